"""The browser front end (``server/ui``) without a browser: every script must tokenise with balanced brackets and closed
strings, every function it calls must be defined in one of the scripts (or be the browser's), every REST route of the
server must be reachable from some page, and the server must hand the files out. No JavaScript engine is needed (there is
none in the test environment): a small tokenizer for the subset of the language the scripts use does the reading."""

import importlib
import re
import sys
from pathlib import Path

import pytest

UI = Path(__file__).resolve().parents[1] / "language_model_saes_b200" / "server" / "ui"
SCRIPTS = ["core.js", "feature.js", "dictionary.js", "graph.js", "circuit.js", "pages.js"]

PUNCT_BEFORE_REGEX = set("(,=:[!&|?{};+-*%<>~^")
WORDS_BEFORE_REGEX = {"return", "typeof", "case", "of", "in", "do", "else", "void", "throw", "new", "delete"}


def tokenize(src: str, name: str = "?"):
    """Tokens ``(kind, text, position)`` with kinds ``id``, ``num``, ``str``, ``tpl`` (a piece of template text), ``re``, ``op``.
    Template literals are entered and left with the brace depth at which ``${`` opened, so nested templates work."""
    out, i, n = [], 0, len(src)
    tpl_stack: list[int] = []  # brace depth at which each open ${ ... } sits
    depth = 0

    def prev_allows_regex() -> bool:
        for kind, text, _ in reversed(out):
            if kind in ("num", "str", "tpl_end", "re"):
                return False
            if kind == "id":
                return text in WORDS_BEFORE_REGEX
            if kind == "op":
                return text in PUNCT_BEFORE_REGEX or text == "=>"
        return True

    def read_template(j: int) -> int:
        """From just after a backtick or a closing ``}`` of a substitution: consume template text up to the closing backtick
        (returns the position after it) or up to ``${`` (pushes the substitution, returns the position after it)."""
        nonlocal depth
        start = j
        while j < n:
            c = src[j]
            if c == "\\":
                j += 2
                continue
            if c == "`":
                out.append(("tpl", src[start:j], start))
                out.append(("tpl_end", "`", j))
                return j + 1
            if c == "$" and j + 1 < n and src[j + 1] == "{":
                out.append(("tpl", src[start:j], start))
                out.append(("op", "${", j))
                depth += 1
                tpl_stack.append(depth)
                return j + 2
            j += 1
        raise AssertionError(f"{name}: template literal opened before {start} is not closed")

    while i < n:
        c = src[i]
        if c.isspace():
            i += 1
        elif src.startswith("//", i):
            i = src.find("\n", i)
            i = n if i < 0 else i
        elif src.startswith("/*", i):
            j = src.find("*/", i)
            assert j >= 0, f"{name}: comment opened at {i} is not closed"
            i = j + 2
        elif c in "'\"":
            j = i + 1
            while j < n and src[j] != c:
                assert src[j] != "\n", f"{name}: string opened at {i} runs over the end of its line"
                j += 2 if src[j] == "\\" else 1
            assert j < n, f"{name}: string opened at {i} is not closed"
            out.append(("str", src[i + 1 : j], i))
            i = j + 1
        elif c == "`":
            out.append(("tpl_start", "`", i))
            i = read_template(i + 1)
        elif c == "/" and prev_allows_regex():
            j, in_class = i + 1, False
            while j < n and (src[j] != "/" or in_class):
                assert src[j] != "\n", f"{name}: regular expression opened at {i} runs over the end of its line"
                if src[j] == "\\":
                    j += 1
                elif src[j] == "[":
                    in_class = True
                elif src[j] == "]":
                    in_class = False
                j += 1
            j += 1
            while j < n and src[j].isalpha():
                j += 1
            out.append(("re", src[i:j], i))
            i = j
        elif c.isalpha() or c in "_$":
            j = i
            while j < n and (src[j].isalnum() or src[j] in "_$"):
                j += 1
            out.append(("id", src[i:j], i))
            i = j
        elif c.isdigit():
            j = i
            while j < n and (src[j].isalnum() or src[j] == "." or (src[j] in "+-" and src[j - 1] in "eE" and not src[i:j].startswith("0x"))):
                j += 1
            out.append(("num", src[i:j], i))
            i = j
        else:
            if c == "{":
                depth += 1
            elif c == "}":
                if tpl_stack and tpl_stack[-1] == depth:
                    tpl_stack.pop()
                    depth -= 1
                    out.append(("op", "}", i))
                    i = read_template(i + 1)
                    continue
                depth -= 1
                assert depth >= 0, f"{name}: closing brace at {i} has no opening one"
            three, two = src[i : i + 3], src[i : i + 2]
            op = three if three in ("===", "!==", "...", "**=", "<<=", ">>=") else two if two in ("=>", "==", "!=", "<=", ">=", "&&", "||", "++", "--", "+=", "-=", "*=", "/=", "??", "?.") else c
            out.append(("op", op, i))
            i += len(op)
    assert not tpl_stack and depth == 0, f"{name}: {depth} braces left open at the end"
    return out


def check_brackets(tokens, name: str) -> None:
    pairs, stack = {")": "(", "]": "[", "}": "{"}, []
    for kind, text, pos in tokens:
        if kind != "op":
            continue
        if text in ("(", "[", "{", "${"):
            stack.append(("{" if text == "${" else text, pos))
        elif text in pairs:
            assert stack and stack[-1][0] == pairs[text], f"{name}: '{text}' at {pos} does not close '{stack[-1][0] if stack else None}'"
            stack.pop()
    assert not stack, f"{name}: '{stack[-1][0]}' opened at {stack[-1][1]} is never closed"


def test_tokenizer_rejects_what_a_browser_would():
    tokenize("const a = `x ${b ? `y ${c}` : 'z'} w`; f(/[/]\\//g, 1 / 2);", "ok")
    check_brackets(tokenize("f(a[0], {b: (1 + 2)});", "ok"), "ok")
    for bad in ("f(a[0)];", "f(1;", "const s = 'abc;\n", "const t = `a ${b`;", "if (x) { y(); ", "a = [1, 2;"):
        with pytest.raises(AssertionError):
            check_brackets(tokenize(bad, "bad"), "bad")


@pytest.fixture(scope="module")
def scripts():
    return {name: tokenize((UI / name).read_text(), name) for name in SCRIPTS}


def test_index_loads_every_script_in_dependency_order():
    html = (UI / "index.html").read_text()
    listed = re.findall(r'<script src="([^"]+)"></script>', html)
    assert listed == SCRIPTS
    assert 'href="style.css"' in html and (UI / "style.css").exists()
    for ident in ("dict", "dictFilter", "fidx", "go", "rand", "circ", "nth", "eth", "overview", "view", "tip"):
        assert f'id="{ident}"' in html, ident


def test_scripts_have_balanced_brackets_and_closed_strings(scripts):
    for name, tokens in scripts.items():
        check_brackets(tokens, name)


JS_WORDS = {"if", "for", "while", "switch", "catch", "function", "return", "typeof", "new", "await", "async", "super", "constructor", "else", "do", "of", "in"}
BROWSER = {"fetch", "Number", "String", "Array", "Object", "Map", "Set", "Error", "JSON", "Math", "DataView", "Uint8Array", "TextDecoder", "Option",
           "encodeURIComponent", "decodeURIComponent", "setTimeout", "clearTimeout", "confirm", "prompt", "alert", "parseInt", "parseFloat", "isNaN", "Promise",
           "Boolean", "Date", "Infinity", "NaN", "document", "window", "location", "history", "localStorage", "console"}  # fmt: skip


def test_every_called_function_is_defined_somewhere(scripts):
    defined, called = set(BROWSER), {}
    for name, tokens in scripts.items():
        for k, (kind, text, pos) in enumerate(tokens):
            if kind != "id":
                continue
            prev = tokens[k - 1] if k else ("op", "", 0)
            nxt = tokens[k + 1] if k + 1 < len(tokens) else ("op", "", 0)
            if prev[0] == "id" and prev[1] in ("function", "class", "const", "let", "var"):
                defined.add(text)
            # parameters and destructured names: an identifier next to a comma / bracket / arrow may be a binding
            if nxt[1] in ("=>", ",", ")", "]", "=", "}") and prev[1] in ("(", ",", "[", "{", "async", "...") or nxt[1] == "=>":
                defined.add(text)
            # method definitions inside a class body: name(args) {  -- recorded as defined too (called through this.)
            if nxt[1] == "(" and prev[1] != "." and text not in JS_WORDS:
                called.setdefault(text, (name, pos))
    missing = {fn: at for fn, at in called.items() if fn not in defined}
    # methods of LinkGraph / GridIndex are written "name(args) {" in their class bodies and reached through "this." or an instance
    methods = {"key", "insert", "nearest", "layout", "shape", "draw", "select", "togglePin", "setMinWeight", "connections", "get", "set"}
    missing = {fn: at for fn, at in missing.items() if fn not in methods}
    assert not missing, f"called but never defined: {missing}"


def _ui_calls(scripts) -> list[str]:
    """Paths handed to ``api(...)``: the first argument's string or template with substitutions replaced by ``{}``."""
    calls = []
    for tokens in scripts.values():
        for k, (kind, text, _) in enumerate(tokens):
            if kind == "id" and text == "api" and tokens[k + 1][1] == "(":
                j, path = k + 2, ""
                if tokens[j][0] == "str":
                    path = tokens[j][1]
                elif tokens[j][0] == "tpl_start":
                    j += 1
                    level = 0
                    while tokens[j][0] != "tpl_end" or level:
                        kind_j, text_j, _ = tokens[j]
                        if kind_j == "op" and text_j == "${":
                            if level == 0:
                                path += "{}"
                            level += 1
                        elif kind_j == "op" and text_j == "}" and level:
                            level -= 1
                        elif kind_j == "tpl" and level == 0:
                            path += text_j
                        elif kind_j == "tpl_start":
                            level += 1
                        elif kind_j == "tpl_end":
                            level -= 1
                        j += 1
                if path:
                    calls.append(path.split("?")[0])
    return calls


def test_every_rest_route_is_used_by_some_page(scripts, tmp_path_factory):
    root = tmp_path_factory.mktemp("ui_routes")
    mp = pytest.MonkeyPatch()
    mp.setenv("MONGO_URI", f"file://{root / 'db'}")
    mp.setenv("MONGO_DB", "ui")
    mp.setenv("SAE_SERIES", "ser")
    mp.setenv("NUM_WORKERS", "0")
    for name in [m for m in sys.modules if m.startswith("language_model_saes_b200.server")]:
        del sys.modules[name]
    try:
        app_mod = importlib.import_module("language_model_saes_b200.server.app")
        from fastapi.testclient import TestClient

        http = TestClient(app_mod.app)
        for name in SCRIPTS + ["index.html", "style.css"]:
            r = http.get(f"/ui/{name}")
            assert r.status_code == 200 and r.text == (UI / name).read_text(), name
        assert "core.js" in http.get("/ui/").text  # the folder serves its index
        routes = sorted({r.path for r in app_mod.app.routes if getattr(r, "methods", None) and not r.path.startswith(("/docs", "/openapi", "/redoc"))})
    finally:
        mp.undo()
        for name in [m for m in sys.modules if m.startswith("language_model_saes_b200.server")]:
            del sys.modules[name]
    calls = _ui_calls(scripts)
    assert len(calls) > 30
    # the feature card reads "is_bookmarked" from the feature record instead of asking GET .../bookmark
    not_needed = {"/dictionaries/{name}/features/{feature_index}/bookmark"}
    unused = []
    for path in routes:
        pattern = re.compile("^" + re.sub(r"\{[^}]+\}", r"(\\{\\}|[^/{}]+)", path) + "$")
        if not any(pattern.match(c) for c in calls) and path not in not_needed:
            unused.append(path)
    assert not unused, f"routes no page calls: {unused}"
    # and the other way round: nothing the pages call is missing on the server
    patterns = [re.compile("^" + re.sub(r"\{[^}]+\}", r"(\\{\\}|[^/{}]+)", p) + "$") for p in routes]
    unknown = [c for c in calls if not any(p.match(c) for p in patterns)]
    assert not unknown, f"pages call paths the server does not have: {unknown}"
