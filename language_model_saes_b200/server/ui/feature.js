// The feature card: interpretation, bookmark, statistics, logits, activation samples (per sampling, paged), activations on a
// text typed by the user, and an embed snippet. The reference project's counterparts are ui/src/components/feature/*
// (feature-card, sample, feature-logits, feature-interpretation, bookmark-button, inference-card, iframe-integration-card)
// and ui/src/routes/dictionaries.$dictionaryName.features.$featureIndex.tsx.

const sampleStore = new Map();  // sample id -> the record, for the hover handlers
let sampleSeq = 0;

function shade(a, max) {
  const f = max > 0 ? Math.min(a / max, 1) : 0;
  return f < 0.01 ? "" : `background: rgba(255,${Math.round(200 - 160 * f)},0,${(0.25 + 0.6 * f).toFixed(2)})`;
}

// One activation sample as highlighted text. s: the server's sample record (text, origins per token, feature_acts_indices /
// values, token_offset / text_offset when the server cut a window, z_pattern_* for attention features). opts.window: show
// only that many tokens on either side of the strongest one (the rest behind a "show all" switch).
function renderSample(s, max, opts = {}) {
  const id = "s" + (++sampleSeq);
  sampleStore.set(id, s);
  const tokOff = s.token_offset || 0, textOff = s.text_offset || 0;
  // token ranges count characters (code points), a string's own indices count UTF-16 units: cut on an array of characters
  const chars = Array.from(s.text || ""), text = { slice: (a, b) => chars.slice(a, b).join("") };
  const act = new Map((s.feature_acts_indices || []).map((i, k) => [i - tokOff, s.feature_acts_values[k]]));
  let peak = -1, peakV = 0;
  act.forEach((v, i) => { if (v > peakV) { peakV = v; peak = i; } });
  const win = opts.window, lo = win && peak >= 0 ? Math.max(0, peak - win) : 0, hi = win && peak >= 0 ? peak + win : Infinity;
  let html = "", cur = -1, shown = 0, hidden = 0;
  (s.origins || []).forEach((o, i) => {
    if (!o) return;
    if (i < lo || i > hi) { hidden++; return; }
    if (o.key === "image") { html += `<span class="chip" data-i="${i}">image</span>`; return; }
    if (o.key !== "text" || !o.range) return;
    const a = o.range[0] - textOff, b = o.range[1] - textOff;
    if (cur < 0) cur = a;
    if (a > cur) html += esc(text.slice(cur, a));
    const v = act.get(i) || 0;
    html += `<span class="tok${i === peak ? " peak" : ""}" data-i="${i}" style="${shade(v, max)}" data-tip="token ${i + tokOff} · activation ${v.toFixed(3)}">${esc(text.slice(Math.max(a, cur), b))}</span>`;
    cur = Math.max(cur, b);
    shown++;
  });
  if (hi === Infinity && cur >= 0) html += esc(text.slice(cur));  // text after the last token (nothing was cut at the end)
  const more = hidden ? `<a href="#" class="expand" data-sid="${id}" data-max="${max}">… ${hidden} more tokens</a>` : "";
  const meta = opts.meta ? `<span class="meta">${esc(opts.meta)}</span>` : "";
  return `<div class="sample" data-sid="${id}">${meta}${lo > 0 ? "… " : ""}${html}${more ? " " + more : ""}${shown ? "" : "<span class='muted'>(no text tokens)</span>"}</div>`;
}

// attention features: hovering a token marks the tokens its value was read from (z pattern of that query position)
view.addEventListener("mouseover", ev => {
  const t = ev.target.closest ? ev.target.closest(".tok[data-i]") : null;
  const box = t ? t.closest(".sample[data-sid]") : null;
  if (!box) return;
  const s = sampleStore.get(box.dataset.sid);
  box.querySelectorAll(".tok.zsrc").forEach(el => { el.classList.remove("zsrc"); el.style.removeProperty("--z"); });
  if (!s || !s.z_pattern_indices || !s.z_pattern_values || s.z_pattern_indices.length < 2) return;
  const q = +t.dataset.i + (s.token_offset || 0), [qs, ks] = s.z_pattern_indices;
  let m = 0;
  qs.forEach((qq, n) => { if (qq === q) m = Math.max(m, Math.abs(s.z_pattern_values[n])); });
  if (!m) return;
  qs.forEach((qq, n) => {
    if (qq !== q) return;
    const el = box.querySelector(`.tok[data-i="${ks[n] - (s.token_offset || 0)}"]`);
    if (el) { el.classList.add("zsrc"); el.style.setProperty("--z", (0.2 + 0.8 * Math.abs(s.z_pattern_values[n]) / m).toFixed(2)); }
  });
});
view.addEventListener("click", ev => {
  const a = ev.target.closest ? ev.target.closest("a.expand[data-sid]") : null;
  if (!a) return;
  ev.preventDefault();
  const s = sampleStore.get(a.dataset.sid), box = a.closest(".sample");
  if (s && box) box.outerHTML = renderSample(s, +a.dataset.max);
});

function logitBars(logits) {
  if (!logits) return "";
  const pos = logits.top_positive || [], neg = logits.top_negative || [];
  const m = Math.max(1e-9, ...pos.map(t => Math.abs(t.logit)), ...neg.map(t => Math.abs(t.logit)));
  const cell = (t, cls) => t ? `${esc(t.token)} <span class="bar ${cls}" style="width:${Math.round(90 * Math.abs(t.logit) / m)}px"></span> <span class="muted">${t.logit.toFixed(2)}</span>` : "";
  const rows = [];
  for (let i = 0; i < Math.max(pos.length, neg.length); i++) rows.push([cell(pos[i], "pos"), cell(neg[i], "neg")]);
  let h = "<h2>Logits</h2>" + table(["promotes", "suppresses"], rows);
  if (logits.histogram) h += histogram(logits.histogram, 360, 80);
  return h;
}

// per-head figures of a crosscoder feature: decoder norms and the similarity of the heads' decoder rows
function decoderTables(f) {
  let h = "";
  if (Array.isArray(f.decoder_norms) && f.decoder_norms.length > 1)
    h += "<h2>Decoder norms per head</h2>" + table(f.decoder_norms.map((_, i) => "head " + i), [f.decoder_norms.map(v => fmt(v, 3))]);
  const sim = f.decoder_similarity_matrix;
  if (Array.isArray(sim) && sim.length > 1 && Array.isArray(sim[0]))
    h += "<h2>Decoder similarity between heads</h2>" + table([""].concat(sim.map((_, i) => String(i))), sim.map((r, i) => [`<b>${i}</b>`].concat(r.map(v =>
      `<span style="background: rgba(40,120,220,${Math.max(0, Math.min(1, v)).toFixed(2)}); padding: 0 4px">${fmt(v, 2)}</span>`))));
  return h;
}

const SAMPLE_PAGE = 10;
async function loadSamples(dict, f, sampling, start, into) {
  const win = +store.get("visibleRange", 60) || null;
  const got = await api(`/dictionaries/${enc(dict)}/features/${f.feature_index}/sampling/${enc(sampling.name)}` +
    query({ analysis_name: f.analysis_name, start, length: SAMPLE_PAGE }));
  into.insertAdjacentHTML("beforeend", got.map((s, k) => renderSample(s, f.max_feature_act, { window: win, meta: `#${start + k + 1}` })).join(""));
  return got.length;
}

async function showFeature(idx) {
  const d = $("dict").value;
  if (!d) return;
  loading();
  try {
    const f = await api(`/dictionaries/${enc(d)}/features/${idx}` + query({ no_samplings: true, feature_analysis_name: store.get("analysis." + d, null) }));
    const [samplings, analyses] = await Promise.all([
      api(`/dictionaries/${enc(d)}/features/${f.feature_index}/samplings` + query({ analysis_name: f.analysis_name })),
      api(`/dictionaries/${enc(d)}/analyses`).catch(() => [])]);
    $("fidx").value = f.feature_index;
    store.set("lastDictionary", d);
    const here = `#/dictionaries/${enc(d)}/features/${f.feature_index}`;
    if (location.hash !== here && !location.hash.startsWith("#/embed")) history.replaceState(null, "", here);
    let h = `<div class="row"><button id="prevF" ${f.feature_index ? "" : "disabled"}>←</button><h1 style="margin:0">Feature #${f.feature_index} <span class="muted">@ ${esc(f.dictionary_name)}</span></h1><button id="nextF">→</button>
      ${analyses.length > 1 ? `<label class="muted">analysis <select id="anaSel">${analyses.map(a => `<option ${a === f.analysis_name ? "selected" : ""}>${esc(a)}</option>`).join("")}</select></label>` : ""}</div>`;
    h += `<div class="row"><input id="interp" style="flex:1" placeholder="interpretation" value="${esc(interpretationOf(f))}"><button id="saveInterp">Save</button>
          <button id="bm">${f.is_bookmarked ? "★ bookmarked" : "☆ bookmark"}</button>${f.is_bookmarked ? "<button id='bmEdit'>tags / notes</button>" : ""}<span id="saved" class="ok"></span></div>`;
    h += `<p>fired ${count(f.act_times)} times · max ${fmt(f.max_feature_act, 4)} · ${count(f.n_analyzed_tokens)} tokens analysed` +
      (f.n_analyzed_tokens ? ` · density ${(f.act_times / f.n_analyzed_tokens).toExponential(2)}` : "") + "</p>";
    h += `<div class="cols"><div>`;
    h += `<div class="tabs">${samplings.map((s, i) => `<button class="tab${i ? "" : " on"}" data-k="${i}">${esc(s.name)} <span class="muted">${s.length}</span></button>`).join("")}</div>`;
    h += `<div class="row muted"><label>tokens shown around the strongest one <input id="visRange" type="number" min="0" step="10" value="${+store.get("visibleRange", 60)}" style="width:70px"> (0: whole sample)</label></div>`;
    h += `<div id="samples"></div><button id="moreSamples">more samples</button>`;
    h += `<h2>Try a text</h2><div class="row"><input id="txt" style="flex:1" placeholder="text to run through the model"><button id="infer">Run</button></div><div id="inferOut"></div>`;
    h += `</div><div>${logitBars(f.logits)}${decoderTables(f)}
      <h2>Embed</h2><p class="muted">This card without the side bar, for an iframe:</p><code class="snip">${esc(`<iframe src="${location.origin}${location.pathname}#/embed/dictionaries/${enc(d)}/features/${f.feature_index}" width="900" height="600"></iframe>`)}</code></div></div>`;
    view.innerHTML = h;

    let current = 0, loaded = 0;
    const box = $("samples"), moreBtn = $("moreSamples");
    const fill = async reset => {
      if (!samplings.length) { box.innerHTML = "<p class='muted'>No samples stored for this feature.</p>"; moreBtn.hidden = true; return; }
      if (reset) { box.innerHTML = ""; loaded = 0; }
      moreBtn.disabled = true;
      let got = 0;
      try { got = await loadSamples(d, f, samplings[current], loaded, box); } catch (e) { box.insertAdjacentHTML("beforeend", `<p class="err">${esc(e.message)}</p>`); }
      loaded += got;
      moreBtn.disabled = false;
      moreBtn.hidden = !got || loaded >= samplings[current].length;
    };
    view.querySelectorAll(".tab").forEach(b => b.onclick = () => {
      view.querySelectorAll(".tab").forEach(x => x.classList.toggle("on", x === b));
      current = +b.dataset.k;
      fill(true);
    });
    moreBtn.onclick = () => fill(false);
    $("visRange").onchange = () => { store.set("visibleRange", +$("visRange").value); fill(true); };
    fill(true);

    if ($("anaSel")) $("anaSel").onchange = () => { store.set("analysis." + d, $("anaSel").value); showFeature(f.feature_index); };
    $("prevF").onclick = () => showFeature(f.feature_index - 1);
    $("nextF").onclick = () => showFeature(f.feature_index + 1);
    $("saveInterp").onclick = async () => {
      try {
        await api(`/dictionaries/${enc(d)}/features/${f.feature_index}/interpretation`, jsonOpts("PUT", { text: $("interp").value }));
        $("saved").textContent = "saved";
      } catch (e) { $("saved").textContent = e.message; }
    };
    $("bm").onclick = async () => {
      await api(`/dictionaries/${enc(d)}/features/${f.feature_index}/bookmark`, { method: f.is_bookmarked ? "DELETE" : "POST" });
      showFeature(f.feature_index);
    };
    if ($("bmEdit")) $("bmEdit").onclick = () => editBookmark(d, f.feature_index);
    $("infer").onclick = async () => {
      $("inferOut").innerHTML = "<p class='muted'>Running…</p>";
      try {
        const r = await api(`/dictionaries/${enc(d)}/features/${f.feature_index}/infer` + query({ text: $("txt").value }), { method: "POST" });
        $("inferOut").innerHTML = renderSample(r, Math.max(f.max_feature_act, ...(r.feature_acts_values || [0])));
      } catch (e) { $("inferOut").innerHTML = `<p class="err">${esc(e.message)}</p>`; }
    };
    $("txt").onkeydown = ev => { if (ev.key === "Enter") $("infer").click(); };
  } catch (e) { fail(e); }
}

// tags and notes of a bookmark (PUT .../bookmark: the tag list is the JSON body, the notes a query parameter)
function editBookmark(dict, index, done) {
  const dlg = openDialog(`<h1>Bookmark · ${esc(dict)} #${index}</h1>
    <p><label>tags, comma separated<br><input id="bmTags" style="width:100%"></label></p>
    <p><label>notes<br><textarea id="bmNotes" rows="4" style="width:100%"></textarea></label></p>
    <div class="row"><button id="bmSave">Save</button><button id="bmCancel">Cancel</button><span id="bmErr" class="err"></span></div>`);
  dlg.querySelector("#bmCancel").onclick = dlg.close;
  dlg.querySelector("#bmSave").onclick = async () => {
    const tags = dlg.querySelector("#bmTags").value.split(",").map(t => t.trim()).filter(t => t);
    try {
      await api(`/dictionaries/${enc(dict)}/features/${index}/bookmark` + query({ notes: dlg.querySelector("#bmNotes").value }), jsonOpts("PUT", tags));
      dlg.close();
      if (done) done();
    } catch (e) { dlg.querySelector("#bmErr").textContent = e.message; }
  };
}

// left / right arrow keys step through the features of the open card (not while typing in a field)
document.addEventListener("keydown", ev => {
  if (ev.target && ["INPUT", "TEXTAREA", "SELECT"].includes(ev.target.tagName)) return;
  const b = ev.key === "ArrowLeft" ? $("prevF") : ev.key === "ArrowRight" ? $("nextF") : null;
  if (b && !b.disabled) b.click();
});

// a feature in a few lines (lists, the connections panel of a circuit): index, interpretation, one sample
function featureSummary(f, opts = {}) {
  if (!f) return "";
  const name = f.dictionary_name || opts.dictionary || "";
  const head = `<a href="#/dictionaries/${enc(name)}/features/${f.feature_index}">#${f.feature_index}</a> <span class="muted">${esc(name)}</span>`;
  const stats = f.act_times !== undefined ? `<span class="muted"> · fired ${count(f.act_times)} · max ${fmt(f.max_feature_act, 2)}</span>` : "";
  const sample = (f.samples || []).slice(0, opts.samples || 1).map(s => renderSample(s, f.max_feature_act, { window: opts.window || 12 })).join("");
  return `<div class="card">${head}${stats}<div>${esc(interpretationOf(f)) || "<span class='muted'>no interpretation</span>"}</div>${sample}</div>`;
}
