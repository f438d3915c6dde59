// Administration (dictionaries, dictionary sets, circuits: rename, regroup, delete; several circuits at once) and the
// address-bar routing of all pages, including the chrome-less "embed" variants; start-up of the side bar. The reference
// project's counterparts are ui/src/routes/admin.index.tsx, ui/src/routes/__root.tsx and the embed.* routes.

async function showAdmin() {
  loading();
  try {
    const search = store.get("adminSearch", "");
    const [st, saes, sets, circ] = await Promise.all([api("/admin/stats"), api("/admin/saes" + query({ limit: 500, search })), api("/admin/sae-sets"), api("/admin/circuits?limit=500")]);
    let h = `<h1>Administration <span class="muted">series ${esc(st.sae_series)}</span></h1>
      <p>${st.sae_count} dictionaries · ${st.sae_set_count} sets · ${st.circuit_count} circuits · ${st.bookmark_count} bookmarks</p>
      <h2>Dictionaries <span class="muted">${saes.total_count}</span></h2><div class="row"><input id="saeSearch" placeholder="search by name (regular expression)" value="${esc(search)}" style="width:320px"><button id="saeSearchGo">Search</button></div>`;
    h += table(["name", "model", "path", "analyses", "features", ""], saes.saes.map(s => [`<a href="#/dictionaries/${enc(s.name)}">${esc(s.name)}</a>`, esc(s.model_name || ""), esc(s.path || ""), s.analysis_count, count(s.feature_count),
      `<button class="renSae" data-n="${esc(s.name)}">rename</button> <button class="pathSae" data-n="${esc(s.name)}" data-p="${esc(s.path || "")}">path</button>
       <button class="modelSae" data-n="${esc(s.name)}" data-m="${esc(s.model_name || "")}">model</button> <button class="delSae" data-n="${esc(s.name)}">delete</button>`]));
    h += `<h2>Dictionary sets</h2>` + table(["name", "dictionaries", ""], sets.map(s => [esc(s.name), (s.sae_names || []).map(n => `<span class="chip">${esc(n)}</span>`).join(""),
      `<button class="renSet" data-n="${esc(s.name)}">rename</button> <button class="editSet" data-n="${esc(s.name)}" data-s="${esc((s.sae_names || []).join(", "))}">members</button>
       <button class="delSet" data-n="${esc(s.name)}">delete</button>`])) + `<div class="row"><button id="addSet">New set</button></div>`;
    h += `<h2>Circuits <span class="muted">${circ.total_count}</span></h2><div class="row"><input id="bulkGroup" placeholder="group for the ticked circuits (empty: none)"><button id="bulkGo">Move ticked circuits</button></div>` +
      table(["", "name", "group", "status", "prompt", ""], circ.circuits.map(c => [`<input type="checkbox" class="tick" value="${c.id}">`, `<a href="#/circuit/${c.id}">${esc(c.name || c.id)}</a>`, esc(c.group || ""), esc(c.status),
        esc((c.prompt || "").slice(0, 60)), `<button class="renCirc" data-i="${c.id}">rename</button> <button class="grpCirc" data-i="${c.id}">group</button> <button class="delCirc" data-i="${c.id}">delete</button>`]));
    view.innerHTML = h;
    const on = (cls, fn) => view.querySelectorAll("." + cls).forEach(el => el.onclick = async () => { try { if (await fn(el.dataset) !== false) { showAdmin(); refreshLists(); } } catch (e) { fail(e); } });
    const ask = (label, value) => { const v = prompt(label, value || ""); return v === null ? null : v; };
    on("renSae", async d => { const n = ask("New name", d.n); return n ? api(`/admin/saes/${enc(d.n)}`, jsonOpts("PUT", { new_name: n })) : false; });
    on("pathSae", async d => { const p = ask("Path of the weights", d.p); return p ? api(`/admin/saes/${enc(d.n)}`, jsonOpts("PUT", { path: p })) : false; });
    on("modelSae", async d => { const m = ask("Name of the language model record", d.m); return m ? api(`/admin/saes/${enc(d.n)}`, jsonOpts("PUT", { model_name: m })) : false; });
    on("delSae", async d => confirm(`Delete ${d.n} with its analyses and features?`) ? api(`/admin/saes/${enc(d.n)}`, { method: "DELETE" }) : false);
    on("renSet", async d => { const n = ask("New name", d.n); return n ? api(`/admin/sae-sets/${enc(d.n)}`, jsonOpts("PUT", { new_name: n })) : false; });
    on("editSet", async d => { const s = ask("Dictionaries of the set, comma separated", d.s); return s === null ? false :
      api(`/admin/sae-sets/${enc(d.n)}`, jsonOpts("PUT", { sae_names: s.split(",").map(x => x.trim()).filter(x => x) })); });
    on("delSet", async d => confirm(`Delete set ${d.n}?`) ? api(`/admin/sae-sets/${enc(d.n)}`, { method: "DELETE" }) : false);
    on("renCirc", async d => { const n = ask("New name"); return n ? api(`/admin/circuits/${d.i}`, jsonOpts("PUT", { name: n })) : false; });
    on("grpCirc", async d => { const g = ask("Group"); return g ? api(`/admin/circuits/${d.i}`, jsonOpts("PUT", { group: g })) : false; });
    on("delCirc", async d => confirm("Delete this circuit?") ? api(`/circuits/${d.i}`, { method: "DELETE" }) : false);
    $("addSet").onclick = () => newSetDialog(showAdmin);
    $("saeSearchGo").onclick = () => { store.set("adminSearch", $("saeSearch").value); showAdmin(); };
    $("bulkGo").onclick = async () => {
      const ids = [...view.querySelectorAll(".tick:checked")].map(b => b.value);
      if (!ids.length) return;
      try { await api("/admin/circuits/bulk-group", jsonOpts("POST", { circuit_ids: ids, group: $("bulkGroup").value || null })); showAdmin(); refreshLists(); } catch (e) { fail(e); }
    };
  } catch (e) { fail(e); }
}

// ---- routing: the address bar names the page, so that pages can be linked, reloaded and embedded ----
//   #/dictionaries/<name>                      overview          #/dictionaries/<name>/features/<index|random>   feature card
//   #/circuits                                 list              #/circuits/new            form
//   #/circuit/<id>                             graph             #/circuit/<id>/qk/<node>  QK tracing
//   #/bookmarks   #/admin                                        #/embed/<any of the above>  the page without the side bar
function route() {
  let parts = location.hash.split("/").filter(s => s && s !== "#").map(decodeURIComponent);
  const embed = parts[0] === "embed";
  if (embed) parts = parts.slice(1);
  document.body.classList.toggle("embed", embed);
  const [a, b, c, d] = parts;
  if (a === "dictionaries" && b && c === "features" && d !== undefined) { selectOption("dict", b); return showFeature(d); }
  if (a === "dictionaries" && b) { selectOption("dict", b); return showDictionary(b); }
  if (a === "circuits" && b === "new") { showCircuits(); return newCircuitDialog({}); }
  if (a === "circuits") return showCircuits();
  if (a === "circuit" && b && c === "qk" && d) return showQk(b, d);
  if (a === "circuit" && b) { selectOption("circ", b); return showCircuit(); }
  if (a === "bookmarks") return showBookmarks();
  if (a === "admin") return showAdmin();
}

let allDictionaries = [];
function fillDictionaries() {
  const sel = $("dict"), keep = sel.value, f = $("dictFilter").value.toLowerCase();
  sel.innerHTML = "";
  allDictionaries.filter(n => n.toLowerCase().includes(f)).forEach(n => sel.add(new Option(n, n)));
  if (keep) selectOption("dict", keep);
}
async function refreshLists() {
  try { allDictionaries = await api("/dictionaries"); fillDictionaries(); } catch (e) { /* keep what is shown */ }
  refreshCircuitList();
}

window.addEventListener("hashchange", route);
(async () => {
  const th = store.get("thresholds", null);
  if (th) { $("nth").value = th.node; $("eth").value = th.edge; }
  try {
    allDictionaries = await api("/dictionaries");
    fillDictionaries();
    await refreshCircuitList();
  } catch (e) { fail(e); }
  const last = store.get("lastDictionary", null);
  if (last && allDictionaries.includes(last)) $("dict").value = last;
  $("dictFilter").oninput = fillDictionaries;
  $("overview").onclick = ev => { ev.preventDefault(); if ($("dict").value) location.hash = `#/dictionaries/${enc($("dict").value)}`; };
  const go = idx => { if ($("dict").value) location.hash = `#/dictionaries/${enc($("dict").value)}/features/${idx}`; };
  $("go").onclick = () => go($("fidx").value);
  $("fidx").onkeydown = ev => { if (ev.key === "Enter") go($("fidx").value); };
  $("rand").onclick = () => { if ($("dict").value) showFeature("random"); };
  $("dict").onchange = () => go($("fidx").value);
  $("circ").onchange = () => { location.hash = `#/circuit/${$("circ").value}`; };
  $("nth").onchange = () => { if (location.hash.startsWith("#/circuit/")) route(); };
  $("eth").onchange = () => { if (location.hash.startsWith("#/circuit/")) route(); };
  route();
})();
