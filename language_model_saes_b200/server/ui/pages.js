// Pages beyond the feature card and the circuit graph of index.html: dictionary overview, bookmarks, administration,
// circuit jobs (create, poll, delete), QK tracing of an attention node, and address-bar routing (#/...), including the
// chrome-less "embed" variants. Uses the helpers index.html defines (api, $, view, esc, showFeature, showCircuit).
// The reference project's counterparts are the routes under ui/src/routes (dictionaries.*, bookmarks.index,
// admin.index, circuits.index, circuit.$id.index, embed.*).

const enc = encodeURIComponent;
const jsonOpts = (method, body) => ({ method, headers: { "content-type": "application/json" }, body: JSON.stringify(body) });
const fail = e => { view.innerHTML = `<p class="err">${esc(e.message)}</p>`; };
const table = (head, rows) => `<table><tr>${head.map(h => `<th>${esc(h)}</th>`).join("")}</tr>${rows.map(r => `<tr>${r.map(c => `<td>${c}</td>`).join("")}</tr>`).join("")}</table>`;

function histogram(h) {
  // h: {x: bin centres, y: counts} as the server's activation_histogram gives it, or a list of counts
  const y = Array.isArray(h) ? h : (h.y || h.counts || []), x = Array.isArray(h) ? y.map((_, i) => i) : (h.x || h.bins || y.map((_, i) => i));
  if (!y.length) return "";
  const W = 520, H = 120, m = Math.max(1, ...y), bw = (W - 20) / y.length;
  let s = `<svg width="${W}" height="${H + 18}">`;
  y.forEach((v, i) => { const hh = (H - 6) * v / m; s += `<rect x="${10 + i * bw}" y="${H - hh}" width="${Math.max(1, bw - 1)}" height="${hh}" fill="#69c"><title>${esc(x[i])}: ${v}</title></rect>`; });
  return s + `<text x="10" y="${H + 14}" font-size="11">${esc(x[0])}</text><text x="${W - 10}" y="${H + 14}" font-size="11" text-anchor="end">${esc(x[x.length - 1])}</text></svg>`;
}

// ---- dictionary overview: alive features, activation-count histogram, metrics, a page of feature summaries ----
async function showDictionary(name, start = 0) {
  view.innerHTML = "<p class='muted'>Loading…</p>";
  try {
    const [d, metrics] = await Promise.all([api(`/dictionaries/${enc(name)}`), api(`/dictionaries/${enc(name)}/metrics`).catch(() => ({ metrics: [] }))]);
    const page = 20, feats = await api(`/dictionaries/${enc(name)}/features?start=${start}&end=${start + page}&sample_length=1`);
    let h = `<h1>${esc(name)}</h1><p>${(d.alive_feature_count || 0).toLocaleString()} features fired at least once</p>`;
    (d.feature_activation_times_histogram || []).forEach(x => h += histogram(x));
    if ((metrics.metrics || []).length) h += `<p class="muted">metrics: ${metrics.metrics.map(esc).join(", ")}</p>`;
    h += `<h2>Features ${start} – ${start + page - 1}</h2>` + table(["#", "fired", "max", "interpretation"], feats.filter(f => f).map(f => [
      `<a href="#/dictionaries/${enc(name)}/features/${f.feature_index}">${f.feature_index}</a>`, (f.act_times || 0).toLocaleString(),
      (f.max_feature_act || 0).toFixed(3), esc((f.interpretation || {}).text || "")]));
    h += `<div class="row"><button id="prevPage" ${start ? "" : "disabled"}>← previous</button><button id="nextPage">next →</button></div>`;
    view.innerHTML = h;
    $("prevPage").onclick = () => showDictionary(name, Math.max(0, start - page));
    $("nextPage").onclick = () => showDictionary(name, start + page);
  } catch (e) { fail(e); }
}

// ---- bookmarks ----
async function showBookmarks() {
  try {
    const b = await api("/bookmarks?limit=200");
    view.innerHTML = `<h1>Bookmarks <span class="muted">${b.total_count}</span></h1>` + table(["dictionary", "feature", "tags", "notes", "created", ""],
      b.bookmarks.map(m => [esc(m.sae_name), `<a href="#/dictionaries/${enc(m.sae_name)}/features/${m.feature_index}">#${m.feature_index}</a>`,
        esc((m.tags || []).join(", ")), esc(m.notes || ""), esc((m.created_at || "").slice(0, 19)),
        `<button data-d="${esc(m.sae_name)}" data-f="${m.feature_index}" class="unmark">remove</button>`]));
    view.querySelectorAll(".unmark").forEach(el => el.onclick = async () => {
      await api(`/dictionaries/${enc(el.dataset.d)}/features/${el.dataset.f}/bookmark`, { method: "DELETE" }); showBookmarks(); });
  } catch (e) { fail(e); }
}

// ---- administration: counts, dictionaries (rename / delete), dictionary sets, circuits (rename, group, delete) ----
async function showAdmin() {
  try {
    const [st, saes, sets, circ] = await Promise.all([api("/admin/stats"), api("/admin/saes?limit=500"), api("/admin/sae-sets"), api("/admin/circuits?limit=500")]);
    let h = `<h1>Administration <span class="muted">series ${esc(st.sae_series)}</span></h1>
      <p>${st.sae_count} dictionaries · ${st.sae_set_count} sets · ${st.circuit_count} circuits · ${st.bookmark_count} bookmarks</p><h2>Dictionaries</h2>`;
    h += table(["name", "model", "path", "analyses", "features", ""], saes.saes.map(s => [esc(s.name), esc(s.model_name || ""), esc(s.path || ""), s.analysis_count, s.feature_count,
      `<button class="renSae" data-n="${esc(s.name)}">rename</button> <button class="delSae" data-n="${esc(s.name)}">delete</button>`]));
    h += "<h2>Dictionary sets</h2>" + table(["name", "dictionaries", ""], (sets.sae_sets || sets).map(s => [esc(s.name), esc((s.sae_names || []).join(", ")),
      `<button class="delSet" data-n="${esc(s.name)}">delete</button>`]));
    h += `<div class="row"><input id="setName" placeholder="new set name"><input id="setSaes" style="flex:1" placeholder="dictionary names, comma separated"><button id="addSet">Create set</button></div>`;
    h += "<h2>Circuits</h2>" + table(["name", "group", "status", "prompt", ""], circ.circuits.map(c => [`<a href="#/circuit/${c.id}">${esc(c.name || c.id)}</a>`, esc(c.group || ""), esc(c.status),
      esc((c.prompt || "").slice(0, 60)), `<button class="renCirc" data-i="${c.id}">rename</button> <button class="grpCirc" data-i="${c.id}">group</button> <button class="delCirc" data-i="${c.id}">delete</button>`]));
    view.innerHTML = h;
    const on = (cls, fn) => view.querySelectorAll("." + cls).forEach(el => el.onclick = async () => { try { if (await fn(el.dataset) !== false) showAdmin(); } catch (e) { fail(e); } });
    on("renSae", async d => { const n = prompt("New name", d.n); return n ? api(`/admin/saes/${enc(d.n)}`, jsonOpts("PUT", { new_name: n })) : false; });
    on("delSae", async d => confirm(`Delete ${d.n} with its analyses and features?`) ? api(`/admin/saes/${enc(d.n)}`, { method: "DELETE" }) : false);
    on("delSet", async d => confirm(`Delete set ${d.n}?`) ? api(`/admin/sae-sets/${enc(d.n)}`, { method: "DELETE" }) : false);
    on("renCirc", async d => { const n = prompt("New name"); return n ? api(`/admin/circuits/${d.i}`, jsonOpts("PUT", { name: n })) : false; });
    on("grpCirc", async d => { const g = prompt("Group"); return g ? api(`/admin/circuits/${d.i}`, jsonOpts("PUT", { group: g })) : false; });
    on("delCirc", async d => confirm("Delete this circuit?") ? api(`/circuits/${d.i}`, { method: "DELETE" }) : false);
    $("addSet").onclick = async () => { try {
      await api("/sae-sets", jsonOpts("POST", { name: $("setName").value, sae_names: $("setSaes").value.split(",").map(s => s.trim()).filter(s => s) })); showAdmin();
    } catch (e) { fail(e); } };
  } catch (e) { fail(e); }
}

// ---- circuit jobs: start one from a prompt and a dictionary set, poll its status, open it when it is done ----
async function showNewCircuit() {
  try {
    const sets = await api("/sae-sets");
    view.innerHTML = `<h1>New circuit</h1>
      <div class="row"><label>dictionary set <select id="ncSet">${sets.map(s => `<option>${esc(s)}</option>`).join("")}</select></label>
      <label>name <input id="ncName"></label><label>group <input id="ncGroup"></label></div>
      <textarea id="ncText" rows="4" style="width:100%" placeholder="prompt"></textarea>
      <div class="row"><label>logit probability mass <input id="ncProb" type="number" step="0.01" value="0.98" style="width:70px"></label>
      <label>feature nodes <input id="ncNodes" type="number" value="256" style="width:70px"></label>
      <label>logits <input id="ncLogits" type="number" value="1" style="width:50px"></label>
      <label>QK tracing top-k <input id="ncQk" type="number" value="10" style="width:50px"></label><button id="ncGo">Start</button></div><div id="ncOut"></div>`;
    $("ncGo").onclick = async () => { try {
      const body = { input: { input_type: "plain_text", text: $("ncText").value }, name: $("ncName").value || null, group: $("ncGroup").value || null,
        desired_logit_prob: +$("ncProb").value, max_feature_nodes: +$("ncNodes").value, max_n_logits: +$("ncLogits").value, qk_tracing_topk: +$("ncQk").value };
      const job = await api(`/circuits?sae_set_name=${enc($("ncSet").value)}`, jsonOpts("POST", body));
      const poll = async () => {
        if (!$("ncOut")) return;  // the user went elsewhere
        const s = await api(`/circuits/${job.circuit_id}/status`);
        $("ncOut").innerHTML = `<p>${esc(s.status)}${s.progress_phase ? " · " + esc(s.progress_phase) : ""}${s.progress != null ? " · " + Math.round(100 * s.progress) + "%" : ""}
          ${s.error_message ? `<span class="err">${esc(s.error_message)}</span>` : ""}</p>`;
        if (s.status === "completed") location.hash = `#/circuit/${job.circuit_id}`; else if (s.status !== "failed") setTimeout(poll, 1500);
      };
      poll();
    } catch (e) { $("ncOut").innerHTML = `<p class="err">${esc(e.message)}</p>`; } };
  } catch (e) { fail(e); }
}

// ---- QK tracing of one attention-feature node: which upstream nodes feed its query and its key side ----
async function showQk(circuitId, nodeId) {
  try {
    const r = await api(`/circuits/${circuitId}/qk/${enc(nodeId)}?node_threshold=${$("nth").value}&edge_threshold=${$("eth").value}`);
    const label = n => n ? esc(n.token != null ? n.token : ((n.feature || {}).interpretation || {}).text || n.node_id) : "";
    const by = Object.fromEntries(r.referenced_nodes.map(n => [n.node_id, n])), qk = r.target_node.qk_tracing_results;
    const side = rows => table(["node", "label", "contribution"], (rows || []).map(([id, w]) => [esc(id), label(by[id]), (+w).toFixed(4)]));
    view.innerHTML = `<h1>QK tracing · ${esc(nodeId)} <span class="muted">${label(r.target_node)}</span></h1>
      <p><a href="#/circuit/${circuitId}">← back to the circuit</a></p><h2>Query side</h2>${side(qk.top_q_marginal_contributors)}
      <h2>Key side</h2>${side(qk.top_k_marginal_contributors)}<h2>Pairs</h2>` +
      table(["query node", "key node", "contribution"], (qk.pair_wise_contributors || []).map(([q, k, w]) => [`${esc(q)} ${label(by[q])}`, `${esc(k)} ${label(by[k])}`, (+w).toFixed(4)]));
  } catch (e) { fail(e); }
}

// ---- routing: the address bar names the page, so that pages can be linked, reloaded and embedded ----
//   #/dictionaries/<name>                      overview          #/dictionaries/<name>/features/<index|random>   feature card
//   #/circuits/new                             job form          #/circuit/<id>            graph        #/circuit/<id>/qk/<node>   QK tracing
//   #/bookmarks   #/admin                                        #/embed/<any of the above>             the page without the side bar
function route() {
  let parts = location.hash.replace(/^#\/?/, "").split("/").filter(s => s).map(decodeURIComponent);
  const embed = parts[0] === "embed";
  if (embed) parts = parts.slice(1);
  document.body.classList.toggle("embed", embed);
  const [a, b, c, d] = parts;
  if (a === "dictionaries" && b && c === "features" && d != null) { selectOption("dict", b); return showFeature(d); }
  if (a === "dictionaries" && b) { selectOption("dict", b); return showDictionary(b); }
  if (a === "circuits" && b === "new") return showNewCircuit();
  if (a === "circuit" && b && c === "qk" && d) return showQk(b, d);
  if (a === "circuit" && b) { selectOption("circ", b); return showCircuit(); }
  if (a === "bookmarks") return showBookmarks();
  if (a === "admin") return showAdmin();
}
function selectOption(id, value) {
  const sel = $(id);
  if (![...sel.options].some(o => o.value === value)) sel.add(new Option(value, value));  // lists still loading, or an id that is not listed
  sel.value = value;
}
window.addEventListener("hashchange", route);
window.addEventListener("load", () => setTimeout(route, 0));
// clicking an attention node of a drawn circuit opens its QK tracing
view.addEventListener("click", ev => {
  const n = ev.target.closest && ev.target.closest("circle.node[data-qk]");
  if (n && $("circ").value) location.hash = `#/circuit/${$("circ").value}/qk/${enc(n.dataset.qk)}`;
});
