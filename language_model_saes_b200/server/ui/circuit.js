// Circuit pages: the list of circuits by group, the form that starts a new one (with a preview of the rendered prompt and
// its most likely next tokens), the dictionary-set form, the graph page with its threshold controls, the connections of
// the selected node, the pinned nodes (from which a sub-circuit can be traced) and the QK tracing of an attention
// feature. The reference project's counterparts are ui/src/routes/circuits.index.tsx, circuit.$id.index.tsx,
// embed.circuit.$id.qk.$nodeId.tsx and ui/src/components/circuits/* (graph-selector, new-graph-dialog,
// create-sae-set-dialog, threshold-controls, node-connections, selected-features-list).

// ---- list of circuits, grouped ----
async function showCircuits() {
  loading();
  try {
    const rows = await api("/circuits?limit=500");
    const groups = new Map();
    rows.forEach(c => { const g = c.group || ""; if (!groups.has(g)) groups.set(g, []); groups.get(g).push(c); });
    let h = `<div class="row"><h1 style="margin:0">Circuits <span class="muted">${rows.length}</span></h1><button id="newCirc">New circuit</button><button id="newSet">New dictionary set</button></div>`;
    [...groups.keys()].sort().forEach(g => {
      h += `<h2>${g ? esc(g) : "<span class='muted'>no group</span>"}</h2>` + table(["name", "status", "prompt", "dictionary set", "created", ""], groups.get(g).map(c => [
        c.status === "completed" ? `<a href="#/circuit/${c.id}">${esc(c.name || c.id)}</a>` : esc(c.name || c.id),
        `<span class="${c.status === "failed" ? "err" : c.status === "completed" ? "ok" : "muted"}">${esc(c.status)}</span>` + (c.error_message ? ` <span class="err" data-tip="${esc(c.error_message)}">(why)</span>` : ""),
        esc((c.prompt || "").slice(0, 70)), esc(c.sae_set_name || ""), esc((c.created_at || "").slice(0, 19).replace("T", " ")),
        (c.parent_id ? `<a href="#/circuit/${c.parent_id}" class="muted">parent</a> ` : "") + `<button class="delCirc" data-i="${c.id}">delete</button>`]));
    });
    if (!rows.length) h += "<p class='muted'>No circuit yet.</p>";
    view.innerHTML = h;
    $("newCirc").onclick = () => newCircuitDialog({});
    $("newSet").onclick = () => newSetDialog(showCircuits);
    view.querySelectorAll(".delCirc").forEach(el => el.onclick = async () => {
      if (!confirm("Delete this circuit?")) return;
      try { await api(`/circuits/${el.dataset.i}`, { method: "DELETE" }); refreshCircuitList(); showCircuits(); } catch (e) { fail(e); }
    });
  } catch (e) { fail(e); }
}

async function refreshCircuitList() {
  const sel = $("circ"), keep = sel.value;
  try {
    const rows = await api("/circuits");
    sel.innerHTML = "";
    rows.forEach(c => sel.add(new Option((c.group ? c.group + " / " : "") + (c.name || c.id) + " · " + c.status, c.id)));
    sel.value = keep;
  } catch (e) { /* the list stays as it was */ }
}

// ---- dictionary set: a named list of dictionaries that a circuit is traced through ----
async function newSetDialog(done) {
  const names = [...$("dict").options].map(o => o.value);
  const dlg = openDialog(`<h1>New dictionary set</h1><p><label>name <input id="setName"></label></p>
    <p class="muted">Dictionaries of the set (one transcoder and, if there is one, one attention dictionary per block):</p>
    <div class="row"><input id="setFilter" placeholder="filter" style="flex:1"><button id="setAll">all shown</button><button id="setNone">none</button></div>
    <div id="setList" style="max-height:45vh; overflow:auto">${names.map(n => `<label style="display:block"><input type="checkbox" value="${esc(n)}"> ${esc(n)}</label>`).join("")}</div>
    <div class="row"><button id="setGo">Create</button><button id="setCancel">Cancel</button><span id="setErr" class="err"></span></div>`);
  const boxes = () => [...dlg.querySelectorAll("#setList input")];
  const shown = () => boxes().filter(b => !b.parentElement.hidden);
  dlg.querySelector("#setFilter").oninput = ev => boxes().forEach(b => { b.parentElement.hidden = !b.value.toLowerCase().includes(ev.target.value.toLowerCase()); });
  dlg.querySelector("#setAll").onclick = () => shown().forEach(b => { b.checked = true; });
  dlg.querySelector("#setNone").onclick = () => boxes().forEach(b => { b.checked = false; });
  dlg.querySelector("#setCancel").onclick = dlg.close;
  dlg.querySelector("#setGo").onclick = async () => {
    try {
      await api("/sae-sets", jsonOpts("POST", { name: dlg.querySelector("#setName").value, sae_names: boxes().filter(b => b.checked).map(b => b.value) }));
      dlg.close();
      if (done) done();
    } catch (e) { dlg.querySelector("#setErr").textContent = e.message; }
  };
}

// ---- new circuit: prompt (plain text or chat turns), targets, limits; preview; start; poll ----
// preset: {text, sae_set_name, list_of_features, parent_id, name, group} fills the form (tracing from pinned features)
async function newCircuitDialog(preset) {
  let sets = [];
  try { sets = await api("/sae-sets"); } catch (e) { fail(e); return; }
  const feats = preset.list_of_features || null;
  const dlg = openDialog(`<h1>New circuit</h1>
    <div class="row"><label>dictionary set <select id="ncSet">${sets.map(s => `<option ${s === preset.sae_set_name ? "selected" : ""}>${esc(s)}</option>`).join("")}</select></label>
      <button id="ncNewSet">new set…</button><label>name <input id="ncName" value="${esc(preset.name || "")}"></label><label>group <input id="ncGroup" value="${esc(preset.group || "")}"></label></div>
    <div class="row"><label><input type="radio" name="ncKind" value="plain_text" checked> plain text</label><label><input type="radio" name="ncKind" value="chat_template"> chat turns</label></div>
    <div id="ncPlain"><textarea id="ncText" rows="4" style="width:100%" placeholder="prompt">${esc(preset.text || "")}</textarea></div>
    <div id="ncChat" hidden><div id="ncTurns"></div><button id="ncAddTurn">add turn</button></div>
    <div class="row"><button id="ncPreview">Preview</button><span class="muted">the prompt as the model sees it, and what it would say next</span></div><div id="ncPrevOut"></div>
    <h3>Targets</h3>${feats ? `<p>${feats.length} pinned features are the targets: ${feats.map(f => `<span class="chip">L${f[0]}${f[3] ? "A" : "M"} #${f[1]} @${f[2]}</span>`).join("")}</p>` :
      `<div class="row"><label>logits <input id="ncLogits" type="number" value="1" min="1" style="width:60px"></label>
       <label>or as many as hold this probability mass <input id="ncProb" type="number" step="0.01" value="0.98" style="width:70px"></label></div>`}
    <h3>Limits</h3><div class="row"><label>feature nodes <input id="ncNodes" type="number" value="256" style="width:80px"></label>
      <label>QK tracing top-k (0: off) <input id="ncQk" type="number" value="10" min="0" max="10" style="width:60px"></label></div>
    <div class="row"><button id="ncGo">Start</button><button id="ncCancel">Close</button></div><div id="ncOut"></div>`);
  const q = s => dlg.querySelector(s);
  const addTurn = (role, content) => q("#ncTurns").insertAdjacentHTML("beforeend",
    `<div class="row turn"><select class="role"><option ${role === "user" ? "selected" : ""}>user</option><option ${role === "assistant" ? "selected" : ""}>assistant</option><option ${role === "system" ? "selected" : ""}>system</option></select>
     <textarea class="content" rows="2" style="flex:1">${esc(content || "")}</textarea><button class="rm">×</button></div>`);
  addTurn("user", "");
  q("#ncTurns").addEventListener("click", ev => { if (ev.target.classList.contains("rm")) ev.target.closest(".turn").remove(); });
  q("#ncAddTurn").onclick = () => addTurn("assistant", "");
  dlg.querySelectorAll("[name=ncKind]").forEach(r => r.onchange = () => { q("#ncPlain").hidden = r.value !== "plain_text"; q("#ncChat").hidden = r.value === "plain_text"; });
  const input = () => dlg.querySelector("[name=ncKind]:checked").value === "plain_text" ? { input_type: "plain_text", text: q("#ncText").value } :
    { input_type: "chat_template", messages: [...dlg.querySelectorAll(".turn")].map(t => ({ role: t.querySelector(".role").value, content: t.querySelector(".content").value })) };
  q("#ncNewSet").onclick = () => newSetDialog(async () => {
    const names = await api("/sae-sets");
    q("#ncSet").innerHTML = names.map(s => `<option>${esc(s)}</option>`).join("");
  });
  q("#ncCancel").onclick = dlg.close;
  q("#ncPreview").onclick = async () => {
    q("#ncPrevOut").innerHTML = "<p class='muted'>Running…</p>";
    try {
      const p = await api("/preview", jsonOpts("POST", { input: input(), sae_set_name: q("#ncSet").value }));
      q("#ncPrevOut").innerHTML = `<div class="sample">${esc(p.prompt)}</div><p>next: ${p.next_tokens.map(t => `<span class="chip">${esc(JSON.stringify(t.token))} ${fmt(t.prob, 3)}</span>`).join("")}</p>`;
    } catch (e) { q("#ncPrevOut").innerHTML = `<p class="err">${esc(e.message)}</p>`; }
  };
  q("#ncGo").onclick = async () => {
    try {
      const body = { input: input(), name: q("#ncName").value || null, group: q("#ncGroup").value || null, max_feature_nodes: +q("#ncNodes").value,
        qk_tracing_topk: +q("#ncQk").value, parent_id: preset.parent_id || null };
      if (feats) body.list_of_features = feats; else { body.max_n_logits = +q("#ncLogits").value; body.desired_logit_prob = +q("#ncProb").value; }
      const job = await api("/circuits" + query({ sae_set_name: q("#ncSet").value }), jsonOpts("POST", body));
      q("#ncGo").disabled = true;
      const poll = async () => {
        if (!document.body.contains(dlg)) return;  // closed: the job goes on, the list shows it
        try {
          const s = await api(`/circuits/${job.circuit_id}/status`);
          q("#ncOut").innerHTML = `<p>${esc(s.status)}${s.progress_phase ? " · " + esc(s.progress_phase) : ""}${s.progress !== null && s.progress !== undefined ? " · " + Math.round(s.progress) + "%" : ""}
            ${s.error_message ? `<span class="err">${esc(s.error_message)}</span>` : ""}</p>`;
          if (s.status === "completed") { dlg.close(); refreshCircuitList(); location.hash = `#/circuit/${job.circuit_id}`; return; }
          if (s.status === "failed") { q("#ncGo").disabled = false; return; }
        } catch (e) { q("#ncOut").innerHTML = `<p class="err">${esc(e.message)}</p>`; }
        setTimeout(poll, 1500);
      };
      poll();
    } catch (e) { q("#ncOut").innerHTML = `<p class="err">${esc(e.message)}</p>`; }
  };
}

// ---- the graph page ----
let currentGraph = null;
async function showCircuit() {
  const id = $("circ").value;
  if (!id) return;
  loading();
  try {
    const c = await api(`/circuits/${id}` + query({ node_threshold: $("nth").value, edge_threshold: $("eth").value }));
    store.set("thresholds", { node: +$("nth").value, edge: +$("eth").value });
    const g = c.graph_data;
    view.innerHTML = `<div class="row"><h1 style="margin:0">${esc(c.name || c.circuit_id)}</h1>${c.group ? `<span class="chip">${esc(c.group)}</span>` : ""}
        ${c.parent_id ? `<a class="muted" href="#/circuit/${c.parent_id}">parent circuit</a>` : ""}</div><p class="muted">${esc(c.prompt)}</p>
      <div class="row card"><label>nodes holding this share of the influence <input id="nthS" type="range" min="0.1" max="1" step="0.05" value="${$("nth").value}"> <span id="nthV">${$("nth").value}</span></label>
        <label>edges <input id="ethS" type="range" min="0.1" max="1" step="0.01" value="${$("eth").value}"> <span id="ethV">${$("eth").value}</span></label>
        <label>hide links below <input id="minW" type="range" min="0" max="0.5" step="0.01" value="0"> <span id="minWV">0</span> of the strongest</label>
        <span class="muted">${g.nodes.length} nodes · ${g.links.length} links</span></div>
      <div class="cols"><div><div id="graphHost"></div><p class="muted">click: select a node · shift-click: pin it · click the background: clear</p>
        <h2>Pinned nodes</h2><div id="pins"><p class="muted">None. Pinned feature nodes can be the targets of a new circuit.</p></div></div>
      <div id="sidePanel"><p class="muted">Select a node to see what feeds it and what it feeds.</p></div></div>`;
    const graph = new LinkGraph($("graphHost"), g, { select: n => showConnections(c, graph, n), pin: nodes => showPins(c, graph, nodes) });
    currentGraph = graph;
    const refetch = debounce(() => { $("nth").value = $("nthS").value; $("eth").value = $("ethS").value; showCircuit(); }, 400);
    $("nthS").oninput = () => { $("nthV").textContent = $("nthS").value; refetch(); };
    $("ethS").oninput = () => { $("ethV").textContent = $("ethS").value; refetch(); };
    $("minW").oninput = () => { $("minWV").textContent = $("minW").value; graph.setMinWeight(+$("minW").value); };
  } catch (e) { fail(e); }
}

function connectionRows(graph, links, other) {
  const m = Math.max(1e-9, ...links.map(l => Math.abs(l.weight)));
  return table(["weight", "node"], links.slice(0, 40).map(l => {
    const n = graph.byId.get(l[other]);
    return [`<span class="bar ${l.weight >= 0 ? "pos" : "neg"}" style="width:${Math.round(70 * Math.abs(l.weight) / m)}px"></span> ${fmt(l.weight, 4)}`,
      `<a href="#" class="goNode" data-id="${esc(l[other])}">${esc(n ? n.feature_type : "")}</a> <span class="muted">${esc(n ? layerName(n.layer, graph.maxLayer) + " @" + n.ctx_idx : "")}</span><br>${esc(nodeLabel(n).slice(0, 160))}`];
  })) + (links.length > 40 ? `<p class="muted">${links.length - 40} weaker links not listed</p>` : "");
}

function showConnections(c, graph, n) {
  const box = $("sidePanel");
  if (!n) { box.innerHTML = "<p class='muted'>Select a node to see what feeds it and what it feeds.</p>"; return; }
  const con = graph.connections(n.node_id), f = n.feature && typeof n.feature === "object" ? n.feature : null;
  let h = `<h2>${esc(n.feature_type)} <span class="muted">${layerName(n.layer, graph.maxLayer)} · position ${n.ctx_idx}</span></h2><p>${esc(nodeLabel(n))}</p>`;
  if (n.activation !== undefined && n.activation !== null) h += `<p class="muted">activation ${fmt(n.activation, 4)}</p>`;
  if (f) h += featureSummary(f, { dictionary: n.sae_name, samples: 2 }) +
    `<div class="row"><input id="nodeInterp" style="flex:1" placeholder="interpretation of this feature" value="${esc(interpretationOf(f))}"><button id="nodeInterpSave">Save</button><span id="nodeInterpMsg" class="ok"></span></div>`;
  h += `<div class="row"><button id="pinNode">${graph.pinned.has(n.node_id) ? "unpin" : "pin"}</button>` +
    (n.qk_tracing_results ? `<button id="qkNode">QK tracing</button>` : "") + "</div>";
  h += `<h3>Inputs <span class="muted">${con.inputs.length}</span></h3>${con.inputs.length ? connectionRows(graph, con.inputs, "source") : "<p class='muted'>none kept at these thresholds</p>"}`;
  h += `<h3>Outputs <span class="muted">${con.outputs.length}</span></h3>${con.outputs.length ? connectionRows(graph, con.outputs, "target") : "<p class='muted'>none kept at these thresholds</p>"}`;
  box.innerHTML = h;
  $("pinNode").onclick = () => { graph.togglePin(n.node_id); showConnections(c, graph, n); };
  if ($("nodeInterpSave")) $("nodeInterpSave").onclick = async () => {
    // the label of every node of this feature changes with it: the record is shared by reference between the nodes of one fetch
    try {
      const text = $("nodeInterp").value;
      await api(`/dictionaries/${enc(n.sae_name)}/features/${f.feature_index}/interpretation`, jsonOpts("PUT", { text }));
      graph.g.nodes.forEach(m => { if (m.sae_name === n.sae_name && m.feature && typeof m.feature === "object" && m.feature.feature_index === f.feature_index) m.feature.interpretation = { text }; });
      graph.draw();
      $("nodeInterpMsg").textContent = "saved";
    } catch (e) { $("nodeInterpMsg").textContent = e.message; }
  };
  if ($("qkNode")) $("qkNode").onclick = () => { location.hash = `#/circuit/${c.circuit_id}/qk/${enc(n.node_id)}`; };
  box.querySelectorAll(".goNode").forEach(a => a.onclick = ev => { ev.preventDefault(); graph.select(a.dataset.id); });
}

// pinned nodes; the feature nodes among them can be the targets of a new circuit on the same prompt
function showPins(c, graph, nodes) {
  const box = $("pins");
  if (!nodes.length) { box.innerHTML = "<p class='muted'>None. Pinned feature nodes can be the targets of a new circuit.</p>"; return; }
  const feats = nodes.filter(n => n.feature_type === "lorsa" || n.feature_type === "cross layer transcoder");
  box.innerHTML = nodes.map(n => `<div class="row"><a href="#" class="goNode" data-id="${esc(n.node_id)}">${esc(n.feature_type)}</a>
    <span class="muted">${layerName(n.layer, graph.maxLayer)} @${n.ctx_idx}</span> ${esc(nodeLabel(n).slice(0, 120))} <button class="unpin" data-id="${esc(n.node_id)}">×</button></div>`).join("") +
    (feats.length ? `<button id="traceFrom">Trace a circuit from the ${feats.length} pinned features</button>` : "");
  box.querySelectorAll(".goNode").forEach(a => a.onclick = ev => { ev.preventDefault(); graph.select(a.dataset.id); });
  box.querySelectorAll(".unpin").forEach(b => b.onclick = () => graph.togglePin(b.dataset.id));
  if ($("traceFrom")) $("traceFrom").onclick = () => newCircuitDialog({
    text: (c.input || {}).text || c.prompt, sae_set_name: c.sae_set_name, parent_id: c.circuit_id, group: c.group, name: (c.name || "circuit") + " · sub",
    // (block, feature index, position, is attention dictionary): the row of a node is 2 x block (+ 1 for the transcoder)
    list_of_features: feats.map(n => [Math.floor(n.layer / 2), typeof n.feature === "object" ? n.feature.feature_index : n.feature, n.ctx_idx, n.feature_type === "lorsa"]) });
}

// ---- QK tracing of one attention-feature node: which upstream nodes feed its query and its key side ----
async function showQk(circuitId, nodeId) {
  loading();
  try {
    const r = await api(`/circuits/${circuitId}/qk/${enc(nodeId)}` + query({ node_threshold: $("nth").value, edge_threshold: $("eth").value }));
    const by = new Map(r.referenced_nodes.map(n => [n.node_id, n])), qk = r.target_node.qk_tracing_results, t = r.target_node;
    const cell = id => { const n = by.get(id); return `${esc(n ? n.feature_type : id)} <span class="muted">${n ? "@" + n.ctx_idx : ""}</span><br>${esc((nodeLabel(n) || id).slice(0, 140))}`; };
    const side = rows => {
      const m = Math.max(1e-9, ...(rows || []).map(x => Math.abs(x[1])));
      return table(["contribution", "node"], (rows || []).map(([id, w]) => [`<span class="bar ${w >= 0 ? "pos" : "neg"}" style="width:${Math.round(80 * Math.abs(w) / m)}px"></span> ${fmt(w, 4)}`, cell(id)]));
    };
    const pm = Math.max(1e-9, ...(qk.pair_wise_contributors || []).map(x => Math.abs(x[2])));
    view.innerHTML = `<h1>QK tracing · ${esc(nodeLabel(t))} <span class="muted">${esc(nodeId)} · position ${t.ctx_idx}</span></h1>
      <p><a href="#/circuit/${circuitId}">← back to the circuit</a></p>${t.feature && typeof t.feature === "object" ? featureSummary(t.feature, { dictionary: t.sae_name }) : ""}
      <div class="cols" style="grid-template-columns: 1fr 1fr"><div><h2>Query side</h2>${side(qk.top_q_marginal_contributors)}</div><div><h2>Key side</h2>${side(qk.top_k_marginal_contributors)}</div></div>
      <h2>Pairs (query node x key node)</h2>` + table(["contribution", "query node", "key node"], (qk.pair_wise_contributors || []).map(([q, k, w]) =>
        [`<span class="bar ${w >= 0 ? "pos" : "neg"}" style="width:${Math.round(80 * Math.abs(w) / pm)}px"></span> ${fmt(w, 4)}`, cell(q), cell(k)]));
  } catch (e) { fail(e); }
}
