// Dictionary pages: overview (alive features, activation-count histogram, a filtered, paged list of features with their
// strongest sample), the features that fire on a text typed by the user, and the bookmark list. The reference project's
// counterparts are ui/src/routes/dictionaries.$dictionaryName.index.tsx, ui/src/components/dictionary/* and
// ui/src/routes/bookmarks.index.tsx.

const FEATURE_PAGE = 20;

// metric filters: one row per metric the dictionary's analyses carry, "min" and "max" bounds -> {"metric": {"$gte": a, "$lte": b}}
function readFilters(box) {
  const out = {};
  box.querySelectorAll("[data-metric]").forEach(row => {
    const lo = row.querySelector(".lo").value, hi = row.querySelector(".hi").value, f = {};
    if (lo !== "") f["$gte"] = +lo;
    if (hi !== "") f["$lte"] = +hi;
    if (Object.keys(f).length) out[row.dataset.metric] = f;
  });
  return Object.keys(out).length ? JSON.stringify(out) : null;
}

async function showDictionary(name, start = 0) {
  loading();
  try {
    const [d, metrics, analyses] = await Promise.all([
      api(`/dictionaries/${enc(name)}`),
      api(`/dictionaries/${enc(name)}/metrics`).catch(() => ({ metrics: [] })),
      api(`/dictionaries/${enc(name)}/analyses`).catch(() => [])]);
    store.set("lastDictionary", name);
    let h = `<h1>${esc(name)}</h1><p>${count(d.alive_feature_count)} features fired at least once` +
      (analyses.length ? ` · analyses: ${analyses.map(a => `<span class="chip">${esc(a)}</span>`).join("")}` : "") + "</p>";
    (d.feature_activation_times_histogram || []).forEach(x => { h += `<div><span class="muted">log10 of how often each feature fired</span><br>${histogram(x)}</div>`; });
    h += `<h2>Features that fire on a text</h2><div class="row"><input id="infText" style="flex:1" placeholder="text to run through the model and this dictionary">
      <label>features <input id="infMax" type="number" value="10" min="1" max="100" style="width:60px"></label><button id="infGo">Run</button></div><div id="infOut"></div>`;
    h += `<h2>Features</h2>`;
    if ((metrics.metrics || []).length)
      h += `<div id="filters" class="card"><span class="muted">keep features whose metrics lie within</span>` + metrics.metrics.map(m =>
        `<div class="row" data-metric="${esc(m)}"><span style="width:220px">${esc(m)}</span><input class="lo" type="number" step="any" placeholder="min" style="width:90px">
         <input class="hi" type="number" step="any" placeholder="max" style="width:90px"></div>`).join("") +
        `<div class="row"><button id="countGo">Count</button><button id="randGo">Random feature within the bounds</button><span id="countOut" class="muted"></span></div></div>`;
    h += `<div class="row"><button id="prevPage" ${start ? "" : "disabled"}>← previous</button><span class="muted">${start} – ${start + FEATURE_PAGE - 1}</span><button id="nextPage">next →</button>
      <label class="muted">jump to <input id="jump" type="number" min="0" style="width:90px"></label></div><div id="featList"><p class="muted">Loading…</p></div>`;
    view.innerHTML = h;
    $("prevPage").onclick = () => showDictionary(name, Math.max(0, start - FEATURE_PAGE));
    $("nextPage").onclick = () => showDictionary(name, start + FEATURE_PAGE);
    $("jump").onchange = () => showDictionary(name, Math.max(0, Math.floor(+$("jump").value / FEATURE_PAGE) * FEATURE_PAGE));
    $("infGo").onclick = () => dictionaryInference(name);
    $("infText").onkeydown = ev => { if (ev.key === "Enter") dictionaryInference(name); };
    if ($("countGo")) {
      $("countGo").onclick = async () => {
        try {
          const r = await api(`/dictionaries/${enc(name)}/features/count` + query({ metric_filters: readFilters($("filters")) }));
          $("countOut").textContent = count(r.count) + " features";
        } catch (e) { $("countOut").textContent = e.message; }
      };
      $("randGo").onclick = async () => {
        try {
          const f = await api(`/dictionaries/${enc(name)}/features/random` + query({ metric_filters: readFilters($("filters")), no_samplings: true }));
          location.hash = `#/dictionaries/${enc(name)}/features/${f.feature_index}`;
        } catch (e) { $("countOut").textContent = e.message; }
      };
    }
    const feats = await api(`/dictionaries/${enc(name)}/features` + query({ start, end: start + FEATURE_PAGE, sample_length: 1, visible_range: 12 }));
    const shown = feats.filter(f => f);
    if (!$("featList")) return;  // the user went elsewhere while the list was loading
    $("featList").innerHTML = shown.length ? shown.map(f => featureSummary(f, { dictionary: name })).join("") : "<p class='muted'>No analysed features in this range.</p>";
  } catch (e) { fail(e); }
}

// POST /dictionaries/<name>/inference: the features with the largest summed activation on the text, each with its
// activations on that text and a few stored samples
async function dictionaryInference(name) {
  const out = $("infOut");
  out.innerHTML = "<p class='muted'>Running…</p>";
  try {
    const rows = await api(`/dictionaries/${enc(name)}/inference` + query({ text: $("infText").value, max_features: $("infMax").value }), { method: "POST" });
    if (!rows.length) { out.innerHTML = "<p class='muted'>No feature fired.</p>"; return; }
    out.innerHTML = rows.map(r => {
      const inf = r.inference || {}, m = Math.max(r.max_feature_act || 0, ...(inf.feature_acts_values || [0]));
      const total = (inf.feature_acts_values || []).reduce((a, b) => a + b, 0);
      return `<div class="card"><a href="#/dictionaries/${enc(name)}/features/${r.feature_index}">#${r.feature_index}</a>
        <span class="muted"> · summed activation ${fmt(total, 3)} · max over the data ${fmt(r.max_feature_act, 3)}</span>
        <div>${esc(interpretationOf(r)) || "<span class='muted'>no interpretation</span>"}</div>${renderSample(inf, m)}
        ${(r.samples || []).slice(0, 2).map(s => renderSample(s, r.max_feature_act, { window: 12, meta: "stored sample" })).join("")}</div>`;
    }).join("");
  } catch (e) { out.innerHTML = `<p class="err">${esc(e.message)}</p>`; }
}

// ---- bookmarks: paged, optionally of one dictionary, with the features' summaries ----
async function showBookmarks(skip = 0) {
  const page = 25;
  loading();
  try {
    const only = store.get("bookmarkDictionary", "");
    const b = await api("/bookmarks" + query({ limit: page, skip, include_features: true, sae_name: only }));
    let h = `<h1>Bookmarks <span class="muted">${b.total_count}</span></h1>
      <div class="row"><label>dictionary <select id="bmDict"><option value="">all</option>${[...$("dict").options].map(o =>
        `<option ${o.value === only ? "selected" : ""}>${esc(o.value)}</option>`).join("")}</select></label>
      <button id="bmPrev" ${skip ? "" : "disabled"}>← previous</button><button id="bmNext" ${skip + page < b.total_count ? "" : "disabled"}>next →</button></div>`;
    h += b.bookmarks.map(m => `<div class="card"><div class="row"><b>${esc(m.sae_name)}</b>
        ${(m.tags || []).map(t => `<span class="chip">${esc(t)}</span>`).join("")}<span class="muted">${esc((m.created_at || "").slice(0, 19).replace("T", " "))}</span>
        <button class="bmTags" data-d="${esc(m.sae_name)}" data-f="${m.feature_index}">tags / notes</button>
        <button class="unmark" data-d="${esc(m.sae_name)}" data-f="${m.feature_index}">remove</button></div>
        ${m.notes ? `<div>${esc(m.notes)}</div>` : ""}${featureSummary(m.feature, { dictionary: m.sae_name })}</div>`).join("") || "<p class='muted'>Nothing bookmarked yet.</p>";
    view.innerHTML = h;
    $("bmDict").onchange = () => { store.set("bookmarkDictionary", $("bmDict").value); showBookmarks(0); };
    $("bmPrev").onclick = () => showBookmarks(Math.max(0, skip - page));
    $("bmNext").onclick = () => showBookmarks(skip + page);
    view.querySelectorAll(".unmark").forEach(el => el.onclick = async () => {
      try { await api(`/dictionaries/${enc(el.dataset.d)}/features/${el.dataset.f}/bookmark`, { method: "DELETE" }); showBookmarks(skip); } catch (e) { fail(e); }
    });
    view.querySelectorAll(".bmTags").forEach(el => el.onclick = () => editBookmark(el.dataset.d, +el.dataset.f, () => showBookmarks(skip)));
  } catch (e) { fail(e); }
}
