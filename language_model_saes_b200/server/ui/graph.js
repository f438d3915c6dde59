// The attribution graph of a circuit as an SVG: one column per prompt token, one row per layer (embeddings at the bottom,
// attention and MLP dictionaries of each block above one another, logits on top), nodes of a cell side by side, links
// coloured by sign and as wide as their weight. Hovering snaps to the nearest node (a uniform grid over the node
// positions answers "what is near this point"); clicking selects a node, shift-clicking pins it. The reference project's
// counterparts are ui/src/components/circuits/link-graph/* (link-graph, nodes, links, grid-lines, row-backgrounds, y-axis,
// token-labels, tooltips) and ui/src/utils/circuit-index.ts (there an R-tree).

// ---- points in buckets of `cell` pixels; nearest(x, y, r) looks at the buckets the circle touches ----
class GridIndex {
  constructor(cell = 24) { this.cell = cell; this.buckets = new Map(); }
  key(cx, cy) { return cx + ":" + cy; }
  insert(x, y, item) {
    const k = this.key(Math.floor(x / this.cell), Math.floor(y / this.cell));
    if (!this.buckets.has(k)) this.buckets.set(k, []);
    this.buckets.get(k).push({ x, y, item });
  }
  nearest(x, y, r) {
    const c = this.cell, x0 = Math.floor((x - r) / c), x1 = Math.floor((x + r) / c), y0 = Math.floor((y - r) / c), y1 = Math.floor((y + r) / c);
    let best = null, bestD = r * r;
    for (let cx = x0; cx <= x1; cx++) for (let cy = y0; cy <= y1; cy++) {
      const b = this.buckets.get(this.key(cx, cy));
      if (!b) continue;
      for (const p of b) {
        const d = (p.x - x) * (p.x - x) + (p.y - y) * (p.y - y);
        if (d <= bestD) { bestD = d; best = p.item; }
      }
    }
    return best;
  }
}

const NODE_COLORS = { embedding: "#888", logit: "#36c", lorsa: "#d80", "cross layer transcoder": "#2a7", "lorsa error": "#b9a", "mlp reconstruction error": "#b9a", bias: "#bbb" };

function nodeLabel(n) {
  if (!n) return "";
  if (n.token !== null && n.token !== undefined) return (n.feature_type === "logit" ? "→ " : "") + JSON.stringify(n.token) + (n.token_prob !== null && n.token_prob !== undefined ? ` (p ${fmt(n.token_prob, 3)})` : "");
  const f = n.feature;
  if (f && typeof f === "object") return `#${f.feature_index} ${interpretationOf(f)}`.trim();
  return n.node_id;
}

function layerName(layer, maxLayer) {
  if (layer < 0) return "Emb";
  if (layer === maxLayer && layer % 2 === 0) return "Logit";
  return "L" + Math.floor(layer / 2) + (layer % 2 ? " M" : " A");  // even rows: attention dictionaries, odd rows: MLP transcoders
}

class LinkGraph {
  // host: element to draw into; g: {nodes, links, metadata.prompt_tokens}; on: {select(node|null), pin(node)}
  constructor(host, g, on = {}) {
    this.host = host; this.g = g; this.on = on;
    this.selected = null; this.pinned = new Set(); this.minWeight = 0;
    this.byId = new Map(g.nodes.map(n => [n.node_id, n]));
    this.inOf = new Map(); this.outOf = new Map();
    for (const l of g.links) {
      if (!this.inOf.has(l.target)) this.inOf.set(l.target, []);
      if (!this.outOf.has(l.source)) this.outOf.set(l.source, []);
      this.inOf.get(l.target).push(l); this.outOf.get(l.source).push(l);
    }
    this.layout();
    this.draw();
  }

  layout() {
    const g = this.g, tokens = (g.metadata || {}).prompt_tokens || [];
    this.layers = [...new Set(g.nodes.map(n => n.layer))].sort((a, b) => a - b);
    this.maxLayer = this.layers.length ? this.layers[this.layers.length - 1] : 0;
    const nctx = Math.max(tokens.length, ...g.nodes.map(n => n.ctx_idx + 1), 1);
    // nodes of one (layer, position) cell sit side by side, the most influential (largest total |weight|) first
    const strength = n => (this.inOf.get(n.node_id) || []).concat(this.outOf.get(n.node_id) || []).reduce((a, l) => a + Math.abs(l.weight), 0);
    const cells = new Map();
    for (const n of g.nodes) {
      const k = n.layer + ":" + n.ctx_idx;
      if (!cells.has(k)) cells.set(k, []);
      cells.get(k).push(n);
    }
    const perCol = new Array(nctx).fill(1);
    cells.forEach((list, k) => {
      list.sort((a, b) => strength(b) - strength(a));
      const c = +k.split(":")[1];
      perCol[c] = Math.max(perCol[c], Math.min(list.length, 8));
    });
    const step = 13, padL = 58, rowH = 46;
    this.colX = []; let x = padL;
    for (let c = 0; c < nctx; c++) { const w = Math.max(64, perCol[c] * step + 18); this.colX.push([x, w]); x += w; }
    this.W = x + 12;
    this.H = this.layers.length * rowH + 44;
    this.rowY = l => this.H - 36 - (this.layers.indexOf(l) + 0.5) * rowH;
    this.rowH = rowH;
    this.pos = new Map();
    this.index = new GridIndex(24);
    cells.forEach((list, k) => {
      const [l, c] = k.split(":").map(Number), [cx, cw] = this.colX[c], per = Math.min(list.length, 8);
      list.forEach((n, i) => {
        const px = cx + cw / 2 + ((i % per) - (per - 1) / 2) * step, py = this.rowY(l) + (Math.floor(i / per) - Math.floor((list.length - 1) / per) / 2) * step;
        this.pos.set(n.node_id, [px, py]);
        this.index.insert(px, py, n);
      });
    });
  }

  shape(n, p, cls) {
    const fill = NODE_COLORS[n.feature_type] || "#bbb", tip = esc(`${n.feature_type} · ${nodeLabel(n)}` + (n.activation !== undefined && n.activation !== null ? `\nactivation ${fmt(n.activation, 3)}` : "") + (n.is_from_qk_tracing ? "\n(only referenced by QK tracing)" : ""));
    const common = `class="node ${cls}" data-id="${esc(n.node_id)}" data-tip="${tip}" fill="${fill}"`;
    if (n.feature_type === "embedding" || n.feature_type === "logit") return `<rect ${common} x="${p[0] - 4.5}" y="${p[1] - 4.5}" width="9" height="9"${n.is_target_logit ? ' stroke="#000"' : ""}/>`;
    if (n.feature_type.endsWith("error")) return `<path ${common} d="M${p[0]},${p[1] - 5.5} L${p[0] + 5.5},${p[1]} L${p[0]},${p[1] + 5.5} L${p[0] - 5.5},${p[1]} Z"/>`;
    return `<circle ${common} cx="${p[0]}" cy="${p[1]}" r="${n.qk_tracing_results ? 5.5 : 4.5}"${n.is_from_qk_tracing ? ' opacity="0.55"' : ""}/>`;
  }

  draw() {
    const g = this.g, tokens = (g.metadata || {}).prompt_tokens || [], sel = this.selected;
    const near = new Set();
    if (sel) {
      near.add(sel);
      (this.inOf.get(sel) || []).forEach(l => near.add(l.source));
      (this.outOf.get(sel) || []).forEach(l => near.add(l.target));
    }
    const wmax = Math.max(1e-9, ...g.links.map(l => Math.abs(l.weight)));
    let s = `<svg width="${this.W}" height="${this.H}">`;
    this.layers.forEach((l, i) => {  // row backgrounds and the layer axis
      const y = this.rowY(l) - this.rowH / 2;
      s += `<rect x="0" y="${y}" width="${this.W}" height="${this.rowH}" fill="${i % 2 ? "#fafafa" : "#f1f3f6"}" stroke="none"/>`;
      s += `<text x="6" y="${this.rowY(l) + 4}" font-size="11" fill="#555">${layerName(l, this.maxLayer)}</text>`;
    });
    this.colX.forEach(([x, w], c) => {  // column separators and token labels
      s += `<line x1="${x}" y1="0" x2="${x}" y2="${this.H - 36}" stroke="#e2e2e2"/>`;
      const t = tokens[c] === undefined ? "" : String(tokens[c]);
      s += `<text x="${x + w / 2}" y="${this.H - 20}" text-anchor="middle" font-size="11" data-tip="${esc("position " + c + ": " + JSON.stringify(t))}">${esc(t.length > 9 ? t.slice(0, 8) + "…" : t)}</text>`;
      s += `<text x="${x + w / 2}" y="${this.H - 6}" text-anchor="middle" font-size="9" fill="#999">${c}</text>`;
    });
    for (const l of g.links) {
      const a = this.pos.get(l.source), b = this.pos.get(l.target);
      if (!a || !b || Math.abs(l.weight) < this.minWeight * wmax) continue;
      const hot = sel && (l.source === sel || l.target === sel), my = (a[1] + b[1]) / 2;
      s += `<path class="link${sel && !hot ? " dim" : ""}" d="M${a[0]},${a[1]} C${a[0]},${my} ${b[0]},${my} ${b[0]},${b[1]}" stroke-width="${(0.3 + 2.7 * Math.abs(l.weight) / wmax).toFixed(2)}"
        stroke="${l.weight >= 0 ? "#2a7" : "#c44"}" opacity="${hot ? 0.9 : 0.5}"/>`;
    }
    for (const n of g.nodes) {
      const p = this.pos.get(n.node_id);
      if (!p) continue;
      const cls = (n.node_id === sel ? "sel " : "") + (this.pinned.has(n.node_id) ? "pin " : "") + (sel && !near.has(n.node_id) ? "dim" : "");
      s += this.shape(n, p, cls);
    }
    const before = this.host.firstElementChild, scrollLeft = before ? before.scrollLeft : 0;  // a redraw keeps the view where it was
    this.host.innerHTML = `<div style="overflow:auto; max-width:100%">${s}</svg></div>`;
    this.host.firstElementChild.scrollLeft = scrollLeft;
    const svg = this.host.querySelector("svg");
    // the pointer snaps to the nearest node within 14 px, so that small nodes are easy to hit
    const pick = ev => {
      const r = svg.getBoundingClientRect();
      return this.index.nearest(ev.clientX - r.left, ev.clientY - r.top, 14);
    };
    svg.addEventListener("click", ev => {
      const n = pick(ev);
      if (n && ev.shiftKey) { this.togglePin(n.node_id); return; }
      this.select(n ? n.node_id : null);
    });
    svg.addEventListener("mousemove", ev => {
      const n = pick(ev);
      svg.style.cursor = n ? "pointer" : "default";
    });
  }

  select(id) {
    this.selected = id && this.byId.has(id) ? id : null;
    this.draw();
    if (this.on.select) this.on.select(this.selected ? this.byId.get(this.selected) : null);
  }

  togglePin(id) {
    if (this.pinned.has(id)) this.pinned.delete(id); else this.pinned.add(id);
    this.draw();
    if (this.on.pin) this.on.pin([...this.pinned].map(i => this.byId.get(i)));
  }

  setMinWeight(f) { this.minWeight = f; this.draw(); }

  // links into and out of a node, strongest first
  connections(id) {
    const by = (a, b) => Math.abs(b.weight) - Math.abs(a.weight);
    return { inputs: (this.inOf.get(id) || []).slice().sort(by), outputs: (this.outOf.get(id) || []).slice().sort(by) };
  }
}
