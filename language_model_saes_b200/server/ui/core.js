// Shared pieces of the browser: msgpack decoding, the REST helper, small HTML builders, the tooltip, dialogs and
// settings kept in the browser's local storage. Every other file of this folder uses these names. The reference
// project's counterparts are ui/src/api/*.ts (fetch + msgpack), ui/src/hooks/useLocalStorage.ts and ui/src/components/ui.

// ---- msgpack decoding (the subset the server emits: nil, bool, ints, floats, str, bin, array, map) ----
function unpack(buf) {
  const v = new DataView(buf), u8 = new Uint8Array(buf), td = new TextDecoder();
  let p = 0;
  const str = n => { const s = td.decode(u8.subarray(p, p + n)); p += n; return s; };
  const bin = n => { p += n; return u8.subarray(p - n, p); };
  const arr = n => { const a = new Array(n); for (let i = 0; i < n; i++) a[i] = rd(); return a; };
  const map = n => { const o = {}; for (let i = 0; i < n; i++) { const k = rd(); o[k] = rd(); } return o; };
  function rd() {
    const b = u8[p++];
    if (b < 0x80) return b;
    if (b >= 0xe0) return b - 256;
    if (b >= 0xa0 && b <= 0xbf) return str(b & 31);
    if (b >= 0x90 && b <= 0x9f) return arr(b & 15);
    if (b >= 0x80 && b <= 0x8f) return map(b & 15);
    switch (b) {
      case 0xc0: return null;
      case 0xc2: return false;
      case 0xc3: return true;
      case 0xc4: return bin(u8[p++]);
      case 0xc5: { const n = v.getUint16(p); p += 2; return bin(n); }
      case 0xc6: { const n = v.getUint32(p); p += 4; return bin(n); }
      case 0xca: p += 4; return v.getFloat32(p - 4);
      case 0xcb: p += 8; return v.getFloat64(p - 8);
      case 0xcc: return u8[p++];
      case 0xcd: p += 2; return v.getUint16(p - 2);
      case 0xce: p += 4; return v.getUint32(p - 4);
      case 0xcf: p += 8; return Number(v.getBigUint64(p - 8));
      case 0xd0: return v.getInt8(p++);
      case 0xd1: p += 2; return v.getInt16(p - 2);
      case 0xd2: p += 4; return v.getInt32(p - 4);
      case 0xd3: p += 8; return Number(v.getBigInt64(p - 8));
      case 0xd9: return str(u8[p++]);
      case 0xda: { const n = v.getUint16(p); p += 2; return str(n); }
      case 0xdb: { const n = v.getUint32(p); p += 4; return str(n); }
      case 0xdc: { const n = v.getUint16(p); p += 2; return arr(n); }
      case 0xdd: { const n = v.getUint32(p); p += 4; return arr(n); }
      case 0xde: { const n = v.getUint16(p); p += 2; return map(n); }
      case 0xdf: { const n = v.getUint32(p); p += 4; return map(n); }
    }
    throw new Error("unsupported msgpack byte 0x" + b.toString(16));
  }
  return rd();
}

// ---- REST ----
async function api(path, opts) {
  const r = await fetch(path, opts);
  if (!r.ok) throw new Error(r.status + " " + await r.text());
  if (r.status === 202) throw new Error("not ready yet: " + await r.text());
  return (r.headers.get("content-type") || "").includes("msgpack") ? unpack(await r.arrayBuffer()) : r.json();
}
const enc = encodeURIComponent;
const jsonOpts = (method, body) => ({ method, headers: { "content-type": "application/json" }, body: JSON.stringify(body) });
function query(params) {
  const parts = [];
  for (const k of Object.keys(params)) if (params[k] !== null && params[k] !== undefined && params[k] !== "") parts.push(enc(k) + "=" + enc(params[k]));
  return parts.length ? "?" + parts.join("&") : "";
}

// ---- HTML helpers ----
const $ = id => document.getElementById(id), view = $("view");
const ESC = { "&": "&amp;", "<": "&lt;", ">": "&gt;", '"': "&quot;" };
function esc(s) {
  let out = "";
  for (const c of String(s === null || s === undefined ? "" : s)) out += ESC[c] || c;
  return out;
}
const fail = e => { view.innerHTML = `<p class="err">${esc(e.message)}</p>`; };
const loading = () => { view.innerHTML = "<p class='muted'>Loading…</p>"; };
const table = (head, rows) => `<table><tr>${head.map(h => `<th>${esc(h)}</th>`).join("")}</tr>${rows.map(r => `<tr>${r.map(c => `<td>${c}</td>`).join("")}</tr>`).join("")}</table>`;
const fmt = (x, d = 3) => (x === null || x === undefined || Number.isNaN(+x)) ? "" : (+x).toFixed(d);
const count = x => (x || 0).toLocaleString();
function interpretationOf(f) { return ((f || {}).interpretation || {}).text || ""; }

// Bars of a histogram. h: {x: bin centres, y: counts} as the server's activation_histogram gives it, or a list of counts.
function histogram(h, W = 520, H = 120) {
  const y = Array.isArray(h) ? h : (h.y || h.counts || []);
  const x = Array.isArray(h) ? y.map((_, i) => i) : (h.x || h.bins || y.map((_, i) => i));
  if (!y.length) return "";
  const m = Math.max(1, ...y), bw = (W - 20) / y.length;
  let s = `<svg width="${W}" height="${H + 18}">`;
  y.forEach((v, i) => {
    const hh = (H - 6) * v / m;
    s += `<rect x="${10 + i * bw}" y="${H - hh}" width="${Math.max(1, bw - 1)}" height="${hh}" fill="#69c"><title>${esc(fmt(x[i], 2))}: ${v}</title></rect>`;
  });
  return s + `<text x="10" y="${H + 14}" font-size="11">${esc(fmt(x[0], 2))}</text><text x="${W - 10}" y="${H + 14}" font-size="11" text-anchor="end">${esc(fmt(x[x.length - 1], 2))}</text></svg>`;
}

// ---- tooltip that follows the pointer: any element with a data-tip attribute ----
const tipBox = $("tip");
document.addEventListener("mousemove", ev => {
  const el = ev.target.closest ? ev.target.closest("[data-tip]") : null;
  if (!el) { tipBox.hidden = true; return; }
  tipBox.textContent = el.dataset.tip;
  tipBox.hidden = false;
  tipBox.style.left = Math.min(ev.clientX + 14, window.innerWidth - 380) + "px";
  tipBox.style.top = (ev.clientY + 16) + "px";
});

// ---- modal dialog: body is HTML; returns the element so that the caller can wire its controls; close() removes it ----
function openDialog(html) {
  const wrap = document.createElement("div");
  wrap.className = "dialog";
  wrap.innerHTML = `<div>${html}</div>`;
  wrap.addEventListener("mousedown", ev => { if (ev.target === wrap) wrap.remove(); });
  document.body.appendChild(wrap);
  wrap.close = () => wrap.remove();
  return wrap;
}

// ---- settings that survive a reload (thresholds, visible range, last dictionary) ----
const store = {
  get(key, fallback) {
    try { const v = localStorage.getItem("lmsae." + key); return v === null ? fallback : JSON.parse(v); } catch (e) { return fallback; }
  },
  set(key, value) { try { localStorage.setItem("lmsae." + key, JSON.stringify(value)); } catch (e) { /* private mode: keep going without it */ } },
};

// ---- debounce: run fn once the calls have stopped for ms ----
function debounce(fn, ms) {
  let t = null;
  return (...args) => { clearTimeout(t); t = setTimeout(() => fn(...args), ms); };
}

function selectOption(id, value) {
  const sel = $(id);
  if (![...sel.options].some(o => o.value === value)) sel.add(new Option(value, value));  // lists still loading, or an id that is not listed
  sel.value = value;
}
