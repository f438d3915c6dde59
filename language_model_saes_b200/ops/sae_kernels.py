"""Python entry points of the sm_100a kernels, each paired with a plain PyTorch definition.

The ``ref_*`` functions state the math of each kernel in fp32 PyTorch. They are the oracles of the GPU
numerics tests and what the CPU code paths run. On a CUDA device the kernel wrappers call the compiled
extension (``ops/native.py``) and raise if it is missing.

Layouts shared by all kernels: encoder and decoder weights are feature-major ``[F, d]``; sparse codes are
``(idx int32 [B, k], val fp32 [B, k])`` with ``idx == -1`` marking an empty slot.
"""

from __future__ import annotations

import os

import torch

from . import native

NUM_SMS_B200 = 148

_status_buffers: dict[torch.device, torch.Tensor] = {}


class KernelStatusError(RuntimeError):
    """A kernel reported a bounded-wait expiry or a bad argument through its status word. ``code`` is the status code
    (5 = a peer's flag did not arrive in time: a collective timed out)."""

    code: int = 0


class CollectiveTimeout(KernelStatusError):
    """A bounded wait on another GPU's flag ran out: the peer is late, stuck or gone. The kernels involved have left
    through their normal exit and the context is usable; the data of that step is not."""


_STATUS_NAMES = {
    1: "timeout waiting for a TMA stage (full barrier)",
    2: "timeout waiting for a free smem stage (empty barrier)",
    3: "timeout waiting for an accumulator (tmem full)",
    4: "timeout waiting for the epilogue (tmem empty)",
    5: "timeout waiting for a peer flag",
    6: "bad argument",
    7: "capacity overflow",
}


class _Counting:
    """Proxy of the extension module that counts the device kernels each entry point launches."""

    KERNELS_PER_CALL = {"csc_build": 5, "exclusive_scan": 3}

    def __init__(self, mod):
        self._mod = mod
        self.launches = 0

    def __getattr__(self, name):
        fn = getattr(self._mod, name)
        n = self.KERNELS_PER_CALL.get(name, 1)

        def call(*args, **kwargs):
            self.launches += n
            return fn(*args, **kwargs)

        self.__dict__[name] = call
        return call


_counting: _Counting | None = None


def _ext():
    global _counting
    if _counting is None:
        _counting = _Counting(native.load(required=True))
    return _counting


def kernel_launch_count() -> int:
    """Number of kernels of this package launched so far in this process."""
    return _counting.launches if _counting is not None else 0


def status_buffer(device: torch.device) -> torch.Tensor:
    device = torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    buf = _status_buffers.get(device)
    if buf is None:
        buf = torch.zeros(4, dtype=torch.int32, device=device)
        _status_buffers[device] = buf
    return buf


def check_status(device: torch.device) -> None:
    """Synchronising read of the status word; raises if any kernel on ``device`` recorded an error."""
    buf = status_buffer(device)
    vals = buf.tolist()
    if vals[0] != 0:
        buf.zero_()
        err = (CollectiveTimeout if vals[0] == 5 else KernelStatusError)(
            f"kernel status {vals[0]} ({_STATUS_NAMES.get(vals[0], 'unknown')}), detail={vals[1]}, block={vals[2]}, aux={vals[3]}"
        )
        err.code = vals[0]
        raise err


GEMM_PAIR_DEFAULT = os.environ.get("LMSAE_GEMM_PAIR", "1") == "1"


def choose_splits(M: int, N: int, num_sms: int = NUM_SMS_B200) -> int:
    """How many CTAs share one 128-row panel of the encoder GEMM (each sweeps a range of 256-column tiles)."""
    panels = (M + 127) // 128
    n_tiles = (N + 255) // 256
    return max(1, min(n_tiles, num_sms // max(panels, 1)))


def choose_units(M: int, N: int, pair: bool, num_sms: int = NUM_SMS_B200) -> tuple[int, int]:
    """Ragged deal of the encoder GEMM's work: ``(units, num_splits)``. A unit is one CTA, or one CTA pair covering two
    adjacent 128-row panels; with ``P`` panel units and room for ``Q`` units on the GPU every panel unit sweeps
    ``Q // P`` column ranges and the first ``Q % P`` of them one more, so that batch sizes whose panel count does not
    divide the SM count (4096 rows = 16 pairs on 74 SM pairs) still occupy every SM. ``num_splits`` is the larger count
    (it sizes the candidate lists). ``units == 0``: the uniform deal of ``choose_splits`` is already full or the only
    one possible."""
    panels = (M + 127) // 128
    if pair and panels % 2:
        pair = False
    P = panels // 2 if pair else panels
    Q = num_sms // 2 if pair else num_sms
    n_tiles = (N + 255) // 256
    uniform = choose_splits(M, N, num_sms)
    if P >= Q or Q % P == 0:
        return 0, uniform
    base, extra = Q // P, Q % P
    if base + 1 > n_tiles:
        return 0, min(uniform, n_tiles)
    return Q, base + 1


def candidate_slots(k: int) -> int:
    return 32 if k <= 32 else 64


# --------------------------------------------------------------------------------------------------
# encoder
# --------------------------------------------------------------------------------------------------
def ref_hidden(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None) -> torch.Tensor:
    h = x.float() @ w.float().t()
    if bias is not None:
        h = h + bias.float()
    return h


def ref_topk_codes(
    h: torch.Tensor, k: int, gate: torch.Tensor | None = None, alive: torch.Tensor | None = None
) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-row top-k of the positive gated values; returns (idx int32, act fp32 = h at the winners)."""
    g = h.float()
    if gate is not None:
        g = g * gate.float()
    if alive is not None:
        g = g * alive.to(g.dtype)
    g = torch.where(g > 0, g, torch.zeros_like(g))
    k_eff = min(k, g.shape[-1])
    vals, idx = torch.topk(g, k_eff, dim=-1)
    if k_eff < k:
        pad = k - k_eff
        vals = torch.cat([vals, vals.new_zeros(*vals.shape[:-1], pad)], dim=-1)
        idx = torch.cat([idx, idx.new_zeros(*idx.shape[:-1], pad)], dim=-1)
    keep = vals > 0
    act = vals
    if gate is not None:
        act = vals / gate.float()[idx.clamp_min(0)]
    act = torch.where(keep, act, torch.zeros_like(act))
    idx = torch.where(keep, idx, torch.full_like(idx, -1))
    return idx.to(torch.int32), act


def _pair_bit(pair: bool | None) -> int:
    """Mode bit 3 of the encoder GEMM: run on CTA pairs (tcgen05 cta_group::2). The extension falls back to the
    single-CTA kernel by itself when the batch is not a whole number of 256-row panel pairs."""
    use = GEMM_PAIR_DEFAULT if pair is None else pair
    return 8 if use else 0


def encoder_hidden(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, pair: bool | None = None,
                   gate: torch.Tensor | None = None) -> torch.Tensor:  # fmt: skip
    """H = x @ w.T + bias as bf16 via the tcgen05 GEMM (x [M,K] bf16, w [N,K] bf16, bias fp32); with ``gate`` (fp32 [N])
    the stored value is ``H * gate`` (gated pre-activations)."""
    if not x.is_cuda:
        h = ref_hidden(x, w, bias)
        return (h * gate if gate is not None else h).to(torch.bfloat16)
    M, N = x.shape[0], w.shape[0]
    H = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    units, S = _deal(M, N, pair, None)
    _ext().encoder_gemm(x, w, bias, gate, 1 | _pair_bit(pair), 0, S, H, None, None, status_buffer(x.device), 0, False, units)
    return H


def _deal(M: int, N: int, pair: bool | None, num_splits: int | None) -> tuple[int, int]:
    """(units, num_splits) of an encoder GEMM launch: the uniform deal of ``choose_splits`` (or an explicit
    ``num_splits``) unless ``LMSAE_GEMM_RAGGED=1`` asks for the ragged one. Measured at batch 4096 x 131072 features the
    ragged deal (148 instead of 128 SMs busy) is SLOWER, 3.20 against 2.95 ms: the kernel runs at the power cap either
    way, and panels that sweep different column ranges no longer share their B tiles in L2."""
    if num_splits:
        return 0, num_splits
    if os.environ.get("LMSAE_GEMM_RAGGED", "0") != "1":
        return 0, choose_splits(M, N)
    return choose_units(M, N, bool(_pair_bit(pair)))


def encoder_topk_candidates(
    x: torch.Tensor,
    w: torch.Tensor,
    bias: torch.Tensor | None,
    gate: torch.Tensor | None,
    k: int,
    num_splits: int | None = None,
    H: torch.Tensor | None = None,
    pair: bool | None = None,
    n_index_offset: int = 0,
    resume: tuple[torch.Tensor, torch.Tensor] | None = None,
    compact_smem: bool = False,
) -> tuple[torch.Tensor, torch.Tensor, int]:
    """Run the GEMM with the fused top-k epilogue; returns (cand_val [M, C], cand_idx [M, C], C).

    A dictionary can be swept in several calls, one per chunk of its rows: pass the chunk as ``w`` (with the matching
    slices of ``bias`` / ``gate``), its first row as ``n_index_offset`` and, from the second chunk on, the previous
    call's ``(cand_val, cand_idx)`` as ``resume``; the buffers are updated in place and the result equals one sweep."""
    M, N = x.shape[0], w.shape[0]
    units, S = _deal(M, N, pair, num_splits)
    KS = candidate_slots(k)
    C = S * KS
    if resume is not None:
        cand_val, cand_idx = resume
        assert cand_val.shape == (M, C) and cand_idx.shape == (M, C), "resume buffers do not match this launch's splits"
    else:
        cand_val = torch.empty(M, C, dtype=torch.float32, device=x.device)
        cand_idx = torch.empty(M, C, dtype=torch.int32, device=x.device)
    mode = 2 | (1 if H is not None else 0) | _pair_bit(pair) | (16 if compact_smem else 0)
    _ext().encoder_gemm(x, w, bias, gate, mode, k, S, H, cand_val, cand_idx, status_buffer(x.device), n_index_offset, resume is not None,
                        units)  # fmt: skip
    return cand_val, cand_idx, C


def ref_topk_merge(cand_val, cand_idx, k: int, gate, own: tuple[int, int] | None = None, emit_gated: bool = False):
    """Plain-torch statement of ``topk_merge`` (any device): the ``k`` largest positive candidates of every row; only
    winners whose candidate slot lies in ``own`` are kept, packed in value-descending order from slot 0 on (the rest of
    the row is -1 / 0); values divided by ``gate[idx]`` unless ``emit_gated``."""
    M, C = cand_val.shape
    lo, hi = own if own is not None else (0, C)
    score = torch.where(cand_idx >= 0, cand_val.float(), torch.full_like(cand_val, -1.0, dtype=torch.float32))
    kk = min(k, C)
    top, pos = torch.topk(score, kk, dim=-1)
    keep = (top > 0) & (pos >= lo) & (pos < hi)
    idx = torch.where(keep, torch.gather(cand_idx, 1, pos), torch.full_like(pos, -1, dtype=cand_idx.dtype))
    val = torch.where(keep, top, torch.zeros_like(top))
    if not emit_gated and gate is not None:
        val = torch.where(keep, val / gate.float()[idx.clamp_min(0).long()], val)
    # pack the kept entries to the front, order preserved
    order = torch.sort((~keep).to(torch.int8), dim=1, stable=True).indices
    idx, val = torch.gather(idx, 1, order), torch.gather(val, 1, order)
    if kk < k:
        idx = torch.cat([idx, idx.new_full((M, k - kk), -1)], dim=1)
        val = torch.cat([val, val.new_zeros(M, k - kk)], dim=1)
    return idx.to(torch.int32), val


def topk_merge(
    cand_val: torch.Tensor,
    cand_idx: torch.Tensor,
    k: int,
    gate: torch.Tensor | None,
    own: tuple[int, int] | None = None,
    emit_gated: bool = False,
) -> tuple[torch.Tensor, torch.Tensor]:
    M, C = cand_val.shape
    lo, hi = own if own is not None else (0, C)
    if not cand_val.is_cuda:
        return ref_topk_merge(cand_val, cand_idx, k, gate, own, emit_gated)
    out_idx = torch.empty(M, k, dtype=torch.int32, device=cand_val.device)
    out_val = torch.empty(M, k, dtype=torch.float32, device=cand_val.device)
    _ext().topk_merge(cand_val, cand_idx, M, C, k, gate, lo, hi, emit_gated, out_idx, out_val, 0, [], 0, None, None)
    return out_idx, out_val


def encoder_topk(
    x: torch.Tensor,
    w: torch.Tensor,
    bias: torch.Tensor | None,
    gate: torch.Tensor | None,
    k: int,
    return_hidden: bool = False,
    pair: bool | None = None,
) -> tuple[torch.Tensor, torch.Tensor] | tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Sparse codes of a TopK encoder: (idx [M,k], act [M,k]) (+ hidden_pre bf16 when asked).

    ``k <= 64`` uses the GEMM's fused top-k epilogue (the dense pre-activations are never written unless
    ``return_hidden``); larger k materialises H and selects with the radix row-top-k kernel.
    """
    if not x.is_cuda:
        h = ref_hidden(x, w, bias)
        idx, act = ref_topk_codes(h, k, gate)
        return (idx, act, h.to(torch.bfloat16)) if return_hidden else (idx, act)
    M, N = x.shape[0], w.shape[0]
    H = torch.empty(M, N, dtype=torch.bfloat16, device=x.device) if (return_hidden or k > 64) else None
    if k <= 64:
        cv, ci, _ = encoder_topk_candidates(x, w, bias, gate, k, H=H, pair=pair)
        idx, act = topk_merge(cv, ci, k, gate)
    else:
        units, S = _deal(M, N, pair, None)
        _ext().encoder_gemm(x, w, bias, None, 1 | _pair_bit(pair), 0, S, H, None, None, status_buffer(x.device), 0, False, units)
        idx, act = row_topk(H, k, gate, None)
    return (idx, act, H) if return_hidden else (idx, act)


def row_topk(
    H: torch.Tensor, k: int, gate: torch.Tensor | None = None, alive: torch.Tensor | None = None
) -> tuple[torch.Tensor, torch.Tensor]:
    if not H.is_cuda:
        return ref_topk_codes(H.float(), k, gate, alive)
    M = H.shape[0]
    out_idx = torch.empty(M, k, dtype=torch.int32, device=H.device)
    out_val = torch.empty(M, k, dtype=torch.float32, device=H.device)
    alive_u8 = alive.to(torch.uint8).contiguous() if alive is not None else None
    _ext().row_topk(H.contiguous(), k, gate, alive_u8, out_idx, out_val)
    return out_idx, out_val


# --------------------------------------------------------------------------------------------------
# decoder
# --------------------------------------------------------------------------------------------------
def ref_sparse_decode(idx: torch.Tensor, val: torch.Tensor, W: torch.Tensor, bias: torch.Tensor | None) -> torch.Tensor:
    safe = idx.clamp_min(0).long()
    rows = W.float()[safe]  # [B, k, d]
    coef = torch.where(idx >= 0, val.float(), torch.zeros_like(val, dtype=torch.float32))
    out = (rows * coef.unsqueeze(-1)).sum(dim=1)
    if bias is not None:
        out = out + bias.float()
    return out


def sparse_decode(
    idx: torch.Tensor, val: torch.Tensor, W: torch.Tensor, bias: torch.Tensor | None, out_dtype: torch.dtype = torch.float32
) -> torch.Tensor:
    if not idx.is_cuda:
        return ref_sparse_decode(idx, val, W, bias).to(out_dtype)
    B, d = idx.shape[0], W.shape[1]
    out = torch.empty(B, d, dtype=out_dtype, device=idx.device)
    f32 = out if out_dtype == torch.float32 else None
    b16 = out if out_dtype == torch.bfloat16 else None
    assert f32 is not None or b16 is not None, "out_dtype must be float32 or bfloat16"
    _ext().sparse_decode(idx, val, W, bias, f32, b16, None, None, 0.0, None, None, None, None)
    return out


def ref_decode_loss(idx, val, W, bias, label, row_weight, grad_scale):
    xhat = ref_sparse_decode(idx, val, W, bias)
    e = xhat - label.float()
    row_loss = (e * e).sum(-1)
    rw = row_weight.float() if row_weight is not None else torch.ones_like(row_loss)
    loss_sum = (row_loss * rw).sum()
    dxhat = (e * grad_scale * rw.unsqueeze(-1)).to(torch.bfloat16)
    safe = idx.clamp_min(0).long()
    dval = torch.einsum("bd,bkd->bk", dxhat.float(), W.float()[safe])
    dval = torch.where(idx >= 0, dval, torch.zeros_like(dval))
    return xhat, dxhat, loss_sum, row_loss, dval


def sparse_decode_loss(
    idx: torch.Tensor,
    val: torch.Tensor,
    W: torch.Tensor,
    bias: torch.Tensor | None,
    label: torch.Tensor,
    row_weight: torch.Tensor | None,
    grad_scale: float,
    loss_sum: torch.Tensor,
    want_dval: bool = True,
    want_xhat: bool = False,
    row_loss: torch.Tensor | None = None,
):
    """Decode, accumulate sum_b w_b * ||x_hat_b - label_b||^2 into ``loss_sum`` and return
    (dxhat bf16, dval fp32 | None, xhat fp32 | None)."""
    B, k = idx.shape
    d = W.shape[1]
    dxhat = torch.empty(B, d, dtype=torch.bfloat16, device=idx.device)
    dval = torch.empty(B, k, dtype=torch.float32, device=idx.device) if want_dval else None
    xhat = torch.empty(B, d, dtype=torch.float32, device=idx.device) if want_xhat else None
    if not idx.is_cuda:
        xh, dx, ls, rl, dv = ref_decode_loss(idx, val, W, bias, label, row_weight, grad_scale)
        loss_sum += ls
        if row_loss is not None:
            row_loss.copy_(rl)
        return dx, (dv if want_dval else None), (xh if want_xhat else None)
    _ext().sparse_decode(idx, val, W, bias, xhat, None, label, row_weight, grad_scale, dxhat, loss_sum, row_loss, dval)
    return dxhat, dval, xhat


def sparse_dact(idx: torch.Tensor, W: torch.Tensor, dxhat: torch.Tensor) -> torch.Tensor:
    if not idx.is_cuda:
        safe = idx.clamp_min(0).long()
        dv = torch.einsum("bd,bkd->bk", dxhat.float(), W.float()[safe])
        return torch.where(idx >= 0, dv, torch.zeros_like(dv))
    dval = torch.empty(idx.shape, dtype=torch.float32, device=idx.device)
    _ext().sparse_dact(idx, W, dxhat, dval, [], 0, None)
    return dval


def mse_loss_grad(xhat, label, bias, row_weight, grad_scale, loss_sum, row_loss=None):
    """dxhat (bf16) and loss accumulation for dense fp32 rows (x_hat optionally still missing its bias)."""
    if not xhat.is_cuda:
        xh = xhat + (bias if bias is not None else 0.0)
        e = xh - label.float()
        rl = (e * e).sum(-1)
        rw = row_weight.float() if row_weight is not None else torch.ones_like(rl)
        loss_sum += (rl * rw).sum()
        if row_loss is not None:
            row_loss.copy_(rl)
        return (e * grad_scale * rw.unsqueeze(-1)).to(torch.bfloat16)
    dxhat = torch.empty(xhat.shape, dtype=torch.bfloat16, device=xhat.device)
    _ext().mse_loss_grad(xhat, label, bias, row_weight, grad_scale, dxhat, loss_sum, row_loss)
    return dxhat


def auxk_loss_grad(xhat, aux_rec, label, bias, row_weight, grad_scale, alpha, loss_sum, aux_sum, alpha_factor=None):
    """Main and auxiliary (dead-feature) reconstruction losses and their output gradients for fp32 rows:
    ``e = label - (xhat + bias)``, ``r = e - aux_rec``; accumulates ``sum rw * |e|^2`` into ``loss_sum`` and
    ``alpha * sum rw * |r|^2`` into ``aux_sum``; returns bf16 ``(g_main, g_aux)`` with
    ``g_main = -(e + alpha r) * grad_scale * rw`` and ``g_aux = -alpha r * grad_scale * rw``. ``alpha_factor``: optional
    one-element fp32 device tensor that multiplies ``alpha`` (0 switches the auxiliary term off without a host read)."""
    if not xhat.is_cuda:
        if alpha_factor is not None:
            alpha = alpha * float(alpha_factor)
        xh = xhat + (bias if bias is not None else 0.0)
        e = label.float() - xh
        r = e - aux_rec
        rw = row_weight.float() if row_weight is not None else torch.ones(xhat.shape[0])
        loss_sum += ((e * e).sum(-1) * rw).sum()
        aux_sum += alpha * ((r * r).sum(-1) * rw).sum()
        sc = (grad_scale * rw).unsqueeze(-1)
        return (-(e + alpha * r) * sc).to(torch.bfloat16), (-alpha * r * sc).to(torch.bfloat16)
    g_main = torch.empty(xhat.shape, dtype=torch.bfloat16, device=xhat.device)
    g_aux = torch.empty_like(g_main)
    _ext().auxk_loss_grad(xhat, aux_rec, label, bias, row_weight, grad_scale, alpha, g_main, g_aux, loss_sum, aux_sum, alpha_factor)
    return g_main, g_aux


# --------------------------------------------------------------------------------------------------
# backward / optimizer
# --------------------------------------------------------------------------------------------------
class FeatureGroups:
    """(row, slot) pairs grouped by feature: ``entries[offsets[f]:offsets[f+1]]`` are flat positions
    ``row * k + slot`` whose code index is ``f``. Buffers are reused across steps."""

    def __init__(self, F: int, capacity: int, device: torch.device):
        self.F = F
        self.counts = torch.zeros(F, dtype=torch.int32, device=device)
        self.offsets = torch.zeros(F + 1, dtype=torch.int32, device=device)
        self.cursor = torch.zeros(F, dtype=torch.int32, device=device)
        self.entries = torch.zeros(capacity, dtype=torch.int32, device=device)
        self.block_sums = torch.zeros((F + 4095) // 4096, dtype=torch.int32, device=device)

    def build(self, idx: torch.Tensor) -> "FeatureGroups":
        n = idx.numel()
        if self.entries.numel() < n:
            self.entries = torch.zeros(n, dtype=torch.int32, device=idx.device)
        if idx.is_cuda:
            _ext().csc_build(idx, self.F, self.counts, self.offsets, self.cursor, self.entries, self.block_sums)
        else:
            flat = idx.reshape(-1)
            valid = flat >= 0
            order = torch.argsort(torch.where(valid, flat, torch.full_like(flat, self.F)), stable=True)
            nvalid = int(valid.sum())
            self.entries[:nvalid] = order[:nvalid].to(torch.int32)
            counts = torch.bincount(flat[valid].long(), minlength=self.F)
            self.counts.copy_(counts.to(torch.int32))
            self.offsets[0] = 0
            self.offsets[1:] = torch.cumsum(counts, 0).to(torch.int32)
        return self


def ref_sparse_grads(idx, act, dact, x, dxhat, F):
    """Dense fp32 gradients (dW_D [F,d], dW_E^T [F,d], db_E [F]) of the sparse codes, for tests / CPU."""
    B, k = idx.shape
    d = x.shape[1]
    flat = idx.reshape(-1).long()
    valid = flat >= 0
    rows = torch.arange(B, device=idx.device).repeat_interleave(k)[valid]
    f = flat[valid]
    a = act.reshape(-1)[valid].float()
    da = dact.reshape(-1)[valid].float()
    gD = torch.zeros(F, d, dtype=torch.float32, device=idx.device)
    gE = torch.zeros(F, d, dtype=torch.float32, device=idx.device)
    gb = torch.zeros(F, dtype=torch.float32, device=idx.device)
    gD.index_add_(0, f, a.unsqueeze(1) * dxhat.float()[rows])
    gE.index_add_(0, f, da.unsqueeze(1) * x.float()[rows])
    gb.index_add_(0, f, da)
    return gD, gE, gb


def ref_adam(p, g, m, v, lr, beta1, beta2, eps, step):
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1 = 1 - beta1**step
    bc2 = 1 - beta2**step
    denom = v.sqrt() / (bc2**0.5) + eps
    p.addcdiv_(m, denom, value=-lr / bc1)


def sparse_grad_adam(
    groups: FeatureGroups,
    act,
    dact,
    x,
    dxhat,
    WD,
    mD,
    vD,
    WD_bf16,
    WE,
    mE,
    vE,
    WE_bf16,
    bE,
    mbE,
    vbE,
    dec_norm,
    grad_mul,
    grad_sq_sum,
    lr,
    beta1,
    beta2,
    eps,
    step,
    update=True,
    f_range: tuple[int, int] | None = None,
    ctas_per_sm: int = 0,
    dxhat_aux=None,
    k_main: int = 0,
    grad_out: tuple[torch.Tensor | None, torch.Tensor | None] = (None, None),
    state_f0: int = 0,
    publish: tuple[list[int], list[int], int, torch.Tensor] | None = None,
    extra: tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor | None] | None = None,
    wd_self_scale: torch.Tensor | None = None,
    norm_sq_accum: torch.Tensor | None = None,
):
    """Rebuild the two sparse gradient rows per feature and apply Adam in the same pass (in place). ``f_range``
    restricts the launch to feature rows ``[begin, end)``. With ``dxhat_aux`` the code slots ``>= k_main`` of every row
    take their output gradient from that matrix instead of ``dxhat`` (auxiliary codes). ``state_f0``: the moment arrays
    start at that feature row (optimizer state sharded by feature row). ``publish`` = ``DataParallelComm.pub_args()``:
    the new shadow rows, norms and biases are stored into every replica's copy. ``extra`` = ``(row_of_feature int32 [F],
    gD fp32 [R, d], gE fp32 [R, d], gb fp32 [R] | None)``: dense gradient rows that are added for the features with
    ``row_of_feature >= 0`` (e.g. the auxiliary loss over a compact dictionary of dead features). ``wd_self_scale`` fp32
    ``[F]``: the decoder row's gradient gets ``wd_self_scale[f] * W_D[f, :]`` added (the gradient that a penalty on the
    row's norm sends into the row). One-sided launches: pass ``WD = mD = vD = WD_bf16 = None`` to update the encoder side
    only, or the ``WE`` group as None for the decoder side only. ``norm_sq_accum`` fp32 ``[F]``: the squared norm of every
    new decoder row is ADDED there instead of writing ``dec_norm``. A non-zero kernel status word turns the update into
    a no-op (CUDA path)."""
    ref_w = WD if WD is not None else WE
    if not ref_w.is_cuda:
        if WD is None or WE is None:  # one-sided: run the two-sided statement on a scratch copy of the missing side
            zero = lambda: torch.zeros_like(ref_w)  # noqa: E731
            if WD is None:
                sparse_grad_adam(groups, act, dact, x, dxhat, zero(), zero(), zero(), torch.zeros_like(WE_bf16), WE, mE, vE, WE_bf16, bE, mbE,
                                 vbE, None, grad_mul, None, lr, beta1, beta2, eps, step, update, f_range, 0, dxhat_aux, k_main,
                                 state_f0=state_f0, extra=extra)  # fmt: skip
            else:
                norms = torch.zeros(ref_w.shape[0]) if (dec_norm is not None or norm_sq_accum is not None) else None
                sparse_grad_adam(groups, act, dact, x, dxhat, WD, mD, vD, WD_bf16, zero(), zero(), zero(), torch.zeros_like(WD_bf16), None,
                                 None, None, norms, grad_mul, None, lr, beta1, beta2, eps, step, update, f_range, 0, dxhat_aux,
                                 k_main, state_f0=state_f0, extra=extra, wd_self_scale=wd_self_scale)  # fmt: skip
                if norm_sq_accum is not None and update:
                    norm_sq_accum += norms.square()
                elif dec_norm is not None and update:
                    dec_norm.copy_(norms)
            return
        if f_range is not None and tuple(f_range) != (0, groups.F):
            lo, hi = f_range
            sub = FeatureGroups.__new__(FeatureGroups)
            sub.F = hi - lo
            sub.offsets, sub.entries = groups.offsets[lo : hi + 1], groups.entries
            sl = slice(lo, hi)
            st = slice(lo - state_f0, hi - state_f0)
            sub_extra = (extra[0][sl], *extra[1:]) if extra is not None else None
            sparse_grad_adam(sub, act, dact, x, dxhat, WD[sl], mD[st], vD[st], WD_bf16[sl], WE[sl], mE[st], vE[st], WE_bf16[sl],
                             bE[sl] if bE is not None else None, mbE[st] if mbE is not None else None,
                             vbE[st] if vbE is not None else None, dec_norm[sl] if dec_norm is not None else None, grad_mul,
                             grad_sq_sum, lr, beta1, beta2, eps, step, update, None, 0, dxhat_aux, k_main, extra=sub_extra,
                             wd_self_scale=wd_self_scale[sl] if wd_self_scale is not None else None)  # fmt: skip
            return
        idx_like = torch.full((act.numel(),), -1, dtype=torch.int64)
        off = groups.offsets.long()
        n_ent = int(off[groups.F] - off[0])
        owner = torch.repeat_interleave(torch.arange(groups.F), (off[1 : groups.F + 1] - off[:groups.F]))
        idx_like[groups.entries[int(off[0]) : int(off[0]) + n_ent].long()] = owner
        idx_like = idx_like.reshape(act.shape)
        if dxhat_aux is None:
            gD, gE, gb = ref_sparse_grads(idx_like, act, dact, x, dxhat, groups.F)
        else:
            parts = [ref_sparse_grads(idx_like[:, sl], act[:, sl], dact[:, sl], x, g, groups.F)
                     for sl, g in ((slice(0, k_main), dxhat), (slice(k_main, None), dxhat_aux))]  # fmt: skip
            gD, gE, gb = (a + b for a, b in zip(*parts))
        if extra is not None:
            row_of, xD, xE, xb = extra
            sel = (row_of >= 0).nonzero().squeeze(-1)
            r = row_of[sel].long()
            if xD is not None:
                gD[sel] += xD[r]
            if xE is not None:
                gE[sel] += xE[r]
            if xb is not None:
                gb[sel] += xb[r]
        mul = float(grad_mul) if grad_mul is not None else 1.0
        gD, gE, gb = gD * mul, gE * mul, gb * mul
        if grad_sq_sum is not None:
            grad_sq_sum += gD.pow(2).sum() + gE.pow(2).sum() + gb.pow(2).sum()
        if wd_self_scale is not None:
            gD = gD + (wd_self_scale * mul).unsqueeze(1) * WD
        if update:
            ref_adam(WD, gD, mD, vD, lr, beta1, beta2, eps, step)
            ref_adam(WE, gE, mE, vE, lr, beta1, beta2, eps, step)
            if bE is not None:
                ref_adam(bE, gb, mbE, vbE, lr, beta1, beta2, eps, step)
            WD_bf16.copy_(WD)
            WE_bf16.copy_(WE)
            if dec_norm is not None:
                dec_norm.copy_(WD.norm(dim=1))
        return
    _ext().sparse_grad_adam(
        groups.offsets, groups.entries, act, dact, x, dxhat, WD, mD, vD, WD_bf16, WE, mE, vE, WE_bf16, bE, mbE, vbE,
        dec_norm, grad_mul, grad_sq_sum, lr, beta1, beta2, eps, step, update, *(f_range if f_range is not None else (0, -1)), ctas_per_sm, dxhat_aux, k_main, grad_out[0], grad_out[1],
        status_buffer(ref_w.device), state_f0, *(publish if publish is not None else ([], [], 0, None)),
        *(extra if extra is not None else (None, None, None, None)), wd_self_scale, norm_sq_accum,
    )  # fmt: skip


def colsum_bf16(a: torch.Tensor) -> torch.Tensor:
    if not a.is_cuda:
        return a.float().sum(0)
    out = torch.empty(a.shape[1], dtype=torch.float32, device=a.device)
    _ext().colsum_bf16(a, out)
    return out


def adam_flat(p, g, m, v, lr, beta1, beta2, eps, step, grad_mul=None, shadow=None, grad_sq_sum=None, update=True):
    if not p.is_cuda:
        gg = g * (float(grad_mul) if grad_mul is not None else 1.0)
        if grad_sq_sum is not None:
            grad_sq_sum += gg.pow(2).sum()
        if update:
            ref_adam(p, gg, m, v, lr, beta1, beta2, eps, step)
            if shadow is not None:
                shadow.copy_(p)
        return
    _ext().adam_flat(p, g, m, v, grad_mul, shadow, grad_sq_sum, lr, beta1, beta2, eps, step, update, status_buffer(p.device))


def row_norm_shadow(W: torch.Tensor, norm: torch.Tensor | None, shadow: torch.Tensor | None) -> None:
    """norm[f] = ||W[f,:]||_2 and shadow = bf16(W) in one pass."""
    if not W.is_cuda:
        if norm is not None:
            norm.copy_(W.norm(dim=1))
        if shadow is not None:
            shadow.copy_(W)
        return
    _ext().row_norm_shadow(W, norm, shadow)
