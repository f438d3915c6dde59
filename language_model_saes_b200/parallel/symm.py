"""Peer-memory communicators: symmetric buffers whose peer mappings the kernels of ``ops/csrc/comm_ops.cu`` store into
and load from over NVLink, synchronised by epoch flags inside the same buffers. torch's own collectives are not involved
on these paths.

One symmetric buffer per rank is allocated with ``torch.distributed._symmetric_memory`` (CUDA VMM allocation whose
handle is exchanged over the process group) and rendezvoused over a group; after that every rank holds plain device
pointers to all peers' buffers and, where the group's GPUs hang off an NVSwitch that the driver lets us use, one more
pointer to a multicast mapping of the same buffers (``multimem`` loads reduce over all ranks inside the switch,
``multimem`` stores reach every rank with one message).

``SymmComm`` carries the feature-sharded fused step (candidate all-gather, reduce-scatter of the partial
reconstructions, all-gather of the gradient rows); ``DataParallelComm`` the data-parallel one (row all-gather,
publication of updated parameter rows); ``ShuffleComm``, ``BroadcastComm`` and ``HeadSumComm`` the activation shuffle,
the cached-activation broadcast and the crosscoder head sum.

Every phase keeps its own epoch counter, advanced by the call that publishes it; all ranks make the same calls in the
same order, so the counters agree without any exchange. Re-use of a region across steps needs no extra barrier: every
phase of a step waits for all peers, so a peer can only start writing step t+1's data into a region after this rank has
consumed step t's (its own step-t+1 writes come after kernels that, in stream order, follow this rank's step-t
consumers). The candidate lists are exchanged outside training steps as well (metrics, encoding), where no later phase
orders the ranks, so their landing zone is double-buffered by epoch parity.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist

from ..ops import sae_kernels as K

PHASE_CAND, PHASE_PARTIAL, PHASE_DXHAT, PHASE_AUX, PHASE_ROWS, PHASE_PARAMS = 0, 1, 2, 3, 4, 5
PHASE_NAMES = {PHASE_CAND: "candidates", PHASE_PARTIAL: "partial rows", PHASE_DXHAT: "gradient rows", PHASE_AUX: "auxiliary",
               PHASE_ROWS: "data-parallel rows", PHASE_PARAMS: "parameter rows"}  # fmt: skip
_MAX_PEERS = 8
_NUM_PHASES = 8
FLAG_BYTES = _NUM_PHASES * _MAX_PEERS * 4


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


def peer_table(world: int, rank: int, ptrs: list[int], flags_off: int = 0, cand_val_off: int = 0, cand_idx_off: int = 0,
               partial_off: int = 0, dxhat_off: int = 0, multicast_ptr: int = 0, stats_ptr: int = 0) -> list[int]:  # fmt: skip
    """The integer list the extension turns into its ``PeerTable``: sizes, region offsets, the multicast base (0: none),
    the address of the exposed-wait counters (0: none) and one buffer pointer per rank."""
    assert len(ptrs) == world
    return [world, rank, flags_off, cand_val_off, cand_idx_off, partial_off, dxhat_off, multicast_ptr, stats_ptr, *ptrs]


def _rendezvous(nbytes: int, group: dist.ProcessGroup, device: torch.device):
    """Allocate and map one zero-filled symmetric buffer of ``nbytes`` per rank of ``group``; returns
    ``(buffer, handle, peer pointers, multicast pointer or 0)``."""
    import torch.distributed._symmetric_memory as symm_mem

    try:
        symm_mem.enable_symm_mem_for_group(group.group_name)
    except Exception:  # noqa: BLE001  (newer torch enables groups implicitly)
        pass
    buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
    buf.zero_()
    handle = symm_mem.rendezvous(buf, group.group_name)
    ptrs = [int(p) for p in handle.buffer_ptrs]
    mc = 0
    if os.environ.get("LMSAE_NVLS", "1") != "0":
        try:
            mc = int(getattr(handle, "multicast_ptr", 0) or 0)
        except Exception:  # noqa: BLE001  (no multicast support in this build / on this fabric)
            mc = 0
    return buf, handle, ptrs, mc


def _use_multicast(requested: bool | None, env_name: str, world: int, multicast_ptr: int) -> bool:
    """Whether a communicator sends through the NVSwitch multicast mapping (``multimem`` instructions): an explicit
    argument wins, then the environment variable (``1`` / ``0``), else groups of more than two ranks do. With one peer a
    multicast store saves nothing over a peer store, and the measured in-switch reduction was slower than peer loads at
    two ranks and faster at eight. Always off without a multicast mapping."""
    if requested is None:
        env = os.environ.get(env_name, "")
        requested = env == "1" if env in ("0", "1") else world > 2
    return bool(requested and multicast_ptr)


class WaitStats:
    """Device counters of the time kernels spent in bounded peer-flag waits: ``{cycles, calls}`` per phase, filled by
    block 0 of every waiting kernel. ``read()`` converts to milliseconds with an SM clock in MHz."""

    def __init__(self, device: torch.device):
        self.buf = torch.zeros(2 * _NUM_PHASES, dtype=torch.int64, device=device)

    def reset(self) -> None:
        self.buf.zero_()

    def read(self, sm_mhz: float) -> dict[str, dict[str, float]]:
        vals = self.buf.tolist()
        out = {}
        for ph, name in PHASE_NAMES.items():
            cycles, calls = vals[2 * ph], vals[2 * ph + 1]
            if calls:
                out[name] = {"ms": cycles / (sm_mhz * 1e3), "calls": calls}
        return out


GUARD_BYTES = 256  # width of a guard band between two regions of a step buffer (debug layouts only)
GUARD_PATTERN = 0xA5


def guards_wanted() -> bool:
    """Debug layouts (guard bands between the regions of the step buffers, checked by ``check_guards``) are on with the
    bounds-checked build of the kernels (``LMSAE_NATIVE_CHECKED=1``) or with ``LMSAE_BUFFER_GUARDS=1``."""
    return os.environ.get("LMSAE_NATIVE_CHECKED") == "1" or os.environ.get("LMSAE_BUFFER_GUARDS") == "1"


def step_buffer_layout(batch: int, world: int, k_max: int, d_model: int, partial_itemsize: int = 2, guards: bool = False) -> dict:
    """Byte offsets of the regions of one rank's buffer for the fused step (the same on every rank): ``flags``
    ``[phase][source rank]`` epoch words, two candidate landing zones ``cand_val`` / ``cand_idx`` ``[2][B][world * k]``,
    ``partial`` ``[world][B / world][d]`` (or ``[B][d]`` when the owner reads through the switch) in fp32 or bf16,
    ``dxhat`` ``[B][d]`` bf16, and the total ``nbytes``. With ``guards`` every region is followed by a band of
    ``GUARD_BYTES`` that nothing may write (``lay["guards"]``: their offsets): a store that runs past a region by a row
    or a slot lands there instead of in its neighbour, and ``check_guards`` finds it."""
    lay, off = {}, 0
    cand = _align(batch * world * k_max * 4)
    bands = []
    for name, nbytes in (("flags", FLAG_BYTES), ("cand_val", 2 * cand), ("cand_idx", 2 * cand),
                         ("partial", batch * d_model * partial_itemsize), ("dxhat", batch * d_model * 2)):  # fmt: skip
        lay[name] = off
        off = _align(off + nbytes)
        if guards:
            bands.append((name, off))
            off = _align(off + GUARD_BYTES)
    lay["cand_stride"] = cand
    lay["guards"] = bands
    lay["nbytes"] = off
    return lay


def fill_guards(buf: torch.Tensor, lay: dict) -> None:
    for _, off in lay["guards"]:
        buf[off : off + GUARD_BYTES] = GUARD_PATTERN


def check_guards(buf: torch.Tensor, lay: dict) -> list[str]:
    """Names of the regions whose guard band (the bytes right behind the region) no longer holds the pattern."""
    return [name for name, off in lay["guards"] if not bool((buf[off : off + GUARD_BYTES] == GUARD_PATTERN).all())]


class SymmComm:
    """Collectives of the feature-sharded fused step over the ``model`` group.

    ``partial_dtype``: element type of the partial reconstruction rows on the wire (bf16 halves the NVLink bytes; it is
    what a bf16 all-reduce of the decoder output moves). ``use_multicast`` (default: environment ``LMSAE_STEP_MULTICAST``,
    else off): partial rows stay in the producer's buffer and the row owner sums them with ``multimem.ld_reduce``; the
    gradient rows are published with ``multimem.st``. Needs a multicast mapping and bf16 partials."""

    def __init__(self, group: dist.ProcessGroup, device: torch.device, batch: int, k_max: int, d_model: int,
                 partial_dtype: torch.dtype = torch.bfloat16, use_multicast: bool | None = None):  # fmt: skip
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        assert self.world <= _MAX_PEERS, f"at most {_MAX_PEERS} feature shards per peer-memory group"
        assert batch % self.world == 0, "batch must be divisible by the number of feature shards"
        assert partial_dtype in (torch.float32, torch.bfloat16)
        self.B, self.k_max, self.d = batch, k_max, d_model
        self.partial_dtype = partial_dtype
        lay = step_buffer_layout(batch, self.world, k_max, d_model, partial_dtype.itemsize, guards=guards_wanted())
        self.lay = lay
        self.partial_off, self.dxhat_off, self.nbytes = lay["partial"], lay["dxhat"], lay["nbytes"]
        self.buf, self.handle, self.ptrs, self.multicast_ptr = _rendezvous(self.nbytes, group, device)
        fill_guards(self.buf, lay)  # (no bands in the regular layout)
        if use_multicast is None:
            use_multicast = os.environ.get("LMSAE_STEP_MULTICAST", "0") == "1"
        self.use_multicast = bool(use_multicast and self.multicast_ptr and partial_dtype == torch.bfloat16)
        self.stats = WaitStats(device)
        self.done_counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.epochs = [0] * _NUM_PHASES
        self.device = device
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def check_guards(self) -> None:
        """Debug layouts: raise when a kernel (of any rank) wrote into a guard band of this rank's buffer. Synchronises."""
        bad = check_guards(self.buf, self.lay)
        if bad:
            raise RuntimeError(f"rank {self.rank}: stores ran past the end of the step buffer region(s) {bad}")

    def table(self, cand_parity: int = 0) -> list[int]:
        off = cand_parity * self.lay["cand_stride"]
        return peer_table(self.world, self.rank, self.ptrs, self.lay["flags"], self.lay["cand_val"] + off,
                          self.lay["cand_idx"] + off, self.partial_off, self.dxhat_off, self.multicast_ptr,
                          self.stats.buf.data_ptr())  # fmt: skip

    def _view(self, off: int, shape: tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        return self.buf[off : off + n * dtype.itemsize].view(dtype).view(*shape)

    def _advance(self, phase: int) -> int:
        self.epochs[phase] += 1
        return self.epochs[phase]

    # ---- candidate exchange ------------------------------------------------------------------------
    def merge_push(self, cand_val: torch.Tensor, cand_idx: torch.Tensor, k: int) -> None:
        """Merge this rank's candidate lists (``[B, C]`` from the encoder GEMM) into its ``k`` best per row and store
        them straight into every rank's merge input: the all-gather is the epilogue of the merge kernel."""
        B, C = cand_val.shape
        assert B == self.B and k <= self.k_max
        e = self._advance(PHASE_CAND)
        K._ext().topk_merge(cand_val, cand_idx, B, C, k, None, 0, C, True, None, None, 1, self.table(e & 1), e,
                            self.done_counter, K.status_buffer(self.device))  # fmt: skip

    def push_candidates(self, g_local: torch.Tensor, idx_local: torch.Tensor) -> None:
        """All-gather of ready-made per-rank (gated value, local column) top-k lists by direct peer stores."""
        B, k = g_local.shape
        assert B == self.B and k <= self.k_max
        e = self._advance(PHASE_CAND)
        K._ext().comm_push_candidates(self.table(e & 1), g_local.float().contiguous(), idx_local.contiguous(), e, self.done_counter)

    def merge_shards(self, k: int, gate: torch.Tensor | None) -> tuple[torch.Tensor, torch.Tensor]:
        """Wait (inside the kernel) for every rank's candidates of the exchange just published and keep this rank's
        winners among the ``k`` best of each row: ``(idx, act) [B, k]``, packed from slot 0 on."""
        e = self.epochs[PHASE_CAND]
        off = (e & 1) * self.lay["cand_stride"]
        shape = (self.B, self.world * k)
        all_g = self._view(self.lay["cand_val"] + off, shape, torch.float32)
        all_i = self._view(self.lay["cand_idx"] + off, shape, torch.int32)
        out_idx = torch.empty(self.B, k, dtype=torch.int32, device=self.device)
        out_val = torch.empty(self.B, k, dtype=torch.float32, device=self.device)
        K._ext().topk_merge(all_g, all_i, self.B, self.world * k, k, gate, self.rank * k, (self.rank + 1) * k, False,
                            out_idx, out_val, 2, self.table(e & 1), e, None, K.status_buffer(self.device))  # fmt: skip
        return out_idx, out_val

    # ---- decode: reduce-scatter, loss, all-gather ----------------------------------------------------
    def decode_reduce_loss(self, idx, act, W_bf16, label, bias, row_weight, grad_scale, loss_sum, want_xhat=False,
                           compact_codes: bool = True):  # fmt: skip
        """Sparse decode whose epilogue scatters partial rows to their owners, owner-side reduction + loss +
        gradient, and all-gather of the gradient rows. Returns (dxhat [B, d] bf16 view, xhat or None); the loss
        of the rows this rank owns is accumulated into ``loss_sum``. The view is complete only after every owner's
        gradient flag: consume it with ``dact`` (which waits inside its kernel) or call ``wait_dxhat`` first."""
        ext = K._ext()
        st = K.status_buffer(self.device)
        pd = 0 if self.partial_dtype == torch.float32 else 1
        e_in = self._advance(PHASE_PARTIAL)
        ext.comm_decode_scatter(self.table(), idx, act, W_bf16, pd, self.use_multicast, compact_codes, e_in, self.done_counter)
        xhat = torch.empty(self.B, self.d, dtype=torch.float32, device=self.device) if want_xhat else None
        e_out = self._advance(PHASE_DXHAT)
        ext.comm_reduce_loss_push(self.table(), self.B, self.d, label, bias, row_weight, grad_scale, loss_sum, xhat, pd,
                                  self.use_multicast, e_in, e_out, self.done_counter, st)  # fmt: skip
        return self._view(self.dxhat_off, (self.B, self.d), torch.bfloat16), xhat

    def dact(self, idx: torch.Tensor, W_bf16: torch.Tensor) -> torch.Tensor:
        """Gradient of the codes from the all-gathered gradient rows; the kernel waits for the owners' flags itself."""
        dxhat = self._view(self.dxhat_off, (self.B, self.d), torch.bfloat16)
        dval = torch.empty(idx.shape, dtype=torch.float32, device=self.device)
        K._ext().sparse_dact(idx, W_bf16, dxhat, dval, self.table(), self.epochs[PHASE_DXHAT], K.status_buffer(self.device))
        return dval

    def wait_dxhat(self) -> None:
        K._ext().comm_wait(self.table(), PHASE_DXHAT, self.epochs[PHASE_DXHAT], K.status_buffer(self.device))


class DataParallelComm:
    """Peer-memory plumbing of the data-parallel fused step over the ``data`` group.

    * ``exchange(tensors)``: all-gather of this replica's rows of several tensors in one kernel (peer stores into every
      replica's gather zones, then a bounded wait for the others' rows).
    * parameter publication: the bf16 shadows of ``W_D`` / ``W_E^T``, the decoder norms and the encoder bias live in
      this buffer; each replica updates only its share of the feature rows (optimizer state sharded by feature row)
      and the update kernel stores the new rows into every replica's copy. ``pub_args()`` are the extra arguments of
      ``sparse_grad_adam`` for that, ``wait_params()`` the bounded wait before the next step reads the shadows.
    """

    def __init__(self, group: dist.ProcessGroup, device: torch.device, n_features: int, d_model: int,
                 zones: dict[str, int], use_multicast: bool | None = None):  # fmt: skip
        """``zones``: name -> capacity in bytes of the GATHERED tensor, for every tensor that ``exchange`` moves.
        ``use_multicast``: the row exchange stores through the NVSwitch multicast mapping, one message per 16 bytes for
        all replicas (default: environment variable ``LMSAE_ROWS_MULTICAST``, else groups of more than two ranks)."""
        self.group, self.device = group, device
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        assert self.world <= _MAX_PEERS
        self.F, self.d = n_features, d_model
        off = _align(FLAG_BYTES)
        self.param_off = {}
        for name, nbytes in (("WD_bf16", n_features * d_model * 2), ("WE_bf16", n_features * d_model * 2),
                             ("dec_norm", n_features * 4), ("bE", n_features * 4)):  # fmt: skip
            self.param_off[name] = off
            off = _align(off + nbytes)
        self.zone_off, self.zone_cap = {}, dict(zones)
        for name, nbytes in zones.items():
            self.zone_off[name] = off
            off = _align(off + nbytes)
        self.nbytes = off
        self.buf, self.handle, self.ptrs, self.multicast_ptr = _rendezvous(self.nbytes, group, device)
        self.use_multicast = _use_multicast(use_multicast, "LMSAE_ROWS_MULTICAST", self.world, self.multicast_ptr)
        self.stats = WaitStats(device)
        self.done_counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.epochs = [0] * _NUM_PHASES
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def table(self) -> list[int]:
        return peer_table(self.world, self.rank, self.ptrs, 0, multicast_ptr=self.multicast_ptr if self.use_multicast else 0,
                          stats_ptr=self.stats.buf.data_ptr())  # fmt: skip

    def _view(self, off: int, shape: tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        n = dtype.itemsize
        for s in shape:
            n *= s
        return self.buf[off : off + n].view(dtype).view(*shape)

    def param_views(self) -> dict[str, torch.Tensor]:
        F, d = self.F, self.d
        return {"WD_bf16": self._view(self.param_off["WD_bf16"], (F, d), torch.bfloat16),
                "WE_bf16": self._view(self.param_off["WE_bf16"], (F, d), torch.bfloat16),
                "dec_norm": self._view(self.param_off["dec_norm"], (F,), torch.float32),
                "bE": self._view(self.param_off["bE"], (F,), torch.float32)}  # fmt: skip

    def own_rows(self) -> tuple[int, int]:
        """Feature rows whose optimizer state this replica holds (equal shares; ``F`` must divide by the group size)."""
        assert self.F % self.world == 0
        per = self.F // self.world
        return self.rank * per, (self.rank + 1) * per

    def exchange(self, tensors: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
        """All-gather (dimension 0) of this replica's part of every tensor in one kernel; returns views of the gathered
        tensors inside the symmetric buffer, valid until the next ``exchange``."""
        names = list(tensors)
        parts = [tensors[n].contiguous() for n in names]
        for n, t in zip(names, parts):
            nb = t.numel() * t.element_size()
            assert nb % 16 == 0 and nb * self.world <= self.zone_cap[n], f"zone {n}: {nb} bytes per rank do not fit"
        e = self.epochs[PHASE_ROWS] = self.epochs[PHASE_ROWS] + 1
        K._ext().comm_exchange_rows(self.table(), parts, [self.zone_off[n] for n in names], e, self.done_counter,
                                    K.status_buffer(self.device), self.use_multicast)  # fmt: skip
        return {n: self._view(self.zone_off[n], (self.world * t.shape[0], *t.shape[1:]), t.dtype) for n, t in zip(names, parts)}

    def pub_args(self) -> tuple[list[int], list[int], int, torch.Tensor]:
        e = self.epochs[PHASE_PARAMS] = self.epochs[PHASE_PARAMS] + 1
        offs = [self.param_off[n] for n in ("WD_bf16", "WE_bf16", "dec_norm", "bE")]
        return self.table(), offs, e, self.done_counter

    def wait_params(self) -> None:
        if self.epochs[PHASE_PARAMS] > 0:
            K._ext().comm_wait(self.table(), PHASE_PARAMS, self.epochs[PHASE_PARAMS], K.status_buffer(self.device))


PHASE_SHUFFLE = 3


class ShuffleComm:
    """All-to-all of rows between the ranks of a group by direct peer stores: ``shuffle(x, seed)`` applies ONE seeded
    permutation to the logical concatenation of every rank's rows and returns this rank's slice of the result.

    The reference shuffles its activation buffer per rank only and refuses to do it under a device mesh
    (activation/processors/activation.py:144-163 of the reference project); with this, data-parallel ranks mix their
    buffers, so a batch is a sample of what ALL ranks generated. Two landing buffers alternate between calls: a peer
    can start call t+1 while this rank still copies call t's result out, and nobody can be two calls ahead of anyone
    because every call waits for all peers' flags.
    """

    def __init__(self, group: dist.ProcessGroup, device: torch.device, rows_per_rank: int, max_row_bytes: int):
        self.group, self.device = group, device
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        assert self.world <= _MAX_PEERS
        self.rows_per_rank = rows_per_rank
        self.max_row_bytes = _align(max_row_bytes, 16)
        self.flags_off = 0
        self.recv_off = [_align(FLAG_BYTES)]
        self.recv_off.append(_align(self.recv_off[0] + rows_per_rank * self.max_row_bytes))
        self.nbytes = _align(self.recv_off[1] + rows_per_rank * self.max_row_bytes)
        self.buf, self.handle, ptrs, _ = _rendezvous(self.nbytes, group, device)
        self.table = peer_table(self.world, self.rank, ptrs)
        self.done_counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.epoch = 0
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def permutation(self, n: int, seed: int) -> torch.Tensor:
        """The permutation of ``world * n`` positions that every rank derives from ``seed`` (CPU generator)."""
        g = torch.Generator().manual_seed(int(seed))
        return torch.randperm(self.world * n, generator=g)

    def shuffle(self, x: torch.Tensor, seed: int, perm: torch.Tensor | None = None) -> torch.Tensor:
        """``x``: this rank's ``[n, ...]`` rows (same ``n`` on every rank, ``n <= rows_per_rank``, rows a multiple of
        16 bytes). Row ``i`` of rank ``r`` lands at global position ``perm[r * n + i]``."""
        n = x.shape[0]
        assert n <= self.rows_per_rank and x.is_cuda
        x = x.contiguous()
        row_bytes = (x.numel() // max(n, 1)) * x.element_size()
        assert row_bytes % 16 == 0 and row_bytes <= self.max_row_bytes, f"row of {row_bytes} bytes does not fit"
        if perm is None:
            perm = self.permutation(n, seed)
        dest = perm[self.rank * n : (self.rank + 1) * n].to(self.device, non_blocking=True)
        self.epoch += 1
        off = self.recv_off[self.epoch & 1]
        ext = K._ext()
        ext.comm_shuffle_rows(self.table, x, dest, n, off, PHASE_SHUFFLE, self.epoch, self.done_counter)
        ext.comm_wait(self.table, PHASE_SHUFFLE, self.epoch, K.status_buffer(self.device))
        out = self.buf[off : off + n * row_bytes].view(x.dtype).view(n, *x.shape[1:])
        return out.clone()


PHASE_BCAST_DATA, PHASE_BCAST_ACK = 0, 1


class BroadcastComm:
    """One rank's rows to every rank of the group by direct peer stores, fused with token-mask compaction and a dtype
    cast (``comm_bcast_rows``): the rank that read a chunk of cached activations pushes the cleaned rows into every
    peer's landing zone over NVLink; the others never touch the disk or the host copy engine for that chunk.

    Two landing zones alternate. Before the sender overwrites the zone of call ``t - 2`` it waits (bounded) for every
    rank's acknowledgement of that call, which each rank publishes after it has copied the rows out. The row count
    travels in a one-element all-reduce that also orders the ranks: receivers run behind the sender's launch and the
    sender behind the receivers' previous copies, so the bounded flag waits only cover stores and flags in flight.
    """

    def __init__(self, group: dist.ProcessGroup, device: torch.device, max_rows: int, max_row_bytes: int,
                 use_multicast: bool | None = None):  # fmt: skip
        """``use_multicast``: the sender stores every 16 bytes once through the NVSwitch multicast mapping instead of once
        per peer (default: environment variable ``LMSAE_BCAST_MULTICAST``, else groups of more than two ranks)."""
        self.group, self.device = group, device
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        assert self.world <= _MAX_PEERS
        self.max_rows, self.max_row_bytes = max_rows, _align(max_row_bytes, 16)
        self.flags_off = 0
        zone = _align(max_rows * self.max_row_bytes)
        self.recv_off = [_align(FLAG_BYTES)]
        self.recv_off.append(self.recv_off[0] + zone)
        self.nbytes = self.recv_off[1] + zone
        self.buf, self.handle, ptrs, mc = _rendezvous(self.nbytes, group, device)
        self.use_multicast = _use_multicast(use_multicast, "LMSAE_BCAST_MULTICAST", self.world, mc)
        self.table = peer_table(self.world, self.rank, ptrs, 0, multicast_ptr=mc if self.use_multicast else 0)
        self.done_counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.count = torch.zeros(1, dtype=torch.int64, device=device)
        self.epoch = 0
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def broadcast_rows(self, src_rank: int, d: int, out_dtype: torch.dtype, rows: torch.Tensor | None = None,
                       keep: torch.Tensor | None = None) -> torch.Tensor:  # fmt: skip
        """Every rank calls this with the same ``src_rank`` (rank within the group), ``d`` and ``out_dtype``; the sender
        also passes ``rows [n, d]`` (fp32 or bf16) and optionally ``keep [n]``. Returns the kept rows, cast, on every
        rank."""
        ext = K._ext()
        st = K.status_buffer(self.device)
        self.epoch += 1
        off = self.recv_off[self.epoch & 1]
        row_bytes = d * out_dtype.itemsize
        assert row_bytes <= self.max_row_bytes and d % 8 == 0 and out_dtype in (torch.float32, torch.bfloat16)
        cap_rows = (self.max_rows * self.max_row_bytes) // row_bytes
        if self.rank == src_rank:
            assert rows is not None and rows.is_cuda and rows.ndim == 2 and rows.shape[1] == d
            rows = rows.contiguous()
            n = rows.shape[0]
            keep32 = pos = None
            if keep is not None:
                keep32 = keep.reshape(-1).to(torch.int32).contiguous()
                pos = torch.empty(n + 1, dtype=torch.int32, device=self.device)
                ext.exclusive_scan(keep32, pos, torch.empty((n + 4095) // 4096, dtype=torch.int32, device=self.device))
                self.count.copy_(pos[n : n + 1])
            else:
                self.count.fill_(n)
            if self.epoch > 2:  # the zone still holds call epoch - 2: everyone must have copied it out
                ext.comm_wait(self.table, PHASE_BCAST_ACK, self.epoch - 2, st)
            ext.comm_bcast_rows(self.table, rows, keep32, pos, 0 if out_dtype == torch.float32 else 1, off, cap_rows,
                                PHASE_BCAST_DATA, self.epoch, self.done_counter, self.use_multicast)  # fmt: skip
        else:
            self.count.zero_()
        # the row count, summed (the others add zero): unlike a broadcast, an all-reduce completes on the sender only after
        # every rank has reached this call, i.e. after their copies and acknowledgements of the previous call
        dist.all_reduce(self.count, group=self.group)
        ext.comm_wait_src(self.table, PHASE_BCAST_DATA, self.epoch, src_rank, st)
        m = int(self.count)
        assert m <= cap_rows, f"{m} rows do not fit the landing zone of {cap_rows}"
        out = self.buf[off : off + m * row_bytes].view(out_dtype).view(m, d).clone()
        ext.comm_signal(self.table, PHASE_BCAST_ACK, self.epoch)
        return out


class AllReduceComm:
    """In-place sum over a group of a bf16 matrix that lives in this communicator's symmetric buffer: ``matrix(rows, cols)``
    hands out the view to fill (e.g. as the output of a GEMM), ``all_reduce(rows, cols)`` replaces it on every rank by the
    sum over ranks in ONE kernel (``ops/csrc/comm_ops.cu::allreduce_bf16_inplace_kernel``): with an NVSwitch multicast
    mapping the owner of a share reads the sum with ``multimem.ld_reduce`` (added inside the switch) and writes it to
    every rank with ``multimem.st``; without one, by peer loads and stores. Two buffers alternate between calls, so a
    rank may fill the next matrix while a slower peer still reads the previous sums."""

    PHASE_READY, PHASE_DONE = 0, 1

    def __init__(self, group: dist.ProcessGroup | None, device: torch.device, max_rows: int, n_cols: int, use_multicast: bool | None = None):
        self.group, self.device = group, device
        self.world = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        assert self.world <= _MAX_PEERS and n_cols % 8 == 0
        self.max_rows, self.n_cols = max_rows, n_cols
        zone = _align(max_rows * n_cols * 2)
        self.off = [_align(FLAG_BYTES), _align(FLAG_BYTES) + zone]
        self.nbytes = self.off[1] + zone
        if group is not None and self.world > 1:
            self.buf, self.handle, ptrs, mc = _rendezvous(self.nbytes, group, device)
        else:
            self.buf, ptrs, mc = torch.zeros(self.nbytes, dtype=torch.uint8, device=device), None, 0
            ptrs = [self.buf.data_ptr()]
        self.use_multicast = _use_multicast(use_multicast, "LMSAE_ALLREDUCE_MULTICAST", self.world, mc)
        self.stats = WaitStats(device)
        self.table = peer_table(self.world, self.rank, ptrs, 0, multicast_ptr=mc, stats_ptr=self.stats.buf.data_ptr())
        self.done_counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.epoch = 0
        torch.cuda.synchronize(device)
        if group is not None and self.world > 1:
            dist.barrier(group=group)

    def matrix(self, rows: int, cols: int | None = None) -> torch.Tensor:
        """The bf16 ``[rows, cols]`` view that the NEXT ``all_reduce`` will sum."""
        cols = cols or self.n_cols
        assert rows <= self.max_rows and cols == self.n_cols
        off = self.off[(self.epoch + 1) & 1]
        return self.buf[off : off + rows * cols * 2].view(torch.bfloat16).view(rows, cols)

    def all_reduce(self, rows: int) -> torch.Tensor:
        self.epoch += 1
        off = self.off[self.epoch & 1]
        n16 = rows * self.n_cols * 2 // 16
        K._ext().comm_allreduce_bf16(self.table, off, n16, self.PHASE_READY, self.PHASE_DONE, self.epoch, self.use_multicast,
                                     self.done_counter, K.status_buffer(self.device))  # fmt: skip
        return self.buf[off : off + rows * self.n_cols * 2].view(torch.bfloat16).view(rows, self.n_cols)


class HeadSumComm:
    """Sum of per-rank encoder pre-activations over a ``head`` group.

    ``head_sum(x, w, bias, ...)`` computes ``sum_ranks (sum_local_heads x_h W_h^T + b_h)`` as ``[M, N]`` on every rank:
    the tcgen05 GEMM accumulates the local heads in one K loop (K = heads x d) and stores its bf16 result straight into
    the symmetric buffer of an ``AllReduceComm``, whose one kernel then sums the matrix over the ranks in place (in the
    NVSwitch with ``multimem`` on groups of more than two ranks, by peer loads and stores otherwise; fp32 accumulation).
    models/crosscoder.py:350-375 of the reference project all-reduces the same ``[batch, d_sae]`` tensor with NCCL.
    """

    def __init__(self, group: dist.ProcessGroup | None, device: torch.device, max_rows: int, n_cols: int,
                 use_multicast: bool | None = None):  # fmt: skip
        self.reduce = AllReduceComm(group, device, max_rows, n_cols, use_multicast)
        self.group, self.device = group, device
        self.world, self.rank = self.reduce.world, self.reduce.rank
        self.max_rows, self.n_cols = max_rows, n_cols

    def head_sum(self, x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, heads: int, rows_per_head: int,
                 out_dtype: torch.dtype = torch.float32, pair: bool = True) -> torch.Tensor:  # fmt: skip
        """``x [M, heads * d]`` bf16, ``w [heads * rows_per_head, d]`` bf16 (feature-major blocks, one per local head),
        ``bias [N]`` fp32 = this rank's summed encoder biases. Returns ``[M, N]`` in ``out_dtype`` (a copy: the buffer is
        reused by the call after next)."""
        M = x.shape[0]
        assert M <= self.max_rows
        P = self.reduce.matrix(M)
        K._ext().head_sum_gemm(x, w, bias, heads, rows_per_head, self.n_cols, pair, K.status_buffer(self.device), P)
        if self.world > 1:
            P = self.reduce.all_reduce(M)
        return P.to(out_dtype, copy=True)
