"""Peer-memory communicator for the feature-sharded fused step.

One symmetric buffer per rank is allocated with ``torch.distributed._symmetric_memory`` (CUDA VMM allocation
whose handle is exchanged over the process group) and rendezvoused over the ``model`` group; after that every
rank holds plain device pointers to all peers' buffers. The kernels in ``ops/csrc/comm_ops.cu`` store into and
load from those pointers over NVLink and synchronise with epoch flags inside the same buffers; torch's own
collectives are not involved on this path.

Buffer regions (identical offsets on every rank): epoch flags, merge input for the candidate exchange
``[B][tp*k]`` (values and columns), reduce-scatter landing zone ``[tp][B/tp][d]`` fp32, all-gathered gradient
``[B][d]`` bf16.

Re-use across steps needs no extra barrier: every phase of a step waits for all peers, so a peer can only start
writing step t+1's data into a region after this rank has consumed step t's (its own step-t+1 writes come after
kernels that, in stream order, follow this rank's step-t consumers).
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import sae_kernels as K

PHASE_CAND, PHASE_PARTIAL, PHASE_DXHAT = 0, 1, 2
_MAX_PEERS = 8
_NUM_PHASES = 4


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


def step_buffer_layout(batch: int, world: int, k_max: int, d_model: int) -> dict[str, int]:
    """Byte offsets of the regions of one rank's buffer for the fused step (the same on every rank): ``flags``
    ``[phase][source rank]`` epoch words, ``cand_val`` / ``cand_idx`` ``[B][world * k]``, ``partial``
    ``[world][B / world][d]`` fp32, ``dxhat`` ``[B][d]`` bf16, and the total ``nbytes``."""
    lay, off = {}, 0
    for name, nbytes in (("flags", _NUM_PHASES * _MAX_PEERS * 4), ("cand_val", batch * world * k_max * 4),
                         ("cand_idx", batch * world * k_max * 4), ("partial", batch * d_model * 4),
                         ("dxhat", batch * d_model * 2)):  # fmt: skip
        lay[name] = off
        off = _align(off + nbytes)
    lay["nbytes"] = off
    return lay


class SymmComm:
    def __init__(self, group: dist.ProcessGroup, device: torch.device, batch: int, k_max: int, d_model: int):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        assert self.world <= _MAX_PEERS, f"at most {_MAX_PEERS} feature shards per peer-memory group"
        assert batch % self.world == 0, "batch must be divisible by the number of feature shards"
        self.B, self.k_max, self.d = batch, k_max, d_model
        lay = step_buffer_layout(batch, self.world, k_max, d_model)
        self.flags_off, self.cand_val_off, self.cand_idx_off = lay["flags"], lay["cand_val"], lay["cand_idx"]
        self.partial_off, self.dxhat_off, self.nbytes = lay["partial"], lay["dxhat"], lay["nbytes"]
        try:
            symm_mem.enable_symm_mem_for_group(group.group_name)
        except Exception:  # noqa: BLE001  (newer torch enables groups implicitly)
            pass
        self.buf = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.buf.zero_()
        self.handle = symm_mem.rendezvous(self.buf, group.group_name)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.table = [self.world, self.rank, self.flags_off, self.cand_val_off, self.cand_idx_off, self.partial_off,
                      self.dxhat_off, *ptrs]  # fmt: skip
        self.done_counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.epoch = 0
        self.device = device
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def _view(self, off: int, shape: tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        return self.buf[off : off + n * dtype.itemsize].view(dtype).view(*shape)

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch

    # ---- phases ----------------------------------------------------------------------------------
    def exchange_candidates(self, g_local: torch.Tensor, idx_local: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """All-gather of the per-rank (gated value, local column) top-k lists by direct peer stores.
        Returns views ``[B, tp*k]`` of this rank's merge input."""
        B, k = g_local.shape
        assert B == self.B and k <= self.k_max
        ext = K._ext()
        ext.comm_push_candidates(self.table, g_local, idx_local, self.epoch, self.done_counter)
        ext.comm_wait(self.table, PHASE_CAND, self.epoch, K.status_buffer(self.device))
        shape = (B, self.world * k)
        return self._view(self.cand_val_off, shape, torch.float32), self._view(self.cand_idx_off, shape, torch.int32)

    def decode_reduce_loss(self, idx, act, W_bf16, label, bias, row_weight, grad_scale, loss_sum, want_xhat=False):
        """Sparse decode whose epilogue scatters partial rows to their owners, owner-side reduction + loss +
        gradient, and all-gather of the gradient rows. Returns (dxhat [B, d] bf16 view, xhat or None); the loss
        of the rows this rank owns is accumulated into ``loss_sum``."""
        ext = K._ext()
        st = K.status_buffer(self.device)
        ext.comm_decode_scatter(self.table, idx, act, W_bf16, self.epoch, self.done_counter)
        xhat = torch.empty(self.B, self.d, dtype=torch.float32, device=self.device) if want_xhat else None
        ext.comm_reduce_loss_push(self.table, self.B, self.d, label, bias, row_weight, grad_scale, loss_sum, xhat,
                                  self.epoch, self.done_counter, st)  # fmt: skip
        ext.comm_wait(self.table, PHASE_DXHAT, self.epoch, st)
        return self._view(self.dxhat_off, (self.B, self.d), torch.bfloat16), xhat


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
        import torch.distributed._symmetric_memory as symm_mem

        self.group, self.device = group, device
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        assert self.world <= _MAX_PEERS
        self.rows_per_rank = rows_per_rank
        self.max_row_bytes = _align(max_row_bytes, 16)
        self.flags_off = 0
        self.recv_off = [_align(_NUM_PHASES * _MAX_PEERS * 4)]
        self.recv_off.append(_align(self.recv_off[0] + rows_per_rank * self.max_row_bytes))
        self.nbytes = _align(self.recv_off[1] + rows_per_rank * self.max_row_bytes)
        try:
            symm_mem.enable_symm_mem_for_group(group.group_name)
        except Exception:  # noqa: BLE001
            pass
        self.buf = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.buf.zero_()
        self.handle = symm_mem.rendezvous(self.buf, group.group_name)
        self.table = [self.world, self.rank, self.flags_off, 0, 0, 0, 0, *[int(p) for p in self.handle.buffer_ptrs]]
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

    def __init__(self, group: dist.ProcessGroup, device: torch.device, max_rows: int, max_row_bytes: int):
        import torch.distributed._symmetric_memory as symm_mem

        self.group, self.device = group, device
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        assert self.world <= _MAX_PEERS
        self.max_rows, self.max_row_bytes = max_rows, _align(max_row_bytes, 16)
        self.flags_off = 0
        zone = _align(max_rows * self.max_row_bytes)
        self.recv_off = [_align(_NUM_PHASES * _MAX_PEERS * 4)]
        self.recv_off.append(self.recv_off[0] + zone)
        self.nbytes = self.recv_off[1] + zone
        try:
            symm_mem.enable_symm_mem_for_group(group.group_name)
        except Exception:  # noqa: BLE001
            pass
        self.buf = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.buf.zero_()
        self.handle = symm_mem.rendezvous(self.buf, group.group_name)
        self.table = [self.world, self.rank, self.flags_off, 0, 0, 0, 0, *[int(p) for p in self.handle.buffer_ptrs]]
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
                                PHASE_BCAST_DATA, self.epoch, self.done_counter)  # fmt: skip
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


PHASE_HS_REDUCED, PHASE_HS_GATHERED = 0, 1


class HeadSumComm:
    """Sum of per-rank encoder pre-activations over a ``head`` group, fused into the GEMM that produces them.

    ``head_sum(x, w, bias, ...)`` computes ``sum_ranks (sum_local_heads x_h W_h^T + b_h)`` as ``[M, N]`` on every rank:
    the tcgen05 GEMM accumulates the local heads in one K loop (K = heads x d) and its epilogue adds each finished tile
    into the fp32 slab of the rank that owns those columns with vector reductions through the peer mapping
    (reduce-scatter while other tiles are still being multiplied); the owners then store the sums into every rank's output
    (all-gather by peer stores). Two slabs alternate between calls and are cleared by their owner after use.
    """

    def __init__(self, group: dist.ProcessGroup | None, device: torch.device, max_rows: int, n_cols: int):
        import torch.distributed._symmetric_memory as symm_mem

        self.group, self.device = group, device
        self.world = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        assert self.world <= _MAX_PEERS and n_cols % (self.world * 32) == 0, "d_sae must divide into 32-column slabs per rank"
        self.max_rows, self.n_cols, self.cols = max_rows, n_cols, n_cols // self.world
        off = _align(_NUM_PHASES * _MAX_PEERS * 4)
        self.slab_off = [off, _align(off + max_rows * self.cols * 4)]
        self.out_off = _align(self.slab_off[1] + max_rows * self.cols * 4)
        self.nbytes = _align(self.out_off + max_rows * n_cols * 4)
        if group is not None and self.world > 1:
            try:
                symm_mem.enable_symm_mem_for_group(group.group_name)
            except Exception:  # noqa: BLE001
                pass
            self.buf = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=device)
            self.buf.zero_()
            self.handle = symm_mem.rendezvous(self.buf, group.group_name)
            ptrs = [int(p) for p in self.handle.buffer_ptrs]
        else:
            self.buf = torch.zeros(self.nbytes, dtype=torch.uint8, device=device)
            ptrs = [self.buf.data_ptr()]
        self.ptrs = ptrs
        self.table = [self.world, self.rank, 0, 0, 0, 0, 0, *ptrs]
        self.done_counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.epoch = 0
        torch.cuda.synchronize(device)
        if group is not None and self.world > 1:
            dist.barrier(group=group)

    def head_sum(self, x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, heads: int, rows_per_head: int,
                 out_dtype: torch.dtype = torch.float32, pair: bool = True) -> torch.Tensor:  # fmt: skip
        """``x [M, heads * d]`` bf16, ``w [heads * rows_per_head, d]`` bf16 (feature-major blocks, one per local head),
        ``bias [N]`` fp32 = this rank's summed encoder biases. Returns ``[M, N]`` in ``out_dtype`` (fp32 or bf16)."""
        M = x.shape[0]
        assert M <= self.max_rows and out_dtype in (torch.float32, torch.bfloat16)
        ext = K._ext()
        st = K.status_buffer(self.device)
        self.epoch += 1
        slab_off = self.slab_off[self.epoch & 1]
        ext.head_sum_gemm(x, w, bias, heads, rows_per_head, self.n_cols, [p + slab_off for p in self.ptrs], pair, st)
        ext.comm_signal(self.table, PHASE_HS_REDUCED, self.epoch)
        ext.comm_headsum_gather(self.table, slab_off, self.out_off, M, self.cols, 0 if out_dtype == torch.float32 else 1,
                                PHASE_HS_REDUCED, PHASE_HS_GATHERED, self.epoch, self.done_counter, st)  # fmt: skip
        ext.comm_wait(self.table, PHASE_HS_GATHERED, self.epoch, st)
        n = M * self.n_cols * out_dtype.itemsize
        return self.buf[self.out_off : self.out_off + n].view(out_dtype).view(M, self.n_cols).clone()
