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


class SymmComm:
    def __init__(self, group: dist.ProcessGroup, device: torch.device, batch: int, k_max: int, d_model: int):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        assert self.world <= _MAX_PEERS, f"at most {_MAX_PEERS} feature shards per peer-memory group"
        assert batch % self.world == 0, "batch must be divisible by the number of feature shards"
        self.B, self.k_max, self.d = batch, k_max, d_model
        off = 0
        self.flags_off = off
        off = _align(off + _NUM_PHASES * _MAX_PEERS * 4)
        self.cand_val_off = off
        off = _align(off + batch * self.world * k_max * 4)
        self.cand_idx_off = off
        off = _align(off + batch * self.world * k_max * 4)
        self.partial_off = off
        off = _align(off + batch * d_model * 4)
        self.dxhat_off = off
        off = _align(off + batch * d_model * 2)
        self.nbytes = off
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
