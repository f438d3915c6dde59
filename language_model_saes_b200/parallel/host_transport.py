"""The fused step's peer-memory protocol executed by the host, for machines without GPUs.

``HostPeerComm`` has the interface of ``parallel.symm.SymmComm`` (``merge_push`` / ``push_candidates``,
``merge_shards``, ``decode_reduce_loss``, ``dact``) and the same buffer layout (``symm.step_buffer_layout``), phases,
flag words and per-phase epoch counters, but the "peer memory" is one file in shared memory that every rank of the
group maps, and the stores, flag publications and bounded flag waits that ``ops/csrc/comm_ops.cu`` does on the device
are done by Python on the CPU. It exists so that the protocol can be tested with gloo ranks: buffer re-use across steps
without a barrier, candidate exchanges outside training steps (double-buffered landing zones), a rank that is late, a
flag that never arrives (the wait gives up after ``timeout_s``, the rank skips the work that needed the data, still
publishes its own flags so that peers do not time out in turn, and the call raises ``CollectiveTimeout`` naming phase
and source, which is what the device path reports through its status word).

``faults`` injects failures on the host only: ``{"drop_flag": phase}`` never publishes that phase's flag to the peers,
``{"delay_flag": (phase, seconds)}`` publishes it late. The reference project has no counterpart (its collectives are
DTensor redistributes, utils/distributed/ops.py there).
"""

from __future__ import annotations

import os
import tempfile
import time

import numpy as np
import torch
import torch.distributed as dist

from ..ops import sae_kernels as K
from .symm import (_MAX_PEERS, _NUM_PHASES, PHASE_CAND, PHASE_DXHAT, PHASE_NAMES, PHASE_PARTIAL, check_guards, fill_guards, guards_wanted,
                   step_buffer_layout)  # fmt: skip

_PHASE_NAMES = PHASE_NAMES


class HostPeerComm:
    def __init__(self, group: dist.ProcessGroup | None, batch: int, k_max: int, d_model: int, timeout_s: float = 5.0,
                 faults: dict | None = None, directory: str | None = None, partial_dtype: torch.dtype = torch.bfloat16,
                 guards: bool | None = None):  # fmt: skip
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        assert self.world <= _MAX_PEERS and batch % self.world == 0
        self.B, self.k_max, self.d = batch, k_max, d_model
        self.partial_dtype = partial_dtype
        self.lay = step_buffer_layout(batch, self.world, k_max, d_model, partial_dtype.itemsize,
                                      guards=guards_wanted() if guards is None else guards)
        self.timeout_s = timeout_s
        self.faults = dict(faults or {})
        self.epochs = [0] * _NUM_PHASES
        self.device = torch.device("cpu")
        # rank 0 of the group creates the file (zero-filled: all flags at epoch 0), everyone maps all of it
        box: list = [None]
        if self.rank == 0:
            base = directory or ("/dev/shm" if os.path.isdir("/dev/shm") else tempfile.gettempdir())
            fd, path = tempfile.mkstemp(prefix="lmsae_peer_", dir=base)
            os.ftruncate(fd, self.world * self.lay["nbytes"])
            os.close(fd)
            box[0] = path
        dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        self.path = box[0]
        self._map = np.memmap(self.path, dtype=np.uint8, mode="r+", shape=(self.world, self.lay["nbytes"]))
        self.bufs = [torch.from_numpy(self._map[p]) for p in range(self.world)]
        fill_guards(self.bufs[self.rank], self.lay)  # (no bands in the regular layout)
        dist.barrier(group=group)
        if self.rank == 0:
            os.unlink(self.path)  # the mappings keep the memory alive; nothing is left behind when the ranks exit

    def check_guards(self) -> None:
        """Debug layouts: raise when anyone wrote into a guard band of this rank's buffer."""
        bad = check_guards(self.bufs[self.rank], self.lay)
        if bad:
            raise RuntimeError(f"rank {self.rank}: stores ran past the end of the step buffer region(s) {bad}")

    # ---- views into a rank's buffer -------------------------------------------------------------
    def _region(self, peer: int, name: str, shape: tuple[int, ...], dtype: torch.dtype, extra_off: int = 0) -> torch.Tensor:
        n = dtype.itemsize
        for s in shape:
            n *= s
        off = self.lay[name] + extra_off
        return self.bufs[peer][off : off + n].view(dtype).view(*shape)

    def _flags(self, peer: int) -> torch.Tensor:
        return self._region(peer, "flags", (_NUM_PHASES, _MAX_PEERS), torch.int32)

    def _advance(self, phase: int) -> int:
        self.epochs[phase] += 1
        return self.epochs[phase]

    # ---- flag protocol ----------------------------------------------------------------------------
    def _signal(self, phase: int) -> None:
        """Publish the phase's current epoch in every rank's flag slot ``[phase][our rank]`` (after the data)."""
        late = self.faults.get("delay_flag")
        if late is not None and late[0] == phase:
            time.sleep(late[1])
        for p in range(self.world):
            if p != self.rank and self.faults.get("drop_flag") == phase:
                continue  # the flag words sent to the peers are lost; our own copy arrives
            self._flags(p)[phase, self.rank] = self.epochs[phase]

    def _wait(self, phase: int) -> list[int]:
        """Bounded wait until every source has published the phase's current epoch in OUR slots; returns the sources
        that had not when the time ran out (empty = all arrived)."""
        mine = self._flags(self.rank)
        deadline = time.monotonic() + self.timeout_s
        while True:
            late = [s for s in range(self.world) if int(mine[phase, s]) < self.epochs[phase]]
            if not late or time.monotonic() > deadline:
                return late
            time.sleep(0.0005)

    @staticmethod
    def _raise(phase: int, late: list[int]) -> None:
        err = K.CollectiveTimeout(f"timeout waiting for a peer flag: phase {phase} ({_PHASE_NAMES[phase]}), "
                                  f"no flag from rank(s) {late}")  # fmt: skip
        err.code, err.phase, err.sources = 5, phase, late
        raise err

    # ---- phases -----------------------------------------------------------------------------------
    def push_candidates(self, g_local: torch.Tensor, idx_local: torch.Tensor) -> None:
        B, k = g_local.shape
        assert B == self.B and k <= self.k_max
        e = self._advance(PHASE_CAND)
        zone = (e & 1) * self.lay["cand_stride"]
        lo, hi = self.rank * k, (self.rank + 1) * k
        for p in range(self.world):
            self._region(p, "cand_val", (B, self.world * k), torch.float32, zone)[:, lo:hi] = g_local.float()
            self._region(p, "cand_idx", (B, self.world * k), torch.int32, zone)[:, lo:hi] = idx_local.to(torch.int32)
        self._signal(PHASE_CAND)

    def merge_push(self, cand_val: torch.Tensor, cand_idx: torch.Tensor, k: int) -> None:
        idx_l, g_l = K.ref_topk_merge(cand_val, cand_idx, k, None, None, emit_gated=True)
        self.push_candidates(g_l, idx_l)

    def merge_shards(self, k: int, gate: torch.Tensor | None) -> tuple[torch.Tensor, torch.Tensor]:
        late = self._wait(PHASE_CAND)
        if late:
            self._raise(PHASE_CAND, late)
        zone = (self.epochs[PHASE_CAND] & 1) * self.lay["cand_stride"]
        all_g = self._region(self.rank, "cand_val", (self.B, self.world * k), torch.float32, zone).clone()
        all_i = self._region(self.rank, "cand_idx", (self.B, self.world * k), torch.int32, zone).clone()
        return K.ref_topk_merge(all_g, all_i, k, gate, own=(self.rank * k, (self.rank + 1) * k))

    def decode_reduce_loss(self, idx, act, W_bf16, label, bias, row_weight, grad_scale, loss_sum, want_xhat=False,
                           compact_codes: bool = True):  # fmt: skip
        B, d, rows = self.B, self.d, self.B // self.world
        pdt = self.partial_dtype
        partial = K.ref_sparse_decode(idx, act, W_bf16, None).to(pdt)  # [B, d] from this rank's features
        self._advance(PHASE_PARTIAL)
        for owner in range(self.world):  # reduce-scatter by stores: slot [our rank] of the owner's landing zone
            self._region(owner, "partial", (self.world, rows, d), pdt)[self.rank] = partial[owner * rows : (owner + 1) * rows]
        self._signal(PHASE_PARTIAL)
        late = self._wait(PHASE_PARTIAL)
        xhat = None
        self._advance(PHASE_DXHAT)
        if not late:
            sl = slice(self.rank * rows, (self.rank + 1) * rows)
            x = self._region(self.rank, "partial", (self.world, rows, d), pdt).float().sum(0)
            if bias is not None:
                x = x + bias
            e = x - label[sl].float()
            rw = row_weight[sl].float() if row_weight is not None else torch.ones(rows)
            loss_sum += (e.square().sum(-1) * rw).sum()
            g = (e * (grad_scale * rw)[:, None]).to(torch.bfloat16)
            for p in range(self.world):  # all-gather by stores into every rank's gradient buffer
                self._region(p, "dxhat", (B, d), torch.bfloat16)[sl] = g
            if want_xhat:
                xhat = torch.zeros(B, d)
                xhat[sl] = x
        # published even after a failed wait: peers must not pile their own timeouts on top of the first one
        self._signal(PHASE_DXHAT)
        if late:
            self._raise(PHASE_PARTIAL, late)
        return self._region(self.rank, "dxhat", (B, d), torch.bfloat16), xhat

    def wait_dxhat(self) -> None:
        late = self._wait(PHASE_DXHAT)
        if late:
            self._raise(PHASE_DXHAT, late)

    def dact(self, idx: torch.Tensor, W_bf16: torch.Tensor) -> torch.Tensor:
        self.wait_dxhat()
        return K.sparse_dact(idx, W_bf16, self._region(self.rank, "dxhat", (self.B, self.d), torch.bfloat16).clone())
