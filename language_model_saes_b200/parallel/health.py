"""Host-side failure detection for multi-process runs: heartbeats through the rendezvous store.

The reference project has none (a failed rank leaves the others blocked in their next collective until the backend's
own timeout, trainer.py:666-671 there only logs and re-raises). Here every rank publishes ``(step, time)`` in the
key-value store its process group was built on; before a step's first collective a rank looks at its peers' entries
and raises ``PeerLost`` when one has announced that it is leaving (an exception, the end of its data) or has not
been heard from for ``timeout_s``. Nothing here touches a GPU: a rank learns of a failure between steps, with none of
its kernels or collectives in flight, and can save a checkpoint and exit instead of waiting in a collective.
Device-side waits have their own bound and report through the kernels' status word (``ops.sae_kernels.check_status``).
"""

from __future__ import annotations

import time
from typing import Iterable

import torch.distributed as dist


class PeerLost(RuntimeError):
    """A peer rank left the job or stopped sending heartbeats. ``ranks`` maps rank -> reason."""

    def __init__(self, ranks: dict[int, str]):
        self.ranks = dict(ranks)
        super().__init__("; ".join(f"rank {r}: {why}" for r, why in sorted(self.ranks.items())))


def default_store():
    """The store of the default process group (None when torch.distributed is not initialised)."""
    if not dist.is_available() or not dist.is_initialized():
        return None
    from torch.distributed.distributed_c10d import _get_default_store

    return _get_default_store()


class Heartbeat:
    def __init__(self, store, rank: int, world_size: int, timeout_s: float = 60.0, prefix: str = "lmsae/heartbeat",
                 clock=time.time):  # fmt: skip
        self.store, self.rank, self.world = store, rank, world_size
        self.timeout_s, self.prefix, self.clock = timeout_s, prefix, clock
        self.started = clock()

    def _key(self, rank: int) -> str:
        return f"{self.prefix}/{rank}"

    def beat(self, step: int) -> None:
        self.store.set(self._key(self.rank), f"alive|{step}|{self.clock():.3f}")

    def leave(self, reason: str) -> None:
        """Announce that this rank stops taking part (called from exception handlers and at the end of the data)."""
        self.store.set(self._key(self.rank), f"left|{reason[:200]}|{self.clock():.3f}")

    def peers(self) -> Iterable[int]:
        return (r for r in range(self.world) if r != self.rank)

    def status(self, rank: int) -> tuple[str, str, float] | None:
        """``(state, detail, time)`` of a rank, None when it has not written anything yet. Never blocks."""
        key = self._key(rank)
        if not self.store.check([key]):
            return None
        state, detail, stamp = self.store.get(key).decode().split("|")
        return state, detail, float(stamp)

    def check(self) -> None:
        """Raise ``PeerLost`` if a peer has left or has been silent for longer than ``timeout_s``."""
        now = self.clock()
        lost: dict[int, str] = {}
        for r in self.peers():
            st = self.status(r)
            if st is None:
                if now - self.started > self.timeout_s:
                    lost[r] = f"no heartbeat since start ({now - self.started:.1f} s)"
                continue
            state, detail, stamp = st
            if state == "left":
                lost[r] = f"left: {detail}"
            elif now - stamp > self.timeout_s:
                lost[r] = f"silent for {now - stamp:.1f} s (last step {detail})"
        if lost:
            raise PeerLost(lost)
