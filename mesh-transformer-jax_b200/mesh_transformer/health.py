"""Host-side liveness check of the shard group.

The reference bounds its cluster calls with ``func_set_timeout`` (TPU_cluster.py:17,44,66,127) and otherwise
relies on the collective never returning when a host is gone.  Here every tensor-parallel call is a set of
kernels that wait on each other's GPUs, so a rank that has left must be noticed BEFORE the next launch: each
rank bumps a counter in the process group's key-value store at the start of a call and waits, with a
deadline, until every peer has bumped the same count.  A rank that raised, exited or hung on the host never
bumps, and the others get ``PeerLostError`` instead of launching kernels whose bounded waits would run out.
Nothing here touches a GPU.
"""
from __future__ import annotations

import time


class PeerLostError(RuntimeError):
    def __init__(self, missing, step, timeout_s):
        super().__init__(f"shard(s) {missing} did not reach call {step} within {timeout_s:.1f} s")
        self.missing = missing
        self.step = step


class PeerMonitor:
    """``step()`` = "I am about to make call number n; is everybody else?"."""

    def __init__(self, store, rank: int, world: int, timeout_s: float = 30.0, prefix: str = "mtj/alive"):
        self.store, self.rank, self.world = store, rank, world
        self.timeout_s = float(timeout_s)
        self.prefix = prefix
        self.count = 0

    @classmethod
    def from_process_group(cls, timeout_s: float = 30.0):
        import torch.distributed as dist
        from torch.distributed import distributed_c10d
        store = distributed_c10d._get_default_store()
        return cls(store, dist.get_rank(), dist.get_world_size(), timeout_s)

    def _key(self, rank):
        return f"{self.prefix}/{rank}"

    def step(self) -> int:
        self.count += 1
        self.store.set(self._key(self.rank), str(self.count))
        deadline = time.monotonic() + self.timeout_s
        pending = [r for r in range(self.world) if r != self.rank]
        while pending:
            still = []
            for r in pending:
                try:
                    seen = int(self.store.get(self._key(r))) if self.store.check([self._key(r)]) else 0
                except Exception:                       # the store's host itself is gone
                    seen = 0
                if seen < self.count:
                    still.append(r)
            pending = still
            if pending:
                if time.monotonic() >= deadline:
                    raise PeerLostError(pending, self.count, self.timeout_s)
                time.sleep(0.005)
        return self.count
