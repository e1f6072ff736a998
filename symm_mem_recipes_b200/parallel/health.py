"""Host-side liveness of the ranks of a group, over the group's Store.

The kernels of this package wait for their peers with a deadline and report a
status when it runs out, but a rank that is already known to be gone should not
cost every survivor a full device-side timeout per launch.  `Heartbeat` lets
the survivors learn of it on the host, between steps, before they launch:

    hb = Heartbeat(group)              # every rank, after init_process_group
    for step in ...:
        hb.check()                     # raises PeerLost(rank, reason) instead of launching
        smr.all_gather_matmul(...)
    hb.stop()                          # announces an orderly leave

A rank leaves only between steps, with none of its kernels in flight (the
symmetric memory of a rank that disappears mid-kernel is gone for its peers;
the bounded device waits cover that case).  Upstream has no failure handling at
all: its waits spin for ever (symm_mem_recipes/triton_barrier.py:119-129,
triton_all_gather_matmul.py:80-83).

Timestamps are `time.time()` of the writing rank: all ranks of a group share
one host (intra-node NVLink only), so they are comparable.
"""
from __future__ import annotations

import threading
import time
from typing import Optional

import torch.distributed as dist

from ..errors import SymmMemError
from .store import _store_of


class PeerLost(SymmMemError):
    """A peer announced that it left, or its heartbeat went stale."""

    def __init__(self, rank: int, reason: str):
        self.rank, self.reason = int(rank), reason
        super().__init__(f"rank {rank} is gone: {reason}")


class Heartbeat:
    """Host-side liveness over the group's Store: a background thread of every
    rank publishes a time stamp every `interval_s`; `check()` raises `PeerLost`
    naming a rank that announced its leave (`stop()`) or whose stamp is stale.
    Call `check()` between steps, before launching kernels that wait on peers."""

    def __init__(self, group=None, interval_s: float = 0.5, store=None, rank: Optional[int] = None,
                 world_size: Optional[int] = None, namespace: str = "smr_health"):
        """`store`, `rank`, `world_size` default to those of `group` (the default
        group when None); pass them explicitly to use a Store without a process group."""
        self.rank = dist.get_rank(group) if rank is None else int(rank)
        self.world_size = dist.get_world_size(group) if world_size is None else int(world_size)
        base = _store_of(group) if store is None else store
        name = "world" if group is None else getattr(group, "group_name", str(id(group)))
        self.store = dist.PrefixStore(f"{namespace}/{name}", base)
        self.interval_s = float(interval_s)
        self._stop = threading.Event()
        self._beat()                                   # visible before the constructor returns
        self._thread = threading.Thread(target=self._run, name="smr-heartbeat", daemon=True)
        self._thread.start()

    def _beat(self) -> None:
        self.store.set(f"hb/{self.rank}", repr(time.time()))

    def _run(self) -> None:
        while not self._stop.wait(self.interval_s):
            try:
                self._beat()
            except Exception:      # noqa: BLE001  the Store went away with the job: nothing left to tell
                return

    def stop(self, leaving: bool = True) -> None:
        """Stops the heartbeat; with `leaving` the peers' next `check()` names this rank at once."""
        if self._stop.is_set():
            return
        self._stop.set()
        self._thread.join(timeout=5.0)
        if leaving:
            try:
                self.store.set(f"left/{self.rank}", "1")
            except Exception:      # noqa: BLE001
                pass

    def wait_for_all(self, timeout_s: float = 60.0) -> None:
        """Returns once every rank has written a first heartbeat."""
        deadline = time.time() + timeout_s
        keys = [f"hb/{r}" for r in range(self.world_size)]
        while not self.store.check(keys):
            if time.time() > deadline:
                missing = [r for r in range(self.world_size) if not self.store.check([f"hb/{r}"])]
                raise PeerLost(missing[0], "never started its heartbeat")
            time.sleep(0.01)

    def ages(self) -> dict:
        """rank -> seconds since its last heartbeat (None: none yet; -1.0: it announced a leave)."""
        now = time.time()
        out = {}
        for r in range(self.world_size):
            if self.store.check([f"left/{r}"]):
                out[r] = -1.0
            elif self.store.check([f"hb/{r}"]):
                out[r] = max(0.0, now - float(self.store.get(f"hb/{r}").decode()))
            else:
                out[r] = None
        return out

    def check(self, max_age_s: float = 3.0) -> None:
        """Raises PeerLost for the first peer that left or whose heartbeat is older than `max_age_s`."""
        for r, age in self.ages().items():
            if r == self.rank:
                continue
            if age is not None and age < 0:
                raise PeerLost(r, "it announced that it left")
            if age is None:
                raise PeerLost(r, "it never started its heartbeat")
            if age > max_age_s:
                raise PeerLost(r, f"last heartbeat {age:.1f} s ago")
