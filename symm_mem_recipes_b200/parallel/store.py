"""Out-of-band exchange between ranks through a torch.distributed Store.

The rendezvous of a symmetric allocation needs a few small host-side messages
(socket names, sizes, phase barriers).  They go through the process group's
Store (TCPStore under torchrun), never through the GPU, so the same code
serves `nccl` and `gloo` groups.
"""
from __future__ import annotations

import pickle
from datetime import timedelta

import torch.distributed as dist


def _store_of(group) -> "dist.Store":
    c10d = dist.distributed_c10d
    if group is None or group is dist.group.WORLD:
        return c10d._get_default_store()
    return c10d._get_process_group_store(group)


class StoreExchange:
    """all_gather / barrier of picklable objects among the ranks of a group."""

    def __init__(self, group=None, namespace: str = "smr", timeout_s: float = 120.0):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world_size = dist.get_world_size(group)
        name = "world" if group is None or group is dist.group.WORLD else \
            (getattr(group, "group_name", None) or str(id(group)))
        self.store = dist.PrefixStore(f"{namespace}/{name}", _store_of(group))
        self.timeout = timedelta(seconds=timeout_s)
        self._seq = 0

    def all_gather(self, obj) -> list:
        """Every rank's picklable `obj`, in rank order (collective; raises when a rank stays away past the timeout)."""
        seq = self._seq
        self._seq += 1
        self.store.set(f"{seq}/{self.rank}", pickle.dumps(obj))
        keys = [f"{seq}/{r}" for r in range(self.world_size)]
        self.store.wait(keys, self.timeout)
        out = [pickle.loads(self.store.get(k)) for k in keys]
        # Every rank has now read round seq - 2: a rank can only publish round seq after it has
        # finished reading round seq - 1, and this rank has just seen every rank's round seq.
        # So this rank's own key of round seq - 2 can go; the Store stays at two rounds per group.
        if seq >= 2:
            try:
                self.store.delete_key(f"{seq - 2}/{self.rank}")
            except Exception:  # noqa: BLE001 - a Store without delete support just keeps the key
                pass
        return out

    def barrier(self) -> None:
        self.all_gather(None)
