"""Per-op configuration: one dataclass per op, overridable by `SMR_*`
environment variables (the upstream recipes use module constants and a plain
dict of tile sizes: symm_mem_recipes/triton_one_shot_all_reduce.py:97-100,
symm_mem_recipes/triton_all_gather_matmul.py:380-388)."""
from __future__ import annotations

import json
import os
from dataclasses import dataclass


def _env_int(name: str, default: int) -> int:
    v = os.environ.get(name)
    return int(v) if v not in (None, "") else default


@dataclass
class AllReduceConfig:
    """Thresholds and launch sizes of the all-reduce kernels (the upstream
    wrapper hard-codes its own: 512 threads, at most 24 CTAs,
    symm_mem_recipes/triton_one_shot_all_reduce.py:97-109).  Every field has an
    SMR_AR_* environment override; `from_tuning` loads thresholds derived from
    a measured sweep."""
    # Message sizes (bytes) up to which each algorithm is picked by `algo="auto"`.
    # low-latency push kernel (tagged words, no barrier) up to this size ...
    ll_max_bytes: int = _env_int("SMR_AR_LL_MAX_BYTES", 256 * 1024)
    ll_max_blocks: int = _env_int("SMR_AR_LL_MAX_BLOCKS", 128)
    # ... then one-shot (peer loads) up to this size (only when larger than ll_max_bytes);
    # -1 = by world size (`one_shot_limit`)
    one_shot_max_bytes: int = _env_int("SMR_AR_ONE_SHOT_MAX_BYTES", -1)
    # ... then two-shot up to this size; -1 = by world size (`two_shot_limit`)
    two_shot_max_bytes: int = _env_int("SMR_AR_TWO_SHOT_MAX_BYTES", -1)
    # Above that: multimem when a multicast mapping exists, else two-shot.
    # CTA caps.  Upstream caps its one-shot kernel at 24 CTAs of 512 threads
    # (triton_one_shot_all_reduce.py:97-109); large messages want more.
    one_shot_max_blocks: int = _env_int("SMR_AR_ONE_SHOT_MAX_BLOCKS", 128)
    two_shot_max_blocks: int = _env_int("SMR_AR_TWO_SHOT_MAX_BLOCKS", 128)
    # 0 = by world size (`multimem_blocks`)
    multimem_max_blocks: int = _env_int("SMR_AR_MULTIMEM_MAX_BLOCKS", 0)
    timeout_ms: int = _env_int("SMR_TIMEOUT_MS", 10000)

    def one_shot_limit(self, world_size: int) -> int:
        """Largest message for which `algo="auto"` takes the one-shot kernel.  `all_reduce` works
        in place, and one-shot must then wait for every peer to have read the input before it
        may overwrite it: a second barrier and a second pass, about 5.5 µs.  Measured on two and
        four B200s, the one-shot kernel alone beats two-shot from 256 KiB to 1 MiB (12.2 against
        15.3 µs at 512 KiB on four ranks) but loses with that write-back (17.7 µs), so by default
        the dispatcher never picks it; callers that can take the sum in a new tensor call
        `one_shot_all_reduce` themselves."""
        return self.one_shot_max_bytes if self.one_shot_max_bytes >= 0 else 0

    def two_shot_limit(self, world_size: int) -> int:
        """Largest message for which `algo="auto"` prefers the two-shot kernel (peer loads, peer
        stores) to the in-switch reduction.  Measured: with two ranks the switch has nothing to
        save and its broadcast also returns to the sender (119 against 193 µs at 64 MiB, 15.1
        against 13.4-17.0 at 1 MiB); with four ranks two-shot wins up to 1 MiB (15.3 against
        15.4-18.4 µs at 512 KiB, 16.3 against 17.6-19.9 at 1 MiB) and the two are within noise of
        each other up to 4 MiB, from where multimem wins (35.3 against 41.3 µs at 8 MiB); with
        eight ranks multimem won at every size above the low-latency kernel's range."""
        if self.two_shot_max_bytes >= 0:
            return self.two_shot_max_bytes
        if world_size <= 2:
            return 1 << 62
        return 1024 * 1024 if world_size <= 4 else 0

    def multimem_blocks(self, world_size: int) -> int:
        """CTAs of the multimem kernel: a few CTAs with eight reductions in flight per thread
        saturate the NVSwitch port; more only add barrier traffic.  Measured at 64 MiB, bus
        bandwidth with 4 / 8 / 16 / 24 CTAs: 733 / 741 / 707 / 689 GB/s on eight ranks, 539 / 605 /
        598 / 577 GB/s on four; at 1 MiB 8 and 16 CTAs tie (16.9 / 16.8 µs on eight ranks)."""
        return self.multimem_max_blocks if self.multimem_max_blocks > 0 else 8

    @staticmethod
    def from_tuning(path: str, world_size: int = 0) -> "AllReduceConfig":
        """Thresholds measured on the machine at hand: `path` is the JSON written by
        `python -m symm_mem_recipes_b200.bench.tune_all_reduce` ({"by_world_size": {"8": {...}}}).
        Fields the file does not name keep their defaults; `world_size` 0 takes the
        largest world size in the file."""
        with open(path) as f:
            table = json.load(f)["by_world_size"]
        key = str(world_size) if world_size else max(table, key=int)
        if key not in table:
            raise KeyError(f"{path} has no entry for world size {key}; it has {sorted(table, key=int)}")
        cfg = AllReduceConfig()
        for name, value in table[key].items():
            if name in cfg.__dataclass_fields__:
                setattr(cfg, name, int(value))
        return cfg


def _default_all_reduce() -> AllReduceConfig:
    path = os.environ.get("SMR_AR_TUNING_FILE")
    return AllReduceConfig.from_tuning(path) if path else AllReduceConfig()


DEFAULT_ALL_REDUCE = _default_all_reduce()
