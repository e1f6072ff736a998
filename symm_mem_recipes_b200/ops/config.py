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
    # ... then one-shot (peer loads) up to this size (only when larger than ll_max_bytes)
    one_shot_max_bytes: int = _env_int("SMR_AR_ONE_SHOT_MAX_BYTES", 0)
    # Above one-shot: multimem when a multicast mapping exists, else two-shot.
    # CTA caps.  Upstream caps its one-shot kernel at 24 CTAs of 512 threads
    # (triton_one_shot_all_reduce.py:97-109); large messages want more.
    one_shot_max_blocks: int = _env_int("SMR_AR_ONE_SHOT_MAX_BLOCKS", 128)
    two_shot_max_blocks: int = _env_int("SMR_AR_TWO_SHOT_MAX_BLOCKS", 128)
    multimem_max_blocks: int = _env_int("SMR_AR_MULTIMEM_MAX_BLOCKS", 16)
    timeout_ms: int = _env_int("SMR_TIMEOUT_MS", 10000)


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
