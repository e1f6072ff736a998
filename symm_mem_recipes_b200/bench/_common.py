"""Shared start-up / tear-down of the benchmark CLIs (one process per GPU)."""
from __future__ import annotations

import os

import torch
import torch.distributed as dist


def init_distributed(default_port: int = 29511):
    """Returns (rank, local_rank, world_size, device).  Initialises the NCCL
    process group once; later calls reuse it (the suite runs several benchmarks
    in one process)."""
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", str(default_port))
        dist.init_process_group("nccl", device_id=dev, rank=rank, world_size=world)
    return rank, local_rank, world, dev


def finish() -> None:
    from symm_mem_recipes_b200.parallel import symm_mem

    symm_mem.shutdown()
    if dist.is_initialized():
        dist.destroy_process_group()


def attempt(what: str, fn, dev, emit=None) -> bool:
    """Runs one section of a benchmark so that its failure does not end the run: the ranks agree
    on the outcome; after a device-side timeout they drop all symmetric memory together (the
    counters and barrier slots in use are then in an unknown state), so the sections after it
    start from fresh allocations.  Returns True when the section ran through on every rank;
    otherwise `emit` (if given) gets a record naming the section and the first error seen here."""
    import traceback

    from symm_mem_recipes_b200.errors import SymmMemTimeout
    from symm_mem_recipes_b200.parallel import symm_mem
    from symm_mem_recipes_b200.utils.benchmark import max_over_ranks

    err, timed_out = None, False
    try:
        fn()
    except SymmMemTimeout as e:
        err, timed_out = f"device-side timeout: {e}", True
    except Exception as e:  # noqa: BLE001 - reported; the benchmark goes on with its next section
        err = f"{type(e).__name__}: {e}"
        traceback.print_exc()
    failed = max_over_ranks(0.0 if err is None else 1.0, dev) != 0.0
    any_timeout = max_over_ranks(1.0 if timed_out else 0.0, dev) != 0.0
    if any_timeout:
        if dev.type == "cuda":
            try:                                       # a timeout recorded here but not yet read
                symm_mem.check_status(dev)
            except SymmMemTimeout:
                pass
        symm_mem.reset()
    if failed and emit is not None:
        emit({"op": "section_failed", "section": what, "error": err or "failed on another rank",
              "symmetric_memory_reset": any_timeout})
    return not failed
