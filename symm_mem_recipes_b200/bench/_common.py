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
