"""Launchers of the device barrier (symm_mem_recipes/triton_barrier.py:156-170)."""
from __future__ import annotations

import torch

from .._ext import C
from ..errors import SymmMemError
from ..parallel import symm_mem


def barrier_test(hdl: "symm_mem.SymmetricMemory", num_blocks: int = 32, threads: int = 128,
                 timeout_ms: int = symm_mem.DEFAULT_TIMEOUT_MS) -> None:
    """Launch a kernel whose CTAs only run `blockwise_barrier` against the CTA
    of the same index on every rank; upstream uses grid (32,1,1)
    (triton_barrier.py:165-170).  Success = `hdl.check()` passes and the pad is
    all zero again."""
    if hdl.kind != "cuda":
        raise SymmMemError("barrier_test launches a CUDA kernel; use hdl.barrier() on CPU")
    C.barrier_test(hdl.native, int(num_blocks), int(threads), int(timeout_ms) * 1_000_000)


def wait_flag(flag: torch.Tensor, target: int, timeout_ms: int) -> None:
    """Launch a one-thread kernel that waits (bounded) for `flag[0] >= target`.
    On expiry the device records a timeout status and the kernel returns."""
    C.wait_flag(flag, int(target), int(timeout_ms) * 1_000_000)
