"""Launchers of the device barrier (symm_mem_recipes/triton_barrier.py:156-170)."""
from __future__ import annotations

import torch

from .._ext import C
from ..errors import SymmMemError
from ..parallel import symm_mem


_KINDS = {"cas": 0, "epoch": 1, "nvls": 2}


def barrier_test(hdl: "symm_mem.SymmetricMemory", num_blocks: int = 32, threads: int = 128,
                 timeout_ms: int = symm_mem.DEFAULT_TIMEOUT_MS, kind: str = "cas") -> None:
    """Launch a kernel whose CTAs only run a device barrier against the CTA of
    the same index on every rank; upstream uses grid (32,1,1)
    (triton_barrier.py:165-170).  Success = `hdl.check()` passes and, for the
    default kind, the pad is all zero again.

    `kind`: "cas" = `blockwise_barrier` (upstream's protocol); "epoch" = one
    release store per peer and a poll of the own pad (what the two-shot and
    multimem all-reduce use); "nvls" = one `multimem.red` per rank on a counter
    in the multicast mapping of the pad (needs `hdl.has_multicast`).  The two
    counting kinds run the barrier twice and leave growing counters behind."""
    if hdl.kind != "cuda":
        raise SymmMemError("barrier_test launches a CUDA kernel; use hdl.barrier() on CPU")
    if kind not in _KINDS:
        raise SymmMemError(f"kind must be one of {sorted(_KINDS)}")
    if kind == "nvls" and not hdl.has_multicast:
        raise SymmMemError("the NVLS barrier needs a multicast mapping")
    C.barrier_test(hdl.native, int(num_blocks), int(threads), int(timeout_ms) * 1_000_000, _KINDS[kind])


def wait_flag(flag: torch.Tensor, target: int, timeout_ms: int) -> None:
    """Launch a one-thread kernel that waits (bounded) for `flag[0] >= target`.
    On expiry the device records a timeout status and the kernel returns."""
    C.wait_flag(flag, int(target), int(timeout_ms) * 1_000_000)
