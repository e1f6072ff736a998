"""The upstream recipes' entry points under their own names and signatures,
for code that was written against `symm_mem_recipes` and moves here.

    upstream (symm_mem_recipes.*)                         here
    ---------------------------------------------------   -----------------------------------------
    triton_all_gather_matmul.all_gather_matmul_tma_persistent(a_shard, b, a_out, c_out, configs, mm_only)
                                                          all_gather_matmul_tma_persistent (same arguments)
    triton_all_gather_matmul.all_gather_matmul(a_shard, b)   (NCCL + cuBLAS)
                                                          all_gather_matmul_baseline
    triton_all_gather_matmul.all_gather_with_progress(output, inp, progress, splits_per_rank)
                                                          all_gather_with_progress (same arguments)
    triton_one_shot_all_reduce.one_shot_all_reduce(tensor)   one_shot_all_reduce
    triton_barrier.barrier_test(symm_mem)                 barrier_test
    utils.benchmark_with_event / benchmark_with_profiler  the same names

Note the one name that changes meaning: upstream's `all_gather_matmul` is its
library BASELINE (triton_all_gather_matmul.py:322-326); in this package the
name belongs to the fused op, and the baseline is `reference_all_gather_matmul`
(`all_gather_matmul_baseline` here).
"""
from __future__ import annotations

from typing import Optional

import torch

from .errors import SymmMemError
from .ops import barrier_test, one_shot_all_reduce  # noqa: F401  (re-exported)
from .ops.ag_matmul import DEFAULT_CONFIG, AgMatmulConfig, all_gather_matmul, reference_all_gather_matmul
from .parallel import symm_mem
from .utils.benchmark import benchmark_with_event, benchmark_with_profiler  # noqa: F401  (re-exported)

all_gather_matmul_baseline = reference_all_gather_matmul


def _config_from_dict(configs: Optional[dict]) -> AgMatmulConfig:
    """Upstream passes tile sizes as a dict (triton_all_gather_matmul.py:380-388).  Only
    BLOCK_SIZE_N is a free parameter of the tcgen05 kernels (128, 192, 224 or 256; anything
    else lets the kernel choose); the M tile (128 per CTA), the K tile (64), the stage count
    and the warp roles are fixed by their design and the other keys are accepted and ignored."""
    if not configs:
        return DEFAULT_CONFIG
    bn = int(configs.get("BLOCK_SIZE_N", 0))
    return AgMatmulConfig(block_n=bn if bn in (128, 192, 224, 256) else 0)


def all_gather_matmul_tma_persistent(a_shard: torch.Tensor, b: torch.Tensor, a_out: torch.Tensor,
                                     c_out: torch.Tensor, configs: Optional[dict] = None,
                                     mm_only: bool = False) -> torch.Tensor:
    """Upstream signature (triton_all_gather_matmul.py:219-226) on the fused kernel of this
    package.  `a_out` may be an ordinary tensor, as upstream allocates it (:376): the gather then
    goes through an internal symmetric buffer and one copy; a symmetric one (`symm_mem.empty`)
    is gathered into directly."""
    return all_gather_matmul(a_shard, b, a_out, c_out, _config_from_dict(configs), mm_only)


def all_gather_with_progress(output: torch.Tensor, inp: torch.Tensor, progress: torch.Tensor,
                             splits_per_rank: int) -> None:
    """Host-driven all-gather of the symmetric tensor `inp` into `output` with one flag per
    chunk: chunks are copied from the peers nearest neighbour first and own shard last, and
    `progress[chunk]` becomes 1, in stream order (the driver's stream memory operation on a
    32-bit CUDA tensor, a one-element fill otherwise), once its copy is complete; a barrier at
    the end keeps any rank from overwriting `inp` while a peer still reads it.  Everything is
    queued on the CURRENT stream: a caller that wants the gather beside a kernel enters
    `torch.cuda.stream(side)` around the call, as upstream does.  Same contract as
    upstream (triton_all_gather_matmul.py:20-56), where a kernel on another stream polls the
    flags.  The fused kernel of this package does not use it (its gather runs inside the
    GEMM); it is here for code that consumes the flags itself."""
    if not inp.is_contiguous():
        raise SymmMemError("inp must be contiguous")
    hdl = symm_mem.rendezvous(inp)
    _, inp_offset_bytes = symm_mem._find_record(inp)
    ws, rank = hdl.world_size, hdl.rank
    if inp.numel() % splits_per_rank or progress.numel() != ws * splits_per_rank:
        raise SymmMemError("need inp.numel() % splits_per_rank == 0 and one progress slot per chunk")
    want = [inp.shape[0] * ws, *inp.shape[1:]]
    if list(output.shape) != want:
        raise SymmMemError(f"output must have shape {want}, got {list(output.shape)}")
    chunks = output.chunk(ws * splits_per_rank)
    chunk_numel = chunks[0].numel()
    base = inp_offset_bytes // inp.element_size()
    flags = progress.view(-1)
    for distance in range(1, ws + 1):
        src = (rank + distance) % ws
        for split in range(splits_per_rank):
            idx = src * splits_per_rank + split
            chunks[idx].copy_(hdl.get_buffer(src, chunks[0].shape, inp.dtype, base + chunk_numel * split))
            hdl.stream_write_value32(flags, idx, 1)   # ordered after the copy on the current stream
    hdl.barrier()
