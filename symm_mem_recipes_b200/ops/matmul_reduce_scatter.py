"""Fused GEMM + reduce-scatter: the row-parallel linear layer of a
tensor-parallel block at prefill time (o-proj, down-proj).

    out_r[M/WS, N] = ( sum over ranks s of  A_s[M, K_s] @ B_s[N, K_s]^T ) [rows of rank r]

One tcgen05 kernel (CTA pairs, `cta_group::2`) multiplies, ships every tile
straight from its epilogue to the rank that owns those rows, and reduces what
arrives; see csrc/kernels/matmul_rs_sm100.cu.  Together with `all_gather_matmul` it keeps
activations sharded on tokens between the layers (sequence parallelism).  The
upstream package has no reduce-scatter half; the library baseline is
`reference_matmul_reduce_scatter` (cuBLAS + NCCL).
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist

from .._ext import C
from ..errors import SymmMemError
from ..parallel import symm_mem
from ..utils.trace import traced
from .ag_matmul import _num_sms, matmul

_workspaces: dict[tuple, torch.Tensor] = {}
_TIMEOUT_MS = int(os.environ.get("SMR_TIMEOUT_MS", "10000"))
_PANEL_W = int(os.environ.get("SMR_RS_PANEL_W", "0"))


def _workspace(M: int, N: int, device: torch.device, group) -> torch.Tensor:
    """Symmetric inbox [WS, M/WS, N] bf16 (= M*N*2 bytes per rank), allocated and
    rendezvoused at first use (collective), shared by all calls of that shape."""
    key = (M, N, device.index, symm_mem._group_key(group))
    t = _workspaces.get(key)
    if t is None:
        t = symm_mem.empty(C.matmul_rs_workspace_bytes(M, N), dtype=torch.uint8, device=device)
        symm_mem.rendezvous(t, group)
        _workspaces[key] = t
    return t


@traced("smr.matmul_reduce_scatter")
def matmul_reduce_scatter(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None,
                          group=None, num_sms: int = 0, timeout_ms: int = _TIMEOUT_MS,
                          trace: Optional[torch.Tensor] = None, panel_w: int = _PANEL_W) -> torch.Tensor:
    """`a` [M, K_local] (all tokens, this rank's slice of the reduction
    dimension), `b` [N, K_local]; returns this rank's [M/WS, N] rows of the sum
    over ranks, bitwise identical to what any other summation site would get
    (fp32 sum in rank order of bf16 partials).

    `trace`: optional int64 CUDA tensor [num_sms, 4]; every CTA writes its
    %globaltimer (ns) at kernel start, after the entry barrier, when its GEMM
    tiles are pushed, and when its share of the reduction is done.
    `panel_w`: N tiles (of 256 columns) per column panel of the tile order; 0
    lets the launcher keep a panel's rows of `b` within the L2."""
    if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[1]:
        raise SymmMemError("need a[M, K] and b[N, K]")
    ws = dist.get_world_size(group) if dist.is_initialized() else 1
    M, K = a.shape
    N = b.shape[0]
    if ws == 1:
        return matmul(a, b, out)
    if M % (ws * 128) or N % 8 or K % 8:
        raise SymmMemError("need M a multiple of 128 * world_size, N and K multiples of 8")
    if out is None:
        out = torch.empty(M // ws, N, dtype=torch.bfloat16, device=a.device)
    wsp = _workspace(M, N, a.device, group)
    hdl = symm_mem.rendezvous(wsp, group)
    C.matmul_reduce_scatter(a, b, out, hdl.native, num_sms or _num_sms(a.device),
                            int(timeout_ms) * 1_000_000, trace, int(panel_w))
    return out


_ar_outputs: dict[tuple, torch.Tensor] = {}


@traced("smr.matmul_all_reduce")
def matmul_all_reduce(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None, group=None,
                      num_sms: int = 0, timeout_ms: int = _TIMEOUT_MS) -> torch.Tensor:
    """The same kernel with an all-reduce ending, for tensor parallelism without
    sequence parallelism: every rank gets the whole [M, N] sum.  Rank r reduces
    its M/WS rows as in `matmul_reduce_scatter` and then broadcasts them into
    the output of every rank (one `multimem.st` through the NVSwitch, or plain
    stores to every peer); an exit barrier inside the kernel proves that all
    rows have landed.  Same bits on every rank.

    `out` must live in symmetric memory (peers write into it).  With
    `out=None` an internal symmetric [M, N] buffer per shape is used and
    returned: it is overwritten by the next call of that shape."""
    if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[1]:
        raise SymmMemError("need a[M, K] and b[N, K]")
    ws = dist.get_world_size(group) if dist.is_initialized() else 1
    M, K = a.shape
    N = b.shape[0]
    if ws == 1:
        return matmul(a, b, out)
    if M % (ws * 128) or N % 8 or K % 8:
        raise SymmMemError("need M a multiple of 128 * world_size, N and K multiples of 8")
    if out is None:
        key = (M, N, a.device.index, symm_mem._group_key(group))
        out = _ar_outputs.get(key)
        if out is None:
            out = symm_mem.empty(M, N, dtype=torch.bfloat16, device=a.device)
            symm_mem.rendezvous(out, group)
            _ar_outputs[key] = out
    if not symm_mem.is_symm_mem_tensor(out) or tuple(out.shape) != (M, N):
        raise SymmMemError("out must be a symmetric [M, N] tensor (symm_mem.empty): every rank writes into it")
    _, out_offset = symm_mem._find_record(out)
    out_hdl = symm_mem.rendezvous(out, group)
    wsp = _workspace(M, N, a.device, group)
    hdl = symm_mem.rendezvous(wsp, group)
    C.matmul_all_reduce(a, b, out, out_hdl.native, out_offset, hdl.native, num_sms or _num_sms(a.device),
                        int(timeout_ms) * 1_000_000, _PANEL_W)
    return out


def reference_matmul_all_reduce(a: torch.Tensor, b: torch.Tensor, group=None) -> torch.Tensor:
    """Library baseline: cuBLAS GEMM, then NCCL all-reduce (bf16)."""
    full = torch.matmul(a, b.t())
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(full, group=group)
    return full


def reference_matmul_reduce_scatter(a: torch.Tensor, b: torch.Tensor, group=None) -> torch.Tensor:
    """Library baseline: cuBLAS GEMM, then NCCL reduce-scatter (bf16)."""
    full = torch.matmul(a, b.t())
    ws = dist.get_world_size(group) if dist.is_initialized() else 1
    if ws == 1:
        return full
    out = torch.empty(full.shape[0] // ws, full.shape[1], dtype=full.dtype, device=full.device)
    dist.reduce_scatter_tensor(out, full, group=group)
    return out
