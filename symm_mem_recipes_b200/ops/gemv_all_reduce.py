"""Fused GEMV + all-reduce for tensor-parallel decode.

    out[b, :] = sum over ranks of x_r[b, :] @ W_r          (b <= 16)

Row-parallel linear layer at decode time (for example the Llama-3-70B
down-projection at TP8: x [b, 3584], W [3584, 8192] per rank).  One kernel
streams the weight shard and reduces the partials across ranks through peer
stores; see csrc/kernels/gemv_allreduce.cu.  There is no upstream counterpart;
the library baseline is `reference_gemv_all_reduce` (cuBLAS + NCCL).
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
from .ag_matmul import _num_sms

_workspaces: dict[tuple, torch.Tensor] = {}
_LOCAL = "local"          # in place of a group: the workspace of the rank-local GEMV (a world of one)
_TIMEOUT_MS = int(os.environ.get("SMR_TIMEOUT_MS", "10000"))


def _workspace(batch_tile: int, N: int, K: int, device: torch.device, group, tensor_core: bool,
               sms: int, tagged: bool = False) -> torch.Tensor:
    """Symmetric scratch (inboxes, flags, epoch) for one (kernel, batch tile,
    N, K): allocated and rendezvoused at the first call, which is therefore
    collective; all ranks must make the same sequence of first calls."""
    local = group is _LOCAL
    ws = 1 if local or not dist.is_initialized() else dist.get_world_size(group)
    key = (tensor_core, tagged, batch_tile, N, K, device.index, _LOCAL if local else symm_mem._group_key(group))
    t = _workspaces.get(key)
    if t is None:
        if tensor_core:
            nbytes = C.gemv_tc_workspace_bytes(N, K, ws, sms, tagged)
        else:
            nbytes = C.gemv_workspace_bytes(batch_tile, N, ws)
        t = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        if local:
            symm_mem.rendezvous_local(t)
        else:
            symm_mem.rendezvous(t, group)
        _workspaces[key] = t
    return t


@traced("smr.gemv_all_reduce")
def gemv_all_reduce(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None,
                    group=None, timeout_ms: int = _TIMEOUT_MS, algo: Optional[str] = None,
                    weights_nk: bool = False) -> torch.Tensor:
    """`x` [B, K] and `w` [K, N] are this rank's (ordinary) tensors; returns the
    all-reduced [B, N] in bf16, bitwise identical on every rank.

    `algo`: "tc" = tcgen05 kernel (weights streamed by TMA, swap-A/B MMA),
    partial sums exchanged through inboxes and flags; "tc_tagged" = the same
    kernel exchanging its sums as {value, call number} words that the reducer
    polls directly (no flags, no release fence: one NVLink crossing on the
    critical path, twice the bytes); "simt" = CUDA-core kernel.  Default from
    SMR_GEMV_ALGO, else "tc_tagged" up to batch 8 and "tc" above (measured on 2
    and 4 GPUs: the tagged exchange is 2 to 9 µs faster up to batch 4 and 1.4 µs
    slower at batch 16).

    `weights_nk=True`: `w` is [N, K] (K contiguous), the layout
    `matmul_reduce_scatter` takes, so that one copy of a row-parallel weight
    serves prefill and decode (tcgen05 kernels only)."""
    k_dim, n_dim = (1, 0) if weights_nk else (0, 1)
    if x.dim() != 2 or w.dim() != 2 or x.shape[1] != w.shape[k_dim]:
        raise SymmMemError("need x[B, K] and w[K, N]" + (" given as [N, K]" if weights_nk else ""))
    B, N = x.shape[0], w.shape[n_dim]
    if not 1 <= B <= 16:
        raise SymmMemError("batch must be between 1 and 16 (decode); use matmul_reduce_scatter for prefill")
    if N % 8:
        raise SymmMemError("N must be a multiple of 8")
    if out is None:
        out = torch.empty(B, N, dtype=torch.bfloat16, device=x.device)
    algo = algo or os.environ.get("SMR_GEMV_ALGO") or ("tc_tagged" if B <= 8 and x.shape[1] % 8 == 0 else "tc")
    if algo not in ("tc", "simt", "tc_tagged"):
        raise SymmMemError('algo must be "tc", "tc_tagged" or "simt"')
    if algo == "tc_tagged" and x.shape[1] % 8:
        raise SymmMemError("the tcgen05 kernels need K to be a multiple of 8")
    tagged = algo == "tc_tagged"
    tensor_core = algo != "simt" and x.shape[1] % 8 == 0
    if weights_nk and not tensor_core:
        raise SymmMemError("weights_nk needs one of the tcgen05 kernels (K a multiple of 8)")
    sms = _num_sms(x.device)
    bt = 16 if tensor_core else C.gemv_batch_tile(B)
    wsp = _workspace(bt, N, x.shape[1], x.device, group, tensor_core, sms, tagged)
    hdl = symm_mem.rendezvous_local(wsp) if group is _LOCAL else symm_mem.rendezvous(wsp, group)
    C.gemv_all_reduce(x.contiguous(), w, out, hdl.native, 0, int(timeout_ms) * 1_000_000, tensor_core, sms, tagged,
                      bool(weights_nk))
    return out


def gemv(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, weights_nk: bool = False,
         timeout_ms: int = _TIMEOUT_MS) -> torch.Tensor:
    """Rank-local `x @ w` for a decode batch (1..16 rows) on the same kernels as `gemv_all_reduce`, with
    nobody to reduce with: the column-parallel projections of a decode step (QKV, gate / up), whose
    weights are streamed once from HBM.  `weights_nk=True`: `w` is [N, K], the layout of the prefill
    GEMMs' B operand.  Not collective; its scratch is a private world of one."""
    return gemv_all_reduce(x, w, out, group=_LOCAL, timeout_ms=timeout_ms, weights_nk=weights_nk)


def reference_gemv_all_reduce(x: torch.Tensor, w: torch.Tensor, group=None,
                              weights_nk: bool = False) -> torch.Tensor:
    """Library baseline: cuBLAS GEMM, then NCCL all-reduce (bf16)."""
    y = torch.matmul(x, w.t() if weights_nk else w)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(y, group=group)
    return y
