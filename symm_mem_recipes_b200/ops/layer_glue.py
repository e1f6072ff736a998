"""Rank-local glue of a decoder layer as single-pass CUDA kernels: RMSNorm
(optionally fused with the residual add before it), rotary embedding in place
on the QKV buffer, and SiLU(gate) * up.  bf16 data, fp32 math.

No upstream counterpart.  They exist because the PyTorch compositions
(`x.float()...`, `torch.cat`, `F.silu(g.float()) * u.float()`) make five to
ten passes with fp32 temporaries over tensors as large as the GEMM outputs,
which at Llama-70B prefill sizes costs more than the o-projection GEMM.
"""
from __future__ import annotations

from typing import Optional, Union

import torch

from .._ext import C
from ..errors import SymmMemError
from ..utils.trace import traced
from .ag_matmul import _num_sms


def _check(name: str, t: torch.Tensor, dim: int) -> None:
    if t.dim() != dim or t.dtype != torch.bfloat16 or not t.is_cuda or not t.is_contiguous():
        raise SymmMemError(f"{name} must be a contiguous {dim}-D bfloat16 CUDA tensor")


@traced("smr.rms_norm")
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: Optional[torch.Tensor] = None,
             residual: Optional[torch.Tensor] = None, sum_out: Optional[torch.Tensor] = None):
    """`out = bf16(bf16(s * rsqrt(mean(s^2) + eps)) * weight)` per row of `s`,
    where `s = x`, or `bf16(x + residual)` when a residual is given (then `s`
    itself is written to `sum_out`, which may be `x` or `residual` for a residual
    stream kept in place).  `out` may be a symmetric buffer, so the result lands
    where `all_gather_matmul` reads it, or `x` itself without a residual.  Returns
    `out`, or `(out, sum_out)` with a residual."""
    _check("x", x, 2)
    _check("weight", weight, 1)
    if x.shape[1] % 8 or weight.shape[0] != x.shape[1]:
        raise SymmMemError("need x[rows, H], weight[H] with H a multiple of 8")
    if out is None:
        out = torch.empty_like(x)
    if residual is not None and sum_out is None:
        sum_out = torch.empty_like(x)
    if residual is None and sum_out is not None:
        raise SymmMemError("sum_out is only written when a residual is given")
    if residual is not None:
        _check("residual", residual, 2)
        _check("sum_out", sum_out, 2)
        if residual.shape != x.shape or sum_out.shape != x.shape:
            raise SymmMemError("residual and sum_out must have the shape of x")
        if out.data_ptr() in (sum_out.data_ptr(), residual.data_ptr()):
            raise SymmMemError("out must not be the buffer of sum_out or of the residual "
                               "(sum_out may be the buffer of x or of the residual)")
    _check("out", out, 2)
    if out.shape != x.shape:
        raise SymmMemError("out must have the shape of x")
    C.rms_norm(x, residual, weight, sum_out, out, float(eps))
    return out if residual is None else (out, sum_out)


@traced("smr.rope_")
def rope_(qkv: torch.Tensor, n_heads: int, head_dim: int, seq: int, theta: float,
          pos0: Union[int, torch.Tensor] = 0) -> torch.Tensor:
    """Rotate heads `[0, n_heads)` of every row of `qkv` [tokens, row] in place
    (Llama pairing `(i, i + head_dim/2)`); token `t` is at position
    `pos0 + t % seq`.  With the Q heads followed by the K heads at the start of
    the row, `n_heads = q_heads + kv_heads` rotates both and leaves V alone.
    `pos0` may be an int32 tensor of one element on the same device: the kernel
    then reads the position when it runs, so a decode step captured in a CUDA
    graph serves every position."""
    _check("qkv", qkv, 2)
    if head_dim % 16 or n_heads * head_dim > qkv.shape[1] or qkv.shape[1] % 8:
        raise SymmMemError("need head_dim % 16 == 0, n_heads * head_dim <= row length, row length % 8 == 0")
    if isinstance(pos0, torch.Tensor):
        if pos0.dtype != torch.int32 or pos0.numel() != 1 or pos0.device != qkv.device:
            raise SymmMemError("a position tensor must be int32, of one element, on qkv's device")
        C.rope_inplace(qkv, int(n_heads), int(head_dim), int(seq), 0, float(theta), _num_sms(qkv.device), pos0)
    else:
        C.rope_inplace(qkv, int(n_heads), int(head_dim), int(seq), int(pos0), float(theta), _num_sms(qkv.device))
    return qkv


@traced("smr.silu_mul")
def silu_mul(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """`out[rows, F] = SiLU(gate_up[:, :F]) * gate_up[:, F:]`."""
    _check("gate_up", gate_up, 2)
    if gate_up.shape[1] % 16:
        raise SymmMemError("gate_up must be [rows, 2F] with F a multiple of 8")
    if out is None:
        out = torch.empty(gate_up.shape[0], gate_up.shape[1] // 2, dtype=torch.bfloat16, device=gate_up.device)
    C.silu_mul(gate_up, out, _num_sms(gate_up.device))
    return out


_attn_scratch: dict[tuple, torch.Tensor] = {}


@traced("smr.decode_attention_")
def decode_attention_(qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, n_q_heads: int,
                      pos: Union[int, torch.Tensor], out: Optional[torch.Tensor] = None,
                      rope_theta: float = 0.0) -> torch.Tensor:
    """Attention of one decode step in one kernel.  `qkv` [B, (hq + 2 hkv) * D]
    holds the new token's queries and keys and its values; with `rope_theta`
    (say 500000.0) queries and key are given unrotated and the kernel applies
    the rotary embedding for position `pos` itself (same bits as `rope_` first),
    otherwise they must be rotated already.  `qkv` is not modified.  The caches
    are [B, S_max, hkv, D].  Writes the new (rotated) key and the value into
    the caches at `pos` (hence the trailing underscore) and returns
    `out[B, hq * D] = softmax(q . K[0..pos] / sqrt(D)) V[0..pos]` per query head
    (grouped-query: head h reads KV head h // (hq / hkv)).  The cached sequence
    is split over CTAs whatever the position, and `pos` may be an int32 tensor
    of one element on the device, so a captured CUDA graph serves every
    position.  Replaces, in a decode step, two cache writes and PyTorch's
    attention under a mask (about ten small kernels).  D is 64 or 128 and
    hq / hkv at most 8.  Calls of one shape share a scratch buffer: issue them
    on one stream (or in one captured graph), not concurrently."""
    _check("qkv", qkv, 2)
    _check("k_cache", k_cache, 4)
    _check("v_cache", v_cache, 4)
    B, s_max, hkv, D = k_cache.shape
    if v_cache.shape != k_cache.shape or qkv.shape != (B, (n_q_heads + 2 * hkv) * D):
        raise SymmMemError("need caches [B, S_max, hkv, D] and qkv [B, (hq + 2 hkv) * D]")
    if n_q_heads % hkv or n_q_heads // hkv > 8 or D not in (64, 128):
        raise SymmMemError("need hq a multiple of hkv with hq / hkv <= 8, and head_dim 64 or 128")
    if rope_theta != 0.0 and rope_theta <= 1.0:
        raise SymmMemError("rope_theta must be 0 (no rotation) or larger than 1")
    if out is None:
        out = torch.empty(B, n_q_heads * D, dtype=torch.bfloat16, device=qkv.device)
    key = (qkv.device.type, qkv.device.index, B, hkv, D, s_max)
    scratch = _attn_scratch.get(key)
    if scratch is None:
        scratch = torch.zeros(C.decode_attention_scratch_bytes(B, hkv, D, s_max), dtype=torch.uint8, device=qkv.device)
        _attn_scratch[key] = scratch
    if isinstance(pos, torch.Tensor):
        if pos.dtype != torch.int32 or pos.numel() != 1 or pos.device != qkv.device:
            raise SymmMemError("a position tensor must be int32, of one element, on qkv's device")
        C.decode_attention(qkv, k_cache, v_cache, out, scratch, int(n_q_heads), int(hkv), 0, pos, float(rope_theta))
    else:
        if not 0 <= int(pos) < s_max:
            raise SymmMemError(f"position {pos} outside the cache of {s_max} entries")
        C.decode_attention(qkv, k_cache, v_cache, out, scratch, int(n_q_heads), int(hkv), int(pos), None,
                           float(rope_theta))
    return out
