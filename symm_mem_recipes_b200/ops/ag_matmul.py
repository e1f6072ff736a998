"""all_gather_matmul: C = all_gather(A_shard) @ B^T with the gather running
inside the GEMM kernel.

API and behaviour follow
symm_mem_recipes/triton_all_gather_matmul.py:219-319
(`all_gather_matmul_tma_persistent(a_shard, b, a_out, c_out, configs,
mm_only)`): A is sharded on rows (tokens), B is given as [N, K], the fully
gathered A is a side output, and `mm_only=True` runs the GEMM alone.  The
NCCL + cuBLAS composition of :322-326 is `reference_all_gather_matmul`.

Dtypes: bfloat16, or float8_e4m3fn for A, B and C at once (upstream's
`FP8_OUTPUT` path, :123 and :311: the output takes the dtype of `a_shard`;
fp32 accumulation, no scale factors; N and K multiples of 16).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from .._ext import C
from ..errors import SymmMemError
from ..parallel import symm_mem
from ..utils.trace import traced

_BLOCK_NS = (256, 224, 192, 128)


def _env_int(name: str, default: int) -> int:
    v = os.environ.get(name)
    return int(v) if v not in (None, "") else default


@dataclass
class AgMatmulConfig:
    """Tile / scheduling knobs (upstream: a dict of BLOCK_SIZE_M/N/K,
    GROUP_SIZE_M, num_stages, num_warps; triton_all_gather_matmul.py:380-388).
    The M tile is 128 and the K tile 64; the stage count follows from BLOCK_N."""
    block_n: int = _env_int("SMR_AGMM_BLOCK_N", 0)        # 0 = pick per shape
    num_sms: int = _env_int("SMR_AGMM_NUM_SMS", 0)        # 0 = all SMs of the device
    # cut the tiles of a thinly filled last wave along K
    split_k_tail: bool = bool(_env_int("SMR_AGMM_SPLIT_K_TAIL", 1))
    # push gather: own 128-row blocks multiplied before the first remote one (-1 = the launcher's choice)
    lead: int = _env_int("SMR_AGMM_LEAD", -1)
    # push gather pacing (0 = the launcher's choice): rounds of tiles by which the broadcast runs ahead of the
    # first need
    push_ahead: int = _env_int("SMR_AGMM_PUSH_AHEAD", 0)
    # push gather by plain stores to every peer even where a multicast mapping exists (-1 = decide by world size)
    push_plain_stores: int = _env_int("SMR_AGMM_PUSH_PLAIN_STORES", -1)
    # pieces a 128-row block is cut into for the broadcast (0 = the launcher's choice)
    push_pieces: int = _env_int("SMR_AGMM_PUSH_PIECES", 0)
    # N tiles per column panel of the tile order (0 = the widest even split whose rows of B stay in L2)
    panel_w: int = _env_int("SMR_AGMM_PANEL_W", 0)
    timeout_ms: int = _env_int("SMR_TIMEOUT_MS", 10000)


DEFAULT_CONFIG = AgMatmulConfig()
_sm_count: dict[int, int] = {}
_tail_scratch: dict[int, torch.Tensor] = {}
_TAIL_SCRATCH_BYTES = 4096 + 37 * 8 * 2 * 128 * 256 * 4     # counters + the largest tail (37 tiles x 8 parts)


def _tail_buffer(device: torch.device, config: "AgMatmulConfig"):
    """Scratch of the split-K tail (fp32 partial accumulators), one per device."""
    if not config.split_k_tail:
        return None
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _tail_scratch.get(idx)
    if t is None:
        t = torch.empty(_TAIL_SCRATCH_BYTES, dtype=torch.uint8, device=device)
        _tail_scratch[idx] = t
    return t


def _push_plain_stores(config: "AgMatmulConfig", world_size: int) -> bool:
    """A multimem.st comes back to its sender too: at two ranks that doubles the bytes every GPU
    receives, so the broadcast through the switch is used from four ranks on."""
    if config.push_plain_stores >= 0:
        return bool(config.push_plain_stores)
    return world_size < 4


def _num_sms(device: torch.device) -> int:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _sm_count:
        _sm_count[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _sm_count[idx]


def choose_block_n(M: int, N: int, gemm_ctas: int) -> int:
    """Measured on B200: a tcgen05.mma of M = 128 rows per CTA takes the same
    time for every N <= 256, so the widest tile is the efficient one; narrower
    tiles only pay off when N itself is narrow (less zero padding streamed)."""
    del M, gemm_ctas
    for bn in sorted(_BLOCK_NS):
        if N <= bn:
            return bn
    return 256


_DTYPES = (torch.bfloat16, torch.float8_e4m3fn)


def _check_2d(name: str, t: torch.Tensor, dtype: Optional[torch.dtype] = None) -> None:
    if t.dim() != 2 or t.dtype not in _DTYPES or not t.is_cuda or not t.is_contiguous():
        raise SymmMemError(f"{name} must be a contiguous 2-D bfloat16 or float8_e4m3fn CUDA tensor")
    if dtype is not None and t.dtype != dtype:
        raise SymmMemError(f"{name} is {t.dtype}, expected {dtype}: A, B and C share one dtype")


def _check_nk(N: int, K: int, b: torch.Tensor, dtype: torch.dtype) -> None:
    align = 16 // dtype.itemsize       # elements per 16 bytes (TMA row pitch, vector stores)
    if b.shape[1] != K or N % align or K % align:
        raise SymmMemError(f"need B[N, K] with N and K multiples of {align}")


_EPILOGUES = {None: 0, "none": 0, "swiglu": 1}

# the words of one CTA's timing record (csrc/kernels/ag_matmul_common.cuh, namespace ag_trace): stamps are
# nanoseconds of %globaltimer, the others accumulated nanoseconds
TRACE_FIELDS = ("start", "entered", "flag_wait", "push", "acc_wait", "tiles_done", "tmem_wait", "operand_wait",
                "stage_wait", "end", "first_flag_wait", "tiles")


def summarize_trace(trace: torch.Tensor) -> dict:
    """Per-field summary (µs) of a timing record filled by `all_gather_matmul(..., trace=...)`:
    stamps relative to the earliest kernel entry, waits as mean and maximum over the CTAs that ran."""
    t = trace.view(-1, len(TRACE_FIELDS)).cpu()
    t = t[t[:, 0] > 0]
    if t.numel() == 0:
        return {}
    t0 = int(t[:, 0].min())
    out = {"ctas": int(t.shape[0])}
    for i, name in enumerate(TRACE_FIELDS):
        col = t[:, i]
        if name in ("start", "entered", "tiles_done", "end"):
            col = col[col > 0] - t0
            if col.numel():
                out[name] = {"min": round(float(col.min()) / 1e3, 1), "max": round(float(col.max()) / 1e3, 1)}
        elif name == "tiles":
            out[name] = {"min": int(col[col > 0].min()) if (col > 0).any() else 0, "max": int(col.max())}
        else:
            out[name] = {"mean": round(float(col.float().mean()) / 1e3, 1), "max": round(float(col.max()) / 1e3, 1)}
    return out


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor, group: int = 128) -> torch.Tensor:
    """Weight layout for `epilogue="swiglu"`: rows `[g*group, (g+1)*group)` of
    `w_gate` [F, K], then the same rows of `w_up`, for g = 0, 1, ...  With it
    every 256-column output tile holds 128 gate columns and their up columns.
    Done once when the weights are loaded.  F must be a multiple of `group`."""
    F, K = w_gate.shape
    if w_up.shape != w_gate.shape or F % group:
        raise SymmMemError(f"need w_gate and w_up of one shape [F, K] with F a multiple of {group}")
    return torch.stack([w_gate.view(F // group, group, K), w_up.view(F // group, group, K)], dim=1) \
        .reshape(2 * F, K).contiguous()


def _epilogue_code(epilogue, dtype: torch.dtype, N: int, config: "AgMatmulConfig") -> int:
    if epilogue not in _EPILOGUES:
        raise SymmMemError('epilogue must be None or "swiglu"')
    code = _EPILOGUES[epilogue]
    if code == 1:
        if dtype != torch.bfloat16 or N % 256 or config.block_n not in (0, 256):
            raise SymmMemError('epilogue="swiglu" needs bfloat16, block_n 256 and N % 256 == 0 '
                               "(B = interleave_gate_up(w_gate, w_up))")
    return code


@traced("smr.matmul")
def matmul(a: torch.Tensor, b: torch.Tensor, c_out: Optional[torch.Tensor] = None,
           config: AgMatmulConfig = DEFAULT_CONFIG, epilogue: Optional[str] = None,
           trace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """C[M, N] = A[M, K] @ B[N, K]^T on the tcgen05 kernel, no communication.
    `epilogue="swiglu"`: see `all_gather_matmul`."""
    _check_2d("a", a)
    _check_2d("b", b, a.dtype)
    M, K = a.shape
    N = b.shape[0]
    _check_nk(N, K, b, a.dtype)
    epi = _epilogue_code(epilogue, a.dtype, N, config)
    if c_out is None:
        c_out = torch.empty(M, N // 2 if epi else N, dtype=a.dtype, device=a.device)
    sms = config.num_sms or _num_sms(a.device)
    bn = 256 if epi else (config.block_n or choose_block_n(M, N, sms))
    C.ag_matmul(a, b, c_out, 0, None, 0, None, bn, sms, config.timeout_ms * 1_000_000,
                _tail_buffer(a.device, config), epi, trace, panel_w=config.panel_w)
    return c_out


_gather_buffers: dict[tuple, torch.Tensor] = {}


def _check_gather_geometry(notes: dict, geometry: tuple) -> None:
    """The arrival counters of the push gather live in the signal pad of the
    a_out allocation and count CALLS: block i has arrived when its counter
    reaches (calls so far) x (pieces per block).  That only holds while every
    call on one allocation gathers the same [M, K] at the same offset, so a
    second geometry on the same allocation is refused here instead of timing
    out on the device.  One symmetric buffer per gathered shape (what
    `gather_buffer` hands out) is the intended use."""
    seen = notes.setdefault("gather_geometry", geometry)
    if seen != geometry:
        raise SymmMemError(f"this symmetric allocation already serves a gather of (offset, M, K, dtype) = {seen}; "
                           f"got {geometry}.  Use one symmetric a_out per gathered shape.")


def gather_buffer(M: int, K: int, device: torch.device, group=None,
                  dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """The symmetric [M, K] buffer that `all_gather_matmul` gathers into when
    the caller passes no `a_out`.  Allocated and rendezvoused at first use
    (collective: every rank must reach it), then reused."""
    key = (M, K, device.index, symm_mem._group_key(group), dtype)
    t = _gather_buffers.get(key)
    if t is None:
        t = symm_mem.empty(M, K, dtype=dtype, device=device)
        symm_mem.rendezvous(t, group)
        _gather_buffers[key] = t
    return t


@traced("smr.all_gather_matmul")
def all_gather_matmul(a_shard: torch.Tensor, b: torch.Tensor, a_out: Optional[torch.Tensor] = None,
                      c_out: Optional[torch.Tensor] = None, config: AgMatmulConfig = DEFAULT_CONFIG,
                      mm_only: bool = False, group=None, epilogue: Optional[str] = None,
                      trace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """`a_shard` is this rank's [M/WS, K] rows of A; `b` is [N, K]; returns
    `c_out` [M, N] = all_gather(A) @ B^T and leaves the gathered A in `a_out`.

    Every rank broadcasts its own shard into the `a_out` of all ranks from
    inside the GEMM kernel (through the NVSwitch from four ranks on), so the
    gathered A has to land in symmetric memory:
      * `a_out` allocated with `symm_mem.empty`, or None (an internal symmetric
        buffer, see `gather_buffer`): gathered in place.
      * `a_out` an ordinary tensor, as in the upstream API: the gather goes into
        the internal buffer and one device-to-device copy fills `a_out`
        (measured on 4 GPUs at the Llama-3-70B shape: 795 µs, against 1940 µs
        for a kernel that pulled the peers' shards with copier CTAs).

    `mm_only=True` skips the gather and multiplies `a_out` (or `a_shard` when
    no `a_out` is given) as it is, to time the GEMM alone.

    `epilogue="swiglu"`: `b` is `interleave_gate_up(w_gate, w_up)` ([2F, K]) and
    the result is `SiLU(A @ w_gate^T) * (A @ w_up^T)`, [M, F], computed on the
    accumulators before they leave the SM (bf16, push gather or no gather).

    `trace`: an int64 CUDA tensor [num_sms, 12] that receives the per-CTA timing
    record of the CTA-pair kernel (`TRACE_FIELDS`; push gather or no gather).
    """
    _check_2d("a_shard", a_shard)
    _check_2d("b", b, a_shard.dtype)
    if mm_only:
        return matmul(a_out if a_out is not None else a_shard, b, c_out, config, epilogue, trace)
    rows, K = a_shard.shape
    N = b.shape[0]
    _check_nk(N, K, b, a_shard.dtype)
    epi = _epilogue_code(epilogue, a_shard.dtype, N, config)
    n_out = N // 2 if epi else N
    ws = dist.get_world_size(group) if dist.is_initialized() else 1
    M = rows * ws
    if c_out is None:
        c_out = torch.empty(M, n_out, dtype=a_shard.dtype, device=a_shard.device)
    if ws == 1:
        # nothing to gather: the shard is the gathered A; copy only on request
        matmul(a_shard, b, c_out, config, epilogue, trace)
        if a_out is not None:
            a_out.copy_(a_shard)
        return c_out
    if rows % 128:
        raise SymmMemError("rows per rank must be a multiple of 128 (the M tile and flag granularity)")
    if a_out is None:
        a_out = gather_buffer(M, K, a_shard.device, group, a_shard.dtype)
    if tuple(a_out.shape) != (M, K) or tuple(c_out.shape) != (M, n_out):
        raise SymmMemError("a_out must be [M, K] and c_out [M, N] ([M, N / 2] with the SwiGLU epilogue), "
                           "M = rows * world_size")
    sms = config.num_sms or _num_sms(a_shard.device)
    t_ns = config.timeout_ms * 1_000_000
    if not symm_mem.is_symm_mem_tensor(a_out):
        staged = gather_buffer(M, K, a_shard.device, group, a_shard.dtype)
        all_gather_matmul(a_shard, b, staged, c_out, config, group=group, epilogue=epilogue, trace=trace)
        a_out.copy_(staged)
        return c_out
    # every CTA is a GEMM CTA, the epilogue warps broadcast the shard
    bn = 256 if epi else (config.block_n or choose_block_n(M, N, sms))
    rec, aout_offset = symm_mem._find_record(a_out)
    hdl = symm_mem.rendezvous(a_out, group)
    if aout_offset % 16:
        raise SymmMemError("a_out must start on a 16-byte boundary of its allocation")
    _check_gather_geometry(rec.notes, (aout_offset, M, K, a_shard.dtype))
    C.ag_matmul(a_shard, b, c_out, 2, hdl.native, aout_offset, a_out, bn, sms, t_ns,
                _tail_buffer(a_shard.device, config), epi, trace, config.lead, config.push_ahead,
                _push_plain_stores(config, ws), config.push_pieces, config.panel_w)
    return c_out


def reference_all_gather_matmul(a_shard: torch.Tensor, b: torch.Tensor, group=None) -> torch.Tensor:
    """The library baseline: NCCL all-gather, then cuBLAS (upstream's
    `all_gather_matmul`, triton_all_gather_matmul.py:322-326).  `b` is [N, K]."""
    ws = dist.get_world_size(group)
    a = torch.empty(a_shard.shape[0] * ws, a_shard.shape[1], dtype=a_shard.dtype, device=a_shard.device)
    if a_shard.dtype == torch.float8_e4m3fn:
        # no fp8 reduction is involved: gather the bytes; the product is taken in bf16 and cast
        dist.all_gather_into_tensor(a.view(torch.uint8), a_shard.view(torch.uint8), group=group)
        return torch.matmul(a.to(torch.bfloat16), b.to(torch.bfloat16).t()).to(torch.float8_e4m3fn)
    dist.all_gather_into_tensor(a, a_shard, group=group)
    return torch.matmul(a, b.t())
