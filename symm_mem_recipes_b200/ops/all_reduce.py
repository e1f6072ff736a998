"""bf16 all-reduce over symmetric memory: one-shot, two-shot, multimem and a
size-based dispatcher.

`one_shot_all_reduce(tensor)` keeps the contract of
symm_mem_recipes/triton_one_shot_all_reduce.py:96-125: bf16, numel % 8 == 0,
symmetric input, a fresh local output, and the same bits on every rank
(ordered bf16 sum).  The in-place variants have no upstream counterpart.
"""
from __future__ import annotations

from typing import Optional

import torch

from .._ext import C
from ..errors import SymmMemError, raise_for_status
from ..parallel import symm_mem
from ..utils.trace import traced
from .config import DEFAULT_ALL_REDUCE, AllReduceConfig

_ALGOS = ("auto", "low_latency", "one_shot", "two_shot", "multimem")
_LL_CAPACITY_NUMEL = 128 * 1024          # elements: messages up to 256 KiB
_ll_workspaces: dict[tuple, torch.Tensor] = {}


def _prepare(t: torch.Tensor):
    if t.dtype != torch.bfloat16:
        raise SymmMemError("only bfloat16 is supported")
    if t.numel() % 8 != 0:
        raise SymmMemError("the number of elements must be a multiple of 8 (128-bit accesses)")
    if not t.is_contiguous():
        raise SymmMemError("the tensor must be contiguous")
    rec, offset = symm_mem._find_record(t)
    hdl = symm_mem.rendezvous(t)
    if offset % 16 != 0:
        raise SymmMemError("the tensor must start on a 16-byte boundary of its allocation")
    return hdl, offset


@traced("smr.one_shot_all_reduce")
def one_shot_all_reduce(t: torch.Tensor, *, exit_barrier: bool = False,
                        out: Optional[torch.Tensor] = None, write_back: bool = False,
                        config: AllReduceConfig = DEFAULT_ALL_REDUCE) -> torch.Tensor:
    """Sum of `t` over all ranks, returned as a new local tensor.

    As upstream, there is no trailing barrier by default: do not overwrite `t`
    until every peer is known to have finished (the next collective on the same
    group proves it), or pass `exit_barrier=True`.  `write_back=True` (implies
    the exit barrier) also stores the sum into `t` once all peers have read it.
    """
    hdl, offset = _prepare(t)
    if out is None:
        out = torch.empty_like(t)
    t_ns = config.timeout_ms * 1_000_000
    exit_barrier = exit_barrier or write_back
    if hdl.kind == "cuda":
        C.one_shot_all_reduce(hdl.native, offset, out, t.numel(), config.one_shot_max_blocks,
                              exit_barrier, t_ns, write_back)
    else:
        raise_for_status(C.host_all_reduce(hdl.native, offset, out, t.numel(), 0, t_ns))
        if exit_barrier:
            hdl.barrier(channel=1, timeout_ms=config.timeout_ms)
        if write_back:
            t.copy_(out)
    return out


def _ll_workspace(device: torch.device, group) -> torch.Tensor:
    """Symmetric inbox of the low-latency kernel (about 8 MiB per rank at 8
    ranks), allocated and rendezvoused at first use: that call is collective."""
    import torch.distributed as dist

    key = (device.type, device.index, symm_mem._group_key(group))
    w = _ll_workspaces.get(key)
    if w is None:
        ws = dist.get_world_size(group) if dist.is_initialized() else 1
        w = symm_mem.empty(C.ll_all_reduce_workspace_bytes(_LL_CAPACITY_NUMEL, ws), dtype=torch.uint8,
                           device=device)
        symm_mem.rendezvous(w, group)
        _ll_workspaces[key] = w
    return w


@traced("smr.low_latency_all_reduce")
def low_latency_all_reduce(t: torch.Tensor, out: Optional[torch.Tensor] = None, group=None,
                           config: AllReduceConfig = DEFAULT_ALL_REDUCE) -> torch.Tensor:
    """All-reduce for small bf16 messages (up to 256 KiB) in one NVLink
    crossing: every rank pushes its data, tagged with the call number, into an
    inbox on every rank and sums what lands in its own; no barrier, no peer
    loads.  `t` is ANY contiguous bf16 CUDA tensor (it need not be symmetric);
    `out` defaults to a new tensor and may be `t` itself.  Same arithmetic as
    `one_shot_all_reduce` (ordered bf16 sum), hence the same bits on all ranks.
    No upstream counterpart."""
    if t.dtype != torch.bfloat16 or not t.is_contiguous() or t.numel() % 8:
        raise SymmMemError("need a contiguous bfloat16 tensor whose size is a multiple of 8")
    if t.numel() > _LL_CAPACITY_NUMEL:
        raise SymmMemError(f"low_latency_all_reduce handles at most {_LL_CAPACITY_NUMEL} elements")
    if out is None:
        out = torch.empty_like(t)
    w = _ll_workspace(t.device, group)
    hdl = symm_mem.rendezvous(w, group)
    if not t.is_cuda:
        # CPU ranks: the same protocol (tagged words, two parities) over shared memory
        raise_for_status(C.host_ll_all_reduce(hdl.native, t, out, _LL_CAPACITY_NUMEL,
                                              config.timeout_ms * 1_000_000))
        return out
    C.ll_all_reduce(hdl.native, t, out, _LL_CAPACITY_NUMEL, config.ll_max_blocks, config.timeout_ms * 1_000_000)
    return out


@traced("smr.two_shot_all_reduce_")
def two_shot_all_reduce_(t: torch.Tensor, *, config: AllReduceConfig = DEFAULT_ALL_REDUCE) -> torch.Tensor:
    """In place: rank r reduces slice r from all peers (ordered bf16 sum) and
    stores it into slice r of every peer.  Returns `t`."""
    hdl, offset = _prepare(t)
    t_ns = config.timeout_ms * 1_000_000
    if hdl.kind == "cuda":
        C.two_shot_all_reduce(hdl.native, offset, t.numel(), config.two_shot_max_blocks, t_ns)
    else:
        raise_for_status(C.host_all_reduce(hdl.native, offset, t, t.numel(), 1, t_ns))
    return t


@traced("smr.multimem_all_reduce_")
def multimem_all_reduce_(t: torch.Tensor, *, config: AllReduceConfig = DEFAULT_ALL_REDUCE) -> torch.Tensor:
    """In place through the NVSwitch: multimem.ld_reduce (fp32 accumulate, one
    bf16 rounding) of slice r, multimem.st of the result.  Returns `t`."""
    hdl, offset = _prepare(t)
    t_ns = config.timeout_ms * 1_000_000
    if hdl.kind == "cuda":
        if hdl.world_size == 1:
            return t
        if not hdl.has_multicast:
            raise SymmMemError("this allocation has no multicast mapping (NVLS unavailable)")
        C.multimem_all_reduce(hdl.native, offset, t.numel(), config.multimem_blocks(hdl.world_size), t_ns)
    else:
        raise_for_status(C.host_all_reduce(hdl.native, offset, t, t.numel(), 2, t_ns))
    return t


_UNROLLED_WORLD_SIZES = frozenset({1, 2, 4, 8})


def choose_algo(nbytes: int, world_size: int, has_multicast: bool,
                config: AllReduceConfig = DEFAULT_ALL_REDUCE) -> str:
    """The dispatcher's decision, exposed for tests and benchmarks."""
    if world_size == 1:
        return "one_shot"
    if world_size not in _UNROLLED_WORLD_SIZES:
        # the peer-to-peer kernels are compiled with the world size unrolled; any other world (say 7
        # ranks left after one was lost) goes through the switch, whose kernel takes it at run time
        if not has_multicast:
            raise SymmMemError(f"all-reduce over {world_size} ranks needs a multicast mapping: the peer-to-peer "
                               f"kernels are built for {sorted(_UNROLLED_WORLD_SIZES)} ranks")
        return "multimem"
    if nbytes <= min(config.ll_max_bytes, _LL_CAPACITY_NUMEL * 2):
        return "low_latency"
    if nbytes <= config.one_shot_limit(world_size):
        return "one_shot"
    if nbytes <= config.two_shot_limit(world_size):
        return "two_shot"
    return "multimem" if has_multicast else "two_shot"


def all_reduce(t: torch.Tensor, algo: str = "auto", *,
               config: AllReduceConfig = DEFAULT_ALL_REDUCE) -> torch.Tensor:
    """All-reduce of a symmetric bf16 tensor; the result is returned in `t`
    itself for the in-place algorithms and copied into `t` for one-shot, so the
    caller always reads the sum from the returned tensor (`t`).  The ranks that
    take part are those of the group `t` was rendezvoused on (the default group
    when this call is its rendezvous)."""
    if algo not in _ALGOS:
        raise SymmMemError(f"algo must be one of {_ALGOS}")
    hdl = symm_mem.rendezvous(t)
    if algo == "auto":
        algo = choose_algo(t.numel() * t.element_size(), hdl.world_size, hdl.has_multicast, config)
    if algo == "low_latency":
        # the inbox workspace belongs to the same group as the tensor: a sub-group's small messages
        # must not land in the inboxes of the whole world
        return low_latency_all_reduce(t, out=t, group=hdl.group, config=config)
    if algo == "one_shot":
        one_shot_all_reduce(t, write_back=True, config=config)
        return t
    if algo == "two_shot":
        return two_shot_all_reduce_(t, config=config)
    return multimem_all_reduce_(t, config=config)
