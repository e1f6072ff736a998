"""Symmetric memory: allocation, rendezvous and the per-allocation handle.

Covers what the upstream recipes borrow from torch's `_SymmetricMemory`
(`empty_strided_p2p`, `rendezvous`, `.rank/.world_size`, `.buffer_ptrs_dev`,
`.signal_pad_ptrs_dev`, `.get_buffer`, `.barrier`; call sites
symm_mem_recipes/triton_all_gather_matmul.py:28-56, 226, 369-375,
symm_mem_recipes/triton_one_shot_all_reduce.py:111-116, 145-151,
symm_mem_recipes/triton_barrier.py:165-198) with this package's own runtime:
CUDA VMM blocks exported as file descriptors, mapped by every rank of the
host and bound to one NVLink multicast object; or POSIX shared memory for CPU
(`gloo`) ranks.

Typical use, one process per GPU::

    dist.init_process_group("nccl")
    t = symm_mem.empty(8192, dtype=torch.bfloat16, device="cuda")
    hdl = symm_mem.rendezvous(t)          # collective, cached
    peer0 = hdl.get_buffer(0, t.shape, t.dtype)
    hdl.barrier()

Beyond that: `hdl.put_signal / wait_signal` (one-to-one signals on a channel),
`check_status()` (turns a kernel's recorded timeout into `SymmMemTimeout`),
`free(t)` (collective), `memory_summary()`, `shutdown()` (orderly teardown
before `destroy_process_group`) and `reset()` (teardown that allows a new
process group to start over).
"""
from __future__ import annotations

import atexit
import os
import uuid
from datetime import timedelta
from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch
import torch.distributed as dist

from .._ext import C
from ..errors import SymmMemError, raise_for_status
from .store import StoreExchange

DEFAULT_TIMEOUT_MS = int(os.environ.get("SMR_TIMEOUT_MS", "10000"))
_RENDEZVOUS_TIMEOUT_MS = int(os.environ.get("SMR_RENDEZVOUS_TIMEOUT_MS", "60000"))


@dataclass
class _GroupState:
    group: object
    exchange: StoreExchange
    channel: object = None          # FdChannel, created at the first CUDA rendezvous
    names: Optional[list] = None    # socket names of all ranks


@dataclass
class _Record:
    alloc: object                   # CudaSymmAllocation | HostSymmAllocation
    kind: str                       # "cuda" | "host"
    base_ptr: int
    nbytes: int
    handle: Optional["SymmetricMemory"] = None
    views: list = field(default_factory=list)
    notes: dict = field(default_factory=dict)   # per-allocation state of the ops (dies with the allocation)


_records: dict[int, _Record] = {}
_groups: dict[int, _GroupState] = {}
_enabled_groups: set[str] = set()
_shutdown_done = False
_generation = 0          # bumped by reset(): caches of symmetric tensors kept elsewhere compare it


def generation() -> int:
    """How many times `reset()` has run in this process.  Code that caches symmetric tensors
    (a model's gather buffers, for instance) keeps the value it saw and drops its cache when
    the number has moved on: those tensors point into released allocations."""
    return _generation


def _group_key(group):
    """Cache key of a process group: its name, which torch never hands out twice in one job (the
    address of a collected group object can be reused by a later one)."""
    if group is None or group is dist.group.WORLD:
        return 0
    return getattr(group, "group_name", None) or id(group)


def _group_state(group) -> _GroupState:
    key = _group_key(group)
    st = _groups.get(key)
    if st is None:
        # a namespace per reset() generation: a new exchange on the same process group must not
        # find the keys its predecessor left in the Store
        st = _GroupState(group=group, exchange=StoreExchange(group, namespace=f"smr/g{_generation}"))
        _groups[key] = st
    return st


def enable_symm_mem_for_group(group_name: Optional[str] = None) -> None:
    """Kept for parity with `torch.distributed._symmetric_memory`
    (symm_mem_recipes/triton_all_gather_matmul.py:366-367).  Groups need no
    registration here: the Store of the group is looked up at rendezvous."""
    _enabled_groups.add(group_name or "world")


def multicast_supported(device: Optional[torch.device] = None) -> bool:
    """Whether the GPU reports NVLink multicast (NVLS) support; False without a GPU."""
    if not torch.cuda.is_available():
        return False
    dev = torch.device(device or "cuda")
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    return bool(C.CudaSymmAllocation.multicast_supported(idx))


def _numel(size: Sequence[int]) -> int:
    n = 1
    for s in size:
        n *= int(s)
    return n


def empty(*size, dtype: torch.dtype = torch.float32, device=None) -> torch.Tensor:
    """A contiguous tensor in a fresh symmetric allocation (not collective).

    The memory is zero-filled, and so is the signal pad behind it.  `device`
    "cpu" gives POSIX shared memory, usable by `gloo` ranks of one host.
    """
    if len(size) == 1 and not isinstance(size[0], int):
        size = tuple(size[0])
    size = tuple(int(s) for s in size)
    dev = torch.device(device if device is not None else ("cuda" if torch.cuda.is_available() else "cpu"))
    nbytes = _numel(size) * torch.empty((), dtype=dtype).element_size()
    if dev.type == "cuda":
        idx = dev.index if dev.index is not None else torch.cuda.current_device()
        alloc = C.CudaSymmAllocation(idx, nbytes)
        t = C.cuda_view(alloc, -1, list(size), dtype, 0)
        kind = "cuda"
    elif dev.type == "cpu":
        alloc = C.HostSymmAllocation(f"/smr_{os.getpid()}_{uuid.uuid4().hex[:12]}", nbytes)
        t = C.host_view(alloc, -1, list(size), dtype, 0)
        kind = "host"
    else:
        raise SymmMemError(f"unsupported device for symmetric memory: {dev}")
    rec = _Record(alloc=alloc, kind=kind, base_ptr=int(alloc.local_ptr), nbytes=nbytes)
    _records[rec.base_ptr] = rec
    return t


def empty_strided_p2p(size, stride, dtype, device, group_name: Optional[str] = None) -> torch.Tensor:
    """Signature of torch's `_SymmetricMemory.empty_strided_p2p`, as the
    upstream drivers call it (symm_mem_recipes/triton_all_gather_matmul.py:369-375).
    Only contiguous strides are supported."""
    size = tuple(int(s) for s in size)
    expect = torch.empty(size, device="meta").stride()
    if tuple(stride) != tuple(expect):
        raise SymmMemError("empty_strided_p2p: only contiguous strides are supported")
    return empty(*size, dtype=dtype, device=device)


def _find_record(t: torch.Tensor) -> tuple[_Record, int]:
    ptr = t.data_ptr()
    base = t.untyped_storage().data_ptr()
    rec = _records.get(base)
    if rec is None:
        for r in _records.values():
            if r.base_ptr <= ptr < r.base_ptr + max(r.nbytes, 1):
                rec = r
                break
    if rec is None:
        raise SymmMemError("tensor was not allocated with symm_mem.empty()")
    return rec, ptr - rec.base_ptr


def is_symm_mem_tensor(t: torch.Tensor) -> bool:
    """Whether `t` (or the storage it views) lives in an allocation made by `empty()`."""
    try:
        _find_record(t)
        return True
    except SymmMemError:
        return False


class SymmetricMemory:
    """Handle of one rendezvoused allocation."""

    def __init__(self, rec: _Record, group):
        self._rec = rec
        self._alloc = rec.alloc
        self.group = group
        self.kind = rec.kind

    # ---- identity ----
    @property
    def rank(self) -> int:
        return self._alloc.rank

    @property
    def world_size(self) -> int:
        return self._alloc.world_size

    @property
    def buffer_size(self) -> int:
        return self._alloc.payload_bytes

    @property
    def signal_pad_size(self) -> int:
        return C.SIGNAL_PAD_BYTES

    @property
    def device(self) -> torch.device:
        return torch.device("cuda", self._alloc.device) if self.kind == "cuda" else torch.device("cpu")

    # ---- raw pointers (device tables of WS pointers, as integers) ----
    @property
    def buffer_ptrs_dev(self) -> int:
        """Device address of the table of WS payload pointers (what upstream's kernels take as `buffer_ptrs_dev`)."""
        self._need_cuda("buffer_ptrs_dev")
        return self._alloc.buffer_ptrs_dev

    @property
    def signal_pad_ptrs_dev(self) -> int:
        """Device address of the table of WS signal-pad pointers (symm_mem_recipes/triton_barrier.py:167-169)."""
        self._need_cuda("signal_pad_ptrs_dev")
        return self._alloc.signal_pad_ptrs_dev

    @property
    def multicast_ptr(self) -> int:
        """Multicast (NVLS) address of the payload, 0 when unavailable."""
        return self._alloc.multicast_ptr if self.kind == "cuda" else 0

    @property
    def has_multicast(self) -> bool:
        return self.multicast_ptr != 0

    def _need_cuda(self, what: str) -> None:
        if self.kind != "cuda":
            raise SymmMemError(f"{what} exists only for CUDA allocations")

    # ---- views ----
    def get_buffer(self, rank: int, sizes, dtype: torch.dtype, storage_offset: int = 0) -> torch.Tensor:
        """Tensor view of `rank`'s payload as mapped in this process.
        `storage_offset` is in elements of `dtype`
        (symm_mem_recipes/triton_all_gather_matmul.py:46-48)."""
        sizes = [int(s) for s in sizes]
        off = int(storage_offset) * torch.empty((), dtype=dtype).element_size()
        if self.kind == "cuda":
            return C.cuda_view(self._alloc, int(rank), sizes, dtype, off)
        return C.host_view(self._alloc, int(rank), sizes, dtype, off)

    def get_multicast_buffer(self, sizes, dtype: torch.dtype, storage_offset: int = 0) -> torch.Tensor:
        """View of the payload through its NVLink multicast mapping: a store lands in every
        rank's copy; only `multimem.*` instructions and plain stores may touch it."""
        self._need_cuda("multicast views")
        off = int(storage_offset) * torch.empty((), dtype=dtype).element_size()
        return C.cuda_view(self._alloc, -1, [int(s) for s in sizes], dtype, off, True)

    def get_signal_pad(self, rank: Optional[int] = None) -> torch.Tensor:
        """int32 view of a rank's signal pad (all zero between operations)."""
        r = self.rank if rank is None else int(rank)
        if self.kind == "cuda":
            return C.cuda_pad_view(self._alloc, r)
        return C.host_pad_view(self._alloc, r)

    # ---- synchronisation ----
    def barrier(self, channel: int = 0, timeout_ms: int = DEFAULT_TIMEOUT_MS) -> None:
        """Cross-rank barrier on a signal-pad channel, ordered on the current
        stream for CUDA (symm_mem_recipes/triton_all_gather_matmul.py:56, 250).
        On CUDA a timeout is reported by the next `check()`."""
        t_ns = int(timeout_ms) * 1_000_000
        if self.kind == "cuda":
            C.channel_barrier(self._alloc, int(channel), t_ns)
        else:
            code, peer = self._alloc.barrier(C.BLOCK_SLOTS + int(channel) * self.world_size, t_ns)
            raise_for_status((code, self.rank, channel, peer, 1, 0))

    def put_signal(self, dst_rank: int, channel: int = 0, timeout_ms: int = DEFAULT_TIMEOUT_MS) -> None:
        """One-to-one signal on a channel: everything this rank wrote before (in
        stream order on CUDA) is visible to `dst_rank` once its `wait_signal`
        returns.  Waits, bounded, while an earlier signal to that rank on that
        channel is still unconsumed.  Signals and `barrier()` share the
        channels: give them different ones."""
        t_ns = int(timeout_ms) * 1_000_000
        if self.kind == "cuda":
            C.put_signal(self._alloc, int(dst_rank), int(channel), t_ns)
        else:
            code = self._alloc.put_signal(int(dst_rank), C.BLOCK_SLOTS + int(channel) * self.world_size, t_ns)
            raise_for_status((code, self.rank, channel, dst_rank, 1, 0))

    def wait_signal(self, src_rank: int, channel: int = 0, timeout_ms: int = DEFAULT_TIMEOUT_MS) -> None:
        """Consumes `src_rank`'s signal on `channel` (see `put_signal`).  On
        CUDA the wait runs on the current stream and a timeout is reported by
        the next `check()`; on CPU it raises SymmMemTimeout itself."""
        t_ns = int(timeout_ms) * 1_000_000
        if self.kind == "cuda":
            C.wait_signal(self._alloc, int(src_rank), int(channel), t_ns)
        else:
            code = self._alloc.wait_signal(int(src_rank), C.BLOCK_SLOTS + int(channel) * self.world_size, t_ns)
            raise_for_status((code, self.rank, channel, src_rank, 1, 0))

    @staticmethod
    def stream_write_value32(flags: torch.Tensor, offset: int, value: int) -> None:
        """`flags[offset] = value`, ordered after everything already queued on
        the current stream, by the driver's stream memory operation
        (cuStreamWriteValue32, a system-scope fence before the write: what
        upstream publishes the progress of its copy-engine all-gather with,
        symm_mem_recipes/triton_all_gather_matmul.py:51-55).  A CPU tensor, or
        a driver without the call, gets a one-element fill instead."""
        flat = flags.view(-1)
        if flat.is_cuda and flat.element_size() == 4 and flat.is_contiguous():
            if C.stream_write_value32(flat, int(offset), int(value) & 0xFFFFFFFF):
                return
        flat[int(offset):int(offset) + 1].fill_(int(value))

    @property
    def buffer_ptrs(self) -> list:
        """Address of every rank's payload as mapped in this process."""
        return [self.get_buffer(r, (1,), torch.uint8).data_ptr() for r in range(self.world_size)]

    @property
    def signal_pad_ptrs(self) -> list:
        """Address of every rank's signal pad as mapped in this process."""
        return [self.get_signal_pad(r).data_ptr() for r in range(self.world_size)]

    def check(self) -> None:
        """Synchronise the device and raise if any kernel reported a failure."""
        if self.kind == "cuda":
            raise_for_status(C.read_status(self._alloc.device))

    @property
    def native(self):
        return self._alloc


def check_status(device=None) -> None:
    """Synchronise `device` and raise `SymmMemTimeout` if a kernel's bounded
    wait ran out since the last check."""
    dev = torch.device(device or "cuda")
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    raise_for_status(C.read_status(idx))


def rendezvous(t: torch.Tensor, group=None) -> SymmetricMemory:
    """Collective over `group`: every rank passes its tensor of the same
    allocation order and size.  Returns the cached handle on later calls."""
    rec, _ = _find_record(t)
    if rec.handle is not None:
        return rec.handle
    if not dist.is_initialized():
        # single process: world of one, nothing to exchange
        if rec.kind == "cuda":
            rec.alloc.begin_rendezvous(0, 1)
            rec.alloc.finish_rendezvous()
        else:
            rec.alloc.rendezvous(0, [rec.alloc.shm_name])
        rec.handle = SymmetricMemory(rec, None)
        return rec.handle

    st = _group_state(group)
    xchg = st.exchange
    rank, ws = xchg.rank, xchg.world_size
    sizes = xchg.all_gather((rec.kind, rec.alloc.block_bytes))
    if any(s != sizes[0] for s in sizes):
        raise SymmMemError(f"rendezvous: allocations differ across ranks: {sizes}")

    if rec.kind == "host":
        names = xchg.all_gather(rec.alloc.shm_name)
        rec.alloc.rendezvous(rank, names)
        xchg.barrier()
    else:
        if st.channel is None:
            st.channel = C.FdChannel(f"smr-{uuid.uuid4().hex}-{rank}")
            st.names = xchg.all_gather(st.channel.name)   # doubles as "every socket is bound"
        alloc = rec.alloc
        alloc.begin_rendezvous(rank, ws)
        alloc.exchange_and_map(st.channel, st.names, _RENDEZVOUS_TIMEOUT_MS)
        xchg.barrier()
        if ws > 1 and os.environ.get("SMR_DISABLE_MULTICAST", "0") != "1":
            _setup_multicast(alloc, st)
        alloc.finish_rendezvous()
        xchg.barrier()
    rec.handle = SymmetricMemory(rec, group)
    return rec.handle


def rendezvous_local(t: torch.Tensor) -> SymmetricMemory:
    """A world of one for `t`'s allocation, whatever process group exists: nothing is exchanged and
    the handle's only rank is this process.  For scratch that a kernel of the library needs in the
    layout of a symmetric workspace while no peer takes part (the rank-local GEMV of a
    column-parallel projection).  Not collective."""
    rec, _ = _find_record(t)
    if rec.handle is not None:
        if rec.handle.world_size != 1:
            raise SymmMemError("this allocation is already rendezvoused with peers")
        return rec.handle
    if rec.kind == "cuda":
        rec.alloc.begin_rendezvous(0, 1)
        rec.alloc.finish_rendezvous()
    else:
        rec.alloc.rendezvous(0, [rec.alloc.shm_name])
    rec.handle = SymmetricMemory(rec, None)
    return rec.handle


def _setup_multicast(alloc, st: _GroupState) -> None:
    """All-or-nothing: if any rank fails a phase, every rank drops multicast
    and the P2P paths remain."""
    xchg = st.exchange
    try:
        ok = bool(alloc.multicast_create_and_add(st.channel, st.names, 20000))
    except Exception:  # noqa: BLE001 - degrade to P2P
        ok = False
    if not all(xchg.all_gather(ok)):
        alloc.multicast_teardown()
        return
    try:
        alloc.multicast_bind_and_map()
        ok = True
    except Exception:  # noqa: BLE001
        ok = False
    if not all(xchg.all_gather(ok)):
        alloc.multicast_teardown()
        xchg.barrier()


def memory_summary() -> dict:
    """Symmetric memory held by this process: one entry per allocation (payload
    bytes, bytes of the mapped block including the signal pad and granularity
    rounding, whether it is rendezvoused and bound to a multicast object) and
    the totals.  A CUDA allocation also occupies (world_size - 1) x block bytes
    of address space for the peers' mappings, but no more physical memory."""
    allocations = []
    for rec in _records.values():
        h = rec.handle
        allocations.append({
            "kind": rec.kind, "payload_bytes": int(rec.nbytes), "block_bytes": int(rec.alloc.block_bytes),
            "rendezvoused": h is not None, "world_size": h.world_size if h is not None else None,
            "multicast": bool(h.has_multicast) if h is not None else False,
        })
    return {"allocations": allocations, "count": len(allocations),
            "payload_bytes": sum(a["payload_bytes"] for a in allocations),
            "block_bytes": sum(a["block_bytes"] for a in allocations)}


def free(t: torch.Tensor) -> None:
    """Release the allocation behind `t`; `t` and every view of it must not be
    used again.  For a rendezvoused allocation this is collective over its
    group: the ranks synchronise their devices and meet (through the Store)
    before anyone unmaps, so that no kernel of a peer still reaches the memory
    and nobody unbinds multicast memory that a peer still uses."""
    rec, _ = _find_record(t)
    if rec.kind == "cuda" and torch.cuda.is_available():
        torch.cuda.synchronize()
    if rec.handle is not None and rec.handle.world_size > 1 and dist.is_initialized():
        _group_state(rec.handle.group).exchange.barrier()
    _records.pop(rec.base_ptr, None)
    _drop_cached_views(rec)
    rec.alloc.release()


def _op_caches():
    """The dictionaries in which the ops keep symmetric workspaces between calls."""
    import importlib
    for mod, names in (("ag_matmul", ("_gather_buffers",)), ("all_reduce", ("_ll_workspaces",)),
                       ("gemv_all_reduce", ("_workspaces",)),
                       ("matmul_reduce_scatter", ("_workspaces", "_ar_outputs"))):
        m = importlib.import_module(f"symm_mem_recipes_b200.ops.{mod}")
        for name in names:
            yield getattr(m, name)


def _drop_cached_views(rec: _Record) -> None:
    """Forget every cached workspace that lives in `rec`: it is about to be unmapped."""
    lo, hi = rec.base_ptr, rec.base_ptr + max(rec.nbytes, 1)
    for cache in _op_caches():
        for key in [k for k, v in cache.items()
                    if any(isinstance(x, torch.Tensor) and lo <= x.data_ptr() < hi
                           for x in (v if isinstance(v, (tuple, list)) else (v,)))]:
            del cache[key]


def shutdown() -> None:
    """Orderly teardown of every allocation: synchronise, meet the other ranks
    (so that nobody unbinds multicast memory a peer still uses), unmap.  Call
    before `dist.destroy_process_group()`; also runs at interpreter exit."""
    global _shutdown_done
    if _shutdown_done:
        return
    _shutdown_done = True
    if torch.cuda.is_available() and any(r.kind == "cuda" for r in _records.values()):
        torch.cuda.synchronize()
    if dist.is_initialized():
        for st in list(_groups.values()):
            try:
                st.exchange.timeout = timedelta(seconds=10)
                st.exchange.barrier()
            except Exception:  # noqa: BLE001 - a peer is gone; continue locally
                pass
    for rec in list(_records.values()):
        try:
            rec.alloc.release()
        except Exception:  # noqa: BLE001
            pass
    _records.clear()
    _groups.clear()


def reset() -> None:
    """`shutdown()`, after which the module accepts new allocations again.  For a
    job that re-forms its process group (for example the survivors after
    `PeerLost`): every symmetric tensor and every cached workspace of the ops
    is gone afterwards and is re-created, collectively, by the new group."""
    global _shutdown_done, _generation
    shutdown()
    _shutdown_done = False
    _generation += 1
    # workspaces the ops keep per (shape, group): they point into released allocations
    for cache in _op_caches():
        cache.clear()


_reset_for_tests = reset


atexit.register(shutdown)
