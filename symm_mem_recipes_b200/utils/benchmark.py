"""Timing helpers with the behaviour of symm_mem_recipes/utils.py.

`benchmark_with_event` (upstream :85-134): warm-up, a process-group barrier,
then per-iteration CUDA-event pairs on the launching stream with an optional
L2 flush before each iteration; returns the median in microseconds.
`benchmark_with_profiler` (upstream :10-82): the same loop under
`torch.profiler`, returning the median device time of the kernels whose name
matches a regex, i.e. pure kernel time without launch overhead.

Additions: `max_over_ranks` (every multi-GPU number of this package is the
maximum over ranks of the device-side time) and a sampler of SM clocks and
throttle reasons for the duration of a timed region.
"""
from __future__ import annotations

import re
import statistics
import subprocess
import threading
from typing import Callable, Optional, Sequence

import torch
import torch.distributed as dist

_L2_FLUSH_BYTES = 256 * 1024 * 1024   # larger than the 126 MB L2 of B200
_flush_buf: dict[int, torch.Tensor] = {}


def flush_l2(device=None) -> None:
    """Overwrite a buffer larger than L2 (upstream zeroes 256 MB: utils.py:37-38, 66-67)."""
    dev = torch.device(device or "cuda")
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    buf = _flush_buf.get(idx)
    if buf is None:
        buf = torch.empty(_L2_FLUSH_BYTES // 4, dtype=torch.int32, device=f"cuda:{idx}")
        _flush_buf[idx] = buf
    buf.zero_()


def _barrier() -> None:
    if dist.is_initialized():
        dist.barrier()


def max_over_ranks(value: float, device=None) -> float:
    """Maximum of a per-rank number over the default process group."""
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return float(value)
    if dist.get_backend() == "nccl":
        t = torch.tensor([value], dtype=torch.float64, device=device or "cuda")
    else:
        t = torch.tensor([value], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def benchmark_with_event(target_fn: Callable[[], None], warmup_iters: int = 200,
                         benchmark_iters: int = 25, profile_ranks: Optional[Sequence[int]] = None,
                         flush_l2: bool = False, reduce: str = "median",
                         all_ranks_max: bool = True, trace_handler=None) -> float:
    """Median (or mean/min) microseconds per call of `target_fn`, timed with CUDA
    events on the current stream.  With `all_ranks_max` the per-rank result is
    replaced by the maximum over ranks.

    `profile_ranks`: ranks on which the timed loop also runs under
    `torch.profiler` (CPU and CUDA activities), `trace_handler(prof)` being its
    `on_trace_ready` callback, as upstream does (utils.py:108-131; there the
    default is rank 0 and the handler an optional importable module).  Here the
    default is no profiler: its bookkeeping shows in event-timed microsecond
    numbers."""
    flush = globals()["flush_l2"] if flush_l2 else None
    rank = dist.get_rank() if dist.is_initialized() else 0
    for _ in range(warmup_iters):
        target_fn()
    _barrier()
    torch.cuda.synchronize()
    begins = [torch.cuda.Event(enable_timing=True) for _ in range(benchmark_iters)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(benchmark_iters)]
    if profile_ranks is not None and rank in profile_ranks:
        from torch.profiler import ProfilerActivity, profile
        prof = profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA], on_trace_ready=trace_handler)
    else:
        import contextlib
        prof = contextlib.nullcontext()
    with prof:
        for i in range(benchmark_iters):
            if flush is not None:
                flush()
            begins[i].record()
            target_fn()
            ends[i].record()
        torch.cuda.synchronize()
    times = [b.elapsed_time(e) * 1000.0 for b, e in zip(begins, ends)]
    if reduce == "median":
        us = statistics.median(times)
    elif reduce == "mean":
        us = statistics.fmean(times)
    else:
        us = min(times)
    return max_over_ranks(us) if all_ranks_max else us


def benchmark_with_profiler(target_fn: Callable[[], None], event_key_regex: str,
                            warmup_iters: int = 200, benchmark_iters: int = 25,
                            profile_ranks: Optional[Sequence[int]] = None,
                            flush_l2: bool = False, trace_handler=None) -> float:
    """Median device time (µs) of the kernels whose name matches
    `event_key_regex`; ranks outside `profile_ranks` (default [0]) return 0.
    `trace_handler(prof)` is passed to the profiler as `on_trace_ready`
    (upstream imports an optional `trace_handler` module for this, utils.py:41-44)."""
    flush = globals()["flush_l2"] if flush_l2 else None
    rank = dist.get_rank() if dist.is_initialized() else 0
    if profile_ranks is None:
        profile_ranks = [0]
    for _ in range(warmup_iters):
        target_fn()
    _barrier()
    torch.cuda.synchronize()
    if rank not in profile_ranks:
        for _ in range(benchmark_iters):
            if flush is not None:
                flush()
            target_fn()
        torch.cuda.synchronize()
        return 0.0
    from torch.profiler import ProfilerActivity, profile

    with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA], on_trace_ready=trace_handler) as prof:
        torch.cuda._sleep(int(2e7))   # queue the launches behind a busy GPU (upstream :64)
        for _ in range(benchmark_iters):
            if flush is not None:
                flush()
            target_fn()
        torch.cuda.synchronize()
    pat = re.compile(event_key_regex)
    times = [e.device_time for e in prof.events() if pat.search(e.key or "") and e.device_time > 0]
    if not times:
        raise RuntimeError(f"no profiler event matches {event_key_regex!r}")
    return float(statistics.median(times))


def benchmark_with_graph(target_fn: Callable[[], None], calls_per_graph: int = 20,
                         warmup_iters: int = 5, replays: int = 10, all_ranks_max: bool = True) -> float:
    """Device time per call (µs) with the CPU launch cost taken out: the call
    is captured `calls_per_graph` times into one CUDA graph and the graph is
    replayed; the median replay time is divided by the number of calls.  This
    is how small-message latencies are reported (upstream gets kernel-only
    time from the profiler instead: utils.py:10-82).  Every op of this package
    is capturable because no launch parameter changes between calls."""
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for _ in range(warmup_iters):
            target_fn()
    stream.synchronize()
    _barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        for _ in range(calls_per_graph):
            target_fn()
    torch.cuda.synchronize()
    _barrier()
    graph.replay()
    torch.cuda.synchronize()
    begins = [torch.cuda.Event(enable_timing=True) for _ in range(replays)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(replays)]
    for i in range(replays):
        begins[i].record()
        graph.replay()
        ends[i].record()
    torch.cuda.synchronize()
    us = statistics.median(b.elapsed_time(e) * 1000.0 / calls_per_graph for b, e in zip(begins, ends))
    del graph
    return max_over_ranks(us) if all_ranks_max else us


class ClockSampler:
    """Samples SM clock, power and throttle reasons of one GPU with nvidia-smi
    while a timed region runs (read-only; changes no GPU setting)."""

    _QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int = 0, period_ms: int = 200):
        self.gpu_index = gpu_index
        self.period_ms = period_ms
        self._proc = None
        self._lines: list[str] = []
        self._thread = None

    def __enter__(self):
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self._QUERY}",
                 "--format=csv,noheader,nounits", "-lms", str(self.period_ms)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self._thread = threading.Thread(target=self._pump, daemon=True)
            self._thread.start()
        except OSError:
            self._proc = None
        return self

    def _pump(self):
        for line in self._proc.stdout:
            self._lines.append(line.strip())

    def __exit__(self, *exc):
        if self._proc is not None:
            self._proc.terminate()
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()
        return False

    def samples_under_load(self) -> int:
        """Samples so far that show the GPU busy (power well above idle)."""
        n = 0
        for line in list(self._lines):
            parts = [p.strip() for p in line.split(",")]
            try:
                if len(parts) >= 3 and float(parts[2]) > 300.0:
                    n += 1
            except ValueError:
                continue
        return n

    def summary(self) -> dict:
        sm, idle, smax, reasons = [], [], 0.0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self._lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                clk, power = float(parts[0]), float(parts[2])
                smax = max(smax, float(parts[1]))
            except ValueError:
                continue
            if power <= 300.0:          # idle sample (before / after the kernels): not "under load"
                idle.append(clk)
                continue
            sm.append(clk)
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else (statistics.median(idle) if idle else None),
                "sm_max_mhz": smax or None, "samples_under_load": len(sm), "samples_idle": len(idle),
                "reasons": sorted(reasons)}
