"""The multi-GPU benchmark drivers on two gloo ranks without a GPU: kernels by
host stand-ins, timers by a single call, the 70B configuration by the tiny
one.  What is checked is the drivers' own code (argument handling, shapes,
reference comparisons, the records they emit), so that a GPU run is not spent
on a typo."""
import contextlib
import io
import json
import pathlib

import pytest
import torch

from symm_mem_recipes_b200.utils.testing import spawn_ranks


def _prepare(rank, world_size):
    import torch.distributed as dist

    import test_fused_ops_flow_cpu as flow
    from symm_mem_recipes_b200.bench import _common
    from symm_mem_recipes_b200.models import llama_tp_layer
    from symm_mem_recipes_b200.utils import benchmark

    flow._install_all_stand_ins()
    dev = torch.device("cpu")
    _common.init_distributed = lambda default_port=0: (rank, rank, world_size, dev)
    _common.finish = lambda: None

    def once(fn, *a, **k):
        fn()
        return 100.0                                   # "microseconds"

    benchmark.benchmark_with_event = once
    benchmark.benchmark_with_graph = once
    torch.cuda.synchronize = lambda device=None: None
    tiny = llama_tp_layer.LlamaTPConfig.tiny(world_size)
    llama_tp_layer.LlamaTPConfig.llama3_70b = staticmethod(lambda: tiny)
    # CUDA events of the per-phase timing: one made-up figure per phase
    llama_tp_layer.LlamaTPDecoderLayer.phase_times_us = (
        lambda self, x, batch, seq, iters=5: {"norm": 1.0, "qkv": 2.0, "rest": 3.0})

    class EagerDecodeGraph:                            # replays by running the static step eagerly
        def __init__(self, layers, batch, max_seq, fused=True, warmup=2, caches=None):
            self.layers, self.fused = list(layers), fused
            cfg = self.layers[0].cfg
            self.pos = torch.zeros(1, dtype=torch.int32)
            self.caches = caches if caches is not None else [
                (torch.zeros(batch, max_seq, lyr.hkv, cfg.head_dim, dtype=torch.bfloat16),
                 torch.zeros(batch, max_seq, lyr.hkv, cfg.head_dim, dtype=torch.bfloat16)) for lyr in self.layers]

        def step(self, x, pos):
            from symm_mem_recipes_b200.models.llama_tp_layer import decode_static_through
            self.pos.fill_(pos)
            return decode_static_through(self.layers, self.caches, x, self.pos, fused=self.fused)

    llama_tp_layer.DecodeGraph = EagerDecodeGraph

    class _Event:
        def __init__(self, enable_timing=False):
            pass

        def record(self):
            pass

        def elapsed_time(self, other):
            return 3.2

    torch.cuda.Event = _Event
    return dist


def _run(main, argv, rank, out_path):
    buf = io.StringIO()
    with contextlib.redirect_stdout(buf):
        assert main(argv, standalone=False) == 0
    if rank == 0:
        pathlib.Path(out_path).write_text(buf.getvalue())


def _layer_worker(rank, world_size, out_path):
    _prepare(rank, world_size)
    from symm_mem_recipes_b200.bench import llama_layer

    _run(llama_layer.main, ["--batch", "2", "--seq", "128", "--warmup", "1", "--iters", "1", "--fused-glue", "all",
                            "--breakdown", "--tp", "--decode-graph", "2", "--decode-cache", "48"], rank, out_path)


def _layer_worker_with_a_timeout(rank, world_size, out_path):
    """The first reduce-scatter section ends in a device-side timeout (on a GPU the peers of a rank whose
    wait ran out run into their own bounded waits, so every rank reports one)."""
    _prepare(rank, world_size)
    import symm_mem_recipes_b200 as smr
    from symm_mem_recipes_b200.bench import llama_layer
    from symm_mem_recipes_b200.errors import SymmMemTimeout

    real = smr.matmul_reduce_scatter

    calls = {"n": 0}

    def flaky(a, b, out=None, **kw):
        calls["n"] += 1
        if calls["n"] == 1:
            raise SymmMemTimeout(3, rank, 0, 0, 7, 0)
        return real(a, b, out, **kw)

    smr.matmul_reduce_scatter = flaky
    _run(llama_layer.main, ["--batch", "2", "--seq", "128", "--warmup", "1", "--iters", "1", "--fused-glue", "both"],
         rank, out_path)


def _agmm_worker(rank, world_size, out_path):
    _prepare(rank, world_size)
    from symm_mem_recipes_b200.bench import all_gather_matmul

    _run(all_gather_matmul.main, ["--M", "512", "--N", "256", "--K", "128", "--warmup", "1", "--iters", "1",
                                  "--with-plain-a-out", "--per-rank", "--leads", "1,2"],
         rank, out_path)


def _gemv_worker(rank, world_size, out_path):
    _prepare(rank, world_size)
    from symm_mem_recipes_b200.bench import gemv_all_reduce

    _run(gemv_all_reduce.main, ["--K", "256", "--N", "512", "--batches", "1,4", "--extra-algos", "tc_tagged,simt"],
         rank, out_path)


def _barrier_worker(rank, world_size, out_path):
    _prepare(rank, world_size)
    import symm_mem_recipes_b200 as smr
    from symm_mem_recipes_b200.bench import barrier

    smr.barrier_test = lambda hdl, num_blocks=32, **k: hdl.barrier()      # the kernel form exists on the GPU only
    _run(barrier.main, ["--blocks", "1,32", "--kinds", "cas,epoch,nvls"], rank, out_path)


def _records(path):
    return [json.loads(ln) for ln in pathlib.Path(path).read_text().splitlines() if ln.startswith("{")]


def test_layer_driver(tmp_path):
    out = tmp_path / "layer.txt"
    spawn_ranks(_layer_worker, 2, "gloo", (str(out),), timeout_s=240.0)
    recs = _records(out)
    ops = [r["op"] for r in recs]
    assert ops.count("matmul_reduce_scatter") == 2
    assert ops.count("llama70b_layer_prefill") == 3 and ops.count("llama70b_layer_prefill_phases") == 3
    assert ops.count("llama70b_layer_prefill_tp") == 1
    decodes = [r for r in recs if r["op"] == "llama70b_layer_decode"]
    assert sorted((r["batch"], r["fused_glue"]) for r in decodes) == [(1, False), (1, True), (4, False), (4, True),
                                                                      (16, False), (16, True)]
    assert ops.count("llama70b_decode_graph") == 3
    assert all(r["matches_library"] for r in recs if "matches_library" in r)
    assert not [r for r in recs if r["op"] == "section_failed"]
    rs = [r for r in recs if r["op"] == "matmul_reduce_scatter"][0]
    assert rs["phases"] == {"entered_us": 1.1, "gemm_done_first_us": 8.0, "gemm_done_last_us": 8.5,
                            "reduced_last_us": 11.5}
    # and the report renders what the driver wrote
    from symm_mem_recipes_b200.bench import report
    text = report.render(recs, None)
    assert "decode steps replayed from one CUDA graph" in text and "GEMM + reduce-scatter" in text


def test_layer_driver_goes_on_after_a_timeout_in_one_section(tmp_path):
    out = tmp_path / "layer_failure.txt"
    spawn_ranks(_layer_worker_with_a_timeout, 2, "gloo", (str(out),), timeout_s=240.0)
    recs = _records(out)
    failed = [r for r in recs if r["op"] == "section_failed"]
    assert [r["section"] for r in failed] == ["matmul_reduce_scatter o_proj"]
    assert all(r["symmetric_memory_reset"] for r in failed)          # every rank dropped its symmetric memory
    assert "device-side timeout" in failed[0]["error"]
    ops = [r["op"] for r in recs]
    # everything after the failing sections still ran, on fresh allocations
    assert ops.count("matmul_reduce_scatter") == 1
    assert ops.count("llama70b_layer_prefill") == 2 and ops.count("llama70b_layer_decode") == 6
    assert all(r["matches_library"] for r in recs if "matches_library" in r)


def test_all_gather_matmul_driver(tmp_path):
    out = tmp_path / "agmm.txt"
    spawn_ranks(_agmm_worker, 2, "gloo", (str(out),), timeout_s=120.0)
    recs = _records(out)
    impls = [(r["impl"], r.get("gather")) for r in recs]
    assert impls == [("cublas_mm_only", None), ("smr_mm_only", None), ("cublas_plus_nccl", None),
                     ("nccl_all_gather_only", None), ("smr_fused", "push"), ("smr_fused", "push"),
                     ("smr_fused", "push"), ("smr_fused", "push_copy")]


def test_gemv_driver(tmp_path):
    out = tmp_path / "gemv.txt"
    spawn_ranks(_gemv_worker, 2, "gloo", (str(out),), timeout_s=120.0)
    recs = _records(out)
    assert len(recs) >= 4 and all(r["op"] == "gemv_all_reduce" for r in recs)


def _all_reduce_worker(rank, world_size, out_path):
    _prepare(rank, world_size)
    from symm_mem_recipes_b200.bench import all_reduce

    _run(all_reduce.main, ["--min-bytes", "4096", "--max-bytes", "65536", "--warmup", "1", "--iters", "1"],
         rank, out_path)


def _one_shot_sweep_worker(rank, world_size, out_path):
    _prepare(rank, world_size)
    from symm_mem_recipes_b200.bench import all_reduce

    _run(all_reduce.main, ["--one-shot-sweep", "--max-bytes", "1048576"], rank, out_path)


def test_one_shot_sweep_driver(tmp_path):
    out = tmp_path / "sweep.txt"
    spawn_ranks(_one_shot_sweep_worker, 2, "gloo", (str(out),), timeout_s=180.0)
    recs = [r for r in _records(out) if r["op"] == "all_reduce_one_shot_sweep"]
    ours = [r for r in recs if r["impl"] == "one_shot"]
    assert {r["bytes"] for r in ours} == {4096, 65536, 1 << 20} and all(r["same_bits_as_default"] for r in ours)
    assert "max_blocks" in ours[0] and any(r["impl"] == "nccl" for r in recs)


def test_all_reduce_driver(tmp_path):
    """Host backend: the ordered-sum kernels run as their host builds, the multimem kernel is skipped
    (no multicast mapping), NCCL is gloo."""
    out = tmp_path / "ar.txt"
    spawn_ranks(_all_reduce_worker, 2, "gloo", (str(out),), timeout_s=120.0)
    recs = _records(out)
    checks = [r for r in recs if r["op"] == "all_reduce_check"]
    assert checks[0]["output_equals_world_size"] is True
    assert {r["impl"] for r in checks[1:]} == {"one_shot", "two_shot", "low_latency"}
    assert all(r["ok"] for r in checks[1:])
    timed = [r for r in recs if r["op"] == "all_reduce"]
    assert {r["bytes"] for r in timed} == {4096, 8192, 16384, 32768, 65536}
    assert {"nccl", "low_latency", "one_shot", "two_shot"} <= {r["impl"] for r in timed}
    # the tuning tool reads what the driver writes
    from symm_mem_recipes_b200.bench import tune_all_reduce
    table = tune_all_reduce.thresholds(timed)
    assert set(table["by_world_size"]) == {"2"}


class _FakeTorchOneGpu:
    """`torch` as the single-GPU driver sees it: the only device is the CPU."""

    def __init__(self):
        import types
        self.cuda = types.SimpleNamespace(set_device=lambda d: None, synchronize=lambda d=None: None)

    def __getattr__(self, name):
        return getattr(torch, name)

    @staticmethod
    def device(*args):
        return torch.device("cpu")


@pytest.mark.parametrize("argv", [
    ["--M", "256", "--N", "512", "--K", "128"],
    ["--M", "256", "--N", "512", "--K", "128", "--variant", "fp8"],
    ["--M", "256", "--N", "512", "--K", "128", "--variant", "swiglu"],
    ["--op", "gemv", "--batch", "4", "--K", "256", "--N", "512", "--gemv-algo", "tc_tagged"],
    ["--op", "gemv", "--batch", "4", "--eager"],
    ["--op", "glue", "--M", "64"],
    ["--op", "all_reduce", "--bytes", "65536"],
])
def test_single_gpu_driver(monkeypatch, capsys, argv):
    import importlib
    import sys

    import test_fused_ops_flow_cpu as flow
    from symm_mem_recipes_b200._ext import C as real
    from symm_mem_recipes_b200.bench import matmul as driver
    from symm_mem_recipes_b200.parallel import symm_mem
    from symm_mem_recipes_b200.utils import benchmark

    ag_mod = importlib.import_module("symm_mem_recipes_b200.ops.ag_matmul")
    gemv_mod = importlib.import_module("symm_mem_recipes_b200.ops.gemv_all_reduce")
    rs_mod = importlib.import_module("symm_mem_recipes_b200.ops.matmul_reduce_scatter")
    glue_mod = importlib.import_module("symm_mem_recipes_b200.ops.layer_glue")
    saved = [(m, k, getattr(m, k)) for m in (ag_mod, gemv_mod, rs_mod, glue_mod)
             for k in ("C", "_num_sms", "_check", "_check_2d", "_tail_buffer") if hasattr(m, k)]
    try:
        flow._install_host_kernels()
        flow._install_row_parallel_and_glue_stand_ins()

        class GemvFake:
            def __getattr__(self, name):
                return getattr(real, name)

            @staticmethod
            def gemv_all_reduce(x, w, out, workspace, ws_offset, timeout_ns, tensor_core=False, num_sms=148,
                                tagged=False, weights_nk=False):
                out.copy_((x.float() @ (w.float().t() if weights_nk else w.float())).to(out.dtype))

        gemv_mod.C = GemvFake()
        gemv_mod._num_sms = lambda device: 148
        monkeypatch.setattr(driver, "torch", _FakeTorchOneGpu())
        monkeypatch.setattr(symm_mem, "check_status", lambda device=None: None)
        monkeypatch.setattr(benchmark, "benchmark_with_event", lambda fn, *a, **k: (fn(), 50.0)[1])
        monkeypatch.setattr(benchmark, "benchmark_with_graph", lambda fn, *a, **k: (fn(), 50.0)[1])

        class Clocks:
            def __init__(self, *a, **k):
                pass

            def __enter__(self):
                return self

            def __exit__(self, *exc):
                return False

            def summary(self):
                return {"sm_mhz": 1500.0}

        monkeypatch.setattr(benchmark, "ClockSampler", Clocks)
        monkeypatch.setattr(sys, "argv", ["matmul"] + argv)
        real_randn = torch.randn
        monkeypatch.setattr(torch, "randn", lambda *shape, device=None, **kw: real_randn(*shape, **kw))
        real_empty, real_ones = torch.empty, torch.ones
        monkeypatch.setattr(torch, "empty", lambda *shape, device=None, **kw: real_empty(*shape, **kw))
        monkeypatch.setattr(torch, "ones", lambda *shape, device=None, **kw: real_ones(*shape, **kw))
        assert driver.main() == 0
    finally:
        for m, k, v in saved:
            setattr(m, k, v)
        symm_mem.reset()
    rec = json.loads([ln for ln in capsys.readouterr().out.splitlines() if ln.startswith("{")][-1])
    assert rec["op"] == (argv[1] if argv[0] == "--op" else "matmul") and "clocks" in rec


def test_barrier_driver(tmp_path):
    out = tmp_path / "barrier.txt"
    spawn_ranks(_barrier_worker, 2, "gloo", (str(out),), timeout_s=120.0)
    recs = _records(out)
    assert [r["op"] for r in recs] == ["blockwise_barrier", "blockwise_barrier", "epoch_barrier_x2", "epoch_barrier_x2",
                                       "channel_barrier", "barrier_test"]      # no multicast on the CPU: nvls skipped
    assert recs[-1]["ok"] is True
