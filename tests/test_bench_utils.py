"""Host-side pieces of the benchmark harness and the op configuration."""
import importlib
import json
import subprocess
import sys

import torch

from symm_mem_recipes_b200.utils.benchmark import ClockSampler


def test_clock_sampler_separates_idle_from_load():
    c = ClockSampler(0)
    c._lines = [
        "1965, 1965, 140.2, Not Active, Not Active, Not Active, Not Active",
        "1410, 1965, 985.0, Not Active, Not Active, Not Active, Active",
        "1395, 1965, 1001.3, Not Active, Not Active, Not Active, Active",
        "garbage line",
    ]
    s = c.summary()
    assert s["samples_under_load"] == 2 and s["samples_idle"] == 1
    assert s["sm_mhz"] == 1402.5 and s["sm_max_mhz"] == 1965.0
    assert s["reasons"] == ["sw_power_cap"]
    assert c.samples_under_load() == 2


def test_clock_sampler_flags_thermal_slowdown():
    c = ClockSampler(0)
    c._lines = ["1200, 1965, 900.0, Active, Active, Not Active, Not Active"]
    assert set(c.summary()["reasons"]) == {"hw_slowdown", "hw_thermal_slowdown"}


def test_all_reduce_config_reads_environment(monkeypatch):
    monkeypatch.setenv("SMR_AR_LL_MAX_BYTES", "4096")
    monkeypatch.setenv("SMR_AR_MULTIMEM_MAX_BLOCKS", "12")
    from symm_mem_recipes_b200.ops import config

    importlib.reload(config)
    try:
        cfg = config.AllReduceConfig()
        assert cfg.ll_max_bytes == 4096 and cfg.multimem_max_blocks == 12
    finally:
        monkeypatch.delenv("SMR_AR_LL_MAX_BYTES")
        monkeypatch.delenv("SMR_AR_MULTIMEM_MAX_BLOCKS")
        importlib.reload(config)


def test_reference_arm_prints_one_json_line():
    import os

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference"],
                         capture_output=True, text=True, timeout=300, cwd=root)
    assert out.returncode == 0
    rec = json.loads(out.stdout.strip().splitlines()[-1])
    assert rec["impl"] == "reference" and "unavailable" in rec


def test_ptxas_report_lists_the_kernels():
    from symm_mem_recipes_b200 import _build

    report = _build.ptxas_report()
    if report:          # present whenever the module was built in this tree
        assert "registers" in report


def test_nvtx_tracing_is_free_when_off_and_balanced_when_on(monkeypatch):
    from symm_mem_recipes_b200.utils import trace

    def op(t, k=1):
        if k < 0:
            raise ValueError("boom")
        return t + k

    assert trace.traced("smr.op", enabled=False)(op) is op        # off: the very same function
    events = []
    monkeypatch.setattr(trace, "_push", lambda msg: events.append(("push", msg)))
    monkeypatch.setattr(trace, "_pop", lambda: events.append(("pop",)))
    wrapped = trace.traced("smr.op", enabled=True)(op)
    assert wrapped.__name__ == "op"
    assert int(wrapped(torch.zeros(2, 3), k=2).sum()) == 12
    assert events == [("push", "smr.op (2, 3)"), ("pop",)]
    events.clear()
    try:
        wrapped(torch.zeros(1), k=-1)
    except ValueError:
        pass
    assert events == [("push", "smr.op (1,)"), ("pop",)]          # popped on the error path too
    events.clear()
    with trace.nvtx_range("phase", enabled=True):
        pass
    with trace.nvtx_range("quiet", enabled=False):
        pass
    assert events == [("push", "phase"), ("pop",)]


def test_guarded_empty_detects_stores_outside():
    from symm_mem_recipes_b200.utils.testing import guarded_empty

    t, intact = guarded_empty((5, 24), torch.bfloat16, "cpu", guard_bytes=256)
    assert t.shape == (5, 24) and t.is_contiguous() and t.data_ptr() % 16 == 0
    t.zero_()
    assert intact()
    flat = t.view(-1)
    # one element past the end / before the start, through the underlying storage
    past = torch.as_strided(flat, (1,), (1,), storage_offset=flat.storage_offset() + flat.numel())
    past.fill_(1.0)
    assert not intact()
    t2, intact2 = guarded_empty((8,), torch.float32, "cpu", guard_bytes=256)
    before = torch.as_strided(t2, (1,), (1,), storage_offset=t2.storage_offset() - 1)
    before.fill_(3.0)
    assert not intact2()


def _one_rank_hangs(rank, world_size):
    import time

    if rank == 1:
        time.sleep(1000)


def test_spawn_ranks_gives_up_on_a_hung_rank_and_lets_it_tear_down():
    import time

    import pytest

    from symm_mem_recipes_b200.utils.testing import spawn_ranks

    t0 = time.monotonic()
    with pytest.raises(RuntimeError, match="did not finish") as e:
        spawn_ranks(_one_rank_hangs, 2, "gloo", timeout_s=25.0)     # long enough for the ranks to come up
    # the hung rank was asked to stop and left (through its teardown, naming where it had been, when it
    # was up far enough to have installed the handler); the parent did not wait for the full join
    assert "did not finish" in str(e.value)
    assert time.monotonic() - t0 < 25.0 + 60.0


def test_build_targets_sm_100a_only_and_covers_every_source():
    from symm_mem_recipes_b200 import _build

    flags = " ".join(_build.NVCC_FLAGS)
    assert "arch=compute_100a,code=sm_100a" in flags and "-lineinfo" in flags
    assert flags.count("-gencode") == 1                      # one architecture, no fallback targets
    cu, cpp = _build.sources()
    names = {p.name for p in cu}
    for must in ("all_reduce.cu", "ag_matmul_2cta_sm100.cu", "gemv_allreduce_tc.cu",
                 "matmul_rs_sm100.cu", "layer_glue.cu"):
        assert must in names, must
    ninja = _build.write_ninja().read_text()
    for src in cu + cpp:
        assert str(src) in ninja
    assert str(_build.so_path()) in ninja


def test_in_tree_extension_is_current():
    """The built extension travels with the tree to the GPU machines: it must not be older than
    any of its sources (a kernel edited without a rebuild would be tested here but not run there)."""
    import shutil

    import pytest

    from symm_mem_recipes_b200 import _build

    if shutil.which("ninja") is None or not _build.so_path().exists():
        pytest.skip("no ninja or no built extension in this tree")
    ninja_file = _build.write_ninja()
    dry = subprocess.run(["ninja", "-C", str(ninja_file.parent), "-n"], capture_output=True, text=True, timeout=120)
    assert dry.returncode == 0 and "no work to do" in dry.stdout, (
        "the extension is stale: run python -m symm_mem_recipes_b200._build\n" + dry.stdout[-600:])
