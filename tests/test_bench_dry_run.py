"""bench.py's control flow on a machine without a GPU: the CUDA runtime calls
are replaced by do-nothing stand-ins, the fused op by a plain product, and the
program must still run from argument parsing to its one JSON line with every
key of the contract.  This catches what a typo in the harness would otherwise
only show on the GPU box (a misspelt name, a wrong keyword, a missing key); it
says nothing about speed."""
import contextlib
import importlib.util
import json
import pathlib
import sys
import types

import pytest
import torch

ROOT = pathlib.Path(__file__).resolve().parent.parent
REQUIRED = {"metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
            "vs_baseline", "dtype", "data", "config", "e2e", "gpu_launches", "clocks"}


class _Event:
    def __init__(self, enable_timing=False):
        pass

    def record(self, stream=None):
        pass

    def elapsed_time(self, other):
        return 0.5                      # ms

    def synchronize(self):
        pass


class _Stream:
    def __init__(self, device=None):
        pass

    def wait_event(self, ev):
        pass

    def wait_stream(self, s):
        pass

    def synchronize(self):
        pass


class _FakeCuda(types.SimpleNamespace):
    pass


class _FakeTorch:
    """`torch` as bench.py sees it: every device is the CPU, the stream and event API does nothing."""

    def __init__(self):
        main = _Stream()
        self.cuda = _FakeCuda(set_device=lambda d: None, synchronize=lambda d=None: None, Event=_Event,
                              Stream=_Stream, current_stream=lambda d=None: main,
                              stream=lambda s: contextlib.nullcontext())

    def __getattr__(self, name):
        return getattr(torch, name)

    @staticmethod
    def device(*args):
        return torch.device("cpu")

    @staticmethod
    def randn(*shape, device=None, **kw):
        return torch.randn(*shape, **kw)

    @staticmethod
    def empty(*shape, device=None, **kw):
        return torch.empty(*shape, **kw)


class _Clocks:
    def __init__(self, *a, **k):
        pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False

    def summary(self):
        return {"sm_mhz": 1500.0, "sm_max_mhz": 1965.0, "reasons": []}


def _load_bench(monkeypatch, shape):
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    bench.torch = _FakeTorch()
    bench.M_TOTAL, bench.N_PER_RANK, bench.K_DIM = shape
    import symm_mem_recipes_b200 as smr
    from symm_mem_recipes_b200.parallel import symm_mem
    from symm_mem_recipes_b200.utils import benchmark

    def product(a_shard, b, a_out=None, c_out=None, *a, **k):
        import torch.distributed as dist
        full = a_shard
        if dist.is_initialized() and dist.get_world_size() > 1:
            full = a_out if a_out is not None else torch.empty(a_shard.shape[0] * dist.get_world_size(),
                                                               a_shard.shape[1], dtype=a_shard.dtype)
            dist.all_gather_into_tensor(full, a_shard.contiguous())
        c = (full.float() @ b.float().t()).to(torch.bfloat16)
        if c_out is None:
            return c
        c_out.copy_(c)
        return c_out

    monkeypatch.setattr(smr, "all_gather_matmul", product)
    monkeypatch.setattr(symm_mem, "check_status", lambda device=None: None)
    monkeypatch.setattr(benchmark, "ClockSampler", _Clocks)
    monkeypatch.setattr(benchmark, "flush_l2", lambda device=None: None)
    monkeypatch.setattr(torch.Tensor, "pin_memory", lambda self, *a, **k: self)
    return bench


@pytest.mark.parametrize("extra", [[], ["--no-extras"]])
def test_bench_runs_to_its_json_line(monkeypatch, capsys, extra):
    bench = _load_bench(monkeypatch, (256, 64, 128))
    monkeypatch.delenv("WORLD_SIZE", raising=False)
    monkeypatch.delenv("RANK", raising=False)
    monkeypatch.setattr(sys, "argv", ["bench.py", "--steps", "2", "--warmup", "1"] + extra)
    assert bench.main() == 0
    from symm_mem_recipes_b200.parallel import symm_mem
    symm_mem.reset()                                         # bench.py shut the module down; later tests allocate again
    lines = [ln for ln in capsys.readouterr().out.splitlines() if ln.startswith("{")]
    assert len(lines) == 1                                   # exactly one JSON line
    rec = json.loads(lines[0])
    assert REQUIRED <= set(rec)
    assert rec["n_gpus"] == 1 and rec["steps"] == 2 and rec["warmup"] == 3      # never fewer than three warm-ups
    assert rec["higher_is_better"] is True and rec["scaling"] == "weak" and rec["dtype"] == "bf16"
    assert rec["gpu_launches"] == 2
    assert set(rec["e2e"]) >= {"value", "unit", "h2d_bytes_per_step", "d2h_bytes_per_step"}
    assert rec["e2e"]["h2d_bytes_per_step"] == 256 * 128 * 2 and rec["e2e"]["d2h_bytes_per_step"] == 4
    assert {"sm_mhz", "sm_max_mhz", "reasons"} <= set(rec["clocks"])
    assert rec["config"]["M"] == 256 and "l2" in rec["config"]
    # value = flops / time, aggregated over the GPUs; 0.5 ms per step by construction
    flops = 2.0 * 256 * 64 * 128
    assert rec["ms_per_step"] == 0.5 and abs(rec["value"] - round(flops / 0.5e-3 / 1e12, 2)) < 1e-9
    assert {"ms_per_step", "h2d_bytes_per_step", "how"} <= set(rec["e2e_serial"]) and "how" in rec["e2e"]
    assert rec["same_box_baseline"]["ms_per_step"] == 0.5


def _two_rank_worker(rank, world_size, out_path):
    import os

    import torch.distributed as dist

    mp = pytest.MonkeyPatch()
    try:
        bench = _load_bench(mp, (256, 64, 128))
        os.environ.update(WORLD_SIZE=str(world_size), RANK=str(rank), LOCAL_RANK=str(rank))
        mp.setattr(dist, "init_process_group", lambda *a, **k: None)          # the harness has formed the gloo group
        mp.setattr(dist, "destroy_process_group", lambda *a, **k: None)
        mp.setattr(sys, "argv", ["bench.py", "--gpus", str(world_size), "--steps", "2", "--warmup", "1",
                                 "--no-extras"])
        import io
        buf = io.StringIO()
        with contextlib.redirect_stdout(buf):
            assert bench.main() == 0
        if rank == 0:
            pathlib.Path(out_path).write_text(buf.getvalue())
        else:
            assert "{" not in buf.getvalue()                 # only rank 0 prints
    finally:
        mp.undo()


def test_bench_two_ranks_over_gloo(tmp_path):
    """The N > 1 branch (rendezvous of the symmetric buffers, collective verdict, NCCL + cuBLAS
    composition as the same-box baseline, rank-uniform repeat loop) with two gloo ranks."""
    from symm_mem_recipes_b200.utils.testing import spawn_ranks

    out = tmp_path / "rank0.txt"
    spawn_ranks(_two_rank_worker, 2, "gloo", (str(out),), timeout_s=120.0)
    lines = [ln for ln in out.read_text().splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    assert REQUIRED <= set(rec) and rec["n_gpus"] == 2 and rec["config"]["parallelism"] == "tp2"
    assert rec["config"]["a_shard_rows"] == 128
    assert "NCCL" in rec["same_box_baseline"]["what"] and "e2e_serial" in rec
