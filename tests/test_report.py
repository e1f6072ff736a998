"""The Markdown renderer of the benchmark JSON lines (no GPU involved)."""
import json

from symm_mem_recipes_b200.bench import report

LINES = [
    'some log line that is not JSON',
    '{"op": "all_reduce", "impl": "nccl", "world_size": 8, "bytes": 4096, "timing": "graph", "us": 28.81}',
    '{"op": "all_reduce", "impl": "low_latency", "world_size": 8, "bytes": 4096, "timing": "graph", "us": 5.4}',
    '{"op": "all_reduce", "impl": "reference_triton", "world_size": 8, "bytes": 4096, "timing": "graph", "us": 7.96}',
    '{"op": "all_reduce", "impl": "auto:low_latency", "world_size": 8, "bytes": 4096, "timing": "graph", "us": 5.5}',
    '{"op": "all_reduce", "impl": "nccl", "world_size": 8, "bytes": 67108864, "timing": "event", "us": 279.04}',
    '{"op": "all_reduce", "impl": "multimem", "world_size": 8, "bytes": 67108864, "timing": "event", "us": 166.38}',
    '{"op": "all_gather_matmul", "impl": "cublas_plus_nccl", "world_size": 8, "M": 16384,'
    ' "N": 3584, "K": 8192, "us": 1341.5}',
    '{"op": "all_gather_matmul", "impl": "smr_fused", "world_size": 8, "M": 16384, "N": 3584,'
    ' "K": 8192, "us": 772.1, "gather": "push"}',
    '{"op": "gemv_all_reduce", "impl": "smr_fused", "world_size": 8, "batch": 1, "K": 3584, "N": 8192, "us": 22.6}',
    '{"op": "gemv_all_reduce", "impl": "cublas_plus_nccl", "world_size": 8, "batch": 1, "K": 3584,'
    ' "N": 8192, "us": 39.52}',
    '{"op": "llama70b_layer_decode", "world_size": 8, "batch": 1, "smr_fused_us": 197.2,'
    ' "nccl_cublas_us": 237.6, "speedup": 1.205}',
    '{"op": "llama70b_decode_graph", "world_size": 8, "batch": 4, "layers": 2, "cache_entries": 4096,'
    ' "first_position": 2048, "steps": 32, "graph_us_per_step": 410.0, "eager_us_per_step": 615.0, "speedup": 1.5}',
    '{"truncated": ',
]
PEAKS = {"bf16_tflops": 1647.3, "bf16_tflops_sustained": 1411.0, "hbm_gbs": 6541.5}


def test_report_tables(tmp_path):
    f = tmp_path / "r.jsonl"
    f.write_text("\n".join(LINES) + "\n")
    recs = report.read_records([str(f)])
    assert len(recs) == 12                       # the log line and the truncated object are skipped
    text = report.render(recs, PEAKS)
    # all-reduce: best of this package and both speed-ups
    row = [ln for ln in text.splitlines() if ln.startswith("| 8 | 4 KiB")][0]
    assert "5.40" in row and "5.34x" in row and "1.47x" in row
    # bus bandwidth of the 64 MiB row: 2 * 7/8 * 64 MiB / 166.38 µs = 705.9 GB/s = 78.4 % of 900
    row = [ln for ln in text.splitlines() if ln.startswith("| 8 | 64 MiB")][0]
    assert "705.9" in row and "78.4 %" in row
    # fused all_gather_matmul against the library composition, and its roofline line
    assert "1.74x" in text
    assert "584 µs of math" in text and "224 MiB of remote A" in text
    # GEMV: the 56 MiB weight shard at the measured HBM rate is 9.0 µs
    row = [ln for ln in text.splitlines() if ln.startswith("| 8 | 3584 x 8192 | 1 |")][0]
    assert "1.75x" in row and "9.0" in row
    assert "decode batch 1" in text and "1.21x" in text
    row = [ln for ln in text.splitlines() if ln.startswith("| 8 | 2 | 4 | 4096")][0]
    assert "410.0" in row and "1.50x" in row


def test_report_cli_without_peaks(tmp_path, capsys):
    f = tmp_path / "r.jsonl"
    f.write_text("\n".join(LINES) + "\n")
    out = tmp_path / "t.md"
    assert report.main([str(f), "--out", str(out)]) == 0
    text = out.read_text()
    assert "of measured" not in text and "### all-reduce" in text
    empty = tmp_path / "e.jsonl"
    empty.write_text(json.dumps({"no": "op"}) + "\n")
    assert report.main([str(empty)]) == 0
    assert "no benchmark records" in capsys.readouterr().out


def test_all_reduce_thresholds_from_a_sweep(tmp_path, monkeypatch):
    from symm_mem_recipes_b200.bench import tune_all_reduce
    from symm_mem_recipes_b200.ops.config import AllReduceConfig

    def rec(impl, nbytes, us, ws=8):
        return json.dumps({"op": "all_reduce", "impl": impl, "world_size": ws, "bytes": nbytes, "us": us})

    lines = [
        # 4 KiB, 8 KiB: low_latency wins; 16 KiB: one_shot wins; 32 KiB on: multimem wins
        rec("nccl", 4096, 1.0), rec("low_latency", 4096, 5), rec("one_shot", 4096, 12), rec("multimem", 4096, 10),
        rec("low_latency", 8192, 6), rec("one_shot", 8192, 12), rec("multimem", 8192, 10),
        rec("low_latency", 16384, 14), rec("one_shot", 16384, 4), rec("two_shot", 16384, 13),
        rec("multimem", 16384, 10),                                    # one-shot: 4 + 5.5 for its write-back < 10
        rec("one_shot", 32768, 9), rec("two_shot", 32768, 10.5), rec("multimem", 32768, 11),   # 9 + 5.5 loses
        rec("two_shot", 49152, 13), rec("multimem", 49152, 12),
        rec("low_latency", 65536, 1), rec("two_shot", 65536, 1), rec("multimem", 65536, 12),   # past the breaks: ranges must not reopen
        rec("low_latency", 4096, 5, ws=2), rec("two_shot", 4096, 9, ws=2),
    ]
    f = tmp_path / "sweep.jsonl"
    f.write_text("\n".join(lines) + "\n")
    out = tmp_path / "tuning.json"
    assert tune_all_reduce.main([str(f), "--out", str(out)]) == 0
    table = json.loads(out.read_text())["by_world_size"]
    assert table["8"] == {"ll_max_bytes": 8192, "one_shot_max_bytes": 16384, "two_shot_max_bytes": 32768}
    assert table["2"] == {"ll_max_bytes": 4096, "one_shot_max_bytes": 0}    # two-shot never met multimem: no entry
    cfg = AllReduceConfig.from_tuning(str(out), world_size=8)
    assert (cfg.ll_max_bytes, cfg.one_shot_max_bytes) == (8192, 16384)
    assert AllReduceConfig.from_tuning(str(out)).ll_max_bytes == 8192           # largest world size in the file
    from symm_mem_recipes_b200.ops.all_reduce import choose_algo
    assert [choose_algo(n, 8, True, cfg) for n in (4096, 16384, 32768, 49152)] == [
        "low_latency", "one_shot", "two_shot", "multimem"]
    assert choose_algo(49152, 8, False, cfg) == "two_shot"


def test_roofline_expectations():
    from symm_mem_recipes_b200.bench.expect import DEFAULT_PEAKS, expect

    e = expect("all_gather_matmul", 8, DEFAULT_PEAKS, M=16384, N=3584, K=8192)
    assert e["bound_by"] == "tensor" and e["target_us"] == 584.0 and e["nvlink_in_us"] == 305.0
    e = expect("matmul_reduce_scatter", 8, DEFAULT_PEAKS, M=32768, N=8192, K=1024)
    assert e["bound_by"] == "nvlink_out" and abs(e["target_us"] - 610.1) < 0.2       # the o-projection is wire-bound
    e = expect("matmul_reduce_scatter", 8, DEFAULT_PEAKS, M=32768, N=8192, K=3584)
    assert e["bound_by"] == "tensor"
    e = expect("gemv_all_reduce", 8, DEFAULT_PEAKS, K=3584, N=8192, batch=1)
    assert e["bound_by"] == "hbm" and e["target_us"] == 9.0
    nvls = expect("all_reduce", 8, DEFAULT_PEAKS, nbytes=64 << 20)
    p2p = expect("all_reduce", 8, DEFAULT_PEAKS, nbytes=64 << 20, nvls=False)
    assert nvls["target_us"] < p2p["target_us"] and nvls["bound_by"] == "nvlink"


def test_suite_hands_each_benchmark_arguments_its_parser_accepts(monkeypatch, tmp_path):
    """The suite runner builds argument lists for the other drivers; each list must parse with the
    driver's own parser (a misspelt flag would otherwise end an 8-GPU run at that benchmark)."""
    import sys

    import torch

    from symm_mem_recipes_b200.bench import (_common, all_gather_matmul, all_reduce, barrier, gemv_all_reduce,
                                             llama_layer, suite)

    seen = {}
    for mod in (all_gather_matmul, all_reduce, barrier, gemv_all_reduce, llama_layer):
        def fake_main(argv=None, standalone=True, _mod=mod):
            ns = _mod.build_parser().parse_args(argv)          # argparse exits on an unknown flag
            seen.setdefault(_mod.__name__.rsplit(".", 1)[1], []).append(ns)
            return 0
        monkeypatch.setattr(mod, "main", fake_main)
    monkeypatch.setattr(_common, "init_distributed", lambda: (0, 0, 8, torch.device("cpu")))
    monkeypatch.setattr(_common, "finish", lambda: None)
    monkeypatch.setattr(sys, "argv", ["suite", "--out-dir", str(tmp_path), "--layer-detail", "--with-reference-triton",
                                      "--only", "barrier,all_reduce,all_gather_matmul,upstream_table,gemv,layer"])
    assert suite.main() == 0
    assert set(seen) == {"all_gather_matmul", "all_reduce", "barrier", "gemv_all_reduce", "llama_layer"}
    assert len(seen["all_gather_matmul"]) == 2 and seen["all_gather_matmul"][1].upstream_table
    layer = seen["llama_layer"][0]
    assert layer.fused_glue == "all" and layer.breakdown and layer.tp and layer.decode_graph == 2
    assert seen["gemv_all_reduce"][0].extra_algos == "tc_tagged"
    assert seen["all_reduce"][0].with_reference_triton and seen["all_reduce"][0].out.endswith("all_reduce_ws8.jsonl")


def test_suite_runs_an_explicit_job_list(monkeypatch, tmp_path, capsys):
    """`--jobs`: every job's arguments go through its driver's own parser; a job that raises is
    reported and the next one still runs."""
    import sys

    import torch

    from symm_mem_recipes_b200.bench import (_common, all_gather_matmul, all_reduce, barrier, gemv_all_reduce,
                                             llama_layer, suite)

    seen = []
    for mod in (all_gather_matmul, all_reduce, barrier, gemv_all_reduce, llama_layer):
        def fake_main(argv=None, standalone=True, _mod=mod):
            ns = _mod.build_parser().parse_args(argv)
            seen.append((_mod.__name__.rsplit(".", 1)[1], ns))
            if _mod is gemv_all_reduce:
                raise RuntimeError("boom")
            return 0
        monkeypatch.setattr(mod, "main", fake_main)
    monkeypatch.setattr(_common, "init_distributed", lambda: (0, 0, 8, torch.device("cpu")))
    monkeypatch.setattr(_common, "finish", lambda: None)
    jobs = ("all_gather_matmul --M 16384 --N 3584 --K 8192 --warmup 10 --iters 25 --trace --per-rank "
            "--pacings 1:12:0,1:4:1,1:12:1,2:12:0 --out x.jsonl; "
            "gemv_all_reduce --extra-algos tc_tagged; "
            "all_reduce --one-shot-sweep --with-reference-triton --max-bytes 8388608; "
            "all_reduce --multimem-sweep --max-bytes 268435456; "
            "llama_layer --skip-layer")
    monkeypatch.setattr(sys, "argv", ["suite", "--jobs", jobs])
    assert suite.main() == 0
    assert [n for n, _ in seen] == ["all_gather_matmul", "gemv_all_reduce", "all_reduce", "all_reduce", "llama_layer"]
    assert seen[0][1].trace and seen[0][1].pacings.count(",") == 3 and seen[2][1].one_shot_sweep
    assert '"section_failed"' in capsys.readouterr().out          # the job that raised


def test_ncu_summary_from_raw_csv():
    """The raw-page CSV of Nsight Compute (header row, unit row, one row per launch) into the
    Markdown summary kept under profiles/, with the derived roofline figures."""
    from symm_mem_recipes_b200.bench import ncu_summary

    header = ["ID", "Kernel Name", "gpu__time_duration.sum", "dram__bytes_read.sum", "dram__bytes_write.sum",
              "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active", "launch__registers_per_thread",
              "launch__shared_mem_per_block_dynamic", "launch__grid_size"]
    units = ["", "", "us", "Mbyte", "Mbyte", "%", "register/thread", "Kbyte/block", ""]
    row = ["0", "void smr::kernel<256, 6>(Params)", "182.912", "249.496064", "22.527232", "92.063681", "151",
           "197.8", "148"]
    text = "==PROF== some banner\n" + "\n".join(",".join(f'"{c}"' for c in r) for r in (header, units, row)) + "\n"
    launches = ncu_summary.parse_raw_csv(text)
    assert len(launches) == 1 and launches[0]["launch__grid_size"] == ("148", "")
    md = ncu_summary.render(launches, title="GEMM", command="ncu ... python -m x", flops=2.405e11, nbytes=1.55e8,
                            peaks={"hbm_gbs": 6541.5, "bf16_tflops": 1647.3})
    assert "# GEMM" in md and "182.9 µs" in md and "92.1 %" in md and "249.5 MB" in md and "197.8 KB" in md
    # 272.0 MB in 182.9 µs = 1487 GB/s = 0.23 of the copy rate; 1.75x the algorithmic bytes; 1315 TFLOPS = 0.80
    assert "272.0 MB at 1487 GB/s" in md and "1.75x" in md and "0.23 of the measured copy rate" in md
    assert "1315 TFLOPS" in md and "0.80 of the measured burst" in md
    assert ncu_summary.render([], "x") == "no captured launch in the report\n"


def test_layer_roofline_expectations():
    from symm_mem_recipes_b200.bench.expect import DEFAULT_PEAKS, expect_layer

    pre = expect_layer(8, DEFAULT_PEAKS, batch=16, seq=2048)
    assert pre["phases"]["qkv"]["bound_by"] == "nvlink_in" and pre["phases"]["o_proj"]["bound_by"] == "nvlink_out"
    assert pre["phases"]["gate_up"]["bound_by"] == "tensor" and pre["phases"]["down_proj"]["bound_by"] == "tensor"
    assert abs(pre["target_us"] - sum(p["target_us"] for p in pre["phases"].values())) < 0.2
    assert 4900 < pre["target_us"] < 5100                      # about 5.0 ms for the 70B layer at TP8
    dec = expect_layer(8, DEFAULT_PEAKS, batch=1, decode=True)
    # every weight of the rank once: (1280 + 7168 + 1024 + 3584) x 8192 x 2 B = 214 MB at 6541 GB/s
    assert abs(dec["target_us"] - 214.0e6 / 6541.5e3) < 0.3 and set(dec["phases"]) == {"qkv", "gate_up", "o_proj",
                                                                                         "down_proj"}
