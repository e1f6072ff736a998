"""Render the JSON lines of the benchmark CLIs as Markdown tables with roofline
fractions.

    python -m symm_mem_recipes_b200.bench.report results.jsonl [more.jsonl ...] \
        [--peaks MEASURED_PEAKS.json] [--out tables.md]

Every benchmark of this package prints one JSON object per measurement (and
appends it to `--out FILE`); upstream prints medians as text on rank 0
(symm_mem_recipes/triton_all_gather_matmul.py:395-418,
triton_one_shot_all_reduce.py:161-162).  This tool needs no GPU: it only reads
those lines.  Non-JSON lines and records of unknown ops are skipped, and when a
measurement occurs more than once the last one wins.

Roofline denominators: `--peaks` names a JSON file with `bf16_tflops`,
`bf16_tflops_sustained` and `hbm_gbs` measured on the same kind of GPU (a
cuBLAS GEMM and a device copy); without it the fractions are left out.  NVLink
figures are per direction per GPU: 900 GB/s nominal, 770 GB/s measured peer copy.
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import Iterable, Optional

NVLINK_NOMINAL_GBS = 900.0
NVLINK_MEASURED_GBS = 770.0

OURS_AR = ("low_latency", "one_shot", "two_shot", "multimem")


def read_records(paths: Iterable[str]) -> list[dict]:
    recs = []
    for path in paths:
        with open(path) as f:
            for line in f:
                line = line.strip()
                if not line.startswith("{"):
                    continue
                try:
                    rec = json.loads(line)
                except json.JSONDecodeError:
                    continue
                if isinstance(rec, dict) and "op" in rec:
                    recs.append(rec)
    return recs


def _size(nbytes: int) -> str:
    for unit, shift in (("GiB", 30), ("MiB", 20), ("KiB", 10)):
        if nbytes >= 1 << shift and nbytes % (1 << shift) == 0:
            return f"{nbytes >> shift} {unit}"
    return f"{nbytes} B"


def _table(header: list[str], rows: list[list[str]]) -> str:
    out = ["| " + " | ".join(header) + " |", "|" + "---|" * len(header)]
    out += ["| " + " | ".join(r) + " |" for r in rows]
    return "\n".join(out)


def _fmt(x: Optional[float], digits: int = 1) -> str:
    return "-" if x is None else f"{x:.{digits}f}"


def all_reduce_table(recs: list[dict]) -> Optional[str]:
    """One row per message size: every implementation's latency, the best of
    this package, its speed-up over NCCL and the upstream Triton kernel, and its
    bus bandwidth as a fraction of nominal NVLink."""
    by_size: dict[tuple[int, int], dict[str, float]] = {}
    for r in recs:
        if r.get("op") != "all_reduce" or "us" not in r:
            continue
        impl = "auto" if r["impl"].startswith("auto:") else r["impl"]    # "auto:<algorithm picked>"
        by_size.setdefault((r["world_size"], r["bytes"]), {})[impl] = float(r["us"])
    if not by_size:
        return None
    impls = ["nccl", "reference_triton", *OURS_AR, "auto"]
    present = [i for i in impls if any(i in v for v in by_size.values())]
    rows = []
    for (ws, nbytes), v in sorted(by_size.items()):
        ours = [v[i] for i in OURS_AR if i in v]
        best = min(ours) if ours else None
        bus = 2.0 * (ws - 1) / ws * nbytes / best / 1e3 if best else None
        row = [str(ws), _size(nbytes)] + [_fmt(v.get(i), 2) for i in present]
        row.append(_fmt(best, 2))
        row.append(_fmt(v["nccl"] / best, 2) + "x" if best and "nccl" in v else "-")
        row.append(_fmt(v["reference_triton"] / best, 2) + "x" if best and "reference_triton" in v else "-")
        row.append(_fmt(bus, 1))
        row.append(_fmt(100.0 * bus / NVLINK_NOMINAL_GBS, 1) + " %" if bus else "-")
        rows.append(row)
    header = ["WS", "bytes"] + [f"{i} µs" for i in present] + \
             ["best of this package µs", "vs NCCL", "vs upstream Triton", "bus GB/s", "of 900 GB/s nominal"]
    return "### all-reduce (bf16)\n\n" + _table(header, rows)


def ag_matmul_table(recs: list[dict], peaks: Optional[dict]) -> Optional[str]:
    """Per shape: the four upstream timings plus the fused kernel, TFLOPS per
    GPU, fraction of the measured cuBLAS peak, speed-up over NCCL + cuBLAS, and
    the time the roofline allows (the slower of the FLOPs at the measured peak
    and the remote bytes at the measured NVLink rate)."""
    groups: dict[tuple, dict[str, dict]] = {}
    for r in recs:
        if r.get("op") != "all_gather_matmul" or "us" not in r:
            continue
        name = r["impl"]
        if name == "smr_fused":
            name = f"smr_fused ({r.get('gather', 'push')})"
        groups.setdefault((r["world_size"], r["M"], r["N"], r["K"]), {})[name] = r
    if not groups:
        return None
    parts = []
    for (ws, M, N, K), impls in sorted(groups.items()):
        flops = 2.0 * M * N * K
        base = impls.get("cublas_plus_nccl", {}).get("us")
        with_upstream = any("upstream_8xh100_us" in r for r in impls.values())
        rows = []
        for name, r in impls.items():
            us = float(r["us"])
            tf = flops / us / 1e6
            row = [name, _fmt(us, 1), _fmt(tf if name != "nccl_all_gather_only" else None, 1)]
            if peaks:
                row.append(_fmt(100.0 * tf / peaks["bf16_tflops"], 1) + " %" if name != "nccl_all_gather_only" else "-")
            row.append(_fmt(base / us, 2) + "x" if base else "-")
            if with_upstream:
                up = r.get("upstream_8xh100_us")
                row.append(f"{up} ({up / us:.2f}x)" if up else "-")
            rows.append(row)
        header = ["impl", "µs", "TFLOPS / GPU"] + (["of measured cuBLAS burst peak"] if peaks else []) + \
                 ["vs NCCL all-gather + cuBLAS"] + \
                 (["same row of the upstream table, 8 x H100 µs (ratio)"] if with_upstream else [])
        text = f"### all_gather_matmul, WS {ws}, M {M}, N {N}, K {K}\n\n" + _table(header, rows)
        if peaks:
            t_math = flops / peaks["bf16_tflops"] / 1e6
            remote = (ws - 1) / ws * M * K * 2.0
            t_wire = remote / NVLINK_MEASURED_GBS / 1e3
            bound = max(t_math, t_wire)
            fused = [float(r["us"]) for n, r in impls.items() if n.startswith("smr_fused")]
            text += (f"\n\nRoofline: {t_math:.0f} µs of math at the measured {peaks['bf16_tflops']:.0f} TFLOPS, "
                     f"{t_wire:.0f} µs for {remote / 2**20:.0f} MiB of remote A at {NVLINK_MEASURED_GBS:.0f} GB/s "
                     f"-> {bound:.0f} µs")
            if fused:
                text += f"; best fused kernel reaches {100.0 * bound / min(fused):.1f} % of it (of measured)."
        parts.append(text)
    return "\n\n".join(parts)


def gemv_table(recs: list[dict], peaks: Optional[dict]) -> Optional[str]:
    groups: dict[tuple, dict[str, float]] = {}
    for r in recs:
        if r.get("op") != "gemv_all_reduce" or "us" not in r:
            continue
        groups.setdefault((r["world_size"], r["K"], r["N"], r["batch"]), {})[r["impl"]] = float(r["us"])
    if not groups:
        return None
    rows = []
    for (ws, K, N, batch), v in sorted(groups.items()):
        fused, lib = v.get("smr_fused"), v.get("cublas_plus_nccl")
        row = [str(ws), f"{K} x {N}", str(batch), _fmt(fused, 2), _fmt(lib, 2), _fmt(v.get("cublas_gemv_only"), 2),
               _fmt(lib / fused, 2) + "x" if fused and lib else "-"]
        if peaks:
            floor = K * N * 2.0 / peaks["hbm_gbs"] / 1e3       # the weight shard must cross HBM once
            row.append(_fmt(floor, 1))
            row.append(_fmt(100.0 * floor / fused, 1) + " %" if fused else "-")
        rows.append(row)
    header = ["WS", "W shard", "batch", "fused µs", "cuBLAS + NCCL µs", "cuBLAS GEMV alone µs", "speed-up"] + \
             (["weight stream at measured HBM rate µs", "fused reaches (of measured)"] if peaks else [])
    return "### GEMV + all-reduce (decode)\n\n" + _table(header, rows)


def layer_tables(recs: list[dict]) -> Optional[str]:
    rs = [r for r in recs if r.get("op") == "matmul_reduce_scatter"]
    pre = [r for r in recs if r.get("op") in ("llama70b_layer_prefill", "llama70b_layer_prefill_tp")]
    dec = [r for r in recs if r.get("op") == "llama70b_layer_decode"]
    parts = []
    if rs:
        last = {(r["world_size"], r["shape"]): r for r in rs}
        rows = [[str(ws), shape, f"{r['M']} x {r['N']} x {r['K_local']}", _fmt(r["smr_fused_us"]),
                 _fmt(r["cublas_plus_nccl_us"]), _fmt(r.get("cublas_mm_only_us")), _fmt(r.get("fused_tflops")),
                 _fmt(r.get("wire_gbs")), f"{r['speedup']:.2f}x"] for (ws, shape), r in sorted(last.items())]
        parts.append("### GEMM + reduce-scatter\n\n" + _table(
            ["WS", "shape", "M x N x K per rank", "fused µs", "cuBLAS + NCCL µs", "cuBLAS alone µs", "fused TFLOPS",
             "outbound GB/s", "speed-up"], rows))
    if pre or dec:
        rows = []
        for r in {(r["op"], r["world_size"], r["batch"], r["seq"], r.get("fused_glue", False),
                   r.get("fused_swiglu", False)): r for r in pre}.values():
            glue = ", no sequence parallelism" if r["op"].endswith("_tp") else ""
            glue += ", single-pass norm / RoPE / SiLU kernels" if r.get("fused_glue") else ""
            glue += ", SwiGLU in the GEMM epilogue" if r.get("fused_swiglu") else ""
            rows.append([str(r["world_size"]), f"prefill {r['batch']} x {r['seq']}{glue}", _fmt(r["smr_fused_us"]),
                         _fmt(r["nccl_cublas_us"]), f"{r['speedup']:.2f}x"])
        for r in {(r["world_size"], r["batch"], r.get("fused_glue", False)): r for r in dec}.values():
            glue = ", single-pass norm / RoPE / SiLU kernels" if r.get("fused_glue") else ""
            rows.append([str(r["world_size"]), f"decode batch {r['batch']}{glue}", _fmt(r["smr_fused_us"]),
                         _fmt(r["nccl_cublas_us"]), f"{r['speedup']:.2f}x"])
        parts.append("### Llama-3-70B TP decoder layer\n\n" + _table(
            ["WS", "step", "this package µs", "NCCL + cuBLAS µs", "speed-up"], rows))
    for r in recs:
        if r.get("op") == "llama70b_layer_prefill_phases":
            total = sum(r["us"].values())
            rows = [[k, _fmt(v), _fmt(100.0 * v / total) + " %"] for k, v in r["us"].items()]
            glue = "single-pass glue kernels" if r.get("fused_glue") else "PyTorch glue"
            glue += " + SwiGLU epilogue" if r.get("fused_swiglu") else ""
            parts.append(f"### prefill phases, WS {r['world_size']}, {glue} (rank 0)\n\n" +
                         _table(["phase", "µs", "share"], rows))
    graphs = {(r["world_size"], r["layers"], r["batch"]): r for r in recs if r.get("op") == "llama70b_decode_graph"}
    if graphs:
        rows = [[str(ws), str(layers), str(batch), str(r["cache_entries"]), _fmt(r["graph_us_per_step"]),
                 _fmt(r["eager_us_per_step"]), f"{r['speedup']:.2f}x"]
                for (ws, layers, batch), r in sorted(graphs.items())]
        parts.append("### decode steps replayed from one CUDA graph\n\n" + _table(
            ["WS", "layers", "batch", "KV cache entries", "graph µs / step", "eager µs / step", "speed-up"], rows))
    return "\n\n".join(parts) if parts else None


def barrier_table(recs: list[dict]) -> Optional[str]:
    rows = []
    for r in recs:
        if r.get("op") == "blockwise_barrier":
            rows.append([str(r["world_size"]), f"blockwise_barrier, {r['blocks']} CTAs", _fmt(r["us"], 2)])
        elif r.get("op") == "channel_barrier":
            rows.append([str(r["world_size"]), "host-launched channel barrier", _fmt(r["us"], 2)])
    if not rows:
        return None
    return "### barriers\n\n" + _table(["WS", "what", "µs"], rows)


def render(recs: list[dict], peaks: Optional[dict] = None) -> str:
    sections = [all_reduce_table(recs), ag_matmul_table(recs, peaks), gemv_table(recs, peaks), layer_tables(recs),
                barrier_table(recs)]
    body = "\n\n".join(s for s in sections if s)
    return body + "\n" if body else "no benchmark records found\n"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("files", nargs="+", help="files of JSON lines written by the benchmark CLIs")
    ap.add_argument("--peaks", default=None, help="JSON file with bf16_tflops, bf16_tflops_sustained, hbm_gbs")
    ap.add_argument("--out", default=None, help="write the Markdown here instead of stdout")
    args = ap.parse_args(argv)
    peaks = None
    if args.peaks:
        with open(args.peaks) as f:
            peaks = json.load(f)
    text = render(read_records(args.files), peaks)
    if args.out:
        with open(args.out, "w") as f:
            f.write(text)
    else:
        sys.stdout.write(text)
    return 0


if __name__ == "__main__":
    sys.exit(main())
