"""Turns an Nsight Compute report into the short Markdown summary kept under
profiles/: one row per metric that the roofline reading needs, one column per
captured launch, plus the figures derived from them (DRAM bytes against the
algorithmic bytes, achieved rate against a peaks file).  Reads the report with
`ncu -i <report> --page raw --csv`; no GPU is needed for that.

    python -m symm_mem_recipes_b200.bench.ncu_summary prof.ncu-rep \
        --title "tcgen05 GEMM, M 4096" --command "ncu --set full ... python -m ..." \
        --flops 2.405e11 --bytes 1.55e8 --peaks MEASURED_PEAKS.json > profiles/gemm.md

The upstream recipes extract one number, the median kernel time, from
torch.profiler events (symm_mem_recipes/utils.py:74-77); this is the same step
for the counters Nsight Compute collects.
"""
from __future__ import annotations

import argparse
import csv
import io
import json
import subprocess
import sys
from typing import Optional

# metric, label, unit conversion to the unit shown
METRICS = [
    ("gpu__time_duration.sum", "duration"),
    ("sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active", "tensor pipe active (% of active cycles)"),
    ("dram__bytes_read.sum", "DRAM read"),
    ("dram__bytes_write.sum", "DRAM written"),
    ("gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed", "DRAM throughput (% of peak)"),
    ("dram__cycles_active.avg.pct_of_peak_sustained_elapsed", "DRAM cycles active (% of elapsed)"),
    ("lts__t_sector_hit_rate.pct", "L2 sector hit rate"),
    ("l1tex__m_xbar2l1tex_read_bytes.sum", "L2 -> SM bytes"),
    ("sm__warps_active.avg.pct_of_peak_sustained_active", "warps active (% of peak)"),
    ("smsp__average_warps_issue_stalled_long_scoreboard_per_issue_active.ratio", "stall: long scoreboard (per issue)"),
    ("smsp__average_warps_issue_stalled_barrier_per_issue_active.ratio", "stall: barrier (per issue)"),
    ("smsp__average_warps_issue_stalled_membar_per_issue_active.ratio", "stall: membar (per issue)"),
    ("launch__registers_per_thread", "registers per thread"),
    ("launch__shared_mem_per_block_dynamic", "dynamic shared memory per CTA"),
    ("launch__grid_size", "grid"),
    ("launch__block_size", "block"),
]
_TO_BYTES = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9, "Tbyte": 1e12}
_TO_US = {"ns": 1e-3, "us": 1.0, "ms": 1e3, "s": 1e6, "usecond": 1.0, "nsecond": 1e-3, "msecond": 1e3, "second": 1e6}


def read_report(path: str, ncu: str = "ncu") -> str:
    out = subprocess.run([ncu, "-i", path, "--page", "raw", "--csv"], capture_output=True, text=True, check=False)
    if out.returncode != 0:
        raise RuntimeError(f"ncu could not read {path}: {out.stderr.strip() or out.stdout.strip()[:200]}")
    return out.stdout


def parse_raw_csv(text: str) -> list[dict]:
    """One dict per captured launch: metric name -> (value string, unit), plus "Kernel Name" etc."""
    lines = text.splitlines()
    start = next((i for i, ln in enumerate(lines) if ln.startswith('"ID"')), None)
    if start is None:
        raise ValueError("no raw-page CSV header in the ncu output")
    rows = list(csv.reader(io.StringIO("\n".join(lines[start:]))))
    header, units = rows[0], rows[1]
    launches = []
    for r in rows[2:]:
        if len(r) != len(header):
            continue
        launches.append({h: (v, u) for h, u, v in zip(header, units, r)})
    return launches


def _num(cell) -> Optional[float]:
    try:
        return float(cell[0].replace(",", ""))
    except (ValueError, AttributeError, IndexError):
        return None


def _bytes(cell) -> Optional[float]:
    v = _num(cell)
    return None if v is None else v * _TO_BYTES.get(cell[1].split("/")[0], 1.0)


def _us(cell) -> Optional[float]:
    v = _num(cell)
    return None if v is None else v * _TO_US.get(cell[1], 1.0)


def _show(metric: str, cell) -> str:
    if cell is None or cell[0] == "":
        return "-"
    if metric.startswith("dram__bytes") or metric.endswith("read_bytes.sum") or "shared_mem" in metric:
        b = _bytes(cell)
        return f"{b / 1e6:.1f} MB" if b >= 1e6 else f"{b / 1e3:.1f} KB"
    if metric == "gpu__time_duration.sum":
        return f"{_us(cell):.1f} µs"
    v = _num(cell)
    if v is None:
        return cell[0]
    if cell[1] == "%":
        return f"{v:.1f} %"
    return f"{v:.2f}" if v != int(v) else str(int(v))


def render(launches: list[dict], title: str = "", command: str = "", flops: float = 0.0, nbytes: float = 0.0,
           peaks: Optional[dict] = None) -> str:
    if not launches:
        return "no captured launch in the report\n"
    out = []
    if title:
        out.append(f"# {title}\n")
    if command:
        out.append("Command (run directly after the same command had exited 0 without `ncu`):\n\n```\n" + command +
                   "\n```\n")
    names = [launch.get("Kernel Name", ("?", ""))[0] for launch in launches]
    out.append("| metric (ncu, one launch each) | " + " | ".join(f"launch {i}" for i in range(len(launches))) + " |")
    out.append("|---|" + "---|" * len(launches))
    out.append("| kernel | " + " | ".join(f"`{n[:90]}`" for n in names) + " |")
    for metric, label in METRICS:
        cells = [launch.get(metric) for launch in launches]
        if all(c is None or c[0] == "" for c in cells):
            continue
        out.append(f"| {label} (`{metric.split('.')[0]}`) | " + " | ".join(_show(metric, c) for c in cells) + " |")
    out.append("")
    for i, launch in enumerate(launches):
        us = _us(launch["gpu__time_duration.sum"]) if "gpu__time_duration.sum" in launch else None
        rd, wr = _bytes(launch.get("dram__bytes_read.sum")), _bytes(launch.get("dram__bytes_write.sum"))
        notes = []
        if us and rd is not None and wr is not None:
            traffic = rd + wr
            notes.append(f"DRAM traffic {traffic / 1e6:.1f} MB at {traffic / us / 1e3:.0f} GB/s")
            if nbytes:
                notes.append(f"{traffic / nbytes:.2f}x the algorithmic {nbytes / 1e6:.1f} MB")
            if peaks and peaks.get("hbm_gbs"):
                notes.append(f"{traffic / us / 1e3 / peaks['hbm_gbs']:.2f} of the measured copy rate "
                             f"({peaks['hbm_gbs']:.0f} GB/s)")
        if us and flops:
            tf = flops / us / 1e6
            notes.append(f"{tf:.0f} TFLOPS under ncu (clocks as ncu found them)")
            if peaks and peaks.get("bf16_tflops"):
                notes.append(f"{tf / peaks['bf16_tflops']:.2f} of the measured burst bf16 rate "
                             f"({peaks['bf16_tflops']:.0f} TFLOPS)")
        if notes:
            out.append(f"Launch {i}: " + "; ".join(notes) + ".")
    out.append("\nTimes taken under `ncu` are for the counters' context only; the timed figures come from CUDA events "
               "in runs without a profiler.")
    return "\n".join(out) + "\n"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("report", help=".ncu-rep file, or a file with the output of `ncu --page raw --csv`")
    ap.add_argument("--title", default="")
    ap.add_argument("--command", default="", help="the full command that made the report (printed in the summary)")
    ap.add_argument("--flops", type=float, default=0.0, help="algorithmic FLOPs of one launch")
    ap.add_argument("--bytes", type=float, default=0.0, help="algorithmic bytes of one launch")
    ap.add_argument("--peaks", default=None, help="JSON with hbm_gbs / bf16_tflops (the measured peaks)")
    ap.add_argument("--ncu", default="ncu")
    args = ap.parse_args(argv)
    text = read_report(args.report, args.ncu) if args.report.endswith(".ncu-rep") else open(args.report).read()
    peaks = json.load(open(args.peaks)) if args.peaks else None
    sys.stdout.write(render(parse_raw_csv(text), args.title, args.command, args.flops, args.bytes, peaks))
    return 0


if __name__ == "__main__":
    sys.exit(main())
