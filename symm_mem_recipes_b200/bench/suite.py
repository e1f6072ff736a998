"""Runs every multi-GPU benchmark of the package in ONE set of processes
(start-up of a torchrun job costs more than most of the benchmarks).

    torchrun --nnodes 1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m symm_mem_recipes_b200.bench.suite --out-dir results --tag ws8

`--jobs` runs an explicit list instead: driver names with their own arguments,
separated by ';', for example
    --jobs "all_reduce --one-shot-sweep --max-bytes 8388608; gemv_all_reduce --extra-algos tc_tagged"
A job that raises is reported and the next one starts from fresh symmetric memory.
"""
from __future__ import annotations

import argparse
import os
import sys


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out-dir", default=".")
    ap.add_argument("--tag", default="")
    ap.add_argument("--only", default="barrier,all_reduce,all_gather_matmul,gemv,layer")
    ap.add_argument("--with-reference-triton", action="store_true")
    ap.add_argument("--ar-max-bytes", type=int, default=256 * 1024 * 1024)
    ap.add_argument("--layer-detail", action="store_true",
                    help="also time the opt-in kernel variants: the layer with the single-pass glue kernels and the "
                         "SwiGLU epilogue, its phases, the prefill without sequence parallelism, the tagged GEMV "
                         "exchange, decode from one CUDA graph")
    ap.add_argument("--jobs", default="",
                    help="';'-separated list of '<driver> <its arguments>' (drivers: barrier, all_reduce, "
                         "all_gather_matmul, gemv_all_reduce, llama_layer) run in this order instead of --only")
    args = ap.parse_args()
    from symm_mem_recipes_b200.bench import (all_gather_matmul, all_reduce, barrier, gemv_all_reduce,
                                             llama_layer)
    from symm_mem_recipes_b200.bench._common import attempt, finish, init_distributed

    rank, _, world, dev = init_distributed()
    tag = args.tag or f"ws{world}"
    only = set(args.only.split(","))
    if args.jobs:
        import json
        import shlex
        drivers = {"barrier": barrier, "all_reduce": all_reduce, "all_gather_matmul": all_gather_matmul,
                   "gemv_all_reduce": gemv_all_reduce, "llama_layer": llama_layer}
        for job in [j.strip() for j in args.jobs.split(";") if j.strip()]:
            name, *argv = shlex.split(job)
            if name not in drivers:
                raise SystemExit(f"unknown driver {name!r}; known: {sorted(drivers)}")
            attempt(job, lambda name=name, argv=argv: drivers[name].main(argv, standalone=False), dev,
                    lambda rec: print(json.dumps(rec), flush=True) if rank == 0 else None)
        finish()
        return 0

    def out(name):
        return os.path.join(args.out_dir, f"{name}_{tag}.jsonl")

    if "barrier" in only:
        barrier.main([], standalone=False)
    if "all_reduce" in only:
        argv = ["--max-bytes", str(args.ar_max_bytes), "--out", out("all_reduce")]
        if args.with_reference_triton:
            argv.append("--with-reference-triton")
        all_reduce.main(argv, standalone=False)
    if "all_gather_matmul" in only:
        all_gather_matmul.main(["--M", "16384", "--N", "3584", "--K", "8192", "--out", out("agmm")],
                               standalone=False)
    if "upstream_table" in only:         # not in the default list: nine shapes, a few minutes
        all_gather_matmul.main(["--upstream-table", "--out", out("agmm_table")], standalone=False)
    if "gemv" in only:
        gemv_all_reduce.main(["--out", out("gemv")] + (["--extra-algos", "tc_tagged"] if args.layer_detail else []),
                             standalone=False)
    if "layer" in only:
        llama_layer.main(["--out", out("layer")] + (["--fused-glue", "all", "--breakdown", "--tp",
                                                     "--decode-graph", "2"]
                                                    if args.layer_detail
                                                    else []), standalone=False)
    finish()
    return 0


if __name__ == "__main__":
    sys.exit(main())
