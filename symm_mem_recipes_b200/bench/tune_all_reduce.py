"""Derive the all-reduce dispatcher's thresholds from a measured sweep.

    torchrun ... -m symm_mem_recipes_b200.bench.all_reduce --out sweep.jsonl       # measure (GPUs)
    python -m symm_mem_recipes_b200.bench.tune_all_reduce sweep.jsonl --out ar_tuning.json
    SMR_AR_TUNING_FILE=ar_tuning.json python serve.py                             # use

`all_reduce(algo="auto")` picks the low-latency push kernel up to
`ll_max_bytes`, then the one-shot kernel up to `one_shot_max_bytes`, then the
two-shot kernel up to `two_shot_max_bytes`, then multimem (or two-shot without
a multicast mapping).  This tool reads the JSON lines of the sweep and sets
each threshold to the largest message size up to which that kernel is still
the fastest of this package's kernels, per world size.  The sweep times the
one-shot kernel writing into a new tensor; `all_reduce` works in place, which
costs that kernel a second barrier and a write-back pass: `--write-back-us`
(default 5.5, measured on 2 and 4 B200s) is added to its times before they
are compared.  Upstream has one kernel and no dispatcher
(symm_mem_recipes/triton_one_shot_all_reduce.py:96-125).  No GPU needed here.
"""
from __future__ import annotations

import argparse
import json
import sys

from .report import read_records

LARGE = ("multimem", "two_shot")


def thresholds(recs: list[dict], write_back_us: float = 5.5) -> dict:
    """{"by_world_size": {"<ws>": {"ll_max_bytes": ..., "one_shot_max_bytes": ..., "two_shot_max_bytes": ...}}}"""
    by_ws: dict[int, dict[int, dict[str, float]]] = {}
    for r in recs:
        if r.get("op") == "all_reduce" and "us" in r and not r["impl"].startswith(("auto", "nccl", "reference")):
            by_ws.setdefault(int(r["world_size"]), {}).setdefault(int(r["bytes"]), {})[r["impl"]] = float(r["us"])
    out = {}
    for ws, sizes in sorted(by_ws.items()):
        ll_max = one_shot_max = two_shot_max = 0
        phase = "low_latency"          # the size axis is cut into four consecutive ranges
        for nbytes in sorted(sizes):
            v = sizes[nbytes]
            large = min((v[k] for k in LARGE if k in v), default=float("inf"))
            ll, one = v.get("low_latency", float("inf")), v.get("one_shot", float("inf")) + write_back_us
            if phase == "low_latency":
                if ll <= min(one, large):
                    ll_max = nbytes
                    continue
                phase = "one_shot"
            if phase == "one_shot":
                if one < large:
                    one_shot_max = nbytes
                    continue
                phase = "two_shot"
            if phase == "two_shot":
                if "two_shot" in v and v["two_shot"] <= v.get("multimem", float("inf")):
                    two_shot_max = nbytes
                    continue
                phase = "large"
        out[str(ws)] = {"ll_max_bytes": ll_max, "one_shot_max_bytes": one_shot_max}
        # only where the sweep compared the two: without such rows the built-in choice by world size stays
        if any("two_shot" in v and "multimem" in v for v in sizes.values()):
            out[str(ws)]["two_shot_max_bytes"] = two_shot_max
    return {"by_world_size": out}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("files", nargs="+", help="JSON lines written by bench.all_reduce --out")
    ap.add_argument("--out", default=None, help="write the tuning JSON here instead of stdout")
    ap.add_argument("--write-back-us", type=float, default=5.5,
                    help="added to the one-shot kernel's times: the cost of its in-place form")
    args = ap.parse_args(argv)
    text = json.dumps(thresholds(read_records(args.files), args.write_back_us), indent=1) + "\n"
    if args.out:
        with open(args.out, "w") as f:
            f.write(text)
    else:
        sys.stdout.write(text)
    return 0


if __name__ == "__main__":
    sys.exit(main())
