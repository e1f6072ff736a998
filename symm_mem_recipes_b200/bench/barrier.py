"""Barrier smoke test and latency: what `python -m symm_mem_recipes.triton_barrier`
does upstream (symm_mem_recipes/triton_barrier.py:173-200: 32 CTAs that only run
the barrier; success = it terminates), plus the device time per barrier.

    torchrun --nnodes 1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m symm_mem_recipes_b200.bench.barrier
"""
from __future__ import annotations

import argparse
import json
import sys

import torch


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser()
    ap.add_argument("--blocks", default="1,32,148")
    ap.add_argument("--kinds", default="cas",
                    help="comma-separated: cas (blockwise_barrier), epoch, nvls; the counting kinds run the barrier "
                         "twice per launch and are timed on a second allocation")
    return ap


def main(argv=None, standalone: bool = True) -> int:
    args = build_parser().parse_args(argv)
    from symm_mem_recipes_b200.bench._common import finish, init_distributed

    rank, local_rank, world, dev = init_distributed()

    import symm_mem_recipes_b200 as smr
    from symm_mem_recipes_b200.parallel import symm_mem
    from symm_mem_recipes_b200.utils.benchmark import benchmark_with_graph

    t = symm_mem.empty(4096, dtype=torch.int32, device=dev)     # as upstream: 4096 x u32, zero-filled
    hdl = symm_mem.rendezvous(t)
    for blocks in [int(b) for b in args.blocks.split(",")]:
        smr.barrier_test(hdl, num_blocks=blocks)
        hdl.check()
        us = benchmark_with_graph(lambda: smr.barrier_test(hdl, num_blocks=blocks), calls_per_graph=50)
        if rank == 0:
            print(json.dumps({"op": "blockwise_barrier", "world_size": world, "blocks": blocks,
                              "us": round(us, 2), "timing": "graph"}), flush=True)
    us = benchmark_with_graph(lambda: hdl.barrier(0), calls_per_graph=50)
    hdl.check()
    pad_sum = int(hdl.get_signal_pad().abs().sum())     # before the counting kinds: they leave counters behind
    counting = [k for k in args.kinds.split(",") if k in ("epoch", "nvls")]
    if counting:
        t2 = symm_mem.empty(4096, dtype=torch.int32, device=dev)
        hdl2 = symm_mem.rendezvous(t2)
        for kind in counting:
            if kind == "nvls" and not hdl2.has_multicast:
                continue
            for blocks in [int(b) for b in args.blocks.split(",")]:
                smr.barrier_test(hdl2, num_blocks=blocks, kind=kind)
                hdl2.check()
                us_k = benchmark_with_graph(lambda: smr.barrier_test(hdl2, num_blocks=blocks, kind=kind),
                                            calls_per_graph=50)
                if rank == 0:
                    print(json.dumps({"op": f"{kind}_barrier_x2", "world_size": world, "blocks": blocks,
                                      "us": round(us_k, 2), "timing": "graph"}), flush=True)
    if rank == 0:
        print(json.dumps({"op": "channel_barrier", "world_size": world, "us": round(us, 2), "timing": "graph"}))
        print(json.dumps({"op": "barrier_test", "signal_pad_abs_sum": pad_sum, "ok": pad_sum == 0}))
    if standalone:
        finish()
    return 0


if __name__ == "__main__":
    sys.exit(main())
