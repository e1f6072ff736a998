"""All-reduce sweep: latency (µs) and bus bandwidth per message size for the
one-shot, two-shot and multimem kernels, against NCCL and (optionally) the
upstream Triton kernel.

    torchrun --nnodes 1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m symm_mem_recipes_b200.bench.all_reduce --min-bytes 4096 --max-bytes 268435456

Mirrors the upstream driver (symm_mem_recipes/triton_one_shot_all_reduce.py:128-164),
which times one 16 KiB message; here every power of two in the range is timed.
Device-side CUDA events, maximum over ranks, one JSON line per (size, impl).
busBW = 2 (WS-1)/WS * bytes / time.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser()
    ap.add_argument("--min-bytes", type=int, default=4096)
    ap.add_argument("--max-bytes", type=int, default=256 * 1024 * 1024)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--algos", default="low_latency,one_shot,two_shot,multimem,auto")
    ap.add_argument("--one-shot-limit", type=int, default=8 * 1024 * 1024,
                    help="largest message timed with the one-shot kernels")
    ap.add_argument("--with-reference-triton", action="store_true")
    ap.add_argument("--timing", default="graph", choices=["graph", "event"],
                    help="graph: CUDA-graph replay (device time per call) up to --graph-limit bytes")
    ap.add_argument("--graph-limit", type=int, default=4 * 1024 * 1024)
    ap.add_argument("--out", default=None, help="also append the JSON lines to this file")
    ap.add_argument("--multimem-blocks", type=int, default=0,
                    help="CTAs of the multimem kernel (0: configured default)")
    ap.add_argument("--multimem-sweep", action="store_true",
                    help="instead of the size sweep: the multimem kernel over CTA counts at 1, 64 and 256 MiB "
                         "(clamped to --max-bytes), one start-up")
    ap.add_argument("--one-shot-sweep", action="store_true",
                    help="instead of the size sweep: the one-shot kernel over its CTA cap at 4 KiB, 64 KiB, 1 MiB and "
                         "8 MiB beside NCCL and the upstream Triton kernel, each first compared bit for bit with the "
                         "default launch")
    return ap


def main(argv=None, standalone: bool = True) -> int:
    args = build_parser().parse_args(argv)

    from symm_mem_recipes_b200.bench._common import attempt, finish, init_distributed

    rank, local_rank, world, dev = init_distributed()

    import symm_mem_recipes_b200 as smr
    from symm_mem_recipes_b200.ops.config import AllReduceConfig
    from symm_mem_recipes_b200.parallel import symm_mem
    from symm_mem_recipes_b200.utils.benchmark import benchmark_with_event, benchmark_with_graph

    max_numel = args.max_bytes // 2
    torch.manual_seed(42 + rank)
    buf = symm_mem.empty(max_numel, dtype=torch.bfloat16, device=dev)
    buf.normal_()
    hdl = symm_mem.rendezvous(buf)
    plain = torch.randn(max_numel, device=dev).to(torch.bfloat16)
    cfg = AllReduceConfig()
    if args.multimem_blocks:
        cfg.multimem_max_blocks = args.multimem_blocks
    ref_fn = ref_buf = None
    if args.with_reference_triton:
        try:
            sys.path.insert(0, os.getcwd())
            from baseline.reference_triton import load_reference_one_shot
            ref_fn, ref_alloc = load_reference_one_shot()
            ref_buf = ref_alloc(min(max_numel, args.one_shot_limit // 2), dev)
            ref_buf.normal_()
        except Exception as e:  # noqa: BLE001
            if rank == 0:
                print(json.dumps({"impl": "reference_triton", "unavailable": f"{type(e).__name__}: {e}"}))
            ref_fn = None

    lines = []

    # the upstream driver's own check (triton_one_shot_all_reduce.py:145-154): all ones in, world size out
    ones = buf[:8192]
    ones.fill_(1)
    hdl.barrier()
    ones_ok = bool(smr.one_shot_all_reduce(ones, exit_barrier=True).eq(world).all())
    hdl.check()
    if rank == 0:
        print(json.dumps({"op": "all_reduce_check", "impl": "one_shot", "input": "ones[8192]",
                          "output_equals_world_size": ones_ok}), flush=True)
    # correctness gate before timing: every kernel against NCCL at two sizes
    if world > 1:
        for check_numel in (4096, 1 << 20):
            if check_numel > max_numel:
                continue
            torch.manual_seed(7 + rank)
            ref_in = torch.randn(check_numel, device=dev).to(torch.bfloat16)
            ref = ref_in.clone()
            dist.all_reduce(ref)
            tc = buf[:check_numel]
            results = {}
            tc.copy_(ref_in); hdl.barrier(); results["one_shot"] = smr.one_shot_all_reduce(tc, exit_barrier=True)
            tc.copy_(ref_in); hdl.barrier(); results["two_shot"] = smr.two_shot_all_reduce_(tc).clone()
            if hdl.has_multicast:
                hdl.barrier(); tc.copy_(ref_in); hdl.barrier()
                results["multimem"] = smr.multimem_all_reduce_(tc).clone()
            if check_numel * 2 <= 256 * 1024:
                results["low_latency"] = smr.low_latency_all_reduce(ref_in)
            hdl.barrier()
            hdl.check()
            scale = float(ref.float().abs().max())
            for name, got in results.items():
                err = float((got.float() - ref.float()).abs().max()) / scale
                if rank == 0:
                    print(json.dumps({"op": "all_reduce_check", "impl": name, "numel": check_numel,
                                      "max_rel_err_vs_nccl": round(err, 5), "ok": err < 2e-2}), flush=True)
        buf.normal_()

    def emit(rec):
        if rank == 0:
            s = json.dumps(rec)
            print(s, flush=True)
            lines.append(s)

    if args.one_shot_sweep:
        import itertools

        def variants(nbytes):
            for blocks in (24, 32, 64, 128, 192):
                if blocks == 32 or blocks * 512 * 16 <= nbytes:      # more CTAs than there is work: the same launch
                    yield dict(one_shot_max_blocks=blocks)

        for nbytes in (4096, 65536, 1 << 20, 8 << 20):
            if nbytes > args.max_bytes:
                continue
            t = buf[:nbytes // 2]
            out = torch.empty_like(t)
            hdl.barrier()
            want = smr.one_shot_all_reduce(t, exit_barrier=True).clone()
            if ref_fn is not None and nbytes // 2 <= ref_buf.numel():
                rt = ref_buf[:nbytes // 2]
                us = benchmark_with_graph(lambda: ref_fn(rt), calls_per_graph=20, warmup_iters=5, replays=10)
                emit({"op": "all_reduce_one_shot_sweep", "impl": "reference_triton", "world_size": world,
                      "bytes": nbytes, "us": round(us, 2)})
            us = benchmark_with_graph(lambda: dist.all_reduce(plain[:nbytes // 2]), calls_per_graph=20,
                                      warmup_iters=5, replays=10)
            emit({"op": "all_reduce_one_shot_sweep", "impl": "nccl", "world_size": world, "bytes": nbytes,
                  "us": round(us, 2)})
            for knobs in variants(nbytes):
                def one(knobs=knobs, t=t, out=out, nbytes=nbytes, want=want):
                    c = AllReduceConfig(**knobs)
                    smr.one_shot_all_reduce(t, out=out, exit_barrier=True, config=c)
                    hdl.check()
                    same = bool(torch.equal(out, want))
                    us = benchmark_with_graph(lambda: smr.one_shot_all_reduce(t, out=out, config=c),
                                              calls_per_graph=20, warmup_iters=5, replays=10)
                    hdl.check()
                    emit({"op": "all_reduce_one_shot_sweep", "impl": "one_shot", "world_size": world,
                          "bytes": nbytes, **{k.replace("one_shot_", ""): v for k, v in knobs.items()},
                          "same_bits_as_default": same, "us": round(us, 2),
                          "bus_gbs": round(2 * (world - 1) / world * nbytes / us / 1e3, 1)})

                if not attempt(f"one-shot sweep: {nbytes} bytes, {knobs}", one, dev, emit):
                    if not symm_mem.is_symm_mem_tensor(buf):
                        break
            if not symm_mem.is_symm_mem_tensor(buf):
                break
        if args.out and rank == 0:
            with open(args.out, "a") as f:
                f.write("\n".join(lines) + "\n")
        if standalone:
            finish()
        return 0

    if args.multimem_sweep:
        if world > 1 and hdl.has_multicast:
            for nbytes in (1 << 20, 64 << 20, 256 << 20):
                if nbytes > args.max_bytes:
                    continue
                t = buf[:nbytes // 2]
                for blocks in (4, 6, 8, 12, 16, 24):
                    def one(blocks=blocks, t=t, nbytes=nbytes):
                        c = AllReduceConfig(multimem_max_blocks=blocks)
                        if nbytes <= (4 << 20):
                            us = benchmark_with_graph(lambda: smr.multimem_all_reduce_(t, config=c),
                                                      calls_per_graph=20, warmup_iters=5, replays=10)
                        else:
                            us = benchmark_with_event(lambda: smr.multimem_all_reduce_(t, config=c), 5, 15,
                                                      flush_l2=False)
                        hdl.check()
                        buf.normal_()
                        emit({"op": "all_reduce_multimem_sweep", "world_size": world, "bytes": nbytes,
                              "blocks": blocks, "us": round(us, 2),
                              "bus_gbs": round(2 * (world - 1) / world * nbytes / us / 1e3, 1)})

                    if not attempt(f"multimem sweep: {nbytes} bytes, {blocks} CTAs", one, dev, emit):
                        # after a device-side timeout the buffer itself is gone (reset): stop the sweep
                        if not symm_mem.is_symm_mem_tensor(buf):
                            if args.out and rank == 0:
                                with open(args.out, "a") as f:
                                    f.write("\n".join(lines) + "\n")
                            if standalone:
                                finish()
                            return 1
        if args.out and rank == 0:
            with open(args.out, "a") as f:
                f.write("\n".join(lines) + "\n")
        if standalone:
            finish()
        return 0

    algos = [a for a in args.algos.split(",") if a]
    nbytes = args.min_bytes
    while nbytes <= args.max_bytes:
        numel = nbytes // 2
        t = buf[:numel]
        iters = args.iters if nbytes <= (16 << 20) else max(10, args.iters // 4)
        warm = args.warmup if nbytes <= (16 << 20) else 5
        impls = {}
        impls["nccl"] = lambda: dist.all_reduce(plain[:numel])
        for a in algos:
            if a == "low_latency" and nbytes <= 256 * 1024 and world > 1:
                src_ll = plain[:numel]
                out_ll = torch.empty_like(src_ll)
                impls["low_latency"] = lambda s_=src_ll, o_=out_ll: smr.low_latency_all_reduce(s_, out=o_, config=cfg)
            elif a == "one_shot" and nbytes <= args.one_shot_limit:
                out = torch.empty_like(t)
                impls["one_shot"] = lambda out=out: smr.one_shot_all_reduce(t, out=out, config=cfg)
            elif a == "two_shot" and world > 1:
                impls["two_shot"] = lambda: smr.two_shot_all_reduce_(t, config=cfg)
            elif a == "multimem" and world > 1 and hdl.has_multicast:
                impls["multimem"] = lambda: smr.multimem_all_reduce_(t, config=cfg)
            elif a == "auto":
                impls["auto:" + smr.ops.choose_algo(nbytes, world, hdl.has_multicast, cfg)] = \
                    lambda: smr.all_reduce(t, config=cfg)
        if ref_fn is not None and numel <= ref_buf.numel():
            rt = ref_buf[:numel]
            impls["reference_triton"] = lambda: ref_fn(rt)
        for name, fn in impls.items():
            if args.timing == "graph" and nbytes <= args.graph_limit:
                # device time per call; the eager number would mostly be CPU launch cost
                us = benchmark_with_graph(fn, calls_per_graph=20, warmup_iters=5, replays=10)
                how = "graph"
            else:
                us = benchmark_with_event(fn, warm, iters, flush_l2=False)
                how = "event"
            buf.normal_()   # in-place algorithms grow the values; refresh
            extra = {}
            if name == "multimem":
                extra = {"multimem_blocks": cfg.multimem_blocks(world)}
            emit({"op": "all_reduce", "impl": name, "world_size": world, "bytes": nbytes, "timing": how, **extra,
                  "us": round(us, 2), "alg_gbs": round(nbytes / us / 1e3, 2),
                  "bus_gbs": round(2 * (world - 1) / world * nbytes / us / 1e3, 2)})
        hdl.check()
        nbytes *= 2
    if args.out and rank == 0:
        with open(args.out, "a") as f:
            f.write("\n".join(lines) + "\n")
    if standalone:
        finish()
    return 0


if __name__ == "__main__":
    sys.exit(main())
