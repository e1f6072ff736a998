"""Llama-3-70B decoder layer under TP: fused kernels against NCCL + cuBLAS.

    torchrun --nnodes 1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m symm_mem_recipes_b200.bench.llama_layer --batch 16 --seq 2048

Times (device, CUDA events, max over ranks, L2 flushed before every timed call):
  * the two row-parallel projections alone (fused GEMM + reduce-scatter against
    cuBLAS + NCCL reduce-scatter): o-proj [T, 1024] x [8192, 1024]^T and
    down-proj [T, 3584] x [8192, 3584]^T per rank at TP8;
  * the whole prefill layer, fused and reference;
  * one decode step (batch 1/4/16), fused GEMV + all-reduce against cuBLAS + NCCL.
Random-init weights (seeded per rank), synthetic activations.  No upstream
counterpart: the upstream recipes time single ops (the fused all-gather
matmul, symm_mem_recipes/triton_all_gather_matmul.py:394-418); this is the
workload those ops were written for, with the shapes of its README.md:24-29 rows.
"""
from __future__ import annotations

import argparse
import json
import sys

import torch
import torch.distributed as dist


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--rs-panels", default="", help="matmul_reduce_scatter: comma-separated column-panel widths of the "
                                                    "tile order (N tiles of 256 columns per panel), each timed")
    ap.add_argument("--skip-layer", action="store_true")
    ap.add_argument("--fused-glue", default="env", choices=["env", "0", "1", "both", "all"],
                    help="norms / RoPE / SiLU-mul as single-pass kernels (1) or PyTorch compositions (0); "
                         "both: time the two; all: also with SiLU-mul inside the gate/up epilogue; "
                         "env: SMR_FUSED_GLUE / SMR_FUSED_SWIGLU")
    ap.add_argument("--breakdown", action="store_true", help="also print the device time of every phase of the layer")
    ap.add_argument("--tp", action="store_true",
                    help="also time the prefill without sequence parallelism (replicated activations, "
                         "matmul_all_reduce endings) against cuBLAS + NCCL all-reduce")
    ap.add_argument("--decode-graph", type=int, default=0, metavar="LAYERS",
                    help="also time serving-style decode: LAYERS layers captured in one CUDA graph (DecodeGraph, "
                         "cache of --decode-cache entries, position in a device tensor), replayed per token, "
                         "against the same steps launched eagerly")
    ap.add_argument("--decode-cache", type=int, default=4096)
    ap.add_argument("--out", default=None)
    return ap


def main(argv=None, standalone: bool = True) -> int:
    args = build_parser().parse_args(argv)
    from symm_mem_recipes_b200.bench._common import attempt, finish, init_distributed

    rank, local_rank, world, dev = init_distributed()

    import symm_mem_recipes_b200 as smr
    from symm_mem_recipes_b200.models.llama_tp_layer import LlamaTPConfig, LlamaTPDecoderLayer
    from symm_mem_recipes_b200.parallel import symm_mem
    from symm_mem_recipes_b200.utils.benchmark import benchmark_with_event, benchmark_with_graph

    cfg = LlamaTPConfig.llama3_70b()
    T = args.batch * args.seq
    assert T % (world * 128) == 0
    lines = []

    def emit(rec):
        if rank == 0:
            s = json.dumps(rec)
            print(s, flush=True)
            lines.append(s)

    bench = dict(warmup_iters=args.warmup, benchmark_iters=args.iters, flush_l2=True)
    torch.manual_seed(42 + rank)

    def section(what, fn) -> bool:
        """One part of the benchmark; its failure is recorded and the run goes on (see `attempt`)."""
        return attempt(what, fn, dev, emit)

    # ---- row-parallel projections alone ----
    for name, k_local in (("o_proj", cfg.n_heads // world * cfg.head_dim), ("down_proj", cfg.ffn // world)):
        a = (torch.randn(T, k_local, device=dev) * 0.02).to(torch.bfloat16)
        b = (torch.randn(cfg.hidden, k_local, device=dev) * 0.02).to(torch.bfloat16)
        wire = T * cfg.hidden * 2 * (world - 1) / world          # bytes leaving each GPU
        shared = {}

        def default_kernel(name=name, k_local=k_local, a=a, b=b, shared=shared, wire=wire):
            out = smr.matmul_reduce_scatter(a, b)
            symm_mem.check_status(dev)
            ref = smr.reference_matmul_reduce_scatter(a, b)
            ok = bool(torch.allclose(out.float(), ref.float(), rtol=5e-2, atol=5e-2))
            flops = 2.0 * T * cfg.hidden * k_local
            us_f = benchmark_with_event(lambda: smr.matmul_reduce_scatter(a, b, out), **bench)
            us_r = benchmark_with_event(lambda: smr.reference_matmul_reduce_scatter(a, b), **bench)
            us_mm = benchmark_with_event(lambda: torch.matmul(a, b.t()), **bench)
            symm_mem.check_status(dev)
            # phase breakdown from the kernel's own time stamps (one traced call)
            trace = torch.zeros(148, 4, dtype=torch.int64, device=dev)
            smr.matmul_reduce_scatter(a, b, out, trace=trace)
            torch.cuda.synchronize()
            tr = trace[trace[:, 0] > 0].double()
            t0 = tr[:, 0].min()
            phases = {"entered_us": float((tr[:, 1].max() - t0) / 1e3),
                      "gemm_done_first_us": float((tr[:, 2].min() - t0) / 1e3),
                      "gemm_done_last_us": float((tr[:, 2].max() - t0) / 1e3),
                      "reduced_last_us": float((tr[:, 3].max() - t0) / 1e3)}
            emit({"op": "matmul_reduce_scatter", "shape": name, "world_size": world, "M": T, "N": cfg.hidden,
                  "K_local": k_local, "matches_library": ok, "smr_fused_us": round(us_f, 1),
                  "cublas_plus_nccl_us": round(us_r, 1), "cublas_mm_only_us": round(us_mm, 1),
                  "fused_tflops": round(flops / us_f / 1e6, 1), "wire_gbs": round(wire / us_f / 1e3, 1),
                  "speedup": round(us_r / us_f, 3), "phases": {k: round(v, 1) for k, v in phases.items()}})
            shared.update(ref=ref, us_r=us_r)
            widths = [int(v) for v in args.rs_panels.split(",") if v]
            if widths:
                # candidates timed in turns (three cycles): the GPU's clock drifts by several per cent over the run
                import statistics

                short = dict(warmup_iters=2, benchmark_iters=max(3, args.iters // 3), flush_l2=True)
                runs, okay = {}, {}
                for cycle in range(3):
                    for pw in widths:
                        us_p = benchmark_with_event(lambda: smr.matmul_reduce_scatter(a, b, out, panel_w=pw), **short)
                        symm_mem.check_status(dev)
                        runs.setdefault(pw, []).append(round(us_p, 1))
                        okay[pw] = bool(torch.allclose(out.float(), ref.float(), rtol=5e-2, atol=5e-2))
                for pw, vals in runs.items():
                    emit({"op": "matmul_reduce_scatter", "shape": name, "world_size": world, "panel_w": pw,
                          "smr_fused_us": statistics.median(vals), "cycles_us": vals, "matches_library": okay[pw]})

        if not section(f"matmul_reduce_scatter {name}", default_kernel):
            continue
        del a, b, shared
    # ---- whole layer ----
    if not args.skip_layer:
        # (fused_glue, fused_swiglu)
        glue_variants = {"env": [(None, None)], "0": [(False, False)], "1": [(True, False)],
                         "both": [(False, False), (True, False)],
                         "all": [(False, False), (True, False), (True, True)]}[args.fused_glue]
        x = (torch.randn(T // world, cfg.hidden, device=dev) * 0.5).to(torch.bfloat16)
        lib = {}                               # timings of the library composition, measured once
        decode_layers = {}                     # fused_glue -> a layer built that way (decode ignores fused_swiglu)
        for glue, swiglu in glue_variants:
            def prefill(glue=glue, swiglu=swiglu):
                layer = LlamaTPDecoderLayer(cfg, dev, seed=1, fused_glue=glue, fused_swiglu=swiglu)
                y = layer.forward(x, args.batch, args.seq)
                symm_mem.check_status(dev)
                y_ref = layer.forward_reference(x, args.batch, args.seq)
                # the two forwards round partial sums at different places (bf16 partials summed in fp32 here,
                # bf16 reduce-scatter in NCCL): compare relative to the output's scale
                rel = float((y.float() - y_ref.float()).abs().max() / y_ref.float().abs().max())
                ok = rel < 3e-2
                us_f = benchmark_with_event(lambda: layer.forward(x, args.batch, args.seq), **bench)
                if "prefill" not in lib:
                    lib["prefill"] = benchmark_with_event(lambda: layer.forward_reference(x, args.batch, args.seq),
                                                          **bench)
                us_r = lib["prefill"]
                symm_mem.check_status(dev)
                emit({"op": "llama70b_layer_prefill", "world_size": world, "batch": args.batch, "seq": args.seq,
                      "fused_glue": layer.fused_glue, "fused_swiglu": layer.fused_swiglu, "matches_library": ok,
                      "max_rel_diff": round(rel, 5),
                      "smr_fused_us": round(us_f, 1), "nccl_cublas_us": round(us_r, 1),
                      "tokens_per_s_fused": round(T / us_f * 1e6), "speedup": round(us_r / us_f, 3)})
                decode_layers.setdefault(layer.fused_glue, layer)
                if args.breakdown:
                    phases = layer.phase_times_us(x, args.batch, args.seq)
                    symm_mem.check_status(dev)
                    emit({"op": "llama70b_layer_prefill_phases", "world_size": world, "fused_glue": layer.fused_glue,
                          "fused_swiglu": layer.fused_swiglu,
                          "rank": 0, "us": {k: round(v, 1) for k, v in phases.items()}})

            section(f"prefill, fused_glue={glue}, fused_swiglu={swiglu}", prefill)
        if not decode_layers:                  # every prefill section failed: decode still gets a plain layer
            decode_layers[False] = LlamaTPDecoderLayer(cfg, dev, seed=1, fused_glue=False, fused_swiglu=False)
        if args.tp:
            def tp_prefill():
                layer = decode_layers[max(decode_layers)]
                x_full = (torch.randn(T, cfg.hidden, device=dev) * 0.5).to(torch.bfloat16)
                if world > 1:
                    dist.broadcast(x_full, 0)
                y = layer.forward_tp(x_full, args.batch, args.seq)
                symm_mem.check_status(dev)
                y_ref = layer.forward_tp_reference(x_full, args.batch, args.seq)
                rel = float((y.float() - y_ref.float()).abs().max() / y_ref.float().abs().max())
                us_f = benchmark_with_event(lambda: layer.forward_tp(x_full, args.batch, args.seq), **bench)
                us_r = benchmark_with_event(lambda: layer.forward_tp_reference(x_full, args.batch, args.seq), **bench)
                symm_mem.check_status(dev)
                emit({"op": "llama70b_layer_prefill_tp", "world_size": world, "batch": args.batch, "seq": args.seq,
                      "fused_glue": layer.fused_glue, "fused_swiglu": layer.fused_swiglu,
                      "matches_library": rel < 3e-2, "max_rel_diff": round(rel, 5), "smr_fused_us": round(us_f, 1),
                      "nccl_cublas_us": round(us_r, 1), "speedup": round(us_r / us_f, 3)})

            section("prefill without sequence parallelism", tp_prefill)
        for B in (1, 4, 16):
            xd = (torch.randn(B, cfg.hidden, device=dev) * 0.5).to(torch.bfloat16)
            if world > 1:
                dist.broadcast(xd, 0)
            for glue_on, dlayer in sorted(decode_layers.items()):
                def decode(B=B, xd=xd, glue_on=glue_on, dlayer=dlayer):
                    kc = torch.zeros(B, 64, dlayer.hkv, cfg.head_dim, dtype=torch.bfloat16, device=dev)
                    vc = torch.zeros_like(kc)
                    y_f = dlayer.decode(xd, kc, vc, 0, fused=True)
                    symm_mem.check_status(dev)
                    y_r = dlayer.decode(xd, kc, vc, 0, fused=False)
                    rel = float((y_f.float() - y_r.float()).abs().max() / y_r.float().abs().max())
                    us_f = benchmark_with_graph(lambda: dlayer.decode(xd, kc, vc, 8, fused=True), calls_per_graph=5)
                    if ("decode", B) not in lib:           # the library composition does not depend on the glue switch
                        lib["decode", B] = benchmark_with_graph(lambda: dlayer.decode(xd, kc, vc, 8, fused=False),
                                                                calls_per_graph=5)
                    us_r = lib["decode", B]
                    symm_mem.check_status(dev)
                    emit({"op": "llama70b_layer_decode", "world_size": world, "batch": B, "timing": "graph",
                          "fused_glue": bool(glue_on), "matches_library": rel < 3e-2, "max_rel_diff": round(rel, 5),
                          "smr_fused_us": round(us_f, 1), "nccl_cublas_us": round(us_r, 1),
                          "speedup": round(us_r / us_f, 3)})

                section(f"decode batch {B}, fused_glue={bool(glue_on)}", decode)
    if args.decode_graph > 0:
        from symm_mem_recipes_b200.models.llama_tp_layer import DecodeGraph
        from symm_mem_recipes_b200.utils.benchmark import max_over_ranks

        stack = [LlamaTPDecoderLayer(cfg, dev, seed=100 + i) for i in range(args.decode_graph)]
        for B in (1, 4, 16):
            def decode_from_graph(B=B):
                xd = (torch.randn(B, cfg.hidden, device=dev) * 0.5).to(torch.bfloat16)
                if world > 1:
                    dist.broadcast(xd, 0)
                graph = DecodeGraph(stack, B, args.decode_cache)
                steps = min(32, args.decode_cache)
                first = min(args.decode_cache // 2, args.decode_cache - steps)

                def replayed():
                    for i in range(steps):
                        graph.step(xd, first + i)

                def eager():
                    for i in range(steps):
                        h = xd
                        for lyr, (kc, vc) in zip(stack, graph.caches):
                            h = lyr.decode(h, kc, vc, first + i, fused=True)

                times = {}
                for name, fn in (("graph", replayed), ("eager", eager)):
                    fn()
                    beg, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    torch.cuda.synchronize()
                    if world > 1:
                        dist.barrier()
                    beg.record()
                    fn()
                    end.record()
                    torch.cuda.synchronize()
                    times[name] = max_over_ranks(beg.elapsed_time(end) * 1e3 / steps, dev)
                symm_mem.check_status(dev)
                emit({"op": "llama70b_decode_graph", "world_size": world, "batch": B, "layers": args.decode_graph,
                      "cache_entries": args.decode_cache, "first_position": first, "steps": steps,
                      "graph_us_per_step": round(times["graph"], 1), "eager_us_per_step": round(times["eager"], 1),
                      "speedup": round(times["eager"] / times["graph"], 3)})

            section(f"decode from one CUDA graph, batch {B}", decode_from_graph)
    if args.out and rank == 0:
        with open(args.out, "a") as f:
            f.write("\n".join(lines) + "\n")
    if standalone:
        finish()
    return 0


if __name__ == "__main__":
    sys.exit(main())
