"""Single-GPU timing of the tcgen05 GEMM (the `mm_only` arm of the upstream
driver, symm_mem_recipes/triton_all_gather_matmul.py:394-405) against cuBLAS,
and of the world-of-one GEMV and all-reduce kernels.  Also the program that
`ncu` wraps for the per-kernel profiles under profiles/.

    python -m symm_mem_recipes_b200.bench.matmul --M 16384 --N 3584 --K 8192
    python -m symm_mem_recipes_b200.bench.matmul --op gemv --batch 16
    python -m symm_mem_recipes_b200.bench.matmul --op glue --M 32768          # RMSNorm, RoPE, SiLU-mul kernels
    python -m symm_mem_recipes_b200.bench.matmul --op matmul --variant fp8    # or swiglu
"""
from __future__ import annotations

import argparse
import json
import sys

import torch


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="matmul", choices=["matmul", "gemv", "all_reduce", "glue"])
    ap.add_argument("--variant", default="bf16", choices=["bf16", "fp8", "swiglu"],
                    help="matmul: float8_e4m3fn operands and output, or the SwiGLU epilogue (N = 2 x FFN width)")
    ap.add_argument("--gemv-algo", default=None, help="gemv: tc, tc_tagged or simt")
    ap.add_argument("--weights-nk", action="store_true",
                    help="gemv: weights stored [N, K] (the column-parallel projections of a decode step: "
                         "--N 1280 --K 8192 is QKV, --N 7168 --K 8192 gate / up at TP8)")
    ap.add_argument("--M", type=int, default=16384)
    ap.add_argument("--N", type=int, default=3584)
    ap.add_argument("--K", type=int, default=8192)
    ap.add_argument("--block-n", type=int, default=0)
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--bytes", type=int, default=64 * 1024 * 1024)
    ap.add_argument("--ar-algo", default="one_shot", choices=["one_shot", "low_latency"],
                    help="all_reduce: the kernel to time in a world of one")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--no-cublas", action="store_true")
    ap.add_argument("--eager", action="store_true",
                    help="gemv: time eager launches with events instead of graph replay (for profilers)")
    args = ap.parse_args()

    import symm_mem_recipes_b200 as smr
    from symm_mem_recipes_b200.ops.ag_matmul import AgMatmulConfig, choose_block_n
    from symm_mem_recipes_b200.parallel import symm_mem
    from symm_mem_recipes_b200.utils.benchmark import (ClockSampler, benchmark_with_event,
                                                       benchmark_with_graph)

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    bench = dict(warmup_iters=args.warmup, benchmark_iters=args.iters, flush_l2=True, all_ranks_max=False)
    out = {"op": args.op}
    with ClockSampler(0, period_ms=100) as clocks:
        if args.op == "matmul":
            M, N, K = args.M, args.N, args.K
            dt = torch.float8_e4m3fn if args.variant == "fp8" else torch.bfloat16
            a = (torch.randn(M, K, device=dev) * 0.02).to(dt)
            b = (torch.randn(N, K, device=dev) * 0.02).to(dt)
            epilogue = "swiglu" if args.variant == "swiglu" else None
            c = torch.empty(M, N // 2 if epilogue else N, dtype=dt, device=dev)
            flops = 2.0 * M * N * K
            cfg = AgMatmulConfig(block_n=args.block_n)
            us = benchmark_with_event(lambda: smr.matmul(a, b, c, cfg, epilogue), **bench)
            out.update(smr_us=round(us, 1), smr_tflops=round(flops / us / 1e6, 1))
            out.update(M=M, N=N, K=K, variant=args.variant, block_n=args.block_n or choose_block_n(M, N, 148))
            if not args.no_cublas and args.variant == "bf16":
                bt = b.t()
                us2 = benchmark_with_event(lambda: torch.matmul(a, bt, out=c), **bench)
                out.update(cublas_us=round(us2, 1), cublas_tflops=round(flops / us2 / 1e6, 1))
        elif args.op == "gemv":
            # decode shape: x [b, 3584], W [3584, 8192] unless given; device time from graph replay
            # over four weight copies (224 MB > L2) so that every call streams from HBM
            K = args.K if args.K != 8192 or args.N != 3584 else 3584
            N = args.N if args.K != 8192 or args.N != 3584 else 8192
            x = (torch.randn(args.batch, K, device=dev) * 0.02).to(torch.bfloat16)
            wshape = (N, K) if args.weights_nk else (K, N)
            n_copies = max(4, -(-256 * 1024 * 1024 // (K * N * 2)))      # cycled copies: more than the L2 holds
            ws_ = [(torch.randn(*wshape, device=dev) * 0.02).to(torch.bfloat16) for _ in range(n_copies)]
            y = torch.empty(args.batch, N, dtype=torch.bfloat16, device=dev)
            state = {"i": 0}

            def fused():
                state["i"] = (state["i"] + 1) % n_copies
                smr.gemv_all_reduce(x, ws_[state["i"]], y, algo=args.gemv_algo, weights_nk=args.weights_nk)

            def lib():
                state["i"] = (state["i"] + 1) % n_copies
                torch.matmul(x, ws_[state["i"]].t() if args.weights_nk else ws_[state["i"]])

            fused()
            if args.eager:
                us = benchmark_with_event(fused, **bench)
            else:
                us = benchmark_with_graph(fused, calls_per_graph=2 * n_copies, replays=10, all_ranks_max=False)
            out.update(batch=args.batch, K=K, N=N, smr_us=round(us, 2), timing="event" if args.eager else "graph",
                       weight_gbs=round(K * N * 2 / us / 1e3, 1))
            if not args.no_cublas and not args.eager:
                us2 = benchmark_with_graph(lib, calls_per_graph=2 * n_copies, replays=10, all_ranks_max=False)
                out.update(cublas_us=round(us2, 2))
        elif args.op == "glue":
            # the layer-glue kernels at the decoder layer's per-rank sizes: T tokens, hidden 8192,
            # 8 + 1 + 1 heads of 128 in the QKV buffer, FFN 3584 per rank; all bound by HBM
            from symm_mem_recipes_b200 import ops
            T = args.M
            x = (torch.randn(T // 8, 8192, device=dev) * 0.5).to(torch.bfloat16)
            r = (torch.randn(T // 8, 8192, device=dev) * 0.5).to(torch.bfloat16)
            w = torch.ones(8192, dtype=torch.bfloat16, device=dev)
            o1, s1 = torch.empty_like(x), torch.empty_like(x)
            qkv = (torch.randn(T, 1280, device=dev) * 0.5).to(torch.bfloat16)
            gu = (torch.randn(T, 7168, device=dev) * 0.5).to(torch.bfloat16)
            act = torch.empty(T, 3584, dtype=torch.bfloat16, device=dev)
            cases = {
                "rms_norm": (lambda: ops.rms_norm(x, w, 1e-5, out=o1), 2 * x.numel() * 2),
                "add_rms_norm": (lambda: ops.rms_norm(x, w, 1e-5, out=o1, residual=r, sum_out=s1), 4 * x.numel() * 2),
                "rope": (lambda: ops.rope_(qkv, 9, 128, 2048, 500000.0), 2 * T * 9 * 128 * 2),
                "silu_mul": (lambda: ops.silu_mul(gu, act), (gu.numel() + act.numel()) * 2),
            }
            # one decode step's attention over a full cache of 4096 entries (8 query heads on one KV head of 128)
            for batch in (1, 16):
                kc = (torch.randn(batch, 4096, 1, 128, device=dev) * 0.5).to(torch.bfloat16)
                vc = torch.randn_like(kc)
                step = (torch.randn(batch, 10 * 128, device=dev) * 0.5).to(torch.bfloat16)
                cases[f"decode_attention_b{batch}_s4096"] = (
                    lambda step=step, kc=kc, vc=vc: ops.decode_attention_(step, kc, vc, 8, 4095),
                    2 * kc.numel() * 2)
            for name, (fn, nbytes) in cases.items():
                us = benchmark_with_event(fn, **bench)
                out[name] = {"us": round(us, 1), "gbs": round(nbytes / us / 1e3, 1)}
            out["tokens"] = T
        else:
            numel = args.bytes // 2
            t = symm_mem.empty(numel, dtype=torch.bfloat16, device=dev)
            t.normal_()
            o = torch.empty_like(t)
            if args.ar_algo == "low_latency":
                us = benchmark_with_event(lambda: smr.low_latency_all_reduce(t, out=o), **bench)
                out.update(bytes=args.bytes, low_latency_us=round(us, 2))
            else:
                us = benchmark_with_event(lambda: smr.one_shot_all_reduce(t, out=o), **bench)
                out.update(bytes=args.bytes, one_shot_us=round(us, 2),
                           read_write_gbs=round(2 * args.bytes / us / 1e3, 1))
        symm_mem.check_status(dev)
    out["clocks"] = clocks.summary()
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
