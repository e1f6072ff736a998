"""all_gather_matmul benchmark with the flags and the four timings of the
upstream driver (symm_mem_recipes/triton_all_gather_matmul.py:329-427):
cuBLAS mm only, this package's mm only, cuBLAS + NCCL, fused.

    torchrun --nnodes 1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m symm_mem_recipes_b200.bench.all_gather_matmul --M 16384 --N 3584 --K 8192

M is the gathered row count; N and K are the per-rank weight dims.  Median of
`--iters` timed calls after `--warmup`, L2 flushed before each, CUDA events,
maximum over ranks.  `--upstream-table` runs the nine shapes of the upstream
README (three models x M in 4096, 8192, 16384, README.md:17-36) and attaches the
numbers published there (8 x H100) to every record.
"""
from __future__ import annotations

import argparse
import json
import sys

import torch
import torch.distributed as dist


# upstream README.md:20-36, µs on 8 x H100: (N, K) -> M -> (cuBLAS, Triton mm, cuBLAS + NCCL, fused)
UPSTREAM_TABLE = {
    (1792, 4096): {4096: (105, 125, 230, 213), 8192: (194, 236, 416, 318), 16384: (391, 434, 819, 514)},
    (3584, 8192): {4096: (403, 483, 652, 543), 8192: (828, 849, 1291, 948), 16384: (1672, 1655, 2541, 1846)},
    (6656, 16384): {4096: (1558, 1595, 2077, 1776), 8192: (2879, 2953, 3847, 3243),
                    16384: (5842, 5948, 7801, 6538)},
}


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser()
    ap.add_argument("--M", type=int, default=4096)
    ap.add_argument("--N", type=int, default=6656)
    ap.add_argument("--K", type=int, default=16384)
    ap.add_argument("--BLOCK_SIZE_N", "--block-n", dest="block_n", type=int, default=0)
    # accepted for command-line compatibility with the upstream driver (:330-339); the M tile (128 per
    # CTA), the K tile (64), the stage count and the warp roles are fixed by the kernel design
    ap.add_argument("--BLOCK_SIZE_M", type=int, default=128, help="fixed: 128 rows per CTA (256 per CTA pair)")
    ap.add_argument("--BLOCK_SIZE_K", type=int, default=64, help="fixed: one 128-byte swizzle row")
    ap.add_argument("--GROUP_SIZE_M", type=int, default=1, help="ignored: tiles are scheduled N-fastest")
    ap.add_argument("--num_stages", type=int, default=0, help="ignored: follows from the tile (4-8 stages)")
    ap.add_argument("--num_warps", type=int, default=6, help="fixed: TMA, MMA and four epilogue warps")
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--iters", type=int, default=25)
    ap.add_argument("--out", default=None)
    ap.add_argument("--with-plain-a-out", "--with-push-copy", dest="with_plain_a_out", action="store_true",
                    help="also time the upstream calling convention: an ordinary (non-symmetric) a_out, served "
                         "through the internal symmetric buffer plus one local copy")
    ap.add_argument("--leads", default="", help="push mode: comma-separated counts of own 128-row blocks multiplied "
                                                "before the first remote one, each timed")
    ap.add_argument("--pacings", default="", help="push mode: comma-separated AHEAD[:LEAD[:PLAIN[:PIECES]]] settings, each timed "
                                                  "(rounds of lookahead of the broadcast; own blocks first, -1 = default; "
                                                  "1 = plain peer stores, 0 = multimem, -1 = by world size; pieces per block)")
    ap.add_argument("--panels", default="", help="comma-separated column-panel widths of the tile order (N tiles per "
                                                 "panel), each timed for the GEMM alone and for the fused op")
    ap.add_argument("--trace", action="store_true",
                    help="print the per-CTA timing record of one fused call and one GEMM-only call, per rank")
    ap.add_argument("--per-rank", action="store_true", help="also print every rank's own median beside the maximum")
    ap.add_argument("--upstream-table", action="store_true",
                    help="run the nine (model, M) shapes of the upstream README instead of --M/--N/--K")
    ap.add_argument("--print-ptxas", "--print_ptx", dest="print_ptxas", action="store_true",
                    help="print what the compiler made of the kernels (registers, spills, shared memory from "
                         "`ptxas -v`); upstream's --print_ptx dumps Triton's PTX at this point")
    return ap


def main(argv=None, standalone: bool = True) -> int:
    args = build_parser().parse_args(argv)

    from symm_mem_recipes_b200.bench._common import finish, init_distributed

    rank, local_rank, world, dev = init_distributed()

    lines = []
    if args.upstream_table:
        shapes = [(M, N, K) for (N, K), by_m in UPSTREAM_TABLE.items() for M in by_m]
    else:
        shapes = [(args.M, args.N, args.K)]
    for M, N, K in shapes:
        _one_shape(args, M, N, K, rank, world, dev, lines)
    if args.print_ptxas and rank == 0:
        from symm_mem_recipes_b200 import _build
        print(_build.ptxas_report())
    if args.out and rank == 0:
        with open(args.out, "a") as f:
            f.write("\n".join(lines) + "\n")
    if standalone:
        finish()
    return 0


def _one_shape(args, M, N, K, rank, world, dev, lines) -> None:
    import symm_mem_recipes_b200 as smr
    from symm_mem_recipes_b200.ops.ag_matmul import AgMatmulConfig
    from symm_mem_recipes_b200.parallel import symm_mem
    from symm_mem_recipes_b200.utils.benchmark import benchmark_with_event

    assert M % world == 0
    torch.manual_seed(42 + rank)
    a_shard = symm_mem.empty(M // world, K, dtype=torch.bfloat16, device=dev)
    a_shard.copy_((torch.randn(M // world, K, device=dev) * 0.02).to(torch.bfloat16))
    a = (torch.randn(M, K, device=dev) * 0.02).to(torch.bfloat16)
    b = (torch.randn(N, K, device=dev) * 0.02).to(torch.bfloat16)
    bt = b.t()
    c = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    a_out = symm_mem.empty(M, K, dtype=torch.bfloat16, device=dev)       # push (broadcast) path
    a_out_plain = torch.empty(M, K, dtype=torch.bfloat16, device=dev)    # the upstream calling convention
    symm_mem.rendezvous(a_shard)
    symm_mem.rendezvous(a_out)
    flops = 2.0 * M * N * K
    published = UPSTREAM_TABLE.get((N, K), {}).get(M)
    published_by_impl = {} if published is None or world != 8 else {
        "cublas_mm_only": published[0], "smr_mm_only": published[1], "cublas_plus_nccl": published[2],
        "smr_fused": published[3]}

    def emit(name, us, **extra):
        rec = {"op": "all_gather_matmul", "impl": name, "world_size": world, "M": M, "N": N, "K": K,
               "us": round(us, 1), "tflops": round(flops / us / 1e6, 1), **extra}
        if name in published_by_impl:
            # the same row of the upstream table (for smr_mm_only: upstream's Triton mm only)
            rec["upstream_8xh100_us"] = published_by_impl[name]
        if rank == 0:
            s = json.dumps(rec)
            print(s, flush=True)
            lines.append(s)

    c0 = smr.reference_all_gather_matmul(a_shard, b)
    c1 = smr.all_gather_matmul(a_shard, b, a_out, c)
    symm_mem.check_status(dev)
    assert torch.allclose(c0.float(), c1.float(), rtol=2e-2, atol=2e-3), "fused != NCCL + cuBLAS"

    bench = dict(warmup_iters=args.warmup, benchmark_iters=args.iters, flush_l2=True)

    def timed(fn):
        """Maximum over ranks of the per-rank medians; with --per-rank also the list of them."""
        own = benchmark_with_event(fn, all_ranks_max=False, **bench)
        per_rank = [None] * world
        if world > 1:
            dist.all_gather_object(per_rank, round(own, 1))
        else:
            per_rank = [round(own, 1)]
        return max(per_rank), ({"per_rank_us": per_rank} if args.per_rank else {})

    us, extra = timed(lambda: torch.matmul(a, bt, out=c))
    emit("cublas_mm_only", us, **extra)
    cfg0 = AgMatmulConfig(block_n=args.block_n)
    us, extra = timed(lambda: smr.matmul(a, b, c, cfg0))
    emit("smr_mm_only", us, **extra)
    us, extra = timed(lambda: smr.reference_all_gather_matmul(a_shard, b))
    emit("cublas_plus_nccl", us, **extra)
    gathered = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
    us, extra = timed(lambda: dist.all_gather_into_tensor(gathered, a_shard))
    emit("nccl_all_gather_only", us, **extra)
    us, extra = timed(lambda: smr.all_gather_matmul(a_shard, b, a_out, c, cfg0))
    emit("smr_fused", us, gather="push", **extra)
    symm_mem.check_status(dev)
    for lead in [int(x) for x in args.leads.split(",") if x]:
        cfgl = AgMatmulConfig(block_n=args.block_n, lead=lead)
        us, extra = timed(lambda: smr.all_gather_matmul(a_shard, b, a_out, c, cfgl))
        emit("smr_fused", us, gather="push", lead=lead, **extra)
        symm_mem.check_status(dev)
    widths = [int(x) for x in args.panels.split(",") if x]
    if widths:
        # the GPU's clock drifts by several per cent over a run of this length, so the candidates are
        # timed in turns (three cycles over all of them) and the median of a candidate's cycles is reported
        import statistics

        short = dict(warmup_iters=2, benchmark_iters=max(3, args.iters // 3), flush_l2=True)
        runs = {}
        for cycle in range(3):
            for pw in widths:
                cfgw = AgMatmulConfig(block_n=args.block_n, panel_w=pw)
                for what, fn in (("cublas_mm_only", lambda: torch.matmul(a, bt, out=c)),
                                 ("smr_mm_only", lambda: smr.matmul(a, b, c, cfgw)),
                                 ("smr_fused", lambda: smr.all_gather_matmul(a_shard, b, a_out, c, cfgw))):
                    if what == "cublas_mm_only" and pw != widths[0]:
                        continue
                    own = benchmark_with_event(fn, all_ranks_max=True, **short)
                    runs.setdefault((what, pw), []).append(round(own, 1))
                symm_mem.check_status(dev)
        for (what, pw), vals in runs.items():
            extra = {} if what == "cublas_mm_only" else {"panel_w": pw}
            emit(what, statistics.median(vals), timing="three interleaved cycles", cycles_us=vals, **extra)
    for spec in [x for x in args.pacings.split(",") if x]:
        parts = [int(v) for v in spec.split(":")]
        cfgp = AgMatmulConfig(block_n=args.block_n, push_ahead=parts[0],
                              lead=parts[1] if len(parts) > 1 else -1,
                              push_plain_stores=parts[2] if len(parts) > 2 else -1,
                              push_pieces=parts[3] if len(parts) > 3 else 0)
        us, extra = timed(lambda: smr.all_gather_matmul(a_shard, b, a_out, c, cfgp))
        emit("smr_fused", us, gather="push", pacing=spec, **extra)
        symm_mem.check_status(dev)
    if args.trace:
        from symm_mem_recipes_b200.ops.ag_matmul import summarize_trace
        from symm_mem_recipes_b200.utils.benchmark import flush_l2

        for what, fn in (("smr_fused", lambda tr: smr.all_gather_matmul(a_shard, b, a_out, c, cfg0, trace=tr)),
                         ("smr_mm_only", lambda tr: smr.matmul(a, b, c, cfg0, trace=tr))):
            tr = torch.zeros(160, 12, dtype=torch.int64, device=dev)
            for _ in range(3):
                fn(tr)
            torch.cuda.synchronize()
            dist.barrier() if world > 1 else None
            tr.zero_()
            flush_l2(dev)
            fn(tr)
            torch.cuda.synchronize()
            summ = summarize_trace(tr)
            all_s = [None] * world
            if world > 1:
                dist.all_gather_object(all_s, summ)
            else:
                all_s = [summ]
            if rank == 0:
                for r, s_ in enumerate(all_s):
                    line = json.dumps({"op": "all_gather_matmul_trace", "impl": what, "world_size": world,
                                       "rank": r, "M": M, "N": N, "K": K, "us": s_})
                    print(line, flush=True)
                    lines.append(line)
        symm_mem.check_status(dev)
    if args.with_plain_a_out:
        def plain_a_out():
            us = benchmark_with_event(lambda: smr.all_gather_matmul(a_shard, b, a_out_plain, c, cfg0), **bench)
            symm_mem.check_status(dev)
            if not torch.allclose(c0.float(), c.float(), rtol=2e-2, atol=2e-3):
                raise RuntimeError("the result with an ordinary a_out differs from NCCL + cuBLAS")
            emit("smr_fused", us, gather="push_copy")

        from symm_mem_recipes_b200.bench._common import attempt
        attempt("all_gather_matmul with an ordinary a_out", plain_a_out, dev,
                lambda rec: (print(json.dumps(rec), flush=True), lines.append(json.dumps(rec))) if rank == 0 else None)


if __name__ == "__main__":
    sys.exit(main())
