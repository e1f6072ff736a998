"""Every op of the package once, on small shapes, against the library
composition or a PyTorch reference, in ONE start-up.

    python -m symm_mem_recipes_b200.selfcheck                       # one GPU: world-of-one forms
    torchrun --nnodes 1 --nproc-per-node 2 --master-addr 127.0.0.1 -m symm_mem_recipes_b200.selfcheck
    ... -m symm_mem_recipes_b200.selfcheck --only gemv,glue --list

An installation check for users, and the cheapest way to try many kernel
variants on hardware: the pytest suite starts a fresh set of processes per
case, this program starts once.  Rank 0 prints one line per check and a JSON
summary; the exit code is the number of failed checks.  After every check the
ranks agree on its outcome; after a check that ends in a device-side timeout
(the allocations it used are then in an unknown state) the ranks drop all
symmetric memory together and carry on with fresh allocations.
No upstream counterpart (the upstream drivers check one op each:
symm_mem_recipes/triton_one_shot_all_reduce.py:145-154,
triton_all_gather_matmul.py:390-392).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
import traceback

import torch
import torch.distributed as dist


def _close(got: torch.Tensor, ref: torch.Tensor, rtol: float = 3e-2, atol: float = 3e-2) -> tuple[bool, float]:
    err = (got.float() - ref.float()).abs()
    ok = bool((err <= ref.float().abs() * rtol + atol).all())
    return ok, float(err.max())


_SHARED_STATE: list = []
_MAX_RECOVERIES = 8


def build_checks(world: int, rank: int, dev: torch.device) -> list:
    """[(group, name, is_variant, fn)]; fn() -> (ok, detail).  `is_variant`: an opt-in variant of an op
    (run after the default forms)."""
    import symm_mem_recipes_b200 as smr
    from symm_mem_recipes_b200 import ops
    from symm_mem_recipes_b200.models.llama_tp_layer import LlamaTPConfig, LlamaTPDecoderLayer
    from symm_mem_recipes_b200.ops.ag_matmul import AgMatmulConfig, gather_buffer
    from symm_mem_recipes_b200.ops.config import AllReduceConfig
    from symm_mem_recipes_b200.parallel import symm_mem

    multi = world > 1
    checks: list = []

    def add(group, name, fn, variant=False):
        checks.append((group, name, variant, fn))

    def randn(*shape, std=0.05, seed=0):
        g = torch.Generator(device="cpu").manual_seed(seed)
        return (torch.randn(*shape, generator=g) * std).to(torch.bfloat16).to(dev)

    # ------------------------------------------------------------------ all-reduce and barriers
    numel = 1 << 16
    state: dict = {}
    _SHARED_STATE.append(state)      # symmetric tensors kept between checks; dropped when main() resets the module

    def ar_setup():
        if "t" not in state:
            t = symm_mem.empty(numel, dtype=torch.bfloat16, device=dev)
            state["t"], state["hdl"] = t, symm_mem.rendezvous(t)
            state["src"] = randn(numel, std=1.0, seed=100 + rank)
            ref = state["src"].clone()
            if multi:
                dist.all_reduce(ref)
            state["ref"] = ref
        state["hdl"].barrier()
        state["t"].copy_(state["src"])
        state["hdl"].barrier()
        return state["t"], state["hdl"], state["ref"]

    def ar(algo, cfg=None):
        def fn():
            t, hdl, ref = ar_setup()
            kw = {"config": cfg} if cfg is not None else {}
            if algo == "one_shot":
                got = smr.one_shot_all_reduce(t, exit_barrier=True, **kw)
            elif algo == "low_latency":
                got = smr.low_latency_all_reduce(state["src"], **kw)
            else:
                got = {"two_shot": smr.two_shot_all_reduce_, "multimem": smr.multimem_all_reduce_,
                       "auto": smr.all_reduce}[algo](t, **kw)
            hdl.check()
            return _close(got, ref, 2e-2, 5e-2)
        return fn

    add("all_reduce", "one_shot", ar("one_shot"))
    add("all_reduce", "two_shot", ar("two_shot"))
    add("all_reduce", "low_latency", ar("low_latency"))
    add("all_reduce", "auto", ar("auto"))
    if multi:
        add("all_reduce", "multimem", ar("multimem"))
        add("all_reduce", "multimem, 16 CTAs", ar("multimem", AllReduceConfig(multimem_max_blocks=16)),
            True)

    def barriers(kind):
        def fn():
            _, hdl, _ = ar_setup()
            if kind == "nvls" and not hdl.has_multicast:
                return True, "skipped: no multicast mapping"
            for blocks in (1, 32, 148):
                for _ in range(20):
                    smr.barrier_test(hdl, num_blocks=blocks, kind=kind, timeout_ms=2000)
            hdl.check()
            return True, ""
        return fn

    add("barrier", "blockwise_barrier (CAS)", barriers("cas"))
    add("barrier", "epoch barrier", barriers("epoch"), True)
    if multi:
        add("barrier", "NVLS barrier", barriers("nvls"), True)

        def signals():
            _, hdl, _ = ar_setup()
            nxt, prv = (rank + 1) % world, (rank - 1) % world
            probe = symm_mem.empty(1024, dtype=torch.float32, device=dev)
            ph = symm_mem.rendezvous(probe)
            for it in range(5):
                probe.fill_(float(10 * it + rank))
                ph.put_signal(nxt, channel=3, timeout_ms=2000)
                ph.wait_signal(prv, channel=3, timeout_ms=2000)
                got = ph.get_buffer(prv, (1024,), torch.float32).clone()
                ph.barrier(channel=1)
                if float(got[-1]) != float(10 * it + prv):
                    return False, f"iteration {it}: read {float(got[-1])}"
            ph.check()
            return True, ""

        add("barrier", "put_signal / wait_signal", signals, True)

    # ------------------------------------------------------------------ all_gather_matmul
    rows, N, K = 256, 512, 1024
    M = rows * world

    def agmm(mode, dtype=torch.bfloat16, epilogue=None, cfg=None):
        def fn():
            cfg_ = cfg or AgMatmulConfig(timeout_ms=5000)
            a_full = randn(M, K, std=0.25, seed=7).to(dtype)
            b = randn(N, K, std=0.25, seed=8).to(dtype)
            a_shard = symm_mem.empty(rows, K, dtype=dtype, device=dev)
            a_shard.copy_(a_full[rank * rows:(rank + 1) * rows])
            if multi:
                symm_mem.rendezvous(a_shard)
            if mode == "push":
                a_out = symm_mem.empty(M, K, dtype=dtype, device=dev)
            elif mode == "plain":
                a_out = torch.zeros(M, K, dtype=dtype, device=dev)
            else:
                a_out = None
            got = smr.all_gather_matmul(a_shard, b, a_out, config=cfg_, epilogue=epilogue)
            symm_mem.check_status(dev)
            ref = a_full.float() @ b.float().t()
            if epilogue == "swiglu":
                tiles = ref.view(M, -1, 2, 128)
                ref = (torch.nn.functional.silu(tiles[:, :, 0]) * tiles[:, :, 1]).reshape(M, -1)
            if a_out is None and multi:
                a_out = gather_buffer(M, K, dev, None, dtype)
            gathered_ok = a_out is None or torch.equal(a_out.view(torch.uint8), a_full.view(torch.uint8))
            ok, err = _close(got, ref, 2.0 ** -3 if dtype != torch.bfloat16 else 3e-2, 3e-2)
            return ok and gathered_ok, f"max err {err:.4f}" + ("" if gathered_ok else "; a_out differs from the gather")
        return fn

    add("all_gather_matmul", "push (symmetric a_out)", agmm("push"))
    add("all_gather_matmul", "internal buffer", agmm("internal"))
    if multi:
        add("all_gather_matmul", "ordinary a_out (gather into the internal buffer, one copy)", agmm("plain"))
    add("all_gather_matmul", "float8_e4m3fn", agmm("push", dtype=torch.float8_e4m3fn), True)
    add("all_gather_matmul", "SwiGLU epilogue", agmm("push", epilogue="swiglu"), True)

    # ------------------------------------------------------------------ row-parallel GEMMs
    def row_parallel(op, **kw):
        def fn():
            Mr, Nr, Kr = 256 * world, 328, 192
            a = randn(Mr, Kr, seed=20 + rank)
            b = randn(Nr, Kr, seed=40 + rank)
            full = (a.float() @ b.float().t()).to(torch.bfloat16).float()
            if multi:
                dist.all_reduce(full)
            if op == "rs":
                got = smr.matmul_reduce_scatter(a, b, **kw)
                r = Mr // world
                ref = full[rank * r:(rank + 1) * r]
            else:
                got = smr.matmul_all_reduce(a, b, **kw)
                ref = full
            symm_mem.check_status(dev)
            ok, err = _close(got, ref)
            return ok, f"max err {err:.4f}"
        return fn

    add("matmul_reduce_scatter", "default", row_parallel("rs"))
    add("matmul_all_reduce", "default", row_parallel("ar"))

    # ------------------------------------------------------------------ GEMV + all-reduce
    def gemv(algo, B, nk=False):
        def fn():
            x = randn(B, 1024, std=0.5, seed=60 + rank)
            w = randn(1024, 512, seed=80 + rank)
            ref = x.float() @ w.float()
            if multi:
                dist.all_reduce(ref)
            w_arg = w.t().contiguous() if nk else w
            for _ in range(3):
                got = smr.gemv_all_reduce(x, w_arg, algo=algo, weights_nk=nk)
            symm_mem.check_status(dev)
            ok, err = _close(got, ref, 2.0 ** -6, 3e-2)
            return ok, f"max err {err:.4f}"
        return fn

    for B in (1, 16):
        add("gemv", f"tcgen05, batch {B}", gemv("tc", B))
        add("gemv", f"CUDA cores, batch {B}", gemv("simt", B))
        add("gemv", f"tcgen05 tagged words, batch {B}", gemv("tc_tagged", B), True)
        add("gemv", f"tcgen05, weights stored [N, K], batch {B}", gemv("tc", B, nk=True), True)

    # ------------------------------------------------------------------ layer glue and the layer
    def glue():
        from symm_mem_recipes_b200._ext import C
        x, r = randn(64, 1024, std=0.7, seed=1), randn(64, 1024, std=0.3, seed=2)
        w = (1.0 + randn(1024, std=0.1, seed=3).float()).to(torch.bfloat16)
        ref, ref_sum = C.oracle_rms_norm_bf16(x.cpu(), r.cpu(), w.cpu(), 1e-5)
        out, s = ops.rms_norm(x, w, 1e-5, residual=r)
        ok1 = torch.equal(s.cpu(), ref_sum) and _close(out.cpu(), ref, 2.0 ** -7, 1e-6)[0]
        qkv = randn(96, 6 * 64, std=1.0, seed=4)
        ref_q = C.oracle_rope_bf16(qkv.cpu(), 5, 64, 24, 0, 500000.0)
        ok2 = _close(ops.rope_(qkv.clone(), 5, 64, 24, 500000.0).cpu(), ref_q, 2.0 ** -7, 4e-3)[0]
        gu = randn(50, 2 * 48, std=3.0, seed=5)
        ok3 = _close(ops.silu_mul(gu).cpu(), C.oracle_silu_mul_bf16(gu.cpu()), 2.0 ** -7, 1e-6)[0]
        kc, vc = randn(2, 300, 1, 128, std=0.7, seed=6), randn(2, 300, 1, 128, std=0.7, seed=7)
        step = randn(2, (8 + 2) * 128, std=0.7, seed=8)
        kc_cpu, vc_cpu = kc.cpu(), vc.cpu()
        ref_a = C.oracle_decode_attention_bf16(step.cpu(), kc_cpu, vc_cpu, 8, 1, 257)
        got_a = ops.decode_attention_(step, kc, vc, 8, 257)
        ok4 = _close(got_a.cpu(), ref_a, 2.0 ** -6, 4e-3)[0] and torch.equal(kc.cpu(), kc_cpu)
        symm_mem.check_status(dev)
        return ok1 and ok2 and ok3 and ok4, f"rms_norm {ok1}, rope {ok2}, silu_mul {ok3}, decode_attention {ok4}"

    add("glue", "rms_norm / rope / silu_mul / decode_attention", glue, True)

    def layer(kind, fused_glue=False, fused_swiglu=False):
        def fn():
            cfg = LlamaTPConfig.tiny(world)
            lay = LlamaTPDecoderLayer(cfg, dev, seed=11, fused_glue=fused_glue, fused_swiglu=fused_swiglu)
            batch, seq = 2, 64 * world
            x = randn(batch * seq, cfg.hidden, std=0.5, seed=9)
            r = batch * seq // world
            if kind == "sp":
                got = lay.forward(x[rank * r:(rank + 1) * r].contiguous(), batch, seq)
                ref = lay.forward_reference(x[rank * r:(rank + 1) * r].contiguous(), batch, seq)
            elif kind == "tp":
                got, ref = lay.forward_tp(x, batch, seq), lay.forward_tp_reference(x, batch, seq)
            else:
                xd = x[:4].contiguous()
                kc = torch.zeros(4, 8, lay.hkv, cfg.head_dim, dtype=torch.bfloat16, device=dev)
                vc, kc2, vc2 = torch.zeros_like(kc), torch.zeros_like(kc), torch.zeros_like(kc)
                got, ref = lay.decode(xd, kc, vc, 0, fused=True), lay.decode(xd, kc2, vc2, 0, fused=False)
            symm_mem.check_status(dev)
            ok, err = _close(got, ref, 5e-2, 5e-2)
            return ok, f"max diff from the library composition {err:.4f}"
        return fn

    add("layer", "prefill, sequence parallel", layer("sp"))
    add("layer", "decode", layer("decode"))
    add("layer", "prefill, single-pass glue kernels", layer("sp", True), True)
    add("layer", "prefill, glue kernels + SwiGLU epilogue", layer("sp", True, True), True)
    add("layer", "prefill, no sequence parallelism", layer("tp"), True)
    add("layer", "decode, single-pass glue kernels", layer("decode", True), True)

    def decode_graph():
        from symm_mem_recipes_b200.models.llama_tp_layer import DecodeGraph
        cfg = LlamaTPConfig.tiny(world)
        lay = LlamaTPDecoderLayer(cfg, dev, seed=11)
        graph = DecodeGraph([lay], batch=4, max_seq=8)
        kc = torch.zeros(4, 8, lay.hkv, cfg.head_dim, dtype=torch.bfloat16, device=dev)
        vc = torch.zeros_like(kc)
        all_ok, worst = True, 0.0
        for pos in range(3):
            xd = randn(4, cfg.hidden, std=0.5, seed=20 + pos)
            got = graph.step(xd, pos).clone()
            ref = lay.decode(xd, kc, vc, pos, fused=True)
            ok, err = _close(got, ref, 5e-2, 5e-2)
            all_ok, worst = all_ok and ok, max(worst, err)
        symm_mem.check_status(dev)
        return all_ok, f"three replayed positions, max diff from the eager step {worst:.4f}"

    if dev.type == "cuda":                          # CUDA graphs: nothing to capture on the CPU backend
        add("layer", "decode through one captured CUDA graph", decode_graph, True)
    # The default forms go first; the variants follow, the rank-local kernels before the ones that
    # talk to peers (a fault in one of them would end the process and take the checks after it along).
    order = {"glue": 0, "all_gather_matmul": 1, "gemv": 2, "barrier": 3, "all_reduce": 4,
             "matmul_reduce_scatter": 5, "matmul_all_reduce": 6, "layer": 7}
    return sorted(checks, key=lambda c: (c[2], order.get(c[0], 8) if c[2] else 0))


def run_checks(checks: list, rank: int, dev: torch.device, only=()) -> tuple:
    """Runs the checks in order; returns (results, recoveries, stopped_early).  Collective: every
    rank runs the same list and learns every rank's outcome after each check."""
    from symm_mem_recipes_b200.errors import SymmMemTimeout
    from symm_mem_recipes_b200.parallel import symm_mem
    from symm_mem_recipes_b200.utils.benchmark import max_over_ranks

    results, stop, recoveries = [], False, 0
    for group, name, variant, fn in checks:
        if only and group not in only:
            continue
        t0 = time.monotonic()
        timed_out = False
        try:
            ok, detail = fn()
        except SymmMemTimeout as e:
            ok, detail, timed_out = False, f"device-side timeout: {e}", True
        except Exception as e:  # noqa: BLE001 - reported, the run goes on
            ok, detail = False, f"{type(e).__name__}: {e}"
            if rank == 0:
                traceback.print_exc()
        # every rank learns the outcome of every rank
        bad = max_over_ranks(0.0 if ok else 1.0, dev) != 0.0
        stop = max_over_ranks(1.0 if timed_out else 0.0, dev) != 0.0
        results.append({"group": group, "check": name, "variant": variant, "ok": not bad,
                        "detail": detail if not ok or detail else "", "seconds": round(time.monotonic() - t0, 2)})
        if rank == 0:
            print(f"[{'ok' if not bad else 'FAILED'}] {group}: {name}  {results[-1]['detail']}", flush=True)
        if stop:
            # A bounded wait ran out somewhere: counters and barrier slots of the allocations in use are no longer
            # trustworthy.  The kernels have returned, so the ranks drop ALL symmetric memory together and the
            # next check starts from fresh allocations.
            recoveries += 1
            if recoveries > _MAX_RECOVERIES:
                if rank == 0:
                    print("stopping: too many device-side timeouts", flush=True)
                break
            for shared in _SHARED_STATE:
                shared.clear()
            if dev.type == "cuda":
                try:                                   # a timeout recorded on this rank but not yet read
                    symm_mem.check_status(dev)
                except SymmMemTimeout:
                    pass
            symm_mem.reset()
            stop = False
            if rank == 0:
                print("a bounded wait ran out: symmetric memory dropped and re-created for the next check", flush=True)
    return results, recoveries, recoveries > _MAX_RECOVERIES


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--only", default="", help="comma-separated groups (all_reduce, barrier, all_gather_matmul, "
                                               "matmul_reduce_scatter, matmul_all_reduce, gemv, glue, layer)")
    ap.add_argument("--list", action="store_true", help="print the checks and exit (no GPU needed)")
    args = ap.parse_args(argv)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    only = {g for g in args.only.split(",") if g}
    if args.list:
        for group, name, variant, _ in build_checks(max(world, 2), 0, torch.device("cpu")):
            if not only or group in only:
                print(f"{group:24s} {name}{'   [variant]' if variant else ''}")
        return 0

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    from symm_mem_recipes_b200.parallel import symm_mem

    results, recoveries, stopped = run_checks(build_checks(world, rank, dev), rank, dev, only)
    failed = [r for r in results if not r["ok"]]
    if rank == 0:
        print(json.dumps({"op": "selfcheck", "world_size": world, "checks": len(results), "failed": len(failed),
                          "stopped_early": stopped, "recoveries": recoveries,
                          "failures": [f"{r['group']}: {r['check']}" for r in failed]}))
    symm_mem.shutdown()
    if world > 1:
        dist.destroy_process_group()
    return len(failed)


if __name__ == "__main__":
    sys.exit(main())
