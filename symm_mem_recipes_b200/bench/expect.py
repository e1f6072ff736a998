"""What the roofline allows for an op, before it is measured.

    python -m symm_mem_recipes_b200.bench.expect all_gather_matmul --M 16384 --N 3584 --K 8192 --ws 8 \
        --peaks MEASURED_PEAKS.json
    python -m symm_mem_recipes_b200.bench.expect all_reduce --bytes 67108864 --ws 8
    python -m symm_mem_recipes_b200.bench.expect gemv_all_reduce --batch 4 --K 3584 --N 8192 --ws 8
    python -m symm_mem_recipes_b200.bench.expect matmul_reduce_scatter --M 32768 --N 8192 --K 1024 --ws 8
    python -m symm_mem_recipes_b200.bench.expect layer_prefill --batch 16 --seq 2048 --ws 8     # Llama-3-70B layer
    python -m symm_mem_recipes_b200.bench.expect layer_decode --batch 1 --ws 8

Prints one JSON object: the time each resource needs on its own (tensor cores
at the measured cuBLAS rate, HBM at the measured copy rate, NVLink at the
measured peer-copy rate per direction and GPU) and the largest of them, which
is the target a fused kernel is held against.  Peaks default to figures measured
on B200 (1647 TFLOPS bf16 burst, 6541 GB/s copy, 770 GB/s NVLink per direction);
`--peaks FILE` overrides the first two.  No GPU needed.  No upstream counterpart.
"""
from __future__ import annotations

import argparse
import json
import sys

DEFAULT_PEAKS = {"bf16_tflops": 1647.3, "hbm_gbs": 6541.5}
NVLINK_GBS = 770.0          # measured peer copy, per direction per GPU (nominal 900)


def _us(amount: float, rate_per_s: float) -> float:
    return amount / rate_per_s * 1e6


def expect(op: str, ws: int, peaks: dict, M: int = 0, N: int = 0, K: int = 0, batch: int = 0,
           nbytes: int = 0, nvls: bool = True) -> dict:
    """Time each resource needs for one call of `op` at world size `ws` (tensor
    cores, HBM, NVLink in and out, at the given peaks), the largest of them as
    `target_us`, and which one it is (`bound_by`)."""
    tflops, hbm = peaks["bf16_tflops"] * 1e12, peaks["hbm_gbs"] * 1e9
    link = NVLINK_GBS * 1e9
    parts: dict[str, float] = {}
    if op == "all_gather_matmul":            # M = gathered rows; every rank multiplies all of them
        parts["tensor_us"] = _us(2.0 * M * N * K, tflops)
        parts["hbm_us"] = _us((M * K + N * K + M * N) * 2.0, hbm)
        parts["nvlink_in_us"] = _us((ws - 1) / ws * M * K * 2.0, link)      # the remote shards arrive once
    elif op == "matmul_reduce_scatter":      # K = this rank's slice of the reduction dimension
        parts["tensor_us"] = _us(2.0 * M * N * K, tflops)
        # operands once; the bf16 partials land in the inboxes and are read back by the reduction
        parts["hbm_us"] = _us((M * K + N * K) * 2.0 + 2.0 * (M * N * 2.0), hbm)
        parts["nvlink_out_us"] = _us((ws - 1) / ws * M * N * 2.0, link)     # bf16 partials to their owners
    elif op == "gemv_all_reduce":            # W [K, N] per rank is streamed once
        parts["hbm_us"] = _us(K * N * 2.0, hbm)
        parts["nvlink_in_us"] = _us((ws - 1) * batch * N * 4.0, link)       # fp32 partials from every peer
    elif op == "all_reduce":
        # in-switch reduction: each rank sends its buffer once and receives the sum once;
        # peer-to-peer two-shot: (ws-1)/ws of it out for the reduce-scatter and again for the all-gather
        factor = 1.0 if nvls else 2.0 * (ws - 1) / ws
        parts["nvlink_us"] = _us(factor * nbytes, link)
        parts["hbm_us"] = _us(2.0 * nbytes, hbm)
    else:
        raise ValueError(f"unknown op {op!r}")
    bound = max(parts, key=parts.get)
    return {"op": op, "world_size": ws, **{k: round(v, 1) for k, v in parts.items()},
            "bound_by": bound.rsplit("_us", 1)[0], "target_us": round(parts[bound], 1)}


def expect_layer(ws: int, peaks: dict, batch: int = 16, seq: int = 2048, hidden: int = 8192, n_heads: int = 64,
                 n_kv_heads: int = 8, head_dim: int = 128, ffn: int = 28672, decode: bool = False) -> dict:
    """The same for a whole decoder layer under TP (`models/llama_tp_layer.py`): the sum of the targets
    of its phases.  Prefill (sequence parallel): QKV and gate/up as all_gather_matmul, o- and
    down-projection as matmul_reduce_scatter, causal attention on the rank's heads at the tensor
    rate, and the rank-local glue (norms, RoPE, SiLU-mul) as single passes at the copy rate.
    Decode (`batch` <= 16 tokens): every weight streamed once from HBM, the two row-parallel
    projections as gemv_all_reduce; attention and glue are negligible."""
    T = batch * seq
    hq, hkv = n_heads // ws, n_kv_heads // ws
    qkv_n, ffn_local = (hq + 2 * hkv) * head_dim, ffn // ws
    tflops, hbm = peaks["bf16_tflops"] * 1e12, peaks["hbm_gbs"] * 1e9
    phases: dict[str, dict] = {}
    if decode:
        for name, rows in (("qkv", qkv_n), ("gate_up", 2 * ffn_local)):
            phases[name] = {"target_us": round(_us(rows * hidden * 2.0, hbm), 1), "bound_by": "hbm"}
        phases["o_proj"] = expect("gemv_all_reduce", ws, peaks, K=hq * head_dim, N=hidden, batch=batch)
        phases["down_proj"] = expect("gemv_all_reduce", ws, peaks, K=ffn_local, N=hidden, batch=batch)
    else:
        phases["qkv"] = expect("all_gather_matmul", ws, peaks, M=T, N=qkv_n, K=hidden)
        attn_flops = 4.0 * batch * hq * seq * seq * head_dim / 2.0          # QK^T and PV, causal half
        phases["attention"] = {"target_us": round(_us(attn_flops, tflops), 1), "bound_by": "tensor"}
        phases["o_proj"] = expect("matmul_reduce_scatter", ws, peaks, M=T, N=hidden, K=hq * head_dim)
        phases["gate_up"] = expect("all_gather_matmul", ws, peaks, M=T, N=2 * ffn_local, K=hidden)
        phases["down_proj"] = expect("matmul_reduce_scatter", ws, peaks, M=T, N=hidden, K=ffn_local)
        # per rank: two norms over its T / ws rows (read x (+ residual), write the sum and the normed row),
        # RoPE in place on Q and K of all T tokens, SiLU-mul reading 2 F and writing F per token
        rows = T / ws
        glue_bytes = (2 * rows * hidden + 4 * rows * hidden + 2 * T * (hq + hkv) * head_dim + 3 * T * ffn_local) * 2.0
        phases["glue"] = {"target_us": round(_us(glue_bytes, hbm), 1), "bound_by": "hbm"}
    total = round(sum(p["target_us"] for p in phases.values()), 1)
    return {"op": "llama_layer_decode" if decode else "llama_layer_prefill", "world_size": ws, "batch": batch,
            **({} if decode else {"seq": seq}), "target_us": total,
            "phases": {k: {"target_us": v["target_us"], "bound_by": v["bound_by"]} for k, v in phases.items()}}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("op", choices=["all_gather_matmul", "matmul_reduce_scatter", "gemv_all_reduce", "all_reduce",
                                   "layer_prefill", "layer_decode"])
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--ws", type=int, default=8)
    ap.add_argument("--M", type=int, default=0)
    ap.add_argument("--N", type=int, default=0)
    ap.add_argument("--K", type=int, default=0)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--bytes", type=int, default=0, dest="nbytes")
    ap.add_argument("--no-nvls", action="store_true", help="all_reduce: peer-to-peer two-shot instead of in-switch")
    ap.add_argument("--peaks", default=None)
    args = ap.parse_args(argv)
    peaks = dict(DEFAULT_PEAKS)
    if args.peaks:
        with open(args.peaks) as f:
            peaks.update({k: v for k, v in json.load(f).items() if k in DEFAULT_PEAKS})
    if args.op.startswith("layer_"):
        print(json.dumps(expect_layer(args.ws, peaks, batch=args.batch, seq=args.seq,
                                      decode=args.op == "layer_decode")))
        return 0
    print(json.dumps(expect(args.op, args.ws, peaks, args.M, args.N, args.K, args.batch, args.nbytes,
                            not args.no_nvls)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
