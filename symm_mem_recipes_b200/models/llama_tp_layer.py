"""A Llama-style decoder layer under tensor + sequence parallelism, built from
this package's fused kernels.

Prefill (`forward`), activations sharded on tokens between the blocks:

    x_shard [T/WS, H]
      -> RMSNorm -> all_gather_matmul with W_qkv            (gather fused into the GEMM)
      -> RoPE, causal GQA attention on the rank's heads     (rank-local)
      -> matmul_reduce_scatter with W_o                     (reduce fused into the GEMM)
      -> + residual -> RMSNorm -> all_gather_matmul with W_gate|W_up
      -> SiLU(gate) * up -> matmul_reduce_scatter with W_down -> + residual

Decode (`decode`), activations replicated, batch <= 16: the two row-parallel
projections use the fused GEMV + all-reduce.  It continues from KV caches that
the prefill fills when given `kv_cache=(k_cache, v_cache)`.  `decode_static` is the same step
with shapes and launches independent of the position, and `DecodeGraph`
captures it (through any number of layers) in one CUDA graph that is replayed
per token.

Prefill without sequence parallelism (`forward_tp`), activations replicated:
local GEMMs for the column-parallel projections, `matmul_all_reduce` for the
row-parallel ones.

`forward_reference` / `forward_tp_reference` / `decode(fused=False)` build the same layer from NCCL
collectives and cuBLAS and are the baseline the fused layer is timed against.
The upstream recipes stop at the single fused op; this module is how the ops
compose in the workload they were written for (Llama-3-70B at TP8: hidden
8192, 64 query / 8 KV heads of 128, FFN 28672).  Attention is PyTorch's
scaled_dot_product_attention (rank-local).  Norms, RoPE and the activation are
the single-pass kernels of `ops.layer_glue` (`fused_glue`, on by default;
SMR_FUSED_GLUE=0 or `fused_glue=False` falls back to PyTorch compositions):
RMSNorm writes straight into the symmetric buffer the next all_gather_matmul
reads (and folds in the residual add before it), RoPE rotates Q and K in place
inside the QKV buffer, SiLU(gate) * up is one pass; in a decode step the
column-parallel projections run on the package's tcgen05 GEMV and the
attention of the new token is one kernel.  `fused_swiglu=True` (SMR_FUSED_SWIGLU=1) goes one
step further for prefill: the gate and up weights are interleaved so that the
activation is applied to the accumulators inside the all_gather_matmul epilogue.
"""
from __future__ import annotations

import contextlib
import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F

from .. import ops
from ..parallel import symm_mem


@dataclass
class LlamaTPConfig:
    """Shape of the un-sharded layer; the defaults are Llama-3-70B.  Heads, KV
    heads and the FFN width must divide by the world size."""
    hidden: int = 8192
    n_heads: int = 64
    n_kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 28672
    rope_theta: float = 500000.0
    eps: float = 1e-5

    @staticmethod
    def llama3_70b() -> "LlamaTPConfig":
        return LlamaTPConfig()

    @staticmethod
    def tiny(world_size: int) -> "LlamaTPConfig":
        """Same structure at a size a unit test can check against fp32."""
        return LlamaTPConfig(hidden=512, n_heads=4 * world_size, n_kv_heads=world_size, head_dim=64,
                             ffn=512 * world_size)


def _sdpa_backends():
    """Context for the prefill attention call.  Attention is rank-local library code
    (`scaled_dot_product_attention`); with SMR_SDPA_CUDNN=1 PyTorch is asked to try its cuDNN
    backend first and fall back to its usual order.  Off by default."""
    if os.environ.get("SMR_SDPA_CUDNN", "0") != "1":
        return contextlib.nullcontext()
    from torch.nn.attention import SDPBackend, sdpa_kernel
    return sdpa_kernel([SDPBackend.CUDNN_ATTENTION, SDPBackend.FLASH_ATTENTION, SDPBackend.EFFICIENT_ATTENTION,
                        SDPBackend.MATH], set_priority=True)


def _rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


def _rope(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """x [B, S, heads, D]; rotate pairs (i, i + D/2), Llama convention."""
    d = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, device=x.device, dtype=torch.float32) / d))
    ang = positions.float()[..., None] * inv                      # [B, S, D/2]
    cos, sin = ang.cos()[:, :, None, :], ang.sin()[:, :, None, :]
    x1, x2 = x.float()[..., : d // 2], x.float()[..., d // 2:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype)


class LlamaTPDecoderLayer:
    """Weights of one rank (random-init from `seed + rank`) and the fused /
    reference forward passes.  Plain object, inference only."""

    def __init__(self, cfg: LlamaTPConfig, device: torch.device, group=None, seed: int = 0,
                 dtype: torch.dtype = torch.bfloat16, fused_glue: Optional[bool] = None,
                 fused_swiglu: Optional[bool] = None, shared_row_weights: Optional[bool] = None):
        self.cfg, self.device, self.group = cfg, device, group
        self.fused_glue = (os.environ.get("SMR_FUSED_GLUE", "1") == "1") if fused_glue is None else bool(fused_glue)
        # SiLU(gate) * up inside the epilogue of the gate/up all_gather_matmul (prefill only)
        self.fused_swiglu = ((os.environ.get("SMR_FUSED_SWIGLU", "0") == "1") if fused_swiglu is None
                             else bool(fused_swiglu))
        self.ws = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        ws = self.ws
        assert cfg.n_heads % ws == 0 and cfg.n_kv_heads % ws == 0 and cfg.ffn % ws == 0
        self.hq, self.hkv = cfg.n_heads // ws, cfg.n_kv_heads // ws
        self.ffn_local = cfg.ffn // ws
        H, D = cfg.hidden, cfg.head_dim
        g = torch.Generator(device="cpu").manual_seed(seed + self.rank)

        def w(*shape, std=0.02):
            return (torch.randn(*shape, generator=g) * std).to(dtype).to(device)

        # column-parallel weights are [N_local, K = H]; row-parallel ones [N = H, K_local]
        self.w_qkv = w((self.hq + 2 * self.hkv) * D, H)
        self.w_o = w(H, self.hq * D)
        self.w_gate_up = w(2 * self.ffn_local, H)
        self.w_down = w(H, self.ffn_local)
        # The decode GEMV streams [K_local, N] weights by default, which costs a transposed copy of the
        # two row-parallel weights; `shared_row_weights` (SMR_GEMV_WEIGHTS_NK=1) lets it read the [N, K_local]
        # layout of the prefill GEMMs instead: one copy serves both.
        self.shared_row_weights = ((os.environ.get("SMR_GEMV_WEIGHTS_NK", "0") == "1") if shared_row_weights is None
                                   else bool(shared_row_weights))
        self.w_o_t = None if self.shared_row_weights else self.w_o.t().contiguous()
        self.w_down_t = None if self.shared_row_weights else self.w_down.t().contiguous()
        self.w_gate_up_interleaved = None
        if self.fused_swiglu:
            if self.ffn_local % 128:
                raise ValueError("fused_swiglu needs the FFN width per rank to be a multiple of 128")
            self.w_gate_up_interleaved = ops.interleave_gate_up(self.w_gate_up[: self.ffn_local],
                                                                self.w_gate_up[self.ffn_local:])
        gn = torch.Generator(device="cpu").manual_seed(seed + 7919)   # norms are replicated
        self.norm1 = (1.0 + 0.1 * torch.randn(H, generator=gn)).to(dtype).to(device)
        self.norm2 = (1.0 + 0.1 * torch.randn(H, generator=gn)).to(dtype).to(device)
        self._sym: dict[tuple, torch.Tensor] = {}
        self._sym_generation = symm_mem.generation()
        # set to a list to get (phase name, CUDA event) pairs appended by `forward` (see `phase_times_us`)
        self.phase_marks: Optional[list] = None

    def _mark(self, name: str) -> None:
        if self.phase_marks is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.phase_marks.append((name, ev))

    def phase_times_us(self, x_shard: torch.Tensor, batch: int, seq: int, iters: int = 5) -> dict:
        """Device time of every phase of `forward` (CUDA events between the
        phases, mean over `iters` calls after one warm-up), in µs."""
        self.forward(x_shard, batch, seq)
        totals: dict[str, float] = {}
        for _ in range(iters):
            self.phase_marks = []
            self.forward(x_shard, batch, seq)
            marks, self.phase_marks = self.phase_marks, None
            torch.cuda.synchronize(self.device)
            for (_, e0), (name, e1) in zip(marks[:-1], marks[1:]):
                totals[name] = totals.get(name, 0.0) + e0.elapsed_time(e1) * 1e3 / iters
        return totals

    # ---- symmetric staging for the gather inputs ----
    def _symmetric(self, tag: str, rows: int) -> torch.Tensor:
        if self._sym_generation != symm_mem.generation():       # symm_mem.reset() ran: the cached buffers are gone
            self._sym.clear()
            self._sym_generation = symm_mem.generation()
        key = (tag, rows)
        t = self._sym.get(key)
        if t is None:
            t = symm_mem.empty(rows, self.cfg.hidden, dtype=torch.bfloat16, device=self.device)
            symm_mem.rendezvous(t, self.group)
            self._sym[key] = t
        return t

    # ---- rank-local attention on [T, (hq + 2 hkv) * D] ----
    def _attention(self, qkv: torch.Tensor, batch: int, seq: int, glue: bool = False, kv_cache=None) -> torch.Tensor:
        """Causal attention of this rank's heads over `batch` sequences of `seq` tokens.  With
        `kv_cache = (k_cache, v_cache)` ([batch, S_max, hkv, D] each) the keys (rotated) and values of
        positions [0, seq) are also written there, which is what `decode` continues from."""
        D, hq, hkv = self.cfg.head_dim, self.hq, self.hkv
        if glue:
            ops.rope_(qkv, hq + hkv, D, seq, self.cfg.rope_theta)      # Q and K heads, in place
        q, k, v = qkv.split([hq * D, hkv * D, hkv * D], dim=-1)
        q = q.view(batch, seq, hq, D)
        k = k.view(batch, seq, hkv, D)
        v = v.view(batch, seq, hkv, D)
        if not glue:
            pos = torch.arange(seq, device=qkv.device)[None, :].expand(batch, seq)
            q, k = _rope(q, pos, self.cfg.rope_theta), _rope(k, pos, self.cfg.rope_theta)
        if kv_cache is not None:
            k_cache, v_cache = kv_cache
            if k_cache.shape[0] != batch or k_cache.shape[1] < seq or v_cache.shape != k_cache.shape:
                raise ValueError("kv_cache: two [batch, S_max >= seq, kv heads per rank, head_dim] tensors")
            k_cache[:, :seq].copy_(k)
            v_cache[:, :seq].copy_(v)
        with _sdpa_backends():
            o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                               is_causal=True, enable_gqa=True)
        return o.transpose(1, 2).reshape(batch * seq, hq * D).contiguous()

    @staticmethod
    def _mlp_act_torch(gu: torch.Tensor, ffn_local: int) -> torch.Tensor:
        gate, up = gu.split(ffn_local, dim=-1)
        return (F.silu(gate.float()) * up.float()).to(gu.dtype).contiguous()

    def _mlp_act(self, gu: torch.Tensor) -> torch.Tensor:
        return ops.silu_mul(gu) if self.fused_glue else self._mlp_act_torch(gu, self.ffn_local)

    # ------------------------------------------------------------------
    def forward(self, x_shard: torch.Tensor, batch: int, seq: int, barrier_between_phases: bool = False,
                kv_cache=None) -> torch.Tensor:
        """x_shard [batch*seq/WS, H] (this rank's tokens) -> same shape.  `kv_cache = (k_cache,
        v_cache)` receives this rank's keys and values of the prompt, for `decode` to continue from."""
        cfg = self.cfg
        rows = x_shard.shape[0]
        assert rows * self.ws == batch * seq
        h = self._symmetric("attn_in", rows)
        self._mark("start")
        if self.fused_glue:
            ops.rms_norm(x_shard, self.norm1, cfg.eps, out=h)
        else:
            h.copy_(_rms_norm(x_shard, self.norm1, cfg.eps))
        self._mark("norm1")
        qkv = ops.all_gather_matmul(h, self.w_qkv, group=self.group)
        self._mark("qkv_all_gather_matmul")
        attn = self._attention(qkv, batch, seq, glue=self.fused_glue, kv_cache=kv_cache)
        self._mark("rope_attention")
        if barrier_between_phases:
            symm_mem.rendezvous(h, self.group).barrier(channel=1)
        h2 = self._symmetric("mlp_in", rows)
        o = ops.matmul_reduce_scatter(attn, self.w_o, group=self.group)
        self._mark("o_proj_reduce_scatter")
        if self.fused_glue:
            _, x1 = ops.rms_norm(x_shard, self.norm2, cfg.eps, out=h2, residual=o)    # x1 = x_shard + o
        else:
            x1 = x_shard + o
            h2.copy_(_rms_norm(x1, self.norm2, cfg.eps))
        self._mark("residual_norm2")
        if self.fused_swiglu:
            act = ops.all_gather_matmul(h2, self.w_gate_up_interleaved, group=self.group, epilogue="swiglu")
            self._mark("gate_up_all_gather_matmul")
        else:
            gu = ops.all_gather_matmul(h2, self.w_gate_up, group=self.group)
            self._mark("gate_up_all_gather_matmul")
            act = self._mlp_act(gu)
        self._mark("silu_mul")
        if barrier_between_phases:
            symm_mem.rendezvous(h2, self.group).barrier(channel=2)
        d = ops.matmul_reduce_scatter(act, self.w_down, group=self.group)
        self._mark("down_proj_reduce_scatter")
        y = x1 + d
        self._mark("residual")
        return y

    # ------------------------------------------------------------------
    def forward_tp(self, x: torch.Tensor, batch: int, seq: int, kv_cache=None) -> torch.Tensor:
        """Prefill under plain tensor parallelism (no sequence parallelism):
        `x` [batch*seq, H] is replicated on every rank, the column-parallel
        projections are local tcgen05 GEMMs, and the two row-parallel ones end
        in an all-reduce inside the kernel (`matmul_all_reduce`).  Returns the
        full [batch*seq, H] output, identical on every rank."""
        cfg = self.cfg
        assert x.shape[0] == batch * seq
        h = ops.rms_norm(x, self.norm1, cfg.eps) if self.fused_glue else _rms_norm(x, self.norm1, cfg.eps)
        qkv = ops.matmul(h, self.w_qkv)
        attn = self._attention(qkv, batch, seq, glue=self.fused_glue, kv_cache=kv_cache)
        o = ops.matmul_all_reduce(attn, self.w_o, group=self.group)      # internal symmetric buffer: consume it
        if self.fused_glue:                                              # before the next call of this shape
            h2, x1 = ops.rms_norm(x, self.norm2, cfg.eps, residual=o)
        else:
            x1 = x + o
            h2 = _rms_norm(x1, self.norm2, cfg.eps)
        if self.fused_swiglu:
            act = ops.matmul(h2, self.w_gate_up_interleaved, epilogue="swiglu")
        else:
            act = self._mlp_act(ops.matmul(h2, self.w_gate_up))
        return x1 + ops.matmul_all_reduce(act, self.w_down, group=self.group)

    def forward_tp_reference(self, x: torch.Tensor, batch: int, seq: int) -> torch.Tensor:
        """`forward_tp` from cuBLAS and NCCL all-reduce."""
        cfg = self.cfg

        def reduced(t):
            if self.ws > 1:
                dist.all_reduce(t, group=self.group)
            return t

        h = _rms_norm(x, self.norm1, cfg.eps)
        attn = self._attention(h @ self.w_qkv.t(), batch, seq)
        x1 = x + reduced(attn @ self.w_o.t())
        h2 = _rms_norm(x1, self.norm2, cfg.eps)
        act = self._mlp_act_torch(h2 @ self.w_gate_up.t(), self.ffn_local)
        return x1 + reduced(act @ self.w_down.t())

    def forward_reference(self, x_shard: torch.Tensor, batch: int, seq: int) -> torch.Tensor:
        """The same layer from NCCL all-gather / reduce-scatter and cuBLAS."""
        cfg = self.cfg

        def gather(t):
            if self.ws == 1:
                return t
            out = torch.empty(t.shape[0] * self.ws, t.shape[1], dtype=t.dtype, device=t.device)
            dist.all_gather_into_tensor(out, t.contiguous(), group=self.group)
            return out

        def scatter(t):
            if self.ws == 1:
                return t
            out = torch.empty(t.shape[0] // self.ws, t.shape[1], dtype=t.dtype, device=t.device)
            dist.reduce_scatter_tensor(out, t.contiguous(), group=self.group)
            return out

        h = gather(_rms_norm(x_shard, self.norm1, cfg.eps))
        attn = self._attention(h @ self.w_qkv.t(), batch, seq)
        x1 = x_shard + scatter(attn @ self.w_o.t())
        h2 = gather(_rms_norm(x1, self.norm2, cfg.eps))
        act = self._mlp_act_torch(h2 @ self.w_gate_up.t(), self.ffn_local)
        return x1 + scatter(act @ self.w_down.t())

    # ------------------------------------------------------------------
    def _row_parallel_decode(self, act: torch.Tensor, which: str, fused: bool) -> torch.Tensor:
        """act [B, K_local] times this rank's rows of the o- or down-projection, summed over the ranks."""
        nk = self.shared_row_weights
        w = {"o": self.w_o if nk else self.w_o_t, "down": self.w_down if nk else self.w_down_t}[which]
        if fused and self.ws > 1:
            return ops.gemv_all_reduce(act, w, group=self.group, weights_nk=nk)
        return ops.reference_gemv_all_reduce(act, w, group=self.group, weights_nk=nk)

    def _column_parallel_decode(self, h: torch.Tensor, w_nk: torch.Tensor, fused: bool) -> torch.Tensor:
        """h [B, H] times this rank's rows of a column-parallel weight ([N_local, H]); nothing to reduce.
        On the package's tcgen05 GEMV (the weight streamed once by TMA) when `fused`, else cuBLAS."""
        if fused and h.is_cuda and h.shape[0] <= 16:
            return ops.gemv(h, w_nk, weights_nk=True)
        return h @ w_nk.t()

    def _decode_norm(self, t: torch.Tensor, w: torch.Tensor, glue: bool) -> torch.Tensor:
        return ops.rms_norm(t, w, self.cfg.eps) if glue else _rms_norm(t, w, self.cfg.eps)

    def _decode_mlp(self, x: torch.Tensor, o_proj: torch.Tensor, fused: bool, glue: bool,
                    defer_residual: bool = False):
        """Second half of a decode step: residual add of the attention output, norm, MLP, residual add.
        `defer_residual`: return `(down, x1)` and leave `x1 + down` to the next layer's first kernel."""
        if glue:
            h2, x1 = ops.rms_norm(o_proj, self.norm2, self.cfg.eps, residual=x)    # x1 = x + o_proj, one kernel
        else:
            x1 = x + o_proj
            h2 = _rms_norm(x1, self.norm2, self.cfg.eps)
        gu = self._column_parallel_decode(h2, self.w_gate_up, glue)
        act = ops.silu_mul(gu) if glue else LlamaTPDecoderLayer._mlp_act_torch(gu, self.ffn_local)
        down = self._row_parallel_decode(act, "down", fused)
        return (down, x1) if defer_residual else x1 + down

    def decode(self, x: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, pos: int,
               fused: bool = True) -> torch.Tensor:
        """One decode step.  x [B, H] replicated on all ranks; caches
        [B, S_max, hkv, D] hold this rank's KV heads and are updated at `pos`."""
        cfg = self.cfg
        B, D, hq, hkv = x.shape[0], cfg.head_dim, self.hq, self.hkv
        glue = fused and self.fused_glue
        qkv = self._column_parallel_decode(self._decode_norm(x, self.norm1, glue), self.w_qkv, glue)
        if glue:
            # ONE kernel rotates the new Q and K, writes the caches and attends over positions 0..pos
            attn = ops.decode_attention_(qkv, k_cache, v_cache, hq, pos, rope_theta=cfg.rope_theta)
            return self._decode_mlp(x, self._row_parallel_decode(attn, "o", fused), fused, glue)
        q, k, v = qkv.split([hq * D, hkv * D, hkv * D], dim=-1)
        q, k = q.view(B, 1, hq, D), k.view(B, 1, hkv, D)
        if not glue:
            p = torch.full((B, 1), pos, device=x.device)
            q, k = _rope(q, p, cfg.rope_theta), _rope(k, p, cfg.rope_theta)
        k_cache[:, pos] = k[:, 0]
        v_cache[:, pos] = v.view(B, hkv, D)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k_cache[:, : pos + 1].transpose(1, 2),
                                           v_cache[:, : pos + 1].transpose(1, 2), enable_gqa=True)
        o_proj = self._row_parallel_decode(o.transpose(1, 2).reshape(B, hq * D).contiguous(), "o", fused)
        return self._decode_mlp(x, o_proj, fused, glue)

    def chains_residual(self, fused: bool = True) -> bool:
        """Whether `decode_static` can take and hand on an unfinished residual add (glue kernels only)."""
        return bool(fused and self.fused_glue)

    def decode_static(self, x: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, pos: torch.Tensor,
                      fused: bool = True, pending_residual: Optional[torch.Tensor] = None,
                      defer_residual: bool = False):
        """`decode` with every shape and every launch independent of the
        position, so that ONE captured CUDA graph serves all positions: `pos`
        is an int32 tensor of one element on the device, the caches are written
        with `index_copy_`, and attention runs over the whole cache under a
        mask that hides the entries beyond `pos`.  Same result as `decode`.

        Between stacked layers the closing residual add of one layer can ride
        in the first RMSNorm kernel of the next (`chains_residual`): with
        `defer_residual` the layer returns `(down, x1)` instead of `x1 + down`,
        and the next layer takes them as `x=down, pending_residual=x1`."""
        cfg = self.cfg
        B, D, hq, hkv = x.shape[0], cfg.head_dim, self.hq, self.hkv
        s_max = k_cache.shape[1]
        glue = fused and self.fused_glue
        if (pending_residual is not None or defer_residual) and not glue:
            raise ValueError("chaining the residual add needs the glue kernels (see chains_residual)")
        if pending_residual is not None:
            h1, x = ops.rms_norm(x, self.norm1, cfg.eps, residual=pending_residual)    # x = previous x1 + down
        else:
            h1 = self._decode_norm(x, self.norm1, glue)
        qkv = self._column_parallel_decode(h1, self.w_qkv, glue)
        if glue:
            attn = ops.decode_attention_(qkv, k_cache, v_cache, hq, pos, rope_theta=cfg.rope_theta)
            return self._decode_mlp(x, self._row_parallel_decode(attn, "o", fused), fused, glue, defer_residual)
        q, k, v = qkv.split([hq * D, hkv * D, hkv * D], dim=-1)
        q, k = q.view(B, 1, hq, D), k.view(B, 1, hkv, D)
        if not glue:
            p = pos.view(1, 1).expand(B, 1)
            q, k = _rope(q, p, cfg.rope_theta), _rope(k, p, cfg.rope_theta)
        idx = pos.view(1).long()
        k_cache.index_copy_(1, idx, k)
        v_cache.index_copy_(1, idx, v.reshape(B, 1, hkv, D))
        visible = (torch.arange(s_max, device=x.device, dtype=torch.int32) <= pos.view(1)).view(1, 1, 1, s_max)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k_cache.transpose(1, 2), v_cache.transpose(1, 2),
                                           attn_mask=visible, enable_gqa=True)
        o_proj = self._row_parallel_decode(o.transpose(1, 2).reshape(B, hq * D).contiguous(), "o", fused)
        return self._decode_mlp(x, o_proj, fused, glue)


def decode_static_through(layers, caches, x: torch.Tensor, pos: torch.Tensor, fused: bool = True) -> torch.Tensor:
    """One decode step through stacked layers; where two neighbours both run the glue kernels the
    residual add that closes the first rides in the RMSNorm kernel that opens the second."""
    layers = list(layers)
    h, pending = x, None
    for i, (lyr, (kc, vc)) in enumerate(zip(layers, caches)):
        defer = (i + 1 < len(layers) and lyr.chains_residual(fused) and layers[i + 1].chains_residual(fused))
        out = lyr.decode_static(h, kc, vc, pos, fused=fused, pending_residual=pending, defer_residual=defer)
        h, pending = out if defer else (out, None)
    return h


def new_kv_caches(layers, batch: int, max_seq: int) -> list:
    """One zeroed (k_cache, v_cache) pair per layer, [batch, max_seq, kv heads per rank, head_dim] each."""
    return [(torch.zeros(batch, max_seq, lyr.hkv, lyr.cfg.head_dim, dtype=torch.bfloat16, device=lyr.device),
             torch.zeros(batch, max_seq, lyr.hkv, lyr.cfg.head_dim, dtype=torch.bfloat16, device=lyr.device))
            for lyr in layers]


class DecodeGraph:
    """A decode step through a stack of layers captured once in a CUDA graph
    and replayed for every token: the launch-bound part of serving (a dozen
    kernels of a few microseconds per layer) costs one graph launch per step.

        g = DecodeGraph(layers, batch=4, max_seq=4096)
        for lyr, cache in zip(layers, g.caches):   # prompt: prefill straight into the graph's caches
            h = lyr.forward(h, batch, prompt_len, kv_cache=cache)
        for pos, x in enumerate(tokens, start=prompt_len):     # x [B, H], replicated on all ranks
            y = g.step(x, pos)                     # y is overwritten by the next step

    Every rank builds and replays the same graph (the fused GEMV + all-reduce
    kernels inside meet their peers as in eager mode).  The KV caches live in
    the object; `reset()` starts a new sequence.  The graph holds the addresses
    of the ops' symmetric workspaces: after `symm_mem.reset()` build a new one.
    No upstream counterpart: the upstream recipes time single kernels.
    """

    def __init__(self, layers, batch: int, max_seq: int, fused: bool = True, warmup: int = 2, caches=None):
        self.layers = list(layers)
        first = self.layers[0]
        dev, cfg = first.device, first.cfg
        self.max_seq = int(max_seq)
        self.fused = fused
        self.x = torch.zeros(batch, cfg.hidden, dtype=torch.bfloat16, device=dev)
        self.pos = torch.zeros(1, dtype=torch.int32, device=dev)
        # `caches`: one (k_cache, v_cache) pair per layer owned by the caller; zeroed here like the own ones
        self.caches = caches if caches is not None else new_kv_caches(self.layers, batch, max_seq)
        if len(self.caches) != len(self.layers) or any(kc.shape[:2] != (batch, max_seq) for kc, _ in self.caches):
            raise ValueError("caches: one ([batch, max_seq, kv heads per rank, head_dim] x 2) pair per layer")
        # first calls allocate workspaces and rendezvous: outside the capture, on a side stream
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup)):
                self._run()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.y = self._run()
        self.reset()

    def _run(self) -> torch.Tensor:
        return decode_static_through(self.layers, self.caches, self.x, self.pos, fused=self.fused)

    def reset(self) -> None:
        """Start a new sequence: the KV caches are zeroed (the graph is kept)."""
        for kc, vc in self.caches:
            kc.zero_()
            vc.zero_()

    def step(self, x: torch.Tensor, pos: int) -> torch.Tensor:
        """One token at position `pos` for every sequence of the batch: copies
        `x` [B, H] into the graph's input, replays, and returns the graph's
        output tensor (overwritten by the next step)."""
        if not 0 <= pos < self.max_seq:
            raise ValueError(f"position {pos} outside the cache of {self.max_seq} entries")
        self.x.copy_(x)
        self.pos.fill_(pos)
        self.graph.replay()
        return self.y


class LlamaTPStack:
    """A stack of decoder layers with their KV caches, the way a serving loop
    drives them: `prefill` a prompt (sequence parallel; fills the caches), then
    `decode_step` token by token, replayed from ONE CUDA graph on a GPU
    (`use_graph`, default on CUDA devices) or run eagerly.  Embedding, final norm
    and the LM head are outside (they involve none of this package's ops).

        stack = LlamaTPStack(cfg, n_layers=4, device=dev, batch=4, max_seq=4096)
        y_shard = stack.prefill(x_shard, seq=prompt_len)      # [batch * prompt_len / WS, H] in and out
        for pos in range(prompt_len, prompt_len + new_tokens):
            y = stack.decode_step(x, pos)                      # [batch, H] in and out, replicated on all ranks
    """

    def __init__(self, cfg: LlamaTPConfig, n_layers: int, device: torch.device, batch: int, max_seq: int,
                 group=None, seed: int = 0, use_graph: Optional[bool] = None, **layer_kwargs):
        self.cfg, self.batch, self.max_seq = cfg, int(batch), int(max_seq)
        self.layers = [LlamaTPDecoderLayer(cfg, device, group=group, seed=seed + 1000 * i, **layer_kwargs)
                       for i in range(n_layers)]
        self.caches = new_kv_caches(self.layers, batch, max_seq)
        self.use_graph = (device.type == "cuda") if use_graph is None else bool(use_graph)
        self._pos = torch.zeros(1, dtype=torch.int32, device=device)
        # built before any prefill: capturing runs warm-up steps that write into the caches
        self.graph = DecodeGraph(self.layers, batch, max_seq, caches=self.caches) if self.use_graph else None

    def reset(self) -> None:
        """Start new sequences: zero the caches."""
        for kc, vc in self.caches:
            kc.zero_()
            vc.zero_()

    def prefill(self, x_shard: torch.Tensor, seq: int) -> torch.Tensor:
        """The prompt's hidden states, this rank's [batch * seq / WS, H] rows, through every layer;
        each layer leaves its keys and values of positions [0, seq) in its cache."""
        if seq > self.max_seq:
            raise ValueError(f"a prompt of {seq} tokens does not fit the cache of {self.max_seq}")
        h = x_shard
        for lyr, cache in zip(self.layers, self.caches):
            h = lyr.forward(h, self.batch, seq, kv_cache=cache)
        return h

    def decode_step(self, x: torch.Tensor, pos: int) -> torch.Tensor:
        """One token per sequence at position `pos`: [batch, H] in (replicated), [batch, H] out.  With
        the graph the result tensor is overwritten by the next step."""
        if self.graph is not None:
            return self.graph.step(x, pos)
        if not 0 <= pos < self.max_seq:
            raise ValueError(f"position {pos} outside the cache of {self.max_seq} entries")
        self._pos.fill_(pos)
        return decode_static_through(self.layers, self.caches, x, self._pos)


def full_precision_reference(layers_weights: list, cfg: LlamaTPConfig, x: torch.Tensor, batch: int,
                             seq: int) -> torch.Tensor:
    """Single-process fp32 forward of the un-sharded layer, from the per-rank
    weights `[(w_qkv, w_o, w_gate_up, w_down, norm1, norm2), ...]` (CPU)."""
    ws = len(layers_weights)
    D = cfg.head_dim
    hq, hkv = cfg.n_heads // ws, cfg.n_kv_heads // ws
    ffn_local = cfg.ffn // ws
    norm1, norm2 = layers_weights[0][4].float(), layers_weights[0][5].float()
    xf = x.float()

    def rms(t, w):
        return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + cfg.eps) * w

    h = rms(xf, norm1)
    o_sum = torch.zeros_like(xf)
    pos = torch.arange(seq)[None, :].expand(batch, seq)
    for w_qkv, w_o, _, _, _, _ in layers_weights:
        qkv = h @ w_qkv.float().t()
        q, k, v = qkv.split([hq * D, hkv * D, hkv * D], dim=-1)
        q = _rope(q.view(batch, seq, hq, D), pos, cfg.rope_theta)
        k = _rope(k.view(batch, seq, hkv, D), pos, cfg.rope_theta)
        v = v.view(batch, seq, hkv, D)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                           is_causal=True, enable_gqa=True)
        o_sum += o.transpose(1, 2).reshape(batch * seq, hq * D) @ w_o.float().t()
    x1 = xf + o_sum
    h2 = rms(x1, norm2)
    d_sum = torch.zeros_like(xf)
    for _, _, w_gu, w_down, _, _ in layers_weights:
        gate, up = (h2 @ w_gu.float().t()).split(ffn_local, dim=-1)
        d_sum += (F.silu(gate) * up) @ w_down.float().t()
    return x1 + d_sum


def smoke(device: Optional[torch.device] = None) -> None:
    """One tiny forward of the layer on one GPU (world of one): exercises the
    tcgen05 GEMM behind both fused ops and checks against fp32."""
    device = device or torch.device("cuda", 0)
    cfg = LlamaTPConfig.tiny(1)
    layer = LlamaTPDecoderLayer(cfg, device, seed=1)
    batch, seq = 2, 128
    torch.manual_seed(3)
    x = (torch.randn(batch * seq, cfg.hidden, device=device) * 0.5).to(torch.bfloat16)
    y = layer.forward(x, batch, seq)
    weights = [(layer.w_qkv.cpu(), layer.w_o.cpu(), layer.w_gate_up.cpu(), layer.w_down.cpu(),
                layer.norm1.cpu(), layer.norm2.cpu())]
    ref = full_precision_reference(weights, cfg, x.cpu(), batch, seq)
    err = (y.float().cpu() - ref).abs().max().item()
    assert err < 0.1, f"decoder layer differs from fp32 reference: {err}"
