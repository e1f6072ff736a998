"""RMSNorm, rotary embedding and SiLU-mul kernels against their CPU oracles
(same rounding points) and, through the decoder layer, against fp32.
"""
import pytest
import torch

pytestmark = [pytest.mark.gpu]


def _ulp_close(got, ref, extra_abs=1e-6):
    # fast-math exp / rsqrt / sincos may flip the final bf16 rounding: one ulp
    err = (got.float().cpu() - ref.float()).abs()
    return bool((err <= ref.float().abs() * 2.0 ** -7 + extra_abs).all()), float(err.max())


@pytest.mark.parametrize("rows,H", [(1, 8), (37, 512), (300, 8192), (5, 16384 + 8)])
def test_rms_norm(rows, H):
    from symm_mem_recipes_b200 import ops
    from symm_mem_recipes_b200._ext import C
    from symm_mem_recipes_b200.utils.testing import guarded_empty

    g = torch.Generator().manual_seed(rows + H)
    x = (torch.randn(rows, H, generator=g) * 0.7).to(torch.bfloat16)
    r = (torch.randn(rows, H, generator=g) * 0.3).to(torch.bfloat16)
    w = (1.0 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16)
    ref, _ = C.oracle_rms_norm_bf16(x, None, w, 1e-5)
    out, intact = guarded_empty((rows, H), torch.bfloat16, "cuda")
    ops.rms_norm(x.cuda(), w.cuda(), 1e-5, out=out)
    ok, err = _ulp_close(out, ref)
    assert ok and intact(), err
    ref2, sum2 = C.oracle_rms_norm_bf16(x, r, w, 1e-5)
    out2, s2 = ops.rms_norm(x.cuda(), w.cuda(), 1e-5, residual=r.cuda())
    assert torch.equal(s2.cpu(), sum2)
    ok, err = _ulp_close(out2, ref2)
    assert ok, err
    # residual stream kept in place: sum_out is the residual's own buffer
    stream = r.cuda()
    out3, s3 = ops.rms_norm(x.cuda(), w.cuda(), 1e-5, residual=stream, sum_out=stream)
    assert s3 is stream and torch.equal(stream.cpu(), sum2)
    ok, err = _ulp_close(out3, ref2)
    assert ok, err
    with pytest.raises(Exception, match="out must not be"):
        ops.rms_norm(x.cuda(), w.cuda(), 1e-5, out=stream, residual=stream)


@pytest.mark.parametrize("batch,seq,hq,hkv,D,pos0",
                         [(2, 24, 4, 1, 64, 0), (1, 2048, 8, 1, 128, 0), (4, 1, 8, 1, 128, 1777)])
def test_rope(batch, seq, hq, hkv, D, pos0):
    from symm_mem_recipes_b200 import ops
    from symm_mem_recipes_b200._ext import C

    g = torch.Generator().manual_seed(seq + D)
    qkv = torch.randn(batch * seq, (hq + 2 * hkv) * D, generator=g).to(torch.bfloat16)
    ref = C.oracle_rope_bf16(qkv, hq + hkv, D, seq, pos0, 500000.0)
    got = ops.rope_(qkv.cuda(), hq + hkv, D, seq, 500000.0, pos0=pos0)
    # fp32 angles (the oracle's are fp64): up to ~2e-4 rad at position 2048
    ok, err = _ulp_close(got, ref, extra_abs=4e-3)
    assert ok, err
    assert torch.equal(got[:, (hq + hkv) * D:].cpu(), qkv[:, (hq + hkv) * D:])     # V untouched


@pytest.mark.parametrize("rows,F", [(1, 8), (19, 48), (4096, 3584)])
def test_silu_mul(rows, F):
    from symm_mem_recipes_b200 import ops
    from symm_mem_recipes_b200._ext import C
    from symm_mem_recipes_b200.utils.testing import guarded_empty

    g = torch.Generator().manual_seed(rows + F)
    gu = (torch.randn(rows, 2 * F, generator=g) * 3.0).to(torch.bfloat16)
    ref = C.oracle_silu_mul_bf16(gu)
    out, intact = guarded_empty((rows, F), torch.bfloat16, "cuda")
    ops.silu_mul(gu.cuda(), out)
    ok, err = _ulp_close(out, ref)
    assert ok and intact(), err


def test_layer_with_fused_glue_matches_fp32():
    from symm_mem_recipes_b200.models.llama_tp_layer import (LlamaTPConfig, LlamaTPDecoderLayer,
                                                             full_precision_reference)

    dev = torch.device("cuda", 0)
    cfg = LlamaTPConfig.tiny(1)
    layer = LlamaTPDecoderLayer(cfg, dev, seed=1, fused_glue=True)
    batch, seq = 2, 128
    torch.manual_seed(3)
    x = (torch.randn(batch * seq, cfg.hidden, device=dev) * 0.5).to(torch.bfloat16)
    y = layer.forward(x, batch, seq)
    y_plain = LlamaTPDecoderLayer(cfg, dev, seed=1, fused_glue=False).forward(x, batch, seq)
    weights = [(layer.w_qkv.cpu(), layer.w_o.cpu(), layer.w_gate_up.cpu(), layer.w_down.cpu(),
                layer.norm1.cpu(), layer.norm2.cpu())]
    ref = full_precision_reference(weights, cfg, x.cpu(), batch, seq)
    assert (y.float().cpu() - ref).abs().max().item() < 0.1
    assert (y.float() - y_plain.float()).abs().max().item() < 0.1


@pytest.mark.parametrize("M,F,K", [(128, 128, 64), (200, 384, 96), (640, 1024, 1024), (4096, 3584, 2048)])
def test_matmul_with_swiglu_epilogue(M, F, K):
    from symm_mem_recipes_b200 import ops
    from symm_mem_recipes_b200.ops.ag_matmul import AgMatmulConfig
    from symm_mem_recipes_b200.parallel import symm_mem
    from symm_mem_recipes_b200.utils.testing import guarded_empty

    torch.manual_seed(M + F + K)
    a = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16)
    wg = (torch.randn(F, K, device="cuda") * 0.2).to(torch.bfloat16)
    wu = (torch.randn(F, K, device="cuda") * 0.2).to(torch.bfloat16)
    out, intact = guarded_empty((M, F), torch.bfloat16, "cuda")
    out.fill_(float("nan"))
    ops.matmul(a, ops.interleave_gate_up(wg, wu), out, AgMatmulConfig(timeout_ms=2000), epilogue="swiglu")
    symm_mem.check_status("cuda")
    g, u = a.float() @ wg.float().t(), a.float() @ wu.float().t()
    ref = torch.nn.functional.silu(g) * u
    err = (out.float() - ref).abs()
    tol = ref.abs() * 2.0 ** -6 + 2e-3 * (K ** 0.5) * 0.1
    assert bool((err <= tol).all()), float(err.max())
    assert intact()


def test_layer_with_fused_swiglu_matches_fp32():
    from symm_mem_recipes_b200.models.llama_tp_layer import (LlamaTPConfig, LlamaTPDecoderLayer,
                                                             full_precision_reference)

    dev = torch.device("cuda", 0)
    cfg = LlamaTPConfig.tiny(1)
    layer = LlamaTPDecoderLayer(cfg, dev, seed=1, fused_glue=True, fused_swiglu=True)
    batch, seq = 2, 128
    torch.manual_seed(3)
    x = (torch.randn(batch * seq, cfg.hidden, device=dev) * 0.5).to(torch.bfloat16)
    y = layer.forward(x, batch, seq)
    weights = [(layer.w_qkv.cpu(), layer.w_o.cpu(), layer.w_gate_up.cpu(), layer.w_down.cpu(),
                layer.norm1.cpu(), layer.norm2.cpu())]
    ref = full_precision_reference(weights, cfg, x.cpu(), batch, seq)
    assert (y.float().cpu() - ref).abs().max().item() < 0.1


@pytest.mark.parametrize("B,hq,hkv,D,s_max,positions", [
    (1, 8, 1, 128, 4096, (0, 1, 255, 256, 2047, 4095)),      # the 70B shape per rank at TP8, long cache
    (16, 8, 1, 128, 512, (0, 300, 511)),
    (3, 4, 2, 64, 40, (0, 7, 39)),                            # two KV heads, 64-wide heads, one split
    (2, 4, 4, 64, 700, (5, 699)),                             # no grouping (one query head per KV head)
])
def test_decode_attention(B, hq, hkv, D, s_max, positions):
    """One kernel for a decode step's attention (cache write + softmax(QK^T)V over 0..pos) against the
    CPU oracle; the position both as a launch argument and from a device tensor; repeated calls reuse
    the scratch and its arrival counters."""
    from symm_mem_recipes_b200 import ops
    from symm_mem_recipes_b200._ext import C

    g = torch.Generator().manual_seed(B * 1000 + s_max)
    k_cache = (torch.randn(B, s_max, hkv, D, generator=g) * 0.7).to(torch.bfloat16)
    v_cache = (torch.randn(B, s_max, hkv, D, generator=g) * 0.7).to(torch.bfloat16)
    k_dev, v_dev = k_cache.cuda(), v_cache.cuda()
    pos_dev = torch.zeros(1, dtype=torch.int32, device="cuda")
    for i, pos in enumerate(positions):
        qkv = (torch.randn(B, (hq + 2 * hkv) * D, generator=g) * 0.7).to(torch.bfloat16)
        # odd steps: the kernel rotates the new queries and key itself (oracle: RoPE first, then attention)
        theta = 500000.0 if i % 2 else 0.0
        rotated = C.oracle_rope_bf16(qkv, hq + hkv, D, 1, pos, theta) if theta else qkv
        want = C.oracle_decode_attention_bf16(rotated, k_cache, v_cache, hq, hkv, pos)   # updates the CPU caches
        qkv_dev = qkv.cuda()
        if i % 2 == 0:
            got = ops.decode_attention_(qkv_dev, k_dev, v_dev, hq, pos, rope_theta=theta)
        else:
            pos_dev.fill_(pos)
            got = ops.decode_attention_(qkv_dev, k_dev, v_dev, hq, pos_dev, rope_theta=theta)
        assert torch.equal(qkv_dev.cpu(), qkv)                                           # the input row is left alone
        err = (got.float().cpu() - want.float()).abs()
        # fp32 sums in another order and fast exp: a bf16 ulp of the output, which is an average of values ~0.7
        assert bool((err <= want.float().abs() * 2.0 ** -6 + 4e-3).all()), (pos, float(err.max()))
        # caches written: bit-exact for the value, within the fast sine / cosine (a bf16 ulp) for a rotated key
        assert torch.equal(v_dev.cpu(), v_cache), pos
        k_err = (k_dev.cpu().float() - k_cache.float()).abs()
        assert bool((k_err <= k_cache.float().abs() * 2.0 ** -7 + (4e-3 if theta else 0.0)).all()), pos
        k_dev.copy_(k_cache)                                                             # keep both histories equal
    torch.cuda.synchronize()
