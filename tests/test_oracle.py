"""CPU oracles against plain PyTorch arithmetic."""
import torch

from symm_mem_recipes_b200._ext import C


def test_ordered_sum_matches_sequential_bf16_adds():
    torch.manual_seed(0)
    srcs = [torch.randn(4096).to(torch.bfloat16) for _ in range(8)]
    acc = torch.zeros(4096, dtype=torch.bfloat16)
    for s in srcs:
        acc = acc + s          # bf16 add = one RNE rounding per step
    out = C.oracle_ordered_sum_bf16(srcs)
    assert torch.equal(out.view(torch.int16), acc.view(torch.int16))


def test_ordered_sum_depends_on_order():
    torch.manual_seed(1)
    srcs = [(torch.randn(1 << 14) * (10.0 ** (i % 3))).to(torch.bfloat16) for i in range(8)]
    a = C.oracle_ordered_sum_bf16(srcs)
    b = C.oracle_ordered_sum_bf16(srcs[::-1])
    assert not torch.equal(a, b)   # the contract is a fixed rank order


def test_fp32_sum():
    torch.manual_seed(2)
    srcs = [torch.randn(1000).to(torch.bfloat16) for _ in range(4)]
    ref = sum(s.float() for s in srcs).to(torch.bfloat16)
    assert torch.equal(C.oracle_fp32_sum_bf16(srcs), ref)


def test_gemm_nt():
    torch.manual_seed(3)
    a = (torch.randn(33, 64) * 0.1).to(torch.bfloat16)
    b = (torch.randn(17, 64) * 0.1).to(torch.bfloat16)
    ref = (a.float() @ b.float().T)
    out = C.oracle_gemm_nt_bf16(a, b).float()
    assert torch.allclose(out, ref, rtol=1e-2, atol=1e-2)


def test_gemv():
    torch.manual_seed(4)
    x = (torch.randn(4, 96) * 0.1).to(torch.bfloat16)
    w = (torch.randn(96, 40) * 0.1).to(torch.bfloat16)
    ref = x.float() @ w.float()
    assert torch.allclose(C.oracle_gemv_f32(x, w), ref, rtol=1e-4, atol=1e-5)


# ---- layer glue: the oracles restate the kernels' rounding points; PyTorch restates the layer's math ----
def _glue_inputs(rows, H, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(rows, H, generator=g) * 0.7).to(torch.bfloat16)
    r = (torch.randn(rows, H, generator=g) * 0.3).to(torch.bfloat16)
    w = (1.0 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16)
    return x, r, w


def test_rms_norm_oracle_matches_the_layer_math():
    from symm_mem_recipes_b200._ext import C
    from symm_mem_recipes_b200.models.llama_tp_layer import _rms_norm

    x, r, w = _glue_inputs(37, 512)
    out, s = C.oracle_rms_norm_bf16(x, None, w, 1e-5)
    assert s.data_ptr() == x.data_ptr() or torch.equal(s, x)
    ref = _rms_norm(x, w, 1e-5)
    # the same rounding points; the mean is summed in another order, which may flip a rounding
    diff = (out.float() - ref.float()).abs()
    assert float((diff > 0).float().mean()) < 0.01
    assert bool((diff <= ref.float().abs() * 2.0 ** -7 + 1e-6).all())
    out2, s2 = C.oracle_rms_norm_bf16(x, r, w, 1e-5)
    assert torch.equal(s2, x + r)
    ref2 = _rms_norm(x + r, w, 1e-5)
    diff2 = (out2.float() - ref2.float()).abs()
    assert bool((diff2 <= ref2.float().abs() * 2.0 ** -7 + 1e-6).all())


def test_rope_oracle_matches_the_layer_math():
    from symm_mem_recipes_b200._ext import C
    from symm_mem_recipes_b200.models.llama_tp_layer import _rope

    batch, seq, hq, hkv, D = 2, 24, 4, 1, 64
    g = torch.Generator().manual_seed(3)
    qkv = (torch.randn(batch * seq, (hq + 2 * hkv) * D, generator=g)).to(torch.bfloat16)
    out = C.oracle_rope_bf16(qkv, hq + hkv, D, seq, 0, 500000.0)
    pos = torch.arange(seq)[None, :].expand(batch, seq)
    q, k, v = qkv.split([hq * D, hkv * D, hkv * D], dim=-1)
    ref_q = _rope(q.reshape(batch, seq, hq, D), pos, 500000.0).reshape(batch * seq, hq * D)
    ref_k = _rope(k.reshape(batch, seq, hkv, D), pos, 500000.0).reshape(batch * seq, hkv * D)
    got_q, got_k, got_v = out.split([hq * D, hkv * D, hkv * D], dim=-1)
    assert torch.equal(got_v, v)                                   # V is not rotated
    for got, ref in ((got_q, ref_q), (got_k, ref_k)):
        assert bool(((got.float() - ref.float()).abs() <= 2.0 ** -7 * ref.float().abs() + 2e-3).all())
    # decode form: one token per sequence at position 17
    one = qkv[:batch].clone()
    dec = C.oracle_rope_bf16(one, hq + hkv, D, 1, 17, 500000.0)
    p17 = torch.full((batch, 1), 17)
    ref17 = _rope(one[:, : hq * D].reshape(batch, 1, hq, D), p17, 500000.0).reshape(batch, hq * D)
    assert bool(((dec[:, : hq * D].float() - ref17.float()).abs() <= 2.0 ** -7 * ref17.float().abs() + 2e-3).all())


def test_silu_mul_oracle_matches_the_layer_math():
    from symm_mem_recipes_b200._ext import C

    g = torch.Generator().manual_seed(5)
    gu = (torch.randn(19, 2 * 48, generator=g) * 3.0).to(torch.bfloat16)
    out = C.oracle_silu_mul_bf16(gu)
    gate, up = gu.split(48, dim=-1)
    ref = (torch.nn.functional.silu(gate.float()) * up.float()).to(torch.bfloat16)
    diff = (out.float() - ref.float()).abs()
    assert bool((diff <= ref.float().abs() * 2.0 ** -7 + 1e-6).all())
