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


def _emulate_decode_attention(qkv, k_cache, v_cache, hq, hkv, pos, n_split, warps=8, no_score=-1.0e30):
    """The decode-attention kernel's algorithm step by step in fp32 (units of strided positions with an
    online softmax, merge of a CTA's warps, merge of the CTAs), with its finite stand-in for "no
    position seen": what the kernel computes if its code follows its design."""
    import math

    B, s_max, _, D = k_cache.shape
    G = hq // hkv
    n_units = n_split * warps
    scale = 1.0 / math.sqrt(D)
    out = torch.zeros(B, hq * D)

    def merge(parts):                                   # [(m, l, acc[D])] -> (m, l, acc)
        big = max([no_score] + [m for m, _, _ in parts])
        lsum, acc = 0.0, torch.zeros(D)
        for m, l, a in parts:
            w = math.exp(max(m - big, -745.0))          # exp underflows to 0 like __expf
            lsum += w * l
            acc = acc + w * a
        return big, lsum, acc

    for b in range(B):
        row = qkv[b].float()
        for kvh in range(hkv):
            k_new = row[(hq + kvh) * D:(hq + kvh + 1) * D]
            v_new = row[(hq + hkv + kvh) * D:(hq + hkv + kvh + 1) * D]
            for g in range(G):
                q = row[(kvh * G + g) * D:(kvh * G + g + 1) * D] * scale
                cta_parts = []
                for split in range(n_split):
                    warp_parts = []
                    for warp in range(warps):
                        unit = split * warps + warp
                        m, l, acc = no_score, 0.0, torch.zeros(D)
                        for p in range(unit, pos + 1, n_units):
                            k = k_new if p == pos else k_cache[b, p, kvh].float()
                            v = v_new if p == pos else v_cache[b, p, kvh].float()
                            s = float(q @ k)
                            m_new = max(m, s)
                            corr, w = math.exp(max(m - m_new, -745.0)), math.exp(s - m_new)
                            l = l * corr + w
                            acc = acc * corr + w * v
                            m = m_new
                        warp_parts.append((m, l, acc))
                    cta_parts.append(merge(warp_parts))
                _, l, acc = merge(cta_parts)
                out[b, (kvh * G + g) * D:(kvh * G + g + 1) * D] = acc / l
    return out


def test_decode_attention_algorithm_and_oracle():
    """The split / merge scheme of the decode-attention kernel (emulated in fp32) against the C++
    oracle and against PyTorch's attention, including positions where most units see nothing."""
    import torch.nn.functional as F

    from symm_mem_recipes_b200._ext import C

    g = torch.Generator().manual_seed(4)
    B, hq, hkv, D, s_max = 2, 4, 2, 64, 300
    for pos, n_split in ((0, 2), (1, 2), (15, 2), (16, 1), (150, 2), (299, 2)):
        qkv = (torch.randn(B, (hq + 2 * hkv) * D, generator=g) * 0.7).to(torch.bfloat16)
        kc = (torch.randn(B, s_max, hkv, D, generator=g) * 0.7).to(torch.bfloat16)
        vc = (torch.randn(B, s_max, hkv, D, generator=g) * 0.7).to(torch.bfloat16)
        emulated = _emulate_decode_attention(qkv, kc, vc, hq, hkv, pos, n_split)
        kc2, vc2 = kc.clone(), vc.clone()
        oracle = C.oracle_decode_attention_bf16(qkv, kc2, vc2, hq, hkv, pos)
        assert torch.isfinite(emulated).all()
        assert (emulated - oracle.float()).abs().max().item() < 1e-2, pos
        # the oracle wrote the new key / value rows, and agrees with PyTorch on the updated caches
        q, k, v = qkv.split([hq * D, hkv * D, hkv * D], dim=-1)
        assert torch.equal(kc2[:, pos], k.view(B, hkv, D)) and torch.equal(vc2[:, pos], v.view(B, hkv, D))
        assert torch.equal(kc2[:, :pos], kc[:, :pos]) and torch.equal(kc2[:, pos + 1:], kc[:, pos + 1:])
        ref = F.scaled_dot_product_attention(q.view(B, 1, hq, D).transpose(1, 2).float(),
                                             kc2[:, :pos + 1].transpose(1, 2).float(),
                                             vc2[:, :pos + 1].transpose(1, 2).float(), enable_gqa=True)
        assert (oracle.float() - ref.transpose(1, 2).reshape(B, hq * D)).abs().max().item() < 1e-2, pos
