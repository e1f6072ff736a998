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
