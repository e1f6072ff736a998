"""float8_e4m3fn form of the tcgen05 GEMM and of all_gather_matmul (the dtype
follows `a_shard`, as upstream's FP8_OUTPUT switch does,
symm_mem_recipes/triton_all_gather_matmul.py:123, 311).

Every case runs in a child process.
"""
import pytest
import torch

from symm_mem_recipes_b200.utils.testing import spawn_ranks

pytestmark = [pytest.mark.gpu]

FP8 = torch.float8_e4m3fn


def _close_fp8(c, ref):
    # fp32 accumulation in another order, then ONE rounding to 3 mantissa bits
    # (half an ulp = 2^-4 relative; a different summation order may flip it to a
    # full ulp); below 2^-6 the format is subnormal with a step of 2^-9
    err = (c.float() - ref).abs()
    tol = ref.abs() * 2.0 ** -3 + 2.0 ** -8
    return bool((err <= tol).all()), float(err.max())


def _mm_worker(rank, world_size, M, N, K, block_n, num_sms, split):
    from symm_mem_recipes_b200.ops.ag_matmul import AgMatmulConfig, matmul
    from symm_mem_recipes_b200.parallel import symm_mem

    dev = torch.device("cuda", rank)
    torch.manual_seed(M + N + K)
    a = (torch.randn(M, K, device=dev) * 0.5).to(FP8)
    b = (torch.randn(N, K, device=dev) * 0.5).to(FP8)
    c = torch.zeros(M, N, dtype=torch.uint8, device=dev).view(FP8)
    cfg = AgMatmulConfig(block_n=block_n, num_sms=num_sms, split_k_tail=split, timeout_ms=2000)
    for _ in range(2):
        matmul(a, b, c, cfg)
    symm_mem.check_status(dev)
    ok, err = _close_fp8(c, a.float() @ b.float().t())
    assert ok, f"max abs error {err}"


@pytest.mark.parametrize("block_n", [128, 192, 224, 256])
@pytest.mark.parametrize("shape", [(128, 256, 128), (256, 512, 256), (200, 336, 208), (640, 1008, 1024)])
def test_matmul_fp8_small(block_n, shape):
    spawn_ranks(_mm_worker, 1, "nccl", (*shape, block_n, 0, True))


@pytest.mark.parametrize("shape,num_sms", [((768, 768, 2048), 8), ((1280, 512, 1024), 8)])
def test_matmul_fp8_split_k_tail(shape, num_sms):
    spawn_ranks(_mm_worker, 1, "nccl", (*shape, 0, num_sms, True))


def _agmm_worker(rank, world_size, rows, N, K):
    import symm_mem_recipes_b200 as smr
    from symm_mem_recipes_b200.ops.ag_matmul import AgMatmulConfig
    from symm_mem_recipes_b200.parallel import symm_mem

    dev = torch.device("cuda", rank)
    M = rows * world_size
    torch.manual_seed(7)
    b = (torch.randn(N, K, device=dev) * 0.25).to(FP8)
    a_shard = symm_mem.empty(rows, K, dtype=FP8, device=dev)
    a_out = symm_mem.empty(M, K, dtype=FP8, device=dev)
    c_out = torch.zeros(M, N, dtype=torch.uint8, device=dev).view(FP8)
    cfg = AgMatmulConfig(timeout_ms=5000)
    failures = []
    for it in range(3):
        torch.manual_seed(42 + rank + 100 * it)
        a_shard.copy_((torch.randn(rows, K, device=dev) * 0.25).to(FP8))
        torch.cuda.synchronize()
        torch.distributed.barrier()
        smr.all_gather_matmul(a_shard, b, a_out, c_out, cfg)
        symm_mem.check_status(dev)
        ref_a = torch.empty(M, K, dtype=torch.uint8, device=dev)
        torch.distributed.all_gather_into_tensor(ref_a, a_shard.view(torch.uint8))
        if not torch.equal(a_out.view(torch.uint8), ref_a):
            failures.append(f"iteration {it}: a_out differs from the all-gather")
        ok, err = _close_fp8(c_out, ref_a.view(FP8).float() @ b.float().t())
        if not ok:
            failures.append(f"iteration {it}: c_out max err {err}")
        torch.cuda.synchronize()
        torch.distributed.barrier()
    lib = smr.reference_all_gather_matmul(a_shard, b)
    ok, err = _close_fp8(c_out, lib.float())
    if not ok:
        failures.append(f"library composition differs: {err}")
    assert not failures, failures


@pytest.mark.multigpu(2)
@pytest.mark.parametrize("rows,N,K", [(128, 256, 256), (384, 512, 1024), (2048, 3584, 8192)])
def test_all_gather_matmul_fp8_2gpu(rows, N, K):
    spawn_ranks(_agmm_worker, 2, "nccl", (rows, N, K))
