"""Fused GEMV + all-reduce against an fp64 reference; identical bits on all ranks."""
import pytest
import torch

from symm_mem_recipes_b200.utils.testing import guarded_empty, spawn_ranks


def _inputs(rank, B, K, N):
    g = torch.Generator().manual_seed(100 + rank)
    x = (torch.randn(B, K, generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn(K, N, generator=g) * 0.05).to(torch.bfloat16)
    return x, w


def _gemv_worker(rank, world_size, B, K, N, algo="tc"):
    import symm_mem_recipes_b200 as smr
    from symm_mem_recipes_b200.parallel import symm_mem

    dev = torch.device("cuda", rank) if torch.cuda.device_count() > rank else torch.device("cuda", 0)
    failures = []
    ref = torch.zeros(B, N, dtype=torch.float64)
    for r in range(world_size):
        x, w = _inputs(r, B, K, N)
        ref += x.double() @ w.double()
    x, w = _inputs(rank, B, K, N)
    x, w = x.to(dev), w.to(dev)
    out, intact = guarded_empty((B, N), torch.bfloat16, dev)     # canaries before and after the output
    for it in range(4):          # repeated calls exercise the epoch / parity logic
        out.fill_(float("nan"))
        smr.gemv_all_reduce(x, w, out, algo=algo)
        symm_mem.check_status(dev)
        if not intact():
            failures.append(f"call {it}: the kernel stored outside its output")
        err = (out.double().cpu() - ref).abs()
        tol = ref.abs() * 2.0 ** -7 + 2e-2
        if not bool((err <= tol).all()):
            failures.append(f"call {it}: max err {float(err.max())}")
    if world_size > 1:
        gathered = [torch.empty_like(out) for _ in range(world_size)]
        torch.distributed.all_gather(gathered, out)
        if not all(torch.equal(g.view(torch.int16), out.view(torch.int16)) for g in gathered):
            failures.append("ranks disagree bitwise")
        lib = smr.reference_gemv_all_reduce(x, w)
        if not torch.allclose(lib.float(), out.float(), rtol=5e-2, atol=5e-2):
            failures.append("differs from cuBLAS + NCCL")
    torch.cuda.synchronize()
    assert not failures, failures


@pytest.mark.gpu
@pytest.mark.parametrize("algo", ["tc", "simt"])
@pytest.mark.parametrize("B,K,N", [(1, 512, 256), (4, 3584, 8192), (16, 3584, 8192), (3, 1000, 328), (8, 256, 64)])
def test_gemv_world_of_one(B, K, N, algo):
    torch.cuda.set_device(0)
    _gemv_worker(0, 1, B, K, N, algo)


@pytest.mark.gpu
@pytest.mark.multigpu(2)
@pytest.mark.parametrize("algo", ["tc", "simt"])
@pytest.mark.parametrize("B", [1, 4, 16])
def test_gemv_all_reduce_2gpu(B, algo):
    spawn_ranks(_gemv_worker, 2, "nccl", (B, 3584, 8192, algo))


@pytest.mark.gpu
@pytest.mark.multigpu(8)
def test_gemv_all_reduce_8gpu():
    spawn_ranks(_gemv_worker, 8, "nccl", (16, 3584, 8192))


# The tagged-word exchange of the tcgen05 kernel.
@pytest.mark.gpu
@pytest.mark.parametrize("B,K,N", [(1, 512, 256), (4, 3584, 8192), (16, 3584, 8192), (3, 1000, 328)])
def test_gemv_tagged_world_of_one(B, K, N):
    torch.cuda.set_device(0)
    _gemv_worker(0, 1, B, K, N, "tc_tagged")


@pytest.mark.gpu
@pytest.mark.multigpu(2)
@pytest.mark.parametrize("B", [1, 4, 16])
def test_gemv_tagged_2gpu(B):
    spawn_ranks(_gemv_worker, 2, "nccl", (B, 3584, 8192, "tc_tagged"))


def _gemv_nk_worker(rank, world_size, B, K, N, algo):
    """Weights stored [N, K] (the prefill layout): same result as the [K, N] form."""
    import symm_mem_recipes_b200 as smr
    from symm_mem_recipes_b200.parallel import symm_mem

    dev = torch.device("cuda", rank)
    x, w = _inputs(rank, B, K, N)
    x, w = x.to(dev), w.to(dev)
    want = smr.gemv_all_reduce(x, w, algo="tc")
    symm_mem.check_status(dev)
    w_nk = w.t().contiguous()
    for _ in range(3):
        got = smr.gemv_all_reduce(x, w_nk, algo=algo, weights_nk=True)
    symm_mem.check_status(dev)
    worst = (got.float() - want.float()).abs().max()
    assert torch.allclose(got.float(), want.float(), rtol=2.0 ** -6, atol=2e-2), worst
    torch.cuda.synchronize()


@pytest.mark.gpu
@pytest.mark.parametrize("algo", ["tc", "tc_tagged"])
@pytest.mark.parametrize("B,K,N", [(1, 512, 256), (4, 3584, 8192), (3, 1000, 328)])
def test_gemv_weights_nk_world_of_one(B, K, N, algo):
    torch.cuda.set_device(0)
    _gemv_nk_worker(0, 1, B, K, N, algo)


@pytest.mark.gpu
@pytest.mark.multigpu(2)
def test_gemv_weights_nk_2gpu():
    spawn_ranks(_gemv_nk_worker, 2, "nccl", (4, 3584, 8192, "tc"))


def _local_gemv_worker(rank, world_size):
    """`ops.gemv` inside a job with peers: every rank multiplies its own operands, nothing is
    exchanged, and the fused op still works beside it on the same shapes."""
    import symm_mem_recipes_b200 as smr
    from symm_mem_recipes_b200.parallel import symm_mem

    dev = torch.device("cuda", rank)
    for B, K, N in [(1, 8192, 1280), (16, 8192, 7168), (3, 1000, 328)]:
        g = torch.Generator().manual_seed(7 + rank)
        x = (torch.randn(B, K, generator=g) * 0.5).to(torch.bfloat16).to(dev)
        w_nk = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(dev)
        for _ in range(3):
            y = smr.gemv(x, w_nk, weights_nk=True)
        symm_mem.check_status(dev)
        ref = x.double() @ w_nk.double().t()
        assert bool(((y.double() - ref).abs() <= ref.abs() * 2.0 ** -7 + 2e-2).all()), (B, K, N)
    if world_size > 1:
        _gemv_worker(rank, world_size, 4, 1000, 328)
    torch.cuda.synchronize()


@pytest.mark.gpu
def test_local_gemv_one_gpu():
    torch.cuda.set_device(0)
    _local_gemv_worker(0, 1)


@pytest.mark.gpu
@pytest.mark.multigpu(2)
def test_local_gemv_beside_peers_2gpu():
    spawn_ranks(_local_gemv_worker, 2, "nccl")
