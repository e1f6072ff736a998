"""Fused GEMM + reduce-scatter against an fp32 reference and cuBLAS + NCCL."""
import pytest
import torch

from symm_mem_recipes_b200.utils.testing import spawn_ranks


def _rs_worker(rank, world_size, M, N, K, panel_w=0):
    import symm_mem_recipes_b200 as smr
    from symm_mem_recipes_b200.parallel import symm_mem

    dev = torch.device("cuda", rank)
    failures = []
    rows = M // world_size
    out = None
    for it in range(3):          # repeated calls exercise the call counters and the entry barrier
        gens = [torch.Generator().manual_seed(1000 * it + r) for r in range(world_size)]
        parts = []
        for r in range(world_size):
            a_r = (torch.randn(M, K, generator=gens[r]) * 0.05).to(torch.bfloat16)
            b_r = (torch.randn(N, K, generator=gens[r]) * 0.05).to(torch.bfloat16)
            parts.append((a_r, b_r))
        a, b = parts[rank][0].to(dev), parts[rank][1].to(dev)
        out = smr.matmul_reduce_scatter(a, b, panel_w=panel_w)
        symm_mem.check_status(dev)
        ref = torch.zeros(rows, N, dtype=torch.float32)
        for a_r, b_r in parts:
            # every partial is rounded to bf16 on the wire, then summed in fp32
            full = (a_r[rank * rows:(rank + 1) * rows].float() @ b_r.float().t())
            ref += full.to(torch.bfloat16).float()
        err = (out.float().cpu() - ref).abs()
        tol = ref.abs() * 2.0 ** -6 + 3e-2
        if not bool((err <= tol).all()):
            failures.append(f"call {it}: max err {float(err.max())}")
        lib = smr.reference_matmul_reduce_scatter(a, b)
        if not torch.allclose(lib.float(), out.float(), rtol=5e-2, atol=5e-2):
            failures.append(f"call {it}: differs from cuBLAS + NCCL")
    torch.cuda.synchronize()
    assert not failures, failures


@pytest.mark.gpu
@pytest.mark.multigpu(2)
# (768, 328, 192): 3 row blocks per rank, so a CTA pair straddles two destinations, and a ragged N edge
@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (512, 328, 192), (768, 328, 192), (4096, 8192, 1024)])
def test_matmul_reduce_scatter_2gpu(M, N, K):
    spawn_ranks(_rs_worker, 2, "nccl", (M, N, K))


@pytest.mark.gpu
@pytest.mark.multigpu(2)
@pytest.mark.parametrize("panel_w", [1, 3])
def test_matmul_reduce_scatter_column_panels_2gpu(panel_w):
    """Tiles walked in column panels: the own rows come last inside every panel, and their tiles wait
    for the peers' tiles of the same panel."""
    spawn_ranks(_rs_worker, 2, "nccl", (1024, 1280, 256, panel_w))


@pytest.mark.gpu
@pytest.mark.multigpu(8)
def test_matmul_reduce_scatter_8gpu():
    spawn_ranks(_rs_worker, 8, "nccl", (2048, 1024, 512))


@pytest.mark.gpu
def test_matmul_reduce_scatter_world_of_one():
    import symm_mem_recipes_b200 as smr

    torch.cuda.set_device(0)
    a = (torch.randn(256, 128, device="cuda") * 0.1).to(torch.bfloat16)
    b = (torch.randn(64, 128, device="cuda") * 0.1).to(torch.bfloat16)
    out = smr.matmul_reduce_scatter(a, b)
    assert torch.allclose(out.float(), a.float() @ b.float().t(), rtol=2e-2, atol=2e-2)


def _ar_worker(rank, world_size, M, N, K):
    import symm_mem_recipes_b200 as smr
    from symm_mem_recipes_b200.parallel import symm_mem

    dev = torch.device("cuda", rank)
    failures = []
    for it in range(3):
        gens = [torch.Generator().manual_seed(2000 * it + r) for r in range(world_size)]
        parts = [((torch.randn(M, K, generator=g) * 0.05).to(torch.bfloat16),
                  (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)) for g in gens]
        a, b = parts[rank][0].to(dev), parts[rank][1].to(dev)
        out = smr.matmul_all_reduce(a, b)
        symm_mem.check_status(dev)
        ref = torch.zeros(M, N, dtype=torch.float32)
        for a_r, b_r in parts:
            ref += (a_r.float() @ b_r.float().t()).to(torch.bfloat16).float()    # bf16 partials, fp32 sum
        err = (out.float().cpu() - ref).abs()
        if not bool((err <= ref.abs() * 2.0 ** -6 + 3e-2).all()):
            failures.append(f"call {it}: max err {float(err.max())}")
        gathered = [torch.empty_like(out) for _ in range(world_size)]
        torch.distributed.all_gather(gathered, out.clone())
        if not all(torch.equal(g.view(torch.int16), out.view(torch.int16)) for g in gathered):
            failures.append(f"call {it}: ranks disagree bitwise")
        rs = smr.matmul_reduce_scatter(a, b)
        rows = M // world_size
        if not torch.equal(rs.view(torch.int16), out[rank * rows:(rank + 1) * rows].view(torch.int16)):
            failures.append(f"call {it}: own rows differ from matmul_reduce_scatter")
        torch.cuda.synchronize()
        torch.distributed.barrier()
    assert not failures, failures


@pytest.mark.gpu
@pytest.mark.multigpu(2)
@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (768, 328, 192), (4096, 8192, 1024)])
def test_matmul_all_reduce_2gpu(M, N, K):
    spawn_ranks(_ar_worker, 2, "nccl", (M, N, K))
