"""tcgen05 GEMM and the fused all-gather + GEMM against fp32 references."""
import pytest
import torch

from symm_mem_recipes_b200.utils.testing import guarded_empty, spawn_ranks


def _ref(a, b):
    return a.float() @ b.float().t()


def _close(c, ref, K):
    # fp32 accumulation in another order plus one bf16 rounding
    err = (c.float() - ref).abs()
    tol = ref.abs() * 2.0 ** -7 + 1e-3 * (K ** 0.5) * 0.02
    return bool((err <= tol).all()), float(err.max())


@pytest.mark.gpu
@pytest.mark.parametrize("block_n", [128, 192, 224, 256])
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 256), (200, 328, 96), (640, 1000, 1024)])
def test_matmul_small(block_n, shape):
    from symm_mem_recipes_b200.ops.ag_matmul import AgMatmulConfig, matmul
    from symm_mem_recipes_b200.parallel import symm_mem

    M, N, K = shape
    torch.manual_seed(M + N + K)
    a = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16)
    b = (torch.randn(N, K, device="cuda") * 0.5).to(torch.bfloat16)
    c, intact = guarded_empty((M, N), torch.bfloat16, "cuda")    # canaries before and after the output
    c.fill_(float("nan"))
    matmul(a, b, c, AgMatmulConfig(block_n=block_n, timeout_ms=2000))
    symm_mem.check_status("cuda")
    ok, err = _close(c, _ref(a, b), K)
    assert ok, f"max abs error {err}"
    assert intact(), "the kernel stored outside its output"


@pytest.mark.gpu
@pytest.mark.parametrize("panel_w", [1, 2, 3, 5])
@pytest.mark.parametrize("shape", [(640, 1280, 256), (1152, 1000, 512)])
def test_matmul_column_panels(panel_w, shape):
    """The tile order in column panels (whole, uneven and single-tile panels, with and without the
    split-K tail) computes every tile exactly once: same bits as the one-panel order."""
    from symm_mem_recipes_b200.ops.ag_matmul import AgMatmulConfig, matmul
    from symm_mem_recipes_b200.parallel import symm_mem

    M, N, K = shape
    torch.manual_seed(M + N + K)
    a = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16)
    b = (torch.randn(N, K, device="cuda") * 0.5).to(torch.bfloat16)
    for split in (False, True):
        want = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        matmul(a, b, want, AgMatmulConfig(block_n=256, num_sms=8, split_k_tail=split, panel_w=1000, timeout_ms=2000))
        c, intact = guarded_empty((M, N), torch.bfloat16, "cuda")
        c.fill_(float("nan"))
        matmul(a, b, c, AgMatmulConfig(block_n=256, num_sms=8, split_k_tail=split, panel_w=panel_w, timeout_ms=2000))
        symm_mem.check_status("cuda")
        ok, err = _close(c, _ref(a, b), K)
        assert ok, f"max abs error {err}"
        assert intact(), "the kernel stored outside its output"
        if not split:
            assert torch.equal(c, want), "whole tiles: the order of the tiles must not change a bit"


@pytest.mark.gpu
@pytest.mark.parametrize("shape,num_sms", [((768, 768, 1024), 8), ((1280, 512, 512), 8), ((768, 768, 4096), 8),
                                           ((16384, 3584, 1024), 0)])
def test_matmul_split_k_tail(shape, num_sms):
    """Tile counts that leave a thin last wave: its tiles are cut along K and
    reduced through scratch memory; the result must not differ from the plain
    schedule by more than summation order."""
    from symm_mem_recipes_b200.ops.ag_matmul import AgMatmulConfig, matmul
    from symm_mem_recipes_b200.parallel import symm_mem

    M, N, K = shape
    torch.manual_seed(M + N + K)
    a = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16)
    b = (torch.randn(N, K, device="cuda") * 0.5).to(torch.bfloat16)
    outs = []
    for split in (True, False):
        c = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        for _ in range(2):       # second call reuses the scratch and its counters
            matmul(a, b, c, AgMatmulConfig(num_sms=num_sms, split_k_tail=split, timeout_ms=2000))
        symm_mem.check_status("cuda")
        outs.append(c)
    ok, err = _close(outs[0], _ref(a, b), K)
    assert ok, f"split-K tail: max abs error {err}"
    ok, err = _close(outs[1], _ref(a, b), K)
    assert ok, f"plain schedule: max abs error {err}"


@pytest.mark.gpu
def test_matmul_llama70b_shape_vs_cublas():
    from symm_mem_recipes_b200.ops.ag_matmul import AgMatmulConfig, matmul
    from symm_mem_recipes_b200.parallel import symm_mem

    M, N, K = 4096, 3584, 8192
    torch.manual_seed(0)
    a = (torch.randn(M, K, device="cuda") * 0.02).to(torch.bfloat16)
    b = (torch.randn(N, K, device="cuda") * 0.02).to(torch.bfloat16)
    c = matmul(a, b, config=AgMatmulConfig(timeout_ms=2000))
    symm_mem.check_status("cuda")
    ref = torch.matmul(a, b.t())
    assert torch.allclose(c.float(), ref.float(), rtol=2e-2, atol=2e-3)


def _agmm_worker(rank, world_size, rows, N, K, mode):
    import symm_mem_recipes_b200 as smr
    from symm_mem_recipes_b200.ops.ag_matmul import AgMatmulConfig
    from symm_mem_recipes_b200.parallel import symm_mem

    dev = torch.device("cuda", rank)
    torch.manual_seed(42 + rank)
    a_shard = symm_mem.empty(rows, K, dtype=torch.bfloat16, device=dev)
    a_shard.copy_((torch.randn(rows, K, device=dev) * 0.02).to(torch.bfloat16))
    torch.manual_seed(7)
    b = (torch.randn(N, K, device=dev) * 0.02).to(torch.bfloat16)
    M = rows * world_size
    if mode in ("push", "push_multicast", "push_plain", "push_panels"):   # gathered A lands in symmetric memory
        a_out = symm_mem.empty(M, K, dtype=torch.bfloat16, device=dev)
    elif mode == "plain":       # ordinary a_out, as in the upstream API: internal buffer plus one copy
        a_out = torch.zeros(M, K, dtype=torch.bfloat16, device=dev)
    else:                       # internal symmetric buffer
        from symm_mem_recipes_b200.ops.ag_matmul import gather_buffer
        a_out = None
    c_out = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    # the broadcast through the switch (multimem.st) and the plain peer stores, whatever the world size picks
    cfg = AgMatmulConfig(timeout_ms=5000, push_plain_stores={"push_multicast": 0, "push_plain": 1}.get(mode, -1),
                         panel_w=1 if mode == "push_panels" else 0)
    failures = []
    for it in range(3):
        smr.all_gather_matmul(a_shard, b, a_out, c_out, cfg)
        symm_mem.check_status(dev)
        if a_out is None:
            a_out = gather_buffer(M, K, dev)
        ref_a = torch.empty_like(a_out)
        torch.distributed.all_gather_into_tensor(ref_a, a_shard)
        if not torch.equal(a_out, ref_a):
            failures.append(f"iteration {it}: a_out differs from the all-gather")
        ref = ref_a.float() @ b.float().t()
        if not torch.allclose(c_out.float(), ref, rtol=2e-2, atol=2e-3):
            failures.append(f"iteration {it}: c_out max err {(c_out.float() - ref).abs().max().item()}")
        # new data every iteration: stale flags or stale a_out would show
        a_shard.copy_((torch.randn(rows, K, device=dev) * 0.02).to(torch.bfloat16))
        a_out.zero_()
        if mode == "internal":
            a_out = None
        torch.cuda.synchronize()
        torch.distributed.barrier()
    c_lib = smr.reference_all_gather_matmul(a_shard, b)
    c_mm = smr.all_gather_matmul(a_shard, b, a_out=ref_a, mm_only=True)
    symm_mem.check_status(dev)
    if c_mm.shape != c_lib.shape:
        failures.append("mm_only shape mismatch")
    torch.cuda.synchronize()
    assert not failures, failures


@pytest.mark.gpu
@pytest.mark.multigpu(2)
@pytest.mark.parametrize("mode", ["push_multicast", "push_plain", "push_panels", "internal", "plain"])
@pytest.mark.parametrize("rows,N,K", [(128, 256, 256), (384, 512, 1024), (2048, 3584, 8192)])
def test_all_gather_matmul_2gpu(rows, N, K, mode):
    spawn_ranks(_agmm_worker, 2, "nccl", (rows, N, K, mode))


@pytest.mark.gpu
@pytest.mark.multigpu(2)
def test_all_gather_matmul_push_without_multicast(monkeypatch):
    monkeypatch.setenv("SMR_DISABLE_MULTICAST", "1")     # plain peer stores instead of multimem.st
    spawn_ranks(_agmm_worker, 2, "nccl", (256, 512, 1024, "push"))


@pytest.mark.gpu
@pytest.mark.multigpu(8)
def test_all_gather_matmul_8gpu():
    spawn_ranks(_agmm_worker, 8, "nccl", (2048, 3584, 8192, "push"))
