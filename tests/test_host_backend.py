"""The public API end to end on CPU: gloo ranks, POSIX-shm symmetric memory,
host implementation of the barrier and all-reduce protocols."""
import pytest
import torch

from symm_mem_recipes_b200.utils.testing import seeded_normal_bf16, spawn_ranks

NUMEL = 8192


def _all_reduce_worker(rank, world_size, algo):
    import symm_mem_recipes_b200 as smr
    from symm_mem_recipes_b200._ext import C
    from symm_mem_recipes_b200.parallel import symm_mem

    t = symm_mem.empty(NUMEL, dtype=torch.bfloat16, device="cpu")
    t.copy_(seeded_normal_bf16(NUMEL, rank))
    hdl = symm_mem.rendezvous(t)
    assert hdl.rank == rank and hdl.world_size == world_size
    assert symm_mem.rendezvous(t) is hdl          # cached
    srcs = [seeded_normal_bf16(NUMEL, r) for r in range(world_size)]
    if algo == "one_shot":
        out = smr.one_shot_all_reduce(t, exit_barrier=True)
        ref = C.oracle_ordered_sum_bf16(srcs)
        assert torch.equal(t, srcs[rank])         # input untouched
    elif algo == "two_shot":
        out = smr.two_shot_all_reduce_(t)
        ref = C.oracle_ordered_sum_bf16(srcs)
    elif algo == "multimem":
        out = smr.multimem_all_reduce_(t)
        ref = C.oracle_fp32_sum_bf16(srcs)
    else:
        out = smr.all_reduce(t, algo="auto")
        ref = C.oracle_ordered_sum_bf16(srcs)
    assert torch.equal(out.view(torch.int16), ref.view(torch.int16))
    hdl.barrier()
    assert int(hdl.get_signal_pad().abs().sum()) == 0   # zero-pad invariant


@pytest.mark.parametrize("algo", ["one_shot", "two_shot", "multimem", "auto"])
def test_all_reduce_gloo_ws2(algo):
    spawn_ranks(_all_reduce_worker, 2, "gloo", (algo,))


def test_all_reduce_gloo_ws4():
    spawn_ranks(_all_reduce_worker, 4, "gloo", ("one_shot",))


def _low_latency_worker(rank, world_size):
    """The tagged-word protocol over shared memory: sizes change from call to
    call, parities alternate, the last call is in place."""
    import symm_mem_recipes_b200 as smr
    from symm_mem_recipes_b200._ext import C

    for call, numel in enumerate([8192, 64, 8192, 131072, 1024, 1024, 1024]):
        srcs = [seeded_normal_bf16(numel, r, seed=100 + call) for r in range(world_size)]
        mine = srcs[rank].clone()              # an ordinary tensor: the input need not be symmetric
        ref = C.oracle_ordered_sum_bf16(srcs)
        if call % 2:
            out = smr.low_latency_all_reduce(mine, out=mine)   # in place
        else:
            out = smr.low_latency_all_reduce(mine)
        assert torch.equal(out.view(torch.int16), ref.view(torch.int16)), f"call {call}"


@pytest.mark.parametrize("world_size", [2, 4])
def test_low_latency_all_reduce_gloo(world_size):
    spawn_ranks(_low_latency_worker, world_size, "gloo")


def _peer_view_worker(rank, world_size):
    from symm_mem_recipes_b200.parallel import symm_mem

    t = symm_mem.empty(4, 16, dtype=torch.float32, device="cpu")
    t.fill_(float(rank + 1))
    hdl = symm_mem.rendezvous(t)
    hdl.barrier()
    for r in range(world_size):
        peer = hdl.get_buffer(r, (4, 16), torch.float32)
        assert float(peer[0, 0]) == r + 1 and float(peer[3, 15]) == r + 1
    row = hdl.get_buffer((rank + 1) % world_size, (16,), torch.float32, storage_offset=32)
    assert float(row.sum()) == 16.0 * ((rank + 1) % world_size + 1)
    hdl.barrier(channel=3)


def test_peer_views_and_channels():
    spawn_ranks(_peer_view_worker, 2, "gloo")


def _timeout_worker(rank, world_size):
    from symm_mem_recipes_b200.errors import SymmMemTimeout
    from symm_mem_recipes_b200.parallel import symm_mem

    t = symm_mem.empty(64, dtype=torch.bfloat16, device="cpu")
    hdl = symm_mem.rendezvous(t)
    if rank == 0:
        # rank 1 never joins channel 5: the wait must give up, not hang
        with pytest.raises(SymmMemTimeout) as e:
            hdl.barrier(channel=5, timeout_ms=200)
        assert e.value.code == 2 and e.value.peer == 1
    hdl.barrier(channel=0)


def test_barrier_timeout_reports_missing_peer():
    spawn_ranks(_timeout_worker, 2, "gloo")


def test_single_process_world_of_one():
    import symm_mem_recipes_b200 as smr
    from symm_mem_recipes_b200.parallel import symm_mem

    t = symm_mem.empty(256, dtype=torch.bfloat16, device="cpu")
    t.copy_(seeded_normal_bf16(256, 0))
    out = smr.one_shot_all_reduce(t)
    assert torch.equal(out, t)
    symm_mem.free(t)


def test_rejects_foreign_tensor():
    import symm_mem_recipes_b200 as smr
    from symm_mem_recipes_b200.errors import SymmMemError

    with pytest.raises(SymmMemError):
        smr.one_shot_all_reduce(torch.zeros(64, dtype=torch.bfloat16))
