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


def _sub_group_worker(rank, world_size):
    """Two sub-groups of two ranks each, reducing at the same time: `all_reduce(auto)` on a tensor
    that was rendezvoused on a sub-group must reduce over that sub-group only, small messages
    (the low-latency inbox, a workspace per group) included."""
    import torch.distributed as dist

    import symm_mem_recipes_b200 as smr
    from symm_mem_recipes_b200._ext import C
    from symm_mem_recipes_b200.parallel import symm_mem

    groups = [dist.new_group([0, 1]), dist.new_group([2, 3])]      # every rank creates both
    mine = groups[rank // 2]
    members = [0, 1] if rank < 2 else [2, 3]
    for numel in (1024, 8192, 1 << 18):                            # low-latency sizes and one beyond them
        t = symm_mem.empty(numel, dtype=torch.bfloat16, device="cpu")
        t.copy_(seeded_normal_bf16(numel, rank))
        hdl = symm_mem.rendezvous(t, mine)
        assert hdl.world_size == 2 and hdl.rank == rank % 2
        out = smr.all_reduce(t, algo="auto")
        ref = C.oracle_ordered_sum_bf16([seeded_normal_bf16(numel, r) for r in members])
        assert torch.equal(out.view(torch.int16), ref.view(torch.int16)), numel
    dist.barrier()


def test_all_reduce_on_sub_groups():
    spawn_ranks(_sub_group_worker, 4, "gloo")


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


# ---- host-side liveness: a rank that leaves between steps is noticed before the next launch ----
def _heartbeat_worker(rank, world_size):
    import time

    import symm_mem_recipes_b200 as smr
    from symm_mem_recipes_b200.parallel import symm_mem
    from symm_mem_recipes_b200.parallel.health import Heartbeat, PeerLost

    hb = Heartbeat(interval_s=0.05)
    hb.wait_for_all(timeout_s=30)
    t = symm_mem.empty(4096, dtype=torch.bfloat16, device="cpu")
    t.copy_(seeded_normal_bf16(4096, rank))
    hdl = symm_mem.rendezvous(t)
    for step in range(2):                       # everybody is there: the check passes, the op runs
        hb.check(max_age_s=5.0)
        hdl.barrier()
        smr.one_shot_all_reduce(t)
        hdl.barrier()
    if rank == world_size - 1:
        hb.stop()                               # leaves between steps, nothing of it in flight
        return
    lost = None
    deadline = time.time() + 20
    while lost is None and time.time() < deadline:
        try:
            hb.check(max_age_s=5.0)
            time.sleep(0.02)
        except PeerLost as e:
            lost = e
    assert lost is not None and lost.rank == world_size - 1 and "left" in lost.reason
    hb.stop(leaving=False)


@pytest.mark.parametrize("world_size", [2, 3])
def test_heartbeat_names_the_rank_that_left(world_size):
    spawn_ranks(_heartbeat_worker, world_size, "gloo")


def test_heartbeat_goes_stale_without_a_goodbye():
    """A rank whose process stops beating (no orderly leave) is reported by age."""
    import time

    from torch.distributed import HashStore

    from symm_mem_recipes_b200.parallel.health import Heartbeat, PeerLost

    store = HashStore()
    a = Heartbeat(store=store, rank=0, world_size=2, interval_s=0.02)
    b = Heartbeat(store=store, rank=1, world_size=2, interval_s=0.02)
    a.wait_for_all(5)
    a.check(max_age_s=1.0)
    b.stop(leaving=False)                       # as if its process had died
    time.sleep(0.3)
    with pytest.raises(PeerLost) as e:
        a.check(max_age_s=0.2)
    assert e.value.rank == 1 and "ago" in e.value.reason
    a.stop()
    # a rank that never came up
    c = Heartbeat(store=HashStore(), rank=0, world_size=2, interval_s=0.02)
    with pytest.raises(PeerLost):
        c.wait_for_all(timeout_s=0.2)
    c.stop()


# ---- upstream entry points under their own names ----
def _compat_worker(rank, world_size):
    from symm_mem_recipes_b200 import compat
    from symm_mem_recipes_b200.parallel import symm_mem

    rows, cols, splits = 8, 16, 2
    big = symm_mem.empty(2, rows, cols, dtype=torch.bfloat16, device="cpu")
    inp = big[1]                                                   # a view at an offset inside the allocation
    inp.copy_(torch.full((rows, cols), float(rank + 1)).to(torch.bfloat16))
    symm_mem.rendezvous(big).barrier()
    out = torch.zeros(rows * world_size, cols, dtype=torch.bfloat16)
    progress = torch.zeros(world_size * splits, dtype=torch.int32)
    compat.all_gather_with_progress(out, inp, progress, splits)
    assert bool((progress == 1).all())
    for r in range(world_size):
        assert bool((out[r * rows:(r + 1) * rows] == r + 1).all())
    ones = symm_mem.empty(64, dtype=torch.bfloat16, device="cpu")
    ones.fill_(1)
    symm_mem.rendezvous(ones).barrier()
    assert bool(compat.one_shot_all_reduce(ones).eq(world_size).all())   # upstream's own check
    cfg = compat._config_from_dict({"BLOCK_SIZE_M": 128, "BLOCK_SIZE_N": 256, "BLOCK_SIZE_K": 64, "num_stages": 3})
    assert cfg.block_n == 256 and compat._config_from_dict({"BLOCK_SIZE_N": 64}).block_n == 0
    assert compat.all_gather_matmul_baseline is not None and compat.benchmark_with_event is not None


@pytest.mark.parametrize("world_size", [2, 3])
def test_upstream_names(world_size):
    spawn_ranks(_compat_worker, world_size, "gloo")


def _signal_worker(rank, world_size):
    from symm_mem_recipes_b200.errors import SymmMemTimeout
    from symm_mem_recipes_b200.parallel import symm_mem

    t = symm_mem.empty(1024, dtype=torch.float32, device="cpu")
    hdl = symm_mem.rendezvous(t)
    assert len(hdl.buffer_ptrs) == world_size and hdl.buffer_ptrs[rank] == t.data_ptr()
    assert len(set(hdl.signal_pad_ptrs)) == world_size
    nxt, prv = (rank + 1) % world_size, (rank - 1) % world_size
    for it in range(50):                       # a ring of one-to-one signals: write, signal, wait, read
        t.fill_(float(100 * it + rank))
        hdl.put_signal(nxt, channel=3)
        hdl.wait_signal(prv, channel=3)
        got = hdl.get_buffer(prv, (1024,), torch.float32)
        assert float(got[0]) == float(100 * it + prv) and float(got[-1]) == float(100 * it + prv)
        hdl.barrier(channel=1)                 # nobody overwrites before everybody has read
    assert int(hdl.get_signal_pad().abs().sum()) == 0          # every signal was consumed
    # a rendezvous that does not touch the pad: a fast rank's next pad barrier would otherwise raise
    # a slot on a rank that is still summing its pad above
    import torch.distributed as dist
    dist.barrier()
    flags = torch.zeros(4, dtype=torch.int32)
    hdl.stream_write_value32(flags, 2, 7)
    assert flags.tolist() == [0, 0, 7, 0]
    if rank == 0:
        with pytest.raises(SymmMemTimeout) as e:              # nobody signals on channel 9
            hdl.wait_signal(nxt, channel=9, timeout_ms=50)
        assert e.value.peer == nxt
    hdl.barrier(channel=1)


@pytest.mark.parametrize("world_size", [2, 4])
def test_one_to_one_signals(world_size):
    spawn_ranks(_signal_worker, world_size, "gloo")


# ---- elastic: the survivors of a lost rank re-form a smaller group and carry on ----
def _reform_worker(rank, world_size, rdzv_file):
    import time

    import torch.distributed as dist

    import symm_mem_recipes_b200 as smr
    from symm_mem_recipes_b200._ext import C
    from symm_mem_recipes_b200.parallel import symm_mem
    from symm_mem_recipes_b200.parallel.health import Heartbeat, PeerLost

    hb = Heartbeat(interval_s=0.05)
    hb.wait_for_all(timeout_s=30)
    numel = 4096
    t = symm_mem.empty(numel, dtype=torch.bfloat16, device="cpu")
    t.copy_(seeded_normal_bf16(numel, rank))
    hdl = symm_mem.rendezvous(t)
    hdl.barrier()
    out3 = smr.one_shot_all_reduce(t)
    hdl.barrier()
    assert torch.equal(out3, C.oracle_ordered_sum_bf16([seeded_normal_bf16(numel, r) for r in range(world_size)]))
    small = smr.low_latency_all_reduce(t[:512].clone())          # leaves a cached workspace behind
    assert small.shape == (512,)
    if rank == world_size - 1:
        hb.stop()                                                # the rank that goes away, between steps
        return
    while True:                                                  # survivors notice on the host ...
        try:
            hb.check(max_age_s=10.0)
            time.sleep(0.02)
        except PeerLost as e:
            assert e.rank == world_size - 1
            break
    hb.stop(leaving=False)
    symm_mem.reset()                                             # ... drop everything tied to the old group,
    dist.destroy_process_group()
    survivors = world_size - 1
    dist.init_process_group("gloo", init_method=f"file://{rdzv_file}", rank=rank, world_size=survivors)
    t2 = symm_mem.empty(numel, dtype=torch.bfloat16, device="cpu")   # ... and carry on as a smaller world
    t2.copy_(seeded_normal_bf16(numel, rank))
    hdl2 = symm_mem.rendezvous(t2)
    assert hdl2.world_size == survivors
    hdl2.barrier()
    out2 = smr.one_shot_all_reduce(t2)
    hdl2.barrier()
    assert torch.equal(out2, C.oracle_ordered_sum_bf16([seeded_normal_bf16(numel, r) for r in range(survivors)]))
    again = smr.low_latency_all_reduce(t2[:512].clone())         # the cached workspace was re-created
    assert torch.equal(again, out2[:512])


def test_survivors_reform_a_smaller_group(tmp_path):
    spawn_ranks(_reform_worker, 3, "gloo", (str(tmp_path / "rdzv2"),))


def _free_worker(rank, world_size):
    import time

    from symm_mem_recipes_b200.parallel import symm_mem

    a = symm_mem.empty(1024, dtype=torch.float32, device="cpu")
    b = symm_mem.empty(1024, dtype=torch.float32, device="cpu")
    ha, hb = symm_mem.rendezvous(a), symm_mem.rendezvous(b)
    a.fill_(float(rank + 1))
    ha.barrier()
    if rank == 0:
        time.sleep(0.5)                          # a slow reader: rank 1 must not unmap under it
        assert float(ha.get_buffer(1, (1024,), torch.float32)[-1]) == 2.0
    symm_mem.free(a)                             # collective: nobody releases before everybody is here
    assert not symm_mem.is_symm_mem_tensor(a)
    b.fill_(float(rank))
    hb.barrier()
    assert float(hb.get_buffer((rank + 1) % world_size, (1024,), torch.float32)[0]) == float((rank + 1) % world_size)
    hb.barrier()


def test_free_is_collective():
    spawn_ranks(_free_worker, 2, "gloo")


def test_memory_summary_counts_allocations():
    from symm_mem_recipes_b200.parallel import symm_mem

    before = symm_mem.memory_summary()
    t = symm_mem.empty(1000, dtype=torch.float32, device="cpu")
    u = symm_mem.empty(16, 16, dtype=torch.bfloat16, device="cpu")
    symm_mem.rendezvous(u)
    s = symm_mem.memory_summary()
    assert s["count"] == before["count"] + 2
    assert s["payload_bytes"] == before["payload_bytes"] + 4000 + 512
    assert s["block_bytes"] >= s["payload_bytes"] + 2 * 128 * 1024          # each block carries its signal pad
    assert sum(a["rendezvoused"] for a in s["allocations"]) == sum(a["rendezvoused"] for a in before["allocations"]) + 1
    symm_mem.free(t)
    symm_mem.free(u)
    assert symm_mem.memory_summary()["count"] == before["count"]


def _reset_same_group_worker(rank, world_size):
    """reset() and carry on with the SAME process group (what a driver does after a device-side
    timeout): the new allocations rendezvous through a Store that still holds the old exchange's
    keys, and must not read them."""
    import symm_mem_recipes_b200 as smr
    from symm_mem_recipes_b200._ext import C
    from symm_mem_recipes_b200.parallel import symm_mem

    for generation, numel in enumerate((4096, 1024, 8192)):
        assert symm_mem.generation() == generation
        t = symm_mem.empty(numel, dtype=torch.bfloat16, device="cpu")
        t.copy_(seeded_normal_bf16(numel, rank + 10 * generation))
        hdl = symm_mem.rendezvous(t)
        hdl.barrier()
        peer = hdl.get_buffer((rank + 1) % world_size, (numel,), torch.bfloat16)
        assert torch.equal(peer, seeded_normal_bf16(numel, (rank + 1) % world_size + 10 * generation))
        out = smr.one_shot_all_reduce(t, exit_barrier=True)
        want = C.oracle_ordered_sum_bf16([seeded_normal_bf16(numel, r + 10 * generation) for r in range(world_size)])
        assert torch.equal(out, want)
        assert smr.low_latency_all_reduce(t[:512].clone()).shape == (512,)      # a cached workspace to drop
        symm_mem.reset()
        assert symm_mem.memory_summary()["count"] == 0


def test_reset_and_carry_on_with_the_same_group():
    spawn_ranks(_reset_same_group_worker, 3, "gloo")
