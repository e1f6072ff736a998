"""Allocator, rendezvous, barrier and all-reduce on real GPUs.

World of one runs in-process; worlds of 2/4/8 run one process per GPU over
NCCL.  Every all-reduce result is compared with the CPU oracle (bit-exact for
the ordered-sum algorithms, one bf16 ulp for the in-switch reduction).
"""
import pytest
import torch

from symm_mem_recipes_b200.utils.testing import seeded_normal_bf16, spawn_ranks


@pytest.mark.gpu
def test_world_of_one_all_paths():
    import symm_mem_recipes_b200 as smr
    from symm_mem_recipes_b200.parallel import symm_mem

    torch.cuda.set_device(0)
    t = symm_mem.empty(8192, dtype=torch.bfloat16, device="cuda")
    assert int(t.float().abs().sum()) == 0           # zero-filled
    t.copy_(seeded_normal_bf16(8192, 0, "cuda"))
    hdl = symm_mem.rendezvous(t)
    assert (hdl.rank, hdl.world_size) == (0, 1)
    out = smr.one_shot_all_reduce(t, exit_barrier=True)
    assert torch.equal(out, t)
    before = t.clone()
    smr.two_shot_all_reduce_(t)
    assert torch.equal(t, before)
    smr.barrier_test(hdl, num_blocks=32)
    hdl.barrier()
    hdl.check()
    from symm_mem_recipes_b200._ext import C
    # barrier slots are back to zero; the all-reduce epoch counters beyond them only ever grow
    assert int(hdl.get_signal_pad()[:C.FLAG_SLOTS_BASE].abs().sum()) == 0
    view = hdl.get_buffer(0, (16,), torch.bfloat16, storage_offset=64)
    assert torch.equal(view, t[64:80])


@pytest.mark.gpu
def test_bounded_wait_reports_and_device_survives():
    """A flag that nothing sets: the kernel gives up after ~20 ms, records a
    timeout status and returns; the context stays usable."""
    from symm_mem_recipes_b200 import ops
    from symm_mem_recipes_b200.errors import SymmMemTimeout
    from symm_mem_recipes_b200.parallel import symm_mem

    torch.cuda.set_device(0)
    flag = torch.zeros(4, dtype=torch.int32, device="cuda")
    ops.wait_flag(flag, 1, timeout_ms=20)
    with pytest.raises(SymmMemTimeout) as e:
        symm_mem.check_status("cuda:0")
    assert e.value.code == 3
    symm_mem.check_status("cuda:0")                  # record was cleared
    flag.fill_(1)
    ops.wait_flag(flag, 1, timeout_ms=20)            # satisfied at once
    symm_mem.check_status("cuda:0")
    x = torch.ones(1024, device="cuda")
    assert float(x.sum()) == 1024.0


def _ar_worker(rank, world_size, numel):
    import torch.distributed as dist

    import symm_mem_recipes_b200 as smr
    from symm_mem_recipes_b200._ext import C
    from symm_mem_recipes_b200.parallel import symm_mem

    dev = torch.device("cuda", rank)
    failures = []
    t = symm_mem.empty(numel, dtype=torch.bfloat16, device=dev)
    hdl = symm_mem.rendezvous(t)
    srcs = [seeded_normal_bf16(numel, r) for r in range(world_size)]
    ordered = C.oracle_ordered_sum_bf16(srcs)
    fp32 = torch.stack([s.float() for s in srcs]).sum(0)

    # pointer-table round trip: every rank reads every peer's payload
    t.copy_(srcs[rank].to(dev))
    hdl.barrier()
    for r in range(world_size):
        peer = hdl.get_buffer(r, (numel,), torch.bfloat16).cpu()
        if not torch.equal(peer, srcs[r]):
            failures.append(f"peer view of rank {r} differs")
    hdl.barrier()

    out = smr.one_shot_all_reduce(t, exit_barrier=True)
    hdl.check()
    if not torch.equal(out.cpu().view(torch.int16), ordered.view(torch.int16)):
        failures.append("one_shot differs from the ordered-sum oracle")

    smr.two_shot_all_reduce_(t)
    hdl.check()
    if not torch.equal(t.cpu().view(torch.int16), ordered.view(torch.int16)):
        failures.append("two_shot differs from the ordered-sum oracle")

    # low-latency push kernel: plain (non-symmetric) input, several calls, then in place
    n_ll = min(numel, 65536)
    plain = srcs[rank][:n_ll].to(dev)
    ordered_ll = C.oracle_ordered_sum_bf16([s[:n_ll] for s in srcs])
    for _ in range(3):
        out_ll = smr.low_latency_all_reduce(plain)
        hdl.check()
        if not torch.equal(out_ll.cpu().view(torch.int16), ordered_ll.view(torch.int16)):
            failures.append("low_latency differs from the ordered-sum oracle")
    smr.low_latency_all_reduce(plain, out=plain)
    hdl.check()
    if not torch.equal(plain.cpu().view(torch.int16), ordered_ll.view(torch.int16)):
        failures.append("in-place low_latency differs from the ordered-sum oracle")

    if hdl.has_multicast:
        hdl.barrier()
        t.copy_(srcs[rank].to(dev))
        hdl.barrier()
        smr.multimem_all_reduce_(t)
        hdl.check()
        got = t.cpu().float()
        # one rounding of the fp32 sum: within one bf16 ulp of it
        tol = fp32.abs() * 2.0 ** -7 + 1e-6
        if not bool(((got - fp32).abs() <= tol).all()):
            failures.append("multimem differs from the fp32-accumulate oracle")
        mc = hdl.get_multicast_buffer((8,), torch.bfloat16)
        assert mc.data_ptr() == hdl.multicast_ptr
    elif world_size > 1:
        failures.append("no multicast mapping on an NVSwitch machine")

    # dispatcher: in place, whichever kernel it picks
    hdl.barrier()
    t.copy_(srcs[rank].to(dev))
    hdl.barrier()
    picked = smr.ops.choose_algo(numel * 2, world_size, hdl.has_multicast)
    smr.all_reduce(t, "auto")
    hdl.check()
    if picked == "multimem":                  # in-switch fp32 summation, one rounding
        tol = fp32.abs() * 2.0 ** -7 + 1e-6
        if not bool(((t.cpu().float() - fp32).abs() <= tol).all()):
            failures.append("all_reduce(auto) -> multimem is off")
    elif not torch.equal(t.cpu().view(torch.int16), ordered.view(torch.int16)):
        # every other kernel adds bf16 values in rank order: the oracle's bits
        failures.append(f"all_reduce(auto) -> {picked} differs from the ordered-sum oracle")

    # barrier stress, 10^4 barriers over four grid sizes: the pad must be all zero afterwards
    for blocks in (1, 7, 32, 148):
        for _ in range(2500):
            smr.barrier_test(hdl, num_blocks=blocks)
    hdl.barrier()
    hdl.check()
    if int(hdl.get_signal_pad()[:C.FLAG_SLOTS_BASE].abs().sum()) != 0:
        failures.append("barrier slots are not zero after the barrier stress")
    dist.barrier()        # not through the pad: a fast rank's next pad barrier must not race the read above
    hdl.barrier()
    torch.cuda.synchronize()
    assert not failures, failures


@pytest.mark.gpu
@pytest.mark.multigpu(2)
@pytest.mark.parametrize("numel", [8192, 1 << 20])
def test_all_reduce_2gpu(numel):
    spawn_ranks(_ar_worker, 2, "nccl", (numel,))


@pytest.mark.gpu
@pytest.mark.multigpu(4)
def test_all_reduce_4gpu():
    spawn_ranks(_ar_worker, 4, "nccl", (1 << 16,))


@pytest.mark.gpu
@pytest.mark.multigpu(8)
def test_all_reduce_8gpu():
    spawn_ranks(_ar_worker, 8, "nccl", (1 << 18,))


def _counting_barriers_worker(rank, world_size, numel):
    """The epoch barrier and the NVLS (multimem.red) barrier as kernels of their
    own, then the multimem all-reduce on the same pad."""
    import symm_mem_recipes_b200 as smr
    from symm_mem_recipes_b200.ops.config import AllReduceConfig
    from symm_mem_recipes_b200.parallel import symm_mem

    dev = torch.device("cuda", rank)
    failures = []
    t = symm_mem.empty(numel, dtype=torch.bfloat16, device=dev)
    hdl = symm_mem.rendezvous(t)
    kinds = ["epoch"] + (["nvls"] if hdl.has_multicast else [])
    for kind in kinds:
        for blocks in (1, 7, 32, 148):
            for _ in range(20):
                smr.barrier_test(hdl, num_blocks=blocks, kind=kind, timeout_ms=2000)
        hdl.barrier()
        hdl.check()
    if hdl.has_multicast:
        srcs = [seeded_normal_bf16(numel, r) for r in range(world_size)]
        results = []
        for blocks in (16, 4, 8, 16):        # after the barrier tests, at several CTA counts
            hdl.barrier()
            t.copy_(srcs[rank].to(dev))
            hdl.barrier()
            smr.multimem_all_reduce_(t, config=AllReduceConfig(multimem_max_blocks=blocks, timeout_ms=2000))
            hdl.check()
            results.append(t.clone())
        ref = results[0].float()
        for r in results[1:]:
            # the switch's summation order is its own: within one bf16 ulp
            if not bool(((r.float() - ref).abs() <= ref.abs() * 2.0 ** -7 + 1e-6).all()):
                failures.append("multimem all-reduce differs between CTA counts")
    elif world_size > 1:
        failures.append("no multicast mapping on an NVSwitch machine")
    torch.cuda.synchronize()
    assert not failures, failures


@pytest.mark.gpu
@pytest.mark.multigpu(2)
def test_counting_barriers_2gpu():
    spawn_ranks(_counting_barriers_worker, 2, "nccl", (1 << 20,))


def _leaving_rank_worker(rank, world_size):
    """A rank stops taking part between steps (nothing of it in flight); the
    others learn of it on the host and do not launch.  The leaver stays alive
    until the survivors are done, so no mapping of a dead process is involved."""
    import time

    import symm_mem_recipes_b200 as smr
    from symm_mem_recipes_b200.parallel import symm_mem
    from symm_mem_recipes_b200.parallel.health import Heartbeat, PeerLost
    from symm_mem_recipes_b200.parallel.store import _store_of

    dev = torch.device("cuda", rank)
    store = _store_of(None)
    hb = Heartbeat(interval_s=0.05)
    hb.wait_for_all(timeout_s=60)
    t = symm_mem.empty(1 << 16, dtype=torch.bfloat16, device=dev)
    t.copy_(seeded_normal_bf16(1 << 16, rank).to(dev))
    hdl = symm_mem.rendezvous(t)
    assert not hdl.has_multicast                 # plain peer loads only in this test
    for _ in range(3):                           # all present: check passes, kernels run
        hb.check(max_age_s=10.0)
        smr.one_shot_all_reduce(t, exit_barrier=True)
        hdl.check()
    torch.cuda.synchronize()
    torch.distributed.barrier()
    leaver = world_size - 1
    if rank == leaver:
        hb.stop()                                # announces the leave; launches nothing from here on
        store.wait([f"leaving_test/done/{r}" for r in range(world_size - 1)])
        return
    lost = None
    deadline = time.time() + 30
    while lost is None and time.time() < deadline:
        try:
            hb.check(max_age_s=10.0)             # what a serving loop calls before every launch
            time.sleep(0.02)
        except PeerLost as e:
            lost = e
    ok = lost is not None and lost.rank == leaver
    # the device is untouched and healthy: a local kernel still runs, the status record is clean
    x = torch.ones(1024, device=dev)
    ok = ok and float(x.sum()) == 1024.0
    hdl.check()
    hb.stop(leaving=False)
    store.set(f"leaving_test/done/{rank}", "1")
    assert ok, f"expected PeerLost for rank {leaver}, got {lost!r}"


@pytest.mark.gpu
@pytest.mark.multigpu(2)
def test_rank_leaving_between_steps_is_noticed_before_the_next_launch(monkeypatch):
    monkeypatch.setenv("NCCL_NVLS_ENABLE", "0")
    monkeypatch.setenv("SMR_DISABLE_MULTICAST", "1")
    spawn_ranks(_leaving_rank_worker, 2, "nccl", ())


def _compat_gpu_worker(rank, world_size):
    from symm_mem_recipes_b200 import compat
    from symm_mem_recipes_b200.parallel import symm_mem

    dev = torch.device("cuda", rank)
    rows, cols, splits = 256, 1024, 2
    inp = symm_mem.empty(rows, cols, dtype=torch.bfloat16, device=dev)
    inp.copy_(seeded_normal_bf16(rows * cols, rank).view(rows, cols).to(dev))
    symm_mem.rendezvous(inp).barrier()
    out = torch.zeros(rows * world_size, cols, dtype=torch.bfloat16, device=dev)
    progress = torch.zeros(world_size * splits, dtype=torch.int32, device=dev)
    compat.all_gather_with_progress(out, inp, progress, splits)    # contiguous peer copies: copy engine
    torch.cuda.synchronize()
    assert bool((progress == 1).all())
    for r in range(world_size):
        want = seeded_normal_bf16(rows * cols, r).view(rows, cols)
        assert torch.equal(out[r * rows:(r + 1) * rows].cpu(), want)
    symm_mem.check_status(dev)


@pytest.mark.gpu
@pytest.mark.multigpu(2)
def test_upstream_all_gather_with_progress_2gpu():
    spawn_ranks(_compat_gpu_worker, 2, "nccl", ())


def _signals_gpu_worker(rank, world_size):
    from symm_mem_recipes_b200.parallel import symm_mem

    dev = torch.device("cuda", rank)
    t = symm_mem.empty(1 << 16, dtype=torch.float32, device=dev)
    hdl = symm_mem.rendezvous(t)
    nxt, prv = (rank + 1) % world_size, (rank - 1) % world_size
    for it in range(20):                       # ring: write, signal the next rank, wait for the previous, read it
        t.fill_(float(100 * it + rank))
        hdl.put_signal(nxt, channel=3, timeout_ms=2000)
        hdl.wait_signal(prv, channel=3, timeout_ms=2000)
        got = hdl.get_buffer(prv, (1 << 16,), torch.float32).clone()
        hdl.barrier(channel=1)
        assert float(got[0]) == float(100 * it + prv) and float(got[-1]) == float(100 * it + prv)
    hdl.check()
    assert int(hdl.get_signal_pad().abs().sum()) == 0
    assert len(hdl.buffer_ptrs) == world_size and hdl.buffer_ptrs[rank] == t.data_ptr()


@pytest.mark.gpu
@pytest.mark.multigpu(2)
def test_one_to_one_signals_2gpu():
    spawn_ranks(_signals_gpu_worker, 2, "nccl", ())
