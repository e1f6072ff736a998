"""The signal-pad barrier protocol compiled for the host and hammered by
threads acting as ranks, plus the pure-Python pieces (dispatcher, config)."""
import pytest

from symm_mem_recipes_b200._ext import C


@pytest.mark.parametrize("world_size,blocks", [(2, 1), (4, 8), (8, 32)])
def test_barrier_completes_and_restores_the_pad(world_size, blocks):
    codes, pad_sum, skew = C.host_barrier_stress(world_size, blocks, 200, 5_000_000_000, -1)
    assert list(codes) == [0] * world_size
    assert pad_sum == 0            # zero-pad invariant: re-entrant without any host-side epoch
    assert skew <= 1               # nobody got past a barrier a peer had not reached


def test_barrier_with_a_dead_rank_times_out_everywhere():
    codes, _, _ = C.host_barrier_stress(4, 2, 10, 100_000_000, 2)
    live = [c for r, c in enumerate(codes) if r != 2]
    assert all(c in (1, 2) for c in live)    # send or wait timed out, nobody hung


@pytest.mark.parametrize("world_size,blocks", [(2, 1), (4, 8), (8, 24)])
def test_epoch_barrier_keeps_ranks_in_step(world_size, blocks):
    codes, skew = C.host_epoch_barrier_stress(world_size, blocks, 300, 5_000_000_000)
    assert list(codes) == [0] * world_size
    assert skew <= 1


def test_dispatcher_thresholds():
    from symm_mem_recipes_b200.ops import choose_algo
    from symm_mem_recipes_b200.ops.config import AllReduceConfig

    cfg = AllReduceConfig(ll_max_bytes=1 << 16, one_shot_max_bytes=1 << 18)
    assert choose_algo(4096, 8, True, cfg) == "low_latency"
    assert choose_algo((1 << 16) + 16, 8, True, cfg) == "one_shot"
    assert choose_algo(1 << 18, 8, True, cfg) == "one_shot"
    assert choose_algo((1 << 18) + 16, 8, True, cfg) == "multimem"
    assert choose_algo(1 << 26, 8, False, cfg) == "two_shot"
    assert choose_algo(1 << 26, 1, False, cfg) == "one_shot"   # nothing to reduce
    # the defaults depend on the world size: one-shot reads every peer's whole buffer
    dflt = AllReduceConfig(ll_max_bytes=256 * 1024, one_shot_max_bytes=-1, multimem_max_blocks=0)
    assert [choose_algo(1 << 20, ws, True, dflt) for ws in (2, 4, 8)] == ["two_shot", "two_shot", "multimem"]
    assert [choose_algo(1 << 22, ws, True, dflt) for ws in (2, 4, 8)] == ["two_shot", "multimem", "multimem"]
    assert [choose_algo(1 << 26, ws, True, dflt) for ws in (2, 4, 8)] == ["two_shot", "multimem", "multimem"]
    assert choose_algo(1 << 23, 4, False, dflt) == "two_shot"
    assert (dflt.multimem_blocks(4), dflt.multimem_blocks(8)) == (8, 8)
    assert AllReduceConfig(multimem_max_blocks=12).multimem_blocks(8) == 12


def test_block_n_choice():
    from symm_mem_recipes_b200.ops.ag_matmul import choose_block_n

    assert choose_block_n(16384, 3584, 148) == 256
    assert choose_block_n(256, 128, 148) == 128
    assert choose_block_n(256, 200, 148) == 224


def test_gemv_workspace_sizes_grow_with_world():
    a = C.gemv_tc_workspace_bytes(8192, 3584, 1, 148)
    b = C.gemv_tc_workspace_bytes(8192, 3584, 8, 148)
    assert b > a > 0
    assert C.matmul_rs_workspace_bytes(32768, 8192) == 32768 * 8192 * 2      # strip-major, no padding here
    assert C.matmul_rs_workspace_bytes(256, 328) == 2 * 2 * 4 * 16384          # padded to whole tiles


def test_status_decoding():
    from symm_mem_recipes_b200.errors import SymmMemTimeout, raise_for_status

    raise_for_status((0, 0, 0, 0, 0, 0))
    with pytest.raises(SymmMemTimeout) as e:
        raise_for_status((2, 3, 7, 5, 10, 0))
    assert (e.value.rank, e.value.block, e.value.peer) == (3, 7, 5)
    assert "never arrived" in str(e.value)


def test_one_gather_geometry_per_symmetric_allocation():
    import torch

    from symm_mem_recipes_b200.errors import SymmMemError
    from symm_mem_recipes_b200.ops.ag_matmul import _check_gather_geometry

    notes = {}
    _check_gather_geometry(notes, (0, 4096, 8192, torch.bfloat16))
    _check_gather_geometry(notes, (0, 4096, 8192, torch.bfloat16))        # same again: fine
    with pytest.raises(SymmMemError):
        _check_gather_geometry(notes, (0, 8192, 8192, torch.bfloat16))    # another M on the same counters
    _check_gather_geometry({}, (0, 8192, 8192, torch.bfloat16))           # a new allocation starts clean


def test_interleaved_gate_up_puts_matching_columns_in_one_tile():
    """Layout contract of the SwiGLU epilogue: tile ni of A @ B^T (256 columns)
    holds gate columns [128 ni, 128 ni + 128) followed by the same up columns."""
    import torch

    from symm_mem_recipes_b200.errors import SymmMemError
    from symm_mem_recipes_b200.ops.ag_matmul import interleave_gate_up

    F, K, M = 384, 32, 8
    g = torch.Generator().manual_seed(0)
    wg, wu, a = torch.randn(F, K, generator=g), torch.randn(F, K, generator=g), torch.randn(M, K, generator=g)
    b = interleave_gate_up(wg, wu)
    assert b.shape == (2 * F, K) and b.is_contiguous()
    full = a @ b.t()
    want = torch.nn.functional.silu(a @ wg.t()) * (a @ wu.t())
    got = torch.empty(M, F)
    for ni in range(2 * F // 256):
        tile = full[:, ni * 256:(ni + 1) * 256]
        got[:, ni * 128:(ni + 1) * 128] = torch.nn.functional.silu(tile[:, :128]) * tile[:, 128:]
    assert torch.allclose(got, want, atol=1e-5)
    with pytest.raises(SymmMemError):
        interleave_gate_up(wg[:100], wu[:100])


def test_dispatcher_sends_odd_world_sizes_through_the_switch():
    from symm_mem_recipes_b200.errors import SymmMemError
    from symm_mem_recipes_b200.ops.all_reduce import choose_algo

    for ws in (3, 5, 6, 7):
        assert choose_algo(4096, ws, True) == "multimem" and choose_algo(1 << 26, ws, True) == "multimem"
        with pytest.raises(SymmMemError, match="multicast"):
            choose_algo(4096, ws, False)
    assert choose_algo(4096, 8, True) == "low_latency" and choose_algo(4096, 1, False) == "one_shot"
