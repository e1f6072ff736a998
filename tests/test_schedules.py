"""The scheduling arithmetic of the fused kernels, run on the CPU.

The kernels decide when a CTA pushes which piece of its shard, and how the
last wave of GEMM tiles is cut along K, with small integer functions.  If those
were wrong a kernel would wait for data nobody sends (its bounded waits would
then report a timeout).  The same functions are compiled for the host and
checked here over many shapes, including the ones the benchmarks use.
"""
import itertools

import pytest

from symm_mem_recipes_b200._ext import C


def _pieces(K):
    block_vecs = 128 * K * 2 // 16
    return 16 if block_vecs >= 8192 else (4 if block_vecs >= 1024 else 1)


@pytest.mark.parametrize("ws", [2, 4, 8])
def test_push_schedule_headline_shape(ws):
    # M = 16384 gathered rows, N = 3584 (14 tiles of 256), K = 8192, 148 CTAs / 74 pairs
    bpr = 16384 // ws // 128
    for rank in range(ws):
        assert C.check_push_schedule(ws, rank, bpr, 14, 148, 1, _pieces(8192)) == 0
        assert C.check_push_schedule(ws, rank, bpr, 14, 74, 2, _pieces(8192)) == 0


def test_push_schedule_many_shapes():
    bad = []
    for ws, bpr, n_tiles_n, units, pieces in itertools.product(
            (2, 3, 4, 8), (1, 2, 3, 5, 16, 32), (1, 2, 5, 14, 28), (1, 2, 7, 74, 148), (1, 4, 16)):
        for pos in (1, 2):
            for rank in {0, ws - 1, ws // 2}:
                rc = C.check_push_schedule(ws, rank, bpr, n_tiles_n, units, pos, pieces)
                if rc != 0:
                    bad.append((ws, rank, bpr, n_tiles_n, units, pos, pieces, rc))
    assert not bad, bad[:10]


def test_decoder_layer_shapes():
    # QKV (N = 1280 -> 5 tiles) and gate/up (N = 7168 -> 28 tiles) at TP8, 32768 tokens
    for n_tiles_n in (5, 28):
        for rank in range(8):
            assert C.check_push_schedule(8, rank, 32, n_tiles_n, 74, 2, 16) == 0


@pytest.mark.parametrize("ws,pieces", [(2, 16), (4, 32), (8, 64), (8, 256)])
def test_push_schedule_fine_pieces(ws, pieces):
    """The piece counts the launcher picks for small shards (about six pieces per CTA over the shard)."""
    bpr = 16384 // ws // 128
    for rank in range(ws):
        assert C.check_push_schedule(ws, rank, bpr, 14, 74, 2, pieces) == 0


def test_split_k_tail_covers_every_tile_once():
    # headline: 896 pair tiles on 74 pairs -> 8 tail tiles cut in 8
    assert C.check_pair_work(896, 74, 128, 8, 8) == 0
    assert C.check_pair_work(896, 74, 128, 0, 1) == 0          # tail off
    bad = []
    for total, pairs, kb in itertools.product((1, 2, 9, 10, 75, 224, 896, 1000), (1, 4, 37, 74), (1, 7, 16, 128)):
        if pairs > total:
            continue
        rem = total % pairs
        configs = [(0, 1)]
        if rem > 0 and rem * 2 <= pairs:
            s = pairs // rem
            s = 8 if s >= 8 else (4 if s >= 4 else 2)
            if kb >= 2 * s:
                configs.append((rem, s))
        for tail, splits in configs:
            rc = C.check_pair_work(total, pairs, kb, tail, splits)
            if rc != 0:
                bad.append((total, pairs, kb, tail, splits, rc))
    assert not bad, bad[:10]


def test_reduce_scatter_pair_schedule_covers_every_tile_once():
    # decoder-layer shapes at TP8: 32 row blocks per rank, N = 8192 (32 tiles), 74 pairs
    for rank in range(8):
        assert C.check_rs_pair_schedule(8, rank, 32, 32, 74) == 0
    bad = []
    for ws, bpr, n_tiles_n, pairs in itertools.product((2, 3, 4, 8), (1, 2, 3, 5, 32), (1, 2, 5, 32), (1, 3, 74)):
        for rank in {0, ws - 1, ws // 2}:
            rc = C.check_rs_pair_schedule(ws, rank, bpr, n_tiles_n, pairs)
            if rc != 0:
                bad.append((ws, rank, bpr, n_tiles_n, pairs, rc))
    assert not bad, bad[:10]


def test_reduce_scatter_progress_with_column_panels():
    """All ranks simulated together: with the own rows last inside every column panel no cycle of waits
    can form, whatever the panel width, also when a CTA pair straddles two destinations (odd blocks per
    rank) and when there are fewer pairs than tiles in a panel."""
    bad = []
    for ws, bpr, n_tiles_n, pairs in itertools.product((2, 3, 4, 8), (1, 2, 3, 32), (1, 5, 32), (1, 3, 74)):
        for panel_w in {n_tiles_n, (n_tiles_n + 1) // 2, 1}:
            if C.check_rs_progress(ws, bpr, n_tiles_n, pairs, panel_w) != 0:
                bad.append((ws, bpr, n_tiles_n, pairs, panel_w))
    assert not bad, bad[:10]
