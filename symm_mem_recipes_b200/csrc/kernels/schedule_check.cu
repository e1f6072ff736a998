// Host-side self-checks of the scheduling arithmetic that the fused kernels
// rely on for progress: the M schedule, the just-in-time push of the own
// shard, and the split-K tail.  The functions under test are the very ones
// the kernels call (`__host__ __device__` in ag_matmul_common.cuh); the checks
// run on the CPU and need no GPU.
#include <vector>

#include "ag_matmul_common.cuh"
#include "matmul_rs_common.cuh"

namespace smr {

using namespace agmm;

// 0 = all invariants hold, otherwise a code saying which one failed:
//  1 the M schedule is not a permutation of the blocks / `local` is wrong
//  2 a tile could wait for a piece that no CTA has been told to push yet
//  3 not every piece is pushed by the end
//  4 the column-panel tile order does not visit every tile exactly once
static int check_push_schedule_with_lead(int world_size, int rank, int blocks_per_rank, int n_tiles_n, int n_units,
                                         int pos_per_tile, int pieces, int lead, int panel_w) {
  AgMatmulParams p{};
  p.mode = 2;
  p.world_size = world_size;
  p.rank = rank;
  p.blocks_per_rank = blocks_per_rank;
  p.n_blocks_m = world_size * blocks_per_rank;
  p.n_tiles_n = n_tiles_n;
  p.panel_w = panel_w;
  p.lead = lead;
  p.pieces = pieces;
  // 1. permutation + locality
  std::vector<int> seen(p.n_blocks_m, 0);
  for (int mi = 0; mi < p.n_blocks_m; ++mi) {
    bool local = false;
    int blk = scheduled_block(p, mi, local);
    if (blk < 0 || blk >= p.n_blocks_m || seen[blk]++) return 1;
    if (local != (blk / blocks_per_rank == rank)) return 1;
  }
  // 2. before any CTA blocks in the epilogue of round j, every piece of every remote block that a tile
  //    of rounds <= j reads has been assigned for pushing (pieces with index < the limit of round j)
  const int m_tiles = (p.n_blocks_m + pos_per_tile - 1) / pos_per_tile;
  const int total_tiles = m_tiles * n_tiles_n;
  const int rounds = (total_tiles + n_units - 1) / n_units;
  {
    std::vector<int> visited((size_t)total_tiles, 0);
    for (int t = 0; t < total_tiles; ++t) {
      int row, ni;
      tile_coords(p, m_tiles, t, row, ni);
      if (row < 0 || row >= m_tiles || ni < 0 || ni >= n_tiles_n || visited[(size_t)row * n_tiles_n + ni]++) return 4;
    }
  }
  for (int j = 0; j < rounds; ++j) {
    const int limit = pieces_needed_through_round(p, j + 1, n_units, pos_per_tile);
    const long long t_end = (long long)(j + 1) * n_units;
    for (int t = 0; t < total_tiles && t < t_end; ++t) {
      for (int c = 0; c < pos_per_tile; ++c) {
        int row, ni;
        tile_coords(p, m_tiles, t, row, ni);
        const int mi = row * pos_per_tile + c;
        if (mi >= p.n_blocks_m) continue;
        bool local = false;
        const int blk = scheduled_block(p, mi, local);
        if (local) continue;
        const int k = blk % blocks_per_rank;          // index of the block inside its shard
        if ((k + 1) * pieces > limit) return 2;
      }
    }
  }
  // 3. the last limit covers the whole shard
  if (pieces_needed_through_round(p, rounds, n_units, pos_per_tile) < blocks_per_rank * pieces) return 3;
  return 0;
}

// Every number of own blocks scheduled first that a launcher may pick (none, a few, the first round of
// tiles (the default), the whole shard), for one column panel and for narrower ones (an even split in
// two, an uneven one with a narrow last panel, single-tile panels).
int check_push_schedule(int world_size, int rank, int blocks_per_rank, int n_tiles_n, int n_units,
                        int pos_per_tile, int pieces) {
  const int widths[4] = {n_tiles_n, (n_tiles_n + 1) / 2, n_tiles_n > 3 ? n_tiles_n - n_tiles_n / 3 : n_tiles_n, 1};
  for (int panel_w : widths) {
    const int first_round = pos_per_tile * ((n_units + panel_w - 1) / panel_w);
    const int leads[4] = {0, blocks_per_rank < 4 ? blocks_per_rank : 4,
                          first_round < blocks_per_rank ? first_round : blocks_per_rank, blocks_per_rank};
    for (int lead : leads) {
      int rc = check_push_schedule_with_lead(world_size, rank, blocks_per_rank, n_tiles_n, n_units, pos_per_tile,
                                             pieces, lead, panel_w);
      if (rc != 0) return rc;
    }
  }
  return 0;
}

// 0 = every (tile, K block) is computed exactly once and every pair gets at most one tail unit.
int check_pair_work(int total_tiles, int n_pairs, int k_blocks, int tail_tiles, int tail_splits) {
  AgMatmulParams p{};
  p.tail_tiles = tail_tiles;
  p.tail_splits = tail_splits;
  std::vector<int> cover((size_t)total_tiles * k_blocks, 0);
  for (int pair = 0; pair < n_pairs; ++pair) {
    int tail_units = 0;
    PairWork w;
    for (int i = 0; pair_work(p, pair, n_pairs, total_tiles, k_blocks, i, w); ++i) {
      if (w.tile < 0 || w.tile >= total_tiles || w.kb0 < 0 || w.kb1 > k_blocks) return 1;
      if (w.part >= 0 && ++tail_units > 1) return 2;
      for (int kb = w.kb0; kb < w.kb1; ++kb) cover[(size_t)w.tile * k_blocks + kb]++;
      if (i > total_tiles) return 3;
    }
  }
  for (int v : cover)
    if (v != 1) return 4;
  return 0;
}

// CTA-pair reduce-scatter kernel: over all pairs, both CTAs and all tiles, every (destination, row
// block, N tile) is produced exactly once, own rows last inside every column panel (a tile of the own
// rows waits for the peers' tiles of the same panel, which therefore all come earlier in every
// rank's order); entries past the end are skipped.
// 0 = holds; 1 = a tile is missing or doubled; 2 = inside a panel, a destination other than the own one
// follows it.
static int check_rs_pair_schedule_panel(int world_size, int rank, int blocks_per_rank, int n_tiles_n, int n_pairs,
                                        int panel_w);
int check_rs_pair_schedule(int world_size, int rank, int blocks_per_rank, int n_tiles_n, int n_pairs) {
  const int widths[4] = {n_tiles_n, (n_tiles_n + 1) / 2, n_tiles_n > 3 ? n_tiles_n - n_tiles_n / 3 : n_tiles_n, 1};
  for (int w : widths)
    if (int rc = check_rs_pair_schedule_panel(world_size, rank, blocks_per_rank, n_tiles_n, n_pairs, w)) return rc;
  return 0;
}
static int check_rs_pair_schedule_panel(int world_size, int rank, int blocks_per_rank, int n_tiles_n, int n_pairs,
                                        int panel_w) {
  rs::RsParams p{};
  p.panel_w = panel_w;
  p.world_size = world_size;
  p.rank = rank;
  p.blocks_per_rank = blocks_per_rank;
  p.n_tiles_n = n_tiles_n;
  const int n_rb = world_size * blocks_per_rank;
  const int total_tiles = ((n_rb + 1) / 2) * n_tiles_n;
  std::vector<int> cover((size_t)n_rb * n_tiles_n, 0);
  for (int pair = 0; pair < n_pairs; ++pair)
    for (int cta = 0; cta < 2; ++cta) {
      bool own_seen = false;
      int last_panel = -1;
      for (int t = pair; t < total_tiles; t += n_pairs) {
        int pr, ni;
        panel_tile_coords(n_tiles_n, panel_w, (n_rb + 1) / 2, t, pr, ni);
        if (ni / panel_w != last_panel) {
          last_panel = ni / panel_w;
          own_seen = false;
        }
        const int rb = 2 * pr + cta;
        if (rb >= n_rb) continue;
        int dest, mb;
        rs::row_block_coords(p, rb, dest, mb);
        if (dest < 0 || dest >= world_size || mb < 0 || mb >= blocks_per_rank) return 1;
        if (own_seen && dest != rank) return 2;
        own_seen = own_seen || dest == rank;
        cover[((size_t)dest * blocks_per_rank + mb) * n_tiles_n + ni]++;
      }
    }
  for (int v : cover)
    if (v != 1) return 1;
  return 0;
}

// Progress of the reduce-scatter kernel over all ranks at once, under a model that is stricter than the
// kernel: a CTA pair moves to its next tile only when both of its CTAs have finished the current one (the
// kernel lets the MMA run one tile ahead); a tile of another rank's rows ships at once, a tile of the own
// rows finishes when all peers have shipped their tile of the same (row block, N tile).  Every pair of
// every rank is assumed resident (the launcher checks that).  0 = every tile of every rank finishes;
// 1 = the ranks end up waiting for one another (a cycle of waits).
int check_rs_progress(int world_size, int blocks_per_rank, int n_tiles_n, int n_pairs, int panel_w) {
  const int n_rb = world_size * blocks_per_rank;
  const int n_rows = (n_rb + 1) / 2;
  const int total_tiles = n_rows * n_tiles_n;
  if (panel_w < 1 || panel_w > n_tiles_n) panel_w = n_tiles_n;
  std::vector<rs::RsParams> params(world_size);
  for (int r = 0; r < world_size; ++r) {
    params[r].world_size = world_size;
    params[r].rank = r;
    params[r].blocks_per_rank = blocks_per_rank;
    params[r].n_tiles_n = n_tiles_n;
    params[r].panel_w = panel_w;
  }
  std::vector<int> arrived((size_t)world_size * blocks_per_rank * n_tiles_n, 0);
  std::vector<int> next((size_t)world_size * n_pairs, 0);          // index of the pair's current tile in its own order
  std::vector<char> done((size_t)world_size * n_pairs * 2, 0);     // CTA c of the pair has finished the current tile
  bool moved = true;
  while (moved) {
    moved = false;
    for (int r = 0; r < world_size; ++r)
      for (int pair = 0; pair < n_pairs; ++pair) {
        const size_t slot = (size_t)r * n_pairs + pair;
        for (;;) {
          const int t = pair + next[slot] * n_pairs;
          if (t >= total_tiles) break;
          int pr, ni;
          panel_tile_coords(n_tiles_n, panel_w, n_rows, t, pr, ni);
          for (int c = 0; c < 2; ++c) {
            if (done[slot * 2 + c]) continue;
            const int rb = 2 * pr + c;
            if (rb >= n_rb) { done[slot * 2 + c] = 1; moved = true; continue; }
            int dest, mb;
            rs::row_block_coords(params[r], rb, dest, mb);
            int& count = arrived[((size_t)dest * blocks_per_rank + mb) * n_tiles_n + ni];
            if (dest != r) {
              ++count;                                             // shipped
              done[slot * 2 + c] = 1;
              moved = true;
            } else if (count == world_size - 1) {
              done[slot * 2 + c] = 1;                              // all partials are in: reduced
              moved = true;
            }
          }
          if (!(done[slot * 2] && done[slot * 2 + 1])) break;
          done[slot * 2] = done[slot * 2 + 1] = 0;
          ++next[slot];
          moved = true;
        }
      }
  }
  for (int r = 0; r < world_size; ++r)
    for (int pair = 0; pair < n_pairs; ++pair)
      if (pair + next[(size_t)r * n_pairs + pair] * n_pairs < total_tiles) return 1;
  return 0;
}

}  // namespace smr
