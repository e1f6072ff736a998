// Order in which the persistent GEMM kernels walk their output tiles, shared by the fused
// all-gather + GEMM and GEMM + reduce-scatter kernels and their host-side schedule checks.
//
// Tiles are walked in column panels of `panel_w` N tiles; inside a panel row by row (N fastest), so
// that the B rows of a panel (panel_w x BN x K elements) stay in L2 while every row block of A
// streams past them once.  With one panel this is the plain row-major order.  Upstream reaches the
// same end with a grouped-M swizzle of pid (symm_mem_recipes/triton_all_gather_matmul.py:143-155);
// here M is the streamed dimension because its order is fixed by the collective (arrival order of
// the gathered blocks, destination order of the scattered ones).
#pragma once
#include <cstddef>

namespace smr {

__host__ __device__ __forceinline__ void panel_tile_coords(int n_tiles_n, int panel_w, int n_rows, int t, int& row,
                                                           int& ni) {
  const int per_panel = n_rows * panel_w;
  const int panel = t / per_panel;
  const int within = t - panel * per_panel;
  const int n0 = panel * panel_w;
  int w = n_tiles_n - n0;            // the last panel may be narrower
  if (w > panel_w) w = panel_w;
  row = within / w;
  ni = n0 + within - row * w;
}

// Panel width for a B of `n_tiles_n` tiles of `tile_bytes` each: the widest even split whose panel
// stays under `budget` bytes.  kPanelBudgetHalfL2: each die keeps its own copy of what it reads
// (measured DRAM reads are twice the operands), so half of the 126 MB is what a panel can count on.
constexpr size_t kPanelBudgetHalfL2 = (size_t)60 << 20;
constexpr size_t kPanelBudgetL2 = (size_t)120 << 20;
__host__ __device__ __forceinline__ int pick_panel_w(int n_tiles_n, size_t tile_bytes,
                                                     size_t budget = kPanelBudgetHalfL2) {
  int fit = (int)(budget / (tile_bytes ? tile_bytes : 1));
  if (fit < 1) fit = 1;
  if (fit >= n_tiles_n) return n_tiles_n;
  const int panels = (n_tiles_n + fit - 1) / fit;
  return (n_tiles_n + panels - 1) / panels;
}

}  // namespace smr
