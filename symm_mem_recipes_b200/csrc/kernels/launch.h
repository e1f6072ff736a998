// C launchers of every kernel in the library.  They take raw device pointers
// and a stream, include no framework header, and return a cudaError_t-style
// int (0 = launched).  The Python bindings and the C ABI both go through them.
#pragma once
#include <cuda_runtime_api.h>
#include <stdint.h>

#include "../device/status.h"

namespace smr {

// Pointers a kernel needs to reach its peers; all tables live in device memory.
struct PeerView {
  void* const* buffers;        // [world_size] payload base of every rank (mapped locally)
  uint32_t* const* pads;       // [world_size] signal-pad base of every rank
  void* multicast;             // multicast payload base or nullptr
  int rank;
  int world_size;
};

// The same addresses by value (kernel parameters), for latency-bound kernels that cannot afford a
// dependent load from the tables before their first remote access; worlds of up to 8 ranks.
struct PeerPtrs {
  void* buffers[8];
  uint32_t* pads[8];
};

// ---- barrier ---------------------------------------------------------------
// `kind`: 0 = blockwise_barrier (CAS protocol, pad returns to zero), 1 = epoch barrier (one store per
// peer, counters only grow), 2 = NVLS barrier (one multimem.red per rank; needs a multicast mapping).
int launch_barrier_test(const PeerView& pv, int num_blocks, int threads, uint64_t timeout_ns,
                        Status* status, cudaStream_t stream, int kind = 0);
int launch_channel_barrier(const PeerView& pv, int channel, uint64_t timeout_ns, Status* status,
                           cudaStream_t stream);
// One-to-one signalling on a channel (the two halves of the channel barrier): `put_signal` raises
// this rank's slot on `dst` (release; waits while an earlier signal is unconsumed), `wait_signal`
// consumes `src`'s signal on this rank (acquire).  Stream-ordered, bounded, status on expiry.
int launch_put_signal(const PeerView& pv, int dst, int channel, uint64_t timeout_ns, Status* status,
                      cudaStream_t stream);
int launch_wait_signal(const PeerView& pv, int src, int channel, uint64_t timeout_ns, Status* status,
                       cudaStream_t stream);
// Waits on a flag nothing sets unless `*flag >= target`; used to prove that a
// timed-out wait returns an error status and leaves the device usable.
int launch_wait_flag(const uint32_t* flag, uint32_t target, uint64_t timeout_ns, int rank,
                     Status* status, cudaStream_t stream);

// ---- all-reduce (bf16) -----------------------------------------------------
// `offset_bytes` is the offset of the tensor inside the symmetric payload.
// `write_back` (needs exit_barrier): after the exit barrier the sum also replaces this
// rank's symmetric input, i.e. the in-place form used by the dispatcher.
int launch_one_shot_all_reduce(const PeerView& pv, const PeerPtrs& ptrs, size_t offset_bytes, void* out,
                               size_t numel, int max_blocks, bool exit_barrier, bool write_back,
                               uint64_t timeout_ns, Status* status, cudaStream_t stream);
// Low-latency (push, tagged words) all-reduce for small messages.  `pv` is the view of a
// symmetric workspace of ll_all_reduce_workspace_bytes(capacity_numel, WS); `in` / `out` are
// ordinary device buffers (they may be the same).
size_t ll_all_reduce_workspace_bytes(size_t max_numel, int world_size);
int launch_ll_all_reduce(const PeerView& pv, const void* in, void* out, size_t numel, size_t capacity_numel,
                         int max_blocks, uint64_t timeout_ns, Status* status, cudaStream_t stream);
int launch_two_shot_all_reduce(const PeerView& pv, size_t offset_bytes, size_t numel,
                               int max_blocks, uint64_t timeout_ns, Status* status,
                               cudaStream_t stream);
int launch_multimem_all_reduce(const PeerView& pv, size_t offset_bytes, size_t numel,
                               int max_blocks, uint64_t timeout_ns, Status* status,
                               cudaStream_t stream);

// ---- all_gather_matmul (tcgen05 GEMM on CTA pairs + in-kernel all-gather) ---
struct AgMatmulArgs {
  const void* a_local;   // own A shard [rows_per_rank, K] (all of A [M, K] when mode == 0)
  const void* b;         // [N, K] bf16, K-major
  void* c;               // [M, N] bf16
  int M, N, K;
  // 0 or 2: bf16.  1: A, B, C and a_out hold fp8 e4m3 (fp32 accumulation, no scale factors,
  // as upstream's FP8_OUTPUT path); N and K multiples of 16.
  int elem_bytes;
  // 0: C[M, N] = A B^T.  1 (bf16, block_n 256, N % 256 == 0): B's rows are interleaved
  // in groups of 128 (gate rows, then the matching up rows) and C[M, N / 2] = SiLU(gate) * up.
  int epilogue;
  int block_n;           // 128, 192, 224 or 256
  int num_sms;           // CTAs to launch at most
  // communication: mode 0 = none (GEMM over a_local only), 2 = push (a_out symmetric; the
  // epilogue warps of the GEMM CTAs broadcast the own shard into every rank's a_out)
  int mode;
  int rank, world_size;
  int rows_per_rank;     // multiple of 128
  void* a_out;           // local gathered A [M, K]
  uint32_t* const* pads; // signal pads of the a_out allocation
  void* const* aout_buffers;  // device table: payload base of the a_out allocation on every rank
  void* aout_mc;              // its multicast base or nullptr
  size_t aout_offset;         // offset of a_out inside that payload
  uint32_t* local_pad;        // this rank's signal pad of the a_out allocation
  uint32_t barrier_block_base;
  uint64_t timeout_ns;
  Status* status;
  // optional scratch of the split-K tail (nullptr = never split)
  void* tail_scratch;
  size_t tail_scratch_bytes;
  uint32_t* tail_counters;
  size_t tail_counter_slots;
  // optional [num_sms][12] words of per-CTA timing (ag_trace:: in ag_matmul_common.cuh)
  uint64_t* trace;
  // push mode: own 128-row blocks multiplied before the first remote one (-1 = chosen by the launcher)
  int lead;
  // push mode pacing (0 = the launcher's choice): rounds of lookahead of the broadcast over the first need
  int push_ahead;
  // push mode: 0 = broadcast the shard with multimem.st when the allocation has a multicast mapping
  // (the shard leaves this GPU once; every rank, the sender included, receives it from the switch),
  // 1 = plain stores to every peer and a local copy (nothing loops back through the switch)
  int push_plain_stores;
  // push mode: pieces a 128-row block is cut into for the broadcast (0 = the launcher's choice); a block
  // has arrived when all of its pieces have, each pushed by another CTA
  int push_pieces;
  // N tiles per column panel of the tile order (0 = the launcher's choice: the widest even split of the
  // N tiles whose rows of B stay in L2)
  int panel_w;
};
int launch_ag_matmul_2cta(const AgMatmulArgs& args, cudaStream_t stream);

// Host-side checks of the kernels' scheduling arithmetic (schedule_check.cu); 0 = invariants hold.
int check_push_schedule(int world_size, int rank, int blocks_per_rank, int n_tiles_n, int n_units,
                        int pos_per_tile, int pieces);
int check_pair_work(int total_tiles, int n_pairs, int k_blocks, int tail_tiles, int tail_splits);
int check_rs_pair_schedule(int world_size, int rank, int blocks_per_rank, int n_tiles_n, int n_pairs);
int check_rs_progress(int world_size, int blocks_per_rank, int n_tiles_n, int n_pairs, int panel_w);

// ---- fused GEMV + all-reduce (decode) -------------------------------------
struct GemvArgs {
  const void* x;      // [batch, K] bf16, batch <= 16
  const void* w;      // [K, N] bf16 ([N, K] for the tcgen05 kernel with weights_nk)
  void* out;          // [batch, N] bf16
  int batch, K, N;
  PeerView pv;        // of the symmetric workspace
  size_t ws_offset;   // offset of the workspace inside the payload
  uint64_t timeout_ns;
  Status* status;
};
// Bytes of symmetric workspace for a batch tile (1, 2, 4, 8 or 16), N columns.
size_t gemv_workspace_bytes(int batch_tile, int N, int world_size, size_t* flags_offset,
                            size_t* inbox_offset, int* max_tiles);
int gemv_batch_tile(int batch);   // smallest supported tile >= batch, -1 if none
int launch_gemv_all_reduce(const GemvArgs& args, cudaStream_t stream);
// Tensor-core (tcgen05, swap A/B) variant; its workspace layout differs.
// `tagged`: partials travel as {fp32, call number} words and are polled directly (no flags, no
// release fence); twice the inbox.  Meant for batch <= 4.
size_t gemv_tc_workspace_bytes(int N, int K, int world_size, int num_sms, size_t* flags_offset,
                               size_t* inbox_offset, int* tiles, int* ksplit, bool tagged = false,
                               size_t* counters_offset = nullptr);
// `weights_nk`: `args.w` is [N, K] (K contiguous), the layout of the prefill GEMMs' B operand.
int launch_gemv_all_reduce_tc(const GemvArgs& args, int num_sms, cudaStream_t stream, bool tagged = false,
                              bool weights_nk = false);

// ---- fused GEMM + reduce-scatter (prefill, row-parallel linear) --------------
struct MatmulRsArgs {
  const void* a;      // [M, K] bf16: all tokens, this rank's slice of the reduction dim
  const void* b;      // [N, K] bf16
  void* out;          // [M / WS, N] bf16: this rank's rows of the sum
  int M, N, K;
  PeerView pv;        // of the symmetric workspace (inbox)
  size_t inbox_offset;
  void* peer_base[16]; // host copy: workspace payload base of every rank as mapped here
  uint32_t* local_pad;
  int num_sms;
  uint64_t timeout_ns;
  Status* status;
  uint64_t* trace;     // optional [num_sms][4] %globaltimer stamps per CTA (start, entered, GEMM done, reduced)
  // all-reduce form: every rank ends up with the whole [M, N] sum in a SYMMETRIC output (`out` is unused);
  // each rank reduces its rows and broadcasts them (multimem.st when `ar_mc`, else stores to every peer)
  bool all_reduce;
  void* const* ar_peers;   // device table: payload base of the output allocation on every rank
  void* ar_mc;             // its multicast base or nullptr
  size_t ar_offset;        // offset of the output tensor inside that payload
  // N tiles per column panel of the tile order (0 = the widest even split whose rows of B stay in L2)
  int panel_w;
};
size_t matmul_rs_workspace_bytes(int M, int N);
int launch_matmul_reduce_scatter(const MatmulRsArgs& args, cudaStream_t stream);

// ---- rank-local layer glue (layer_glue.cu): bf16 data, fp32 math, one pass each ----
// out[rows, H] = RMSNorm(x (+ residual)) * w.  With `residual`, `sum_out` (optional) receives
// bf16(x + residual).  `sum_out` may be the buffer of `x` or of `residual`, `out` the buffer of `x`;
// `out` must not be the buffer of `sum_out` or `residual`.  H % 8 == 0, 16-byte aligned pointers.
int launch_rms_norm(const void* x, const void* residual, const void* w, void* sum_out, void* out, int rows, int H,
                    float eps, cudaStream_t stream);
// Rotary embedding in place on heads [0, n_heads) of every row (`row_stride` elements per row);
// token t is at position pos0 + t % seq, with pos0 read from `pos_dev` on the device when that is
// not null (graph-captured decode).  head_dim % 16 == 0.
int launch_rope_inplace(void* qkv, long long tokens, int row_stride, int n_heads, int head_dim, int seq, int pos0,
                        const int* pos_dev, float theta, int num_sms, cudaStream_t stream);
// out[rows, F] = SiLU(gate_up[:, :F]) * gate_up[:, F:].  F % 8 == 0.
int launch_silu_mul(const void* gate_up, void* out, long long rows, int F, int num_sms, cudaStream_t stream);
// Attention of one decode step: qkv [batch, (hq + 2 hkv) * head_dim] (new token, keys already rotated),
// caches [batch, s_max, hkv, head_dim]; writes the new key / value into the caches at the position
// and out [batch, hq * head_dim].  The position is `pos0`, or read from `pos_dev` on the device.
// `scratch`: decode_attention_scratch_bytes(...) bytes, zero-filled once; head_dim 64 or 128,
// hq / hkv <= 8.
size_t decode_attention_scratch_bytes(int batch, int hkv, int head_dim, int s_max, int* n_split_out);
// `rope_theta` != 0: the new token's queries and key are taken unrotated and rotated in the kernel.
int launch_decode_attention(const void* qkv, void* k_cache, void* v_cache, void* out, void* scratch,
                            size_t scratch_bytes, int batch, int hq, int hkv, int head_dim, int s_max, int pos0,
                            const int* pos_dev, float rope_theta, cudaStream_t stream);

}  // namespace smr
