// smr_gemv_bf16_noalloc: a decode GEMV for callers that must not allocate.
//
// This entry point has no counterpart in the upstream recipes.  It exists for
// hosts that drive the GPU from a context in which device allocation is off
// limits: a serving loop that has handed all of its memory to a pool and
// forbids cudaMalloc on the hot path, a plugin loaded into someone else's
// process that may not touch that process's allocator, or code running between
// the begin and end of a region where allocation would synchronise the device.
// Such a caller cannot create the symmetric workspace that `gemv_all_reduce`
// sets up on first use, so the library carries what the kernel needs itself.
//
//     out[b, n] = sum_k x[b, k] * w[k, n]      bf16 in, fp32 accumulate, bf16 out
//
// on ONE GPU (a world of one: nothing crosses NVLink), computed by the same
// tcgen05 kernel as `gemv_all_reduce`.  The global memory that kernel needs
// besides its operands — the table through which it finds its workspace and
// the status record its bounded waits report into — sits in a file-scope
// `static __device__` array of SMR_GEMV_NOALLOC_SCRATCH_BYTES (4 KiB) that
// every GPU loading the library holds until the process exits.  (The K splits
// of a column tile meet in shared memory; with one rank nothing else is parked
// in global memory.)
//
// What the caller must know:
//  * Limits: 1 <= batch <= SMR_GEMV_NOALLOC_MAX_BATCH, N <= SMR_GEMV_NOALLOC_MAX_N,
//    N % 8 == 0, K % 8 == 0, K >= 8.  Anything else is refused with a non-zero
//    return value and a message in `err` (when `err` is not NULL); nothing is
//    launched.
//  * x is [batch, K], w is [K, N], out is [batch, N]; contiguous bf16 in device
//    memory of the current device, 16-byte aligned.  The caller owns them.
//  * The first call on each device resolves the device address of the array
//    (cudaGetSymbolAddress) and writes one pointer into it with a blocking
//    copy.  Make that first call before any stream capture and outside any
//    region that must not synchronise.  Later calls only enqueue work on
//    `stream`.
//  * No call allocates: no cudaMalloc, no cudaFree, no framework allocator.
//  * All calls on a device share the one array, which keeps whatever the
//    previous call left in it (the pointer table, and the status record of a
//    failed call until it is queried).  Two calls that overlap in time on the
//    same GPU — different streams, or two host threads — would share the status
//    record; order them on one stream or with events.
//  * A return value of 0 means "enqueued", not "done".  The CTAs of the kernel
//    wait for one another (the K splits of a column tile form a cluster), each
//    wait bounded at 2 s.  If a wait runs out the kernel records why in the
//    status record and returns with `out` UNWRITTEN.
//    smr_gemv_bf16_noalloc_status() reads that record; call it wherever you
//    would otherwise synchronise.
//
// Returns 0 when the kernel was enqueued, otherwise:
//   1 a size is outside the limits above      2 a pointer is null or misaligned
//   3 a CUDA call failed (the message names it)
#pragma once
#include <stddef.h>

#define SMR_GEMV_NOALLOC_MAX_BATCH 16
#define SMR_GEMV_NOALLOC_MAX_N 8192
#define SMR_GEMV_NOALLOC_SCRATCH_BYTES 4096

#ifdef __cplusplus
extern "C" {
#endif

// `stream` is a cudaStream_t passed as a pointer (NULL = the default stream).
// `err`/`err_len`: optional buffer that receives a NUL-terminated message on failure.
int smr_gemv_bf16_noalloc(const void* x, const void* w, void* out, int batch, int K, int N,
                          void* stream, char* err, int err_len);

// Waits for `stream` (cudaStreamSynchronize), then reads the status word of the current
// device's scratch array: 0 = every call since the last query ran to its end; 4 = a bounded
// wait ran out in one of them and that call left `out` unwritten (the word is cleared, so the
// failure is reported once); 3 = a CUDA call failed.  `record` (optional, 6 words) receives
// {code, rank, block, peer, where, aux} of the kernel's Status record.  Allocates nothing.
int smr_gemv_bf16_noalloc_status(void* stream, unsigned int record[6], char* err, int err_len);

#ifdef __cplusplus
}
#endif
