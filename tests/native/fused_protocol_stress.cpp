// Host model of the protocol the fused GEMM + collective kernels share (matmul_reduce_scatter, the
// push gather of all_gather_matmul), run under ThreadSanitizer with one thread per CTA:
//
//   * every CTA reads the call number from the header of its rank's pad (epoch = header[0] + 1);
//   * entry barrier among the CTAs with the same index on every rank (the CAS barrier on block slot
//     1024 + index): "every rank has entered this call", which by stream order means that every
//     rank has finished the previous call and its reads of the inboxes;
//   * producer: plain stores of a tile's payload into the destination rank's inbox, then a release
//     add on that tile's arrival counter in the destination's pad;
//   * consumer: acquire wait until the counter reads epoch x world size, then plain reads;
//   * the last CTA of the rank to finish publishes the call number.
//
// Counters count calls and nothing is reset; kernels of one rank do not overlap (stream order is a
// pthread barrier among the rank's CTA threads here).  argv: world size, CTAs per rank, calls,
// and "no-entry-barrier" to leave the entry barrier out, which must make the run fail (a data race
// between call n + 1's stores and call n's reads, or a wrong value).
#include <pthread.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <thread>
#include <vector>

#include "device/pad_layout.h"
#include "symm/host_backend.h"

using namespace smr;

namespace {
constexpr int kTilesPerRank = 6;     // not a multiple of the CTA count: uneven shares
constexpr int kWords = 32;           // payload words per (source, tile)

uint32_t value_of(int call, int src, int tile, int w) { return (uint32_t)(call * 1000003 + src * 8191 + tile * 131 + w); }
}  // namespace

// The exchange of the fused GEMV + all-reduce (gemv_allreduce*.cu): no barrier at all.  CTA (tile) of
// every rank stores its partial into slot [rank] of the tile's inbox on EVERY rank, in the half
// selected by the parity of the call number, then release-stores the call number into its flag there;
// it acquire-waits until all world-size flags of the tile (its own rank's copy) carry the call
// number and reads the partials in slot order.  Two halves suffice because a rank can be at most
// one call ahead of any other: it cannot finish call n + 1 without the partial that the slowest
// rank pushes only after its own call n has ended.  `one_parity` uses a single half, which must fail.
int gemv_model(int ws, int tiles, int calls, bool one_parity) {
  const int halves = one_parity ? 1 : 2;
  std::vector<std::vector<uint32_t>> inbox(ws, std::vector<uint32_t>((size_t)halves * tiles * ws * kWords, 0));
  std::vector<std::vector<uint32_t>> flags(ws, std::vector<uint32_t>((size_t)halves * tiles * ws, 0));
  std::vector<uint32_t> header(ws * 2, 0);                  // per rank: [0] call number, [1] CTAs done
  std::vector<pthread_barrier_t> stream(ws);
  for (auto& b : stream) pthread_barrier_init(&b, nullptr, tiles);
  std::vector<int> bad((size_t)ws * tiles, 0);
  std::vector<std::thread> th;
  for (int r = 0; r < ws; ++r)
    for (int t = 0; t < tiles; ++t)
      th.emplace_back([&, r, t] {
        int& failures = bad[(size_t)r * tiles + t];
        for (int call = 1; call <= calls; ++call) {
          const uint32_t epoch = __atomic_load_n(&header[r * 2], __ATOMIC_RELAXED) + 1u;
          if (epoch != (uint32_t)call) failures++;
          const size_t half = one_parity ? 0 : (epoch & 1u);
          for (int j = 1; j <= ws; ++j) {                       // own inbox last
            const int peer = (r + j) % ws;
            uint32_t* dst = inbox[peer].data() + ((half * tiles + t) * ws + r) * kWords;
            for (int w = 0; w < kWords; ++w) dst[w] = value_of(call, r, t, w);
          }
          for (int peer = 0; peer < ws; ++peer)
            __atomic_store_n(&flags[peer][(half * tiles + t) * ws + r], epoch, __ATOMIC_RELEASE);
          for (int s = 0; s < ws; ++s) {
            long spins = 0;
            while (__atomic_load_n(&flags[r][(half * tiles + t) * ws + s], __ATOMIC_ACQUIRE) != epoch) {
              // with one half a flag can be overwritten by the next call before it is seen: give up soon there
              if (++spins > (one_parity ? 200000L : 400000000L)) { failures++; break; }
              std::this_thread::yield();
            }
            const uint32_t* src = inbox[r].data() + ((half * tiles + t) * ws + s) * kWords;
            for (int w = 0; w < kWords; ++w)
              if (src[w] != value_of(call, s, t, w)) failures++;
          }
          const uint32_t done = __atomic_fetch_add(&header[r * 2 + 1], 1u, __ATOMIC_ACQ_REL);
          if (done == (uint32_t)tiles - 1u) {
            __atomic_store_n(&header[r * 2 + 1], 0u, __ATOMIC_RELAXED);
            __atomic_store_n(&header[r * 2], epoch, __ATOMIC_RELEASE);
          }
          pthread_barrier_wait(&stream[r]);
        }
      });
  for (auto& t : th) t.join();
  int total = 0;
  for (int b : bad) total += b;
  printf("gemv ws=%d tiles=%d calls=%d halves=%d failures=%d\n", ws, tiles, calls, halves, total);
  return total != 0;
}

int main(int argc, char** argv) {
  const int ws = argc > 1 ? atoi(argv[1]) : 4;
  const int ctas = argc > 2 ? atoi(argv[2]) : 3;
  const int calls = argc > 3 ? atoi(argv[3]) : 100;
  if (argc > 4 && strncmp(argv[4], "gemv", 4) == 0) return gemv_model(ws, ctas, calls, strcmp(argv[4], "gemv-one-parity") == 0);
  const bool entry_barrier = !(argc > 4 && strcmp(argv[4], "no-entry-barrier") == 0);
  const uint64_t timeout_ns = 20000000000ull;

  std::vector<uint32_t*> pads(ws);
  for (auto& p : pads) p = (uint32_t*)calloc(kSignalPadSlots, 4);
  // inbox[rank][src][tile][word], plain memory
  std::vector<std::vector<uint32_t>> inbox(ws, std::vector<uint32_t>((size_t)ws * kTilesPerRank * kWords, 0));
  std::vector<pthread_barrier_t> stream(ws);
  for (auto& b : stream) pthread_barrier_init(&b, nullptr, ctas);
  std::vector<int> bad((size_t)ws * ctas, 0);

  std::vector<std::thread> th;
  for (int r = 0; r < ws; ++r)
    for (int c = 0; c < ctas; ++c)
      th.emplace_back([&, r, c] {
        int& failures = bad[(size_t)r * ctas + c];
        uint32_t* header = pads[r] + kFlagSlotsBase;          // [0] call number, [1] CTAs done
        uint32_t* counters = pads[r] + kFlagSlotsBase + 2;    // one per tile of this rank
        for (int call = 1; call <= calls; ++call) {
          const uint32_t epoch = __atomic_load_n(&header[0], __ATOMIC_RELAXED) + 1u;
          if (epoch != (uint32_t)call) failures++;
          if (entry_barrier) {
            int peer = -1;
            if (host_barrier_signal_wait(pads.data(), (1024u + (uint32_t)c) * (uint32_t)ws, r, ws, timeout_ns, &peer))
              failures++;
          }
          // producer: tiles c, c + ctas, ... of the ws x kTilesPerRank (destination, tile) pairs
          for (int t = c; t < ws * kTilesPerRank; t += ctas) {
            const int dest = (t / kTilesPerRank + r + 1) % ws;   // own rows last, as the kernels visit them
            const int tile = t % kTilesPerRank;
            uint32_t* dst = inbox[dest].data() + ((size_t)r * kTilesPerRank + tile) * kWords;
            for (int w = 0; w < kWords; ++w) dst[w] = value_of(call, r, tile, w);
            __atomic_fetch_add(pads[dest] + kFlagSlotsBase + 2 + tile, 1u, __ATOMIC_RELEASE);
          }
          // consumer: this rank's tiles c, c + ctas, ...
          for (int tile = c; tile < kTilesPerRank; tile += ctas) {
            const uint32_t target = epoch * (uint32_t)ws;
            long spins = 0;
            while ((int32_t)(__atomic_load_n(&counters[tile], __ATOMIC_ACQUIRE) - target) < 0) {
              if (++spins > 2000000000L) { failures++; break; }
              std::this_thread::yield();
            }
            for (int s = 0; s < ws; ++s) {
              const uint32_t* src = inbox[r].data() + ((size_t)s * kTilesPerRank + tile) * kWords;
              for (int w = 0; w < kWords; ++w)
                if (src[w] != value_of(call, s, tile, w)) failures++;
            }
          }
          // the last CTA to finish publishes the call number
          const uint32_t done = __atomic_fetch_add(&header[1], 1u, __ATOMIC_ACQ_REL);
          if (done == (uint32_t)ctas - 1u) {
            __atomic_store_n(&header[1], 0u, __ATOMIC_RELAXED);
            __atomic_store_n(&header[0], epoch, __ATOMIC_RELEASE);
          }
          pthread_barrier_wait(&stream[r]);                    // stream order: the next kernel starts after this one
        }
      });
  for (auto& t : th) t.join();
  for (auto p : pads) free(p);
  int total = 0;
  for (int b : bad) total += b;
  printf("ws=%d ctas=%d calls=%d entry_barrier=%d failures=%d\n", ws, ctas, calls, (int)entry_barrier, total);
  return total != 0;
}
