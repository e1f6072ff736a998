// Race check of the cross-rank protocols under ThreadSanitizer: threads play the ranks over heap
// "signal pads" and run the host builds of the CAS barrier (as a litmus: plain writes, barrier,
// plain reads of every peer), the epoch barrier and the low-latency all-reduce (tagged words, two
// parities).  The host builds use the same slot layout and the same release / acquire placement as
// the device code, so a missing ordering shows up here as a reported race or a wrong value.
// Built and run by tests/test_tsan_protocols.py with -fsanitize=thread and with
// -fsanitize=address,undefined; exit code 0 = clean.
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <thread>
#include <vector>
#include "symm/host_backend.h"
#include "device/pad_layout.h"
#include "oracle/cpu_reference.h"
using namespace smr;
int main(int argc, char** argv) {
  const int ws = argc > 1 ? atoi(argv[1]) : 4, iters = argc > 2 ? atoi(argv[2]) : 300;
  std::vector<uint32_t*> pads(ws);
  std::vector<std::vector<uint32_t>> data(ws, std::vector<uint32_t>(64, 0));
  for (auto& p : pads) p = (uint32_t*)calloc(kSignalPadSlots, 4);
  const size_t cap = 256;
  std::vector<void*> wsp(ws);
  for (auto& w : wsp) w = calloc(1, 256 + 2 * ws * (cap / 8) * 32);
  std::vector<int> bad(ws, 0);
  std::vector<std::thread> th;
  for (int r = 0; r < ws; ++r)
    th.emplace_back([&, r] {
      int peer = -1;
      uint32_t count = 0;
      std::vector<uint16_t> in(cap), out(cap);
      for (int it = 1; it <= iters; ++it) {
        for (auto& v : data[r]) v = (uint32_t)(it * 100 + r);               // plain writes
        if (host_barrier_signal_wait(pads.data(), 5 * ws, r, ws, 5000000000ull, &peer)) bad[r]++;
        for (int s = 0; s < ws; ++s)                                         // plain reads of every peer
          if (data[s][7] != (uint32_t)(it * 100 + s)) bad[r]++;
        if (host_epoch_barrier(pads.data(), 3, r, ws, &count, 5000000000ull, &peer)) bad[r]++;   // before overwrite
        for (size_t i = 0; i < cap; ++i) in[i] = f32_to_bf16((float)((it + r + i) % 7));
        if (host_ll_all_reduce(wsp.data(), r, ws, in.data(), out.data(), cap, cap, 5000000000ull, &peer)) bad[r]++;
        float want = 0; for (int s = 0; s < ws; ++s) want += (float)((it + s + 3) % 7);
        if (bf16_to_f32(out[3]) != want) bad[r]++;
      }
    });
  for (auto& t : th) t.join();
  for (auto p : pads) free(p);
  for (auto w : wsp) free(w);
  int total = 0; for (int b : bad) total += b;
  printf("ws=%d iters=%d failures=%d\n", ws, iters, total);
  return total != 0;
}
