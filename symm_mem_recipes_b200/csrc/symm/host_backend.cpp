#include "host_backend.h"

#include <errno.h>
#include <fcntl.h>
#include <sched.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <time.h>
#include <unistd.h>

#include <stdexcept>

namespace smr {

namespace {
size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

uint64_t now_ns() {
  timespec t;
  clock_gettime(CLOCK_MONOTONIC, &t);
  return (uint64_t)t.tv_sec * 1000000000ull + (uint64_t)t.tv_nsec;
}

void* map_shm(const std::string& name, size_t bytes, bool create) {
  int fd = shm_open(name.c_str(), create ? (O_CREAT | O_EXCL | O_RDWR) : O_RDWR, 0600);
  if (fd < 0) throw std::runtime_error("shm_open(" + name + "): " + strerror(errno));
  if (create && ftruncate(fd, (off_t)bytes) != 0) {
    int e = errno;
    close(fd);
    shm_unlink(name.c_str());
    throw std::runtime_error("ftruncate(" + name + "): " + strerror(e));
  }
  void* p = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  int e = errno;
  close(fd);
  if (p == MAP_FAILED) throw std::runtime_error("mmap(" + name + "): " + strerror(e));
  return p;
}
}  // namespace

HostSymmAllocation::HostSymmAllocation(const std::string& shm_name, size_t payload_bytes)
    : name_(shm_name), payload_bytes_(payload_bytes) {
  pad_offset_ = round_up(payload_bytes == 0 ? 16 : payload_bytes, 256);
  block_bytes_ = round_up(pad_offset_ + kSignalPadBytes, 4096);
  base_ = map_shm(name_, block_bytes_, /*create=*/true);  // fresh shm pages read as zero
}

HostSymmAllocation::~HostSymmAllocation() { release(); }

void HostSymmAllocation::rendezvous(int rank, const std::vector<std::string>& names) {
  if (rendezvoused_) throw std::runtime_error("allocation is already rendezvoused");
  int ws = (int)names.size();
  if (ws < 1 || ws > kMaxWorldSize || rank < 0 || rank >= ws || names[rank] != name_)
    throw std::runtime_error("bad rank / names for host rendezvous");
  rank_ = rank;
  world_size_ = ws;
  peers_.assign(ws, nullptr);
  peers_[rank] = base_;
  for (int r = 0; r < ws; ++r)
    if (r != rank) peers_[r] = map_shm(names[r], block_bytes_, /*create=*/false);
  rendezvoused_ = true;
}

void HostSymmAllocation::release() {
  if (released_) return;
  released_ = true;
  for (int r = 0; r < (int)peers_.size(); ++r)
    if (r != rank_ && peers_[r] != nullptr) munmap(peers_[r], block_bytes_);
  peers_.clear();
  if (base_ != nullptr) {
    munmap(base_, block_bytes_);
    shm_unlink(name_.c_str());
    base_ = nullptr;
  }
}

uint32_t host_barrier_signal_wait(uint32_t* const* pads, uint32_t slot_base, int rank,
                                  int world_size, uint64_t timeout_ns, int* failed_peer) {
  const uint64_t deadline = now_ns() + timeout_ns;
  // signal every peer (release), spinning while an earlier signal is unconsumed
  for (int peer = 0; peer < world_size; ++peer) {
    uint32_t* send = pads[peer] + slot_base + rank;
    for (uint32_t spins = 0;; ++spins) {
      uint32_t expected = 0;
      if (__atomic_compare_exchange_n(send, &expected, 1u, false, __ATOMIC_RELEASE, __ATOMIC_RELAXED))
        break;
      if ((spins & 255u) == 255u) {
        if (now_ns() > deadline) {
          if (failed_peer) *failed_peer = peer;
          return kTimeoutBarrierSend;
        }
        sched_yield();
      }
    }
  }
  // consume every peer's signal (acquire)
  for (int peer = 0; peer < world_size; ++peer) {
    uint32_t* wait = pads[rank] + slot_base + peer;
    for (uint32_t spins = 0;; ++spins) {
      uint32_t expected = 1;
      if (__atomic_compare_exchange_n(wait, &expected, 0u, false, __ATOMIC_ACQUIRE, __ATOMIC_RELAXED))
        break;
      if ((spins & 255u) == 255u) {
        if (now_ns() > deadline) {
          if (failed_peer) *failed_peer = peer;
          return kTimeoutBarrierWait;
        }
        sched_yield();
      }
    }
  }
  return kOk;
}

uint32_t host_epoch_barrier(uint32_t* const* pads, uint32_t block_id, int rank, int world_size,
                            uint32_t* count, uint64_t timeout_ns, int* failed_peer) {
  const uint64_t deadline = now_ns() + timeout_ns;
  const uint32_t base = kArFlagBase + block_id * kArFlagStride;
  const uint32_t c = ++*count;
  for (int peer = 0; peer < world_size; ++peer)
    __atomic_store_n(pads[peer] + base + 16u + (uint32_t)rank, c, __ATOMIC_RELEASE);
  for (int peer = 0; peer < world_size; ++peer) {
    const uint32_t* wait = pads[rank] + base + 16u + (uint32_t)peer;
    for (uint32_t spins = 0;; ++spins) {
      // a peer can be one barrier ahead, never behind once it has arrived: signed comparison
      if ((int32_t)(__atomic_load_n(wait, __ATOMIC_ACQUIRE) - c) >= 0) break;
      if ((spins & 255u) == 255u) {
        if (now_ns() > deadline) {
          if (failed_peer) *failed_peer = peer;
          return kTimeoutBarrierWait;
        }
        sched_yield();
      }
    }
  }
  return kOk;
}

uint32_t host_ll_all_reduce(void* const* workspaces, int rank, int world_size, const uint16_t* in,
                            uint16_t* out, size_t numel, size_t capacity_numel, uint64_t timeout_ns,
                            int* failed_peer) {
  const uint64_t deadline = now_ns() + timeout_ns;
  char* my_ws = static_cast<char*>(workspaces[rank]);
  uint32_t* header = reinterpret_cast<uint32_t*>(my_ws);
  const uint32_t tag = header[0] + 1u;                    // this call's number
  const size_t cap_vec = capacity_numel / 8, n_vec = numel / 8;
  const size_t parity_off = 256 + (size_t)(tag & 1u) * world_size * cap_vec * 32;
  // push: every 8 bytes on the "wire" = 4 bytes of data + the tag
  for (size_t i = 0; i < n_vec; ++i) {
    uint32_t x[4];
    memcpy(x, in + i * 8, 16);
    for (int j = 1; j <= world_size; ++j) {               // own inbox last
      const int peer = (rank + j) % world_size;
      uint64_t* dst = reinterpret_cast<uint64_t*>(static_cast<char*>(workspaces[peer]) + parity_off +
                                                  ((size_t)rank * cap_vec + i) * 32);
      for (int q = 0; q < 4; ++q)
        __atomic_store_n(dst + q, (uint64_t)x[q] | ((uint64_t)tag << 32), __ATOMIC_RELAXED);
    }
  }
  // poll the own inbox, sum in rank order (bf16 adds from +0: same bits on every rank)
  for (size_t i = 0; i < n_vec; ++i) {
    uint16_t acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int r = 0; r < world_size; ++r) {
      const uint64_t* src = reinterpret_cast<const uint64_t*>(my_ws + parity_off + ((size_t)r * cap_vec + i) * 32);
      uint32_t w[4];
      for (int q = 0; q < 4; ++q) {
        for (uint32_t spins = 0;; ++spins) {
          const uint64_t v = __atomic_load_n(src + q, __ATOMIC_RELAXED);
          if ((uint32_t)(v >> 32) == tag) {
            w[q] = (uint32_t)v;
            break;
          }
          if ((spins & 255u) == 255u) {
            if (now_ns() > deadline) {
              if (failed_peer) *failed_peer = r;
              return kTimeoutFlag;
            }
            sched_yield();
          }
        }
      }
      uint16_t h[8];
      memcpy(h, w, 16);
      for (int e = 0; e < 8; ++e) {
        uint32_t a = (uint32_t)acc[e] << 16, b = (uint32_t)h[e] << 16;
        float fa, fb;
        memcpy(&fa, &a, 4);
        memcpy(&fb, &b, 4);
        float f = fa + fb;
        uint32_t u;
        memcpy(&u, &f, 4);
        if ((u & 0x7fffffffu) <= 0x7f800000u) u += 0x7fffu + ((u >> 16) & 1u);   // round to nearest even
        acc[e] = (uint16_t)(u >> 16);
      }
    }
    memcpy(out + i * 8, acc, 16);
  }
  header[0] = tag;                                         // single-threaded per rank: no "last CTA" needed
  return kOk;
}

namespace {
// 0 -> 1 (release) or 1 -> 0 (acquire) on one slot, bounded
uint32_t flip_slot(uint32_t* slot, uint32_t from, uint32_t to, int order, uint64_t timeout_ns, uint32_t on_timeout) {
  const uint64_t deadline = now_ns() + timeout_ns;
  for (uint32_t spins = 0;; ++spins) {
    uint32_t expected = from;
    if (__atomic_compare_exchange_n(slot, &expected, to, false, order, __ATOMIC_RELAXED)) return kOk;
    if ((spins & 255u) == 255u) {
      if (now_ns() > deadline) return on_timeout;
      sched_yield();
    }
  }
}
}  // namespace

uint32_t HostSymmAllocation::put_signal(int dst, uint32_t slot_base, uint64_t timeout_ns) {
  if (!rendezvoused_) throw std::runtime_error("put_signal on an allocation that is not rendezvoused");
  return flip_slot(peer_pad(dst) + slot_base + rank_, 0u, 1u, __ATOMIC_RELEASE, timeout_ns, kTimeoutBarrierSend);
}

uint32_t HostSymmAllocation::wait_signal(int src, uint32_t slot_base, uint64_t timeout_ns) {
  if (!rendezvoused_) throw std::runtime_error("wait_signal on an allocation that is not rendezvoused");
  return flip_slot(peer_pad(rank_) + slot_base + src, 1u, 0u, __ATOMIC_ACQUIRE, timeout_ns, kTimeoutBarrierWait);
}

uint32_t HostSymmAllocation::barrier(uint32_t slot_base, uint64_t timeout_ns, int* failed_peer) {
  if (!rendezvoused_) throw std::runtime_error("barrier on an allocation that is not rendezvoused");
  std::vector<uint32_t*> pads(world_size_);
  for (int r = 0; r < world_size_; ++r) pads[r] = peer_pad(r);
  return host_barrier_signal_wait(pads.data(), slot_base, rank_, world_size_, timeout_ns, failed_peer);
}

}  // namespace smr
