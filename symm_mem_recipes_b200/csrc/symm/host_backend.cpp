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

uint32_t HostSymmAllocation::barrier(uint32_t slot_base, uint64_t timeout_ns, int* failed_peer) {
  if (!rendezvoused_) throw std::runtime_error("barrier on an allocation that is not rendezvoused");
  std::vector<uint32_t*> pads(world_size_);
  for (int r = 0; r < world_size_; ++r) pads[r] = peer_pad(r);
  return host_barrier_signal_wait(pads.data(), slot_base, rank_, world_size_, timeout_ns, failed_peer);
}

}  // namespace smr
