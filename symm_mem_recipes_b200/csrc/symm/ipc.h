// File-descriptor passing between the ranks of one host.
//
// Each rank binds one abstract-namespace unix datagram socket; an FD travels
// as SCM_RIGHTS ancillary data with a small header saying who sent it and what
// it is.  The socket names themselves are exchanged through the
// torch.distributed Store by the Python layer.
//
// Upstream has no code for this: its `rendezvous` calls
// (symm_mem_recipes/triton_all_gather_matmul.py:28, 226;
// triton_one_shot_all_reduce.py:111; triton_barrier.py:198) rely on torch's
// own handle exchange.
#pragma once
#include <stdint.h>

#include <string>

namespace smr {

struct FdMessage {
  int fd = -1;
  int32_t src_rank = -1;
  int32_t tag = 0;
};

class FdChannel {
 public:
  // `name` without the leading NUL of the abstract namespace.
  explicit FdChannel(const std::string& name);
  ~FdChannel();
  FdChannel(const FdChannel&) = delete;
  FdChannel& operator=(const FdChannel&) = delete;

  const std::string& name() const { return name_; }
  void send_fd(const std::string& dst_name, int fd, int32_t src_rank, int32_t tag,
               int timeout_ms) const;
  // Blocks up to timeout_ms; throws on timeout.
  FdMessage recv_fd(int timeout_ms) const;

 private:
  std::string name_;
  int sock_ = -1;
};

}  // namespace smr
