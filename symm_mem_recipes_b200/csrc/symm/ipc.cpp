#include "ipc.h"

#include <errno.h>
#include <poll.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <time.h>
#include <unistd.h>

#include <stdexcept>

namespace smr {

namespace {
socklen_t make_addr(const std::string& name, sockaddr_un* addr) {
  if (name.size() + 2 > sizeof(addr->sun_path))
    throw std::runtime_error("FdChannel: socket name too long: " + name);
  memset(addr, 0, sizeof(*addr));
  addr->sun_family = AF_UNIX;
  addr->sun_path[0] = '\0';  // abstract namespace: no file, gone when the socket closes
  memcpy(addr->sun_path + 1, name.data(), name.size());
  return (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + name.size());
}
}  // namespace

FdChannel::FdChannel(const std::string& name) : name_(name) {
  sock_ = socket(AF_UNIX, SOCK_DGRAM | SOCK_CLOEXEC, 0);
  if (sock_ < 0) throw std::runtime_error(std::string("FdChannel: socket(): ") + strerror(errno));
  sockaddr_un addr;
  socklen_t len = make_addr(name_, &addr);
  if (bind(sock_, reinterpret_cast<sockaddr*>(&addr), len) != 0) {
    int e = errno;
    close(sock_);
    sock_ = -1;
    throw std::runtime_error("FdChannel: bind(" + name_ + "): " + strerror(e));
  }
}

FdChannel::~FdChannel() {
  if (sock_ >= 0) close(sock_);
}

void FdChannel::send_fd(const std::string& dst_name, int fd, int32_t src_rank, int32_t tag,
                        int timeout_ms) const {
  sockaddr_un addr;
  socklen_t len = make_addr(dst_name, &addr);
  int32_t header[2] = {src_rank, tag};
  iovec iov{header, sizeof(header)};
  alignas(cmsghdr) char control[CMSG_SPACE(sizeof(int))];
  memset(control, 0, sizeof(control));
  msghdr msg{};
  msg.msg_name = &addr;
  msg.msg_namelen = len;
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = control;
  msg.msg_controllen = sizeof(control);
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  c->cmsg_level = SOL_SOCKET;
  c->cmsg_type = SCM_RIGHTS;
  c->cmsg_len = CMSG_LEN(sizeof(int));
  memcpy(CMSG_DATA(c), &fd, sizeof(int));
  // The peer may not have bound its socket yet: retry until the deadline.
  timespec t0;
  clock_gettime(CLOCK_MONOTONIC, &t0);
  for (;;) {
    if (sendmsg(sock_, &msg, 0) >= 0) return;
    int e = errno;
    if (e != ECONNREFUSED && e != ENOENT && e != EAGAIN && e != ENOBUFS && e != EINTR)
      throw std::runtime_error("FdChannel: sendmsg to " + dst_name + ": " + strerror(e));
    timespec t1;
    clock_gettime(CLOCK_MONOTONIC, &t1);
    long ms = (t1.tv_sec - t0.tv_sec) * 1000L + (t1.tv_nsec - t0.tv_nsec) / 1000000L;
    if (ms > timeout_ms)
      throw std::runtime_error("FdChannel: timed out sending to " + dst_name + ": " + strerror(e));
    usleep(1000);
  }
}

FdMessage FdChannel::recv_fd(int timeout_ms) const {
  pollfd p{sock_, POLLIN, 0};
  int pr;
  do {
    pr = poll(&p, 1, timeout_ms);
  } while (pr < 0 && errno == EINTR);
  if (pr == 0) throw std::runtime_error("FdChannel: timed out waiting for a file descriptor on " + name_);
  if (pr < 0) throw std::runtime_error(std::string("FdChannel: poll(): ") + strerror(errno));
  int32_t header[2] = {-1, 0};
  iovec iov{header, sizeof(header)};
  alignas(cmsghdr) char control[CMSG_SPACE(sizeof(int))];
  msghdr msg{};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = control;
  msg.msg_controllen = sizeof(control);
  ssize_t n = recvmsg(sock_, &msg, MSG_CMSG_CLOEXEC);
  if (n != (ssize_t)sizeof(header))
    throw std::runtime_error(std::string("FdChannel: recvmsg(): ") + (n < 0 ? strerror(errno) : "short message"));
  FdMessage out;
  out.src_rank = header[0];
  out.tag = header[1];
  for (cmsghdr* c = CMSG_FIRSTHDR(&msg); c != nullptr; c = CMSG_NXTHDR(&msg, c)) {
    if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS) {
      memcpy(&out.fd, CMSG_DATA(c), sizeof(int));
      break;
    }
  }
  if (out.fd < 0) throw std::runtime_error("FdChannel: message carried no file descriptor (dropped?)");
  return out;
}

}  // namespace smr
