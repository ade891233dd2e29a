#include "bootstrap.h"

#include <errno.h>
#include <poll.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <time.h>
#include <unistd.h>

#include <cstddef>

namespace tileccl {

namespace {

int64_t now_ms() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return static_cast<int64_t>(ts.tv_sec) * 1000 + ts.tv_nsec / 1000000;
}

struct WireHeader {
  uint32_t magic;
  uint32_t tag;
  int32_t from_rank;
  int32_t has_fd;
  uint64_t payload;
};
constexpr uint32_t kMagic = 0x7C11B200u;

// Abstract-namespace address: sun_path[0] == 0, no file-system entry to clean up.
socklen_t fill_addr(sockaddr_un* addr, const std::string& name) {
  memset(addr, 0, sizeof(*addr));
  addr->sun_family = AF_UNIX;
  size_t n = name.size();
  if (n > sizeof(addr->sun_path) - 2) n = sizeof(addr->sun_path) - 2;
  memcpy(addr->sun_path + 1, name.data(), n);
  return static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + n);
}

}  // namespace

Bootstrap::Bootstrap(int rank, int world_size, std::string job_id, int timeout_ms)
    : rank_(rank), world_size_(world_size), job_id_(std::move(job_id)), timeout_ms_(timeout_ms) {}

Bootstrap::~Bootstrap() {
  if (listen_fd_ >= 0) close(listen_fd_);
  for (auto& kv : inbox_)
    if (kv.second.fd >= 0) close(kv.second.fd);
}

std::string Bootstrap::socket_name(int rank) const {
  return "tileccl-b200-" + job_id_ + "-" + std::to_string(rank);
}

bool Bootstrap::open() {
  listen_fd_ = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (listen_fd_ < 0) {
    error_ = std::string("socket(): ") + strerror(errno);
    return false;
  }
  sockaddr_un addr;
  socklen_t len = fill_addr(&addr, socket_name(rank_));
  if (bind(listen_fd_, reinterpret_cast<sockaddr*>(&addr), len) != 0) {
    error_ = "bind(" + socket_name(rank_) + "): " + strerror(errno);
    return false;
  }
  if (listen(listen_fd_, 64) != 0) {
    error_ = std::string("listen(): ") + strerror(errno);
    return false;
  }
  return true;
}

bool Bootstrap::send(int to_rank, uint32_t tag, uint64_t payload, int fd) {
  const int64_t deadline = now_ms() + timeout_ms_;
  int s = -1;
  // The peer may not have bound its socket yet: retry until the deadline.
  for (;;) {
    s = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (s < 0) {
      error_ = std::string("socket(): ") + strerror(errno);
      return false;
    }
    sockaddr_un addr;
    socklen_t len = fill_addr(&addr, socket_name(to_rank));
    if (connect(s, reinterpret_cast<sockaddr*>(&addr), len) == 0) break;
    int err = errno;
    close(s);
    s = -1;
    if (err != ECONNREFUSED && err != ENOENT && err != EAGAIN) {
      error_ = "connect(rank " + std::to_string(to_rank) + "): " + strerror(err);
      return false;
    }
    if (now_ms() > deadline) {
      error_ = "timed out connecting to rank " + std::to_string(to_rank) + " (" +
               socket_name(to_rank) + ")";
      return false;
    }
    usleep(2000);
  }
  WireHeader h{kMagic, tag, rank_, fd >= 0 ? 1 : 0, payload};
  iovec iov{&h, sizeof(h)};
  msghdr msg;
  memset(&msg, 0, sizeof(msg));
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  if (fd >= 0) {
    memset(ctrl, 0, sizeof(ctrl));
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    cmsghdr* c = CMSG_FIRSTHDR(&msg);
    c->cmsg_level = SOL_SOCKET;
    c->cmsg_type = SCM_RIGHTS;
    c->cmsg_len = CMSG_LEN(sizeof(int));
    memcpy(CMSG_DATA(c), &fd, sizeof(int));
  }
  ssize_t n = sendmsg(s, &msg, MSG_NOSIGNAL);
  int err = errno;
  close(s);
  if (n != static_cast<ssize_t>(sizeof(h))) {
    error_ = "sendmsg(rank " + std::to_string(to_rank) + "): " + strerror(err);
    return false;
  }
  return true;
}

bool Bootstrap::pump_one(int64_t deadline_ms) {
  int64_t left = deadline_ms - now_ms();
  if (left < 0) left = 0;
  pollfd pfd{listen_fd_, POLLIN, 0};
  int pr = poll(&pfd, 1, static_cast<int>(left));
  if (pr == 0) {
    error_ = "timed out waiting for a peer message";
    return false;
  }
  if (pr < 0) {
    if (errno == EINTR) return true;
    error_ = std::string("poll(): ") + strerror(errno);
    return false;
  }
  int s = accept4(listen_fd_, nullptr, nullptr, SOCK_CLOEXEC);
  if (s < 0) {
    error_ = std::string("accept(): ") + strerror(errno);
    return false;
  }
  WireHeader h;
  memset(&h, 0, sizeof(h));
  iovec iov{&h, sizeof(h)};
  msghdr msg;
  memset(&msg, 0, sizeof(msg));
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  memset(ctrl, 0, sizeof(ctrl));
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  // The sender may be between connect() and sendmsg(): wait for the payload.
  pollfd dfd{s, POLLIN, 0};
  left = deadline_ms - now_ms();
  if (left < 0) left = 0;
  if (poll(&dfd, 1, static_cast<int>(left)) <= 0) {
    close(s);
    error_ = "peer connected but sent nothing (it may have exited)";
    return false;
  }
  ssize_t n = recvmsg(s, &msg, MSG_CMSG_CLOEXEC);
  close(s);
  if (n != static_cast<ssize_t>(sizeof(h)) || h.magic != kMagic) {
    error_ = "malformed or truncated bootstrap message (peer closed its socket?)";
    return false;
  }
  int fd = -1;
  for (cmsghdr* c = CMSG_FIRSTHDR(&msg); c != nullptr; c = CMSG_NXTHDR(&msg, c)) {
    if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS)
      memcpy(&fd, CMSG_DATA(c), sizeof(int));
  }
  if (h.has_fd && fd < 0) {
    error_ = "bootstrap message announced a descriptor but carried none";
    return false;
  }
  if (h.from_rank < 0 || h.from_rank >= world_size_) {
    if (fd >= 0) close(fd);
    error_ = "bootstrap message from an out-of-range rank";
    return false;
  }
  inbox_[{h.tag, h.from_rank}] = Message{h.payload, fd};
  return true;
}

bool Bootstrap::recv(int from_rank, uint32_t tag, uint64_t* payload, int* fd) {
  const int64_t deadline = now_ms() + timeout_ms_;
  for (;;) {
    auto it = inbox_.find({tag, from_rank});
    if (it != inbox_.end()) {
      if (payload) *payload = it->second.payload;
      if (fd) *fd = it->second.fd;
      else if (it->second.fd >= 0) close(it->second.fd);
      inbox_.erase(it);
      return true;
    }
    if (now_ms() > deadline) {
      error_ = "timed out waiting for rank " + std::to_string(from_rank) + " (tag " +
               std::to_string(tag) + ")";
      return false;
    }
    if (!pump_one(deadline)) return false;
  }
}

bool Bootstrap::all_gather(uint32_t tag, uint64_t payload, int fd, std::vector<uint64_t>* payloads,
                           std::vector<int>* fds) {
  for (int d = 1; d < world_size_; ++d)
    if (!send((rank_ + d) % world_size_, tag, payload, fd)) return false;
  if (payloads) payloads->assign(world_size_, 0);
  if (fds) fds->assign(world_size_, -1);
  if (payloads) (*payloads)[rank_] = payload;
  if (fds) (*fds)[rank_] = fd;
  for (int r = 0; r < world_size_; ++r) {
    if (r == rank_) continue;
    uint64_t pl = 0;
    int f = -1;
    if (!recv(r, tag, &pl, fds ? &f : nullptr)) return false;
    if (payloads) (*payloads)[r] = pl;
    if (fds) (*fds)[r] = f;
  }
  return true;
}

bool Bootstrap::broadcast(uint32_t tag, int root, uint64_t* payload, int* fd) {
  if (rank_ == root) {
    for (int r = 0; r < world_size_; ++r)
      if (r != root && !send(r, tag, payload ? *payload : 0, fd ? *fd : -1)) return false;
    return true;
  }
  return recv(root, tag, payload, fd);
}

bool Bootstrap::barrier(uint32_t tag) { return all_gather(tag, 0, -1, nullptr, nullptr); }

}  // namespace tileccl
