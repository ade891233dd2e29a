// Host-side rendezvous between the ranks of one node: tagged all-to-all message
// exchange over abstract Unix-domain sockets, with file descriptors riding along
// as SCM_RIGHTS ancillary data.  The symmetric heap uses it to hand cuMem
// allocation handles (and the NVLS multicast handle) to every peer, and as a
// host barrier between the steps of multicast set-up.  No GPU involved, so it is
// tested with plain processes/threads on a CPU-only machine.
#pragma once
#include <stdint.h>

#include <map>
#include <string>
#include <utility>
#include <vector>

namespace tileccl {

class Bootstrap {
 public:
  Bootstrap(int rank, int world_size, std::string job_id, int timeout_ms);
  ~Bootstrap();
  Bootstrap(const Bootstrap&) = delete;
  Bootstrap& operator=(const Bootstrap&) = delete;

  // Binds and listens on this rank's socket.  Returns false (see error()) on failure.
  bool open();

  // Sends (payload, fd) to `to_rank` under `tag`; fd < 0 sends no descriptor.
  bool send(int to_rank, uint32_t tag, uint64_t payload, int fd);
  // Receives the message `from_rank` sent under `tag` (buffers anything else that arrives).
  bool recv(int from_rank, uint32_t tag, uint64_t* payload, int* fd);

  // Every rank contributes (payload, fd); afterwards payloads[r] / fds[r] hold
  // rank r's contribution (own entry copied, own fd not duplicated).
  bool all_gather(uint32_t tag, uint64_t payload, int fd, std::vector<uint64_t>* payloads,
                  std::vector<int>* fds);
  // Root sends (payload, fd) to everyone.
  bool broadcast(uint32_t tag, int root, uint64_t* payload, int* fd);
  bool barrier(uint32_t tag);

  const std::string& error() const { return error_; }
  int rank() const { return rank_; }
  int world_size() const { return world_size_; }

 private:
  struct Message {
    uint64_t payload;
    int fd;
  };
  bool pump_one(int64_t deadline_ms);
  std::string socket_name(int rank) const;

  int rank_, world_size_;
  std::string job_id_;
  int timeout_ms_;
  int listen_fd_ = -1;
  std::map<std::pair<uint32_t, int>, Message> inbox_;
  std::string error_;
};

}  // namespace tileccl
