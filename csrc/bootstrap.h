// Out-of-band bootstrap between the processes of one box: a full mesh of
// Unix-domain stream sockets in the abstract namespace, named after a shared
// unique id.  It carries small blobs (all-gather, barrier) and, the reason it
// exists, file descriptors (SCM_RIGHTS) – the exportable handles of CUDA VMM
// allocations and of the NVLS multicast object.
//
// Plays the role of NVSHMEM's unique-id bootstrap in the reference
// (csrc/torch_interface.cpp:16-25,57-64): get_unique_id() on one rank, ship the
// id through any channel (torch.distributed, a file, argv), init_with_uid() on
// all.  No network, no MPI, no torch: every call has a deadline and throws
// std::runtime_error instead of blocking forever.
#pragma once
#include <stddef.h>

#include <string>
#include <vector>

namespace penny {

std::string make_unique_id();  // 32 hex characters

class Bootstrap {
 public:
  Bootstrap(const std::string& uid, int rank, int world, int timeout_ms = 120000);
  ~Bootstrap();
  Bootstrap(const Bootstrap&) = delete;
  Bootstrap& operator=(const Bootstrap&) = delete;

  int rank() const { return rank_; }
  int world() const { return world_; }

  // out receives world * bytes, ordered by rank.
  void all_gather(const void* in, size_t bytes, void* out);
  void barrier();
  void send_bytes(int peer, const void* p, size_t bytes);
  void recv_bytes(int peer, void* p, size_t bytes);
  void send_fd(int peer, int fd);
  int recv_fd(int peer);

 private:
  int rank_, world_, timeout_ms_;
  int listen_fd_ = -1;
  std::vector<int> conn_;  // conn_[peer], -1 for self
};

}  // namespace penny
