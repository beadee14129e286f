// Per-node rendezvous between the local rank processes: small all-gathers,
// barriers and file-descriptor passing, all with timeouts.
//
// Capability parity: the reference's Broker (src/system/broker.cpp:469-887)
// does the same job with a POSIX shared-memory vault, a process-shared
// condition-variable barrier and SCM_RIGHTS datagrams, and waits without
// limit.  Here rank 0 is a hub on an abstract-namespace UNIX stream socket
// (nothing to unlink, nothing left behind after a crash); every message
// carries an operation tag and a sequence number, and every wait has a
// deadline, so a rank that died or never joined turns into an error on the
// others instead of a hang.
#pragma once
#include <cstddef>
#include <string>
#include <vector>

namespace oob {

class Bootstrap {
 public:
  // Returns nullptr and fills *err on failure (bad key, timeout, ...).
  static Bootstrap* create(int rank, int world, const std::string& key, int timeout_ms, std::string* err);
  ~Bootstrap();

  int rank() const { return rank_; }
  int world() const { return world_; }
  const std::string& last_error() const { return err_; }

  // out must hold world * bytes; slot r receives rank r's `in`.
  bool allgather(const void* in, void* out, size_t bytes);
  bool barrier();
  // Every rank contributes one descriptor (or -1); on return fds[r] is a
  // descriptor in this process that refers to rank r's file (fds[rank] is a
  // dup of the caller's own).  The caller closes them.
  bool exchange_fds(int my_fd, std::vector<int>* fds);
  // Rank `root` sends *fd to everybody else.
  bool broadcast_fd(int root, int* fd);

  // Longest key accepted (the reference keeps its socket prefix under 90
  // characters for sun_path, src/system/broker.cpp:46-103).
  static constexpr size_t kMaxKeyLen = 80;
  static bool sanitize_key(const std::string& key, std::string* out, std::string* err);

 private:
  Bootstrap() = default;
  bool fail(const std::string& what);
  bool send_msg(int sock, int op, const void* data, size_t bytes, int fd);
  bool recv_msg(int sock, int op, void* data, size_t bytes, int* fd);

  int rank_ = 0, world_ = 1, timeout_ms_ = 30000;
  unsigned seq_ = 0;
  int listen_fd_ = -1;
  int hub_fd_ = -1;             // non-root: connection to rank 0
  std::vector<int> peer_fd_;    // root: connection to each rank (index = rank; [0] unused)
  std::string err_;
};

}  // namespace oob
