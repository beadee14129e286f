#include "bootstrap.h"

#include <errno.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <time.h>
#include <unistd.h>

#include <cstdint>
#include <cstring>

namespace oob {
namespace {

constexpr uint32_t kMagic = 0x4f4f4232;  // "OOB2"
enum Op : int { kOpHello = 1, kOpGather = 2, kOpFd = 3, kOpBcastFd = 4 };

struct Header {
  uint32_t magic;
  int32_t op;
  uint32_t seq;
  int32_t rank;
  uint64_t bytes;
  int32_t has_fd;
  int32_t pad;
};

int64_t now_ms() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return int64_t(ts.tv_sec) * 1000 + ts.tv_nsec / 1000000;
}

bool wait_fd(int fd, short events, int64_t deadline) {
  while (true) {
    const int64_t left = deadline - now_ms();
    if (left <= 0) return false;
    pollfd p{fd, events, 0};
    const int r = poll(&p, 1, static_cast<int>(left > 1000 ? 1000 : left));
    if (r > 0) return (p.revents & (events | POLLHUP | POLLERR)) != 0;
    if (r < 0 && errno != EINTR) return false;
  }
}

socklen_t make_addr(const std::string& key, sockaddr_un* addr) {
  std::memset(addr, 0, sizeof(*addr));
  addr->sun_family = AF_UNIX;
  // Abstract namespace: first byte of sun_path is NUL.
  const std::string name = "oob_b200_" + key;
  std::memcpy(addr->sun_path + 1, name.data(), name.size());
  return static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + name.size());
}

}  // namespace

bool Bootstrap::sanitize_key(const std::string& key, std::string* out, std::string* err) {
  if (key.empty()) {
    if (err) *err = "bootstrap key is empty";
    return false;
  }
  if (key.size() > kMaxKeyLen) {
    if (err) *err = "bootstrap key longer than " + std::to_string(kMaxKeyLen) + " characters";
    return false;
  }
  out->clear();
  for (char c : key) {
    const bool ok = (c >= 'a' && c <= 'z') || (c >= 'A' && c <= 'Z') || (c >= '0' && c <= '9') || c == '_' ||
                    c == '-' || c == '.';
    out->push_back(ok ? c : '_');
  }
  return true;
}

bool Bootstrap::fail(const std::string& what) {
  err_ = "bootstrap rank " + std::to_string(rank_) + ": " + what;
  return false;
}

bool Bootstrap::send_msg(int sock, int op, const void* data, size_t bytes, int fd) {
  const int64_t deadline = now_ms() + timeout_ms_;
  Header h{kMagic, op, seq_, rank_, bytes, fd >= 0 ? 1 : 0, 0};
  // Header (with the optional descriptor as ancillary data).
  {
    iovec iov{&h, sizeof(h)};
    msghdr m{};
    m.msg_iov = &iov;
    m.msg_iovlen = 1;
    alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
    if (fd >= 0) {
      std::memset(ctrl, 0, sizeof(ctrl));
      m.msg_control = ctrl;
      m.msg_controllen = sizeof(ctrl);
      cmsghdr* c = CMSG_FIRSTHDR(&m);
      c->cmsg_level = SOL_SOCKET;
      c->cmsg_type = SCM_RIGHTS;
      c->cmsg_len = CMSG_LEN(sizeof(int));
      std::memcpy(CMSG_DATA(c), &fd, sizeof(int));
    }
    if (!wait_fd(sock, POLLOUT, deadline)) return fail("timeout sending header");
    const ssize_t n = sendmsg(sock, &m, MSG_NOSIGNAL);
    if (n != static_cast<ssize_t>(sizeof(h))) return fail(std::string("sendmsg failed: ") + strerror(errno));
  }
  const char* p = static_cast<const char*>(data);
  size_t left = bytes;
  while (left > 0) {
    if (!wait_fd(sock, POLLOUT, deadline)) return fail("timeout sending payload");
    const ssize_t n = send(sock, p, left, MSG_NOSIGNAL);
    if (n < 0) {
      if (errno == EINTR || errno == EAGAIN) continue;
      return fail(std::string("send failed: ") + strerror(errno));
    }
    p += n;
    left -= static_cast<size_t>(n);
  }
  return true;
}

bool Bootstrap::recv_msg(int sock, int op, void* data, size_t bytes, int* fd) {
  const int64_t deadline = now_ms() + timeout_ms_;
  Header h{};
  {
    iovec iov{&h, sizeof(h)};
    msghdr m{};
    m.msg_iov = &iov;
    m.msg_iovlen = 1;
    alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
    std::memset(ctrl, 0, sizeof(ctrl));
    m.msg_control = ctrl;
    m.msg_controllen = sizeof(ctrl);
    if (!wait_fd(sock, POLLIN, deadline)) return fail("timeout waiting for a peer (op " + std::to_string(op) + ")");
    const ssize_t n = recvmsg(sock, &m, MSG_WAITALL);
    if (n == 0) return fail("peer closed the connection");
    if (n != static_cast<ssize_t>(sizeof(h))) return fail(std::string("recvmsg failed: ") + strerror(errno));
    int got = -1;
    for (cmsghdr* c = CMSG_FIRSTHDR(&m); c != nullptr; c = CMSG_NXTHDR(&m, c)) {
      if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS) std::memcpy(&got, CMSG_DATA(c), sizeof(int));
    }
    if (fd != nullptr)
      *fd = got;
    else if (got >= 0)
      close(got);
  }
  if (h.magic != kMagic) return fail("bad magic (foreign or corrupted message)");
  if (h.op != op || h.seq != seq_)
    return fail("out-of-step message: expected op " + std::to_string(op) + " seq " + std::to_string(seq_) + ", got op " +
                std::to_string(h.op) + " seq " + std::to_string(h.seq) + " from rank " + std::to_string(h.rank));
  if (h.bytes != bytes) return fail("size mismatch between ranks");
  char* p = static_cast<char*>(data);
  size_t left = bytes;
  while (left > 0) {
    if (!wait_fd(sock, POLLIN, deadline)) return fail("timeout receiving payload");
    const ssize_t n = recv(sock, p, left, 0);
    if (n == 0) return fail("peer closed the connection");
    if (n < 0) {
      if (errno == EINTR || errno == EAGAIN) continue;
      return fail(std::string("recv failed: ") + strerror(errno));
    }
    p += n;
    left -= static_cast<size_t>(n);
  }
  return true;
}

Bootstrap* Bootstrap::create(int rank, int world, const std::string& key, int timeout_ms, std::string* err) {
  std::string clean;
  if (!sanitize_key(key, &clean, err)) return nullptr;
  if (world < 1 || rank < 0 || rank >= world) {
    if (err) *err = "bad rank/world";
    return nullptr;
  }
  Bootstrap* b = new Bootstrap();
  b->rank_ = rank;
  b->world_ = world;
  b->timeout_ms_ = timeout_ms > 0 ? timeout_ms : 30000;
  auto bail = [&](const std::string& what) -> Bootstrap* {
    if (err) *err = "bootstrap rank " + std::to_string(rank) + ": " + what;
    delete b;
    return nullptr;
  };
  if (world == 1) return b;
  sockaddr_un addr;
  const socklen_t alen = make_addr(clean, &addr);
  const int64_t deadline = now_ms() + b->timeout_ms_;
  if (rank == 0) {
    b->listen_fd_ = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (b->listen_fd_ < 0) return bail("socket() failed");
    if (bind(b->listen_fd_, reinterpret_cast<sockaddr*>(&addr), alen) != 0)
      return bail(std::string("bind failed (key in use?): ") + strerror(errno));
    if (listen(b->listen_fd_, world) != 0) return bail("listen failed");
    b->peer_fd_.assign(world, -1);
    for (int i = 1; i < world; ++i) {
      if (!wait_fd(b->listen_fd_, POLLIN, deadline))
        return bail("timeout: only " + std::to_string(i) + " of " + std::to_string(world) + " ranks joined");
      const int c = accept4(b->listen_fd_, nullptr, nullptr, SOCK_CLOEXEC);
      if (c < 0) return bail("accept failed");
      int32_t who = -1;
      if (!b->recv_msg(c, kOpHello, &who, sizeof(who), nullptr)) {
        close(c);
        return bail(b->err_);
      }
      if (who <= 0 || who >= world || b->peer_fd_[who] >= 0) {
        close(c);
        return bail("duplicate or invalid rank " + std::to_string(who) + " joined");
      }
      b->peer_fd_[who] = c;
    }
  } else {
    while (true) {
      b->hub_fd_ = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
      if (b->hub_fd_ < 0) return bail("socket() failed");
      if (connect(b->hub_fd_, reinterpret_cast<sockaddr*>(&addr), alen) == 0) break;
      close(b->hub_fd_);
      b->hub_fd_ = -1;
      if (now_ms() > deadline) return bail("timeout: rank 0 never opened the rendezvous");
      usleep(2000);
    }
    int32_t who = rank;
    if (!b->send_msg(b->hub_fd_, kOpHello, &who, sizeof(who), -1)) return bail(b->err_);
  }
  b->seq_ = 1;
  if (!b->barrier()) return bail(b->err_);
  return b;
}

Bootstrap::~Bootstrap() {
  if (listen_fd_ >= 0) close(listen_fd_);
  if (hub_fd_ >= 0) close(hub_fd_);
  for (int fd : peer_fd_)
    if (fd >= 0) close(fd);
}

bool Bootstrap::allgather(const void* in, void* out, size_t bytes) {
  char* o = static_cast<char*>(out);
  if (world_ == 1) {
    if (bytes) std::memcpy(o, in, bytes);
    return true;
  }
  ++seq_;
  if (rank_ == 0) {
    if (bytes) std::memcpy(o, in, bytes);
    for (int r = 1; r < world_; ++r)
      if (!recv_msg(peer_fd_[r], kOpGather, o + size_t(r) * bytes, bytes, nullptr)) return false;
    for (int r = 1; r < world_; ++r)
      if (!send_msg(peer_fd_[r], kOpGather, o, bytes * world_, -1)) return false;
    return true;
  }
  if (!send_msg(hub_fd_, kOpGather, in, bytes, -1)) return false;
  return recv_msg(hub_fd_, kOpGather, o, bytes * world_, nullptr);
}

bool Bootstrap::barrier() {
  std::vector<char> scratch(world_);
  char z = 0;
  return allgather(&z, scratch.data(), 1);
}

bool Bootstrap::exchange_fds(int my_fd, std::vector<int>* fds) {
  fds->assign(world_, -1);
  if (world_ == 1) {
    (*fds)[0] = my_fd >= 0 ? dup(my_fd) : -1;
    return true;
  }
  ++seq_;
  char z = 0;
  if (rank_ == 0) {
    (*fds)[0] = my_fd >= 0 ? dup(my_fd) : -1;
    for (int r = 1; r < world_; ++r)
      if (!recv_msg(peer_fd_[r], kOpFd, &z, 1, &(*fds)[r])) return false;
    for (int r = 1; r < world_; ++r)
      for (int s = 0; s < world_; ++s)
        if (!send_msg(peer_fd_[r], kOpFd, &z, 1, (*fds)[s])) return false;
    return true;
  }
  if (!send_msg(hub_fd_, kOpFd, &z, 1, my_fd)) return false;
  for (int s = 0; s < world_; ++s)
    if (!recv_msg(hub_fd_, kOpFd, &z, 1, &(*fds)[s])) return false;
  return true;
}

bool Bootstrap::broadcast_fd(int root, int* fd) {
  std::vector<int> all;
  if (!exchange_fds(rank_ == root ? *fd : -1, &all)) return false;
  for (int r = 0; r < world_; ++r) {
    if (r == root) continue;
    if (all[r] >= 0) close(all[r]);
  }
  if (rank_ == root) {
    if (all[root] >= 0) close(all[root]);
  } else {
    *fd = all[root];
  }
  return true;
}

}  // namespace oob
