// Host-only stress of the node-local rendezvous (csrc/runtime/bootstrap.cpp), meant to be built with
// -fsanitize=address,undefined and with -fsanitize=thread: `world` ranks run as threads of one process, many rounds,
// every primitive (all-gather, barrier, descriptor exchange, descriptor broadcast), plus a round in which one rank
// never shows up and the others must fail by their deadline without leaking.
//
// Capability parity: the reference's Broker has no such test (its waits are unbounded, src/system/broker.cpp:112-131).
#include <fcntl.h>
#include <sys/mman.h>
#include <unistd.h>

#include <atomic>
#include <cstdio>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "../../csrc/runtime/bootstrap.h"

namespace {

std::atomic<int> g_failures{0};

void fail(const char* what, int rank, int round) {
  std::fprintf(stderr, "FAIL %s (rank %d, round %d)\n", what, rank, round);
  g_failures.fetch_add(1);
}

int make_file_with(int value) {
  int fd = memfd_create("oob_stress", 0);
  if (fd < 0) return -1;
  if (write(fd, &value, sizeof(value)) != static_cast<ssize_t>(sizeof(value))) {
    close(fd);
    return -1;
  }
  return fd;
}

int read_value(int fd) {
  int v = -1;
  if (pread(fd, &v, sizeof(v), 0) != static_cast<ssize_t>(sizeof(v))) return -1;
  return v;
}

void rank_main(int rank, int world, const std::string& key, int round) {
  std::string err;
  oob::Bootstrap* b = oob::Bootstrap::create(rank, world, key, 20000, &err);
  if (b == nullptr) return fail(("create: " + err).c_str(), rank, round);
  struct Blob {
    int rank, round;
    char pad[56];
  } mine{};
  mine.rank = rank;
  mine.round = round;
  std::vector<Blob> all(world);
  if (!b->allgather(&mine, all.data(), sizeof(Blob))) fail("allgather", rank, round);
  for (int r = 0; r < world; ++r)
    if (all[r].rank != r || all[r].round != round) fail("allgather content", rank, round);
  if (!b->barrier()) fail("barrier", rank, round);
  int fd = make_file_with(1000 * round + rank);
  std::vector<int> fds;
  if (fd < 0 || !b->exchange_fds(fd, &fds) || static_cast<int>(fds.size()) != world) {
    fail("exchange_fds", rank, round);
  } else {
    for (int r = 0; r < world; ++r) {
      if (read_value(fds[r]) != 1000 * round + r) fail("exchange_fds content", rank, round);
      close(fds[r]);
    }
  }
  if (fd >= 0) close(fd);
  const int root = round % world;
  int bfd = rank == root ? make_file_with(77 + round) : -1;
  if (!b->broadcast_fd(root, &bfd) || bfd < 0 || read_value(bfd) != 77 + round) fail("broadcast_fd", rank, round);
  if (bfd >= 0) close(bfd);
  if (!b->barrier()) fail("barrier 2", rank, round);
  delete b;
}

}  // namespace

int main(int argc, char** argv) {
  const int world = argc > 1 ? std::atoi(argv[1]) : 4;
  const int rounds = argc > 2 ? std::atoi(argv[2]) : 20;
  const std::string base = "oobstress_" + std::to_string(getpid()) + "_";
  for (int round = 0; round < rounds; ++round) {
    std::vector<std::thread> th;
    const std::string key = base + std::to_string(round);
    for (int r = 0; r < world; ++r) th.emplace_back(rank_main, r, world, key, round);
    for (auto& t : th) t.join();
  }
  // One rank never arrives: the others give up by the deadline (300 ms) and report it.
  {
    std::vector<std::thread> th;
    std::atomic<int> refused{0};
    const std::string key = base + "absent";
    for (int r = 0; r < world - 1; ++r)
      th.emplace_back([&, r] {
        std::string err;
        oob::Bootstrap* b = oob::Bootstrap::create(r, world, key, 300, &err);
        if (b == nullptr && !err.empty()) refused.fetch_add(1);
        delete b;
      });
    for (auto& t : th) t.join();
    if (refused.load() != world - 1) fail("absent rank not detected", -1, -1);
  }
  if (g_failures.load() != 0) {
    std::fprintf(stderr, "%d failure(s)\n", g_failures.load());
    return 1;
  }
  std::printf("ok %d ranks x %d rounds\n", world, rounds);
  return 0;
}
