// oob_topology: prints the topology document of the visible GPUs.
//
// Capability parity: ooverlap_topology_cli (src/topology/topology_cli.cpp:24-114)
// with its --json / --no-probe switches; text mode prints a short table.
#include <cstdio>
#include <cstring>
#include <vector>
#include "../api/oob.h"

int main(int argc, char** argv) {
  bool probes = true, json = false;
  for (int i = 1; i < argc; ++i) {
    if (!std::strcmp(argv[i], "--no-probe")) probes = false;
    else if (!std::strcmp(argv[i], "--json")) json = true;
    else if (!std::strcmp(argv[i], "--help") || !std::strcmp(argv[i], "-h")) {
      std::printf("usage: oob_topology [--json] [--no-probe]\n");
      return 0;
    } else {
      std::fprintf(stderr, "unknown option %s\n", argv[i]);
      return 2;
    }
  }
  std::vector<char> buf(1 << 20);
  if (oob_topology_json(buf.data(), buf.size(), probes ? 1 : 0) != 0) {
    std::fprintf(stderr, "topology failed: %s\n", oob_last_error());
    return 1;
  }
  if (!json) std::printf("# %s\n", oob_version());
  std::fputs(buf.data(), stdout);
  return 0;
}
