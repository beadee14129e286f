// oob_topology: prints the topology document of the visible GPUs (or of the listed ones) as a table or as JSON.
//
// Capability parity: ooverlap_topology_cli (src/topology/topology_cli.cpp:24-114): --json, --no-enable-peer,
// --require-peer, --no-probe, --no-atomic-probe and a device list.  Its --no-tma-probe switches off the probe of
// the data path it uses between GPUs; here that path is multimem, 128-bit ld/st and bulk stores, so the matching
// switches are --no-multimem-probe, --no-copy-probe and --no-bulk-probe (--no-tma-probe is accepted as its alias).  --no-shm is accepted and ignored: no host-staged transport exists here.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>
#include "../api/oob.h"

static void usage(const char* argv0) {
  std::printf(
      "usage: %s [--json] [--no-probe] [--no-enable-peer] [--no-atomic-probe] [--no-copy-probe]\n"
      "          [--no-multimem-probe] [--no-bulk-probe] [--require-peer] [--no-shm] [device ...]\n"
      "  --json               JSON document instead of the table\n"
      "  --no-probe           attributes only: no kernel runs, no memory is allocated\n"
      "  --no-enable-peer     do not switch peer access on (implies no per-pair probes)\n"
      "  --no-atomic-probe    skip the remote-atomic probe\n"
      "  --no-copy-probe      skip the timed 64 MiB peer copy\n"
      "  --no-multimem-probe  skip the multicast (NVLS) probe\n"
      "  --no-bulk-probe      skip the bulk-store probe (shared memory -> peer memory; alias --no-tma-probe)\n"
      "  --require-peer       exit 1 unless every listed pair has peer access\n"
      "  device ...           indices to describe (default: all visible devices)\n",
      argv0);
}

int main(int argc, char** argv) {
  unsigned flags = OOB_TOPO_PROBES | OOB_TOPO_TEXT;
  std::vector<int> devices;
  for (int i = 1; i < argc; ++i) {
    const char* a = argv[i];
    if (!std::strcmp(a, "--json")) flags &= ~OOB_TOPO_TEXT;
    else if (!std::strcmp(a, "--no-probe")) flags &= ~OOB_TOPO_PROBES;
    else if (!std::strcmp(a, "--no-enable-peer")) flags |= OOB_TOPO_NO_ENABLE_PEER;
    else if (!std::strcmp(a, "--no-atomic-probe")) flags |= OOB_TOPO_NO_ATOMIC_PROBE;
    else if (!std::strcmp(a, "--no-copy-probe")) flags |= OOB_TOPO_NO_COPY_PROBE;
    else if (!std::strcmp(a, "--no-multimem-probe")) flags |= OOB_TOPO_NO_MULTIMEM_PROBE;
    else if (!std::strcmp(a, "--no-bulk-probe") || !std::strcmp(a, "--no-tma-probe")) flags |= OOB_TOPO_NO_BULK_PROBE;
    else if (!std::strcmp(a, "--require-peer")) flags |= OOB_TOPO_REQUIRE_PEER;
    else if (!std::strcmp(a, "--no-shm")) continue;
    else if (!std::strcmp(a, "--help") || !std::strcmp(a, "-h")) {
      usage(argv[0]);
      return 0;
    } else {
      char* end = nullptr;
      const long v = std::strtol(a, &end, 10);
      if (end == a || *end != 0 || v < 0) {
        std::fprintf(stderr, "unknown option %s\n", a);
        usage(argv[0]);
        return 2;
      }
      devices.push_back(int(v));
    }
  }
  std::vector<char> buf(1 << 20);
  if (oob_topology_describe(buf.data(), buf.size(), flags, devices.empty() ? nullptr : devices.data(),
                            int(devices.size())) != 0) {
    std::fprintf(stderr, "topology discovery failed: %s\n", oob_last_error());
    return 1;
  }
  if (flags & OOB_TOPO_TEXT) std::printf("# %s\n", oob_version());
  std::fputs(buf.data(), stdout);
  return 0;
}
