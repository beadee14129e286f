// Host-only driver for the tuning-policy parser and selector (csrc/runtime/policy.cpp), meant to be built with
// -fsanitize=address,undefined: loads every file named on the command line (valid, truncated or mutated JSON) and
// queries the selector over a grid of sizes.  Any outcome is fine except memory errors and crashes.
#include <cstdint>
#include <cstdio>
#include <string>

#include "../../csrc/api/oob.h"
#include "../../csrc/runtime/errors.h"

namespace oob {
// The library's error sink lives in comm.cpp (not part of this host-only build).
static std::string g_err;
int set_error(int code, const std::string& msg) {
  g_err = msg;
  return code;
}
int cuda_fail(cudaError_t, const char* what) { return set_error(OOB_ERR_CUDA, what); }
}  // namespace oob

int main(int argc, char** argv) {
  int loaded = 0, rejected = 0;
  unsigned long checksum = 0;
  for (int i = 1; i < argc; ++i) {
    const int rc = oob_policy_load(argv[i]);
    if (rc == OOB_OK)
      ++loaded;
    else
      ++rejected;
    for (int world : {2, 4, 8, 16})
      for (int coll = 0; coll < 3; ++coll)
        for (int nvls = 0; nvls < 2; ++nvls)
          for (uint64_t bytes = 1; bytes <= (1ull << 32); bytes <<= 3) {
            int algo = -7, ctas = -7;
            const int s = oob_policy_select(world, coll, bytes, nvls, &algo, &ctas);
            if (s == OOB_OK) {
              if (ctas < 1 || ctas > 4096 || algo < 0 || algo > 16) {
                std::fprintf(stderr, "implausible selection algo=%d ctas=%d from %s\n", algo, ctas, argv[i]);
                return 2;
              }
              checksum = checksum * 31 + static_cast<unsigned>(algo * 131 + ctas);
            }
          }
  }
  std::printf("ok loaded=%d rejected=%d checksum=%lu\n", loaded, rejected, checksum);
  return 0;
}
