// Topology discovery: per device the SM count, memory, NUMA node, multicast
// (NVLS) and fd-export support; per directed device pair the P2P attributes
// and, optionally, live probes (remote load/store, remote atomic, and a timed
// peer copy for bandwidth) run with peer access enabled.
//
// Capability parity: src/topology/topology.cpp:652-941 (discover_link),
// :183-219 (NUMA node from sysfs), :1328 (JSON dump) and the probe kernels in
// src/topology/topology_probe.cu:108-238.  The bulk-copy-engine probes of the
// reference are replaced by what this library actually uses between GPUs:
// 128-bit ld/st, system-scope atomics and (reported as a capability only)
// multimem.  Host-staged "Shm" transport is not probed: on an NVSwitch machine
// every pair is directly connected, and a pair that is not is reported as
// "unsupported" instead of being routed through host memory.
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "../api/oob.h"
#include "../device/ptx.cuh"
#include "driver_api.h"
#include "errors.h"

namespace oob {
namespace {

__global__ void probe_ldst_kernel(uint32_t* remote, uint32_t* result, uint32_t token) {
  // remote store, remote load back
  remote[0] = token;
  __threadfence_system();
  result[0] = ptx::ld_relaxed_sys(remote);
}

__global__ void probe_atomic_kernel(uint32_t* remote, uint32_t* result) {
  result[0] = atomicAdd_system(remote, 7u);
  __threadfence_system();
  result[1] = ptx::ld_relaxed_sys(remote);
}

__global__ void probe_copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, size_t n) {
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x)
    ptx::st_v4(dst + i, ptx::ld_nc_v4(src + i));
}

int numa_node_of(int dev) {
  char bus[32] = {};
  if (cudaDeviceGetPCIBusId(bus, sizeof(bus), dev) != cudaSuccess) return -1;
  for (char* p = bus; *p; ++p)
    if (*p >= 'A' && *p <= 'Z') *p = char(*p - 'A' + 'a');
  std::string path = std::string("/sys/bus/pci/devices/") + bus + "/numa_node";
  FILE* f = std::fopen(path.c_str(), "r");
  if (f == nullptr) return -1;
  int node = -1;
  if (std::fscanf(f, "%d", &node) != 1) node = -1;
  std::fclose(f);
  return node;
}

void append(std::string* s, const char* fmt, ...) __attribute__((format(printf, 2, 3)));
void append(std::string* s, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  std::vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  s->append(buf);
}

struct PairProbe {
  int ldst = -1, atomic = -1;  // -1 not run, 0 failed, 1 ok
  double copy_gbs = 0.0;
};

PairProbe probe_pair(int src, int dst) {
  PairProbe out;
  // Kernels run on `src` and touch memory that lives on `dst`.
  uint32_t* remote = nullptr;
  uint32_t* result = nullptr;
  uint4 *big_remote = nullptr, *big_local = nullptr;
  const size_t big = size_t(64) << 20;
  cudaSetDevice(dst);
  if (cudaMalloc(&remote, 256) != cudaSuccess || cudaMalloc(&big_remote, big) != cudaSuccess) goto done;
  cudaMemset(remote, 0, 256);
  cudaDeviceSynchronize();
  cudaSetDevice(src);
  {
    cudaError_t e = cudaDeviceEnablePeerAccess(dst, 0);
    if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) {
      (void)cudaGetLastError();
      goto done;
    }
    (void)cudaGetLastError();
  }
  if (cudaMallocManaged(&result, 64) != cudaSuccess || cudaMalloc(&big_local, big) != cudaSuccess) goto done;
  std::memset(result, 0, 64);
  probe_ldst_kernel<<<1, 1>>>(remote, result, 0xB200u);
  if (cudaDeviceSynchronize() != cudaSuccess) goto done;
  out.ldst = result[0] == 0xB200u ? 1 : 0;
  probe_atomic_kernel<<<1, 1>>>(remote, result);
  if (cudaDeviceSynchronize() != cudaSuccess) goto done;
  out.atomic = (result[0] == 0xB200u && result[1] == 0xB200u + 7u) ? 1 : 0;
  {
    cudaEvent_t a, b;
    cudaEventCreate(&a);
    cudaEventCreate(&b);
    const size_t n = big / 16;
    for (int it = 0; it < 3; ++it) probe_copy_kernel<<<64, 512>>>(big_local, big_remote, n);
    cudaEventRecord(a);
    const int iters = 10;
    for (int it = 0; it < iters; ++it) probe_copy_kernel<<<64, 512>>>(big_local, big_remote, n);
    cudaEventRecord(b);
    if (cudaEventSynchronize(b) == cudaSuccess) {
      float ms = 0;
      cudaEventElapsedTime(&ms, a, b);
      if (ms > 0) out.copy_gbs = double(big) * iters / (ms * 1e-3) / 1e9;
    }
    cudaEventDestroy(a);
    cudaEventDestroy(b);
  }
done:
  (void)cudaGetLastError();
  cudaSetDevice(src);
  if (result) cudaFree(result);
  if (big_local) cudaFree(big_local);
  cudaSetDevice(dst);
  if (remote) cudaFree(remote);
  if (big_remote) cudaFree(big_remote);
  return out;
}

}  // namespace
}  // namespace oob

extern "C" int oob_topology_json(char* buf, uint64_t cap, int run_probes) {
  using namespace oob;
  if (buf == nullptr || cap == 0) return set_error(OOB_ERR_INVALID, "null buffer");
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    (void)cudaGetLastError();
    n = 0;
  }
  int prev = 0;
  if (n > 0) cudaGetDevice(&prev);
  const DriverApi* d = n > 0 ? driver_api() : nullptr;
  std::string s = "{\n  \"devices\": [";
  for (int i = 0; i < n; ++i) {
    cudaDeviceProp p{};
    cudaGetDeviceProperties(&p, i);
    int mc = 0, fd = 0;
    if (d != nullptr) {
      CUdevice dev;
      if (d->cuDeviceGet(&dev, i) == CUDA_SUCCESS) {
        d->cuDeviceGetAttribute(&mc, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev);
        d->cuDeviceGetAttribute(&fd, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, dev);
      }
    }
    append(&s,
           "%s\n    {\"index\": %d, \"name\": \"%s\", \"cc\": \"%d.%d\", \"sms\": %d, \"memory_bytes\": %zu, "
           "\"l2_bytes\": %d, \"numa_node\": %d, \"multicast\": %d, \"fd_handles\": %d}",
           i ? "," : "", i, p.name, p.major, p.minor, p.multiProcessorCount, size_t(p.totalGlobalMem), p.l2CacheSize,
           numa_node_of(i), mc, fd);
  }
  s += "\n  ],\n  \"links\": [";
  bool first = true;
  bool all_nvlink = n > 1;
  for (int a = 0; a < n; ++a) {
    for (int b = 0; b < n; ++b) {
      if (a == b) continue;
      int can = 0, atomics = 0, rank = -1;
      cudaDeviceCanAccessPeer(&can, a, b);
      cudaDeviceGetP2PAttribute(&atomics, cudaDevP2PAttrNativeAtomicSupported, a, b);
      cudaDeviceGetP2PAttribute(&rank, cudaDevP2PAttrPerformanceRank, a, b);
      (void)cudaGetLastError();
      // Same inference as the reference: NVLink iff native atomics and the best performance rank.
      const char* kind = !can ? "none" : (atomics && rank == 0 ? "nvlink" : "pcie");
      if (std::strcmp(kind, "nvlink") != 0) all_nvlink = false;
      PairProbe pr;
      if (run_probes && can) pr = probe_pair(a, b);
      append(&s,
             "%s\n    {\"src\": %d, \"dst\": %d, \"p2p\": %d, \"native_atomics\": %d, \"performance_rank\": %d, "
             "\"kind\": \"%s\", \"probe_ldst\": %d, \"probe_atomic\": %d, \"copy_gbs\": %.1f}",
             first ? "" : ",", a, b, can, atomics, rank, kind, pr.ldst, pr.atomic, pr.copy_gbs);
      first = false;
    }
  }
  append(&s, "\n  ],\n  \"all_pairs_nvlink\": %s,\n  \"device_count\": %d\n}\n", all_nvlink ? "true" : "false", n);
  if (n > 0) cudaSetDevice(prev);
  const uint64_t len = s.size() < cap - 1 ? s.size() : cap - 1;
  std::memcpy(buf, s.data(), len);
  buf[len] = 0;
  return OOB_OK;
}
