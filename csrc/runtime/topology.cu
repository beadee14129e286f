// Topology discovery: per device the SM count, memory, NUMA node, multicast
// (NVLS) and fd-export support; per directed device pair the P2P attributes
// and, optionally, live probes (remote load/store, remote atomic, and a timed
// peer copy for bandwidth) run with peer access enabled.
//
// Capability parity: src/topology/topology.cpp:652-941 (discover_link),
// :183-219 (NUMA node from sysfs), :1328 (JSON dump) and the probe kernels in
// src/topology/topology_probe.cu:108-238.  The bulk-copy-engine probes of the
// reference are replaced by what this library actually uses between GPUs:
// 128-bit ld/st, system-scope atomics, bulk stores from shared memory and multimem (a live probe through a
// multicast object over all listed devices: multimem.st, multimem.red and
// multimem.ld_reduce, each checked from every device's own memory).
// Host-staged "Shm" transport is not probed: on an NVSwitch machine every pair
// is directly connected, and a pair that is not is reported as "none" (and
// fails the call under OOB_TOPO_REQUIRE_PEER) instead of being routed through
// host memory.
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

// Untiled bulk store (the copy engine path the one-SM fused GEMM uses for its pushed tiles, here without a tensor map):
// 4 KiB from shared memory of an SM of the source device into memory of the destination device, then a load back.
__global__ void probe_bulk_store_kernel(uint32_t* remote, uint32_t* result, uint32_t token) {
  __shared__ __align__(128) uint32_t tile[1024];
  for (int i = threadIdx.x; i < 1024; i += blockDim.x) tile[i] = token + uint32_t(i);
  __syncthreads();
  if (threadIdx.x == 0) {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes before the async-proxy read
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(remote),
                 "r"(static_cast<uint32_t>(__cvta_generic_to_shared(tile))), "r"(4096u)
                 : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    __threadfence_system();
    uint32_t bad = 0;
    for (int i = 0; i < 1024; i += 101) bad += ptx::ld_relaxed_sys(remote + i) != token + uint32_t(i);
    result[0] = bad;
  }
}

// One thread: store a token to word 0 of every bound device, add 5 to word 1 of every bound device.
__global__ void probe_multimem_write_kernel(uint32_t* mc, uint32_t token) {
  asm volatile("multimem.st.relaxed.sys.global.u32 [%0], %1;" ::"l"(mc), "r"(token) : "memory");
  asm volatile("multimem.red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(mc + 1), "r"(5u) : "memory");
  __threadfence_system();
}

// One thread: the sum over all bound devices of word 2 (each device wrote its index + 1 there).
__global__ void probe_multimem_reduce_kernel(const uint32_t* mc, uint32_t* result) {
  uint32_t v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.u32 %0, [%1];" : "=r"(v) : "l"(mc + 2) : "memory");
  result[0] = v;
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
  int ldst = -1, atomic = -1, bulk = -1;  // -1 not run, 0 failed, 1 ok
  double copy_gbs = 0.0;
};

PairProbe probe_pair(int src, int dst, unsigned flags) {
  PairProbe out;
  // Kernels run on `src` and touch memory that lives on `dst`.
  uint32_t* remote = nullptr;
  uint32_t* result = nullptr;
  uint4 *big_remote = nullptr, *big_local = nullptr;
  const bool copy = !(flags & OOB_TOPO_NO_COPY_PROBE);
  const size_t big = size_t(64) << 20;
  cudaSetDevice(dst);
  if (cudaMalloc(&remote, 8192) != cudaSuccess || (copy && cudaMalloc(&big_remote, big) != cudaSuccess)) goto done;
  cudaMemset(remote, 0, 8192);
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
  if (cudaMallocManaged(&result, 64) != cudaSuccess || (copy && cudaMalloc(&big_local, big) != cudaSuccess)) goto done;
  std::memset(result, 0, 64);
  probe_ldst_kernel<<<1, 1>>>(remote, result, 0xB200u);
  if (cudaDeviceSynchronize() != cudaSuccess) goto done;
  out.ldst = result[0] == 0xB200u ? 1 : 0;
  if (!(flags & OOB_TOPO_NO_ATOMIC_PROBE)) {
    probe_atomic_kernel<<<1, 1>>>(remote, result);
    if (cudaDeviceSynchronize() != cudaSuccess) goto done;
    out.atomic = (result[0] == 0xB200u && result[1] == 0xB200u + 7u) ? 1 : 0;
  }
  if (!(flags & OOB_TOPO_NO_BULK_PROBE)) {
    result[0] = 0xffffffffu;
    probe_bulk_store_kernel<<<1, 128>>>(remote + 1024, result, 0xB2000000u);  // 4 KiB past the words of the other probes
    if (cudaDeviceSynchronize() != cudaSuccess) goto done;
    out.bulk = result[0] == 0u ? 1 : 0;
  }
  if (copy) {
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

// Live multimem probe over `devs` (at least two devices that all report multicast support): one multicast object of
// one granule, one granule of physical memory per device bound to it, then
//   * device devs[0] stores a token and adds 5 through the multicast address; every device must find both in its own
//     memory,
//   * every device writes index + 1 into its own word 2; devs[0] reads the in-switch sum of word 2.
// Returns 1 ok, 0 a check failed, -1 the probe could not be set up (`why` says which call refused).
int probe_multimem(const std::vector<int>& devs, std::string* why) {
  const DriverApi* d = driver_api();
  const int n = int(devs.size());
  if (d == nullptr || d->cuMulticastCreate == nullptr || n < 2) {
    *why = "needs two or more devices and the multicast driver entry points";
    return -1;
  }
  std::vector<CUmemGenericAllocationHandle> mem(n);
  std::vector<char> have(n, 0), bound(n, 0);
  std::vector<CUdeviceptr> va(n, 0);
  CUmemGenericAllocationHandle mc = 0;
  bool have_mc = false;
  CUdeviceptr mc_va = 0;
  bool mc_mapped = false;
  uint32_t* result = nullptr;
  int verdict = -1;
  size_t gran = 0;
  CUresult r = CUDA_SUCCESS;
  auto fail = [&](const char* what) {
    const char* msg = nullptr;
    if (d->cuGetErrorString) d->cuGetErrorString(r, &msg);
    *why = std::string(what) + ": " + (msg ? msg : "error");
  };

  CUmulticastObjectProp mprop{};
  mprop.numDevices = unsigned(n);
  mprop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  mprop.size = 2u << 20;
  r = d->cuMulticastGetGranularity(&gran, &mprop, CU_MULTICAST_GRANULARITY_RECOMMENDED);
  if (r != CUDA_SUCCESS || gran == 0) { fail("cuMulticastGetGranularity"); return -1; }
  mprop.size = gran;
  for (int i = 0; i < n; ++i) {  // primary contexts must exist before devices join the object
    cudaSetDevice(devs[i]);
    cudaFree(nullptr);
  }
  r = d->cuMulticastCreate(&mc, &mprop);
  if (r != CUDA_SUCCESS) { fail("cuMulticastCreate"); return -1; }
  have_mc = true;
  for (int i = 0; i < n; ++i) {
    CUdevice dev;
    r = d->cuDeviceGet(&dev, devs[i]);
    if (r == CUDA_SUCCESS) r = d->cuMulticastAddDevice(mc, dev);
    if (r != CUDA_SUCCESS) { fail("cuMulticastAddDevice"); goto cleanup; }
  }
  for (int i = 0; i < n; ++i) {
    CUmemAllocationProp prop{};
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = devs[i];
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    CUmemAccessDesc acc{};
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = devs[i];
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    r = d->cuMemCreate(&mem[i], gran, &prop, 0);
    if (r != CUDA_SUCCESS) { fail("cuMemCreate"); goto cleanup; }
    have[i] = 1;
    r = d->cuMemAddressReserve(&va[i], gran, gran, 0, 0);
    if (r != CUDA_SUCCESS) { va[i] = 0; fail("cuMemAddressReserve"); goto cleanup; }
    r = d->cuMemMap(va[i], gran, 0, mem[i], 0);
    if (r == CUDA_SUCCESS) r = d->cuMemSetAccess(va[i], gran, &acc, 1);
    if (r != CUDA_SUCCESS) { fail("mapping the probe memory"); goto cleanup; }
    cudaSetDevice(devs[i]);
    const uint32_t init[4] = {0u, 0u, uint32_t(i + 1), 0u};
    if (cudaMemcpy(reinterpret_cast<void*>(va[i]), init, sizeof(init), cudaMemcpyHostToDevice) != cudaSuccess) {
      *why = "initialising the probe memory failed";
      goto cleanup;
    }
    r = d->cuMulticastBindMem(mc, 0, mem[i], 0, gran, 0);
    if (r != CUDA_SUCCESS) { fail("cuMulticastBindMem"); goto cleanup; }
    bound[i] = 1;
  }
  {
    std::vector<CUmemAccessDesc> acc(n);
    for (int i = 0; i < n; ++i) {
      acc[i].location.type = CU_MEM_LOCATION_TYPE_DEVICE;
      acc[i].location.id = devs[i];
      acc[i].flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    }
    r = d->cuMemAddressReserve(&mc_va, gran, gran, 0, 0);
    if (r != CUDA_SUCCESS) { mc_va = 0; fail("cuMemAddressReserve(multicast)"); goto cleanup; }
    r = d->cuMemMap(mc_va, gran, 0, mc, 0);
    if (r == CUDA_SUCCESS) {
      mc_mapped = true;
      r = d->cuMemSetAccess(mc_va, gran, acc.data(), size_t(n));
    }
    if (r != CUDA_SUCCESS) { fail("mapping the multicast object"); goto cleanup; }
  }
  cudaSetDevice(devs[0]);
  if (cudaMallocManaged(&result, 64) != cudaSuccess) { *why = "cudaMallocManaged failed"; goto cleanup; }
  result[0] = 0;
  probe_multimem_write_kernel<<<1, 1>>>(reinterpret_cast<uint32_t*>(mc_va), 0xB200u);
  if (cudaDeviceSynchronize() != cudaSuccess) { *why = "the multimem store kernel failed"; goto cleanup; }
  probe_multimem_reduce_kernel<<<1, 1>>>(reinterpret_cast<const uint32_t*>(mc_va), result);
  if (cudaDeviceSynchronize() != cudaSuccess) { *why = "the multimem reduce kernel failed"; goto cleanup; }
  verdict = result[0] == uint32_t(n * (n + 1) / 2) ? 1 : 0;
  if (!verdict) *why = "multimem.ld_reduce returned a wrong sum";
  for (int i = 0; i < n && verdict == 1; ++i) {
    uint32_t got[2] = {0, 0};
    cudaSetDevice(devs[i]);
    if (cudaMemcpy(got, reinterpret_cast<void*>(va[i]), sizeof(got), cudaMemcpyDeviceToHost) != cudaSuccess ||
        got[0] != 0xB200u || got[1] != 5u) {
      verdict = 0;
      *why = "device " + std::to_string(devs[i]) + " did not receive the multimem store / add";
    }
  }
cleanup:
  (void)cudaGetLastError();
  if (result) {
    cudaSetDevice(devs[0]);
    cudaFree(result);
  }
  if (mc_mapped) d->cuMemUnmap(mc_va, gran);
  if (mc_va) d->cuMemAddressFree(mc_va, gran);
  for (int i = 0; i < n; ++i) {
    if (bound[i]) {
      CUdevice dev;
      if (d->cuDeviceGet(&dev, devs[i]) == CUDA_SUCCESS) d->cuMulticastUnbind(mc, dev, 0, gran);
    }
    if (va[i]) {
      if (have[i]) d->cuMemUnmap(va[i], gran);
      d->cuMemAddressFree(va[i], gran);
    }
    if (have[i]) d->cuMemRelease(mem[i]);
  }
  if (have_mc) d->cuMemRelease(mc);
  return verdict;
}

struct DeviceRow {
  int index = 0, major = 0, minor = 0, sms = 0, l2 = 0, numa = -1, multicast = 0, fd = 0;
  size_t mem = 0;
  std::string name;
};
struct LinkRow {
  int src = 0, dst = 0, p2p = 0, atomics = 0, rank = -1;
  const char* kind = "none";
  PairProbe probe;
};
struct TopoDoc {
  std::vector<DeviceRow> devices;
  std::vector<LinkRow> links;
  bool all_nvlink = false, all_p2p = false;
  int multimem = -1;  // -1 not run / not set up, 0 failed, 1 ok
  std::string multimem_note;
};

// Returns OOB_OK or an error code with the message set.
int discover(unsigned flags, const int* devices, int n_devices, TopoDoc* doc) {
  int visible = 0;
  if (cudaGetDeviceCount(&visible) != cudaSuccess) {
    (void)cudaGetLastError();
    visible = 0;
  }
  std::vector<int> devs;
  if (devices != nullptr && n_devices > 0) {
    for (int i = 0; i < n_devices; ++i) {
      if (devices[i] < 0 || devices[i] >= visible)
        return set_error(OOB_ERR_INVALID, "device " + std::to_string(devices[i]) + " is not visible (" +
                                              std::to_string(visible) + " devices)");
      for (int j = 0; j < i; ++j)
        if (devices[j] == devices[i]) return set_error(OOB_ERR_INVALID, "device listed twice");
      devs.push_back(devices[i]);
    }
  } else {
    for (int i = 0; i < visible; ++i) devs.push_back(i);
  }
  const int n = int(devs.size());
  int prev = 0;
  if (n > 0) cudaGetDevice(&prev);
  const DriverApi* d = n > 0 ? driver_api() : nullptr;
  bool all_mc = n > 1;
  for (int i : devs) {
    cudaDeviceProp p{};
    cudaGetDeviceProperties(&p, i);
    DeviceRow row;
    row.index = i;
    row.name = p.name;
    row.major = p.major;
    row.minor = p.minor;
    row.sms = p.multiProcessorCount;
    row.mem = size_t(p.totalGlobalMem);
    row.l2 = p.l2CacheSize;
    row.numa = numa_node_of(i);
    if (d != nullptr) {
      CUdevice dev;
      if (d->cuDeviceGet(&dev, i) == CUDA_SUCCESS) {
        d->cuDeviceGetAttribute(&row.multicast, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev);
        d->cuDeviceGetAttribute(&row.fd, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, dev);
      }
    }
    if (!row.multicast) all_mc = false;
    doc->devices.push_back(row);
  }
  const bool probes = (flags & OOB_TOPO_PROBES) && !(flags & OOB_TOPO_NO_ENABLE_PEER);
  doc->all_nvlink = n > 1;
  doc->all_p2p = n > 1;
  for (int a : devs) {
    for (int b : devs) {
      if (a == b) continue;
      LinkRow l;
      l.src = a;
      l.dst = b;
      cudaDeviceCanAccessPeer(&l.p2p, a, b);
      cudaDeviceGetP2PAttribute(&l.atomics, cudaDevP2PAttrNativeAtomicSupported, a, b);
      cudaDeviceGetP2PAttribute(&l.rank, cudaDevP2PAttrPerformanceRank, a, b);
      (void)cudaGetLastError();
      // Same inference as the reference: NVLink iff native atomics and the best performance rank.
      l.kind = !l.p2p ? "none" : (l.atomics && l.rank == 0 ? "nvlink" : "pcie");
      if (std::strcmp(l.kind, "nvlink") != 0) doc->all_nvlink = false;
      if (!l.p2p) doc->all_p2p = false;
      if (probes && l.p2p) l.probe = probe_pair(a, b, flags);
      doc->links.push_back(l);
    }
  }
  if ((flags & OOB_TOPO_PROBES) && !(flags & OOB_TOPO_NO_MULTIMEM_PROBE)) {
    if (all_mc && doc->all_p2p) doc->multimem = probe_multimem(devs, &doc->multimem_note);
    else doc->multimem_note = n < 2 ? "needs two or more devices" : "not every device supports multicast with peer access";
  } else {
    doc->multimem_note = "not run";
  }
  if (n > 0) cudaSetDevice(prev);
  if ((flags & OOB_TOPO_REQUIRE_PEER) && n > 1 && !doc->all_p2p) {
    std::string bad;
    for (const LinkRow& l : doc->links)
      if (!l.p2p) bad += (bad.empty() ? "" : ", ") + std::to_string(l.src) + "->" + std::to_string(l.dst);
    return set_error(OOB_ERR_UNSUPPORTED, "peer access is required but missing for " + bad);
  }
  return OOB_OK;
}

std::string to_json(const TopoDoc& doc) {
  std::string s = "{\n  \"devices\": [";
  bool first = true;
  for (const DeviceRow& r : doc.devices) {
    append(&s,
           "%s\n    {\"index\": %d, \"name\": \"%s\", \"cc\": \"%d.%d\", \"sms\": %d, \"memory_bytes\": %zu, "
           "\"l2_bytes\": %d, \"numa_node\": %d, \"multicast\": %d, \"fd_handles\": %d}",
           first ? "" : ",", r.index, r.name.c_str(), r.major, r.minor, r.sms, r.mem, r.l2, r.numa, r.multicast, r.fd);
    first = false;
  }
  s += "\n  ],\n  \"links\": [";
  first = true;
  for (const LinkRow& l : doc.links) {
    append(&s,
           "%s\n    {\"src\": %d, \"dst\": %d, \"p2p\": %d, \"native_atomics\": %d, \"performance_rank\": %d, "
           "\"kind\": \"%s\", \"probe_ldst\": %d, \"probe_atomic\": %d, \"probe_bulk_store\": %d, \"copy_gbs\": %.1f}",
           first ? "" : ",", l.src, l.dst, l.p2p, l.atomics, l.rank, l.kind, l.probe.ldst, l.probe.atomic, l.probe.bulk,
           l.probe.copy_gbs);
    first = false;
  }
  std::string note;
  for (char c : doc.multimem_note) note += (c == '"' || c == '\\') ? '\'' : c;
  append(&s, "\n  ],\n  \"all_pairs_nvlink\": %s,\n  \"all_pairs_p2p\": %s,\n  \"probe_multimem\": %d,\n",
         doc.all_nvlink ? "true" : "false", doc.all_p2p ? "true" : "false", doc.multimem);
  s += "  \"probe_multimem_note\": \"" + note + "\",\n";
  append(&s, "  \"device_count\": %d\n}\n", int(doc.devices.size()));
  return s;
}

const char* tri(int v) { return v < 0 ? "-" : (v ? "ok" : "FAIL"); }

std::string to_text(const TopoDoc& doc) {
  std::string s;
  append(&s, "%d device(s)\n", int(doc.devices.size()));
  append(&s, "%-4s %-28s %-5s %-4s %-9s %-7s %-5s %-9s %s\n", "dev", "name", "cc", "SMs", "memory", "L2", "NUMA",
         "multicast", "fd handles");
  for (const DeviceRow& r : doc.devices)
    append(&s, "%-4d %-28.28s %d.%-3d %-4d %-6.1f GB %-4d MB %-5d %-9s %s\n", r.index, r.name.c_str(), r.major, r.minor,
           r.sms, double(r.mem) / 1e9, r.l2 >> 20, r.numa, r.multicast ? "yes" : "no", r.fd ? "yes" : "no");
  if (!doc.links.empty()) {
    append(&s, "\n%-9s %-7s %-4s %-8s %-5s %-6s %-7s %-5s %s\n", "src->dst", "kind", "p2p", "atomics", "rank", "ld/st",
           "atomic", "bulk", "copy GB/s");
    for (const LinkRow& l : doc.links)
      append(&s, "%3d->%-4d %-7s %-4s %-8s %-5d %-6s %-7s %-5s %.1f\n", l.src, l.dst, l.kind, l.p2p ? "yes" : "no",
             l.atomics ? "native" : "no", l.rank, tri(l.probe.ldst), tri(l.probe.atomic), tri(l.probe.bulk),
             l.probe.copy_gbs);
  }
  append(&s, "\nall pairs NVLink: %s   all pairs peer access: %s   multimem probe: %s", doc.all_nvlink ? "yes" : "no",
         doc.all_p2p ? "yes" : "no", tri(doc.multimem));
  if (doc.multimem != 1 && !doc.multimem_note.empty()) s += " (" + doc.multimem_note + ")";
  s += "\n";
  return s;
}

}  // namespace
}  // namespace oob

extern "C" int oob_topology_describe(char* buf, uint64_t cap, unsigned flags, const int* devices, int n_devices) {
  using namespace oob;
  if (buf == nullptr || cap == 0) return set_error(OOB_ERR_INVALID, "null buffer");
  TopoDoc doc;
  const int rc = discover(flags, devices, n_devices, &doc);
  if (rc != OOB_OK) {
    buf[0] = 0;
    return rc;
  }
  const std::string s = (flags & OOB_TOPO_TEXT) ? to_text(doc) : to_json(doc);
  const uint64_t len = s.size() < cap - 1 ? s.size() : cap - 1;
  std::memcpy(buf, s.data(), len);
  buf[len] = 0;
  return OOB_OK;
}

extern "C" int oob_topology_json(char* buf, uint64_t cap, int run_probes) {
  return oob_topology_describe(buf, cap, run_probes ? OOB_TOPO_PROBES : 0u, nullptr, 0);
}
