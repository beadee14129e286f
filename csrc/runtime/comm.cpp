#include "comm.h"

#include <unistd.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "../api/oob.h"
#include "../api/oob_model.h"
#include "../collectives/collectives.h"
#include "../gemm/gemm.h"
#include "../gemm/gemm_pair.h"
#include "driver_api.h"
#include "errors.h"
#include "log.h"

using namespace oob;

// ---------------------------------------------------------------------------
// helpers
// ---------------------------------------------------------------------------
namespace oob {

thread_local std::string g_last_error;

int set_error(int code, const std::string& msg) {
  g_last_error = msg;
  OOB_LOG(kLogInfo, "error %d: %s", code, msg.c_str());
  return code;
}

int cuda_fail(cudaError_t e, const char* what) {
  (void)cudaGetLastError();
  return set_error(OOB_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}

static std::string cu_str(const DriverApi* d, CUresult r) {
  const char* s = nullptr;
  if (d && d->cuGetErrorString) d->cuGetErrorString(r, &s);
  return s ? s : ("CUresult " + std::to_string(int(r)));
}

}  // namespace oob

CommCtx oob_comm::make_ctx() const {
  CommCtx c{};
  c.world = world;
  c.rank = rank;
  for (int r = 0; r < world; ++r) c.pad[r] = reinterpret_cast<uint32_t*>(heap[r]);
  c.pad_mc = heap_mc ? reinterpret_cast<uint32_t*>(heap_mc) : nullptr;
  c.status = status_dev;
  c.timeout_ns = timeout_ns;
  c.emu_table = emulated ? emu_table_dev : nullptr;
  return c;
}

bool oob_comm::peer_ptrs(int reg, uint64_t off, uint64_t bytes, PeerPtrs* out) const {
  std::memset(out, 0, sizeof(*out));
  if (reg == 0) {
    if (off > heap_bytes || bytes > heap_bytes - off) return false;
    for (int r = 0; r < world; ++r) out->p[r] = heap[r] + off;
    out->mc = heap_mc ? heap_mc + off : nullptr;
    return true;
  }
  auto it = regs.find(reg);
  if (it == regs.end() || off > it->second.bytes || bytes > it->second.bytes - off) return false;
  for (int r = 0; r < world; ++r) out->p[r] = static_cast<char*>(it->second.peer[r]) + off;
  out->mc = nullptr;
  return true;
}

namespace {

constexpr uint64_t kAllocAlign = 1024;

uint64_t round_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

void allocator_init(oob_comm* c) {
  c->live.clear();
  c->free_blocks.clear();
  const uint64_t start = round_up(kPadBytes, kAllocAlign);
  if (c->heap_bytes > start) c->free_blocks[start] = c->heap_bytes - start;
}

int refresh_emu_table(oob_comm* c) {
  if (!c->emulated) return OOB_OK;
  std::vector<CommCtx> table(c->world);
  for (int r = 0; r < c->world; ++r) {
    CommCtx x = c->make_ctx();
    x.rank = r;
    x.emu_table = nullptr;
    x.status = c->status_dev + r;
    table[r] = x;
  }
  cudaError_t e = cudaMemcpy(c->emu_table_dev, table.data(), sizeof(CommCtx) * c->world, cudaMemcpyHostToDevice);
  if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpy(emu table)");
  return OOB_OK;
}

int alloc_status(oob_comm* c, int n) {
  cudaError_t e = cudaHostAlloc(reinterpret_cast<void**>(&c->status_host), sizeof(DeviceStatus) * n, cudaHostAllocMapped);
  if (e != cudaSuccess) return cuda_fail(e, "cudaHostAlloc(status)");
  std::memset(c->status_host, 0, sizeof(DeviceStatus) * n);
  e = cudaHostGetDevicePointer(reinterpret_cast<void**>(&c->status_dev), c->status_host, 0);
  if (e != cudaSuccess) return cuda_fail(e, "cudaHostGetDevicePointer(status)");
  return OOB_OK;
}

// Collective agreement: true only if every rank passed `ok`.
bool all_agree(oob_comm* c, bool ok) {
  if (c->boot == nullptr || c->world == 1) return ok;
  char mine = ok ? 1 : 0;
  std::vector<char> all(c->world);
  if (!c->boot->allgather(&mine, all.data(), 1)) return false;
  for (char v : all)
    if (!v) return false;
  return true;
}

void release_vmm(oob_comm* c) {
  const DriverApi* d = driver_api();
  if (d == nullptr) return;
  if (c->heap_mc) {
    d->cuMemUnmap(reinterpret_cast<CUdeviceptr>(c->heap_mc), c->map_bytes);
    d->cuMemAddressFree(reinterpret_cast<CUdeviceptr>(c->heap_mc), c->map_bytes);
    c->heap_mc = nullptr;
  }
  if (c->mc_bound && d->cuMulticastUnbind) {
    CUdevice dev;
    if (d->cuDeviceGet(&dev, c->device) == CUDA_SUCCESS) d->cuMulticastUnbind(c->mc_handle, dev, 0, c->map_bytes);
    c->mc_bound = false;
  }
  if (c->mc_valid) {
    d->cuMemRelease(c->mc_handle);
    c->mc_valid = false;
  }
  for (int r = 0; r < c->world; ++r) {
    if (c->memory_kind == 0 && c->heap[r]) {
      d->cuMemUnmap(reinterpret_cast<CUdeviceptr>(c->heap[r]), c->map_bytes);
      d->cuMemAddressFree(reinterpret_cast<CUdeviceptr>(c->heap[r]), c->map_bytes);
      c->heap[r] = nullptr;
    }
    if (c->handle_valid[r]) {
      d->cuMemRelease(c->handles[r]);
      c->handle_valid[r] = false;
    }
  }
}

// VMM path: one physical allocation per rank exported as a POSIX fd, mapped by everybody.
int setup_vmm(oob_comm* c, unsigned flags, std::string* why) {
  const DriverApi* d = driver_api();
  if (d == nullptr) {
    *why = "CUDA driver entry points unavailable";
    return OOB_ERR_UNSUPPORTED;
  }
  CUdevice dev;
  CUresult r = d->cuDeviceGet(&dev, c->device);
  if (r != CUDA_SUCCESS) {
    *why = "cuDeviceGet: " + cu_str(d, r);
    return OOB_ERR_CUDA;
  }
  int fd_ok = 0, mc_ok = 0;
  d->cuDeviceGetAttribute(&fd_ok, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, dev);
  d->cuDeviceGetAttribute(&mc_ok, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev);
  if (!fd_ok) {
    *why = "device cannot export POSIX file descriptor handles";
    return OOB_ERR_UNSUPPORTED;
  }
  const bool want_mc = mc_ok && !(flags & OOB_FLAG_NO_NVLS) && c->world > 1 && d->cuMulticastCreate != nullptr &&
                       std::getenv("OOB_DISABLE_NVLS") == nullptr;

  CUmemAllocationProp prop{};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = c->device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t gran = 0;
  r = d->cuMemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
  if (r != CUDA_SUCCESS || gran == 0) gran = 2u << 20;
  CUmulticastObjectProp mprop{};
  mprop.numDevices = static_cast<unsigned>(c->world);
  mprop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  mprop.flags = 0;
  if (want_mc) {
    size_t mgran = 0;
    mprop.size = round_up(c->heap_bytes, gran);
    if (d->cuMulticastGetGranularity(&mgran, &mprop, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mgran > gran)
      gran = mgran;
  }
  c->map_bytes = round_up(c->heap_bytes, gran);
  c->heap_bytes = c->map_bytes;
  mprop.size = c->map_bytes;

  // 1. local physical memory + export
  bool ok = true;
  int my_fd = -1;
  r = d->cuMemCreate(&c->handles[c->rank], c->map_bytes, &prop, 0);
  if (r != CUDA_SUCCESS) {
    *why = "cuMemCreate: " + cu_str(d, r);
    ok = false;
  } else {
    c->handle_valid[c->rank] = true;
    r = d->cuMemExportToShareableHandle(&my_fd, c->handles[c->rank], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
    if (r != CUDA_SUCCESS) {
      *why = "cuMemExportToShareableHandle: " + cu_str(d, r);
      ok = false;
    }
  }
  if (!all_agree(c, ok)) {
    if (my_fd >= 0) close(my_fd);
    if (why->empty()) *why = "a peer could not create exportable memory";
    release_vmm(c);
    return OOB_ERR_UNSUPPORTED;
  }
  // 2. exchange descriptors, import, map
  std::vector<int> fds;
  if (!c->boot->exchange_fds(my_fd, &fds)) {
    close(my_fd);
    *why = c->boot->last_error();
    release_vmm(c);
    return OOB_ERR_BOOTSTRAP;
  }
  close(my_fd);
  CUmemAccessDesc acc{};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = c->device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  for (int p = 0; p < c->world && ok; ++p) {
    if (p != c->rank) {
      r = d->cuMemImportFromShareableHandle(&c->handles[p], reinterpret_cast<void*>(static_cast<intptr_t>(fds[p])),
                                            CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      if (r != CUDA_SUCCESS) {
        *why = "cuMemImportFromShareableHandle(rank " + std::to_string(p) + "): " + cu_str(d, r);
        ok = false;
        break;
      }
      c->handle_valid[p] = true;
    }
    CUdeviceptr va = 0;
    r = d->cuMemAddressReserve(&va, c->map_bytes, gran, 0, 0);
    if (r == CUDA_SUCCESS) r = d->cuMemMap(va, c->map_bytes, 0, c->handles[p], 0);
    if (r == CUDA_SUCCESS) r = d->cuMemSetAccess(va, c->map_bytes, &acc, 1);
    if (r != CUDA_SUCCESS) {
      *why = "mapping rank " + std::to_string(p) + "'s heap: " + cu_str(d, r);
      ok = false;
      break;
    }
    c->heap[p] = reinterpret_cast<char*>(va);
  }
  for (int fd : fds)
    if (fd >= 0) close(fd);
  if (!all_agree(c, ok)) {
    if (why->empty()) *why = "a peer could not map the heaps";
    release_vmm(c);
    return OOB_ERR_UNSUPPORTED;
  }
  c->memory_kind = 0;

  // 3. optional NVLS multicast alias of all heaps.  Every stage is agreed on
  // collectively; any refusal leaves the communicator on plain P2P.
  if (want_mc) {
    bool mok = true;
    int mfd = -1;
    if (c->rank == 0) {
      r = d->cuMulticastCreate(&c->mc_handle, &mprop);
      if (r == CUDA_SUCCESS) {
        c->mc_valid = true;
        r = d->cuMemExportToShareableHandle(&mfd, c->mc_handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
      }
      mok = (r == CUDA_SUCCESS);
    }
    // Rank 0's verdict decides whether a descriptor travels at all.
    char go = mok ? 1 : 0;
    std::vector<char> all(c->world);
    if (!c->boot->allgather(&go, all.data(), 1)) mok = false;
    else mok = all[0] != 0;
    if (mok) {
      if (!c->boot->broadcast_fd(0, &mfd)) mok = false;
      if (mok && c->rank != 0) {
        r = d->cuMemImportFromShareableHandle(&c->mc_handle, reinterpret_cast<void*>(static_cast<intptr_t>(mfd)),
                                              CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
        mok = (r == CUDA_SUCCESS);
        if (mok) c->mc_valid = true;
      }
      if (mfd >= 0) close(mfd);
      if (mok) {
        r = d->cuMulticastAddDevice(c->mc_handle, dev);
        mok = (r == CUDA_SUCCESS);
      }
      mok = all_agree(c, mok);  // every device added before anybody binds
      if (mok) {
        r = d->cuMulticastBindMem(c->mc_handle, 0, c->handles[c->rank], 0, c->map_bytes, 0);
        mok = (r == CUDA_SUCCESS);
        if (mok) c->mc_bound = true;
      }
      mok = all_agree(c, mok);
      if (mok) {
        CUdeviceptr va = 0;
        r = d->cuMemAddressReserve(&va, c->map_bytes, gran, 0, 0);
        if (r == CUDA_SUCCESS) r = d->cuMemMap(va, c->map_bytes, 0, c->mc_handle, 0);
        if (r == CUDA_SUCCESS) r = d->cuMemSetAccess(va, c->map_bytes, &acc, 1);
        mok = (r == CUDA_SUCCESS);
        if (mok) c->heap_mc = reinterpret_cast<char*>(va);
      }
      mok = all_agree(c, mok);
    }
    if (!mok) {
      if (c->heap_mc) {
        d->cuMemUnmap(reinterpret_cast<CUdeviceptr>(c->heap_mc), c->map_bytes);
        d->cuMemAddressFree(reinterpret_cast<CUdeviceptr>(c->heap_mc), c->map_bytes);
        c->heap_mc = nullptr;
      }
      if (c->mc_bound) {
        d->cuMulticastUnbind(c->mc_handle, dev, 0, c->map_bytes);
        c->mc_bound = false;
      }
      if (c->mc_valid) {
        d->cuMemRelease(c->mc_handle);
        c->mc_valid = false;
      }
    }
    c->nvls = mok;
    if (!mok)
      OOB_LOG(kLogWarn, "rank %d: the NVLink multicast alias could not be set up (last driver answer: %s); using peer "
              "loads and stores", c->rank, cu_str(d, r).c_str());
  } else if (c->world > 1) {
    OOB_LOG(kLogInfo, "rank %d: no multicast alias (%s)", c->rank,
            !mc_ok ? "the device does not report multicast support" : "switched off by flag or OOB_DISABLE_NVLS");
  }
  return OOB_OK;
}

// Legacy path: cudaMalloc + cudaIpcMemHandle (no multicast).
int setup_legacy_ipc(oob_comm* c, std::string* why) {
  void* local = nullptr;
  cudaError_t e = cudaMalloc(&local, c->heap_bytes);
  bool ok = (e == cudaSuccess);
  cudaIpcMemHandle_t mine{};
  if (ok) {
    e = cudaIpcGetMemHandle(&mine, local);
    ok = (e == cudaSuccess);
  }
  if (!ok) *why = std::string("legacy IPC export: ") + cudaGetErrorString(e);
  (void)cudaGetLastError();
  if (!all_agree(c, ok)) {
    if (local) cudaFree(local);
    if (why->empty()) *why = "a peer could not export its heap";
    return OOB_ERR_UNSUPPORTED;
  }
  std::vector<cudaIpcMemHandle_t> all(c->world);
  if (!c->boot->allgather(&mine, all.data(), sizeof(mine))) {
    *why = c->boot->last_error();
    cudaFree(local);
    return OOB_ERR_BOOTSTRAP;
  }
  c->heap[c->rank] = static_cast<char*>(local);
  for (int p = 0; p < c->world && ok; ++p) {
    if (p == c->rank) continue;
    void* ptr = nullptr;
    e = cudaIpcOpenMemHandle(&ptr, all[p], cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      *why = "cudaIpcOpenMemHandle(rank " + std::to_string(p) + "): " + cudaGetErrorString(e);
      (void)cudaGetLastError();
      ok = false;
      break;
    }
    c->heap[p] = static_cast<char*>(ptr);
  }
  if (!all_agree(c, ok)) {
    for (int p = 0; p < c->world; ++p) {
      if (p != c->rank && c->heap[p]) cudaIpcCloseMemHandle(c->heap[p]);
      c->heap[p] = nullptr;
    }
    cudaFree(local);
    if (why->empty()) *why = "a peer could not open the heaps";
    return OOB_ERR_UNSUPPORTED;
  }
  c->memory_kind = 1;
  c->nvls = false;
  return OOB_OK;
}

int check_comm(const oob_comm* c) {
  if (c == nullptr) return set_error(OOB_ERR_INVALID, "null communicator");
  if (c->poisoned)
    return set_error(OOB_ERR_POISONED, "communicator is poisoned by an earlier device timeout; call oob_comm_recover");
  return OOB_OK;
}

}  // namespace

// ---------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------
extern "C" {

const char* oob_last_error(void) { return g_last_error.c_str(); }
const char* oob_version(void) { return "ooverlap_b200 0.1 (sm_100a)"; }

int oob_comm_create(int rank, int world, int device, const char* key, uint64_t heap_bytes, unsigned flags,
                    int timeout_ms, oob_comm** out) {
  if (out == nullptr || key == nullptr) return set_error(OOB_ERR_INVALID, "null argument");
  *out = nullptr;
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world)
    return set_error(OOB_ERR_INVALID, "world must be 1.." + std::to_string(kMaxRanks) + " and 0 <= rank < world");
  if (heap_bytes < kPadBytes + (1u << 20)) heap_bytes = kPadBytes + (1u << 20);
  cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
  e = cudaFree(nullptr);
  if (e != cudaSuccess) return cuda_fail(e, "context creation");

  oob_comm* c = new oob_comm();
  c->rank = rank;
  c->world = world;
  c->device = device;
  c->heap_bytes = heap_bytes;
  std::string err;
  c->boot = Bootstrap::create(rank, world, key, timeout_ms, &err);
  if (c->boot == nullptr) {
    delete c;
    return set_error(OOB_ERR_BOOTSTRAP, err);
  }
  int rc = OOB_ERR_UNSUPPORTED;
  std::string why;
  if (!(flags & OOB_FLAG_LEGACY_IPC)) rc = setup_vmm(c, flags, &why);
  if (rc != OOB_OK && rc != OOB_ERR_BOOTSTRAP) {
    if (!(flags & OOB_FLAG_LEGACY_IPC))
      OOB_LOG(kLogWarn, "rank %d: no VMM heap (%s); falling back to cudaMalloc + CUDA IPC, without NVLS", rank, why.c_str());
    std::string why2;
    rc = setup_legacy_ipc(c, &why2);
    if (rc != OOB_OK) why = why + "; " + why2;
  }
  if (rc != OOB_OK) {
    delete c->boot;
    delete c;
    return set_error(rc, "cannot build the symmetric heap: " + why);
  }
  e = cudaMemset(c->heap[rank], 0, kPadBytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    rc = cuda_fail(e, "clearing the signal pad");
  } else {
    rc = alloc_status(c, 1);
  }
  if (rc == OOB_OK && !c->boot->barrier()) rc = set_error(OOB_ERR_BOOTSTRAP, c->boot->last_error());
  if (rc != OOB_OK) {
    oob_comm_destroy(c);
    return rc;
  }
  allocator_init(c);
  OOB_LOG(kLogInfo, "rank %d/%d on device %d: heap %llu MiB (%s), NVLS %s, device-wait budget %llu ms", rank, world, device,
          static_cast<unsigned long long>(c->heap_bytes >> 20), c->memory_kind == 0 ? "VMM, fd export" : "cudaMalloc + CUDA IPC",
          c->nvls ? "on" : "off", static_cast<unsigned long long>(c->timeout_ns / 1000000ull));
  *out = c;
  return OOB_OK;
}

int oob_comm_create_emulated(int world, int device, uint64_t heap_bytes, oob_comm** out) {
  if (out == nullptr) return set_error(OOB_ERR_INVALID, "null argument");
  *out = nullptr;
  if (world < 1 || world > kMaxRanks) return set_error(OOB_ERR_INVALID, "bad world size");
  if (heap_bytes < kPadBytes + (1u << 20)) heap_bytes = kPadBytes + (1u << 20);
  heap_bytes = round_up(heap_bytes, 4096);
  cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
  oob_comm* c = new oob_comm();
  c->rank = 0;
  c->world = world;
  c->device = device;
  c->emulated = true;
  c->memory_kind = 2;
  c->heap_bytes = heap_bytes;
  for (int r = 0; r < world; ++r) {
    void* p = nullptr;
    e = cudaMalloc(&p, heap_bytes);
    if (e != cudaSuccess) {
      oob_comm_destroy(c);
      return cuda_fail(e, "cudaMalloc(emulated heap)");
    }
    c->heap[r] = static_cast<char*>(p);
    cudaMemset(p, 0, kPadBytes);
  }
  e = cudaMalloc(reinterpret_cast<void**>(&c->emu_table_dev), sizeof(CommCtx) * kMaxRanks);
  if (e != cudaSuccess) {
    oob_comm_destroy(c);
    return cuda_fail(e, "cudaMalloc(emu table)");
  }
  int rc = alloc_status(c, world);
  if (rc == OOB_OK) rc = refresh_emu_table(c);
  if (rc != OOB_OK) {
    oob_comm_destroy(c);
    return rc;
  }
  cudaDeviceSynchronize();
  allocator_init(c);
  *out = c;
  return OOB_OK;
}

int oob_comm_destroy(oob_comm* c) {
  if (c == nullptr) return OOB_OK;
  cudaSetDevice(c->device);
  cudaDeviceSynchronize();
  // Nobody may unmap while a peer could still be touching the heap.
  if (c->boot && c->world > 1) c->boot->barrier();
  for (int p = 0; p < c->world; ++p)
    for (auto& im : c->imports[p])
      if (im.base) cudaIpcCloseMemHandle(im.base);
  if (c->memory_kind == 0) {
    release_vmm(c);
  } else if (c->memory_kind == 1) {
    for (int p = 0; p < c->world; ++p) {
      if (c->heap[p] == nullptr) continue;
      if (p == c->rank)
        cudaFree(c->heap[p]);
      else
        cudaIpcCloseMemHandle(c->heap[p]);
    }
  } else {
    for (int p = 0; p < c->world; ++p)
      if (c->heap[p]) cudaFree(c->heap[p]);
  }
  if (c->emu_table_dev) cudaFree(c->emu_table_dev);
  if (c->status_host) cudaFreeHost(c->status_host);
  (void)cudaGetLastError();
  delete c->boot;
  delete c;
  return OOB_OK;
}

int oob_comm_info(const oob_comm* c, oob_comm_info_t* info) {
  if (c == nullptr || info == nullptr) return set_error(OOB_ERR_INVALID, "null argument");
  info->rank = c->rank;
  info->world = c->world;
  info->device = c->device;
  info->nvls = c->nvls ? 1 : 0;
  info->emulated = c->emulated ? 1 : 0;
  info->memory_kind = c->memory_kind;
  info->heap_bytes = c->heap_bytes;
  info->user_offset = round_up(kPadBytes, kAllocAlign);
  info->timeout_ns = c->timeout_ns;
  return OOB_OK;
}

int oob_comm_set_timeout_ms(oob_comm* c, int ms) {
  if (c == nullptr || ms <= 0) return set_error(OOB_ERR_INVALID, "bad argument");
  c->timeout_ns = uint64_t(ms) * 1000000ull;
  return refresh_emu_table(c);
}

int oob_comm_barrier(oob_comm* c) {
  if (c == nullptr) return set_error(OOB_ERR_INVALID, "null communicator");
  if (c->boot == nullptr || c->world == 1 || c->emulated) return OOB_OK;
  if (!c->boot->barrier()) return set_error(OOB_ERR_BOOTSTRAP, c->boot->last_error());
  return OOB_OK;
}

int oob_comm_host_allgather(oob_comm* c, const void* in, void* out, uint64_t bytes) {
  if (c == nullptr || in == nullptr || out == nullptr || bytes == 0) return set_error(OOB_ERR_INVALID, "bad argument");
  if (c->boot == nullptr || c->world == 1 || c->emulated) {
    std::memcpy(out, in, bytes);
    return OOB_OK;
  }
  if (!c->boot->allgather(in, out, bytes)) return set_error(OOB_ERR_BOOTSTRAP, c->boot->last_error());
  return OOB_OK;
}

int oob_comm_status(oob_comm* c, oob_device_status_t* s) {
  if (c == nullptr) return set_error(OOB_ERR_INVALID, "null communicator");
  const int n = c->emulated ? c->world : 1;
  for (int i = 0; i < n; ++i) {
    const volatile DeviceStatus* d = c->status_host + i;
    if (d->code != 0) {
      if (s) {
        s->code = d->code;
        s->rank = d->rank;
        s->peer = d->peer;
        s->block = d->block;
        s->expected = d->expected;
        s->observed = d->observed;
        s->where = d->where;
        s->pad = 0;
      }
      if (!c->poisoned)
        OOB_LOG(kLogWarn, "rank %d: a kernel gave up waiting (code %d, peer %d, block %d, expected %u, observed %u, site %d); "
                "the communicator is poisoned until oob_comm_recover", c->rank, int(d->code), int(d->peer), int(d->block),
                unsigned(d->expected), unsigned(d->observed), int(d->where));
      c->poisoned = true;
      return set_error(OOB_ERR_DEVICE_TIMEOUT,
                       "device wait gave up: code " + std::to_string(d->code) + " rank " + std::to_string(d->rank) +
                           " peer " + std::to_string(d->peer) + " block " + std::to_string(d->block) + " expected " +
                           std::to_string(d->expected) + " observed " + std::to_string(d->observed) + " at " +
                           std::to_string(d->where));
    }
  }
  if (s) std::memset(s, 0, sizeof(*s));
  return OOB_OK;
}

int oob_comm_recover(oob_comm* c) {
  if (c == nullptr) return set_error(OOB_ERR_INVALID, "null communicator");
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceSynchronize");
  if (c->boot && c->world > 1 && !c->boot->barrier()) return set_error(OOB_ERR_BOOTSTRAP, c->boot->last_error());
  const int n = c->emulated ? c->world : 1;
  for (int i = 0; i < n; ++i) {
    char* pad = c->emulated ? c->heap[i] : c->heap[c->rank];
    e = cudaMemset(pad, 0, kPadBytes);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemset(pad)");
  }
  e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceSynchronize");
  std::memset(c->status_host, 0, sizeof(DeviceStatus) * n);
  if (c->boot && c->world > 1 && !c->boot->barrier()) return set_error(OOB_ERR_BOOTSTRAP, c->boot->last_error());
  c->poisoned = false;
  OOB_LOG(kLogInfo, "rank %d: signal pad and status cleared, communicator back in service", c->rank);
  return OOB_OK;
}

int oob_alloc(oob_comm* c, uint64_t bytes, uint64_t align, uint64_t* offset) {
  if (c == nullptr || offset == nullptr || bytes == 0) return set_error(OOB_ERR_INVALID, "bad argument");
  if (align < kAllocAlign) align = kAllocAlign;
  if (align & (align - 1)) return set_error(OOB_ERR_INVALID, "alignment must be a power of two");
  bytes = round_up(bytes, kAllocAlign);
  for (auto it = c->free_blocks.begin(); it != c->free_blocks.end(); ++it) {
    const uint64_t start = it->first, size = it->second;
    const uint64_t aligned = round_up(start, align);
    if (aligned + bytes > start + size) continue;
    c->free_blocks.erase(it);
    if (aligned > start) c->free_blocks[start] = aligned - start;
    if (aligned + bytes < start + size) c->free_blocks[aligned + bytes] = start + size - (aligned + bytes);
    c->live[aligned] = bytes;
    *offset = aligned;
    return OOB_OK;
  }
  return set_error(OOB_ERR_NOMEM, "symmetric heap exhausted (asked for " + std::to_string(bytes) + " bytes)");
}

int oob_free(oob_comm* c, uint64_t offset) {
  if (c == nullptr) return set_error(OOB_ERR_INVALID, "null communicator");
  auto it = c->live.find(offset);
  if (it == c->live.end()) return set_error(OOB_ERR_INVALID, "offset was not returned by oob_alloc");
  uint64_t start = it->first, size = it->second;
  c->live.erase(it);
  auto next = c->free_blocks.lower_bound(start);
  if (next != c->free_blocks.end() && next->first == start + size) {
    size += next->second;
    next = c->free_blocks.erase(next);
  }
  if (next != c->free_blocks.begin()) {
    auto prev = std::prev(next);
    if (prev->first + prev->second == start) {
      start = prev->first;
      size += prev->second;
      c->free_blocks.erase(prev);
    }
  }
  c->free_blocks[start] = size;
  return OOB_OK;
}

void* oob_heap_ptr(const oob_comm* c, int rank, uint64_t offset) {
  if (c == nullptr || rank < 0 || rank >= c->world || offset > c->heap_bytes) return nullptr;
  return c->heap[rank] + offset;
}

void* oob_heap_mc_ptr(const oob_comm* c, uint64_t offset) {
  if (c == nullptr || c->heap_mc == nullptr || offset > c->heap_bytes) return nullptr;
  return c->heap_mc + offset;
}

int oob_register_ipc(oob_comm* c, void* ptr, uint64_t bytes, int* reg) {
  int rc = check_comm(c);
  if (rc != OOB_OK) return rc;
  if (ptr == nullptr || reg == nullptr || bytes == 0) return set_error(OOB_ERR_INVALID, "bad argument");
  // The kernels move 16-byte packs: a registered view that starts off a 16-byte boundary (a tensor slice with a
  // storage offset) would trap in them.  Every rank checks its own pointer and all ranks agree on the outcome below,
  // so that nobody registers while a peer refuses.
  const bool aligned = (reinterpret_cast<uintptr_t>(ptr) & 15) == 0;
  if ((c->emulated || c->world == 1) && !aligned)
    return set_error(OOB_ERR_INVALID, "registered memory must start on a 16-byte boundary");
  oob_comm::Registration R;
  R.local = ptr;
  R.bytes = bytes;
  if (c->emulated || c->world == 1) {
    // Same process: the "peers" are given by the caller one by one is not
    // supported; a single rank only sees itself.
    if (c->world != 1) return set_error(OOB_ERR_UNSUPPORTED, "IPC registration is meaningless in the emulated group");
    R.peer[0] = ptr;
    *reg = c->next_reg++;
    c->regs[*reg] = R;
    return OOB_OK;
  }
  const DriverApi* d = driver_api();
  struct Desc {
    cudaIpcMemHandle_t handle;
    uint64_t offset;
    int ok;
    int pad;
  } mine{};
  mine.ok = 0;
  mine.pad = aligned ? 0 : 1;
  CUdeviceptr base = 0;
  size_t range = 0;
  if (d && d->cuMemGetAddressRange(&base, &range, reinterpret_cast<CUdeviceptr>(ptr)) == CUDA_SUCCESS) {
    cudaError_t e = cudaIpcGetMemHandle(&mine.handle, reinterpret_cast<void*>(base));
    if (e == cudaSuccess) {
      mine.offset = reinterpret_cast<CUdeviceptr>(ptr) - base;
      mine.ok = 1;
    } else {
      (void)cudaGetLastError();
    }
  }
  std::vector<Desc> all(c->world);
  if (!c->boot->allgather(&mine, all.data(), sizeof(Desc))) return set_error(OOB_ERR_BOOTSTRAP, c->boot->last_error());
  for (auto& x : all)
    if (x.pad != 0)
      return set_error(OOB_ERR_INVALID, "registered memory must start on a 16-byte boundary on every rank (a rank passed "
                                        "a view with a storage offset that is not a multiple of 16 bytes)");
  for (auto& x : all)
    if (!x.ok)
      return set_error(OOB_ERR_UNSUPPORTED,
                       "a rank could not export this allocation through CUDA IPC (expandable segments or a "
                       "non-cudaMalloc allocation?)");
  bool ok = true;
  std::string why;
  for (int p = 0; p < c->world; ++p) {
    if (p == c->rank) {
      R.peer[p] = ptr;
      continue;
    }
    void* mapped = nullptr;
    auto& cache = c->imports[p];
    for (auto& im : cache) {
      if (std::memcmp(&im.handle, &all[p].handle, sizeof(cudaIpcMemHandle_t)) == 0) {
        mapped = im.base;
        im.last_use = ++c->use_clock;
        break;
      }
    }
    if (mapped == nullptr) {
      cudaError_t e = cudaIpcOpenMemHandle(&mapped, all[p].handle, cudaIpcMemLazyEnablePeerAccess);
      if (e != cudaSuccess) {
        (void)cudaGetLastError();
        why = std::string("cudaIpcOpenMemHandle: ") + cudaGetErrorString(e);
        ok = false;
        break;
      }
      if (cache.size() >= 16) {
        // Evict the least recently used mapping that no live registration still points into.
        auto victim = cache.end();
        for (auto it = cache.begin(); it != cache.end(); ++it)
          if (it->refs == 0 && (victim == cache.end() || it->last_use < victim->last_use)) victim = it;
        if (victim != cache.end()) {
          OOB_LOG(kLogDebug, "rank %d: IPC import cache of peer %d is full, closing the least recently used mapping", c->rank, p);
          cudaIpcCloseMemHandle(victim->base);
          cache.erase(victim);
        }
      }
      cache.push_back({all[p].handle, mapped, ++c->use_clock, 0});
      OOB_LOG(kLogDebug, "rank %d: opened an IPC mapping of peer %d's allocation (%zu cached)", c->rank, p, cache.size());
    }
    for (auto& im : cache)
      if (im.base == mapped) ++im.refs;
    R.import_base[p] = mapped;
    R.peer[p] = static_cast<char*>(mapped) + all[p].offset;
  }
  if (!all_agree(c, ok)) return set_error(OOB_ERR_CUDA, why.empty() ? "a peer failed to import the allocation" : why);
  *reg = c->next_reg++;
  c->regs[*reg] = R;
  return OOB_OK;
}

int oob_unregister(oob_comm* c, int reg) {
  if (c == nullptr) return set_error(OOB_ERR_INVALID, "null communicator");
  auto it = c->regs.find(reg);
  if (it == c->regs.end()) return set_error(OOB_ERR_INVALID, "unknown registration");
  for (int p = 0; p < c->world; ++p)
    for (auto& im : c->imports[p])
      if (im.base != nullptr && im.base == it->second.import_base[p] && im.refs > 0) --im.refs;
  c->regs.erase(it);
  return OOB_OK;
}

// ---- collectives -----------------------------------------------------------

int oob_allreduce(oob_comm* c, int dtype, int op, int algo, int in_reg, uint64_t in_off, int out_reg, uint64_t out_off,
                  void* out_local, uint64_t count, int max_ctas, void* stream) {
  int rc = check_comm(c);
  if (rc != OOB_OK) return rc;
  if (count == 0) return OOB_OK;
  const uint64_t esize = dtype == OOB_F32 ? 4 : 2;
  if (algo == OOB_ALGO_AUTO) {
    int ctas = 0;
    const bool mc_ok = c->nvls && in_reg == 0 && (out_reg == 0 || out_local != nullptr) && !(dtype == OOB_F32 && op != OOB_SUM);
    oob_policy_select(c->world, 0, count * esize, mc_ok ? 1 : 0, &algo, &ctas);
    const bool one_shot = (algo == OOB_AR_ONESHOT_P2P || algo == OOB_AR_ONESHOT_NVLS);
    if (one_shot && out_local == nullptr) algo = (mc_ok && out_reg == 0) ? OOB_AR_TWOSHOT_NVLS : OOB_AR_TWOSHOT_P2P;
    if (!one_shot && out_reg < 0) algo = mc_ok ? OOB_AR_ONESHOT_NVLS : OOB_AR_ONESHOT_P2P;
    if (max_ctas <= 0) max_ctas = ctas;
  }
  if (max_ctas <= 0) max_ctas = 16;
  PeerPtrs in, out;
  if (!c->peer_ptrs(in_reg, in_off, count * esize, &in))
    return set_error(OOB_ERR_INVALID, "bad input buffer (offset + count lies outside the heap / the registration)");
  const bool one_shot = (algo == OOB_AR_ONESHOT_P2P || algo == OOB_AR_ONESHOT_NVLS);
  if (one_shot) {
    if (out_local == nullptr) return set_error(OOB_ERR_INVALID, "one-shot all-reduce needs out_local");
    std::memset(&out, 0, sizeof(out));
  } else if (!c->peer_ptrs(out_reg, out_off, count * esize, &out)) {
    return set_error(OOB_ERR_INVALID, "two-shot all-reduce needs a registered output buffer that holds count elements");
  }
  if ((in_off & 15) || (!one_shot && (out_off & 15)))
    return set_error(OOB_ERR_INVALID, "registered all-reduce buffers must be 16-byte aligned");
  const uint64_t emu_stride = c->emulated ? count * esize : 0;
  cudaError_t e = launch_allreduce(c->make_ctx(), dtype, op, algo, in, out, out_local, emu_stride, count, max_ctas,
                                   static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "all-reduce launch");
  return OOB_OK;
}

int oob_reduce_scatter(oob_comm* c, int dtype, int op, int algo, int in_reg, uint64_t in_off, void* out_local,
                       uint64_t count, int max_ctas, void* stream) {
  int rc = check_comm(c);
  if (rc != OOB_OK) return rc;
  if (count == 0) return OOB_OK;
  const uint64_t esize = dtype == OOB_F32 ? 4 : 2;
  if (algo == OOB_ALGO_AUTO) {
    int ctas = 0;
    const bool mc_ok = c->nvls && in_reg == 0 && !(dtype == OOB_F32 && op != OOB_SUM);
    oob_policy_select(c->world, 1, count * esize, mc_ok ? 1 : 0, &algo, &ctas);
    if (max_ctas <= 0) max_ctas = ctas;
  }
  if (max_ctas <= 0) max_ctas = 16;
  PeerPtrs in;
  if (!c->peer_ptrs(in_reg, in_off, count * esize, &in) || (in_off & 15)) return set_error(OOB_ERR_INVALID, "bad input buffer");
  if (out_local == nullptr) return set_error(OOB_ERR_INVALID, "null output");
  // Emulation: rank r's output block is out_local + r * ceil(count / world) elements.
  const uint64_t emu_stride = c->emulated ? ((count + c->world - 1) / c->world) * esize : 0;
  cudaError_t e = launch_reduce_scatter(c->make_ctx(), dtype, op, algo, in, out_local, emu_stride, count, max_ctas,
                                        static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "reduce-scatter launch");
  return OOB_OK;
}

int oob_all_gather(oob_comm* c, int dtype, int algo, int out_reg, uint64_t out_off, const void* src_local,
                   void* dst_local, uint64_t count, int max_ctas, void* stream) {
  int rc = check_comm(c);
  if (rc != OOB_OK) return rc;
  if (count == 0) return OOB_OK;
  const uint64_t esize = dtype == OOB_F32 ? 4 : 2;
  if (algo == OOB_ALGO_AUTO) {
    int ctas = 0;
    oob_policy_select(c->world, 2, count * esize, (c->nvls && out_reg == 0) ? 1 : 0, &algo, &ctas);
    if (max_ctas <= 0) max_ctas = ctas;
  }
  if (max_ctas <= 0) max_ctas = 16;
  PeerPtrs out;
  // Push: the registered buffer receives all `count` elements.  Pull: it holds this rank's shard.
  const uint64_t reg_elems = algo == OOB_AG_PULL_P2P ? (count + c->world - 1) / c->world : count;
  if (!c->peer_ptrs(out_reg, out_off, reg_elems * esize, &out) || (out_off & 15))
    return set_error(OOB_ERR_INVALID, "bad registered buffer");
  if (algo == OOB_AG_PULL_P2P) {
    if (dst_local == nullptr) return set_error(OOB_ERR_INVALID, "pull all-gather needs dst_local");
  } else if (src_local == nullptr) {
    return set_error(OOB_ERR_INVALID, "push all-gather needs src_local");
  }
  const uint64_t shard = ((count + c->world - 1) / c->world) * esize;
  const uint64_t src_stride = c->emulated ? shard : 0;
  const uint64_t dst_stride = c->emulated ? count * esize : 0;
  cudaError_t e = launch_all_gather(c->make_ctx(), dtype, algo, out, src_local, src_stride, dst_local, dst_stride, count,
                                    max_ctas, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "all-gather launch");
  return OOB_OK;
}

int oob_allreduce_push(oob_comm* c, int dtype, int op, int stage_reg, uint64_t stage_off, uint64_t piece_bytes,
                       const void* in_local, void* out_local, uint64_t count, int use_nvls, int max_ctas, void* stream) {
  int rc = check_comm(c);
  if (rc != OOB_OK) return rc;
  if (count == 0) return OOB_OK;
  if (dtype != OOB_F16 && dtype != OOB_BF16 && dtype != OOB_F32) return set_error(OOB_ERR_INVALID, "bad dtype");
  if (op != OOB_SUM && op != OOB_MIN && op != OOB_MAX) return set_error(OOB_ERR_INVALID, "bad reduction");
  if (in_local == nullptr || out_local == nullptr) return set_error(OOB_ERR_INVALID, "null input or output");
  const uint64_t esize = dtype == OOB_F32 ? 4 : 2;
  if ((piece_bytes & 15) || count * esize > piece_bytes)
    return set_error(OOB_ERR_INVALID, "piece_bytes must be a multiple of 16 and hold the message");
  PeerPtrs st;
  if ((stage_off & 15) || !c->peer_ptrs(stage_reg, stage_off, 2 * piece_bytes * c->world, &st))
    return set_error(OOB_ERR_INVALID, "bad staging area (16-byte aligned, 2 * world * piece_bytes inside the registration)");
  const bool mc = use_nvls != 0 && st.mc != nullptr;
  const uint64_t emu_stride = c->emulated ? count * esize : 0;
  cudaError_t e = launch_allreduce_push(c->make_ctx(), dtype, op, mc, st, piece_bytes, in_local, emu_stride, out_local,
                                        emu_stride, count, max_ctas, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "push all-reduce launch");
  return OOB_OK;
}

int oob_allreduce_ll(oob_comm* c, int dtype, int op, int stage_reg, uint64_t stage_off, uint64_t piece_bytes,
                     const void* in_local, void* out_local, uint64_t count, int use_nvls, int max_ctas, void* stream) {
  int rc = check_comm(c);
  if (rc != OOB_OK) return rc;
  if (count == 0) return OOB_OK;
  if (dtype != OOB_F16 && dtype != OOB_BF16 && dtype != OOB_F32) return set_error(OOB_ERR_INVALID, "bad dtype");
  if (op != OOB_SUM && op != OOB_MIN && op != OOB_MAX) return set_error(OOB_ERR_INVALID, "bad reduction");
  if (in_local == nullptr || out_local == nullptr) return set_error(OOB_ERR_INVALID, "null input or output");
  const uint64_t esize = dtype == OOB_F32 ? 4 : 2;
  const uint64_t words = (count * esize + 3) / 4;
  if ((piece_bytes & 15) || words * 8 > piece_bytes)
    return set_error(OOB_ERR_INVALID, "piece_bytes must be a multiple of 16 and hold 8 bytes per 32-bit word of the message");
  if ((reinterpret_cast<uintptr_t>(in_local) | reinterpret_cast<uintptr_t>(out_local)) & (esize - 1))
    return set_error(OOB_ERR_INVALID, "input and output must be aligned to their element size");
  PeerPtrs st;
  if ((stage_off & 15) || !c->peer_ptrs(stage_reg, stage_off, 2 * piece_bytes * c->world, &st))
    return set_error(OOB_ERR_INVALID, "bad staging area (16-byte aligned, 2 * world * piece_bytes inside the registration)");
  const bool mc = use_nvls != 0 && st.mc != nullptr;
  const uint64_t emu_stride = c->emulated ? count * esize : 0;
  cudaError_t e = launch_allreduce_ll(c->make_ctx(), dtype, op, mc, st, piece_bytes, in_local, emu_stride, out_local,
                                      emu_stride, count, max_ctas, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "flag-in-data all-reduce launch");
  return OOB_OK;
}

int oob_all_to_all(oob_comm* c, int dtype, int out_reg, uint64_t out_off, const void* src_local, uint64_t count_per_peer,
                   int max_ctas, void* stream) {
  int rc = check_comm(c);
  if (rc != OOB_OK) return rc;
  if (count_per_peer == 0) return OOB_OK;
  if (dtype != OOB_F16 && dtype != OOB_BF16 && dtype != OOB_F32) return set_error(OOB_ERR_INVALID, "bad dtype");
  if (src_local == nullptr) return set_error(OOB_ERR_INVALID, "all-to-all needs src_local");
  const uint64_t chunk = count_per_peer * (dtype == OOB_F32 ? 4 : 2);
  PeerPtrs out;
  if (!c->peer_ptrs(out_reg, out_off, chunk * c->world, &out) || (out_off & 15))
    return set_error(OOB_ERR_INVALID, "bad registered buffer");
  const uint64_t src_stride = c->emulated ? chunk * c->world : 0;
  cudaError_t e = launch_all_to_all(c->make_ctx(), out, src_local, src_stride, chunk, max_ctas,
                                    static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "all-to-all launch");
  return OOB_OK;
}

int oob_fused_norm(oob_comm* c, int algo, const oob_norm_args_t* a, int max_ctas, void* stream) {
  if (a == nullptr) return set_error(OOB_ERR_INVALID, "null argument");
  if (c == nullptr) {
    // Local normalisation needs no communicator: x_off carries the address of x.
    if (algo != OOB_NORM_LOCAL) return set_error(OOB_ERR_INVALID, "fused norm algorithms need a communicator");
    if (a->weight == nullptr || a->y_local == nullptr || (a->x_off & 15)) return set_error(OOB_ERR_INVALID, "bad argument");
    NormArgs n{};
    n.dtype = a->dtype;
    n.rows = a->rows;
    n.hidden = a->hidden;
    n.eps = a->eps;
    n.x.p[0] = reinterpret_cast<void*>(static_cast<uintptr_t>(a->x_off));
    n.residual = a->residual;
    n.weight = a->weight;
    n.y_local = a->y_local;
    n.res_out_local = a->res_out_local;
    CommCtx ctx{};
    ctx.world = 1;
    ctx.rank = 0;
    if (max_ctas <= 0) max_ctas = 148 * 8;
    cudaError_t e = launch_fused_norm(ctx, algo, n, max_ctas, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(e, "rmsnorm launch");
    return OOB_OK;
  }
  int rc = check_comm(c);
  if (rc != OOB_OK) return rc;
  NormArgs n{};
  n.dtype = a->dtype;
  n.rows = a->rows;
  n.hidden = a->hidden;
  n.eps = a->eps;
  if (a->rows <= 0 || a->hidden <= 0) return set_error(OOB_ERR_INVALID, "bad shape");
  const uint64_t norm_bytes = uint64_t(a->rows) * a->hidden * (a->dtype == OOB_F32 ? 4 : 2);
  if (!c->peer_ptrs(a->x_reg, a->x_off, norm_bytes, &n.x) || (a->x_off & 15)) return set_error(OOB_ERR_INVALID, "bad x buffer");
  n.residual = a->residual;
  n.residual_emu_stride = c->emulated ? a->emu_stride_local : 0;
  n.weight = a->weight;
  if (a->weight == nullptr) return set_error(OOB_ERR_INVALID, "null norm weight");
  const bool push = (algo == OOB_NORM_AR_TWOSHOT || algo == OOB_NORM_AR_TWOSHOT_NVLS);
  if (push) {
    if (!c->peer_ptrs(a->y_reg, a->y_off, norm_bytes, &n.y) || (a->y_off & 15)) return set_error(OOB_ERR_INVALID, "bad y buffer");
    if (a->res_out_reg >= 0) {
      if (!c->peer_ptrs(a->res_out_reg, a->res_out_off, norm_bytes, &n.res_out) || (a->res_out_off & 15))
        return set_error(OOB_ERR_INVALID, "bad res_out buffer");
    } else {
      std::memset(&n.res_out, 0, sizeof(n.res_out));
    }
  } else {
    if (a->y_local == nullptr) return set_error(OOB_ERR_INVALID, "null y_local");
    n.y_local = a->y_local;
    n.y_local_emu_stride = c->emulated ? a->emu_stride_local : 0;
    n.res_out_local = a->res_out_local;
    n.res_out_local_emu_stride = c->emulated ? a->emu_stride_local : 0;
  }
  if (algo == OOB_NORM_AR_PUSH || algo == OOB_NORM_AR_PUSH_NVLS || algo == OOB_NORM_AR_LL) {
    if ((a->piece_bytes & 15) || a->piece_bytes < norm_bytes * (algo == OOB_NORM_AR_LL ? 2 : 1) || (a->stage_off & 15) ||
        !c->peer_ptrs(a->stage_reg, a->stage_off, 2 * a->piece_bytes * c->world, &n.staging))
      return set_error(OOB_ERR_INVALID,
                       "bad staging area (16-byte aligned, piece_bytes >= the message, 2 * world * piece_bytes registered)");
    n.piece_bytes = a->piece_bytes;
    if (algo == OOB_NORM_AR_PUSH_NVLS && n.staging.mc == nullptr) algo = OOB_NORM_AR_PUSH;
  }
  if (max_ctas <= 0) max_ctas = 32;
  cudaError_t e = launch_fused_norm(c->make_ctx(), algo, n, max_ctas, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "fused norm launch");
  return OOB_OK;
}

int oob_gemm(oob_comm* c, const oob_gemm_args_t* a, void* stream) {
  if (a == nullptr) return set_error(OOB_ERR_INVALID, "null argument");
  if (a->dtype != OOB_F16 && a->dtype != OOB_BF16) return set_error(OOB_ERR_INVALID, "GEMM dtype must be fp16 or bf16");
  CommCtx ctx{};
  if (c != nullptr) {
    int rc = check_comm(c);
    if (rc != OOB_OK) return rc;
    ctx = c->make_ctx();
  } else {
    if (a->mode != OOB_GEMM_PLAIN) return set_error(OOB_ERR_INVALID, "fused GEMM modes need a communicator");
    ctx.world = 1;
    ctx.rank = 0;
    ctx.timeout_ns = 2000000000ull;
  }
  GemmArgs g{};
  g.mode = a->mode;
  g.fmt = a->dtype == OOB_BF16 ? 1 : 0;
  g.M = a->M;
  g.N = a->N;
  g.K = a->K;
  g.A = a->A;
  g.lda = a->lda;
  g.B = a->B;
  g.ldb = a->ldb;
  g.C = a->C;
  g.ldc = a->ldc;
  const bool emu = c != nullptr && c->emulated;
  g.a_emu_stride = emu ? a->a_emu_stride : 0;
  g.b_emu_stride = emu ? a->b_emu_stride : 0;
  g.c_emu_stride = emu ? a->c_emu_stride : 0;
  g.comm_ctas = a->comm_ctas;
  g.max_ctas = a->max_ctas;
  g.use_nvls = a->use_nvls;
  g.splits = a->splits;
  g.no_join = a->no_join;
  g.trace = static_cast<unsigned long long*>(a->trace);
  g.pair = a->pair;
  g.skinny = a->skinny;
  g.splitk_reduce = a->splitk_reduce;
  g.gemv = a->gemv;
  g.stream_k = a->stream_k;
  g.order = static_cast<unsigned long long*>(a->order);
  g.epilogue = a->epilogue;
  g.epilogue_args = a->epilogue_args;
  if (a->epilogue != OOB_EPILOGUE_NONE) {
    if (a->mode != OOB_GEMM_PLAIN || emu) return set_error(OOB_ERR_INVALID, "epilogues apply to the plain GEMM only");
    if (a->epilogue_args == nullptr) return set_error(OOB_ERR_INVALID, "null epilogue arguments");
    if (gemm_plan_splits(a->M, a->N, a->K, a->max_ctas, a->splits) <= 1)
      return set_error(OOB_ERR_UNSUPPORTED, "the epilogue runs in the split-K sum, and this problem is not split "
                                            "(see oob_gemm_plan_splits)");
    if (a->epilogue == OOB_EPILOGUE_SWIGLU) {
      const int F = static_cast<const oob_gemm_epilogue_swiglu_t*>(a->epilogue_args)->F;
      if (F <= 0 || F % 8 != 0 || a->N != 2 * F || a->ldc < F || a->ldc % 8 != 0 || a->C == nullptr)
        return set_error(OOB_ERR_INVALID, "SwiGLU epilogue: N must be 2F, F and ldc multiples of 8, ldc >= F");
    } else if (a->epilogue == OOB_EPILOGUE_ROPE_KV) {
      const oob_rope_args_t* r = static_cast<const oob_rope_args_t*>(a->epilogue_args);
      if (r->B <= 0 || r->T <= 0 || r->H <= 0 || r->KV <= 0 || r->hd <= 0 || r->hd % 8 != 0 ||
          static_cast<long long>(r->B) * r->T != a->M || (r->H + 2 * r->KV) * r->hd != a->N)
        return set_error(OOB_ERR_INVALID, "RoPE epilogue: M must be B*T and N (H + 2 KV) * hd");
      if (r->q_out == nullptr || r->k_cache == nullptr || r->v_cache == nullptr || r->cos_table == nullptr ||
          r->sin_table == nullptr)
        return set_error(OOB_ERR_INVALID, "RoPE epilogue: null pointer");
      const uintptr_t align = reinterpret_cast<uintptr_t>(r->q_out) | reinterpret_cast<uintptr_t>(r->k_cache) |
                              reinterpret_cast<uintptr_t>(r->v_cache) | reinterpret_cast<uintptr_t>(r->cos_table) |
                              reinterpret_cast<uintptr_t>(r->sin_table);
      if ((align & 15) || r->cache_batch_stride % 8 != 0 || r->max_len <= 0 || r->batch0 < 0 ||
          r->cache_batch_stride < static_cast<int64_t>(r->KV) * r->max_len * r->hd)
        return set_error(OOB_ERR_INVALID, "RoPE epilogue: bad cache geometry or alignment");
      if (r->pos_dev == nullptr && (r->pos0 < 0 || r->pos0 + r->T > r->max_len))
        return set_error(OOB_ERR_INVALID, "RoPE epilogue: positions outside the cache");
    } else {
      return set_error(OOB_ERR_INVALID, "unknown epilogue");
    }
  }
  g.splitk_ws = nullptr;
  g.counter_base = a->counter_base;
  g.residual = a->residual;
  g.weight = a->weight;
  g.eps = a->eps;
  g.y_local = a->y_local;
  g.res_out_local = a->res_out_local;
  g.rs_emu_stride = emu ? a->rs_emu_stride : 0;
  if (a->mode == OOB_GEMM_AR || a->mode == OOB_GEMM_RS_NORM) {
    if (a->M <= 0 || a->N <= 0) return set_error(OOB_ERR_INVALID, "bad shape");
    if (!c->peer_ptrs(a->partial_reg, a->partial_off, oob_gemm_partial_bytes(a->M, a->N), &g.partial))
      return set_error(OOB_ERR_INVALID, "bad partial buffer (it must hold oob_gemm_partial_bytes(M, N))");
    if (a->partial_off & 1023) return set_error(OOB_ERR_INVALID, "partial buffer must be 1 KiB aligned");
  }
  if (a->mode == OOB_GEMM_AR) {
    if (!c->peer_ptrs(a->c_reg, a->c_off, uint64_t(a->M) * a->N * 2, &g.c_sym) || (a->c_off & 15))
      return set_error(OOB_ERR_INVALID, "bad C buffer");
  }
  if (a->mode == OOB_GEMM_RS_NORM && a->y_local == nullptr) return set_error(OOB_ERR_INVALID, "null y_local");
  if (a->mode == OOB_GEMM_AG) {
    if (a->M <= 0 || a->K <= 0 || !c->peer_ptrs(a->a_full_reg, a->a_full_off, uint64_t(a->M) * a->K * 2, &g.a_full) ||
        (a->a_full_off & 127))
      return set_error(OOB_ERR_INVALID, "bad gathered-A buffer");
  }
  cudaError_t e = launch_gemm(ctx, g, static_cast<cudaStream_t>(stream));
  if (e == cudaErrorStreamCaptureUnsupported) {
    (void)cudaGetLastError();
    return set_error(OOB_ERR_UNSUPPORTED, "this GEMM needs a larger scratch workspace and the stream is being captured: "
                                          "call oob_gemm_reserve_workspace before the capture");
  }
  if (e != cudaSuccess) return cuda_fail(e, "GEMM launch");
  return OOB_OK;
}

uint64_t oob_pad_counter_offset(void) { return uint64_t(kPadCounterOffset) * sizeof(uint32_t); }
int oob_pad_counter_count(void) { return kNumCounters; }

int oob_gemm_plan_splits(int M, int N, int K, int max_ctas, int splits) {
  if (M <= 0 || N <= 0 || K <= 0) return 1;
  return gemm_plan_splits(M, N, K, max_ctas, splits);
}

int oob_gemm_counters_needed(int mode, int M, int N, int world) { return gemm_counters_needed(mode, M, N, world); }

int oob_gemm_reserve_workspace(uint64_t splitk_bytes) {
  cudaError_t e = gemm_pair_reserve_workspace();
  if (e != cudaSuccess) return cuda_fail(e, "reserving the stream-K workspace");
  e = gemm_reserve_splitk(splitk_bytes);
  if (e != cudaSuccess) return cuda_fail(e, "reserving the split-K workspace");
  return OOB_OK;
}

int oob_test_pair_schedule(int mode, int M, int N, int K, int pairs, int stream_k, int world, int rank, int* out, int cap) {
  if (M <= 0 || N <= 0 || K <= 0 || pairs < 1 || out == nullptr) return -1;
  return pair_schedule_dump(mode, M, N, K, pairs, stream_k, world, rank, out, cap);
}

uint64_t oob_gemm_splitk_bytes(int M, int N, int K, int max_ctas, int splits) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  return gemm_splitk_bytes(M, N, K, max_ctas, splits);
}

uint64_t oob_gemm_partial_bytes(int M, int N) {
  // One slice per (tile, source rank) in the owner's buffer: tiles rounded up to a whole number per rank.
  const uint64_t tm = (M + kTileM - 1) / kTileM, tn = (N + kTileN - 1) / kTileN;
  return (tm * tn + kMaxRanks) * kTileBytes;
}

}  // extern "C"
