// The communicator object behind the C ABI: symmetric heap, peer mappings,
// multicast alias, signal pad, status block, IPC registrations.
//
// Capability parity: oo_group / oo_node / oo_buffer / oo_ipc_slot_set and the
// launch preparation of the reference (src/comm/ooverlap_comm_internal.h:123-416,
// src/comm/ooverlap_comm_public.cu:707-1240, src/comm/ooverlap_comm_private.cu:218-1358).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <map>
#include <string>
#include <vector>
#include "../device/comm_ctx.h"
#include "bootstrap.h"

struct oob_comm {
  int rank = 0, world = 1, device = 0;
  bool emulated = false;
  int memory_kind = 0;  // 0 VMM fd, 1 legacy IPC, 2 same process
  bool nvls = false;
  bool poisoned = false;
  uint64_t heap_bytes = 0;
  uint64_t timeout_ns = 2000000000ull;
  oob::Bootstrap* boot = nullptr;

  char* heap[oob::kMaxRanks] = {};
  char* heap_mc = nullptr;
  // VMM bookkeeping
  CUmemGenericAllocationHandle handles[oob::kMaxRanks] = {};
  bool handle_valid[oob::kMaxRanks] = {};
  CUmemGenericAllocationHandle mc_handle = 0;
  bool mc_valid = false;
  bool mc_bound = false;
  uint64_t map_bytes = 0;

  oob::DeviceStatus* status_host = nullptr;  // pinned, device-visible
  oob::DeviceStatus* status_dev = nullptr;
  oob::CommCtx* emu_table_dev = nullptr;

  // Symmetric allocator: offset -> size of live blocks, and a sorted free list.
  std::map<uint64_t, uint64_t> live;
  std::map<uint64_t, uint64_t> free_blocks;

  // Legacy-IPC registrations of foreign memory.
  struct Registration {
    void* local = nullptr;
    uint64_t bytes = 0;
    void* peer[oob::kMaxRanks] = {};
    void* import_base[oob::kMaxRanks] = {};  // which cached import each peer pointer lives in
  };
  std::map<int, Registration> regs;
  int next_reg = 1;
  // Import cache: peer rank -> (handle bytes -> mapped base), bounded like the
  // reference's 16-entry per-peer cache (src/comm/ooverlap_comm_internal.h:199-335).
  struct Import {
    cudaIpcMemHandle_t handle;
    void* base;
    uint64_t last_use;
    int refs;  // live registrations that point into this mapping
  };
  std::vector<Import> imports[oob::kMaxRanks];
  uint64_t use_clock = 0;

  oob::CommCtx make_ctx() const;
  // Pointer table of the `bytes` bytes at `off` of registration `reg` (0 = the heap); false when the range does not lie
  // inside the heap / the registration.
  bool peer_ptrs(int reg, uint64_t off, uint64_t bytes, oob::PeerPtrs* out) const;
};
