// Plain structs shared between host code and kernels: the per-launch view of a
// communicator (peer pointer tables, flag pads, status word).
//
// Capability parity: plays the role of the reference's CollectiveLaunchState
// (src/comm/ooverlap_comm_private.h:17-113) and of its ready-signal layout
// (src/comm/ooverlap_comm_internal.h:22-45), re-designed for NVSwitch: every
// rank has the same "signal pad" at the same offset of a symmetric heap, all
// counters only ever grow, and each wait has a time budget.
#pragma once
#include <cstdint>

namespace oob {

constexpr int kMaxRanks = 16;        // same ceiling as the reference (ooverlap_comm_internal.h:19)
constexpr int kMaxCommBlocks = 160;  // CTAs of one collective launch that may take part in rank barriers

// Error codes written by kernels into DeviceStatus::code (0 = ok).
enum DeviceError : int {
  kDevOk = 0,
  kDevTimeoutRankBarrier = 1,   // a peer never published the expected epoch
  kDevTimeoutCounter = 2,       // a tile / row-block arrival counter never reached its target
  kDevTimeoutMbarrier = 3,      // an on-chip pipeline wait ran out of polls
  kDevTimeoutChunkFlag = 4,     // an all-gather chunk never landed
  kDevBadArgument = 5,
};

// One per rank, in host-mapped pinned memory so that the host can read it even
// while a kernel is still running.  First writer wins (atomicCAS on code).
struct DeviceStatus {
  int code;
  int rank;
  int peer;
  int block;
  unsigned expected;
  unsigned observed;
  int where;  // kernel-specific location tag
  int pad;
};

// Signal pad layout inside each rank's symmetric heap (all uint32_t):
//   [0, kMaxCommBlocks*kMaxRanks)     barrier inboxes: inbox[block][sender]
//   then kMaxCommBlocks               private per-block epoch counters (only the owner touches them)
//   then kNumCounters                 general arrival counters (tile / row-block / chunk), zeroed at creation,
//                                     monotonically increasing thereafter
constexpr int kNumCounters = 16384;
constexpr int kPadInboxWords = kMaxCommBlocks * kMaxRanks;
constexpr int kPadEpochOffset = kPadInboxWords;
constexpr int kPadCounterOffset = kPadEpochOffset + kMaxCommBlocks;
constexpr int kPadCallEpochOffset = kPadCounterOffset + kNumCounters;  // 64 per-op call counters
constexpr int kNumCallEpochs = 64;
// One word that mirrors "this rank has recorded an error" in DEVICE memory: waiters poll it instead of the
// host-mapped status block (a poll loop must never read over PCIe).
constexpr int kPadErrorFlagOffset = kPadCallEpochOffset + kNumCallEpochs;
constexpr int kPadWords = kPadErrorFlagOffset + 16;
constexpr uint64_t kPadBytes = ((uint64_t(kPadWords) * 4 + 4095) / 4096) * 4096;

// Passed by value to every communicating kernel.
struct CommCtx {
  int world;
  int rank;
  uint32_t* pad[kMaxRanks];   // every rank's signal pad as mapped in THIS process
  uint32_t* pad_mc;           // multicast mapping of the pad (nullptr when NVLS is unavailable)
  DeviceStatus* status;       // this rank's status block (device-visible)
  uint64_t timeout_ns;        // budget of every cross-GPU wait
  // Single-GPU emulation: when non-null, the launch has gridDim.y == world and
  // block row y acts as rank y with context emu_table[y] (all "ranks" live on
  // one device and the launch is cooperative so that every block is resident).
  const CommCtx* emu_table;
};

// Pointer table of one registered buffer: where each rank's copy is mapped in
// this process, plus the multicast alias (or nullptr).
struct PeerPtrs {
  void* p[kMaxRanks];
  void* mc;
};

}  // namespace oob
