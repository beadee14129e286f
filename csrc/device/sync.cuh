// Cross-GPU synchronisation built on monotonically increasing 32-bit words in
// each rank's signal pad.  Nothing is ever reset, every wait has a time budget,
// and a wait that runs out records who waited for whom in the rank's status
// block and returns false; kernels then skip their remaining work and exit
// normally (no trap, no endless spin).
//
// Capability parity: the reference's ready signals and CTA grid barrier
// (src/comm/kernels/multi_gpu_ready_signal.cuh:104-336,
// src/comm/kernels/window_task_executor.cuh:17-56) use the same "values only
// grow" idea (epoch*1024+phase) but spin without limit.
#pragma once
#include "comm_ctx.h"
#include "ptx.cuh"

namespace oob {

__device__ __forceinline__ void report_error(const CommCtx& ctx, int code, int peer, unsigned expected,
                                             unsigned observed, int where) {
  DeviceStatus* s = ctx.status;
  if (ctx.pad[ctx.rank] != nullptr) atomicExch(ctx.pad[ctx.rank] + kPadErrorFlagOffset, static_cast<uint32_t>(code));
  if (s == nullptr) return;
  if (atomicCAS(&s->code, 0, code) == 0) {
    s->rank = ctx.rank;
    s->peer = peer;
    s->block = static_cast<int>(blockIdx.x);
    s->expected = expected;
    s->observed = observed;
    s->where = where;
    __threadfence_system();
  }
}

// Wait until (int)(*p - want) >= 0 with acquire semantics, for at most
// timeout_ns.  Returns false on timeout (and records it).
__device__ __forceinline__ bool wait_word_ge(const CommCtx& ctx, const uint32_t* p, uint32_t want, int code,
                                             int peer, int where) {
  uint32_t v = ptx::ld_acquire_sys(p);
  if (static_cast<int32_t>(v - want) >= 0) return true;
  const uint64_t t0 = ptx::globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    v = ptx::ld_acquire_sys(p);
    if (static_cast<int32_t>(v - want) >= 0) return true;
    if (++spins > 64) __nanosleep(spins > 4096 ? 100 : 20);
    if ((spins & 255) == 0) {
      if (ptx::globaltimer_ns() - t0 > ctx.timeout_ns) {
        report_error(ctx, code, peer, want, v, where);
        return false;
      }
      // Somebody on this rank already failed: do not wait out a second budget.  (Device-memory mirror of the
      // status code; the status block itself lives in host memory.)
      if (ctx.pad[ctx.rank] != nullptr &&
          *reinterpret_cast<volatile uint32_t*>(ctx.pad[ctx.rank] + kPadErrorFlagOffset) != 0)
        return false;
    }
  }
}

// Resolve the context of this block: identity in a real launch, row y of the
// emulation table in a single-GPU emulation launch.
__device__ __forceinline__ CommCtx resolve_ctx(const CommCtx& param) {
  if (param.emu_table != nullptr) return param.emu_table[blockIdx.y];
  return param;
}

// Barrier between block `blockIdx.x` of every rank.  All threads of the block
// must call it.  Data written by any thread of this block (to local or peer
// memory) before the call is visible to every thread of the peer blocks after
// their call returns.  Returns false if a peer did not show up in time; the
// return value is uniform across the block.
//
// `slot` selects the inbox row (defaults to blockIdx.x); launches that give
// different roles to different blocks pass their own numbering.
__device__ __forceinline__ bool rank_barrier(const CommCtx& ctx, int slot, int where) {
  __shared__ uint32_t s_epoch;
  __shared__ int s_ok;
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t* ep = ctx.pad[ctx.rank] + kPadEpochOffset + slot;
    s_epoch = *ep + 1;
    *ep = s_epoch;
    s_ok = 1;
  }
  __syncthreads();
  const uint32_t e = s_epoch;
  if (static_cast<int>(threadIdx.x) < ctx.world) {
    const int peer = static_cast<int>(threadIdx.x);
    // Tell `peer` that this rank's block reached epoch e ...
    ptx::st_release_sys(ctx.pad[peer] + slot * kMaxRanks + ctx.rank, e);
    // ... and wait until `peer` told us the same.
    if (!wait_word_ge(ctx, ctx.pad[ctx.rank] + slot * kMaxRanks + peer, e, kDevTimeoutRankBarrier, peer, where))
      s_ok = 0;
  }
  __syncthreads();
  return s_ok != 0;
}

// Per-operation call counter kept in the pad, so that counter targets are
// computed on the device and a captured CUDA graph can be replayed: returns
// the 1-based index of this call of operation `op_slot` on this rank.  Exactly
// one thread of the whole launch (per rank) must call bump; others read after
// a grid-level ordering of their own.
__device__ __forceinline__ uint32_t* call_epoch_ptr(const CommCtx& ctx, int op_slot) {
  return ctx.pad[ctx.rank] + kPadCallEpochOffset + op_slot;
}

__device__ __forceinline__ uint32_t* counter_ptr(const CommCtx& ctx, int rank, int idx) {
  return ctx.pad[rank] + kPadCounterOffset + idx;
}

}  // namespace oob
