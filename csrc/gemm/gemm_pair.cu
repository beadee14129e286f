// Two-SM tcgen05 GEMM for sm_100a: a pair of CTAs on neighbouring SMs (a cluster of two) computes one 256x256
// output tile with tcgen05.mma.cta_group::2.  The same kernel runs the plain GEMM and the three fused
// GEMM + collective ops.
//
// Why pairs: with one CTA per tile every SM stages the whole 256x64 B block of a K step (32 KiB) next to its
// 128x64 A block.  In a pair each CTA stages only HALF of B (128 of the 256 N rows); the tensor cores of the two
// SMs read both halves.  Per SM and K step that is 32 KiB instead of 48 KiB through L2 and shared memory, which
// leaves room for six pipeline stages instead of four and lowers the power spent on data movement -- the GEMM is
// power-capped on this part, so traffic saved is clock gained.
//
// Roles per GEMM CTA:
//   warp 0    TMA producer (both CTAs): loads this CTA's 128 A rows and its 128 B rows of the K step into its own
//             shared memory; the copy's completion is counted on the LEADER CTA's `full` barrier
//             (cp.async.bulk.tensor ... .cta_group::2, no multicast: every byte is loaded once, from this GPU)
//   warp 1    MMA issuer (leader CTA only): one thread issues M256 N256 K16 instructions; tcgen05.commit with a
//             two-CTA mask releases the stage in both CTAs / publishes the accumulator to both epilogues
//   warps 2-5 epilogue (both CTAs): each CTA drains its own 128 accumulator rows from its own TMEM (two
//             accumulator stages), converts, stages through shared memory and writes whole 256-byte row segments
//   warps 6-11 (fused all-reduce / reduce-scatter) signal warps, sharing the CTA's tiles round robin: when the four
//             epilogue warps have stored a tile, one of them orders those stores system-wide and bumps an arrival
//             counter on the rank that reduces the tile
//
// Work distribution.  Tiles are dealt to the pairs round robin, whole waves first.  When the tile count is not a
// multiple of the pair count, the last wave would leave pairs idle; the host may then ask for a STREAM-K TAIL: the
// last (one wave + remainder) tiles are cut along K into equal unit ranges, one per pair.  A pair that computes only
// part of a tile writes its fp32 accumulator to a workspace slot; whichever part arrives last for a 32-row strip
// sums all parts in pair order (bit-reproducible, and nobody waits for anybody) and writes C.
//
// Fused modes (`comm` CTA clusters beside the GEMM pairs, same launch):
//   GEMM->AR      the epilogue writes the partial product into this rank's copy of C in registered memory.  Every
//                 128x256 half tile has an owner rank; once all ranks have stored it, the owner's reducer CTAs read
//                 the sum of all copies (multimem.ld_reduce through the switch, or peer loads) and broadcast it
//                 into every rank's C in place (multimem.st, or peer stores).  Each byte crosses NVLink once per
//                 direction with the switch doing the reduction.
//   GEMM->RS+norm partial products go to a registered [M, N] buffer; the owner of a 128-row block waits until
//                 every rank has stored all its tiles, then its reducers read the rows' sums, add the residual,
//                 apply RMSNorm and write the rank's rows.
//   AG->GEMM      pusher CTAs broadcast this rank's A shard in 128-row chunks into every rank's gathered buffer
//                 and bump per-chunk flags; each CTA's TMA producer waits for the chunk that holds its A rows and
//                 loads it from LOCAL memory.
// Cross-GPU traffic is ld/st/red and multimem.* only.  TMA loads read this GPU's memory and never use cluster
// multicast.  Every wait is bounded; a CTA that gives up records the failure in the status block and both CTAs of
// the pair still meet at the closing cluster barrier (the peer's waits run out as well), so TMEM is always released.
//
// Capability parity with the reference: the plain GEMM (src/gemm/gemm_plain_sm90.cu), the cluster shapes and
// stream-K instances of its generated tables (src/gemm/gemm_plain_sm90_dispatch.h:19-46,
// src/gemm/gemm_with_signal_sm90.h:238-292), the signalling GEMM + wait kernel + per-segment collective
// (src/gemm/gemm_with_signal_sm90.h:102-513, src/wait.cuh:5-9, src/overlap_impl.cu:450-706) and its SM budget knob
// (active_sm_count, src/gemm/gemm_with_signal_sm90.h:408-410).  Hopper's 2x1 cluster with multicast loads maps to
// the Blackwell CTA pair here.
#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>

#include "gemm_kernel.cuh"
#include "gemm_pair.h"

namespace oob {
namespace gemm_pair {

using namespace gemm_detail;

constexpr int kStagesP = 6;
constexpr int kHalfBBytes = (kTileN / 2) * kTileK * 2;   // 16 KiB: this CTA's half of the B block
constexpr int kStageBytesP = kABytes + kHalfBBytes;      // 32 KiB per CTA and stage
constexpr int kPairTileM = 2 * kTileM;                   // 256
constexpr int kSmemBytesP = kStagesP * kStageBytesP + kEpiBytes + 1024 + 256;
constexpr int kThreadsPlainP = 192;
constexpr int kThreadsFusedP = 384;

struct SmemCtlP {
  uint64_t full[kStagesP];         // used in the leader CTA only: bytes of both CTAs' copies
  uint64_t empty[kStagesP];        // per CTA: one arrival from the leader's commit
  uint64_t tmem_full[kAccStages];  // per CTA: one arrival from the leader's commit
  uint64_t tmem_empty[kAccStages]; // used in the leader CTA only: 8 arrivals (4 epilogue warps x 2 CTAs)
  uint32_t tmem_base;
  int abort;
  uint32_t epi_done[4];            // fused AR / RS: epilogue warps that stored their rows of item (index & 3)
};

// ---- PTX used only by the pair kernel ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ptx::smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Tiled load into THIS CTA's shared memory whose completion bytes are counted on a barrier that may live in the
// peer CTA of the pair (`bar_cluster_addr` is a shared::cluster address).  No multicast.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const void* tmap, uint32_t bar_cluster_addr,
                                                 int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(ptx::smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// One arrival on the barrier at this offset in every CTA of `mask`, once the issuing thread's MMAs have completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar, uint16_t mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          ptx::smem_u32(bar)),
      "h"(mask)
      : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Stream-K workspace: arrival flags (one per tail tile, CTA of the pair and epilogue warp), then one fp32 slot of
// 256x256 per pair (a pair parks at most one accumulator: a part that does not start its tile's K range).  Inside a
// slot the layout is the epilogue's own: [cta][warp][32-column chunk][float4 index][lane], so that both the writer
// and the owner that adds the part move whole 512-byte lines.
constexpr size_t kSkSlotFloat4 = size_t(kPairTileM) * kTileN / 4;  // 16384 float4 = 256 KiB
__device__ __forceinline__ uint32_t* sk_flags(void* ws) { return static_cast<uint32_t*>(ws); }
__device__ __forceinline__ float4* sk_slot(void* ws, int slot, int cta, int q) {
  return reinterpret_cast<float4*>(static_cast<char*>(ws) + kSkFlagBytes) + size_t(slot) * kSkSlotFloat4 +
         size_t(cta) * (kSkSlotFloat4 / 2) + size_t(q) * (kSkSlotFloat4 / 8);
}

// ---- epilogue helpers ------------------------------------------------------------------------------------------
// 32 fp32 columns of one row (one row per lane) -> 16-bit -> four 16-byte units of the warp's staging buffer
// ([32 rows][256 bytes], 16-byte units XOR-swizzled by row so that both the row-wise writes here and the
// line-wise reads of copy_out_half are conflict free).
template <typename T>
__device__ __forceinline__ void stage_chunk(uint32_t stage_u32, int lane, int c, const uint32_t (&r)[32]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float lo = __uint_as_float(r[8 * j + 2 * i]), hi = __uint_as_float(r[8 * j + 2 * i + 1]);
      if constexpr (PackTraits<T>::kDType == kBF16) {
        __nv_bfloat162 hh = __floats2bfloat162_rn(lo, hi);
        w[i] = *reinterpret_cast<uint32_t*>(&hh);
      } else {
        __half2 hh = __floats2half2_rn(lo, hi);
        w[i] = *reinterpret_cast<uint32_t*>(&hh);
      }
    }
    const int u = c * 4 + j;  // 16-byte unit of the 256-byte staged row
    const uint32_t saddr = stage_u32 + lane * 256 + ((u ^ (lane & 7)) << 4);
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(saddr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                 : "memory");
  }
}

// Writes the staged half (32 rows x 128 columns) to global memory, two rows per warp instruction.
__device__ __forceinline__ void copy_out_half(uint32_t stage_u32, int lane, char* dst_rows, size_t dst_row_bytes, int h,
                                              int row0, int col0, int M, int N, bool vec_ok) {
#pragma unroll 4
  for (int i = 0; i < 16; ++i) {
    const int rr = 2 * i + (lane >> 4), u = lane & 15;
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(stage_u32 + rr * 256 + ((u ^ (rr & 7)) << 4))
                 : "memory");
    const int grow = row0 + rr;
    const int gcol = col0 + h * 128 + u * 8;
    if (grow < M && gcol < N) {
      char* dst = dst_rows + size_t(rr) * dst_row_bytes + h * 256 + u * 16;
      if (gcol + 8 <= N && vec_ok) {
        ptx::st_v4(dst, v);
      } else {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        for (int e = 0; e < 8 && gcol + e < N; ++e)
          reinterpret_cast<unsigned short*>(dst)[e] =
              static_cast<unsigned short>((e & 1) ? (w[e >> 1] >> 16) : (w[e >> 1] & 0xffff));
      }
    }
  }
}

// ---- communication roles ---------------------------------------------------------------------------------------
// All of them run in the `comm` CTAs behind the GEMM pairs (j = index among them, R = their number), with
// THREADS = kThreadsFusedP threads each.
//
// The reducers work WARP by warp: every warp draws its own small work items, waits for its own flag and keeps its own
// loads in flight, with no block-wide synchronisation between items.  Loads through the switch (and peer loads) have
// microseconds of latency under load, so throughput is bytes in flight / latency: twelve independent warps with 8 KiB
// each keep ~96 KiB per CTA in flight all the time, where a block that synchronised per item idled half of it.

constexpr int kArSubRows = 16;                        // rows of a 128x256 half tile per work item (8 KiB)
constexpr int kArSubsPerUnit = kTileM / kArSubRows;   // 8

// Work items are handed out by a ticket counter, one ticket per warp and item, in schedule order (the order in which
// the GEMMs finish them).  Dedicated communication CTAs draw from the start; every GEMM CTA joins with all its warps
// once it has run out of tiles, so whatever the reduction still has to do when the GEMM ends is spread over the whole
// GPU.  The counter is re-armed by whoever draws the last ticket that can ever be drawn: `total` in-range tickets plus
// one out-of-range ticket per drawing warp.
__device__ __forceinline__ int draw_ticket_warp(uint32_t* ticket, int total, int drawers, int lane) {
  uint32_t t = 0;
  if (lane == 0) {
    t = atomicAdd(ticket, 1u);
    if (t == uint32_t(total + drawers - 1)) {
      *ticket = 0;
      __threadfence();
    }
  }
  return static_cast<int>(__shfl_sync(0xffffffffu, t, 0));
}

// One work item of the GEMM->AR reduction: kArSubRows rows x 256 columns, one 512-byte row per warp instruction.
template <typename T, int NR, bool MC>
__device__ __forceinline__ void ar_reduce_sub(const GemmArgs& a, int world, int rank, size_t off0, size_t row_bytes,
                                              int rows_valid, int packs_valid_row, int lane) {
  // Rows per batch: bounded by registers (a peer reduction holds NR raw packs per result).
  constexpr int U = MC ? kArSubRows : (NR == 0 ? 1 : (NR >= 8 ? 2 : (NR == 4 ? 4 : 8)));
  const bool col_live = lane < packs_valid_row;
#pragma unroll 1
  for (int u0 = 0; u0 < kArSubRows; u0 += U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (col_live && u0 + u < rows_valid) {
        const size_t off = off0 + size_t(u0 + u) * row_bytes + size_t(lane) * 16;
        if constexpr (MC)
          v[u] = reduce_pack_mc<T, kSum>(static_cast<const char*>(a.c_sym.mc) + off);
        else
          v[u] = reduce_pack_p2p<T, kSum, NR>(a.c_sym, off, world);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (col_live && u0 + u < rows_valid) {
        const size_t off = off0 + size_t(u0 + u) * row_bytes + size_t(lane) * 16;
        if constexpr (MC) {
          ptx::multimem_st_v4(static_cast<char*>(a.c_sym.mc) + off, v[u]);
        } else if constexpr (NR > 0) {
#pragma unroll
          for (int r = 0; r < NR; ++r) ptx::st_v4(static_cast<char*>(a.c_sym.p[(rank + r) % NR]) + off, v[u]);
        } else {
          for (int r = 0; r < world; ++r) ptx::st_v4(static_cast<char*>(a.c_sym.p[(rank + r) % world]) + off, v[u]);
        }
      }
    }
  }
}

// GEMM->AR.  Unit u = 2 * seq + cta is the 128x256 half tile that CTA `cta` of a pair stores for schedule position
// seq.  Its owner is rank u % world; the k-th unit of a rank (u = k * world + rank) has two counters on that rank:
// counter_base + k counts the ranks that have stored it, counter_base + owned_max + k the finished work items (whoever
// finishes the last one re-arms both); counter_base + 2 * owned_max is the ticket counter.  Work item i = (unit i / 8,
// rows 16 * (i % 8) ...).  `drawers` = warps of the launch that draw tickets.
template <typename T, int THREADS>
__device__ void pair_ar_reducer(const CommCtx& ctx, const GemmArgs& a, const PairSched& sc, int drawers,
                                bool stamp_first = true) {
  const int world = ctx.world, rank = ctx.rank;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int W = THREADS / 32;
  const bool use_mc = a.c_sym.mc != nullptr && a.use_nvls != 0;
  const size_t row_bytes = size_t(a.N) * 2;
  const int units = 2 * sc.tiles;
  const int owned = (units - rank + world - 1) / world;
  const int owned_max = (units + world - 1) / world;
  const int items = owned * kArSubsPerUnit;
  uint32_t* ticket = counter_ptr(ctx, rank, a.counter_base + 2 * owned_max);
  (void)W;
  bool ok = true;
  unsigned long long t_wait = 0, n_items = 0;
  // The next ticket is drawn before the current item is processed: its round trip hides behind the item's loads.
  int next = draw_ticket_warp(ticket, items, drawers, lane);
  while (true) {
    const int i = next;
    if (i >= items) break;
    next = draw_ticket_warp(ticket, items, drawers, lane);
    if (!ok) continue;  // after a timeout: keep drawing so that every warp ends with its one out-of-range ticket
    const int k = i / kArSubsPerUnit, sub = i % kArSubsPerUnit;
    uint32_t* cnt = counter_ptr(ctx, rank, a.counter_base + k);
    uint32_t* done = counter_ptr(ctx, rank, a.counter_base + owned_max + k);
    int good = 1;
    if (lane == 0) {
      const unsigned long long tw = (a.trace && warp == 0) ? ptx::globaltimer_ns() : 0;
      good = wait_word_ge(ctx, cnt, world, kDevTimeoutCounter, -1, 52) ? 1 : 0;
      if (a.trace && warp == 0) {
        const unsigned long long now = ptx::globaltimer_ns();
        t_wait += now - tw;
        if (n_items == 0 && threadIdx.x == 0 && stamp_first) trace_put(a, kTraceFirstReady, now);
      }
    }
    good = __shfl_sync(0xffffffffu, good, 0);
    if (!good) {
      ok = false;
      continue;
    }
    ++n_items;
    const int u = k * world + rank;
    int m_blk, n_blk;
    sc.coord(u >> 1, m_blk, n_blk);
    const int m0 = m_blk * kPairTileM + (u & 1) * kTileM + sub * kArSubRows, n0 = n_blk * kTileN;
    const int rows_valid = min(kArSubRows, a.M - m0);
    const int packs_valid_row = min(kPacksPerTileRow, (a.N - n0) / 8);
    if (rows_valid > 0 && packs_valid_row > 0) {
      const size_t off0 = size_t(m0) * row_bytes + size_t(n0) * 2;
      if (use_mc)
        ar_reduce_sub<T, 0, true>(a, world, rank, off0, row_bytes, rows_valid, packs_valid_row, lane);
      else if (world == 2)
        ar_reduce_sub<T, 2, false>(a, world, rank, off0, row_bytes, rows_valid, packs_valid_row, lane);
      else if (world == 4)
        ar_reduce_sub<T, 4, false>(a, world, rank, off0, row_bytes, rows_valid, packs_valid_row, lane);
      else if (world == 8)
        ar_reduce_sub<T, 8, false>(a, world, rank, off0, row_bytes, rows_valid, packs_valid_row, lane);
      else
        ar_reduce_sub<T, 0, false>(a, world, rank, off0, row_bytes, rows_valid, packs_valid_row, lane);
    }
    // Whoever finishes the last item of a unit re-arms its counters.  The next call's arrivals cannot come before
    // this launch has ended on every rank (the closing rank barrier); counters that timed out are zeroed by recover().
    __syncwarp();
    if (lane == 0) {
      if (atomicAdd(done, 1u) == uint32_t(kArSubsPerUnit - 1)) {
        *cnt = 0;
        *done = 0;
        __threadfence();
      }
    }
  }
  const int all_ok = __syncthreads_and(ok ? 1 : 0);
  if (a.trace) {
    trace_put(a, kTraceCommDone, ptx::globaltimer_ns());
    trace_put(a, kTraceItems, n_items);
    trace_put(a, kTraceWaitNs, t_wait);
  }
  // CTA b of every rank is past its last item: together (all drawing CTAs) this means every result has been written
  // into this rank's C, and nobody reads this rank's partial products any more.
  if (all_ok) rank_barrier(ctx, blockIdx.x, 53);
  if (a.trace) trace_put(a, kTraceEnd, ptx::globaltimer_ns());
}

// GEMM->RS + residual + RMSNorm.  The owner of a 128-row block (local index lb) has two counters for it:
// counter_base + lb counts stored half tiles (tiles_n per rank), counter_base + blocks + lb counts finished rows
// (whoever finishes the last one re-arms both).  A work item is ONE ROW of the rank's shard, handled by one warp:
//   pass 1  the row's sums are read 8 packs per lane at a time (through the switch, or from all peers), the residual is
//           added, the 16-bit rounded values are written to the residual output (or to y, as scratch) and their squares
//           accumulated;
//   pass 2  the warp reduces the sum of squares with shuffles, re-reads its own rounded values (each lane the packs it
//           wrote: L2 hits, ordered by program order) and writes the normalised row.
// No block-wide synchronisation, any N that is a multiple of 8.
template <typename T, int NR, bool MC>
__device__ __forceinline__ void rs_row(const GemmArgs& a, int world, size_t grow, size_t lrow, const char* res, char* y,
                                       char* ro, const char* wgt, int lane) {
  using PT = PackTraits<T>;
  constexpr int U = MC ? 8 : (NR == 2 ? 4 : (NR == 4 ? 2 : 1));
  const int packs_per_row = a.N / 8;
  const size_t row_bytes = size_t(a.N) * 2;
  const size_t g_off = grow * row_bytes, l_off = lrow * row_bytes;
  char* stash = ro != nullptr ? ro : y;
  float ss = 0.f;
#pragma unroll 1
  for (int c0 = 0; c0 < packs_per_row; c0 += 32 * U) {
    float f[U][8];
    if constexpr (MC) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int p = c0 + u * 32 + lane;
        v[u] = make_uint4(0u, 0u, 0u, 0u);
        // lanes past the end of the row load nothing: a load through the switch is link traffic on every rank
        if (p < packs_per_row) v[u] = reduce_pack_mc<T, kSum>(static_cast<const char*>(a.partial.mc) + g_off + size_t(p) * 16);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) PT::unpack(v[u], f[u]);
    } else {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int p = c0 + u * 32 + lane;
        if (p < packs_per_row) reduce_pack_p2p_f32<T, kSum, NR>(a.partial, g_off + size_t(p) * 16, world, f[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int p = c0 + u * 32 + lane;
      if (p >= packs_per_row) continue;
      if (res != nullptr) {
        float rf[8];
        PT::unpack(ptx::ld_nc_v4(res + l_off + size_t(p) * 16), rf);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[u][i] += rf[i];
      }
      // The normalisation sees the 16-bit value that is also written out as the new residual.
      const uint4 rounded = PT::pack(f[u]);
      PT::unpack(rounded, f[u]);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += f[u][i] * f[u][i];
      ptx::st_v4(stash + l_off + size_t(p) * 16, rounded);
      if (wgt == nullptr && ro != nullptr) ptx::st_v4(y + l_off + size_t(p) * 16, rounded);
    }
  }
  if (wgt == nullptr) return;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float scale = rsqrtf(ss / float(a.N) + a.eps);
#pragma unroll 2
  for (int p = lane; p < packs_per_row; p += 32) {
    float f[8], wf[8], o[8];
    // Written a moment ago by this same lane: a plain (coherent) load, not the read-only path.
    PT::unpack(*reinterpret_cast<const uint4*>(stash + l_off + size_t(p) * 16), f);
    PT::unpack(*reinterpret_cast<const uint4*>(wgt + size_t(p) * 16), wf);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = f[i] * scale * wf[i];
    ptx::st_v4(y + l_off + size_t(p) * 16, PT::pack(o));
  }
}

template <typename T, int THREADS>
__device__ void pair_rs_reducer(const CommCtx& ctx, const GemmArgs& a, const PairSched& sc, int drawers,
                                bool stamp_first = true) {
  const int world = ctx.world, rank = ctx.rank;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int W = THREADS / 32;
  const bool use_mc = a.partial.mc != nullptr && a.use_nvls != 0;
  const int rows_per_rank = a.M / world;
  const int blocks = rows_per_rank / kTileM;
  const char* res = a.residual ? static_cast<const char*>(a.residual) + a.rs_emu_stride * blockIdx.y : nullptr;
  char* y = static_cast<char*>(a.y_local) + a.rs_emu_stride * blockIdx.y;
  char* ro = a.res_out_local ? static_cast<char*>(a.res_out_local) + a.rs_emu_stride * blockIdx.y : nullptr;
  const char* wgt = static_cast<const char*>(a.weight);
  uint32_t* ticket = counter_ptr(ctx, rank, a.counter_base + 2 * blocks);
  (void)W;
  bool ok = true;
  unsigned long long t_wait = 0, n_items = 0;
  int ready_lb = -1;  // blocks up to here are known to be complete
  int next = draw_ticket_warp(ticket, rows_per_rank, drawers, lane);
  while (true) {
    const int r = next;
    if (r >= rows_per_rank) break;
    next = draw_ticket_warp(ticket, rows_per_rank, drawers, lane);
    if (!ok) continue;
    const int lb = r / kTileM;
    uint32_t* cnt = counter_ptr(ctx, rank, a.counter_base + lb);
    uint32_t* done = counter_ptr(ctx, rank, a.counter_base + blocks + lb);
    if (lb > ready_lb) {
      int good = 1;
      if (lane == 0) {
        const unsigned long long tw = (a.trace && warp == 0) ? ptx::globaltimer_ns() : 0;
        good = wait_word_ge(ctx, cnt, uint32_t(world) * sc.tiles_n, kDevTimeoutCounter, -1, 62) ? 1 : 0;
        if (a.trace && warp == 0) {
          const unsigned long long now = ptx::globaltimer_ns();
          t_wait += now - tw;
          if (n_items == 0 && threadIdx.x == 0 && stamp_first) trace_put(a, kTraceFirstReady, now);
        }
      }
      good = __shfl_sync(0xffffffffu, good, 0);
      if (!good) {
        ok = false;
        continue;
      }
      ready_lb = lb;
    }
    ++n_items;
    const size_t grow = size_t(rank) * rows_per_rank + r;
    if (use_mc)
      rs_row<T, 0, true>(a, world, grow, r, res, y, ro, wgt, lane);
    else if (world == 2)
      rs_row<T, 2, false>(a, world, grow, r, res, y, ro, wgt, lane);
    else if (world == 4)
      rs_row<T, 4, false>(a, world, grow, r, res, y, ro, wgt, lane);
    else if (world == 8)
      rs_row<T, 8, false>(a, world, grow, r, res, y, ro, wgt, lane);
    else
      rs_row<T, 0, false>(a, world, grow, r, res, y, ro, wgt, lane);
    // Whoever finishes the last row of a block re-arms the block's counters for the next call.
    __syncwarp();
    if (lane == 0) {
      if (atomicAdd(done, 1u) == uint32_t(kTileM - 1)) {
        *cnt = 0;
        *done = 0;
        __threadfence();
      }
    }
  }
  const int all_ok = __syncthreads_and(ok ? 1 : 0);
  if (a.trace) {
    trace_put(a, kTraceCommDone, ptx::globaltimer_ns());
    trace_put(a, kTraceItems, n_items);
    trace_put(a, kTraceWaitNs, t_wait);
  }
  // Nobody reads this rank's partial products any more once CTA b of every rank is here.
  if (all_ok) rank_barrier(ctx, blockIdx.x, 63);
  if (a.trace) trace_put(a, kTraceEnd, ptx::globaltimer_ns());
}

// The last CTA of the launch (GEMM CTAs and pushers) to get here zeroes the chunk flags: every flag has reached its
// final value by then.
__device__ __forceinline__ void ag_rearm_flags(const CommCtx& ctx, const GemmArgs& a, int ctas) {
  const int chunks_all = a.M / kTileM;
  uint32_t* done = counter_ptr(ctx, ctx.rank, a.counter_base + chunks_all);
  __threadfence();
  if (atomicAdd(done, 1u) == uint32_t(ctas - 1)) {
    __threadfence();
    for (int i = 0; i < chunks_all; ++i) *counter_ptr(ctx, ctx.rank, a.counter_base + i) = 0;
    *done = 0;
    __threadfence();
  }
}

template <int THREADS>
__device__ void pair_ag_pusher(const CommCtx& ctx, const GemmArgs& a, int j, int R, int gemm_ctas) {
  const int world = ctx.world, rank = ctx.rank;
  const bool use_mc = a.a_full.mc != nullptr && ctx.pad_mc != nullptr && a.use_nvls != 0;
  // Previous call's readers of the gathered buffers are done once every rank has entered this call.
  if (!rank_barrier(ctx, j, 72)) return;
  const char* src = static_cast<const char*>(a.A) + a.a_emu_stride * blockIdx.y;
  const size_t row_bytes = size_t(a.K) * 2;  // gathered buffer is dense [M, K]
  const size_t src_row_bytes = size_t(a.lda) * 2;
  const int packs_per_row = a.K / 8;
  const int shard_rows = a.M / world;
  const int chunks = shard_rows / kTileM;
  for (int c = 0; c < chunks; ++c) {
    const int row0 = c * kTileM;
    const int total = kTileM * packs_per_row;
    constexpr int U = 8;
    for (int pb = j * THREADS + threadIdx.x; pb < total; pb += R * THREADS * U) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int p = pb + u * R * THREADS;
        const int pc = p < total ? p : pb;
        v[u] = ptx::ld_nc_v4(src + size_t(row0 + pc / packs_per_row) * src_row_bytes + size_t(pc % packs_per_row) * 16);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int p = pb + u * R * THREADS;
        if (p >= total) continue;
        const int row = row0 + p / packs_per_row, cp = p % packs_per_row;
        const size_t doff = size_t(rank * shard_rows + row) * row_bytes + size_t(cp) * 16;
        if (use_mc) {
          ptx::multimem_st_v4(static_cast<char*>(a.a_full.mc) + doff, v[u]);
        } else {
          for (int r = 1; r < world; ++r) ptx::st_v4(static_cast<char*>(a.a_full.p[(rank + r) % world]) + doff, v[u]);
        }
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      ptx::fence_acq_rel_sys();
      const int idx = a.counter_base + rank * chunks + c;
      if (use_mc) {
        ptx::multimem_red_add_u32(ctx.pad_mc + kPadCounterOffset + idx, 1u);
      } else {
        for (int r = 1; r < world; ++r) ptx::red_release_sys_add(counter_ptr(ctx, (rank + r) % world, idx), 1u);
      }
    }
  }
  // Through the switch the flags of this rank's own chunks are bumped as well (nobody waits for them), so the pushers
  // take part in the count that decides who re-arms the flags.
  __syncthreads();
  if (threadIdx.x == 0) {
    ptx::fence_acq_rel_sys();
    ag_rearm_flags(ctx, a, gemm_ctas + R);
  }
}

// True when all four epilogue warps have stored item `idx` of this CTA (see epi_done).  Safe for any idx: the four
// warps are never more than the two accumulator stages apart, and the counts only grow.
__device__ __forceinline__ bool ctl_epi_done_ge(const SmemCtlP* ctl, uint32_t idx) {
  return *reinterpret_cast<const volatile uint32_t*>(&ctl->epi_done[idx & 3]) >= 4u * (idx / 4u + 1u);
}

// ---- the kernel ------------------------------------------------------------------------------------------------
// SK: compiled with the stream-K tail (partial items); launches without a tail use the leaner instantiation.
template <typename T, int MODE, bool SK>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(MODE == kGemmPlain ? kThreadsPlainP : kThreadsFusedP, 1)
    gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                     const __grid_constant__ CUtensorMap tmap_a_local, EmuMaps emu, CommCtx ctx_param, GemmArgs a,
                     PairPlan plan) {
  constexpr int THREADS = MODE == kGemmPlain ? kThreadsPlainP : kThreadsFusedP;
  constexpr int FMT = PackTraits<T>::kDType == kBF16 ? 1 : 0;
  constexpr bool kSignals = MODE == kGemmAr || MODE == kGemmRsNorm;
  extern __shared__ uint8_t smem_raw[];
  // The same offset in both CTAs (same kernel, same dynamic shared memory base), as the MMA descriptors require.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  SmemCtlP* ctl = reinterpret_cast<SmemCtlP*>(smem + kStagesP * kStageBytesP + kEpiBytes);

  const CommCtx ctx = resolve_ctx(ctx_param);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();  // 0 = leader
  const bool leader = cta == 0;
  const int pair = blockIdx.x >> 1;
  if (a.trace) {
    trace_put(a, kTraceStart, ptx::globaltimer_ns());
    trace_put(a, kTraceRole, pair >= plan.gemm_pairs ? 1 : 0);
  }

  PairSched sc;
  sc.num_kb = (a.K + kTileK - 1) / kTileK;
  sc.tiles_m = (a.M + kPairTileM - 1) / kPairTileM;
  sc.tiles_n = (a.N + kTileN - 1) / kTileN;
  sc.tiles = sc.tiles_m * sc.tiles_n;
  sc.P = plan.gemm_pairs;
  sc.sk_tiles = plan.sk_tiles;
  sc.sk_pairs = plan.sk_pairs;
  sc.sk_units = plan.sk_tiles * sc.num_kb;
  sc.dp_tiles = sc.tiles - sc.sk_tiles;
  sc.mode = MODE;
  sc.world = ctx.world;
  sc.rank = ctx.rank;
  sc.bpr = 0;
  if constexpr (MODE == kGemmRsNorm || MODE == kGemmAg) {
    const int rows_per_rank = a.M / ctx.world;
    if (rows_per_rank % kPairTileM == 0) sc.bpr = rows_per_rank / kPairTileM;
  }

  // ---- communication CTAs ----------------------------------------------------------------------------------------
  if constexpr (MODE != kGemmPlain) {
    if (pair >= plan.gemm_pairs) {
      const int j = int(blockIdx.x) - 2 * plan.gemm_pairs, R = int(gridDim.x) - 2 * plan.gemm_pairs;
      const int drawers = (a.no_join ? R : int(gridDim.x)) * (THREADS / 32);
      if constexpr (MODE == kGemmAr) pair_ar_reducer<T, THREADS>(ctx, a, sc, drawers);
      if constexpr (MODE == kGemmRsNorm) pair_rs_reducer<T, THREADS>(ctx, a, sc, drawers);
      if constexpr (MODE == kGemmAg) pair_ag_pusher<THREADS>(ctx, a, j, R, 2 * plan.gemm_pairs);
      return;
    }
  }

  // ---- GEMM CTAs -------------------------------------------------------------------------------------------------
  const CUtensorMap* ta = emu.table ? &emu.table[3 * blockIdx.y + 0] : &tmap_a;
  const CUtensorMap* tb = emu.table ? &emu.table[3 * blockIdx.y + 1] : &tmap_b;
  const CUtensorMap* tal = emu.table ? &emu.table[3 * blockIdx.y + 2] : &tmap_a_local;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStagesP; ++s) {
      ptx::mbar_init(&ctl->full[s], 1);
      ptx::mbar_init(&ctl->empty[s], 1);
    }
    for (int s = 0; s < kAccStages; ++s) {
      ptx::mbar_init(&ctl->tmem_full[s], 1);
      ptx::mbar_init(&ctl->tmem_empty[s], 8);
    }
    for (int s = 0; s < 4; ++s) ctl->epi_done[s] = 0;
    ctl->abort = 0;
    ptx::mbar_fence_init();
    ptx::prefetch_tmap(ta);
    ptx::prefetch_tmap(tb);
    if constexpr (MODE == kGemmAg) ptx::prefetch_tmap(tal);
  }
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anything can signal them
  if (warp == 1) {
    tmem_alloc_pair(&ctl->tmem_base, kTmemCols);
    tmem_relinquish_pair();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // both CTAs hold their TMEM before the first MMA writes into it
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;
  volatile int* abort = &ctl->abort;

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------- TMA producer (both CTAs) -------------------------
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      ItemIter iter(sc, pair);
      Item it;
      while (ok && iter.next(sc, pair, it)) {
        int m_blk, n_blk;
        sc.coord(it.seq, m_blk, n_blk);
        const CUtensorMap* tma_a_cur = ta;
        int a_row = m_blk * kPairTileM + int(cta) * kTileM;
        const int b_row = n_blk * kTileN + int(cta) * (kTileN / 2);
        if constexpr (MODE == kGemmAg) {
          const int shard_rows = a.M / ctx.world;
          const int owner = a_row / shard_rows;
          if (a_row < a.M) {
            if (owner == ctx.rank) {
              tma_a_cur = tal;  // own rows are read from the shard itself
              a_row -= owner * shard_rows;
            } else {
              // Gathered rows: wait until all pushers of `owner` delivered this chunk into LOCAL memory.
              const int R = int(gridDim.x) - 2 * plan.gemm_pairs;
              ok = wait_word_ge(ctx, counter_ptr(ctx, ctx.rank, a.counter_base + a_row / kTileM), R, kDevTimeoutChunkFlag,
                                owner, 73);
              if (!ok) {
                *abort = 1;
                break;
              }
              ptx::fence_proxy_async_global();
            }
          }
        }
        for (int kb = it.kb0; kb < it.kb1; ++kb) {
          if (!ptx::mbar_wait(&ctl->empty[stage], phase ^ 1, abort)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * kStageBytesP;
          uint8_t* sb = sa + kABytes;
          const uint32_t full_leader = map_to_cta(ptx::smem_u32(&ctl->full[stage]), 0);
          if (leader) ptx::mbar_arrive_expect_tx(&ctl->full[stage], 2 * kStageBytesP);
          tma_load_2d_pair(sa, tma_a_cur, full_leader, kb * kTileK, a_row);
          tma_load_2d_pair(sb, tb, full_leader, kb * kTileK, b_row);
          if (++stage == kStagesP) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      // ------------------------- MMA issuer (leader CTA) ---------------------------
      constexpr uint32_t idesc = ptx::umma_idesc_f16(FMT, kPairTileM, kTileN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      ItemIter iter(sc, pair);
      Item it;
      while (ok && iter.next(sc, pair, it)) {
        if (!ptx::mbar_wait(&ctl->tmem_empty[acc], acc_phase ^ 1, abort)) break;
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * kTileN;
        for (int kb = it.kb0; kb < it.kb1; ++kb) {
          if (!ptx::mbar_wait(&ctl->full[stage], phase, abort)) {
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint32_t sa = ptx::smem_u32(smem + stage * kStageBytesP);
          const uint64_t da = ptx::umma_desc_kmajor_sw128(sa);
          const uint64_t db = ptx::umma_desc_kmajor_sw128(sa + kABytes);
#pragma unroll
          for (int k = 0; k < kTileK / 16; ++k)
            umma_f16_pair(d_tmem, da + uint64_t(k * 2), db + uint64_t(k * 2), idesc, (kb > it.kb0 || k > 0) ? 1u : 0u);
          umma_commit_pair(&ctl->empty[stage], 3);  // both CTAs may refill this stage
          if (++stage == kStagesP) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit_pair(&ctl->tmem_full[acc], 3);  // accumulator complete, in both CTAs' TMEM
        if (++acc == kAccStages) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else if (warp < 6) {
    // --------------------------- epilogue (both CTAs) -----------------------------
    const int q = warp & 3;  // TMEM lane quadrant this warp may read
    uint8_t* stage_buf = smem + kStagesP * kStageBytesP + (warp - 2) * kEpiWarpBytes;
    const uint32_t stage_u32 = ptx::smem_u32(stage_buf);
    int acc = 0;
    uint32_t acc_phase = 0;
    uint32_t idx = 0;
    // Destination matrix of this rank's tiles: C, this rank's copy of the symmetric C (AR, reduced in place
    // afterwards), or the registered buffer of partial products (RS).
    char* c_base;
    int ldc;
    if constexpr (MODE == kGemmAr) {
      c_base = static_cast<char*>(a.c_sym.p[ctx.rank]);
      ldc = a.N;
    } else if constexpr (MODE == kGemmRsNorm) {
      c_base = static_cast<char*>(a.partial.p[ctx.rank]);
      ldc = a.N;
    } else {
      c_base = static_cast<char*>(a.C) + a.c_emu_stride * blockIdx.y;
      ldc = a.ldc;
    }
    const bool vec_ok = (ldc % 8) == 0;
    const size_t dst_row_bytes = size_t(ldc) * 2;
    ItemIter iter(sc, pair);
    Item it;
    for (; iter.next(sc, pair, it); ++idx) {
      int m_blk, n_blk;
      sc.coord(it.seq, m_blk, n_blk);
      if (!ptx::mbar_wait(&ctl->tmem_full[acc], acc_phase, abort)) break;
      ptx::tc_fence_after_sync();
      const uint32_t t_addr = tmem_base + (uint32_t(q * 32) << 16) + acc * kTileN;
      const int row0 = m_blk * kPairTileM + int(cta) * kTileM + q * 32;  // first of this warp's 32 rows
      const int col0 = n_blk * kTileN;
      char* dst_rows = c_base + (size_t(row0) * ldc + size_t(col0)) * 2;
      bool whole = true;
      if constexpr (SK) whole = !it.partial;
      if (whole) {
#pragma unroll 1
        for (int h = 0; h < 2; ++h) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            ptx::tmem_ld_32x32b_x32(t_addr + h * 128 + c * 32, r);
            ptx::tmem_ld_wait();
            stage_chunk<T>(stage_u32, lane, c, r);
          }
          if (h == 1) {
            // Everything has left TMEM: hand the accumulator stage back to the leader's MMA thread.
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(ptx::smem_u32(&ctl->tmem_empty[acc]), 0));
          }
          __syncwarp();
          copy_out_half(stage_u32, lane, dst_rows, dst_row_bytes, h, row0, col0, a.M, a.N, vec_ok);
          __syncwarp();
        }
        if constexpr (!kSignals) {
          if (a.order != nullptr && q == 3 && lane == 0) {
            unsigned long long* rec = a.order + 2 * (2 * size_t(it.seq) + cta);
            rec[0] = ptx::globaltimer_ns();
            rec[1] = (static_cast<unsigned long long>(pair) << 32) | idx;
          }
        }
        if constexpr (kSignals) {
          // This warp's rows of the tile are stored (to LOCAL memory).  The signal warp publishes the tile once
          // all four epilogue warps are here; the fence below orders this warp's stores before the count.
          if (lane == 0) {
            __threadfence_block();
            atomicAdd(&ctl->epi_done[idx & 3], 1u);
          }
        }
      } else if constexpr (SK) {
        // Stream-K: this pair computed K blocks [kb0, kb1) of the tile only.
        const int u_first = it.sk_tile * sc.num_kb;
        const int p_first = sc.sk_owner(u_first), p_last = sc.sk_owner(u_first + sc.num_kb - 1);
        uint32_t* flag = sk_flags(plan.sk_ws) + (it.sk_tile * 2 + int(cta)) * 4 + q;
        if (it.kb0 > 0) {
          // Not the beginning of the tile's K range: park the fp32 accumulator in this pair's slot and tell the
          // pair that owns the tile.  A pair does this FIRST in its tail range (right after its whole tiles), the
          // owner needs it LAST in its own range, so the owner practically never waits.
          float4* ws = sk_slot(plan.sk_ws, pair, int(cta), q);
#pragma unroll 2
          for (int c = 0; c < kTileN / 32; ++c) {
            uint32_t r[32];
            ptx::tmem_ld_32x32b_x32(t_addr + c * 32, r);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 8; ++i)
              __stcg(&ws[(c * 8 + i) * 32 + lane],
                     make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]), __uint_as_float(r[4 * i + 2]),
                                 __uint_as_float(r[4 * i + 3])));
          }
          ptx::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) {
            mbar_arrive_cluster(map_to_cta(ptx::smem_u32(&ctl->tmem_empty[acc]), 0));
            __threadfence();  // the warp's stores (ordered before this thread by the barrier above) before the flag
            atomicAdd(flag, 1u);
          }
        } else {
          // The beginning of the tile's K range: this pair owns the tile.  It adds the other parts to its own
          // accumulator in pair order (bit-reproducible) and writes C.  The parts are read three 32-column chunks
          // ahead of their use, so that their L2 latency hides behind the TMEM reads and conversions.
          const uint32_t others = uint32_t(p_last - p_first);
          if (lane == 0) {
            uint32_t polls = 0;
            while (ld_acquire_gpu(flag) < others) {
              if (*abort || ++polls > (1u << 24)) {
                *abort = 1;
                break;
              }
              __nanosleep(64);
            }
            *flag = 0;  // re-arm for the next call (all arrivals of this call are in)
          }
          __syncwarp();
          if (*abort) break;
          // (one chunk ahead in the fused kernels: their 384 threads leave 168 registers per thread)
          constexpr int PF = THREADS > kThreadsPlainP ? 1 : 3;
          const float4* src1 = sk_slot(plan.sk_ws, p_first + 1, int(cta), q) + lane;
          float4 pre[PF][8];
#pragma unroll
          for (int c = 0; c < PF; ++c)
#pragma unroll
            for (int i = 0; i < 8; ++i) pre[c][i] = __ldcg(src1 + (c * 8 + i) * 32);
#pragma unroll(PF == 1 ? 1 : kTileN / 32)
          for (int c = 0; c < kTileN / 32; ++c) {
            uint32_t r[32];
            ptx::tmem_ld_32x32b_x32(t_addr + c * 32, r);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float4 v = pre[c % PF][i];
              r[4 * i] = __float_as_uint(__uint_as_float(r[4 * i]) + v.x);
              r[4 * i + 1] = __float_as_uint(__uint_as_float(r[4 * i + 1]) + v.y);
              r[4 * i + 2] = __float_as_uint(__uint_as_float(r[4 * i + 2]) + v.z);
              r[4 * i + 3] = __float_as_uint(__uint_as_float(r[4 * i + 3]) + v.w);
            }
            if (c + PF < kTileN / 32) {
#pragma unroll
              for (int i = 0; i < 8; ++i) pre[c % PF][i] = __ldcg(src1 + ((c + PF) * 8 + i) * 32);
            }
            // A tile cut into more than two parts (ranges shorter than a tile): the further parts, in pair order.
            for (int p = p_first + 2; p <= p_last; ++p) {
              const float4* src = sk_slot(plan.sk_ws, p, int(cta), q) + lane + c * 8 * 32;
              float4 v[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) v[i] = __ldcg(src + i * 32);
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                r[4 * i] = __float_as_uint(__uint_as_float(r[4 * i]) + v[i].x);
                r[4 * i + 1] = __float_as_uint(__uint_as_float(r[4 * i + 1]) + v[i].y);
                r[4 * i + 2] = __float_as_uint(__uint_as_float(r[4 * i + 2]) + v[i].z);
                r[4 * i + 3] = __float_as_uint(__uint_as_float(r[4 * i + 3]) + v[i].w);
              }
            }
            stage_chunk<T>(stage_u32, lane, c & 3, r);
            if ((c & 3) == 3) {
              if (c == kTileN / 32 - 1) {
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(map_to_cta(ptx::smem_u32(&ctl->tmem_empty[acc]), 0));
              }
              __syncwarp();
              copy_out_half(stage_u32, lane, dst_rows, dst_row_bytes, c >> 2, row0, col0, a.M, a.N, vec_ok);
              __syncwarp();
            }
          }
        }
      }
      if (++acc == kAccStages) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
    // Trace: when this CTA's last tile had left the epilogue (the signal warps may still be publishing).
    if constexpr (kSignals) {
      if (a.trace != nullptr && q == 0 && lane == 0)  // not thread 0 of the CTA: written directly
        a.trace[(size_t(blockIdx.y) * gridDim.x + blockIdx.x) * kTraceWords + kTraceFirstReady] = ptx::globaltimer_ns();
    }
  } else if (warp >= 6) {
    // --------------------------- signal warps (fused AR / RS) ----------------------------
    // Warps 6 .. 11 share the CTA's items round robin (item idx belongs to warp 6 + idx % kSignalWarps); one thread of
    // each follows its items in order.  When all four epilogue warps have stored their rows of a tile it orders those
    // stores system-wide (the fence is cumulative over what it observed through the CTA-scope counter) and publishes
    // one arrival on the rank that reduces the tile.  Several warps, because a publication is a chain of a
    // system-scope fence and a remote reduction that takes far longer than a short tile (K / world of a few hundred)
    // takes to compute: one warp alone would publish the tiles later than they are produced.
    if constexpr (kSignals) {
      constexpr int kSignalWarps = THREADS / 32 - 6;
      const int sw = warp - 6;
      if (lane == 0) {
        // Tiles whose epilogue is complete are published in batches: one fence covers every tile of this warp that
        // is ready at that moment, so the publication rate does not depend on how long a fence takes under load.
        constexpr int kMaxPend = 4;
        uint32_t* pend[kMaxPend];
        unsigned long long pend_rec[kMaxPend];
        int npend = 0;
        auto flush = [&]() {
          if (npend == 0) return;
          // The fence is the release (and the acquire of what the epilogue warps published through epi_done); the
          // reductions after it need no ordering of their own.
          ptx::fence_acq_rel_sys();
          for (int j = 0; j < npend; ++j) ptx::red_relaxed_sys_add(pend[j], 1u);
          if (a.order != nullptr) {
            const unsigned long long now = ptx::globaltimer_ns();
            for (int j = 0; j < npend; ++j) {
              unsigned long long* rec = a.order + 2 * (pend_rec[j] >> 32);
              rec[0] = now;
              rec[1] = (static_cast<unsigned long long>(pair) << 32) | (pend_rec[j] & 0xffffffffull);
            }
          }
          npend = 0;
        };
        uint32_t idx = 0;
        ItemIter iter(sc, pair);
        Item it;
        bool ok = true;
        for (; iter.next(sc, pair, it); ++idx) {
          if (int(idx % uint32_t(kSignalWarps)) != sw) continue;
          const uint32_t expected = 4u * (idx / 4u + 1u);
          volatile uint32_t* cnt = &ctl->epi_done[idx & 3];
          uint32_t polls = 0;
          while (*cnt < expected) {
            if (*abort || ++polls > (1u << 26)) {
              ok = false;
              break;
            }
            __nanosleep(40);
          }
          if (!ok) {
            *abort = 1;
            break;
          }
          int m_blk, n_blk;
          sc.coord(it.seq, m_blk, n_blk);
          int owner = -1, cidx = 0;
          if constexpr (MODE == kGemmAr) {
            const int u = 2 * it.seq + int(cta);
            owner = u % ctx.world;
            cidx = a.counter_base + u / ctx.world;
          } else {
            const int m0 = m_blk * kPairTileM + int(cta) * kTileM;
            if (m0 < a.M) {  // a second half past the last row is waited for by nobody
              const int rows_per_rank = a.M / ctx.world;
              owner = m0 / rows_per_rank;
              cidx = a.counter_base + (m0 - owner * rows_per_rank) / kTileM;
            }
          }
          if (owner >= 0) {
            pend[npend] = counter_ptr(ctx, owner, cidx);
            pend_rec[npend] = (static_cast<unsigned long long>(2 * size_t(it.seq) + cta) << 32) | idx;
            ++npend;
          }
          // This warp's next tile: if it is complete already, it shares the fence.
          const uint32_t nxt = idx + uint32_t(kSignalWarps);
          const bool next_ready = ctl_epi_done_ge(ctl, nxt);
          if (npend == kMaxPend || !next_ready) flush();
        }
        if (ok) flush();
      }
    }
  }

  // ---- teardown --------------------------------------------------------------------------------------------------
  __syncthreads();
  if (a.trace) trace_put(a, kTraceGemmDone, ptx::globaltimer_ns());
  const bool aborted = *abort != 0;
  if (aborted) {
    if (threadIdx.x == 0) {
      gemm_report(ctx.status, ctx.rank, kDevTimeoutMbarrier, 90 + int(cta));
      // Copies that may still be in flight get time to land before shared memory is released.
      const uint64_t t0 = ptx::globaltimer_ns();
      while (ptx::globaltimer_ns() - t0 < 200000) __nanosleep(1000);
    }
    __syncthreads();
  }
  if constexpr (MODE == kGemmAg) {
    if (threadIdx.x == 0 && !aborted) ag_rearm_flags(ctx, a, int(gridDim.x));
  }
  ptx::tc_fence_before_sync();
  cluster_sync_all();  // the peer has no MMA, commit or remote arrival left that targets this CTA
  ptx::tc_fence_after_sync();
  if (warp == 1) tmem_dealloc_pair(tmem_base, kTmemCols);
  // GEMM CTAs that are out of tiles help with the reduction of what is still in flight.
  if constexpr (kSignals) {
    if (!aborted && !a.no_join) {
      __syncthreads();
      const int drawers = int(gridDim.x) * (THREADS / 32);
      if constexpr (MODE == kGemmAr) pair_ar_reducer<T, THREADS>(ctx, a, sc, drawers, false);
      if constexpr (MODE == kGemmRsNorm) pair_rs_reducer<T, THREADS>(ctx, a, sc, drawers, false);
      return;
    }
  }
  if (a.trace) trace_put(a, kTraceEnd, ptx::globaltimer_ns());
}

// ---- host side ---------------------------------------------------------------------------------------------------

// Number of CTA pairs that can be resident at once (0 when the device cannot run the kernel).
template <typename T, int MODE, bool SK>
static int pair_capacity(int dev) {
  static int cached[64];
  static bool have[64];
  static std::mutex mu;
  std::lock_guard<std::mutex> g(mu);
  if (have[dev & 63]) return cached[dev & 63];
  auto kernel = gemm_pair_kernel<T, MODE, SK>;
  int clusters = 0;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytesP) == cudaSuccess) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * 74);
    cfg.blockDim = dim3(MODE == kGemmPlain ? kThreadsPlainP : kThreadsFusedP);
    cfg.dynamicSmemBytes = kSmemBytesP;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess) {
      cudaGetLastError();
      clusters = 0;
    }
  } else {
    cudaGetLastError();
  }
  cached[dev & 63] = clusters;
  have[dev & 63] = true;
  return clusters;
}

// Library-owned stream-K workspace, one per device: a fixed size (it depends on the pair count only), allocated on
// first use and never freed or moved, so that launches captured in a CUDA graph stay valid.
static void* g_sk_ws[64];
static std::mutex g_sk_mu;

cudaError_t pair_streamk_workspace(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  std::lock_guard<std::mutex> g(g_sk_mu);
  void*& ws = g_sk_ws[dev & 63];
  if (ws == nullptr) {
    void* p = nullptr;
    e = cudaMalloc(&p, kSkWorkspaceBytes);
    if (e != cudaSuccess) return e;
    e = cudaMemset(p, 0, kSkFlagBytes);
    if (e != cudaSuccess) {
      cudaFree(p);
      return e;
    }
    ws = p;
  }
  *out = ws;
  return cudaSuccess;
}

template <typename T, int MODE>
static cudaError_t launch_pair_mode(const CommCtx& ctx, const GemmArgs& a, cudaStream_t stream, TmapFn make_tmap,
                                    CUtensorMap* emu_table_dev) {
  int dev = 0;
  cudaGetDevice(&dev);
  const int capacity = pair_capacity<T, MODE, false>(dev);
  if (capacity <= 0) return cudaErrorNotSupported;
  const bool emu = ctx.emu_table != nullptr;
  const int world = ctx.world;
  int budget = capacity;  // clusters of this launch
  if (a.max_ctas > 0 && budget > a.max_ctas / 2) budget = a.max_ctas / 2;
  if (emu) budget = budget / world;
  int comm = 0;
  if (MODE != kGemmPlain) {
    comm = ((a.comm_ctas > 0 ? a.comm_ctas : 16) + 1) / 2;  // clusters
    if (comm > budget / 2) comm = budget / 2;
    if (comm < 1) return cudaErrorInvalidValue;
    if (2 * comm > kMaxCommBlocks) comm = kMaxCommBlocks / 2;  // rank-barrier slots
  }
  const int tiles = ((a.M + kPairTileM - 1) / kPairTileM) * ((a.N + kTileN - 1) / kTileN);
  const int num_kb = (a.K + kTileK - 1) / kTileK;
  PairPlan plan{};
  plan.gemm_pairs = budget - comm;
  if (plan.gemm_pairs < 1) return cudaErrorInvalidValue;
  if ((MODE == kGemmPlain || MODE == kGemmAg) && !emu && plan.gemm_pairs <= kSkMaxPairs) {
    // Less than a wave of tiles also profits: the tail then is the whole problem, cut over all pairs.
    const long long operand_bytes = (static_cast<long long>(a.M) + a.N) * a.K * 2;
    const int sk = a.stream_k == 0 ? pair_streamk_auto(tiles, plan.gemm_pairs, num_kb, operand_bytes) : (a.stream_k > 0 ? 1 : 0);
    if (sk) pair_streamk_plan(tiles, plan.gemm_pairs, num_kb, &plan.sk_tiles, &plan.sk_pairs);
    if (plan.sk_tiles > 0) {
      cudaError_t e = pair_streamk_workspace(&plan.sk_ws);
      if (e != cudaSuccess) return e;
    }
  }
  if (plan.sk_tiles == 0 && plan.gemm_pairs > tiles) plan.gemm_pairs = tiles;

  const int shard_rows = a.M / world;
  CUtensorMap ta, tb, tal;
  EmuMaps em{nullptr};
  if (!emu) {
    const void* a_ptr = MODE == kGemmAg ? a.a_full.p[ctx.rank] : a.A;
    const uint64_t a_ld = MODE == kGemmAg ? uint64_t(a.K) : uint64_t(a.lda);
    if (!make_tmap(&ta, a_ptr, a.M, a.K, a_ld, kTileM)) return cudaErrorInvalidValue;
    if (!make_tmap(&tb, a.B, a.N, a.K, a.ldb, kTileN / 2)) return cudaErrorInvalidValue;
    if (MODE == kGemmAg) {
      if (!make_tmap(&tal, a.A, shard_rows, a.K, a.lda, kTileM)) return cudaErrorInvalidValue;
    } else {
      tal = ta;
    }
  } else {
    if (emu_table_dev == nullptr) return cudaErrorInvalidValue;
    CUtensorMap host[3 * kMaxRanks];
    for (int r = 0; r < world; ++r) {
      const char* A_r = static_cast<const char*>(a.A) + a.a_emu_stride * r;
      const char* B_r = static_cast<const char*>(a.B) + a.b_emu_stride * r;
      const void* a_ptr = MODE == kGemmAg ? a.a_full.p[r] : static_cast<const void*>(A_r);
      const uint64_t a_ld = MODE == kGemmAg ? uint64_t(a.K) : uint64_t(a.lda);
      if (!make_tmap(&host[3 * r + 0], a_ptr, a.M, a.K, a_ld, kTileM)) return cudaErrorInvalidValue;
      if (!make_tmap(&host[3 * r + 1], B_r, a.N, a.K, a.ldb, kTileN / 2)) return cudaErrorInvalidValue;
      if (MODE == kGemmAg) {
        if (!make_tmap(&host[3 * r + 2], A_r, shard_rows, a.K, a.lda, kTileM)) return cudaErrorInvalidValue;
      } else {
        host[3 * r + 2] = host[3 * r + 0];
      }
    }
    // Synchronous on purpose: the emulation path is a test harness.
    cudaError_t e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return e;
    e = cudaMemcpy(emu_table_dev, host, sizeof(CUtensorMap) * 3 * world, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return e;
    em.table = emu_table_dev;
    ta = tb = tal = host[0];
  }

  constexpr bool kCanSk = MODE == kGemmPlain || MODE == kGemmAg;
  constexpr int THREADS = MODE == kGemmPlain ? kThreadsPlainP : kThreadsFusedP;
  if constexpr (kCanSk) {
    if (plan.sk_tiles > 0 && pair_capacity<T, MODE, true>(dev) < budget) return cudaErrorNotSupported;
  }
  const int grid_x = 2 * (plan.gemm_pairs + comm);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid_x, emu ? world : 1);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = kSmemBytesP;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  // Emulated ranks wait on one another inside one launch: all blocks must be resident, which a cooperative launch
  // guarantees (or refuses).
  cfg.numAttrs = emu ? 1 : 0;
  if constexpr (kCanSk) {
    if (plan.sk_tiles > 0) return cudaLaunchKernelEx(&cfg, gemm_pair_kernel<T, MODE, true>, ta, tb, tal, em, ctx, a, plan);
  }
  return cudaLaunchKernelEx(&cfg, gemm_pair_kernel<T, MODE, false>, ta, tb, tal, em, ctx, a, plan);
}

}  // namespace gemm_pair

int pair_streamk_auto(int tiles, int pairs, int num_kb, long long operand_bytes) {
  if (pairs < 2 || tiles % pairs == 0 || num_kb < 16) return 0;
  const int waves = tiles / pairs, rem = tiles % pairs;
  // Fraction of the run that the idle pairs of the last wave would waste.
  const double wasted = (1.0 - double(rem) / pairs) / (waves + 1);
  if (wasted <= 0.03) return 0;
  // Whole tiles of a wave walk K in lockstep, so pairs that share an A or B block find it in L2; the ranges of a tail
  // start at different K offsets and lose that reuse.  Measured on B200 (126 MB of L2): with A and B resident in L2 the
  // tail gives its full gain (4096 x 3584 x 8192: 226 -> 189 us); with 168 MB of operands and at least one whole wave a
  // small one (2048 x 8192 x 8192: 185 -> 177 us); with less than a wave of tiles and operands beyond L2 it loses
  // (512 x 8192 x 8192: 61 -> 72 us), and forced on 8192^3 it loses 17 %.
  const long long kL2Resident = 112ll << 20, kL2Streaming = 192ll << 20;
  if (operand_bytes <= kL2Resident) return 1;
  return (waves >= 1 && operand_bytes <= kL2Streaming) ? 1 : 0;
}

void pair_streamk_plan(int tiles, int pairs, int num_kb, int* sk_tiles, int* sk_pairs) {
  *sk_tiles = 0;
  *sk_pairs = 0;
  if (pairs < 2 || tiles % pairs == 0) return;
  const int waves = tiles / pairs, rem = tiles % pairs;
  int t = rem + (waves >= 1 ? pairs : 0);
  if (t > gemm_pair::kSkMaxTiles) return;
  // Ranges of at least eight K blocks: below that the fixed cost of a part (its own pipeline fill, a 256 KiB
  // round trip through the workspace) outweighs what it computes.
  long long units = static_cast<long long>(t) * num_kb;
  int p = pairs;
  if (units / 8 < p) p = static_cast<int>(units / 8);
  if (p < 2) return;
  *sk_tiles = t;
  *sk_pairs = p;
}

bool gemm_pair_supported(const CommCtx& ctx, const GemmArgs& a) {
  if (a.mode == kGemmPlain) return true;
  if (a.mode == kGemmAr) return a.N % 8 == 0;
  const int rows_per_rank = a.M / ctx.world;
  if (a.M % ctx.world != 0 || rows_per_rank % kTileM != 0) return false;
  if (a.mode == kGemmRsNorm) return a.N % 8 == 0;
  return true;
}

cudaError_t launch_gemm_pair(const CommCtx& ctx, const GemmArgs& a, cudaStream_t stream, gemm_detail::TmapFn make_tmap,
                             CUtensorMap* emu_table_dev) {
  using namespace gemm_pair;
#define OOB_PAIR_CASE(MODE)                                                                          \
  case MODE:                                                                                         \
    return a.fmt == 1 ? launch_pair_mode<__nv_bfloat16, MODE>(ctx, a, stream, make_tmap, emu_table_dev) \
                      : launch_pair_mode<__half, MODE>(ctx, a, stream, make_tmap, emu_table_dev);
  switch (a.mode) {
    OOB_PAIR_CASE(kGemmPlain)
    OOB_PAIR_CASE(kGemmAr)
    OOB_PAIR_CASE(kGemmRsNorm)
    OOB_PAIR_CASE(kGemmAg)
  }
#undef OOB_PAIR_CASE
  return cudaErrorInvalidValue;
}

int pair_schedule_dump(int mode, int M, int N, int K, int pairs, int stream_k, int world, int rank, int* out, int cap) {
  using namespace gemm_pair;
  PairSched sc{};
  sc.num_kb = (K + kTileK - 1) / kTileK;
  sc.tiles_m = (M + 2 * kTileM - 1) / (2 * kTileM);
  sc.tiles_n = (N + kTileN - 1) / kTileN;
  sc.tiles = sc.tiles_m * sc.tiles_n;
  const int sk = stream_k == 0 ? pair_streamk_auto(sc.tiles, pairs, sc.num_kb, (static_cast<long long>(M) + N) * K * 2)
                               : (stream_k > 0 ? 1 : 0);
  if (sk && pairs <= kSkMaxPairs) pair_streamk_plan(sc.tiles, pairs, sc.num_kb, &sc.sk_tiles, &sc.sk_pairs);
  if (sc.sk_tiles == 0 && pairs > sc.tiles) pairs = sc.tiles;
  sc.P = pairs;
  sc.sk_units = sc.sk_tiles * sc.num_kb;
  sc.dp_tiles = sc.tiles - sc.sk_tiles;
  sc.mode = mode;
  sc.world = world;
  sc.rank = rank;
  if ((mode == kGemmRsNorm || mode == kGemmAg) && world > 0 && M % world == 0 && (M / world) % (2 * kTileM) == 0)
    sc.bpr = M / world / (2 * kTileM);
  int n = 0;
  for (int p = 0; p < pairs; ++p) {
    ItemIter iter(sc, p);
    Item it;
    while (iter.next(sc, p, it)) {
      if ((n + 1) * 9 > cap) return -1;
      int m_blk, n_blk;
      sc.coord(it.seq, m_blk, n_blk);
      int slot = -1, parts = 1, first = -1;
      if (it.partial) {
        slot = it.kb0 == 0 ? -2 : p;  // -2: the part that starts the tile (its pair owns the tile and parks nothing)
        first = sc.sk_owner(it.sk_tile * sc.num_kb);
        parts = sc.sk_owner(it.sk_tile * sc.num_kb + sc.num_kb - 1) - first + 1;
      }
      int* o = out + n * 9;
      o[0] = p; o[1] = it.seq; o[2] = m_blk; o[3] = n_blk; o[4] = it.kb0; o[5] = it.kb1; o[6] = slot; o[7] = parts; o[8] = first;
      ++n;
    }
  }
  return n;
}

cudaError_t gemm_pair_reserve_workspace() {
  void* p = nullptr;
  return gemm_pair::pair_streamk_workspace(&p);
}

}  // namespace oob
