// tcgen05 / TMEM GEMM for sm_100a with communication fused into the same
// persistent kernel (device code and the launch helper; included by the
// translation units that instantiate it).
//
// Mainloop (all modes): one CTA per SM, 128x256 output tiles, K blocks of 64.
//   warp 0    TMA producer: cp.async.bulk.tensor (this GPU's memory, 128-byte swizzle) into a 4-stage ring
//   warp 1    MMA issuer: one thread issues tcgen05.mma (M128 N256 K16, fp32 accumulate in TMEM);
//             tcgen05.commit releases the smem stage / publishes the accumulator
//   warps 2-5 epilogue: tcgen05.ld the accumulator (two TMEM stages, so the next tile's mainloop overlaps),
//             convert, store
// Plain mode can split K over several CTAs per tile (small-M problems that would otherwise occupy a fraction of
// the SMs): partial accumulators go to an fp32 workspace and the last CTA to arrive for a 32-row quadrant of a tile
// sums the splits in a fixed order and writes C.
// Fused modes add a communication role.  `comm_ctas` CTAs run it from the start and every GEMM CTA joins when it
// has finished its tiles, drawing work from a ticket counter:
//   GEMM->AR      every tile has an owner rank.  The epilogue stages its 32-row strips in shared memory and PUSHES
//                 them into the owner's registered buffer with bulk tensor stores (cp.async.bulk.tensor, smem ->
//                 peer global memory); a signal warp waits for those stores, orders them system-wide and bumps the
//                 tile's arrival counter on the owner, so the epilogue warps never stall on NVLink.  The owner sums
//                 the `world` slices from its LOCAL memory (fp32, rank order) and broadcasts the result into every
//                 rank's C (multimem.st through the switch, or peer stores) while later tiles still compute.
//                 use_nvls == 2 selects the pull variant: tiles stay in the producer's buffer and the owner reads
//                 their in-switch sum with multimem.ld_reduce.
//   GEMM->RS+norm same push, counters per 128-row block on the rank that owns the rows; reducers sum the rows, add
//                 the residual, apply RMSNorm and write the rank's rows.
//   AG->GEMM      pusher CTAs broadcast this rank's A shard chunk by chunk into every rank's gathered buffer and bump
//                 per-chunk flags; the TMA producer waits for the flag of the chunk it is about to load from LOCAL
//                 memory.
// Cross-GPU traffic is ld/st/red, multimem.* and bulk tensor STORES into peer memory.  TMA LOADS only ever read
// this GPU's own memory, and nothing here uses cluster multicast.
//
// Capability parity with the reference: signalling GEMM + reorder epilogue + wait kernel + per-segment all-reduce
// (src/gemm/gemm_with_signal_sm90.h:102-513, src/epilogue/reorder_epilogue.h:324-595, src/wait.cuh:5-9,
// src/overlap_impl.cu:450-706), row remap for reduce-scatter (src/gemm/scatter_row_remap_sm90.cuh:35-82), the plain
// GEMM (src/gemm/gemm_plain_sm90.cu) and its stream-K instances (src/gemm/gemm_with_signal_sm90.h:238-292).  The
// reorder tables / segment search are replaced by a deterministic tile order plus arrival counters; accumulation is
// fp32 (the reference accumulates in fp16, src/gemm/gemm_signal_sm90.cu:108).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include "../device/reduce.cuh"
#include "../device/sync.cuh"
#include "gemm.h"

namespace oob {

// Encodes a 2-D tensor map over a row-major [rows, cols] 16-bit matrix with leading dimension ld (elements):
// box = box_rows x 64 elements, 128-byte swizzle.  Pure host computation through the driver; false on failure.
bool encode_tmap_2d(CUtensorMap* out, const void* p, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows);

namespace gemm_detail {

constexpr int kStages = 4;
constexpr int kABytes = kTileM * kTileK * 2;  // 16 KiB
constexpr int kBBytes = kTileN * kTileK * 2;  // 32 KiB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kAccStages = 2;
constexpr int kTmemCols = 512;
constexpr int kEpiWarpBytes = 32 * 256;  // epilogue staging per warp: 32 rows x 128 16-bit columns
constexpr int kEpiBytes = 4 * kEpiWarpBytes;
constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr int kThreadsPlain = 192;
constexpr int kThreadsFused = 384;
constexpr int kPacksPerTile = kTileBytes / 16;  // 4096
constexpr int kPacksPerTileRow = kTileN / 8;    // 32
constexpr int kRsRowsPerItem = 8;               // GEMM->RS: rows of a 128-row block handled per ticket
constexpr int kRsItemsPerBlock = kTileM / kRsRowsPerItem;

// Split-K workspace layout: kSplitkCounterBytes of arrival counters (one per 32-row tile quadrant, zero between
// calls), then the fp32 partial tiles [tile][split][128][256].
constexpr size_t kSplitkMaxTiles = 16384;
constexpr size_t kSplitkCounterBytes = kSplitkMaxTiles * 4 * sizeof(uint32_t);
__host__ __device__ __forceinline__ float* splitk_partials(void* ws) {
  return reinterpret_cast<float*>(static_cast<char*>(ws) + kSplitkCounterBytes);
}

struct SmemCtl {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tmem_full[kAccStages];
  uint64_t tmem_empty[kAccStages];
  uint32_t tmem_base;
  int abort;
  uint32_t epi_count[8];  // epilogue warps that have issued their rows of a tile (slot = tile iteration & 7; never reset)
};

struct Sched {
  int tiles_m, tiles_n, tiles;
  int splits, items;  // items = tiles * splits (split-K: plain mode only)
  int kb_per_split;
  int mode, world, rank;
  int bps;  // 128-row blocks per rank shard (RS / AG)
  // Logical tile (m_blk, n_blk) of schedule position `seq`.  Every rank walks
  // the same sequence so that arrival counters fill at about the same time.
  __device__ void coord(int seq, int& m_blk, int& n_blk) const {
    if (mode == kGemmRsNorm) {
      // Row-block major; consecutive row blocks belong to consecutive owners.
      const int i = seq / tiles_n;
      n_blk = seq % tiles_n;
      m_blk = (i % world) * bps + i / world;
    } else if (mode == kGemmAg) {
      // Own shard first (it is local), then chunk c of every other rank in ring order.
      const int i = seq / tiles_n;
      n_blk = seq % tiles_n;
      if (i < bps) {
        m_blk = rank * bps + i;
      } else {
        const int k = i - bps;
        const int c = k / (world - 1);
        const int s = (rank + 1 + k % (world - 1)) % world;
        m_blk = s * bps + c;
      }
    } else {
      // Grouped raster: 16 tile rows at a time so that concurrently running
      // CTAs share A and B tiles in L2.
      constexpr int kGroup = 16;
      const int per_group = kGroup * tiles_n;
      const int g = seq / per_group;
      const int first_m = g * kGroup;
      const int rows = (tiles_m - first_m) < kGroup ? (tiles_m - first_m) : kGroup;
      const int in = seq - g * per_group;
      m_blk = first_m + in % rows;
      n_blk = in / rows;
    }
  }
};

__device__ __forceinline__ void gemm_report(DeviceStatus* s, int rank, int code, int where) {
  if (s == nullptr) return;
  if (atomicCAS(&s->code, 0, code) == 0) {
    s->rank = rank;
    s->peer = -1;
    s->block = static_cast<int>(blockIdx.x);
    s->where = where;
    __threadfence_system();
  }
}

template <typename T>
__device__ __forceinline__ void cvt_store_32(char* dst, const uint32_t (&r)[32], bool full_vec, int valid_cols) {
  // r holds 32 consecutive fp32 columns of one row.
  uint32_t packed[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float a = __uint_as_float(r[2 * i]), b = __uint_as_float(r[2 * i + 1]);
    if constexpr (PackTraits<T>::kDType == kBF16) {
      __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
      packed[i] = *reinterpret_cast<uint32_t*>(&h);
    } else {
      __half2 h = __floats2half2_rn(a, b);
      packed[i] = *reinterpret_cast<uint32_t*>(&h);
    }
  }
  if (full_vec) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      *reinterpret_cast<uint4*>(dst + i * 16) =
          make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
  } else {
    for (int i = 0; i < valid_cols; ++i) {
      const uint32_t w = packed[i >> 1];
      *reinterpret_cast<unsigned short*>(dst + i * 2) = static_cast<unsigned short>((i & 1) ? (w >> 16) : (w & 0xffff));
    }
  }
}

template <int THREADS>
__device__ __forceinline__ float cta_sum(float v, float* s_part, float* s_total) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < THREADS / 32 ? s_part[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (threadIdx.x == 0) *s_total = t;
  }
  __syncthreads();
  return *s_total;
}

// Device-side trace (GemmArgs::trace): thread 0 of each CTA records globaltimer stamps and counts.
__device__ __forceinline__ void trace_put(const GemmArgs& a, int slot, unsigned long long v) {
  if (a.trace != nullptr && threadIdx.x == 0)
    a.trace[(size_t(blockIdx.y) * gridDim.x + blockIdx.x) * kTraceWords + slot] = v;
}

// Draws the next ticket of this launch.  The counter is re-armed by whoever draws the last ticket that can ever
// be drawn: `total` in-range tickets plus one out-of-range ticket per CTA of the launch.
__device__ __forceinline__ int draw_ticket(uint32_t* ticket, int total, int* s_slot, int drawers) {
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t t = atomicAdd(ticket, 1u);
    if (t == uint32_t(total + drawers - 1)) {
      *ticket = 0;
      __threadfence();
    }
    *s_slot = static_cast<int>(t);
  }
  __syncthreads();
  return *s_slot;
}

// The partial products of all ranks for one tile sit side by side in the OWNER's memory (every rank's epilogue
// pushed its slice there), kTileBytes apart.  Slices<> holds the raw 16-byte pack of every slice: all loads are
// issued back to back, with no arithmetic in between, so that many local loads are in flight per thread.
template <typename T, int NR>
struct Slices {
  static constexpr int kSlots = NR > 0 ? NR : 1;
  uint4 v[kSlots];
  float generic_[NR == 0 ? 8 : 1];
  __device__ __forceinline__ void load(const char* base, int world) {
    if constexpr (NR > 0) {
#pragma unroll
      for (int r = 0; r < NR; ++r) v[r] = ptx::ld_nc_v4(base + size_t(r) * kTileBytes);
    } else {
      // Generic world size: summed right away (fallback path).
      using PT = PackTraits<T>;
      float acc[8];
      PT::unpack(ptx::ld_nc_v4(base), acc);
      for (int r = 1; r < world; ++r) {
        float f[8];
        PT::unpack(ptx::ld_nc_v4(base + size_t(r) * kTileBytes), f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += f[i];
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) generic_[i] = acc[i];
    }
  }
  __device__ __forceinline__ void sum(float (&acc)[8]) const {
    using PT = PackTraits<T>;
    if constexpr (NR > 0) {
      PT::unpack(v[0], acc);
#pragma unroll
      for (int r = 1; r < NR; ++r) {
        float f[8];
        PT::unpack(v[r], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += f[i];
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = generic_[i];
    }
  }
};

// Packs per thread and batch for the reducer loops: bounded by registers (NR raw packs each).
template <int NR>
constexpr int kReduceBatch = NR == 0 ? 1 : (NR >= 8 ? 3 : (NR == 4 ? 6 : 8));

// All-reduce of one 128x256 tile: sum the `world` local slices (fp32, rank order) and push the result into every
// rank's C, through the switch (multimem.st) or with peer stores.
template <typename T, int THREADS, int NR, bool MC>
__device__ __forceinline__ void ar_reduce_tile(const GemmArgs& a, int world, int rank, const char* slices,
                                               size_t c_off0, size_t row_bytes, int rows_valid, int packs_valid_row) {
  constexpr int U = kReduceBatch<NR>;
  for (int base = 0; base < kPacksPerTile; base += THREADS * U) {
    Slices<T, NR> raw[U];
    bool live[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int p = base + u * THREADS + threadIdx.x;
      const int row = p / kPacksPerTileRow, cp = p % kPacksPerTileRow;
      live[u] = p < kPacksPerTile && row < rows_valid && cp < packs_valid_row;
      // Dead lanes load pack 0 of the tile (always mapped) instead of branching around the load.
      raw[u].load(slices + size_t(live[u] ? p : 0) * 16, world);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (!live[u]) continue;
      const int p = base + u * THREADS + threadIdx.x;
      const int row = p / kPacksPerTileRow, cp = p % kPacksPerTileRow;
      float acc[8];
      raw[u].sum(acc);
      const uint4 v = PackTraits<T>::pack(acc);
      const size_t coff = c_off0 + size_t(row) * row_bytes + size_t(cp) * 16;
      if constexpr (MC) {
        ptx::multimem_st_v4(static_cast<char*>(a.c_sym.mc) + coff, v);
      } else if constexpr (NR > 0) {
#pragma unroll
        for (int r = 0; r < NR; ++r) ptx::st_v4(static_cast<char*>(a.c_sym.p[(rank + r) % NR]) + coff, v);
      } else {
        for (int r = 0; r < world; ++r) ptx::st_v4(static_cast<char*>(a.c_sym.p[(rank + r) % world]) + coff, v);
      }
    }
  }
}

// Pull variant (use_nvls == 2): every rank keeps its partial tile in its OWN buffer at the same offset; the owner
// reads the sum of all ranks with one in-switch multimem.ld_reduce per pack and broadcasts it with multimem.st.
// Per direction this moves the message once (the push variants move it 1.75 times).
template <typename T, int THREADS>
__device__ __forceinline__ void ar_reduce_tile_pull(const GemmArgs& a, size_t tile_off, size_t c_off0, size_t row_bytes,
                                                    int rows_valid, int packs_valid_row) {
  constexpr int U = (kPacksPerTile + THREADS - 1) / THREADS;  // the whole tile in one batch of loads
  uint4 v[U];
  bool live[U];
  const char* src = static_cast<const char*>(a.partial.mc) + tile_off;
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const int p = u * THREADS + threadIdx.x;
    const int row = p / kPacksPerTileRow, cp = p % kPacksPerTileRow;
    live[u] = p < kPacksPerTile && row < rows_valid && cp < packs_valid_row;
    v[u] = reduce_pack_mc<T, kSum>(src + size_t(live[u] ? p : 0) * 16);
  }
#pragma unroll
  for (int u = 0; u < U; ++u) {
    if (!live[u]) continue;
    const int p = u * THREADS + threadIdx.x;
    const int row = p / kPacksPerTileRow, cp = p % kPacksPerTileRow;
    ptx::multimem_st_v4(static_cast<char*>(a.c_sym.mc) + c_off0 + size_t(row) * row_bytes + size_t(cp) * 16, v[u]);
  }
}

template <typename T, int THREADS, bool MC>
__device__ __forceinline__ void ar_reduce_tile_dispatch(const GemmArgs& a, int world, int rank, const char* slices,
                                                        size_t c_off0, size_t row_bytes, int rows_valid,
                                                        int packs_valid_row) {
  if (world == 2)
    ar_reduce_tile<T, THREADS, 2, MC>(a, world, rank, slices, c_off0, row_bytes, rows_valid, packs_valid_row);
  else if (world == 4)
    ar_reduce_tile<T, THREADS, 4, MC>(a, world, rank, slices, c_off0, row_bytes, rows_valid, packs_valid_row);
  else if (world == 8)
    ar_reduce_tile<T, THREADS, 8, MC>(a, world, rank, slices, c_off0, row_bytes, rows_valid, packs_valid_row);
  else
    ar_reduce_tile<T, THREADS, 0, MC>(a, world, rank, slices, c_off0, row_bytes, rows_valid, packs_valid_row);
}

// ---------------------------------------------------------------------------
// Communication roles
// ---------------------------------------------------------------------------

// GEMM->AR: owned tiles are those at schedule positions seq with seq % world == rank; ticket k is the k-th of them.
// Staging layout in the owner's partial buffer: [k][source rank][128][256].
// Counter layout from counter_base: [owned] arrivals per owned tile, then the ticket counter.
template <typename T, int THREADS>
__device__ void ar_reducer_role(const CommCtx& ctx, const GemmArgs& a, const Sched& sc, int drawers) {
  __shared__ int s_ok;
  __shared__ int s_ticket;
  const int world = ctx.world, rank = ctx.rank;
  const bool use_mc = a.c_sym.mc != nullptr && a.use_nvls != 0;  // broadcast of the result through the switch
  const size_t row_bytes = size_t(a.N) * 2;
  const char* staged = static_cast<const char*>(a.partial.p[rank]);
  const int owned = (sc.tiles - rank + world - 1) / world;  // tickets that map to a tile
  const int owned_max = (sc.tiles + world - 1) / world;
  uint32_t* ticket = counter_ptr(ctx, rank, a.counter_base + owned_max);
  bool ok = true;
  unsigned long long t_wait = 0, n_items = 0;
  while (true) {
    const int k = draw_ticket(ticket, owned, &s_ticket, drawers);
    if (k >= owned) break;
    const int seq = k * world + rank;
    if (threadIdx.x == 0) {
      uint32_t* cnt = counter_ptr(ctx, rank, a.counter_base + k);
      const unsigned long long tw = a.trace ? ptx::globaltimer_ns() : 0;
      s_ok = wait_word_ge(ctx, cnt, world, kDevTimeoutCounter, -1, 50) ? 1 : 0;
      *cnt = 0;  // single consumer: re-arm now (next call's arrivals cannot come before this launch ends everywhere)
      if (a.trace) {
        const unsigned long long now = ptx::globaltimer_ns();
        t_wait += now - tw;
        if (n_items == 0) trace_put(a, kTraceFirstReady, now);
        ++n_items;
      }
    }
    __syncthreads();
    if (s_ok == 0) ok = false;
    if (!ok) continue;  // keep drawing so that the ticket counter still gets re-armed
    int m_blk, n_blk;
    sc.coord(seq, m_blk, n_blk);
    const char* slices = staged + size_t(k) * world * kTileBytes;  // [world][128][256] pushed by the epilogues
    const int rows_valid = min(kTileM, a.M - m_blk * kTileM);
    const int packs_valid_row = min(kPacksPerTileRow, (a.N - n_blk * kTileN) / 8);
    const size_t c_off0 = size_t(m_blk * kTileM) * row_bytes + size_t(n_blk * kTileN) * 2;
    if (a.use_nvls == 2 && a.partial.mc != nullptr && use_mc)
      ar_reduce_tile_pull<T, THREADS>(a, size_t(m_blk * sc.tiles_n + n_blk) * kTileBytes, c_off0, row_bytes, rows_valid,
                                      packs_valid_row);
    else if (use_mc)
      ar_reduce_tile_dispatch<T, THREADS, true>(a, world, rank, slices, c_off0, row_bytes, rows_valid, packs_valid_row);
    else
      ar_reduce_tile_dispatch<T, THREADS, false>(a, world, rank, slices, c_off0, row_bytes, rows_valid, packs_valid_row);
  }
  if (a.trace) {
    trace_put(a, kTraceCommDone, ptx::globaltimer_ns());
    trace_put(a, kTraceItems, n_items);
    trace_put(a, kTraceWaitNs, t_wait);
  }
  // Block b of every rank is past its last tile: together (all blocks) this means every push into this rank's C
  // has been issued and released, and nobody reads this rank's partial buffer any more.
  if (ok) rank_barrier(ctx, blockIdx.x, 51);
  if (a.trace) trace_put(a, kTraceEnd, ptx::globaltimer_ns());
}

// One ticket of the GEMM->RS tail: rows [r_begin, r_end) of an owned 128-row block.
struct RsRowCtx {
  const char* row_base0;  // the block's first staged tile: layout [n_blk][source rank][128][256]
  int lrow0;         // rank-local index of the block's first row
  int r_begin, r_end;
  const char* res;
  char* y;
  char* ro;
  const char* wgt;
  float* s_part;
  float* s_total;
};

// PPT = packs per thread and row (N <= PPT * THREADS * 8).  For each row: all raw packs of all ranks are loaded
// first (in batches bounded by registers), then summed, the residual is added, the row's mean square is reduced
// over the CTA, and the normalised row is written.
template <typename T, int THREADS, int NR, int PPT>
__device__ __forceinline__ void rs_process_rows(const GemmArgs& a, int world, const RsRowCtx& rc) {
  using PT = PackTraits<T>;
  constexpr int QB = NR == 0 ? 1 : (NR >= 8 ? (PPT < 3 ? PPT : 3) : PPT);
  const int packs_per_row = a.N / 8;
  const size_t row_bytes = size_t(a.N) * 2;
  for (int r_in = rc.r_begin; r_in < rc.r_end; ++r_in) {
    const size_t lrow_off = size_t(rc.lrow0 + r_in) * row_bytes;
    const char* row_base = rc.row_base0 + size_t(r_in) * (kTileN * 2);
    float v[PPT][8];
#pragma unroll
    for (int q0 = 0; q0 < PPT; q0 += QB) {
      Slices<T, NR> raw[QB];
#pragma unroll
      for (int i = 0; i < QB; ++i) {
        if (q0 + i < PPT) {
          const int p = threadIdx.x + (q0 + i) * THREADS;
          const int pc = p < packs_per_row ? p : 0;  // dead lanes reload pack 0 instead of branching
          raw[i].load(row_base + size_t(pc / kPacksPerTileRow) * world * kTileBytes + size_t(pc % kPacksPerTileRow) * 16,
                      world);
        }
      }
#pragma unroll
      for (int i = 0; i < QB; ++i)
        if (q0 + i < PPT) raw[i].sum(v[q0 + i]);
    }
    float ss = 0.f;
#pragma unroll
    for (int q = 0; q < PPT; ++q) {
      const int p = threadIdx.x + q * THREADS;
      if (p < packs_per_row) {
        if (rc.res != nullptr) {
          const uint4 rv = ptx::ld_nc_v4(rc.res + lrow_off + size_t(p) * 16);
          float rf[8];
          PT::unpack(rv, rf);
#pragma unroll
          for (int i = 0; i < 8; ++i) v[q][i] += rf[i];
          const uint4 rounded = PT::pack(v[q]);
          PT::unpack(rounded, v[q]);
        }
        if (rc.ro != nullptr) ptx::st_v4(rc.ro + lrow_off + size_t(p) * 16, PT::pack(v[q]));
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += v[q][i] * v[q][i];
      }
    }
    float scale = 1.f;
    if (rc.wgt != nullptr) {
      const float total_ss = cta_sum<THREADS>(ss, rc.s_part, rc.s_total);
      scale = rsqrtf(total_ss / float(a.N) + a.eps);
    }
#pragma unroll
    for (int q = 0; q < PPT; ++q) {
      const int p = threadIdx.x + q * THREADS;
      if (p < packs_per_row) {
        float o[8];
        if (rc.wgt != nullptr) {
          const uint4 wv = *reinterpret_cast<const uint4*>(rc.wgt + size_t(p) * 16);
          float wf[8];
          PT::unpack(wv, wf);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = v[q][i] * scale * wf[i];
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = v[q][i];
        }
        ptx::st_v4(rc.y + lrow_off + size_t(p) * 16, PT::pack(o));
      }
    }
  }
}

template <typename T, int THREADS, int PPT>
__device__ __forceinline__ void rs_rows_dispatch(const GemmArgs& a, int world, const RsRowCtx& rc) {
  if (world == 2)
    rs_process_rows<T, THREADS, 2, PPT>(a, world, rc);
  else if (world == 4)
    rs_process_rows<T, THREADS, 4, PPT>(a, world, rc);
  else if (world == 8)
    rs_process_rows<T, THREADS, 8, PPT>(a, world, rc);
  else
    rs_process_rows<T, THREADS, 0, PPT>(a, world, rc);
}

// GEMM->RS + residual + RMSNorm.  Ticket t = (owned row block t / kRsItemsPerBlock, row group t % kRsItemsPerBlock).
// Counter layout from counter_base: [bps] tile arrivals per row block, [bps] finished items per row block, ticket.
// Staging layout in the owner's partial buffer: [owned row block][n_blk][source rank][128][256].
template <typename T, int THREADS>
__device__ void rs_reducer_role(const CommCtx& ctx, const GemmArgs& a, const Sched& sc, int drawers) {
  __shared__ int s_ok;
  __shared__ int s_ticket;
  __shared__ float s_part[THREADS / 32];
  __shared__ float s_total;
  const int world = ctx.world, rank = ctx.rank;
  const char* res = a.residual ? static_cast<const char*>(a.residual) + a.rs_emu_stride * blockIdx.y : nullptr;
  char* y = static_cast<char*>(a.y_local) + a.rs_emu_stride * blockIdx.y;
  char* ro = a.res_out_local ? static_cast<char*>(a.res_out_local) + a.rs_emu_stride * blockIdx.y : nullptr;
  const char* wgt = static_cast<const char*>(a.weight);
  const int total = sc.bps * kRsItemsPerBlock;
  uint32_t* ticket = counter_ptr(ctx, rank, a.counter_base + 2 * sc.bps);
  bool ok = true;
  unsigned long long t_wait = 0, n_items = 0;
  while (true) {
    const int t = draw_ticket(ticket, total, &s_ticket, drawers);
    if (t >= total) break;
    const int lb = t / kRsItemsPerBlock, grp = t % kRsItemsPerBlock;
    uint32_t* cnt = counter_ptr(ctx, rank, a.counter_base + lb);
    uint32_t* done = counter_ptr(ctx, rank, a.counter_base + sc.bps + lb);
    if (threadIdx.x == 0) {
      const unsigned long long tw = a.trace ? ptx::globaltimer_ns() : 0;
      s_ok = wait_word_ge(ctx, cnt, uint32_t(world) * sc.tiles_n, kDevTimeoutCounter, -1, 60) ? 1 : 0;
      if (a.trace) {
        const unsigned long long now = ptx::globaltimer_ns();
        t_wait += now - tw;
        if (n_items == 0) trace_put(a, kTraceFirstReady, now);
        ++n_items;
      }
    }
    __syncthreads();
    if (s_ok == 0) ok = false;
    if (ok) {
      RsRowCtx rc;
      rc.row_base0 = static_cast<const char*>(a.partial.p[rank]) + size_t(lb) * sc.tiles_n * world * kTileBytes;
      rc.lrow0 = lb * kTileM;
      rc.r_begin = grp * kRsRowsPerItem;
      rc.r_end = (grp + 1) * kRsRowsPerItem;
      rc.res = res;
      rc.y = y;
      rc.ro = ro;
      rc.wgt = wgt;
      rc.s_part = s_part;
      rc.s_total = &s_total;
      const int ppt = (a.N / 8 + THREADS - 1) / THREADS;
      if (ppt <= 2)
        rs_rows_dispatch<T, THREADS, 2>(a, world, rc);
      else if (ppt <= 3)
        rs_rows_dispatch<T, THREADS, 3>(a, world, rc);
      else
        rs_rows_dispatch<T, THREADS, 6>(a, world, rc);
    }
    // Whoever finishes the last row group of a block re-arms the block's counters for the next call.
    __syncthreads();
    if (threadIdx.x == 0) {
      if (atomicAdd(done, 1u) == uint32_t(kRsItemsPerBlock - 1)) {
        *cnt = 0;
        *done = 0;
        __threadfence();
      }
    }
  }
  if (a.trace) {
    trace_put(a, kTraceCommDone, ptx::globaltimer_ns());
    trace_put(a, kTraceItems, n_items);
    trace_put(a, kTraceWaitNs, t_wait);
  }
  if (ok) rank_barrier(ctx, blockIdx.x, 61);
  if (a.trace) trace_put(a, kTraceEnd, ptx::globaltimer_ns());
}

// AG->GEMM pusher: broadcasts this rank's shard, one 128-row chunk at a time.
template <int THREADS>
__device__ void ag_pusher_role(const CommCtx& ctx, const GemmArgs& a, const Sched& sc, int j, int R) {
  const int world = ctx.world, rank = ctx.rank;
  const bool use_mc = a.a_full.mc != nullptr && ctx.pad_mc != nullptr && a.use_nvls != 0;
  // Previous call's readers of the gathered buffers are done once every rank has entered this call.
  if (!rank_barrier(ctx, j, 70)) return;
  const char* src = static_cast<const char*>(a.A) + a.a_emu_stride * blockIdx.y;
  const size_t row_bytes = size_t(a.K) * 2;  // gathered buffer is dense [M, K]
  const size_t src_row_bytes = size_t(a.lda) * 2;
  const int packs_per_row = a.K / 8;
  const int shard_rows = a.M / world;
  for (int c = 0; c < sc.bps; ++c) {
    const int row0 = c * kTileM;
    const int rows = min(kTileM, shard_rows - row0);
    const int total = rows * packs_per_row;
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
      const int idx = a.counter_base + rank * sc.bps + c;
      if (use_mc) {
        ptx::multimem_red_add_u32(ctx.pad_mc + kPadCounterOffset + idx, 1u);
      } else {
        for (int r = 1; r < world; ++r) ptx::red_release_sys_add(counter_ptr(ctx, (rank + r) % world, idx), 1u);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------
struct EmuMaps {
  const CUtensorMap* table;  // [world][3]: A, B, A_local per emulated rank (device memory), or nullptr
};

template <typename T, int MODE>
__global__ void __launch_bounds__(MODE == kGemmPlain ? kThreadsPlain : kThreadsFused, 1)
    gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                const __grid_constant__ CUtensorMap tmap_a_local, EmuMaps emu, CommCtx ctx_param, GemmArgs a,
                int gemm_ctas) {
  constexpr int THREADS = MODE == kGemmPlain ? kThreadsPlain : kThreadsFused;
  constexpr int FMT = PackTraits<T>::kDType == kBF16 ? 1 : 0;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  SmemCtl* ctl = reinterpret_cast<SmemCtl*>(smem + kStages * kStageBytes + kEpiBytes);

  const CommCtx ctx = resolve_ctx(ctx_param);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (a.K + kTileK - 1) / kTileK;
  if (a.trace) {
    trace_put(a, kTraceStart, ptx::globaltimer_ns());
    trace_put(a, kTraceRole, static_cast<int>(blockIdx.x) >= gemm_ctas ? 1 : 0);
  }

  Sched sc;
  sc.tiles_m = (a.M + kTileM - 1) / kTileM;
  sc.tiles_n = (a.N + kTileN - 1) / kTileN;
  sc.tiles = sc.tiles_m * sc.tiles_n;
  sc.splits = (MODE == kGemmPlain && a.splits > 1) ? a.splits : 1;
  sc.items = sc.tiles * sc.splits;
  sc.kb_per_split = (num_kb + sc.splits - 1) / sc.splits;
  sc.mode = MODE;
  sc.world = ctx.world;
  sc.rank = ctx.rank;
  sc.bps = (MODE == kGemmRsNorm || MODE == kGemmAg) ? (a.M / ctx.world + kTileM - 1) / kTileM : 0;

  // ---- communication CTAs -------------------------------------------------
  if constexpr (MODE != kGemmPlain) {
    if (static_cast<int>(blockIdx.x) >= gemm_ctas) {
      const int j = blockIdx.x - gemm_ctas, R = gridDim.x - gemm_ctas;
      const int drawers = a.no_join ? R : int(gridDim.x);
      if constexpr (MODE == kGemmAr) ar_reducer_role<T, THREADS>(ctx, a, sc, drawers);
      if constexpr (MODE == kGemmRsNorm) rs_reducer_role<T, THREADS>(ctx, a, sc, drawers);
      if constexpr (MODE == kGemmAg) ag_pusher_role<THREADS>(ctx, a, sc, j, R);
      return;
    }
  }

  // ---- GEMM CTAs ----------------------------------------------------------
  const CUtensorMap* ta = emu.table ? &emu.table[3 * blockIdx.y + 0] : &tmap_a;
  const CUtensorMap* tb = emu.table ? &emu.table[3 * blockIdx.y + 1] : &tmap_b;
  const CUtensorMap* tal = emu.table ? &emu.table[3 * blockIdx.y + 2] : &tmap_a_local;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(&ctl->full[s], 1);
      ptx::mbar_init(&ctl->empty[s], 1);
    }
    for (int s = 0; s < kAccStages; ++s) {
      ptx::mbar_init(&ctl->tmem_full[s], 1);
      ptx::mbar_init(&ctl->tmem_empty[s], 4);  // one arrival per epilogue warp
    }
    for (int s = 0; s < 8; ++s) ctl->epi_count[s] = 0;
    ctl->abort = 0;
    ptx::mbar_fence_init();
    ptx::prefetch_tmap(ta);
    ptx::prefetch_tmap(tb);
    if constexpr (MODE == kGemmAg) ptx::prefetch_tmap(tal);
  }
  if (warp == 1) {
    ptx::tmem_alloc(&ctl->tmem_base, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;
  volatile int* abort = &ctl->abort;
  const int G = gemm_ctas;

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------- TMA producer -------------------------
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < sc.items && ok; item += G) {
        const int seq = item / sc.splits, split = item - seq * sc.splits;
        const int kb0 = split * sc.kb_per_split, kb1 = min(num_kb, kb0 + sc.kb_per_split);
        int m_blk, n_blk;
        sc.coord(seq, m_blk, n_blk);
        const CUtensorMap* tma_a_cur = ta;
        int a_row = m_blk * kTileM;
        if constexpr (MODE == kGemmAg) {
          const int owner = m_blk / sc.bps;
          if (owner == ctx.rank) {
            tma_a_cur = tal;  // own rows are read from the shard itself
            a_row = (m_blk - owner * sc.bps) * kTileM;
          } else {
            // Gathered rows: wait until all pushers of `owner` delivered this chunk into LOCAL memory.
            const int R = gridDim.x - G;
            ok = wait_word_ge(ctx, counter_ptr(ctx, ctx.rank, a.counter_base + m_blk), R, kDevTimeoutChunkFlag, owner,
                              71);
            if (!ok) {
              *abort = 1;
              break;
            }
            ptx::fence_proxy_async_global();
          }
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!ptx::mbar_wait(&ctl->empty[stage], phase ^ 1, abort)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * kStageBytes;
          uint8_t* sb = sa + kABytes;
          ptx::mbar_arrive_expect_tx(&ctl->full[stage], kStageBytes);
          ptx::tma_load_2d(sa, tma_a_cur, &ctl->full[stage], kb * kTileK, a_row);
          ptx::tma_load_2d(sb, tb, &ctl->full[stage], kb * kTileK, n_blk * kTileN);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ------------------------- MMA issuer ---------------------------
      constexpr uint32_t idesc = ptx::umma_idesc_f16(FMT, kTileM, kTileN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < sc.items && ok; item += G) {
        const int split = item % sc.splits;
        const int kb0 = split * sc.kb_per_split, kb1 = min(num_kb, kb0 + sc.kb_per_split);
        if (!ptx::mbar_wait(&ctl->tmem_empty[acc], acc_phase ^ 1, abort)) break;
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * kTileN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!ptx::mbar_wait(&ctl->full[stage], phase, abort)) {
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint32_t sa = ptx::smem_u32(smem + stage * kStageBytes);
          const uint64_t da = ptx::umma_desc_kmajor_sw128(sa);
          const uint64_t db = ptx::umma_desc_kmajor_sw128(sa + kABytes);
#pragma unroll
          for (int k = 0; k < kTileK / 16; ++k) {
            // Advancing 16 K-elements = 32 bytes inside the 128-byte swizzle atom: +2 in the (>>4) address field.
            ptx::umma_f16(d_tmem, da + uint64_t(k * 2), db + uint64_t(k * 2), idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          ptx::umma_commit(&ctl->empty[stage]);  // stage reusable once these MMAs have read it
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        ptx::umma_commit(&ctl->tmem_full[acc]);  // accumulator complete
        if (++acc == kAccStages) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else if (warp < 6) {
    // --------------------------- epilogue -----------------------------
    // Each epilogue warp owns the 32 accumulator rows of its TMEM lane quadrant.  A row is read from TMEM by one
    // thread (tcgen05.ld 32x32b), converted, and staged in shared memory (XOR-swizzled 16-byte units, conflict
    // free both ways); the warp then writes 256-byte row segments with all lanes, so that stores -- to local
    // memory or to the owner rank's memory over NVLink -- are whole lines, not 16-byte fragments.
    const int q = warp & 3;  // TMEM lane quadrant this warp may read
    uint8_t* stage_buf = smem + kStages * kStageBytes + (warp - 2) * kEpiWarpBytes;
    const uint32_t stage_u32 = ptx::smem_u32(stage_buf);
    int acc = 0;
    uint32_t acc_phase = 0;
    uint32_t iter = 0, prev_iter = 0;
    bool have_prev = false;
    char* c_base = nullptr;
    if constexpr (MODE == kGemmPlain || MODE == kGemmAg) c_base = static_cast<char*>(a.C) + a.c_emu_stride * blockIdx.y;
    for (int item = blockIdx.x; item < sc.items; item += G, ++iter) {
      const int seq = item / sc.splits, split = item - seq * sc.splits;
      int m_blk, n_blk;
      sc.coord(seq, m_blk, n_blk);
      if (!ptx::mbar_wait(&ctl->tmem_full[acc], acc_phase, abort)) break;
      ptx::tc_fence_after_sync();
      const int r_in = q * 32 + lane;
      const uint32_t t_addr = tmem_base + (uint32_t(q * 32) << 16) + acc * kTileN;
      const int tile_id = m_blk * sc.tiles_n + n_blk;
      float* ws_tile = nullptr;
      if constexpr (MODE == kGemmPlain) {
        if (sc.splits > 1)
          ws_tile = splitk_partials(a.splitk_ws) + (size_t(tile_id) * sc.splits + split) * (kTileM * kTileN);
      }
      if (ws_tile != nullptr) {
        // split-K: fp32 partial accumulator, tile-packed [128][256]; rows past M are never read back
        const bool row_live = m_blk * kTileM + r_in < a.M;
#pragma unroll 2
        for (int c = 0; c < kTileN / 32; ++c) {
          uint32_t r[32];
          ptx::tmem_ld_32x32b_x32(t_addr + c * 32, r);
          ptx::tmem_ld_wait();
          if (row_live) {
            float4* dst = reinterpret_cast<float4*>(ws_tile + size_t(r_in) * kTileN + c * 32);
#pragma unroll
            for (int i = 0; i < 8; ++i)
              dst[i] = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]),
                                   __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
          }
        }
        // Accumulator drained: hand the TMEM stage back to the MMA warp.
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&ctl->tmem_empty[acc]);
        // The last CTA to deliver this 32-row quadrant sums the splits in split order and writes C -- unless the
        // host asked for the sum to be left to the reduction kernel that follows this launch (many live rows: one
        // warp summing them is a chain of L2 round trips, a whole grid is not).
        uint32_t* qcnt = static_cast<uint32_t*>(a.splitk_ws) + tile_id * 4 + q;
        uint32_t prev = 0xffffffffu;
        if (!a.splitk_defer) {
          __threadfence();
          __syncwarp();
          if (lane == 0) prev = atomicAdd(qcnt, 1u);
          prev = __shfl_sync(0xffffffffu, prev, 0);
        }
        if (prev == uint32_t(sc.splits - 1)) {
          __threadfence();
          if (lane == 0) *qcnt = 0;  // re-arm for the next call
          const float* base = splitk_partials(a.splitk_ws) + size_t(tile_id) * sc.splits * (kTileM * kTileN);
          // Eight rows x two 128-column halves per step: sixteen independent loads per lane are in flight for
          // every split, instead of one dependent chain per row.
          const int rows_live = min(32, a.M - (m_blk * kTileM + q * 32));
          for (int rr0 = 0; rr0 < rows_live; rr0 += 8) {
            float4 sacc8[8][2];
#pragma unroll
            for (int i = 0; i < 8; ++i) sacc8[i][0] = sacc8[i][1] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
            for (int sp = 0; sp < sc.splits; ++sp) {
              const float* sbase = base + size_t(sp) * (kTileM * kTileN) + size_t(q * 32 + rr0) * kTileN + lane * 4;
              float4 v[8][2];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                // rows past the live range re-read the first row instead of branching (result unused)
                const int ro = rr0 + i < rows_live ? i : 0;
                v[i][0] = __ldcg(reinterpret_cast<const float4*>(sbase + size_t(ro) * kTileN));
                v[i][1] = __ldcg(reinterpret_cast<const float4*>(sbase + size_t(ro) * kTileN + 128));
              }
#pragma unroll
              for (int i = 0; i < 8; ++i) {
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                  sacc8[i][hh].x += v[i][hh].x;
                  sacc8[i][hh].y += v[i][hh].y;
                  sacc8[i][hh].z += v[i][hh].z;
                  sacc8[i][hh].w += v[i][hh].w;
                }
              }
            }
#pragma unroll
            for (int idx = 0; idx < 16; ++idx) {
              const int rr = rr0 + (idx >> 1), half = idx & 1;
              if (rr >= rows_live) continue;
              const int grow = m_blk * kTileM + q * 32 + rr;
              const float4 sacc = sacc8[idx >> 1][half];
              const int cc = half * 128 + lane * 4;
              const int gcol = n_blk * kTileN + cc;
              if (gcol < a.N) {
                const float f[4] = {sacc.x, sacc.y, sacc.z, sacc.w};
                char* dst = c_base + (size_t(grow) * a.ldc + gcol) * 2;
                if (gcol + 4 <= a.N && (a.ldc % 4) == 0) {
                  uint2 o;
                  if constexpr (PackTraits<T>::kDType == kBF16) {
                    __nv_bfloat162 h0 = __floats2bfloat162_rn(f[0], f[1]), h1 = __floats2bfloat162_rn(f[2], f[3]);
                    o.x = *reinterpret_cast<uint32_t*>(&h0);
                    o.y = *reinterpret_cast<uint32_t*>(&h1);
                  } else {
                    __half2 h0 = __floats2half2_rn(f[0], f[1]), h1 = __floats2half2_rn(f[2], f[3]);
                    o.x = *reinterpret_cast<uint32_t*>(&h0);
                    o.y = *reinterpret_cast<uint32_t*>(&h1);
                  }
                  *reinterpret_cast<uint2*>(dst) = o;
                } else {
                  for (int i = 0; i < 4 && gcol + i < a.N; ++i)
                    reinterpret_cast<T*>(dst)[i] = PackTraits<T>::from_float(f[i]);
                }
              }
            }
          }
        }
      } else {
        // Destination of this warp's 32 rows: local C, or this rank's slice of the tile in the OWNER's buffer.
        char* dst_rows;        // address of (row q*32, column 0 of the tile)
        size_t dst_row_bytes;  // distance between rows
        int owner = 0, owner_counter = 0;
        size_t push_row0 = 0;
        if constexpr (MODE == kGemmPlain || MODE == kGemmAg) {
          dst_row_bytes = size_t(a.ldc) * 2;
          dst_rows = c_base + (size_t(m_blk * kTileM + q * 32) * a.ldc + size_t(n_blk) * kTileN) * 2;
        } else {
          size_t slice;
          if constexpr (MODE == kGemmAr) {
            owner = seq % ctx.world;
            owner_counter = a.counter_base + seq / ctx.world;
            slice = size_t(seq / ctx.world) * ctx.world + ctx.rank;
            if (a.use_nvls == 2 && a.partial.mc != nullptr && a.c_sym.mc != nullptr) {
              owner = ctx.rank;  // pull variant: the tile stays here, at the offset every rank uses for it
              slice = size_t(tile_id);
            }
          } else {
            owner = m_blk / sc.bps;
            const int lb = m_blk - owner * sc.bps;
            owner_counter = a.counter_base + lb;
            slice = (size_t(lb) * sc.tiles_n + n_blk) * ctx.world + ctx.rank;
          }
          dst_row_bytes = kTileN * 2;
          dst_rows = static_cast<char*>(a.partial.p[owner]) + slice * kTileBytes + size_t(q * 32) * (kTileN * 2);
          push_row0 = slice * kTileM + size_t(q * 32);  // row of the owner's buffer seen as [slices * 128, 256]
        }
        (void)dst_rows;
        (void)dst_row_bytes;
#pragma unroll 1
        for (int h = 0; h < 2; ++h) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            ptx::tmem_ld_32x32b_x32(t_addr + h * 128 + c * 32, r);
            ptx::tmem_ld_wait();
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
              uint32_t saddr;
              if constexpr (MODE == kGemmAr || MODE == kGemmRsNorm) {
                // Two [32 rows][128 B] sub-tiles in the 128-byte-swizzle layout of the TMA store below.
                saddr = stage_u32 + (u >> 3) * 4096 + lane * 128 + (((u & 7) ^ (lane & 7)) << 4);
              } else {
                saddr = stage_u32 + lane * 256 + ((u ^ (lane & 7)) << 4);
              }
              asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(saddr), "r"(w[0]), "r"(w[1]), "r"(w[2]),
                           "r"(w[3])
                           : "memory");
            }
          }
          if (h == 1) {
            // Everything has left TMEM: hand the accumulator stage back before the last copy-out.
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&ctl->tmem_empty[acc]);
          }
          if constexpr (MODE == kGemmAr || MODE == kGemmRsNorm) {
            // Push this half (32 rows x 128 columns) into the owner's buffer with two bulk tensor stores issued
            // by one lane: the copy engine moves the data, no warp waits on NVLink.
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              const CUtensorMap* pm = static_cast<const CUtensorMap*>(a.push_maps) + owner;
              const int y = static_cast<int>(push_row0);
              ptx::tma_store_2d(pm, stage_buf, h * 128, y);
              ptx::tma_store_2d(pm, stage_buf + 4096, h * 128 + 64, y);
              ptx::bulk_commit_group();
              if (h == 0) {
                ptx::bulk_wait_group_read<0>();  // staging buffer is reused by the second half
              } else {
                // Tile i-1 of this warp is complete once only this tile's two groups may still be pending.
                ptx::bulk_wait_group<2>();
                if (have_prev) {
                  ptx::fence_proxy_async_all();
                  __threadfence_block();
                  atomicAdd(&ctl->epi_count[prev_iter & 7], 1u);
                }
                ptx::bulk_wait_group_read<0>();
              }
            }
            __syncwarp();
            if (h == 1) {
              have_prev = true;
              prev_iter = iter;
            }
            continue;
          }
          __syncwarp();
#pragma unroll 4
          for (int i = 0; i < 16; ++i) {
            const int rr = 2 * i + (lane >> 4), u = lane & 15;
            uint4 v;
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                         : "r"(stage_u32 + rr * 256 + ((u ^ (rr & 7)) << 4))
                         : "memory");
            char* dst = dst_rows + size_t(rr) * dst_row_bytes + h * 256 + u * 16;
            if constexpr (MODE == kGemmPlain || MODE == kGemmAg) {
              const int grow = m_blk * kTileM + q * 32 + rr;
              const int gcol = n_blk * kTileN + h * 128 + u * 8;
              if (grow < a.M && gcol < a.N) {
                if (gcol + 8 <= a.N && (a.ldc % 8) == 0) {
                  ptx::st_v4(dst, v);
                } else {
                  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
                  for (int e = 0; e < 8 && gcol + e < a.N; ++e)
                    reinterpret_cast<unsigned short*>(dst)[e] =
                        static_cast<unsigned short>((e & 1) ? (w[e >> 1] >> 16) : (w[e >> 1] & 0xffff));
                }
              }
            } else {
              ptx::st_v4(dst, v);  // the whole padded tile is pushed so that the owner can stream it
            }
          }
          __syncwarp();
        }
        if constexpr (MODE == kGemmAr || MODE == kGemmRsNorm) {
          // This warp's rows of the tile have been issued.  It does NOT wait for the (remote) stores to land:
          // it only tells the signal warp, which takes the wait, and moves on to the next tile.
          (void)owner_counter;
        }
      }
      if (++acc == kAccStages) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
    if constexpr (MODE == kGemmAr || MODE == kGemmRsNorm) {
      // Last tile of this warp: wait for its bulk stores, then tell the signal warp.
      if (lane == 0 && have_prev) {
        ptx::bulk_wait_group<0>();
        ptx::fence_proxy_async_all();
        __threadfence_block();
        atomicAdd(&ctl->epi_count[prev_iter & 7], 1u);
      }
    }
  } else if (warp == 6) {
    // --------------------------- signal warp (fused AR / RS) -----------------------------
    // One thread follows the CTA's tiles in order.  When all four epilogue warps have issued their rows of a
    // tile it orders those stores system-wide (the fence is cumulative over what it observed through the
    // CTA-scope counter) and publishes one arrival on the owner rank.  The epilogue warps never stall on NVLink.
    if constexpr (MODE == kGemmAr || MODE == kGemmRsNorm) {
      if (lane == 0) {
        uint32_t iter = 0;
        for (int item = blockIdx.x; item < sc.items; item += G, ++iter) {
          const uint32_t expected = 4u * (iter / 8u + 1u);
          volatile uint32_t* cnt = &ctl->epi_count[iter & 7];
          uint32_t polls = 0;
          bool ok = true;
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
          sc.coord(item, m_blk, n_blk);
          int owner, idx;
          if constexpr (MODE == kGemmAr) {
            owner = item % ctx.world;
            idx = a.counter_base + item / ctx.world;
          } else {
            owner = m_blk / sc.bps;
            idx = a.counter_base + (m_blk - owner * sc.bps);
          }
          ptx::fence_acq_rel_sys();
          ptx::red_release_sys_add(counter_ptr(ctx, owner, idx), 1u);
        }
      }
    }
  }

  // ---- teardown -----------------------------------------------------------
  __syncthreads();
  if (a.trace) trace_put(a, kTraceGemmDone, ptx::globaltimer_ns());
  const bool aborted = *abort != 0;
  if (aborted) {
    // Give copies that may still be in flight time to land before shared memory is released.
    if (threadIdx.x == 0) {
      gemm_report(ctx.status, ctx.rank, kDevTimeoutMbarrier, 80);
      const uint64_t t0 = ptx::globaltimer_ns();
      while (ptx::globaltimer_ns() - t0 < 200000) __nanosleep(1000);
    }
    __syncthreads();
  }
  if constexpr (MODE == kGemmAg) {
    // Last GEMM CTA out re-arms the chunk flags (every flag has reached its final value by now).
    if (threadIdx.x == 0 && !aborted) {
      uint32_t* done = counter_ptr(ctx, ctx.rank, a.counter_base + sc.tiles_m);
      __threadfence();
      if (atomicAdd(done, 1u) == uint32_t(G - 1)) {
        for (int i = 0; i < sc.tiles_m; ++i) *counter_ptr(ctx, ctx.rank, a.counter_base + i) = 0;
        *done = 0;
        __threadfence();
      }
    }
  }
  if (warp == 1) {
    __syncwarp();
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
  // GEMM CTAs that are done computing help with the reduction of what is still in flight.
  if constexpr (MODE == kGemmAr) {
    if (!aborted && !a.no_join) ar_reducer_role<T, THREADS>(ctx, a, sc, int(gridDim.x));
  }
  if constexpr (MODE == kGemmRsNorm) {
    if (!aborted && !a.no_join) rs_reducer_role<T, THREADS>(ctx, a, sc, int(gridDim.x));
  }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------

// 2-D tensor map over a row-major [rows, cols] 16-bit matrix; box = box_rows x 64 elements, 128-byte swizzle.
typedef bool (*TmapFn)(CUtensorMap* out, const void* p, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows);

inline int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

// `emu_table_dev`: device memory for 3 * kMaxRanks tensor maps (emulation only; may be null otherwise).
template <typename T, int MODE>
cudaError_t launch_mode(const CommCtx& ctx, const GemmArgs& a, cudaStream_t stream, TmapFn make_tmap,
                        CUtensorMap* emu_table_dev) {
  constexpr int THREADS = MODE == kGemmPlain ? kThreadsPlain : kThreadsFused;
  auto kernel = gemm_kernel<T, MODE>;
  static uint64_t attr_set_mask = 0;  // per device (one bit each)
  int dev = 0;
  cudaGetDevice(&dev);
  if (!(attr_set_mask >> (dev & 63) & 1)) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set_mask |= uint64_t(1) << (dev & 63);
  }
  const bool emu = ctx.emu_table != nullptr;
  const int world = ctx.world;
  const int tiles = ((a.M + kTileM - 1) / kTileM) * ((a.N + kTileN - 1) / kTileN);
  const int splits = (MODE == kGemmPlain && a.splits > 1) ? a.splits : 1;
  int budget = a.max_ctas > 0 ? a.max_ctas : sm_count();
  // The fused modes use blockIdx.x as the slot of their rank barriers: the grid must stay inside the inbox rows of
  // the signal pad (a larger part, or a caller asking for more CTAs, would write into the peers' epoch words).
  static_assert(kPadInboxWords == kMaxCommBlocks * kMaxRanks, "one inbox row per CTA that may take part in a rank barrier");
  if (MODE != kGemmPlain && budget > kMaxCommBlocks) budget = kMaxCommBlocks;
  if (emu) budget = budget / world;
  int comm = MODE == kGemmPlain ? 0 : (a.comm_ctas > 0 ? a.comm_ctas : 16);
  if (comm > budget / 2) comm = budget / 2;
  if (MODE != kGemmPlain && comm < 1) return cudaErrorInvalidValue;
  int gemm_ctas = budget - comm;
  if (gemm_ctas > tiles * splits) gemm_ctas = tiles * splits;
  if (gemm_ctas < 1) return cudaErrorInvalidValue;

  const int shard_rows = a.M / world;
  CUtensorMap ta, tb, tal;
  EmuMaps em{nullptr};
  if (!emu) {
    const void* a_ptr = MODE == kGemmAg ? a.a_full.p[ctx.rank] : a.A;
    const uint64_t a_ld = MODE == kGemmAg ? uint64_t(a.K) : uint64_t(a.lda);
    if (!make_tmap(&ta, a_ptr, a.M, a.K, a_ld, kTileM)) return cudaErrorInvalidValue;
    if (!make_tmap(&tb, a.B, a.N, a.K, a.ldb, kTileN)) return cudaErrorInvalidValue;
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
      if (!make_tmap(&host[3 * r + 1], B_r, a.N, a.K, a.ldb, kTileN)) return cudaErrorInvalidValue;
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

  const int grid_x = gemm_ctas + comm;
  if (emu) {
    dim3 grid(grid_x, world);
    CommCtx c = ctx;
    GemmArgs aa = a;
    int g = gemm_ctas;
    void* argv[] = {(void*)&ta, (void*)&tb, (void*)&tal, (void*)&em, (void*)&c, (void*)&aa, (void*)&g};
    return cudaLaunchCooperativeKernel((const void*)kernel, grid, dim3(THREADS), argv, kSmemBytes, stream);
  }
  kernel<<<dim3(grid_x, 1), THREADS, kSmemBytes, stream>>>(ta, tb, tal, em, ctx, a, gemm_ctas);
  return cudaGetLastError();
}

// Sums the split-K partial tiles [tile][split][128][256] in split order and writes C: the second kernel of a
// split-K GEMM whose launch asked for a deferred reduction.  One thread per row and 8 columns.
template <typename T>
__global__ void splitk_reduce_kernel(const float* __restrict__ partials, T* C, int M, int N, int ldc, int tiles_n,
                                     int splits) {
  const int n8 = (N + 7) / 8;
  const long long total = static_cast<long long>(M) * n8;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int m = static_cast<int>(i / n8), n = static_cast<int>(i % n8) * 8;
    const int tile_id = (m / kTileM) * tiles_n + n / kTileN;
    const float* src = partials + static_cast<size_t>(tile_id) * splits * (kTileM * kTileN) + static_cast<size_t>(m % kTileM) * kTileN +
                       (n % kTileN);
    float4 lo = make_float4(0.f, 0.f, 0.f, 0.f), hi = lo;
#pragma unroll 8
    for (int sp = 0; sp < splits; ++sp) {
      const float4 a0 = __ldcg(reinterpret_cast<const float4*>(src + static_cast<size_t>(sp) * (kTileM * kTileN)));
      const float4 a1 = __ldcg(reinterpret_cast<const float4*>(src + static_cast<size_t>(sp) * (kTileM * kTileN) + 4));
      lo.x += a0.x; lo.y += a0.y; lo.z += a0.z; lo.w += a0.w;
      hi.x += a1.x; hi.y += a1.y; hi.z += a1.z; hi.w += a1.w;
    }
    const float f[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
    T* dst = C + static_cast<size_t>(m) * ldc + n;
    if (n + 8 <= N && (ldc % 8) == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0) {
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if constexpr (PackTraits<T>::kDType == kBF16) {
          __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
          w[j] = *reinterpret_cast<uint32_t*>(&h);
        } else {
          __half2 h = __floats2half2_rn(f[2 * j], f[2 * j + 1]);
          w[j] = *reinterpret_cast<uint32_t*>(&h);
        }
      }
      *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
      for (int j = 0; j < 8 && n + j < N; ++j) dst[j] = PackTraits<T>::from_float(f[j]);
    }
  }
}

template <typename T>
cudaError_t launch_splitk_reduce(const GemmArgs& a, cudaStream_t stream) {
  const int tiles_n = (a.N + kTileN - 1) / kTileN;
  const long long total = static_cast<long long>(a.M) * ((a.N + 7) / 8);
  const int threads = 256;
  long long blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 8) blocks = 148 * 8;
  splitk_reduce_kernel<T><<<static_cast<int>(blocks), threads, 0, stream>>>(
      splitk_partials(a.splitk_ws), static_cast<T*>(a.C), a.M, a.N, a.ldc, tiles_n, a.splits);
  return cudaGetLastError();
}

// Bytes of split-K workspace for a problem: the counter block plus the fp32 partial tiles.
inline size_t splitk_workspace_bytes(int M, int N, int splits) {
  const size_t tiles = size_t((M + kTileM - 1) / kTileM) * ((N + kTileN - 1) / kTileN);
  return kSplitkCounterBytes + tiles * splits * (size_t(kTileM) * kTileN * 4);
}

// Number of K splits that leaves no split empty (each split gets ceil(num_kb / splits) K blocks).
inline int normalize_splits(int K, int want) {
  const int num_kb = (K + kTileK - 1) / kTileK;
  if (want < 1) want = 1;
  if (want > num_kb) want = num_kb;
  const int per = (num_kb + want - 1) / want;
  return (num_kb + per - 1) / per;
}

}  // namespace gemm_detail
}  // namespace oob
