// Host interface of the two-SM (CTA pair) GEMM kernel: launch plan, stream-K planning, workspace.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstddef>
#include "gemm.h"

namespace oob {

namespace gemm_pair {

// Stream-K workspace geometry.  The tail holds fewer than two waves of tiles, and a pair parks at most one partial
// accumulator (256x256 fp32), so the size depends on the pair count only.
constexpr int kSkMaxPairs = 80;               // >= 74 pairs of a 148-SM part
constexpr int kSkMaxTiles = 2 * kSkMaxPairs;  // tiles of a tail
constexpr size_t kSkFlagBytes = 8192;         // kSkMaxTiles x 2 CTAs x 4 warps x 4 bytes, rounded up
constexpr size_t kSkSlotBytes = size_t(256) * 256 * 4;
constexpr size_t kSkWorkspaceBytes = kSkFlagBytes + size_t(kSkMaxPairs) * kSkSlotBytes;

// What the host decided for one launch.
struct PairPlan {
  int gemm_pairs;  // CTA pairs that compute tiles (communication clusters follow them in the grid)
  int sk_tiles;    // tiles of the stream-K tail, 0 = every tile is computed whole by one pair
  int sk_pairs;    // pairs that share the tail
  void* sk_ws;     // stream-K workspace (flags + slots), null without a tail
};

// ---- schedule (host and device: the host side exists for tests of the enumeration) ------------------------------
// Everything a role needs to enumerate the work items of its pair.  All roles of a pair (and, in the fused modes,
// all ranks) derive the same sequence from it.
struct PairSched {
  int tiles_m, tiles_n, tiles, num_kb;
  int P;         // GEMM pairs of this launch
  int dp_tiles;  // tiles dealt out whole, round robin (tile s goes to pair s % P)
  int sk_tiles;  // tiles of the stream-K tail (the last ones of the sequence); 0 = none
  int sk_pairs;  // pairs that share the tail
  int sk_units;  // sk_tiles * num_kb
  int mode, world, rank;
  int bpr;       // RS / AG: 256-row blocks per rank when the rows split evenly into such blocks, else 0

  // Logical tile (m_blk, n_blk) of schedule position `seq`.  Every rank walks the same sequence so that arrival
  // counters fill at about the same time.
  __host__ __device__ void coord(int seq, int& m_blk, int& n_blk) const {
    if (mode == kGemmRsNorm && bpr > 0) {
      // Row-block major; consecutive row blocks belong to consecutive owners.
      const int i = seq / tiles_n;
      n_blk = seq % tiles_n;
      m_blk = (i % world) * bpr + i / world;
    } else if (mode == kGemmAg && bpr > 0) {
      // Own shard first (it is local), then block c of every other rank in ring order.
      const int i = seq / tiles_n;
      n_blk = seq % tiles_n;
      if (i < bpr) {
        m_blk = rank * bpr + i;
      } else {
        const int k = i - bpr;
        const int c = k / (world - 1);
        const int s = (rank + 1 + k % (world - 1)) % world;
        m_blk = s * bpr + c;
      }
    } else if (mode == kGemmRsNorm || mode == kGemmAg) {
      m_blk = seq / tiles_n;
      n_blk = seq % tiles_n;
    } else {
      // Grouped raster: 8 tile rows at a time, so that pairs running at the same time share A and B blocks in L2.
      constexpr int kGroup = 8;
      const int per_group = kGroup * tiles_n;
      const int g = seq / per_group;
      const int first_m = g * kGroup;
      const int rows = (tiles_m - first_m) < kGroup ? (tiles_m - first_m) : kGroup;
      const int in = seq - g * per_group;
      m_blk = first_m + in % rows;
      n_blk = in / rows;
    }
  }
  // First unit of the stream-K range of pair p (p may be sk_pairs: one past the last range).
  __host__ __device__ int sk_start(int p) const { return static_cast<int>(static_cast<long long>(sk_units) * p / sk_pairs); }
  // Pair whose range holds unit u.
  __host__ __device__ int sk_owner(int u) const {
    int p = static_cast<int>((static_cast<long long>(u) * sk_pairs) / sk_units);
    if (p >= sk_pairs) p = sk_pairs - 1;
    while (p + 1 < sk_pairs && sk_start(p + 1) <= u) ++p;
    while (p > 0 && sk_start(p) > u) --p;
    return p;
  }
};

struct Item {
  int seq;       // schedule position of the tile
  int sk_tile;   // index inside the stream-K tail (partial items)
  int kb0, kb1;  // K blocks [kb0, kb1)
  bool partial;  // true: this pair computes only part of the tile's K range
};

// Enumerates the items of one pair: whole tiles first, then the pair's range of the stream-K tail (at most three
// items: the end of one tile, a whole tile, the beginning of the next).
struct ItemIter {
  int i, u, u_end;
  __host__ __device__ ItemIter(const PairSched& s, int pair) : i(0), u(0), u_end(0) {
    if (s.sk_tiles > 0 && pair < s.sk_pairs) {
      u = s.sk_start(pair);
      u_end = s.sk_start(pair + 1);
    }
  }
  __host__ __device__ bool next(const PairSched& s, int pair, Item& it) {
    const int seq = i * s.P + pair;
    if (seq < s.dp_tiles) {
      it.seq = seq;
      it.sk_tile = -1;
      it.kb0 = 0;
      it.kb1 = s.num_kb;
      it.partial = false;
      ++i;
      return true;
    }
    if (u < u_end) {
      const int t = u / s.num_kb;
      const int kb0 = u - t * s.num_kb;
      int len = s.num_kb - kb0;
      if (len > u_end - u) len = u_end - u;
      it.seq = s.dp_tiles + t;
      it.sk_tile = t;
      it.kb0 = kb0;
      it.kb1 = kb0 + len;
      it.partial = len < s.num_kb;
      u += len;
      return true;
    }
    return false;
  }
};

}  // namespace gemm_pair

// 1 when a stream-K tail pays for `tiles` 256x256 tiles on `pairs` pairs with `num_kb` K blocks per tile: the last
// wave would leave pairs idle for more than 3 % of the run, K is deep enough to cut, and the operands (`operand_bytes`
// of A and B together) are small enough for L2 to make up for the lost lockstep of the pairs.
int pair_streamk_auto(int tiles, int pairs, int num_kb, long long operand_bytes);
// Size of the tail (one wave + remainder, or everything when there is less than a wave) and the number of pairs
// that share it; both 0 when a tail is not possible.
void pair_streamk_plan(int tiles, int pairs, int num_kb, int* sk_tiles, int* sk_pairs);

// Whether the pair kernel can run this (mode, shape).
bool gemm_pair_supported(const CommCtx& ctx, const GemmArgs& args);

typedef bool (*PairTmapFn)(CUtensorMap* out, const void* p, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows);
// Launches the pair kernel; cudaErrorNotSupported when the device cannot hold a pair.
cudaError_t launch_gemm_pair(const CommCtx& ctx, const GemmArgs& args, cudaStream_t stream, PairTmapFn make_tmap,
                             CUtensorMap* emu_table_dev);

// Test hook: enumerates the work items of every pair for a problem, nine integers per item (pair, schedule position,
// m block, n block, first K block, end K block, workspace slot (-1 whole tile, -2 the owner's part), parts of the tile,
// first pair of the tile).
// Returns the number of items, -1 when `cap` integers do not hold them.
int pair_schedule_dump(int mode, int M, int N, int K, int pairs, int stream_k, int world, int rank, int* out, int cap);

// Allocates the stream-K workspace of the current device now (it is otherwise allocated by the first launch that
// needs it, which must not happen during stream capture).
cudaError_t gemm_pair_reserve_workspace();

}  // namespace oob
