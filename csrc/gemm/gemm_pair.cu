// Two-SM tcgen05 GEMM for sm_100a: a pair of CTAs on neighbouring SMs (a cluster of two) computes one 256x256
// output tile with tcgen05.mma.cta_group::2.
//
// Why a second kernel beside gemm_kernel.cuh: with one CTA per tile every SM stages the whole 256x64 B block of a
// K step (32 KiB) next to its 128x64 A block.  In a pair each CTA stages only HALF of B (128 of the 256 N rows); the
// tensor cores of the two SMs read both halves.  Per SM and K step that is 32 KiB instead of 48 KiB through L2 and
// shared memory, which leaves room for six pipeline stages instead of four and lowers the power spent on data
// movement -- the plain GEMM is power-capped on this part, so traffic saved is clock gained.
//
// Roles per CTA (192 threads):
//   warp 0    TMA producer (both CTAs): loads this CTA's 128 A rows and its 128 B rows of the K step into its own
//             shared memory; the copy's completion is counted on the LEADER CTA's `full` barrier
//             (cp.async.bulk.tensor ... .cta_group::2, no multicast: every byte is loaded once)
//   warp 1    MMA issuer (leader CTA only): one thread issues M256 N256 K16 instructions; tcgen05.commit with a
//             two-CTA mask releases the stage in both CTAs / publishes the accumulator to both epilogues
//   warps 2-5 epilogue (both CTAs): each CTA drains its own 128 accumulator rows from its own TMEM (two
//             accumulator stages), converts, stages through shared memory and writes whole 256-byte row segments
// Every wait is bounded; a CTA that gives up records the failure in the status block and both CTAs of the pair
// still meet at the closing cluster barrier (the peer's waits run out as well), so TMEM is always released.
//
// Capability parity with the reference: the plain GEMM (src/gemm/gemm_plain_sm90.cu) and the cluster shapes of its
// generated instances (src/gemm/gemm_plain_sm90_dispatch.h:19-46); Hopper's 2x1 cluster with multicast loads maps
// to the Blackwell CTA pair here.
#include <cuda.h>
#include <cuda_runtime.h>

#include "gemm_kernel.cuh"

namespace oob {
namespace gemm_pair {

using namespace gemm_detail;

constexpr int kStagesP = 6;
constexpr int kHalfBBytes = (kTileN / 2) * kTileK * 2;   // 16 KiB: this CTA's half of the B block
constexpr int kStageBytesP = kABytes + kHalfBBytes;      // 32 KiB per CTA and stage
constexpr int kPairTileM = 2 * kTileM;                   // 256
constexpr int kSmemBytesP = kStagesP * kStageBytesP + kEpiBytes + 1024 + 256;
constexpr int kThreadsP = 192;

struct SmemCtlP {
  uint64_t full[kStagesP];         // used in the leader CTA only: bytes of both CTAs' copies
  uint64_t empty[kStagesP];        // per CTA: one arrival from the leader's commit
  uint64_t tmem_full[kAccStages];  // per CTA: one arrival from the leader's commit
  uint64_t tmem_empty[kAccStages]; // used in the leader CTA only: 8 arrivals (4 epilogue warps x 2 CTAs)
  uint32_t tmem_base;
  int abort;
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

// Grouped raster over 256x256 tiles: 8 tile rows at a time, so that pairs running at the same time share A and B
// blocks in L2.
__device__ __forceinline__ void pair_coord(int seq, int tiles_m, int tiles_n, int& m_blk, int& n_blk) {
  constexpr int kGroup = 8;
  const int per_group = kGroup * tiles_n;
  const int g = seq / per_group;
  const int first_m = g * kGroup;
  const int rows = (tiles_m - first_m) < kGroup ? (tiles_m - first_m) : kGroup;
  const int in = seq - g * per_group;
  m_blk = first_m + in % rows;
  n_blk = in / rows;
}

template <typename T>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreadsP, 1)
    gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, GemmArgs a,
                     DeviceStatus* status) {
  constexpr int FMT = PackTraits<T>::kDType == kBF16 ? 1 : 0;
  extern __shared__ uint8_t smem_raw[];
  // The same offset in both CTAs (same kernel, same dynamic shared memory base), as the MMA descriptors require.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  SmemCtlP* ctl = reinterpret_cast<SmemCtlP*>(smem + kStagesP * kStageBytesP + kEpiBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();  // 0 = leader
  const bool leader = cta == 0;
  const int pair = blockIdx.x >> 1, P = gridDim.x >> 1;
  const int num_kb = (a.K + kTileK - 1) / kTileK;
  const int tiles_m = (a.M + kPairTileM - 1) / kPairTileM;
  const int tiles_n = (a.N + kTileN - 1) / kTileN;
  const int tiles = tiles_m * tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStagesP; ++s) {
      ptx::mbar_init(&ctl->full[s], 1);
      ptx::mbar_init(&ctl->empty[s], 1);
    }
    for (int s = 0; s < kAccStages; ++s) {
      ptx::mbar_init(&ctl->tmem_full[s], 1);
      ptx::mbar_init(&ctl->tmem_empty[s], 8);
    }
    ctl->abort = 0;
    ptx::mbar_fence_init();
    ptx::prefetch_tmap(&tmap_a);
    ptx::prefetch_tmap(&tmap_b);
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
      for (int item = pair; item < tiles && ok; item += P) {
        int m_blk, n_blk;
        pair_coord(item, tiles_m, tiles_n, m_blk, n_blk);
        const int a_row = m_blk * kPairTileM + int(cta) * kTileM;
        const int b_row = n_blk * kTileN + int(cta) * (kTileN / 2);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!ptx::mbar_wait(&ctl->empty[stage], phase ^ 1, abort)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * kStageBytesP;
          uint8_t* sb = sa + kABytes;
          const uint32_t full_leader = map_to_cta(ptx::smem_u32(&ctl->full[stage]), 0);
          if (leader) ptx::mbar_arrive_expect_tx(&ctl->full[stage], 2 * kStageBytesP);
          tma_load_2d_pair(sa, &tmap_a, full_leader, kb * kTileK, a_row);
          tma_load_2d_pair(sb, &tmap_b, full_leader, kb * kTileK, b_row);
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
      for (int item = pair; item < tiles && ok; item += P) {
        if (!ptx::mbar_wait(&ctl->tmem_empty[acc], acc_phase ^ 1, abort)) break;
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * kTileN;
        for (int kb = 0; kb < num_kb; ++kb) {
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
            umma_f16_pair(d_tmem, da + uint64_t(k * 2), db + uint64_t(k * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
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
  } else {
    // --------------------------- epilogue (both CTAs) -----------------------------
    const int q = warp & 3;  // TMEM lane quadrant this warp may read
    uint8_t* stage_buf = smem + kStagesP * kStageBytesP + (warp - 2) * kEpiWarpBytes;
    const uint32_t stage_u32 = ptx::smem_u32(stage_buf);
    int acc = 0;
    uint32_t acc_phase = 0;
    char* c_base = static_cast<char*>(a.C);
    const bool vec_ok = (a.ldc % 8) == 0;
    for (int item = pair; item < tiles; item += P) {
      int m_blk, n_blk;
      pair_coord(item, tiles_m, tiles_n, m_blk, n_blk);
      if (!ptx::mbar_wait(&ctl->tmem_full[acc], acc_phase, abort)) break;
      ptx::tc_fence_after_sync();
      const uint32_t t_addr = tmem_base + (uint32_t(q * 32) << 16) + acc * kTileN;
      const int row0 = m_blk * kPairTileM + int(cta) * kTileM + q * 32;  // first of this warp's 32 rows
      char* dst_rows = c_base + (size_t(row0) * a.ldc + size_t(n_blk) * kTileN) * 2;
      const size_t dst_row_bytes = size_t(a.ldc) * 2;
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
            const uint32_t saddr = stage_u32 + lane * 256 + ((u ^ (lane & 7)) << 4);
            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(saddr), "r"(w[0]), "r"(w[1]), "r"(w[2]),
                         "r"(w[3])
                         : "memory");
          }
        }
        if (h == 1) {
          // Everything has left TMEM: hand the accumulator stage back to the leader's MMA thread.
          ptx::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(map_to_cta(ptx::smem_u32(&ctl->tmem_empty[acc]), 0));
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
          const int grow = row0 + rr;
          const int gcol = n_blk * kTileN + h * 128 + u * 8;
          if (grow < a.M && gcol < a.N) {
            char* dst = dst_rows + size_t(rr) * dst_row_bytes + h * 256 + u * 16;
            if (gcol + 8 <= a.N && vec_ok) {
              ptx::st_v4(dst, v);
            } else {
              const uint32_t w[4] = {v.x, v.y, v.z, v.w};
              for (int e = 0; e < 8 && gcol + e < a.N; ++e)
                reinterpret_cast<unsigned short*>(dst)[e] =
                    static_cast<unsigned short>((e & 1) ? (w[e >> 1] >> 16) : (w[e >> 1] & 0xffff));
            }
          }
        }
        __syncwarp();
      }
      if (++acc == kAccStages) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }

  // ---- teardown -----------------------------------------------------------
  __syncthreads();
  if (*abort != 0) {
    if (threadIdx.x == 0) {
      gemm_report(status, 0, kDevTimeoutMbarrier, 90 + int(cta));
      // Copies that may still be in flight get time to land before shared memory is released.
      const uint64_t t0 = ptx::globaltimer_ns();
      while (ptx::globaltimer_ns() - t0 < 200000) __nanosleep(1000);
    }
    __syncthreads();
  }
  ptx::tc_fence_before_sync();
  cluster_sync_all();  // the peer has no MMA, commit or remote arrival left that targets this CTA
  ptx::tc_fence_after_sync();
  if (warp == 1) tmem_dealloc_pair(tmem_base, kTmemCols);
}

}  // namespace gemm_pair

// Number of CTA pairs that can be resident at once (0 when the device cannot run the kernel).
template <typename T>
static int pair_capacity(int dev) {
  static int cached[64];
  static bool have[64];
  if (have[dev & 63]) return cached[dev & 63];
  auto kernel = gemm_pair::gemm_pair_kernel<T>;
  int clusters = 0;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, gemm_pair::kSmemBytesP) == cudaSuccess) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * 74);
    cfg.blockDim = dim3(gemm_pair::kThreadsP);
    cfg.dynamicSmemBytes = gemm_pair::kSmemBytesP;
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

template <typename T>
static cudaError_t launch_pair_fmt(const GemmArgs& a, DeviceStatus* status, cudaStream_t stream, gemm_detail::TmapFn make_tmap) {
  int dev = 0;
  cudaGetDevice(&dev);
  int pairs = pair_capacity<T>(dev);
  if (pairs <= 0) return cudaErrorNotSupported;
  if (a.max_ctas > 0 && pairs > a.max_ctas / 2) pairs = a.max_ctas / 2;
  const int tiles = ((a.M + gemm_pair::kPairTileM - 1) / gemm_pair::kPairTileM) * ((a.N + kTileN - 1) / kTileN);
  if (pairs > tiles) pairs = tiles;
  if (pairs < 1) return cudaErrorInvalidValue;
  CUtensorMap ta, tb;
  if (!make_tmap(&ta, a.A, a.M, a.K, a.lda, kTileM)) return cudaErrorInvalidValue;
  if (!make_tmap(&tb, a.B, a.N, a.K, a.ldb, kTileN / 2)) return cudaErrorInvalidValue;
  gemm_pair::gemm_pair_kernel<T><<<dim3(2 * pairs), gemm_pair::kThreadsP, gemm_pair::kSmemBytesP, stream>>>(ta, tb, a, status);
  return cudaGetLastError();
}

cudaError_t launch_gemm_pair(const GemmArgs& a, DeviceStatus* status, cudaStream_t stream, gemm_detail::TmapFn make_tmap) {
  return a.fmt == 1 ? launch_pair_fmt<__nv_bfloat16>(a, status, stream, make_tmap)
                    : launch_pair_fmt<__half>(a, status, stream, make_tmap);
}

}  // namespace oob
