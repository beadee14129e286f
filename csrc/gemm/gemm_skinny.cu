// Weight-streaming tcgen05 GEMM for few rows (M <= 128 tokens): C[M, N] = A[M, K] * B[N, K]^T is computed as
// C^T = B * A^T, so the WEIGHT rows fill the 128-row dimension of the tensor-core instruction and the tokens are
// its narrow N dimension (16 .. 128).  This is the decode-step GEMM: its time is the time to read B once.
//
// What differs from the square-tile kernels (gemm_kernel.cuh, gemm_pair.cu):
//   * a pipeline stage holds 128 weight rows x 128 K elements, i.e. 256 contiguous bytes per row and stage (two
//     128-byte swizzle boxes issued back to back) instead of 128, and no 128-row A tile that is mostly padding;
//     with M = 16 a stage is 36 KiB and six stages fit, so ~200 KiB of loads are in flight per SM;
//   * stream-K work split: the (tile, K block) units are dealt out evenly, every CTA gets one contiguous run of
//     units, so all SMs stream for the same time whatever N / 128 is.  A run that covers only part of a tile's K
//     range leaves an fp32 partial in the workspace; the warp that completes a 32-row quadrant of a tile sums the
//     partials in CTA order (deterministic) and writes C;
//   * one launch = one run per CTA (not persistent): the accumulator is 128 lanes x M columns of TMEM.
// Roles: warp 0 TMA producer, warp 1 MMA issuer (one thread), warps 2-5 epilogue.  All waits are bounded.
//
// Capability parity with the reference: its stream-K GEMM instances
// (src/gemm/gemm_with_signal_sm90.h:238-292) and the small-M end of its plain-GEMM dispatch table
// (src/gemm/gemm_plain_sm90_dispatch.h:19-46).
#include <cuda.h>
#include <cuda_runtime.h>

#include "gemm_kernel.cuh"

namespace oob {

// gemm.cu: the library-owned workspace (arrival counters, zero between calls, then partials).
cudaError_t gemm_library_workspace(size_t bytes, cudaStream_t stream, void** out);

namespace gemm_skinny {

using namespace gemm_detail;

constexpr int kRowsW = 128;              // weight rows per tile (the instruction's M)
constexpr int kKB = 128;                 // K elements per stage: two swizzle boxes of 64
constexpr int kWSubBytes = kRowsW * 128; // one 128-row x 64-element box
constexpr int kMaxTokens = 128;
constexpr int kThreadsS = 192;
constexpr int kMaxStagesS = 8;
constexpr int kSmemLimit = 227 * 1024;
constexpr int kCtlBytes = 256;

struct CtlS {
  uint64_t full[kMaxStagesS];
  uint64_t empty[kMaxStagesS];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort;
};
static_assert(sizeof(CtlS) <= kCtlBytes, "control block");

struct Params {
  int M, N, K, Mp;  // Mp: M rounded up to a multiple of 16 (the instruction's N)
  void* C;
  int ldc;
  int num_kb, num_tiles;
  int upc;          // units per CTA
  long long units;  // num_tiles * num_kb
  int stages, stage_bytes;
  uint32_t tmem_cols;
  uint32_t* counters;  // [num_tiles * 4], zero between calls
  float* partials;     // [gridDim.x * 2][Mp * 128]
};

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) {
  return __float2half_rn(v);
}

template <typename T>
__global__ void __launch_bounds__(kThreadsS, 1)
    gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, Params p,
                       DeviceStatus* status) {
  constexpr int FMT = PackTraits<T>::kDType == kBF16 ? 1 : 0;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  CtlS* ctl = reinterpret_cast<CtlS*>(smem + p.stages * p.stage_bytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long u0 = static_cast<long long>(blockIdx.x) * p.upc;
  const long long u1 = min(p.units, u0 + p.upc);
  const int x_sub_bytes = p.Mp * 128;  // one Mp-row x 64-element box of activations

  // One K block of one tile into pipeline stage `stage` (four boxes: two of weights, two of activations).
  auto load_unit = [&](long long u, int stage) {
    const int t = static_cast<int>(u / p.num_kb), kb = static_cast<int>(u - static_cast<long long>(t) * p.num_kb);
    uint8_t* sw = smem + stage * p.stage_bytes;
    uint8_t* sx = sw + 2 * kWSubBytes;
    ptx::mbar_arrive_expect_tx(&ctl->full[stage], p.stage_bytes);
    ptx::tma_load_2d(sw, &tmap_w, &ctl->full[stage], kb * kKB, t * kRowsW);
    ptx::tma_load_2d(sw + kWSubBytes, &tmap_w, &ctl->full[stage], kb * kKB + 64, t * kRowsW);
    ptx::tma_load_2d(sx, &tmap_x, &ctl->full[stage], kb * kKB, 0);
    ptx::tma_load_2d(sx + x_sub_bytes, &tmap_x, &ctl->full[stage], kb * kKB + 64, 0);
  };
  const int prefill = static_cast<int>(min(static_cast<long long>(p.stages), u1 - u0));

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      ptx::mbar_init(&ctl->full[s], 1);
      ptx::mbar_init(&ctl->empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(&ctl->tmem_full[s], 1);
      ptx::mbar_init(&ctl->tmem_empty[s], 4);
    }
    ctl->abort = 0;
    ptx::mbar_fence_init();
    // The whole ring is free at the start: fill it before the CTA has even allocated its TMEM, so that the
    // first bytes are on their way while the rest of the prologue runs.
    for (int i = 0; i < prefill; ++i) load_unit(u0 + i, i);
  }
  if (warp == 1) {
    ptx::tmem_alloc(&ctl->tmem_base, p.tmem_cols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;
  volatile int* abort = &ctl->abort;

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------- TMA producer (continues after the prefill) -------------------------
      int stage = prefill == p.stages ? 0 : prefill;
      uint32_t phase = prefill == p.stages ? 1 : 0;
      for (long long u = u0 + prefill; u < u1; ++u) {
        if (!ptx::mbar_wait(&ctl->empty[stage], phase ^ 1, abort)) break;
        load_unit(u, stage);
        if (++stage == p.stages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ------------------------- MMA issuer ---------------------------
      const uint32_t idesc = ptx::umma_idesc_f16(FMT, kRowsW, p.Mp);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      long long u = u0;
      while (u < u1 && ok) {
        const int t = static_cast<int>(u / p.num_kb);
        const long long seg_end = min(u1, (static_cast<long long>(t) + 1) * p.num_kb);
        if (!ptx::mbar_wait(&ctl->tmem_empty[acc], acc_phase ^ 1, abort)) break;
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * p.Mp;
        bool first = true;
        for (; u < seg_end; ++u) {
          if (!ptx::mbar_wait(&ctl->full[stage], phase, abort)) {
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint32_t sw = ptx::smem_u32(smem + stage * p.stage_bytes);
          const uint32_t sx = sw + 2 * kWSubBytes;
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const uint64_t da = ptx::umma_desc_kmajor_sw128(sw + j * kWSubBytes);
            const uint64_t db = ptx::umma_desc_kmajor_sw128(sx + j * x_sub_bytes);
#pragma unroll
            for (int k = 0; k < 4; ++k)
              ptx::umma_f16(d_tmem, da + uint64_t(k * 2), db + uint64_t(k * 2), idesc, (first && j == 0 && k == 0) ? 0u : 1u);
          }
          first = false;
          ptx::umma_commit(&ctl->empty[stage]);
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        ptx::umma_commit(&ctl->tmem_full[acc]);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // --------------------------- epilogue -----------------------------
    // Thread = one weight row (TMEM lane) of the tile; its registers hold that row's value for every token.
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    const int first_tile = static_cast<int>(u0 / p.num_kb);
    T* C = static_cast<T*>(p.C);
    long long u = u0;
    while (u < u1) {
      const int t = static_cast<int>(u / p.num_kb);
      const long long seg_end = min(u1, (static_cast<long long>(t) + 1) * p.num_kb);
      const int seg_kb = static_cast<int>(seg_end - u);
      const bool complete = seg_kb == p.num_kb;
      if (!ptx::mbar_wait(&ctl->tmem_full[acc], acc_phase, abort)) break;
      ptx::tc_fence_after_sync();
      const int n = t * kRowsW + q * 32 + lane;
      const uint32_t t_addr = tmem_base + (uint32_t(q * 32) << 16) + acc * p.Mp;
      float* slot = p.partials + (size_t(2) * blockIdx.x + (t == first_tile ? 0 : 1)) * (size_t(p.Mp) * kRowsW) + q * 32 + lane;
      for (int c16 = 0; c16 * 16 < p.M; ++c16) {
        uint32_t r[16];
        ptx::tmem_ld_32x32b_x16(t_addr + c16 * 16, r);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int m = c16 * 16 + j;
          if (m < p.M) {
            if (complete) {
              if (n < p.N) C[size_t(m) * p.ldc + n] = from_f32<T>(__uint_as_float(r[j]));
            } else {
              slot[size_t(m) * kRowsW] = __uint_as_float(r[j]);
            }
          }
        }
      }
      // Accumulator drained: hand the TMEM stage back to the MMA thread.
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&ctl->tmem_empty[acc]);
      if (!complete) {
        // This quadrant's share of the tile's K range has been delivered.  Whoever completes the range sums the
        // partials of all contributing CTAs in CTA order and writes C.
        uint32_t* cnt = p.counters + size_t(t) * 4 + q;
        __threadfence();
        __syncwarp();
        uint32_t prev = 0;
        if (lane == 0) prev = atomicAdd(cnt, static_cast<uint32_t>(seg_kb));
        prev = __shfl_sync(0xffffffffu, prev, 0);
        if (prev + static_cast<uint32_t>(seg_kb) == static_cast<uint32_t>(p.num_kb)) {
          __threadfence();
          if (lane == 0) *cnt = 0;  // re-arm for the next call
          const int c_first = static_cast<int>((static_cast<long long>(t) * p.num_kb) / p.upc);
          const int c_last = static_cast<int>(((static_cast<long long>(t) + 1) * p.num_kb - 1) / p.upc);
          for (int m0 = 0; m0 < p.M; m0 += 8) {
            float sum[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) sum[i] = 0.f;
            // Four contributors at a time: 32 independent loads are in flight per lane, so a tile with many
            // contributors costs a few L2 round trips, not one per contributor.  Summation order is CTA order.
#pragma unroll 1
            for (int c0 = c_first; c0 <= c_last; c0 += 4) {
              float v[4][8];
#pragma unroll
              for (int pp = 0; pp < 4; ++pp) {
                const int c = c0 + pp <= c_last ? c0 + pp : c_last;  // past the end: re-read, result unused
                const int which = static_cast<int>((static_cast<long long>(c) * p.upc) / p.num_kb) == t ? 0 : 1;
                const float* src = p.partials + (size_t(2) * c + which) * (size_t(p.Mp) * kRowsW) + q * 32 + lane;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  const int m = m0 + i < p.M ? m0 + i : m0;  // rows past M re-read a live row instead of branching
                  v[pp][i] = __ldcg(src + size_t(m) * kRowsW);
                }
              }
#pragma unroll
              for (int pp = 0; pp < 4; ++pp) {
                if (c0 + pp <= c_last) {
#pragma unroll
                  for (int i = 0; i < 8; ++i) sum[i] += v[pp][i];
                }
              }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i)
              if (m0 + i < p.M && n < p.N) C[size_t(m0 + i) * p.ldc + n] = from_f32<T>(sum[i]);
          }
        }
      }
      u = seg_end;
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }

  // ---- teardown -----------------------------------------------------------
  __syncthreads();
  if (*abort != 0) {
    if (threadIdx.x == 0) {
      gemm_report(status, 0, kDevTimeoutMbarrier, 95);
      const uint64_t t0 = ptx::globaltimer_ns();
      while (ptx::globaltimer_ns() - t0 < 200000) __nanosleep(1000);  // copies in flight land before smem is released
    }
    __syncthreads();
  }
  if (warp == 1) {
    __syncwarp();
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, p.tmem_cols);
  }
}

template <typename T>
cudaError_t launch_fmt(const GemmArgs& a, DeviceStatus* status, cudaStream_t stream, TmapFn make_tmap) {
  auto kernel = gemm_skinny_kernel<T>;
  static uint64_t attr_set_mask = 0;
  int dev = 0;
  cudaGetDevice(&dev);
  if (!(attr_set_mask >> (dev & 63) & 1)) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e != cudaSuccess) return e;
    attr_set_mask |= uint64_t(1) << (dev & 63);
  }
  Params p{};
  p.M = a.M;
  p.N = a.N;
  p.K = a.K;
  p.Mp = (a.M + 15) / 16 * 16;
  p.C = a.C;
  p.ldc = a.ldc;
  p.num_kb = (a.K + kKB - 1) / kKB;
  p.num_tiles = (a.N + kRowsW - 1) / kRowsW;
  p.units = static_cast<long long>(p.num_tiles) * p.num_kb;
  int cap = a.max_ctas > 0 ? a.max_ctas : sm_count();
  if (cap < 1) cap = 1;
  long long upc = (p.units + cap - 1) / cap;
  if (upc > 0x3fffffff) return cudaErrorInvalidValue;
  p.upc = static_cast<int>(upc);
  const int grid = static_cast<int>((p.units + p.upc - 1) / p.upc);
  p.stage_bytes = 2 * kWSubBytes + 2 * p.Mp * 128;
  p.stages = (kSmemLimit - 1024 - kCtlBytes) / p.stage_bytes;
  if (p.stages > kMaxStagesS) p.stages = kMaxStagesS;
  if (p.stages < 2) return cudaErrorInvalidValue;
  uint32_t cols = 32;
  while (cols < uint32_t(2 * p.Mp)) cols <<= 1;
  p.tmem_cols = cols;
  if (size_t(p.num_tiles) * 4 * sizeof(uint32_t) > kSplitkCounterBytes) return cudaErrorInvalidValue;
  void* ws = nullptr;
  cudaError_t e = gemm_library_workspace(kSplitkCounterBytes + size_t(grid) * 2 * p.Mp * kRowsW * sizeof(float), stream, &ws);
  if (e != cudaSuccess) return e;
  p.counters = static_cast<uint32_t*>(ws);
  p.partials = splitk_partials(ws);
  CUtensorMap tw, tx;
  if (!make_tmap(&tw, a.B, a.N, a.K, a.ldb, kRowsW)) return cudaErrorInvalidValue;
  if (!make_tmap(&tx, a.A, a.M, a.K, a.lda, p.Mp)) return cudaErrorInvalidValue;
  const int smem = p.stages * p.stage_bytes + 1024 + kCtlBytes;
  kernel<<<grid, kThreadsS, smem, stream>>>(tw, tx, p, status);
  return cudaGetLastError();
}

}  // namespace gemm_skinny

bool gemm_skinny_supported(const GemmArgs& a) { return a.mode == kGemmPlain && a.M >= 1 && a.M <= gemm_skinny::kMaxTokens; }

cudaError_t launch_gemm_skinny(const GemmArgs& a, DeviceStatus* status, cudaStream_t stream, gemm_detail::TmapFn make_tmap) {
  return a.fmt == 1 ? gemm_skinny::launch_fmt<__nv_bfloat16>(a, status, stream, make_tmap)
                    : gemm_skinny::launch_fmt<__half>(a, status, stream, make_tmap);
}

}  // namespace oob
