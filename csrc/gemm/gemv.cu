// C[M, N] = A[M, K] * B[N, K]^T for M <= 4 on the CUDA cores: the decode step of one to four sequences.
//
// With so few rows the tensor cores have nothing to amortise: the time is the time to read B once, and what
// decides it is how soon after launch every SM has enough loads in flight and how little happens after the last
// byte arrives.  So this kernel has no TMA ring, no TMEM, no split-K hand-off through global memory: a warp owns
// one weight row (or 1/KS of its K range), every lane keeps eight independent 16-byte loads of the row in flight,
// multiplies them with the matching 16 bytes of each activation row (L1-resident), and the partial sums meet in a
// warp shuffle and, for KS > 1, in shared memory.  fp32 accumulation, fixed summation order (deterministic).
//
// Capability parity: the small-M end of the reference's plain-GEMM dispatch
// (src/gemm/gemm_plain_sm90_dispatch.h:19-46), which it covers with CUTLASS tile instances.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../device/ptx.cuh"
#include "../device/reduce.cuh"
#include "gemm.h"

namespace oob {
namespace gemv {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kUnroll = 8;  // independent 16-byte weight loads per lane

template <typename T>
__device__ __forceinline__ float dot8(const uint4& w, const uint4& x) {
  const uint32_t wv[4] = {w.x, w.y, w.z, w.w}, xv[4] = {x.x, x.y, x.z, x.w};
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 a, b;
    if constexpr (PackTraits<T>::kDType == kBF16) {
      a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wv[i]));
      b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xv[i]));
    } else {
      a = __half22float2(*reinterpret_cast<const __half2*>(&wv[i]));
      b = __half22float2(*reinterpret_cast<const __half2*>(&xv[i]));
    }
    s = fmaf(a.x, b.x, s);
    s = fmaf(a.y, b.y, s);
  }
  return s;
}

// MB: activation rows handled (M <= MB); KS: warps that share one weight row (each takes 1/KS of the K range).
template <typename T, int MB, int KS>
__global__ void __launch_bounds__(kThreads) gemv_kernel(const T* __restrict__ A, int lda, const T* __restrict__ B, int ldb,
                                                        T* __restrict__ C, int ldc, int M, int N, int K) {
  constexpr int kRowsPerCta = kWarps / KS;
  __shared__ float red[kWarps][MB];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row_in_cta = warp / KS, ks = warp % KS;
  const int n = blockIdx.x * kRowsPerCta + row_in_cta;
  float acc[MB];
#pragma unroll
  for (int m = 0; m < MB; ++m) acc[m] = 0.f;
  if (n < N) {
    const T* w = B + static_cast<size_t>(n) * ldb;
    const int chunks = K / 8;  // 16-byte units of a row
    const int per = (chunks + KS - 1) / KS;
    const int c0 = ks * per, c1 = min(chunks, c0 + per);
    for (int c = c0 + lane; c < c1; c += 32 * kUnroll) {
      uint4 wv[kUnroll];
#pragma unroll
      for (int j = 0; j < kUnroll; ++j) {
        const int cc = c + j * 32;
        wv[j] = cc < c1 ? ptx::ld_nc_v4(w + static_cast<size_t>(cc) * 8) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int j = 0; j < kUnroll; ++j) {
        const int cc = c + j * 32;
        if (cc < c1) {
#pragma unroll
          for (int m = 0; m < MB; ++m) {
            if (m < M) {
              const uint4 xv = __ldg(reinterpret_cast<const uint4*>(A + static_cast<size_t>(m) * lda + static_cast<size_t>(cc) * 8));
              acc[m] += dot8<T>(wv[j], xv);
            }
          }
        }
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MB; ++m) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], o);
  }
  if (lane == 0) {
#pragma unroll
    for (int m = 0; m < MB; ++m) red[warp][m] = acc[m];
  }
  __syncthreads();
  if (threadIdx.x < kRowsPerCta * MB) {
    const int r = threadIdx.x / MB, m = threadIdx.x % MB;
    const int n2 = blockIdx.x * kRowsPerCta + r;
    if (n2 < N && m < M) {
      float s = 0.f;
#pragma unroll
      for (int k = 0; k < KS; ++k) s += red[r * KS + k][m];
      C[static_cast<size_t>(m) * ldc + n2] = PackTraits<T>::from_float(s);
    }
  }
}

template <typename T, int MB, int KS>
cudaError_t launch_one(const GemmArgs& a, cudaStream_t stream) {
  constexpr int kRowsPerCta = kWarps / KS;
  const int grid = (a.N + kRowsPerCta - 1) / kRowsPerCta;
  gemv_kernel<T, MB, KS><<<grid, kThreads, 0, stream>>>(static_cast<const T*>(a.A), a.lda, static_cast<const T*>(a.B), a.ldb,
                                                        static_cast<T*>(a.C), a.ldc, a.M, a.N, a.K);
  return cudaGetLastError();
}

template <typename T, int MB>
cudaError_t launch_ks(const GemmArgs& a, int ks, cudaStream_t stream) {
  switch (ks) {
    case 1:
      return launch_one<T, MB, 1>(a, stream);
    case 2:
      return launch_one<T, MB, 2>(a, stream);
    case 4:
      return launch_one<T, MB, 4>(a, stream);
    default:
      return launch_one<T, MB, 8>(a, stream);
  }
}

template <typename T>
cudaError_t launch_fmt(const GemmArgs& a, int ks, cudaStream_t stream) {
  if (a.M == 1) return launch_ks<T, 1>(a, ks, stream);
  if (a.M == 2) return launch_ks<T, 2>(a, ks, stream);
  return launch_ks<T, 4>(a, ks, stream);
}

}  // namespace gemv

// Warps per weight row: the smallest power of two that gives about four CTAs per SM, as long as every warp
// still has a few loads per lane to issue.
int gemv_k_split(int N, int K, int sms) {
  int ks = 1;
  while (ks < 8 && static_cast<long long>(N) * ks / gemv::kWarps < 4LL * sms && K / 8 / (ks * 2) >= 64) ks *= 2;
  return ks;
}

bool gemv_supported(const GemmArgs& a) { return a.mode == kGemmPlain && a.M >= 1 && a.M <= 4 && a.K % 8 == 0; }

cudaError_t launch_gemv(const GemmArgs& a, int sms, cudaStream_t stream) {
  const int ks = gemv_k_split(a.N, a.K, sms);
  return a.fmt == 1 ? gemv::launch_fmt<__nv_bfloat16>(a, ks, stream) : gemv::launch_fmt<__half>(a, ks, stream);
}

}  // namespace oob
