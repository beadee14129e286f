// Epilogues that run in the kernel which sums the K splits of a split-K GEMM: since that kernel reads fp32 sums
// and may write anywhere, an elementwise op that follows the GEMM costs no launch and no round trip through a
// 16-bit intermediate.
//   SwiGLU     the GEMM's N = 2F columns are [gate | up]; the output is silu(gate) * up, [M, F]
//   RoPE + KV  the GEMM's columns are (H + 2 KV) heads of hd; query and key heads are rotated, queries go to
//              q_out, keys and values into the layer's cache (the stand-alone kernel of the same op is
//              rope_kv_write_kernel in csrc/model/decode_ops.cu)
// Both need a problem that launch_gemm splits (oob_gemm_plan_splits > 1), which every decode-step GEMM is.
//
// Capability parity: none in the reference (its GEMM epilogue only reorders and signals,
// src/epilogue/reorder_epilogue.h:324-595).
#pragma once
#include "../api/oob.h"
#include "../api/oob_model.h"
#include "gemm_kernel.cuh"

namespace oob {
namespace gemm_detail {

// Sum over the splits, in split order, of 8 consecutive columns (n % 8 == 0) of row m.
__device__ __forceinline__ void splitk_sum8(const float* __restrict__ partials, int m, int n, int tiles_n, int splits,
                                            float (&f)[8]) {
  const int tile_id = (m / kTileM) * tiles_n + n / kTileN;
  const float* src = partials + static_cast<size_t>(tile_id) * splits * (kTileM * kTileN) +
                     static_cast<size_t>(m % kTileM) * kTileN + (n % kTileN);
  float4 lo = make_float4(0.f, 0.f, 0.f, 0.f), hi = lo;
#pragma unroll 8
  for (int sp = 0; sp < splits; ++sp) {
    const float4 a0 = __ldcg(reinterpret_cast<const float4*>(src + static_cast<size_t>(sp) * (kTileM * kTileN)));
    const float4 a1 = __ldcg(reinterpret_cast<const float4*>(src + static_cast<size_t>(sp) * (kTileM * kTileN) + 4));
    lo.x += a0.x; lo.y += a0.y; lo.z += a0.z; lo.w += a0.w;
    hi.x += a1.x; hi.y += a1.y; hi.z += a1.z; hi.w += a1.w;
  }
  f[0] = lo.x; f[1] = lo.y; f[2] = lo.z; f[3] = lo.w;
  f[4] = hi.x; f[5] = hi.y; f[6] = hi.z; f[7] = hi.w;
}

template <typename T>
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
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
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// out[m, j] = silu(sum[m, j]) * sum[m, F + j]; F % 8 == 0, out rows 16-byte aligned (ld_out % 8 == 0).
template <typename T>
__global__ void splitk_reduce_swiglu_kernel(const float* __restrict__ partials, T* out, int M, int F, int ld_out,
                                            int tiles_n, int splits) {
  const int f8 = F / 8;
  const long long total = static_cast<long long>(M) * f8;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int m = static_cast<int>(i / f8), j = static_cast<int>(i % f8) * 8;
    float g[8], u[8], o[8];
    splitk_sum8(partials, m, j, tiles_n, splits, g);
    splitk_sum8(partials, m, F + j, tiles_n, splits, u);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = g[e] / (1.f + __expf(-g[e])) * u[e];
    *reinterpret_cast<uint4*>(out + static_cast<size_t>(m) * ld_out + j) = pack8<T>(o);
  }
}

// One thread per token and 16-byte unit (8 elements = 4 rotation pairs) of one head; same mapping and the same
// argument block as the stand-alone RoPE + KV-write kernel, with the GEMM's fp32 sums as the input.
template <typename T>
__global__ void splitk_reduce_rope_kv_kernel(const float* __restrict__ partials, oob_rope_args_t a, int tiles_n, int splits) {
  const int upr = a.hd / 8;
  const int heads = a.H + 2 * a.KV;
  const long long units = static_cast<long long>(a.B) * a.T * heads * upr;
  const long long pos_base = a.pos_dev != nullptr ? *a.pos_dev : static_cast<long long>(a.pos0);
  for (long long u = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; u < units;
       u += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(u % upr);
    const long long th = u / upr;
    const int hh = static_cast<int>(th % heads);
    const long long token = th / heads;
    const int b = static_cast<int>(token / a.T), t = static_cast<int>(token % a.T);
    long long p = pos_base + t;
    if (p < 0) p = 0;
    if (p > a.max_len - 1) p = a.max_len - 1;  // the host checks the range; never index outside the tables / cache
    float x[8];
    splitk_sum8(partials, static_cast<int>(token), hh * a.hd + c * 8, tiles_n, splits, x);
    if (hh < a.H + a.KV) {
      const float4 cs = *reinterpret_cast<const float4*>(a.cos_table + p * (a.hd / 2) + c * 4);
      const float4 sn = *reinterpret_cast<const float4*>(a.sin_table + p * (a.hd / 2) + c * 4);
      const float cc[4] = {cs.x, cs.y, cs.z, cs.w}, ss[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float x0 = x[2 * i], x1 = x[2 * i + 1];
        x[2 * i] = x0 * cc[i] - x1 * ss[i];
        x[2 * i + 1] = x0 * ss[i] + x1 * cc[i];
      }
    }
    T* dst;
    if (hh < a.H) {
      dst = static_cast<T*>(a.q_out) + (token * a.H + hh) * a.hd + c * 8;
    } else {
      const int kvh = hh < a.H + a.KV ? hh - a.H : hh - a.H - a.KV;
      T* cache = static_cast<T*>(hh < a.H + a.KV ? a.k_cache : a.v_cache);
      dst = cache + (a.batch0 + b) * a.cache_batch_stride + (static_cast<long long>(kvh) * a.max_len + p) * a.hd + c * 8;
    }
    *reinterpret_cast<uint4*>(dst) = pack8<T>(x);
  }
}

inline int reduce_grid(long long threads_total) {
  long long blocks = (threads_total + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

template <typename T>
cudaError_t launch_splitk_reduce_swiglu(const GemmArgs& a, int F, cudaStream_t stream) {
  const int tiles_n = (a.N + kTileN - 1) / kTileN;
  splitk_reduce_swiglu_kernel<T><<<reduce_grid(static_cast<long long>(a.M) * (F / 8)), 256, 0, stream>>>(
      splitk_partials(a.splitk_ws), static_cast<T*>(a.C), a.M, F, a.ldc, tiles_n, a.splits);
  return cudaGetLastError();
}

template <typename T>
cudaError_t launch_splitk_reduce_rope_kv(const GemmArgs& a, const oob_rope_args_t& r, cudaStream_t stream) {
  const int tiles_n = (a.N + kTileN - 1) / kTileN;
  const long long units = static_cast<long long>(r.B) * r.T * (r.H + 2 * r.KV) * (r.hd / 8);
  splitk_reduce_rope_kv_kernel<T><<<reduce_grid(units), 256, 0, stream>>>(splitk_partials(a.splitk_ws), r, tiles_n, a.splits);
  return cudaGetLastError();
}

}  // namespace gemm_detail
}  // namespace oob
