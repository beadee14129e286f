// Decode-path kernels of the tensor-parallel model runner (sm_100a): rotary embedding + KV-cache write, SwiGLU,
// and grouped-query decode attention over a static cache.
//
// The attention kernel is bound by reading the cache once: a CTA handles one (sequence, KV head, key chunk); its
// four warps take 32-key tiles in turn (cp.async double buffering, per-warp buffers, XOR-swizzled rows), compute
// scores for all query heads of the KV group at once on the tensor cores (the <= 16 query heads are the M rows of
// m16n8k16 MMAs -- too few rows for a tcgen05 tile, which needs 64), keep an online softmax per row and accumulate
// P*V in fp32.  The warps' partial results are merged through shared memory; with several chunks per sequence a
// second small kernel merges the chunks.
//
// Capability parity: none of these exist in the reference (it delegates the model to vLLM,
// patches/vllm/v0.25.0/vllm/model_executor/models/qwen2.py); they make this library's own serving path a fixed
// sequence of kernels per layer.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <type_traits>

#include "../api/oob.h"
#include "../api/oob_model.h"
#include "../runtime/errors.h"

namespace oob {
namespace model {

// ---------------------------------------------------------------------------------------------------------------
// small helpers
// ---------------------------------------------------------------------------------------------------------------
template <typename T>
struct Cvt;
template <>
struct Cvt<__nv_bfloat16> {
  static __device__ __forceinline__ float2 unpack(uint32_t w) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
  }
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
};
template <>
struct Cvt<__half> {
  static __device__ __forceinline__ float2 unpack(uint32_t w) {
    return __half22float2(*reinterpret_cast<const __half2*>(&w));
  }
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
};

// ---------------------------------------------------------------------------------------------------------------
// RoPE + KV-cache write
// ---------------------------------------------------------------------------------------------------------------
// One thread per 16-byte unit (8 elements = 4 rotation pairs) of one head of one token.
template <typename T>
__global__ void rope_kv_write_kernel(oob_rope_args_t a, long long units) {
  const int upr = a.hd / 8;  // units per head
  const int heads = a.H + 2 * a.KV;
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
    const uint4 in = *reinterpret_cast<const uint4*>(static_cast<const T*>(a.qkv) + (token * heads + hh) * a.hd + c * 8);
    uint4 out = in;
    if (hh < a.H + a.KV) {
      const float4 cs = *reinterpret_cast<const float4*>(a.cos_table + p * (a.hd / 2) + c * 4);
      const float4 sn = *reinterpret_cast<const float4*>(a.sin_table + p * (a.hd / 2) + c * 4);
      const float cc[4] = {cs.x, cs.y, cs.z, cs.w}, ss[4] = {sn.x, sn.y, sn.z, sn.w};
      const uint32_t w[4] = {in.x, in.y, in.z, in.w};
      uint32_t o[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 x = Cvt<T>::unpack(w[i]);
        o[i] = Cvt<T>::pack(x.x * cc[i] - x.y * ss[i], x.x * ss[i] + x.y * cc[i]);
      }
      out = make_uint4(o[0], o[1], o[2], o[3]);
    }
    T* dst;
    if (hh < a.H) {
      dst = static_cast<T*>(a.q_out) + (token * a.H + hh) * a.hd + c * 8;
    } else {
      const int kvh = hh < a.H + a.KV ? hh - a.H : hh - a.H - a.KV;
      T* cache = static_cast<T*>(hh < a.H + a.KV ? a.k_cache : a.v_cache);
      dst = cache + (a.batch0 + b) * a.cache_batch_stride + (static_cast<long long>(kvh) * a.max_len + p) * a.hd + c * 8;
    }
    *reinterpret_cast<uint4*>(dst) = out;
  }
}

// ---------------------------------------------------------------------------------------------------------------
// SwiGLU
// ---------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void silu_mul_kernel(const T* gu, long long ld, T* out, long long units, int F) {
  const int upr = F / 8;
  for (long long u = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; u < units;
       u += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = u / upr;
    const int c = static_cast<int>(u % upr);
    const uint4 g = *reinterpret_cast<const uint4*>(gu + r * ld + c * 8);
    const uint4 v = *reinterpret_cast<const uint4*>(gu + r * ld + F + c * 8);
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, vw[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = Cvt<T>::unpack(gw[i]), y = Cvt<T>::unpack(vw[i]);
      o[i] = Cvt<T>::pack(x.x / (1.f + __expf(-x.x)) * y.x, x.y / (1.f + __expf(-x.y)) * y.y);
    }
    *reinterpret_cast<uint4*>(out + r * static_cast<long long>(F) + c * 8) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Decode attention
// ---------------------------------------------------------------------------------------------------------------
constexpr int kHD = 128;
constexpr int kTileKeys = 32;                      // keys per warp tile
constexpr int kAttnWarps = 4;
constexpr int kAttnThreads = kAttnWarps * 32;
constexpr int kRowBytes = kHD * 2;                 // 256
constexpr int kKvTileBytes = kTileKeys * kRowBytes;  // 8 KiB
// Pipeline depth per warp (tiles of K and V in flight or in use): 2 by default (128 KiB per CTA), 3 with
// OOB_ATTN_STAGES=3 (192 KiB: two tiles in flight while one is consumed).  The buffers are reused for the
// cross-warp merge.
__host__ __device__ constexpr int attn_warp_buf_bytes(int stages) { return stages * 2 * kKvTileBytes; }
__host__ __device__ constexpr int attn_smem_bytes(int stages) { return kAttnWarps * attn_warp_buf_bytes(stages); }
constexpr int kPartialStride = kHD + 2;            // fp32 words of one partial result: 128 values, max, sum

template <typename T>
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma_16816<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma_16816<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void cp_async_16(uint32_t smem_addr, const void* gptr) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr), "l"(gptr) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
// Byte offset of 16-byte unit `c` of key row `r` inside a tile (rows of 256 bytes, units XOR-swizzled by the row so
// that the eight rows of an ldmatrix hit different banks).
__device__ __forceinline__ uint32_t kv_off(int r, int c) { return uint32_t(r) * kRowBytes + (uint32_t(c ^ (r & 7)) << 4); }

struct AttnParams {
  const void* q;
  const void* k;
  const void* v;
  void* out;
  float* ws;
  const long long* pos_dev;
  int len;
  int B, H, KV, G;
  long long batch_stride;
  int max_len, batch0;
  int splits, chunk;
  float scale_log2;
};

template <typename T, int STAGES>
__global__ void __launch_bounds__(kAttnThreads, 1) attn_decode_kernel(AttnParams p) {
  constexpr int kWarpBufBytes = attn_warp_buf_bytes(STAGES);
  extern __shared__ __align__(128) uint8_t attn_smem[];
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.G;
  int L = p.pos_dev != nullptr ? static_cast<int>(*p.pos_dev) + 1 : p.len;
  if (L > p.max_len) L = p.max_len;
  if (L < 1) L = 1;
  const int start = split * p.chunk;
  const int end = min(L, start + p.chunk);
  const int h0 = kvh * G;

  if (start >= end) {
    // No keys in this chunk (only with splits > 1): a neutral partial.
    if (threadIdx.x < G) {
      float* w = p.ws + ((static_cast<long long>(b) * p.H + h0 + threadIdx.x) * p.splits + split) * kPartialStride;
      w[kHD] = -INFINITY;
      w[kHD + 1] = 0.f;
    }
    return;
  }

  // ---- Q fragments (A operand, 16 x 128; rows >= G are zero) ----
  const int row0 = lane >> 2, colp = (lane & 3) * 2;
  uint32_t qa[8][4];
  {
    const T* qb = static_cast<const T*>(p.q) + (static_cast<long long>(b) * p.H + h0) * kHD;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const int c0 = ks * 16 + colp;
      qa[ks][0] = row0 < G ? *reinterpret_cast<const uint32_t*>(qb + row0 * kHD + c0) : 0u;
      qa[ks][1] = row0 + 8 < G ? *reinterpret_cast<const uint32_t*>(qb + (row0 + 8) * kHD + c0) : 0u;
      qa[ks][2] = row0 < G ? *reinterpret_cast<const uint32_t*>(qb + row0 * kHD + c0 + 8) : 0u;
      qa[ks][3] = row0 + 8 < G ? *reinterpret_cast<const uint32_t*>(qb + (row0 + 8) * kHD + c0 + 8) : 0u;
    }
  }

  const T* kbase = static_cast<const T*>(p.k) + (p.batch0 + b) * p.batch_stride + static_cast<long long>(kvh) * p.max_len * kHD;
  const T* vbase = static_cast<const T*>(p.v) + (p.batch0 + b) * p.batch_stride + static_cast<long long>(kvh) * p.max_len * kHD;
  uint8_t* wbuf = attn_smem + warp * kWarpBufBytes;
  const uint32_t wbuf_u32 = static_cast<uint32_t>(__cvta_generic_to_shared(wbuf));

  const int ntiles_total = (end - start + kTileKeys - 1) / kTileKeys;
  const int my_tiles = ntiles_total > warp ? (ntiles_total - warp + kAttnWarps - 1) / kAttnWarps : 0;

  auto issue_tile = [&](int i, int stage) {
    const int key0 = start + (warp + i * kAttnWarps) * kTileKeys;
    const uint32_t ks = wbuf_u32 + stage * 2 * kKvTileBytes, vs = ks + kKvTileBytes;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int unit = j * 32 + lane;  // 512 units of 16 bytes per tile
      const int r = unit >> 4, c = unit & 15;
      int key = key0 + r;
      if (key > end - 1) key = end - 1;  // masked later; the address stays inside the written part of the cache
      cp_async_16(ks + kv_off(r, c), kbase + static_cast<long long>(key) * kHD + c * 8);
      cp_async_16(vs + kv_off(r, c), vbase + static_cast<long long>(key) * kHD + c * 8);
    }
  };

  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  // One commit group per tile slot, empty when there is no tile: the group count is then the same for every warp
  // and wait<STAGES - 1> always means "tile i has landed".
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < my_tiles) issue_tile(s, s);
    cp_async_commit();
  }
  for (int i = 0; i < my_tiles; ++i) {
    const int stage = i % STAGES;
    if (i + STAGES - 1 < my_tiles) issue_tile(i + STAGES - 1, (i + STAGES - 1) % STAGES);
    cp_async_commit();
    cp_async_wait<STAGES - 1>();
    __syncwarp();
    const int key0 = start + (warp + i * kAttnWarps) * kTileKeys;
    const uint32_t ks = wbuf_u32 + stage * 2 * kKvTileBytes, vs = ks + kKvTileBytes;

    // ---- S = Q K^T for 32 keys ----
    float s[4][4];
#pragma unroll
    for (int nb = 0; nb < 4; ++nb) {
      s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;
#pragma unroll
      for (int kp = 0; kp < 4; ++kp) {
        uint32_t r[4];
        ldmatrix_x4(r, ks + kv_off(nb * 8 + (lane & 7), kp * 4 + (lane >> 3)));
        mma_16816<T>(s[nb], qa[2 * kp], r[0], r[1]);
        mma_16816<T>(s[nb], qa[2 * kp + 1], r[2], r[3]);
      }
    }
    // ---- mask, online softmax ----
    float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nb = 0; nb < 4; ++nb) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key0 + nb * 8 + colp + (e & 1);
        const float v = key < end ? s[nb][e] * p.scale_log2 : -INFINITY;
        s[nb][e] = v;
        tmax[e >> 1] = fmaxf(tmax[e >> 1], v);
      }
    }
    float corr[2], m_use[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 1));
      tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 2));
      const float m_new = fmaxf(m_run[h], tmax[h]);
      m_use[h] = m_new == -INFINITY ? 0.f : m_new;
      corr[h] = exp2f(m_run[h] - m_use[h]);  // 0 when nothing has been seen yet
      m_run[h] = m_new;
      l_run[h] *= corr[h];
    }
#pragma unroll
    for (int nb = 0; nb < 4; ++nb) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float pv = exp2f(s[nb][e] - m_use[e >> 1]);
        s[nb][e] = pv;
        l_run[e >> 1] += pv;
      }
    }
#pragma unroll
    for (int i2 = 0; i2 < 16; ++i2) {
      o[i2][0] *= corr[0];
      o[i2][1] *= corr[0];
      o[i2][2] *= corr[1];
      o[i2][3] *= corr[1];
    }
    // ---- O += P V ----
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
      uint32_t pa[4];
      pa[0] = Cvt<T>::pack(s[2 * kk][0], s[2 * kk][1]);
      pa[1] = Cvt<T>::pack(s[2 * kk][2], s[2 * kk][3]);
      pa[2] = Cvt<T>::pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      pa[3] = Cvt<T>::pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int dp = 0; dp < 8; ++dp) {
        uint32_t r[4];
        const int j = lane >> 3;
        ldmatrix_x4_trans(r, vs + kv_off(kk * 16 + (j & 1) * 8 + (lane & 7), dp * 2 + (j >> 1)));
        mma_16816<T>(o[2 * dp], pa, r[0], r[1]);
        mma_16816<T>(o[2 * dp + 1], pa, r[2], r[3]);
      }
    }
    __syncwarp();  // every lane is done with this stage before the next iteration's copies overwrite it
  }
  cp_async_wait<0>();
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
  __syncthreads();  // all warps are done with their tile buffers: reuse shared memory for the merge

  // ---- cross-warp merge: [warp][16 rows][128] fp32 values, then [warp][16] max and sum ----
  float* mo = reinterpret_cast<float*>(attn_smem);
  float* mm = mo + kAttnWarps * 16 * kHD;
  float* ml = mm + kAttnWarps * 16;
#pragma unroll
  for (int nb = 0; nb < 16; ++nb) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int row = row0 + (e >> 1) * 8, col = nb * 8 + colp + (e & 1);
      mo[(warp * 16 + row) * kHD + col] = o[nb][e];
    }
  }
  if ((lane & 3) == 0) {
    mm[warp * 16 + row0] = m_run[0];
    mm[warp * 16 + row0 + 8] = m_run[1];
    ml[warp * 16 + row0] = l_run[0];
    ml[warp * 16 + row0 + 8] = l_run[1];
  }
  __syncthreads();
  const int d = threadIdx.x;  // 128 threads = 128 dims
  for (int g = 0; g < G; ++g) {
    float m_tot = -INFINITY;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) m_tot = fmaxf(m_tot, mm[w * 16 + g]);
    float acc = 0.f, l_tot = 0.f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) {
      const float mw = mm[w * 16 + g];
      const float f = mw == -INFINITY ? 0.f : exp2f(mw - m_tot);
      acc += f * mo[(w * 16 + g) * kHD + d];
      l_tot += f * ml[w * 16 + g];
    }
    const long long hrow = static_cast<long long>(b) * p.H + h0 + g;
    if (p.splits == 1) {
      const float y = acc / l_tot;
      T* dst = static_cast<T*>(p.out) + hrow * kHD + d;
      if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        *dst = __float2bfloat16_rn(y);
      } else {
        *dst = __float2half_rn(y);
      }
    } else {
      float* w = p.ws + (hrow * p.splits + split) * kPartialStride;
      w[d] = acc;
      if (d == 0) {
        w[kHD] = m_tot;
        w[kHD + 1] = l_tot;
      }
    }
  }
}

// Merges the key chunks of one (sequence, head): grid = B * H, 128 threads.
template <typename T>
__global__ void attn_combine_kernel(const float* ws, void* out, int splits) {
  const long long hrow = blockIdx.x;
  const int d = threadIdx.x;
  const float* w = ws + hrow * splits * kPartialStride;
  float m_tot = -INFINITY;
  for (int s = 0; s < splits; ++s) m_tot = fmaxf(m_tot, w[s * kPartialStride + kHD]);
  float acc = 0.f, l_tot = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = w[s * kPartialStride + kHD];
    if (ms == -INFINITY) continue;  // empty chunk: its values were never written
    const float f = exp2f(ms - m_tot);
    acc += f * w[s * kPartialStride + d];
    l_tot += f * w[s * kPartialStride + kHD + 1];
  }
  const float y = acc / l_tot;
  T* dst = static_cast<T*>(out) + hrow * kHD + d;
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    *dst = __float2bfloat16_rn(y);
  } else {
    *dst = __float2half_rn(y);
  }
}

int sm_count_model() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

template <typename T, int STAGES>
cudaError_t launch_attn_stages(const AttnParams& p, cudaStream_t stream) {
  static bool attr_done[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_done[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<T, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         attn_smem_bytes(STAGES));
    if (e != cudaSuccess) return e;
    attr_done[dev & 63] = true;
  }
  attn_decode_kernel<T, STAGES><<<dim3(p.splits, p.KV, p.B), kAttnThreads, attn_smem_bytes(STAGES), stream>>>(p);
  return cudaGetLastError();
}

template <typename T>
cudaError_t launch_attn(const AttnParams& p, cudaStream_t stream) {
  static const bool three_stages = [] {
    const char* v = getenv("OOB_ATTN_STAGES");
    return v != nullptr && v[0] == '3';
  }();
  cudaError_t e = three_stages ? launch_attn_stages<T, 3>(p, stream) : launch_attn_stages<T, 2>(p, stream);
  if (e != cudaSuccess) return e;
  if (p.splits > 1) {
    attn_combine_kernel<T><<<p.B * p.H, kHD, 0, stream>>>(p.ws, p.out, p.splits);
    e = cudaGetLastError();
  }
  return e;
}

}  // namespace model
}  // namespace oob

using namespace oob;
using namespace oob::model;

extern "C" {

int oob_rope_kv_write(const oob_rope_args_t* a, void* stream) {
  if (a == nullptr) return set_error(OOB_ERR_INVALID, "null argument");
  if (a->dtype != OOB_F16 && a->dtype != OOB_BF16) return set_error(OOB_ERR_INVALID, "dtype must be fp16 or bf16");
  if (a->B <= 0 || a->T <= 0 || a->H <= 0 || a->KV <= 0 || a->hd <= 0 || a->hd % 8 != 0)
    return set_error(OOB_ERR_INVALID, "bad RoPE shape");
  if (a->qkv == nullptr || a->q_out == nullptr || a->k_cache == nullptr || a->v_cache == nullptr ||
      a->cos_table == nullptr || a->sin_table == nullptr)
    return set_error(OOB_ERR_INVALID, "null pointer");
  if (a->batch0 < 0 || a->max_len <= 0 || a->cache_batch_stride < int64_t(a->KV) * a->max_len * a->hd)
    return set_error(OOB_ERR_INVALID, "bad cache geometry");
  if (a->pos_dev == nullptr && (a->pos0 < 0 || a->pos0 + a->T > a->max_len))
    return set_error(OOB_ERR_INVALID, "positions outside the cache");
  const uintptr_t align = reinterpret_cast<uintptr_t>(a->qkv) | reinterpret_cast<uintptr_t>(a->q_out) |
                          reinterpret_cast<uintptr_t>(a->k_cache) | reinterpret_cast<uintptr_t>(a->v_cache) |
                          reinterpret_cast<uintptr_t>(a->cos_table) | reinterpret_cast<uintptr_t>(a->sin_table);
  if (align & 15) return set_error(OOB_ERR_INVALID, "pointers must be 16-byte aligned");
  if ((a->cache_batch_stride % 8) != 0) return set_error(OOB_ERR_INVALID, "cache stride must be a multiple of 8 elements");
  const long long units = static_cast<long long>(a->B) * a->T * (a->H + 2 * a->KV) * (a->hd / 8);
  const int threads = 256;
  long long blocks = (units + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (a->dtype == OOB_BF16)
    rope_kv_write_kernel<__nv_bfloat16><<<static_cast<int>(blocks), threads, 0, s>>>(*a, units);
  else
    rope_kv_write_kernel<__half><<<static_cast<int>(blocks), threads, 0, s>>>(*a, units);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "rope_kv_write launch");
  return OOB_OK;
}

int oob_silu_mul(int dtype, const void* gu, int64_t ld_gu, void* out, int rows, int F, void* stream) {
  if (dtype != OOB_F16 && dtype != OOB_BF16) return set_error(OOB_ERR_INVALID, "dtype must be fp16 or bf16");
  if (gu == nullptr || out == nullptr || rows <= 0 || F <= 0 || F % 8 != 0 || ld_gu < 2 * int64_t(F) || ld_gu % 8 != 0)
    return set_error(OOB_ERR_INVALID, "bad SwiGLU arguments");
  if ((reinterpret_cast<uintptr_t>(gu) | reinterpret_cast<uintptr_t>(out)) & 15)
    return set_error(OOB_ERR_INVALID, "pointers must be 16-byte aligned");
  const long long units = static_cast<long long>(rows) * (F / 8);
  const int threads = 256;
  long long blocks = (units + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == OOB_BF16)
    silu_mul_kernel<__nv_bfloat16><<<static_cast<int>(blocks), threads, 0, s>>>(
        static_cast<const __nv_bfloat16*>(gu), ld_gu, static_cast<__nv_bfloat16*>(out), units, F);
  else
    silu_mul_kernel<__half><<<static_cast<int>(blocks), threads, 0, s>>>(static_cast<const __half*>(gu), ld_gu,
                                                                         static_cast<__half*>(out), units, F);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "silu_mul launch");
  return OOB_OK;
}

int oob_attn_decode_auto_splits(int B, int KV, int len_bound) {
  if (B <= 0 || KV <= 0 || len_bound <= 0) return 1;
  const int sms = 148;
  const long long ctas = static_cast<long long>(B) * KV;
  int s = static_cast<int>((2 * sms + ctas - 1) / ctas);  // aim at two CTAs' worth of work per SM
  const int max_by_len = (len_bound + 127) / 128;          // at least one pass of the four warps per chunk
  if (s > max_by_len) s = max_by_len;
  if (s > 32) s = 32;
  if (s < 1) s = 1;
  return s;
}

uint64_t oob_attn_decode_workspace_bytes(int B, int H, int splits) {
  if (splits <= 1) return 0;
  return uint64_t(B) * H * splits * kPartialStride * sizeof(float);
}

int oob_attn_decode(const oob_attn_decode_args_t* a, void* stream) {
  if (a == nullptr) return set_error(OOB_ERR_INVALID, "null argument");
  if (a->dtype != OOB_F16 && a->dtype != OOB_BF16) return set_error(OOB_ERR_INVALID, "dtype must be fp16 or bf16");
  if (a->B <= 0 || a->H <= 0 || a->KV <= 0 || a->H % a->KV != 0 || a->H / a->KV > 16)
    return set_error(OOB_ERR_INVALID, "bad head counts (at most 16 query heads per KV head)");
  if (a->q == nullptr || a->k_cache == nullptr || a->v_cache == nullptr || a->out == nullptr)
    return set_error(OOB_ERR_INVALID, "null pointer");
  if (a->max_len <= 0 || a->batch0 < 0 || a->cache_batch_stride < int64_t(a->KV) * a->max_len * kHD ||
      a->cache_batch_stride % 8 != 0)
    return set_error(OOB_ERR_INVALID, "bad cache geometry");
  if (a->pos_dev == nullptr && (a->len < 1 || a->len > a->max_len)) return set_error(OOB_ERR_INVALID, "bad context length");
  if ((reinterpret_cast<uintptr_t>(a->q) | reinterpret_cast<uintptr_t>(a->k_cache) |
       reinterpret_cast<uintptr_t>(a->v_cache) | reinterpret_cast<uintptr_t>(a->out)) & 15)
    return set_error(OOB_ERR_INVALID, "pointers must be 16-byte aligned");
  int bound = a->len_bound > 0 ? a->len_bound : a->max_len;
  if (bound > a->max_len) bound = a->max_len;
  if (a->pos_dev == nullptr && a->len > bound) bound = a->len;
  int splits = a->splits > 0 ? a->splits : oob_attn_decode_auto_splits(a->B, a->KV, bound);
  if (splits > 65535) return set_error(OOB_ERR_INVALID, "too many splits");
  if (splits > 1 && a->workspace == nullptr) return set_error(OOB_ERR_INVALID, "splits > 1 need a workspace");
  AttnParams p{};
  p.q = a->q;
  p.k = a->k_cache;
  p.v = a->v_cache;
  p.out = a->out;
  p.ws = a->workspace;
  p.pos_dev = reinterpret_cast<const long long*>(a->pos_dev);
  p.len = a->len;
  p.B = a->B;
  p.H = a->H;
  p.KV = a->KV;
  p.G = a->H / a->KV;
  p.batch_stride = a->cache_batch_stride;
  p.max_len = a->max_len;
  p.batch0 = a->batch0;
  p.splits = splits;
  // Keys per chunk: whole passes of the CTA (4 warps x 32 keys), covering `bound` keys.
  int chunk = (bound + splits - 1) / splits;
  chunk = (chunk + 127) / 128 * 128;
  p.chunk = chunk;
  p.scale_log2 = a->scale * 1.4426950408889634f;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = a->dtype == OOB_BF16 ? launch_attn<__nv_bfloat16>(p, s) : launch_attn<__half>(p, s);
  if (e != cudaSuccess) return cuda_fail(e, "attn_decode launch");
  return OOB_OK;
}

}  // extern "C"
