// 16-byte pack arithmetic with fp32 accumulation, and the element-range walker
// shared by the collective kernels.
//
// Capability parity: the reference reduces with element-wise atomics in the
// storage dtype at the destination (include/ooverlap/tma/tma_reduce.cuh:110-129,
// eight dtype/op functors in src/comm/pipeline/pipeline_tma_reduce.h:25-184).
// Here every reduction is a pull: the values of all ranks are loaded, summed
// in fp32 in a fixed rank order, and rounded once.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "comm_ctx.h"
#include "ptx.cuh"

namespace oob {

enum ReduceOp : int { kSum = 0, kMin = 1, kMax = 2 };
enum DType : int { kF16 = 0, kBF16 = 1, kF32 = 2 };

template <typename T>
struct PackTraits;
template <>
struct PackTraits<__half> {
  static constexpr int kElems = 8;
  static constexpr int kDType = kF16;
  __device__ static void unpack(const uint4& v, float (&f)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 t = __half22float2(h[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
  __device__ static uint4 pack(const float (&f)[8]) {
    uint4 v;
    __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    return v;
  }
  __device__ static float to_float(__half x) { return __half2float(x); }
  __device__ static __half from_float(float x) { return __float2half_rn(x); }
};
template <>
struct PackTraits<__nv_bfloat16> {
  static constexpr int kElems = 8;
  static constexpr int kDType = kBF16;
  __device__ static void unpack(const uint4& v, float (&f)[8]) {
    const uint32_t* w = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ static uint4 pack(const float (&f)[8]) {
    uint4 v;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return v;
  }
  __device__ static float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
  __device__ static __nv_bfloat16 from_float(float x) { return __float2bfloat16_rn(x); }
};
template <>
struct PackTraits<float> {
  static constexpr int kElems = 4;
  static constexpr int kDType = kF32;
  __device__ static void unpack(const uint4& v, float (&f)[4]) {
    f[0] = __uint_as_float(v.x);
    f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z);
    f[3] = __uint_as_float(v.w);
  }
  __device__ static uint4 pack(const float (&f)[4]) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
  __device__ static float to_float(float x) { return x; }
  __device__ static float from_float(float x) { return x; }
};

template <int OP>
__device__ __forceinline__ float combine(float a, float b) {
  if constexpr (OP == kSum) return a + b;
  if constexpr (OP == kMin) return fminf(a, b);
  return fmaxf(a, b);
}

// Reduce the 16-byte pack at byte offset `off` over all ranks with plain peer
// loads.  NR > 0 fixes the world size at compile time so that all loads are in
// flight together; NR == 0 is the generic loop.
template <typename T, int OP, int NR>
__device__ __forceinline__ void reduce_pack_p2p_f32(const PeerPtrs& in, size_t off, int world,
                                                    float (&acc)[PackTraits<T>::kElems]) {
  using PT = PackTraits<T>;
  constexpr int E = PT::kElems;
  if constexpr (NR > 0) {
    uint4 v[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) v[r] = ptx::ld_nc_v4(static_cast<const char*>(in.p[r]) + off);
    PT::unpack(v[0], acc);
#pragma unroll
    for (int r = 1; r < NR; ++r) {
      float f[E];
      PT::unpack(v[r], f);
#pragma unroll
      for (int i = 0; i < E; ++i) acc[i] = combine<OP>(acc[i], f[i]);
    }
  } else {
    uint4 v0 = ptx::ld_nc_v4(static_cast<const char*>(in.p[0]) + off);
    PT::unpack(v0, acc);
    for (int r = 1; r < world; ++r) {
      uint4 v = ptx::ld_nc_v4(static_cast<const char*>(in.p[r]) + off);
      float f[E];
      PT::unpack(v, f);
#pragma unroll
      for (int i = 0; i < E; ++i) acc[i] = combine<OP>(acc[i], f[i]);
    }
  }
}

template <typename T, int OP, int NR>
__device__ __forceinline__ uint4 reduce_pack_p2p(const PeerPtrs& in, size_t off, int world) {
  float acc[PackTraits<T>::kElems];
  reduce_pack_p2p_f32<T, OP, NR>(in, off, world, acc);
  return PackTraits<T>::pack(acc);
}

// Same reduction done inside the NVSwitch.  fp32 min/max have no multimem
// form; callers route them to the P2P path.
template <typename T, int OP>
__device__ __forceinline__ uint4 reduce_pack_mc(const void* mc_addr) {
  if constexpr (PackTraits<T>::kDType == kBF16) {
    if constexpr (OP == kSum) return ptx::multimem_ld_reduce_add_bf16x8(mc_addr);
    if constexpr (OP == kMin) return ptx::multimem_ld_reduce_min_bf16x8(mc_addr);
    return ptx::multimem_ld_reduce_max_bf16x8(mc_addr);
  } else if constexpr (PackTraits<T>::kDType == kF16) {
    if constexpr (OP == kSum) return ptx::multimem_ld_reduce_add_f16x8(mc_addr);
    if constexpr (OP == kMin) return ptx::multimem_ld_reduce_min_f16x8(mc_addr);
    return ptx::multimem_ld_reduce_max_f16x8(mc_addr);
  } else {
    return ptx::multimem_ld_reduce_add_f32x4(mc_addr);
  }
}

// Single-element accesses with system scope (head / tail of unaligned ranges).
template <typename T>
__device__ __forceinline__ T ld_elem_sys(const void* p) {
  if constexpr (sizeof(T) == 2) {
    unsigned short v;
    asm volatile("ld.relaxed.sys.global.u16 %0, [%1];" : "=h"(v) : "l"(p) : "memory");
    T out;
    *reinterpret_cast<unsigned short*>(&out) = v;
    return out;
  } else {
    uint32_t v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    T out;
    *reinterpret_cast<uint32_t*>(&out) = v;
    return out;
  }
}
template <typename T>
__device__ __forceinline__ void st_elem(void* p, T x) {
  if constexpr (sizeof(T) == 2) {
    unsigned short v = *reinterpret_cast<unsigned short*>(&x);
    asm volatile("st.global.u16 [%0], %1;" ::"l"(p), "h"(v) : "memory");
  } else {
    uint32_t v = *reinterpret_cast<uint32_t*>(&x);
    asm volatile("st.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
  }
}

template <typename T, int OP>
__device__ __forceinline__ T reduce_scalar_p2p(const PeerPtrs& in, size_t off, int world) {
  using PT = PackTraits<T>;
  float acc = PT::to_float(ld_elem_sys<T>(static_cast<const char*>(in.p[0]) + off));
  for (int r = 1; r < world; ++r)
    acc = combine<OP>(acc, PT::to_float(ld_elem_sys<T>(static_cast<const char*>(in.p[r]) + off)));
  return PT::from_float(acc);
}

// Splits the element range [e0, e1) of a buffer whose byte address at element
// 0 is 16-byte aligned into: scalar head, 16-byte body, scalar tail.
template <typename T>
struct RangeSplit {
  size_t head_end;   // elements [e0, head_end) are scalar
  size_t body_end;   // elements [head_end, body_end) are whole packs
  __device__ RangeSplit(size_t e0, size_t e1) {
    constexpr size_t E = PackTraits<T>::kElems;
    size_t a = (e0 + E - 1) / E * E;
    if (a > e1) a = e1;
    head_end = a;
    body_end = a + (e1 - a) / E * E;
  }
};

}  // namespace oob
