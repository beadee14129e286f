// Lowest-latency all-reduce for decode-sized messages: NO barrier and NO fence.  Every rank stores its input into
// piece `rank` of a staging area on all ranks as 8-byte cells {4 data bytes, 4 flag bytes}; the flag is the number
// of this call.  An 8-byte store arrives whole, so a receiver that polls a cell and sees this call's flag also sees its
// data: the receivers spin on the cells themselves and sum them in rank order (fp32) as they arrive.  What is left
// of the latency is the launch, one flight of the stores and the local sum.
//
// The staging area is used by this kernel only and holds two sets of cells; consecutive calls alternate between the
// sets (call counter on the device, so CUDA-graph replays alternate too).  A rank that has finished call k + 1 has seen
// every peer's cells of call k + 1, so every peer has started call k + 1 and therefore finished reading call k: the
// set of call k is free for call k + 2 without any barrier.  Flags only grow, and nothing else ever writes to the
// area (it is zeroed when it is allocated and whenever the call counter is reset), so a cell can never show the flag
// of a call that has not written it.  The 32-bit call number wraps after 2^32 calls; a cell can then alias only if
// it has not been written for a whole period and its first writer afterwards happens to carry exactly the old number.
//
// Cost: twice the bytes of the message per peer, which is why this is for messages of a few KiB to 64 KiB; above
// that the push kernel with one barrier (allreduce_push.cu) moves the plain bytes.
//
// Capability parity: the reference's fast one-shot all-reduce (src/comm/fast_multi_gpu_allreduce_sm90.cu:155-257) for
// messages up to 384 KiB uses three grid barriers and two rendezvous around bulk reduce-copies; NCCL's LL protocol
// is the model for the flag-in-data cells.
#include <cuda_runtime.h>

#include "../device/reduce.cuh"
#include "../device/sync.cuh"
#include "collectives.h"

namespace oob {
namespace {

constexpr int kLlThreads = 512;

__device__ __forceinline__ uint2 ld_cell(const void* p) {
  uint2 v;
  asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_cell(void* p, uint32_t data, uint32_t flag) {
  asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(data), "r"(flag) : "memory");
}
__device__ __forceinline__ void multimem_st_cell(void* mc, uint32_t data, uint32_t flag) {
  asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1, %2};" ::"l"(mc), "r"(data), "r"(flag) : "memory");
}

// One 32-bit word of the message as floats: two 16-bit elements or one fp32 element.
template <typename T>
__device__ __forceinline__ void word_to_float(uint32_t w, float& a, float& b) {
  if constexpr (sizeof(T) == 4) {
    a = __uint_as_float(w);
    b = 0.f;
  } else {
    a = PackTraits<T>::to_float(reinterpret_cast<const T*>(&w)[0]);
    b = PackTraits<T>::to_float(reinterpret_cast<const T*>(&w)[1]);
  }
}
template <typename T>
__device__ __forceinline__ uint32_t float_to_word(float a, float b) {
  if constexpr (sizeof(T) == 4) {
    return __float_as_uint(a);
  } else {
    uint32_t w;
    reinterpret_cast<T*>(&w)[0] = PackTraits<T>::from_float(a);
    reinterpret_cast<T*>(&w)[1] = PackTraits<T>::from_float(b);
    return w;
  }
}

// Word i of a local buffer of `count` elements that may start on any element boundary; elements past the end read 0.
template <typename T>
__device__ __forceinline__ uint32_t load_word(const char* base, size_t i, size_t count, bool aligned4) {
  if constexpr (sizeof(T) == 4) {
    return *reinterpret_cast<const uint32_t*>(base + i * 4);
  } else {
    if (aligned4 && 2 * i + 1 < count) return *reinterpret_cast<const uint32_t*>(base + i * 4);
    uint32_t w = 0;
    reinterpret_cast<unsigned short*>(&w)[0] = *reinterpret_cast<const unsigned short*>(base + i * 4);
    if (2 * i + 1 < count) reinterpret_cast<unsigned short*>(&w)[1] = *reinterpret_cast<const unsigned short*>(base + i * 4 + 2);
    return w;
  }
}
template <typename T>
__device__ __forceinline__ void store_word(char* base, size_t i, size_t count, bool aligned4, uint32_t w) {
  if constexpr (sizeof(T) == 4) {
    *reinterpret_cast<uint32_t*>(base + i * 4) = w;
  } else {
    if (aligned4 && 2 * i + 1 < count) {
      *reinterpret_cast<uint32_t*>(base + i * 4) = w;
      return;
    }
    *reinterpret_cast<unsigned short*>(base + i * 4) = reinterpret_cast<const unsigned short*>(&w)[0];
    if (2 * i + 1 < count) *reinterpret_cast<unsigned short*>(base + i * 4 + 2) = reinterpret_cast<const unsigned short*>(&w)[1];
  }
}

template <typename T, int OP, int NR, bool MC>
__global__ void __launch_bounds__(kLlThreads)
    allreduce_ll_kernel(CommCtx ctx_param, PeerPtrs staging, const char* in_local, size_t in_emu_stride, char* out_local,
                        size_t out_emu_stride, size_t count, size_t piece_bytes) {
  const CommCtx ctx = resolve_ctx(ctx_param);
  const int world = ctx.world, rank = ctx.rank;
  const char* src = in_local + in_emu_stride * blockIdx.y;
  char* dst = out_local + out_emu_stride * blockIdx.y;
  const bool src4 = (reinterpret_cast<uintptr_t>(src) & 3) == 0, dst4 = (reinterpret_cast<uintptr_t>(dst) & 3) == 0;
  const size_t words = (count * sizeof(T) + 3) / 4;
  const size_t per = (words + gridDim.x - 1) / gridDim.x;
  const size_t w0 = min(words, per * blockIdx.x), w1 = min(words, w0 + per);

  __shared__ uint32_t s_seq;
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    s_seq = ptx::ld_relaxed_sys(call_epoch_ptr(ctx, kLlCallSlot));
    s_ok = 1;
  }
  __syncthreads();
  const uint32_t seq = s_seq, flag = seq + 1u;  // never 0: the area starts zeroed
  const size_t set_off = size_t(seq & 1u) * size_t(world) * piece_bytes;
  const size_t my_piece = set_off + size_t(rank) * piece_bytes;

  // ---- store this block's words, flag attached, into piece `rank` on every other rank -----------------------------
  for (size_t i = w0 + threadIdx.x; i < w1; i += kLlThreads) {
    const uint32_t w = load_word<T>(src, i, count, src4);
    if constexpr (MC) {
      multimem_st_cell(static_cast<char*>(staging.mc) + my_piece + i * 8, w, flag);
    } else {
      for (int r = 1; r < world; ++r) st_cell(static_cast<char*>(staging.p[(rank + r) % world]) + my_piece + i * 8, w, flag);
    }
  }

  // ---- poll the peers' cells of the same words and sum in rank order -----------------------------------------------
  const char* mine = static_cast<const char*>(staging.p[rank]) + set_off;
  const uint64_t t0 = ptx::globaltimer_ns();
  bool ok = true;
  for (size_t i = w0 + threadIdx.x; i < w1 && ok; i += kLlThreads) {
    float a = 0.f, b = 0.f;
    if constexpr (NR > 0) {
      // All peers' cells of this word are requested at once and re-requested until each shows this call's flag.
      uint2 v[NR];
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        v[r] = make_uint2(0u, flag);
        if (r != rank) v[r] = ld_cell(mine + size_t(r) * piece_bytes + i * 8);
      }
      uint32_t spins = 0;
      while (true) {
        bool all = true;
#pragma unroll
        for (int r = 0; r < NR; ++r) all = all && (v[r].y == flag);
        if (all) break;
        if (++spins > 32) __nanosleep(20);
        if ((spins & 255u) == 0u) {
          if (ptx::globaltimer_ns() - t0 > ctx.timeout_ns) {
            int late = 0;
#pragma unroll
            for (int r = 0; r < NR; ++r)
              if (v[r].y != flag) late = r;
            report_error(ctx, kDevTimeoutCounter, late, flag, 0u, 44);
            ok = false;
            break;
          }
          if (*reinterpret_cast<volatile uint32_t*>(ctx.pad[rank] + kPadErrorFlagOffset) != 0) {
            ok = false;
            break;
          }
        }
#pragma unroll
        for (int r = 0; r < NR; ++r)
          if (v[r].y != flag) v[r] = ld_cell(mine + size_t(r) * piece_bytes + i * 8);
      }
      if (!ok) break;
      const uint32_t own = load_word<T>(src, i, count, src4);  // the own contribution never travels
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        float x, y;
        word_to_float<T>(r == rank ? own : v[r].x, x, y);
        if (r == 0) {
          a = x;
          b = y;
        } else {
          a = combine<OP>(a, x);
          b = combine<OP>(b, y);
        }
      }
    } else {
      for (int r = 0; r < world; ++r) {
        uint32_t w;
        if (r == rank) {
          w = load_word<T>(src, i, count, src4);
        } else {
          const char* cell = mine + size_t(r) * piece_bytes + i * 8;
          uint2 v = ld_cell(cell);
          uint32_t spins = 0;
          while (v.y != flag) {
            if (++spins > 32) __nanosleep(20);
            if ((spins & 255u) == 0u) {
              if (ptx::globaltimer_ns() - t0 > ctx.timeout_ns) {
                report_error(ctx, kDevTimeoutCounter, r, flag, v.y, 44);
                ok = false;
                break;
              }
              if (*reinterpret_cast<volatile uint32_t*>(ctx.pad[rank] + kPadErrorFlagOffset) != 0) {
                ok = false;
                break;
              }
            }
            v = ld_cell(cell);
          }
          if (!ok) break;
          w = v.x;
        }
        float x, y;
        word_to_float<T>(w, x, y);
        if (r == 0) {
          a = x;
          b = y;
        } else {
          a = combine<OP>(a, x);
          b = combine<OP>(b, y);
        }
      }
    }
    if (ok) store_word<T>(dst, i, count, dst4, float_to_word<T>(a, b));
  }
  if (!ok) s_ok = 0;
  __syncthreads();
  if (!s_ok) return;  // the call counter stays: recover() zeroes it together with the peers'

  // The block that finishes last moves the rank on to the next call number (and the other set of cells).
  if (threadIdx.x == 0) {
    uint32_t* ticket = call_epoch_ptr(ctx, kLlDoneSlot);
    if (atomicAdd(ticket, 1u) == gridDim.x - 1) {
      *ticket = 0;
      atomicAdd(call_epoch_ptr(ctx, kLlCallSlot), 1u);
      __threadfence();
    }
  }
}

template <typename K, typename... Args>
cudaError_t launch_ll(K kernel, const CommCtx& ctx, int ctas, cudaStream_t stream, Args... args) {
  if (ctx.emu_table != nullptr) {
    dim3 grid(ctas, ctx.world);
    CommCtx c = ctx;
    void* argv[] = {(void*)&c, (void*)&args...};
    return cudaLaunchCooperativeKernel((const void*)kernel, grid, dim3(kLlThreads), argv, 0, stream);
  }
  kernel<<<dim3(ctas, 1), kLlThreads, 0, stream>>>(ctx, args...);
  return cudaGetLastError();
}

template <typename T, int OP, int NR>
cudaError_t ll_dispatch_mc(const CommCtx& ctx, bool mc, const PeerPtrs& st, const char* in, size_t in_stride, char* out,
                           size_t out_stride, size_t count, size_t piece, int ctas, cudaStream_t stream) {
  if (mc) return launch_ll(allreduce_ll_kernel<T, OP, NR, true>, ctx, ctas, stream, st, in, in_stride, out, out_stride, count, piece);
  return launch_ll(allreduce_ll_kernel<T, OP, NR, false>, ctx, ctas, stream, st, in, in_stride, out, out_stride, count, piece);
}

template <typename T, int OP>
cudaError_t ll_dispatch_world(const CommCtx& ctx, bool mc, const PeerPtrs& st, const char* in, size_t in_stride, char* out,
                              size_t out_stride, size_t count, size_t piece, int ctas, cudaStream_t stream) {
  switch (ctx.world) {
    case 2:
      return ll_dispatch_mc<T, OP, 2>(ctx, mc, st, in, in_stride, out, out_stride, count, piece, ctas, stream);
    case 4:
      return ll_dispatch_mc<T, OP, 4>(ctx, mc, st, in, in_stride, out, out_stride, count, piece, ctas, stream);
    case 8:
      return ll_dispatch_mc<T, OP, 8>(ctx, mc, st, in, in_stride, out, out_stride, count, piece, ctas, stream);
    default:
      return ll_dispatch_mc<T, OP, 0>(ctx, mc, st, in, in_stride, out, out_stride, count, piece, ctas, stream);
  }
}

template <typename T>
cudaError_t ll_dispatch_op(int op, const CommCtx& ctx, bool mc, const PeerPtrs& st, const char* in, size_t in_stride,
                           char* out, size_t out_stride, size_t count, size_t piece, int ctas, cudaStream_t stream) {
  switch (op) {
    case kSum:
      return ll_dispatch_world<T, kSum>(ctx, mc, st, in, in_stride, out, out_stride, count, piece, ctas, stream);
    case kMin:
      return ll_dispatch_world<T, kMin>(ctx, mc, st, in, in_stride, out, out_stride, count, piece, ctas, stream);
    case kMax:
      return ll_dispatch_world<T, kMax>(ctx, mc, st, in, in_stride, out, out_stride, count, piece, ctas, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace

// `piece_bytes` (a multiple of 16, at least 2 x the message rounded up to whole words) is the distance between the
// ranks' pieces; the staging area holds two sets of world * piece_bytes, is zeroed when it is allocated and is written
// by this kernel only.
cudaError_t launch_allreduce_ll(const CommCtx& ctx, int dtype, int op, bool use_mc, const PeerPtrs& staging,
                                size_t piece_bytes, const void* in_local, size_t in_emu_stride, void* out_local,
                                size_t out_emu_stride, size_t count, int max_ctas, cudaStream_t stream) {
  if (count == 0 || (piece_bytes & 15) != 0) return cudaErrorInvalidValue;
  const size_t esize = dtype == kF32 ? 4 : 2;
  const size_t words = (count * esize + 3) / 4;
  if (words * 8 > piece_bytes) return cudaErrorInvalidValue;
  if (use_mc && staging.mc == nullptr) return cudaErrorInvalidValue;
  // One word per thread while the CTAs last: a thread's words are polled one after the other, and at these sizes the
  // polls, not the bytes, are the cost (2-GPU measurement: 16 KiB on 2 CTAs 8.6 us, 1 KiB on one CTA 6.2 us).
  size_t need = (words + kLlThreads - 1) / kLlThreads;
  if (need < 1) need = 1;
  int ctas = max_ctas < 1 ? 16 : max_ctas;
  if (ctas > kMaxCommBlocks) ctas = kMaxCommBlocks;
  if (static_cast<size_t>(ctas) > need) ctas = static_cast<int>(need);
  const char* in = static_cast<const char*>(in_local);
  char* out = static_cast<char*>(out_local);
  switch (dtype) {
    case kF16:
      return ll_dispatch_op<__half>(op, ctx, use_mc, staging, in, in_emu_stride, out, out_emu_stride, count, piece_bytes, ctas, stream);
    case kBF16:
      return ll_dispatch_op<__nv_bfloat16>(op, ctx, use_mc, staging, in, in_emu_stride, out, out_emu_stride, count, piece_bytes, ctas,
                                           stream);
    case kF32:
      return ll_dispatch_op<float>(op, ctx, use_mc, staging, in, in_emu_stride, out, out_emu_stride, count, piece_bytes, ctas, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace oob
