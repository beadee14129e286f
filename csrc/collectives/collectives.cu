// All-reduce, reduce-scatter and all-gather kernels for NVLink 5 / NVSwitch.
//
// One specialised kernel per (collective, algorithm); every block of a launch
// does: rank barrier -> move/reduce its stripe of 16-byte packs with plain
// 128-bit peer loads/stores or NVLS multimem instructions -> rank barrier.
// There is no copy-engine IR and no per-call planning: the host passes the
// peer pointer table, the element range and a CTA budget.
//
// Capability parity with the reference:
//   fast one-shot kernels          src/comm/fast_multi_gpu_allreduce_sm90.cu:155-257,
//                                  fast_multi_gpu_reduce_scatter_sm90.cu:182-326,
//                                  fast_multi_gpu_all_gather_sm90.cu:178-300
//   general task-executor kernel   src/comm/kernels/multi_gpu_window_task_executor.cuh:34-114
//   two-shot all-reduce plan       src/comm/plan/tma_multi_gpu_allreduce_plan.cuh:936-1049
//   CTA budget knob                src/comm/launch_config.h:8-232 (max_ctas)
// Differences by design: reductions accumulate in fp32 in rank order (the
// reference adds in the storage dtype in arrival order); 8 peers are native;
// every wait is bounded.
#include <cuda_runtime.h>
#include "../device/reduce.cuh"
#include "../device/sync.cuh"
#include "collectives.h"

namespace oob {

namespace {

constexpr int kThreads = 512;

// Packs per thread and loop iteration.  A P2P reduction of NR ranks holds NR loads per pack in registers, so
// wide worlds unroll less; multimem loads (one per pack) unroll most.
template <int NR, bool MC>
constexpr int kUnroll = MC ? 8 : (NR == 0 ? 1 : (NR >= 8 ? 2 : 4));

struct Stripe {
  size_t begin, end;  // pack indices handled by this block
};

// Contiguous stripe of [p0, p1) for this block; contiguous stripes keep each
// block's peer traffic sequential.
__device__ __forceinline__ Stripe block_stripe(size_t p0, size_t p1) {
  const size_t n = p1 - p0;
  const size_t per = (n + gridDim.x - 1) / gridDim.x;
  size_t b = p0 + per * blockIdx.x;
  size_t e = b + per;
  if (b > p1) b = p1;
  if (e > p1) e = p1;
  return {b, e};
}

template <typename T>
__device__ __forceinline__ char* at(void* base, size_t elem) {
  return static_cast<char*>(base) + elem * sizeof(T);
}

// ---------------------------------------------------------------------------
// All-reduce
// ---------------------------------------------------------------------------
// ALGO 0: one-shot P2P   every rank reduces the whole message into its local `out` (out != in)
// ALGO 1: two-shot P2P   rank r reduces shard r and pushes it into every rank's `out` (may alias in)
// ALGO 2: two-shot NVLS  multimem.ld_reduce shard r, multimem.st into every rank's `out`
// ALGO 3: one-shot NVLS  multimem.ld_reduce the whole message into local `out`
template <typename T, int OP, int NR, int ALGO>
__global__ void __launch_bounds__(kThreads) allreduce_kernel(CommCtx ctx_param, PeerPtrs in, PeerPtrs out,
                                                             char* out_local, size_t out_local_emu_stride,
                                                             size_t count) {
  const CommCtx ctx = resolve_ctx(ctx_param);
  const int world = ctx.world, rank = ctx.rank;
  constexpr size_t E = PackTraits<T>::kElems;
  const size_t packs = count / E;

  if (!rank_barrier(ctx, blockIdx.x, 10)) return;

  if constexpr (ALGO == 0 || ALGO == 3) {
    char* dst = out_local + out_local_emu_stride * blockIdx.y;
    // A destination that is not 16-byte aligned takes the element-wise path for everything.
    const size_t vec_packs = (reinterpret_cast<uintptr_t>(dst) & 15) == 0 ? packs : 0;
    const Stripe s = block_stripe(0, vec_packs);
    constexpr int U = kUnroll<NR, ALGO == 3>;
    for (size_t pb = s.begin + threadIdx.x; pb < s.end; pb += size_t(kThreads) * U) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t p = pb + size_t(u) * kThreads;
        if (p < s.end) {
          if constexpr (ALGO == 0)
            v[u] = reduce_pack_p2p<T, OP, NR>(in, p * 16, world);
          else
            v[u] = reduce_pack_mc<T, OP>(static_cast<const char*>(in.mc) + p * 16);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t p = pb + size_t(u) * kThreads;
        if (p < s.end) ptx::st_v4(dst + p * 16, v[u]);
      }
    }
    for (size_t e = vec_packs * E + blockIdx.x * size_t(kThreads) + threadIdx.x; e < count;
         e += size_t(gridDim.x) * kThreads)
      st_elem<T>(dst + e * sizeof(T), reduce_scalar_p2p<T, OP>(in, e * sizeof(T), world));
  } else {
    // Shard r = packs [r*P/n, (r+1)*P/n); the sub-pack tail belongs to the last rank.
    const size_t p0 = packs * rank / world, p1 = packs * (rank + 1) / world;
    const Stripe s = block_stripe(p0, p1);
    // U packs per thread and iteration: all their remote loads are issued before the first store, which is
    // what keeps enough bytes in flight to cover the NVLink round trip.
    constexpr int U = kUnroll<NR, ALGO == 2>;
    for (size_t pb = s.begin + threadIdx.x; pb < s.end; pb += size_t(kThreads) * U) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t p = pb + size_t(u) * kThreads;
        if (p < s.end) {
          if constexpr (ALGO == 1)
            v[u] = reduce_pack_p2p<T, OP, NR>(in, p * 16, world);
          else
            v[u] = reduce_pack_mc<T, OP>(static_cast<const char*>(in.mc) + p * 16);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t p = pb + size_t(u) * kThreads;
        if (p < s.end) {
          if constexpr (ALGO == 1) {
            if constexpr (NR > 0) {
#pragma unroll
              for (int r = 0; r < NR; ++r) ptx::st_v4(static_cast<char*>(out.p[(rank + r) % NR]) + p * 16, v[u]);
            } else {
              for (int r = 0; r < world; ++r)
                ptx::st_v4(static_cast<char*>(out.p[(rank + r) % world]) + p * 16, v[u]);
            }
          } else {
            ptx::multimem_st_v4(static_cast<char*>(out.mc) + p * 16, v[u]);
          }
        }
      }
    }
    if (rank == world - 1 && blockIdx.x == 0) {
      for (size_t e = packs * E + threadIdx.x; e < count; e += kThreads) {
        const T v = reduce_scalar_p2p<T, OP>(in, e * sizeof(T), world);
        for (int r = 0; r < world; ++r) st_elem<T>(static_cast<char*>(out.p[r]) + e * sizeof(T), v);
      }
    }
  }

  rank_barrier(ctx, blockIdx.x, 11);
}

// ---------------------------------------------------------------------------
// Reduce-scatter: rank r reduces elements [begin_r, end_r) of `in` (given by
// the uneven "base+1 for the first rem ranks" partition) into out_local, whose
// element 0 corresponds to begin_r.  ALGO 0 = P2P pull, 1 = NVLS ld_reduce.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void partition(size_t count, int world, int r, size_t& b, size_t& e) {
  const size_t base = count / world, rem = count % world;
  b = base * r + (static_cast<size_t>(r) < rem ? r : rem);
  e = b + base + (static_cast<size_t>(r) < rem ? 1 : 0);
}

template <typename T, int OP, int NR, int ALGO>
__global__ void __launch_bounds__(kThreads) reduce_scatter_kernel(CommCtx ctx_param, PeerPtrs in, char* out_local,
                                                                  size_t out_local_emu_stride, size_t count) {
  const CommCtx ctx = resolve_ctx(ctx_param);
  const int world = ctx.world, rank = ctx.rank;
  constexpr size_t E = PackTraits<T>::kElems;
  size_t e0, e1;
  partition(count, world, rank, e0, e1);
  char* dst = out_local + out_local_emu_stride * blockIdx.y;  // element e maps to dst + (e - e0)

  if (!rank_barrier(ctx, blockIdx.x, 20)) return;

  // Packs are usable only when source and destination agree modulo 16 bytes.
  const bool vec_ok = ((reinterpret_cast<uintptr_t>(dst) - e0 * sizeof(T)) & 15) == 0;
  const RangeSplit<T> sp(e0, vec_ok ? e1 : e0);
  if (vec_ok) {
    const Stripe s = block_stripe(sp.head_end / E, sp.body_end / E);
    constexpr int U = kUnroll<NR, ALGO == 1>;
    for (size_t pb = s.begin + threadIdx.x; pb < s.end; pb += size_t(kThreads) * U) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t p = pb + size_t(u) * kThreads;
        if (p < s.end) {
          if constexpr (ALGO == 0)
            v[u] = reduce_pack_p2p<T, OP, NR>(in, p * 16, world);
          else
            v[u] = reduce_pack_mc<T, OP>(static_cast<const char*>(in.mc) + p * 16);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t p = pb + size_t(u) * kThreads;
        if (p < s.end) ptx::st_v4(dst + (p * E - e0) * sizeof(T), v[u]);
      }
    }
  }
  // Scalar head and tail (or everything, when the alignments disagree).
  {
    const size_t h0 = e0, h1 = vec_ok ? sp.head_end : e1;
    const size_t n = h1 - h0;
    for (size_t i = blockIdx.x * kThreads + threadIdx.x; i < n; i += size_t(gridDim.x) * kThreads)
      st_elem<T>(dst + i * sizeof(T), reduce_scalar_p2p<T, OP>(in, (h0 + i) * sizeof(T), world));
    if (vec_ok && blockIdx.x == 0) {
      for (size_t e = sp.body_end + threadIdx.x; e < e1; e += kThreads)
        st_elem<T>(dst + (e - e0) * sizeof(T), reduce_scalar_p2p<T, OP>(in, e * sizeof(T), world));
    }
  }

  rank_barrier(ctx, blockIdx.x, 21);
}

// ---------------------------------------------------------------------------
// All-gather: rank r contributes elements [begin_r, end_r) of the gathered
// buffer, read from src_local (element 0 = begin_r).
// ALGO 0: P2P push   store own shard into every rank's `out`
// ALGO 1: NVLS push  multimem.st own shard
// ALGO 2: P2P pull   `out` table holds every rank's *source* shard (registered); gather into dst_local
// ---------------------------------------------------------------------------
template <typename T, int ALGO>
__global__ void __launch_bounds__(kThreads) all_gather_kernel(CommCtx ctx_param, PeerPtrs out, const char* src_local,
                                                              size_t src_local_emu_stride, char* dst_local,
                                                              size_t dst_local_emu_stride, size_t count) {
  const CommCtx ctx = resolve_ctx(ctx_param);
  const int world = ctx.world, rank = ctx.rank;
  constexpr size_t E = PackTraits<T>::kElems;

  if (!rank_barrier(ctx, blockIdx.x, 30)) return;

  if constexpr (ALGO == 2) {
    // out.p[r] is rank r's registered source shard; gather all of them locally.
    char* dst = dst_local + dst_local_emu_stride * blockIdx.y;
    for (int i = 0; i < world; ++i) {
      const int r = (rank + i) % world;
      size_t e0, e1;
      partition(count, world, r, e0, e1);
      const char* src = static_cast<const char*>(out.p[r]);
      const bool vec_ok = ((e0 * sizeof(T)) & 15) == 0 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0;
      const size_t n = e1 - e0;
      const size_t packs = vec_ok ? n / E : 0;
      const Stripe s = block_stripe(0, packs);
      for (size_t p = s.begin + threadIdx.x; p < s.end; p += kThreads)
        ptx::st_v4(dst + e0 * sizeof(T) + p * 16, ptx::ld_nc_v4(src + p * 16));
      for (size_t e = packs * E + blockIdx.x * kThreads + threadIdx.x; e < n; e += size_t(gridDim.x) * kThreads)
        st_elem<T>(dst + (e0 + e) * sizeof(T), ld_elem_sys<T>(src + e * sizeof(T)));
    }
  } else {
    const char* src = src_local + src_local_emu_stride * blockIdx.y;
    size_t e0, e1;
    partition(count, world, rank, e0, e1);
    const bool vec_ok = ((reinterpret_cast<uintptr_t>(src) - e0 * sizeof(T)) & 15) == 0;
    const RangeSplit<T> sp(e0, vec_ok ? e1 : e0);
    if (vec_ok) {
      const Stripe s = block_stripe(sp.head_end / E, sp.body_end / E);
      for (size_t p = s.begin + threadIdx.x; p < s.end; p += kThreads) {
        const uint4 v = ptx::ld_nc_v4(src + (p * E - e0) * sizeof(T));
        if constexpr (ALGO == 1) {
          ptx::multimem_st_v4(static_cast<char*>(out.mc) + p * 16, v);
        } else {
          for (int r = 0; r < world; ++r) ptx::st_v4(static_cast<char*>(out.p[(rank + r) % world]) + p * 16, v);
        }
      }
    }
    // Scalar head / tail (or the whole shard when alignments disagree).
    auto scalar_range = [&](size_t a, size_t b) {
      for (size_t e = a + blockIdx.x * kThreads + threadIdx.x; e < b; e += size_t(gridDim.x) * kThreads) {
        const T v = *reinterpret_cast<const T*>(src + (e - e0) * sizeof(T));
        for (int r = 0; r < world; ++r) st_elem<T>(static_cast<char*>(out.p[r]) + e * sizeof(T), v);
      }
    };
    if (vec_ok) {
      scalar_range(e0, sp.head_end);
      scalar_range(sp.body_end, e1);
    } else {
      scalar_range(e0, e1);
    }
  }

  rank_barrier(ctx, blockIdx.x, 31);
}

// ---------------------------------------------------------------------------
// Host-side launchers
// ---------------------------------------------------------------------------
int clamp_ctas(int want, size_t packs) {
  size_t need = (packs + kThreads - 1) / kThreads;
  if (need < 1) need = 1;
  int c = want < 1 ? 1 : want;
  if (c > kMaxCommBlocks) c = kMaxCommBlocks;
  if (static_cast<size_t>(c) > need) c = static_cast<int>(need);
  return c;
}

template <typename K, typename... Args>
cudaError_t launch(K kernel, const CommCtx& ctx, int ctas, cudaStream_t stream, Args... args) {
  if (ctx.emu_table != nullptr) {
    // Emulated ranks wait on one another inside one launch: all blocks must be
    // resident, which a cooperative launch guarantees (or refuses).
    dim3 grid(ctas, ctx.world);
    CommCtx c = ctx;
    void* argv[] = {(void*)&c, (void*)&args...};
    return cudaLaunchCooperativeKernel((const void*)kernel, grid, dim3(kThreads), argv, 0, stream);
  }
  kernel<<<dim3(ctas, 1), kThreads, 0, stream>>>(ctx, args...);
  return cudaGetLastError();
}

template <typename T, int OP, int NR>
cudaError_t ar_dispatch_algo(int algo, const CommCtx& ctx, const PeerPtrs& in, const PeerPtrs& out, char* out_local,
                             size_t emu_stride, size_t count, int ctas, cudaStream_t stream) {
  switch (algo) {
    case kArOneShotP2P:
      return launch(allreduce_kernel<T, OP, NR, 0>, ctx, ctas, stream, in, out, out_local, emu_stride, count);
    case kArTwoShotP2P:
      return launch(allreduce_kernel<T, OP, NR, 1>, ctx, ctas, stream, in, out, out_local, emu_stride, count);
    case kArTwoShotNvls:
      return launch(allreduce_kernel<T, OP, 0, 2>, ctx, ctas, stream, in, out, out_local, emu_stride, count);
    case kArOneShotNvls:
      return launch(allreduce_kernel<T, OP, 0, 3>, ctx, ctas, stream, in, out, out_local, emu_stride, count);
  }
  return cudaErrorInvalidValue;
}

template <typename T, int OP>
cudaError_t ar_dispatch_world(int algo, const CommCtx& ctx, const PeerPtrs& in, const PeerPtrs& out, char* out_local,
                              size_t emu_stride, size_t count, int ctas, cudaStream_t stream) {
  switch (ctx.world) {
    case 2:
      return ar_dispatch_algo<T, OP, 2>(algo, ctx, in, out, out_local, emu_stride, count, ctas, stream);
    case 4:
      return ar_dispatch_algo<T, OP, 4>(algo, ctx, in, out, out_local, emu_stride, count, ctas, stream);
    case 8:
      return ar_dispatch_algo<T, OP, 8>(algo, ctx, in, out, out_local, emu_stride, count, ctas, stream);
    default:
      return ar_dispatch_algo<T, OP, 0>(algo, ctx, in, out, out_local, emu_stride, count, ctas, stream);
  }
}

template <typename T>
cudaError_t ar_dispatch_op(int op, int algo, const CommCtx& ctx, const PeerPtrs& in, const PeerPtrs& out,
                           char* out_local, size_t emu_stride, size_t count, int ctas, cudaStream_t stream) {
  switch (op) {
    case kSum:
      return ar_dispatch_world<T, kSum>(algo, ctx, in, out, out_local, emu_stride, count, ctas, stream);
    case kMin:
      return ar_dispatch_world<T, kMin>(algo, ctx, in, out, out_local, emu_stride, count, ctas, stream);
    case kMax:
      return ar_dispatch_world<T, kMax>(algo, ctx, in, out, out_local, emu_stride, count, ctas, stream);
  }
  return cudaErrorInvalidValue;
}

template <typename T, int OP>
cudaError_t rs_dispatch(int algo, const CommCtx& ctx, const PeerPtrs& in, char* out_local, size_t emu_stride,
                        size_t count, int ctas, cudaStream_t stream) {
  if (algo == kRsNvls) return launch(reduce_scatter_kernel<T, OP, 0, 1>, ctx, ctas, stream, in, out_local, emu_stride, count);
  switch (ctx.world) {
    case 2:
      return launch(reduce_scatter_kernel<T, OP, 2, 0>, ctx, ctas, stream, in, out_local, emu_stride, count);
    case 4:
      return launch(reduce_scatter_kernel<T, OP, 4, 0>, ctx, ctas, stream, in, out_local, emu_stride, count);
    case 8:
      return launch(reduce_scatter_kernel<T, OP, 8, 0>, ctx, ctas, stream, in, out_local, emu_stride, count);
    default:
      return launch(reduce_scatter_kernel<T, OP, 0, 0>, ctx, ctas, stream, in, out_local, emu_stride, count);
  }
}

template <typename T>
cudaError_t rs_dispatch_op(int op, int algo, const CommCtx& ctx, const PeerPtrs& in, char* out_local,
                           size_t emu_stride, size_t count, int ctas, cudaStream_t stream) {
  switch (op) {
    case kSum:
      return rs_dispatch<T, kSum>(algo, ctx, in, out_local, emu_stride, count, ctas, stream);
    case kMin:
      return rs_dispatch<T, kMin>(algo, ctx, in, out_local, emu_stride, count, ctas, stream);
    case kMax:
      return rs_dispatch<T, kMax>(algo, ctx, in, out_local, emu_stride, count, ctas, stream);
  }
  return cudaErrorInvalidValue;
}

template <typename T>
cudaError_t ag_dispatch(int algo, const CommCtx& ctx, const PeerPtrs& out, const char* src, size_t src_stride,
                        char* dst, size_t dst_stride, size_t count, int ctas, cudaStream_t stream) {
  switch (algo) {
    case kAgPushP2P:
      return launch(all_gather_kernel<T, 0>, ctx, ctas, stream, out, src, src_stride, dst, dst_stride, count);
    case kAgPushNvls:
      return launch(all_gather_kernel<T, 1>, ctx, ctas, stream, out, src, src_stride, dst, dst_stride, count);
    case kAgPullP2P:
      return launch(all_gather_kernel<T, 2>, ctx, ctas, stream, out, src, src_stride, dst, dst_stride, count);
  }
  return cudaErrorInvalidValue;
}

}  // namespace

cudaError_t launch_allreduce(const CommCtx& ctx, int dtype, int op, int algo, const PeerPtrs& in, const PeerPtrs& out,
                             void* out_local, size_t out_local_emu_stride, size_t count, int max_ctas,
                             cudaStream_t stream) {
  const bool nvls = (algo == kArTwoShotNvls || algo == kArOneShotNvls);
  if (nvls && (in.mc == nullptr || (algo == kArTwoShotNvls && out.mc == nullptr))) return cudaErrorInvalidValue;
  if (nvls && dtype == kF32 && op != kSum) return cudaErrorInvalidValue;
  const size_t esize = dtype == kF32 ? 4 : 2;
  size_t packs = count * esize / 16;
  if (algo == kArTwoShotP2P || algo == kArTwoShotNvls) packs = (packs + ctx.world - 1) / ctx.world;
  const int ctas = clamp_ctas(max_ctas, packs);
  char* ol = static_cast<char*>(out_local);
  switch (dtype) {
    case kF16:
      return ar_dispatch_op<__half>(op, algo, ctx, in, out, ol, out_local_emu_stride, count, ctas, stream);
    case kBF16:
      return ar_dispatch_op<__nv_bfloat16>(op, algo, ctx, in, out, ol, out_local_emu_stride, count, ctas, stream);
    case kF32:
      return ar_dispatch_op<float>(op, algo, ctx, in, out, ol, out_local_emu_stride, count, ctas, stream);
  }
  return cudaErrorInvalidValue;
}

cudaError_t launch_reduce_scatter(const CommCtx& ctx, int dtype, int op, int algo, const PeerPtrs& in,
                                  void* out_local, size_t out_local_emu_stride, size_t count, int max_ctas,
                                  cudaStream_t stream) {
  if (algo == kRsNvls && in.mc == nullptr) return cudaErrorInvalidValue;
  if (algo == kRsNvls && dtype == kF32 && op != kSum) return cudaErrorInvalidValue;
  const size_t esize = dtype == kF32 ? 4 : 2;
  const int ctas = clamp_ctas(max_ctas, (count * esize / 16 + ctx.world - 1) / ctx.world);
  char* ol = static_cast<char*>(out_local);
  switch (dtype) {
    case kF16:
      return rs_dispatch_op<__half>(op, algo, ctx, in, ol, out_local_emu_stride, count, ctas, stream);
    case kBF16:
      return rs_dispatch_op<__nv_bfloat16>(op, algo, ctx, in, ol, out_local_emu_stride, count, ctas, stream);
    case kF32:
      return rs_dispatch_op<float>(op, algo, ctx, in, ol, out_local_emu_stride, count, ctas, stream);
  }
  return cudaErrorInvalidValue;
}

cudaError_t launch_all_gather(const CommCtx& ctx, int dtype, int algo, const PeerPtrs& out, const void* src_local,
                              size_t src_local_emu_stride, void* dst_local, size_t dst_local_emu_stride,
                              size_t count, int max_ctas, cudaStream_t stream) {
  if (algo == kAgPushNvls && out.mc == nullptr) return cudaErrorInvalidValue;
  const size_t esize = dtype == kF32 ? 4 : 2;
  const size_t packs = count * esize / 16;
  const int ctas = clamp_ctas(max_ctas, algo == kAgPullP2P ? packs : (packs + ctx.world - 1) / ctx.world);
  const char* s = static_cast<const char*>(src_local);
  char* d = static_cast<char*>(dst_local);
  switch (dtype) {
    case kF16:
      return ag_dispatch<__half>(algo, ctx, out, s, src_local_emu_stride, d, dst_local_emu_stride, count, ctas, stream);
    case kBF16:
      return ag_dispatch<__nv_bfloat16>(algo, ctx, out, s, src_local_emu_stride, d, dst_local_emu_stride, count, ctas,
                                        stream);
    case kF32:
      return ag_dispatch<float>(algo, ctx, out, s, src_local_emu_stride, d, dst_local_emu_stride, count, ctas, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace oob
