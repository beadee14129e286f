// Residual-add + RMSNorm, stand-alone and fused into the tail of the
// all-reduce / reduce-scatter: the rank that reduces a token row keeps it in
// registers, adds the residual, computes the row's mean square in fp32,
// scales by the norm weight and writes (or broadcasts) the result.  The
// partial sums never make a round trip through memory between the collective
// and the normalisation.
//
// Capability parity: the reference has a stand-alone fp16 RMSNorm and a
// variant that un-reorders the overlap GEMM's packed tiles
// (src/rmsnorm/rmsnorm.cuh:11-121); it has no residual add and no fusion with
// a collective.  Math here is fp32 with a caller-supplied eps.
#include <cuda_runtime.h>
#include "../device/reduce.cuh"
#include "../device/sync.cuh"
#include "collectives.h"

namespace oob {
namespace {

constexpr int kNormThreads = 256;

__device__ __forceinline__ float block_sum(float v) {
  __shared__ float s_part[kNormThreads / 32];
  __shared__ float s_total;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();  // protects s_part / s_total against the previous row's readers
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < kNormThreads / 32 ? s_part[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (threadIdx.x == 0) s_total = t;
  }
  __syncthreads();
  return s_total;
}

__device__ __forceinline__ void row_partition(int rows, int world, int r, int& b, int& e) {
  const int base = rows / world, rem = rows % world;
  b = base * r + (r < rem ? r : rem);
  e = b + base + (r < rem ? 1 : 0);
}

// PPT = 16-byte packs per thread (hidden <= PPT * 256 * 8).
template <typename T, int PPT, int NR, int ALGO>
__global__ void __launch_bounds__(kNormThreads) fused_norm_kernel(CommCtx ctx_param, NormArgs a) {
  const CommCtx ctx = resolve_ctx(ctx_param);
  const int world = ctx.world, rank = ctx.rank;
  using PT = PackTraits<T>;
  constexpr int E = 8;
  const int hidden = a.hidden;
  const int packs_per_row = hidden / E;
  const size_t row_bytes = size_t(hidden) * sizeof(T);

  constexpr bool kComm = ALGO != kNormLocal;
  constexpr bool kShard = (ALGO == kNormArTwoShot || ALGO == kNormArTwoShotNvls || ALGO == kNormRs || ALGO == kNormRsNvls);
  constexpr bool kRs = (ALGO == kNormRs || ALGO == kNormRsNvls);
  constexpr bool kMc = (ALGO == kNormArTwoShotNvls || ALGO == kNormRsNvls);
  constexpr bool kPush = (ALGO == kNormArTwoShot || ALGO == kNormArTwoShotNvls);

  if constexpr (kComm) {
    if (!rank_barrier(ctx, blockIdx.x, 40)) return;
  }

  int row0 = 0, row1 = a.rows;
  if constexpr (kShard) row_partition(a.rows, world, rank, row0, row1);

  const char* res = a.residual ? static_cast<const char*>(a.residual) + a.residual_emu_stride * blockIdx.y : nullptr;
  char* y_local = a.y_local ? static_cast<char*>(a.y_local) + a.y_local_emu_stride * blockIdx.y : nullptr;
  char* ro_local =
      a.res_out_local ? static_cast<char*>(a.res_out_local) + a.res_out_local_emu_stride * blockIdx.y : nullptr;
  const bool want_res_out = kPush ? (a.res_out.p[rank] != nullptr) : (ro_local != nullptr);

  // Norm weight for this thread's packs stays in registers across rows.
  float w[PPT][E];
#pragma unroll
  for (int j = 0; j < PPT; ++j) {
    const int p = threadIdx.x + j * kNormThreads;
    if (p < packs_per_row) {
      const uint4 wv = *reinterpret_cast<const uint4*>(static_cast<const char*>(a.weight) + size_t(p) * 16);
      PT::unpack(wv, w[j]);
    }
  }

  for (int row = row0 + blockIdx.x; row < row1; row += gridDim.x) {
    const size_t off = size_t(row) * row_bytes;
    // Residual and outputs of the RS form are indexed by the rank-local row.
    const size_t loff = kRs ? size_t(row - row0) * row_bytes : off;
    float v[PPT][E];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < PPT; ++j) {
      const int p = threadIdx.x + j * kNormThreads;
      if (p < packs_per_row) {
        if constexpr (!kComm) {
          PT::unpack(*reinterpret_cast<const uint4*>(static_cast<const char*>(a.x.p[rank]) + off + size_t(p) * 16),
                     v[j]);
        } else if constexpr (kMc) {
          PT::unpack(reduce_pack_mc<T, kSum>(static_cast<const char*>(a.x.mc) + off + size_t(p) * 16), v[j]);
        } else {
          // fp32 sum stays in registers: one rounding, after the residual add.
          reduce_pack_p2p_f32<T, kSum, NR>(a.x, off + size_t(p) * 16, world, v[j]);
        }
        if (res != nullptr) {
          const uint4 rv = ptx::ld_nc_v4(res + loff + size_t(p) * 16);
          float rf[E];
          PT::unpack(rv, rf);
#pragma unroll
          for (int i = 0; i < E; ++i) v[j][i] += rf[i];
          // The normalisation sees the residual stream as it is stored (rounded).
          if (want_res_out) {
            const uint4 ro = PT::pack(v[j]);
            PT::unpack(ro, v[j]);
          }
        }
        if (want_res_out) {
          const uint4 ro = PT::pack(v[j]);
          if constexpr (kPush) {
            if constexpr (kMc) {
              ptx::multimem_st_v4(static_cast<char*>(a.res_out.mc) + off + size_t(p) * 16, ro);
            } else {
              for (int r = 0; r < world; ++r)
                ptx::st_v4(static_cast<char*>(a.res_out.p[(rank + r) % world]) + off + size_t(p) * 16, ro);
            }
          } else {
            ptx::st_v4(ro_local + loff + size_t(p) * 16, ro);
          }
        }
#pragma unroll
        for (int i = 0; i < E; ++i) ss += v[j][i] * v[j][i];
      }
    }
    const float total = block_sum(ss);
    const float scale = rsqrtf(total / float(hidden) + a.eps);
#pragma unroll
    for (int j = 0; j < PPT; ++j) {
      const int p = threadIdx.x + j * kNormThreads;
      if (p < packs_per_row) {
        float o[E];
#pragma unroll
        for (int i = 0; i < E; ++i) o[i] = v[j][i] * scale * w[j][i];
        const uint4 yo = PT::pack(o);
        if constexpr (kPush) {
          if constexpr (kMc) {
            ptx::multimem_st_v4(static_cast<char*>(a.y.mc) + off + size_t(p) * 16, yo);
          } else {
            for (int r = 0; r < world; ++r)
              ptx::st_v4(static_cast<char*>(a.y.p[(rank + r) % world]) + off + size_t(p) * 16, yo);
          }
        } else {
          ptx::st_v4(y_local + loff + size_t(p) * 16, yo);
        }
      }
    }
  }

  if constexpr (kComm) rank_barrier(ctx, blockIdx.x, 41);
}

// One-barrier all-reduce + residual + RMSNorm for decode-sized messages.  Block b of every rank owns rows b, b + G, ...:
// it pushes its rows of this rank's partial sums into piece `rank` of the staging area on all ranks, meets block b of
// the other ranks once, and then sums the `world` pieces of its rows from LOCAL memory (fp32, rank order), adds the
// residual, normalises and writes the outputs locally.  Every rank normalises every row, so nothing has to be
// broadcast afterwards.  The staging area holds two sets of pieces that consecutive push calls alternate between
// (call counter on the device, shared with allreduce_push.cu), which is what makes a closing barrier unnecessary.
template <typename T, int PPT, int NR, bool MC>
__global__ void __launch_bounds__(kNormThreads) push_norm_kernel(CommCtx ctx_param, NormArgs a) {
  const CommCtx ctx = resolve_ctx(ctx_param);
  const int world = ctx.world, rank = ctx.rank;
  using PT = PackTraits<T>;
  constexpr int E = 8;
  const int packs_per_row = a.hidden / E;
  const size_t row_bytes = size_t(a.hidden) * sizeof(T);

  __shared__ uint32_t s_set;
  if (threadIdx.x == 0) s_set = ptx::ld_relaxed_sys(call_epoch_ptr(ctx, kPushCallSlot)) & 1u;
  __syncthreads();
  const size_t set_off = size_t(s_set) * size_t(world) * a.piece_bytes;
  const size_t my_piece = set_off + size_t(rank) * a.piece_bytes;

  const char* x = static_cast<const char*>(a.x.p[rank]);
  const char* res = a.residual ? static_cast<const char*>(a.residual) + a.residual_emu_stride * blockIdx.y : nullptr;
  char* y_local = static_cast<char*>(a.y_local) + a.y_local_emu_stride * blockIdx.y;
  char* ro_local =
      a.res_out_local ? static_cast<char*>(a.res_out_local) + a.res_out_local_emu_stride * blockIdx.y : nullptr;

  // ---- push this block's rows ------------------------------------------------------------------------------------
  for (int row = blockIdx.x; row < a.rows; row += gridDim.x) {
    const size_t off = size_t(row) * row_bytes;
#pragma unroll
    for (int j = 0; j < PPT; ++j) {
      const int p = threadIdx.x + j * kNormThreads;
      if (p < packs_per_row) {
        const uint4 v = *reinterpret_cast<const uint4*>(x + off + size_t(p) * 16);
        if constexpr (MC) {
          ptx::multimem_st_v4(static_cast<char*>(a.staging.mc) + my_piece + off + size_t(p) * 16, v);
        } else if constexpr (NR > 0) {
#pragma unroll
          for (int r = 1; r < NR; ++r)
            ptx::st_v4(static_cast<char*>(a.staging.p[(rank + r) % NR]) + my_piece + off + size_t(p) * 16, v);
        } else {
          for (int r = 1; r < world; ++r)
            ptx::st_v4(static_cast<char*>(a.staging.p[(rank + r) % world]) + my_piece + off + size_t(p) * 16, v);
        }
      }
    }
  }

  // Norm weight for this thread's packs (loaded while the pushes travel).
  float w[PPT][E];
#pragma unroll
  for (int j = 0; j < PPT; ++j) {
    const int p = threadIdx.x + j * kNormThreads;
    if (p < packs_per_row)
      PT::unpack(*reinterpret_cast<const uint4*>(static_cast<const char*>(a.weight) + size_t(p) * 16), w[j]);
  }

  if (!rank_barrier(ctx, blockIdx.x, 42)) return;

  // ---- sum the pieces of this block's rows from local memory, add the residual, normalise -------------------------
  // The own contribution is taken from x: a rank's own multicast store is not ordered with its loads, and without
  // the switch the own piece is not pushed at all.
  const char* mine = static_cast<const char*>(a.staging.p[rank]) + set_off;
  for (int row = blockIdx.x; row < a.rows; row += gridDim.x) {
    const size_t off = size_t(row) * row_bytes;
    float v[PPT][E];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < PPT; ++j) {
      const int p = threadIdx.x + j * kNormThreads;
      if (p < packs_per_row) {
        const size_t po = off + size_t(p) * 16;
#pragma unroll
        for (int i = 0; i < E; ++i) v[j][i] = 0.f;
        if constexpr (NR > 0) {
          uint4 raw[NR];
#pragma unroll
          for (int r = 0; r < NR; ++r)
            raw[r] = r == rank ? *reinterpret_cast<const uint4*>(x + po)
                               : ptx::ld_relaxed_sys_v4(mine + size_t(r) * a.piece_bytes + po);
#pragma unroll
          for (int r = 0; r < NR; ++r) {
            float f[E];
            PT::unpack(raw[r], f);
#pragma unroll
            for (int i = 0; i < E; ++i) v[j][i] += f[i];
          }
        } else {
          for (int r = 0; r < world; ++r) {
            float f[E];
            PT::unpack(r == rank ? *reinterpret_cast<const uint4*>(x + po)
                                 : ptx::ld_relaxed_sys_v4(mine + size_t(r) * a.piece_bytes + po),
                       f);
#pragma unroll
            for (int i = 0; i < E; ++i) v[j][i] += f[i];
          }
        }
        if (res != nullptr) {
          float rf[E];
          PT::unpack(ptx::ld_nc_v4(res + po), rf);
#pragma unroll
          for (int i = 0; i < E; ++i) v[j][i] += rf[i];
        }
        // The normalisation sees the residual stream as it is stored (rounded).
        const uint4 ro = PT::pack(v[j]);
        if (ro_local != nullptr) {
          PT::unpack(ro, v[j]);
          ptx::st_v4(ro_local + po, ro);
        } else if (res != nullptr) {
          PT::unpack(ro, v[j]);
        }
#pragma unroll
        for (int i = 0; i < E; ++i) ss += v[j][i] * v[j][i];
      }
    }
    const float total = block_sum(ss);
    const float scale = rsqrtf(total / float(a.hidden) + a.eps);
#pragma unroll
    for (int j = 0; j < PPT; ++j) {
      const int p = threadIdx.x + j * kNormThreads;
      if (p < packs_per_row) {
        float o[E];
#pragma unroll
        for (int i = 0; i < E; ++i) o[i] = v[j][i] * scale * w[j][i];
        ptx::st_v4(y_local + off + size_t(p) * 16, PT::pack(o));
      }
    }
  }

  // The block that finishes last moves the rank on to the other set of pieces.
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t* ticket = call_epoch_ptr(ctx, kPushDoneSlot);
    if (atomicAdd(ticket, 1u) == gridDim.x - 1) {
      *ticket = 0;
      atomicAdd(call_epoch_ptr(ctx, kPushCallSlot), 1u);
      __threadfence();
    }
  }
}

// The same op without any barrier, for the smallest messages (a few rows): the rows travel as 8-byte cells of 4 data
// bytes + the call number (the cell format, staging area and call counter of allreduce_ll.cu), and every rank spins
// on the cells of its peers before it sums and normalises.  Block b of every rank owns rows b, b + G, ...
template <typename T, int PPT, int NR>
__global__ void __launch_bounds__(kNormThreads) ll_norm_kernel(CommCtx ctx_param, NormArgs a) {
  const CommCtx ctx = resolve_ctx(ctx_param);
  const int world = ctx.world, rank = ctx.rank;
  using PT = PackTraits<T>;
  constexpr int E = 8;
  const int packs_per_row = a.hidden / E;
  const size_t row_bytes = size_t(a.hidden) * sizeof(T);

  __shared__ uint32_t s_seq;
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    s_seq = ptx::ld_relaxed_sys(call_epoch_ptr(ctx, kLlCallSlot));
    s_ok = 1;
  }
  __syncthreads();
  const uint32_t flag = s_seq + 1u;
  const size_t set_off = size_t(s_seq & 1u) * size_t(world) * a.piece_bytes;
  const size_t my_piece = set_off + size_t(rank) * a.piece_bytes;

  const char* x = static_cast<const char*>(a.x.p[rank]);
  const char* res = a.residual ? static_cast<const char*>(a.residual) + a.residual_emu_stride * blockIdx.y : nullptr;
  char* y_local = static_cast<char*>(a.y_local) + a.y_local_emu_stride * blockIdx.y;
  char* ro_local =
      a.res_out_local ? static_cast<char*>(a.res_out_local) + a.res_out_local_emu_stride * blockIdx.y : nullptr;

  // ---- store this block's rows as cells into piece `rank` of every other rank (a pack of 16 bytes = four cells) ----
  for (int row = blockIdx.x; row < a.rows; row += gridDim.x) {
    const size_t off = size_t(row) * row_bytes;
#pragma unroll
    for (int j = 0; j < PPT; ++j) {
      const int p = threadIdx.x + j * kNormThreads;
      if (p < packs_per_row) {
        const uint4 v = *reinterpret_cast<const uint4*>(x + off + size_t(p) * 16);
        const size_t cell0 = my_piece + 2 * (off + size_t(p) * 16);  // 8 bytes of cell per 4 bytes of data
        for (int r = 1; r < world; ++r) {
          char* dst = static_cast<char*>(a.staging.p[(rank + r) % world]) + cell0;
          asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(v.x), "r"(flag) : "memory");
          asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(dst + 8), "r"(v.y), "r"(flag) : "memory");
          asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(dst + 16), "r"(v.z), "r"(flag) : "memory");
          asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(dst + 24), "r"(v.w), "r"(flag) : "memory");
        }
      }
    }
  }

  float w[PPT][E];
#pragma unroll
  for (int j = 0; j < PPT; ++j) {
    const int p = threadIdx.x + j * kNormThreads;
    if (p < packs_per_row)
      PT::unpack(*reinterpret_cast<const uint4*>(static_cast<const char*>(a.weight) + size_t(p) * 16), w[j]);
  }

  // ---- spin on the peers' cells of this block's rows, sum in rank order, add the residual, normalise --------------
  const char* mine = static_cast<const char*>(a.staging.p[rank]) + set_off;
  const uint64_t t0 = ptx::globaltimer_ns();
  bool ok = true;
  for (int row = blockIdx.x; row < a.rows; row += gridDim.x) {
    const size_t off = size_t(row) * row_bytes;
    float v[PPT][E];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < PPT; ++j) {
      const int p = threadIdx.x + j * kNormThreads;
      if (p < packs_per_row) {
        const size_t po = off + size_t(p) * 16;
#pragma unroll
        for (int i = 0; i < E; ++i) v[j][i] = 0.f;
        for (int r = 0; r < world; ++r) {
          uint4 raw;
          if (r == rank) {
            raw = *reinterpret_cast<const uint4*>(x + po);  // the own contribution never travels
          } else {
            const char* cell = mine + size_t(r) * a.piece_bytes + 2 * po;
            uint4 c0, c1;  // two 16-byte loads = four cells {d, f, d, f}
            uint32_t spins = 0;
            while (true) {
              c0 = ptx::ld_relaxed_sys_v4(cell);
              c1 = ptx::ld_relaxed_sys_v4(cell + 16);
              if (c0.y == flag && c0.w == flag && c1.y == flag && c1.w == flag) break;
              if (++spins > 32) __nanosleep(20);
              if ((spins & 255u) == 0u) {
                if (ptx::globaltimer_ns() - t0 > ctx.timeout_ns) {
                  report_error(ctx, kDevTimeoutCounter, r, flag, c0.y, 45);
                  ok = false;
                  break;
                }
                if (*reinterpret_cast<volatile uint32_t*>(ctx.pad[rank] + kPadErrorFlagOffset) != 0) {
                  ok = false;
                  break;
                }
              }
            }
            if (!ok) break;
            raw = make_uint4(c0.x, c0.z, c1.x, c1.z);
          }
          float f[E];
          PT::unpack(raw, f);
#pragma unroll
          for (int i = 0; i < E; ++i) v[j][i] += f[i];
        }
        if (ok && res != nullptr) {
          float rf[E];
          PT::unpack(ptx::ld_nc_v4(res + po), rf);
#pragma unroll
          for (int i = 0; i < E; ++i) v[j][i] += rf[i];
        }
        const uint4 ro = PT::pack(v[j]);
        if (ro_local != nullptr) {
          PT::unpack(ro, v[j]);
          if (ok) ptx::st_v4(ro_local + po, ro);
        } else if (res != nullptr) {
          PT::unpack(ro, v[j]);
        }
#pragma unroll
        for (int i = 0; i < E; ++i) ss += v[j][i] * v[j][i];
      }
    }
    // Every thread reaches the block-wide sum, also after a timeout (the row is then not written).
    const float total = block_sum(ss);
    const float scale = rsqrtf(total / float(a.hidden) + a.eps);
#pragma unroll
    for (int j = 0; j < PPT; ++j) {
      const int p = threadIdx.x + j * kNormThreads;
      if (p < packs_per_row && ok) {
        float o[E];
#pragma unroll
        for (int i = 0; i < E; ++i) o[i] = v[j][i] * scale * w[j][i];
        ptx::st_v4(y_local + off + size_t(p) * 16, PT::pack(o));
      }
    }
  }
  if (!ok) s_ok = 0;
  __syncthreads();
  if (!s_ok) return;  // the call counter stays: recover() zeroes it together with the peers'
  if (threadIdx.x == 0) {
    uint32_t* ticket = call_epoch_ptr(ctx, kLlDoneSlot);
    if (atomicAdd(ticket, 1u) == gridDim.x - 1) {
      *ticket = 0;
      atomicAdd(call_epoch_ptr(ctx, kLlCallSlot), 1u);
      __threadfence();
    }
  }
}

template <typename K>
cudaError_t launch_k(K kernel, const CommCtx& ctx, int ctas, const NormArgs& a, cudaStream_t stream) {
  if (ctx.emu_table != nullptr) {
    dim3 grid(ctas, ctx.world);
    CommCtx c = ctx;
    NormArgs aa = a;
    void* argv[] = {(void*)&c, (void*)&aa};
    return cudaLaunchCooperativeKernel((const void*)kernel, grid, dim3(kNormThreads), argv, 0, stream);
  }
  kernel<<<dim3(ctas, 1), kNormThreads, 0, stream>>>(ctx, a);
  return cudaGetLastError();
}

template <typename T, int PPT, int NR>
cudaError_t dispatch_algo(int algo, const CommCtx& ctx, int ctas, const NormArgs& a, cudaStream_t stream) {
  switch (algo) {
    case kNormLocal:
      return launch_k(fused_norm_kernel<T, PPT, 0, kNormLocal>, ctx, ctas, a, stream);
    case kNormArOneShot:
      return launch_k(fused_norm_kernel<T, PPT, NR, kNormArOneShot>, ctx, ctas, a, stream);
    case kNormArTwoShot:
      return launch_k(fused_norm_kernel<T, PPT, NR, kNormArTwoShot>, ctx, ctas, a, stream);
    case kNormArTwoShotNvls:
      return launch_k(fused_norm_kernel<T, PPT, 0, kNormArTwoShotNvls>, ctx, ctas, a, stream);
    case kNormRs:
      return launch_k(fused_norm_kernel<T, PPT, NR, kNormRs>, ctx, ctas, a, stream);
    case kNormRsNvls:
      return launch_k(fused_norm_kernel<T, PPT, 0, kNormRsNvls>, ctx, ctas, a, stream);
    case kNormArPush:
      return launch_k(push_norm_kernel<T, PPT, NR, false>, ctx, ctas, a, stream);
    case kNormArPushNvls:
      return launch_k(push_norm_kernel<T, PPT, NR, true>, ctx, ctas, a, stream);
    case kNormArLl:
      return launch_k(ll_norm_kernel<T, PPT, NR>, ctx, ctas, a, stream);
  }
  return cudaErrorInvalidValue;
}

template <typename T, int PPT>
cudaError_t dispatch_world(int algo, const CommCtx& ctx, int ctas, const NormArgs& a, cudaStream_t stream) {
  switch (ctx.world) {
    case 2:
      return dispatch_algo<T, PPT, 2>(algo, ctx, ctas, a, stream);
    case 4:
      return dispatch_algo<T, PPT, 4>(algo, ctx, ctas, a, stream);
    case 8:
      return dispatch_algo<T, PPT, 8>(algo, ctx, ctas, a, stream);
    default:
      return dispatch_algo<T, PPT, 0>(algo, ctx, ctas, a, stream);
  }
}

template <typename T>
cudaError_t dispatch_ppt(int algo, const CommCtx& ctx, int ctas, const NormArgs& a, cudaStream_t stream) {
  const int packs = a.hidden / 8;
  const int ppt = (packs + kNormThreads - 1) / kNormThreads;
  if (ppt <= 1) return dispatch_world<T, 1>(algo, ctx, ctas, a, stream);
  if (ppt <= 2) return dispatch_world<T, 2>(algo, ctx, ctas, a, stream);
  if (ppt <= 4) return dispatch_world<T, 4>(algo, ctx, ctas, a, stream);
  if (ppt <= 8) return dispatch_world<T, 8>(algo, ctx, ctas, a, stream);
  return cudaErrorInvalidValue;  // hidden > 16384
}

}  // namespace

cudaError_t launch_fused_norm(const CommCtx& ctx, int algo, const NormArgs& a, int max_ctas, cudaStream_t stream) {
  if (a.hidden % 8 != 0 || a.hidden <= 0 || a.rows < 0) return cudaErrorInvalidValue;
  if (a.dtype != kF16 && a.dtype != kBF16) return cudaErrorInvalidValue;
  const bool mc = (algo == kNormArTwoShotNvls || algo == kNormRsNvls);
  if (mc && a.x.mc == nullptr) return cudaErrorInvalidValue;
  if (algo == kNormArTwoShotNvls && a.y.mc == nullptr) return cudaErrorInvalidValue;
  const bool push = (algo == kNormArPush || algo == kNormArPushNvls || algo == kNormArLl);
  if (push && (a.y_local == nullptr ||
               a.piece_bytes < size_t(a.rows) * a.hidden * 2 * (algo == kNormArLl ? 2 : 1) || (a.piece_bytes & 15) ||
               a.staging.p[ctx.rank] == nullptr || (algo == kNormArPushNvls && a.staging.mc == nullptr)))
    return cudaErrorInvalidValue;
  int rows = a.rows;
  if (algo >= kNormArTwoShot && !push) rows = (a.rows + ctx.world - 1) / ctx.world;
  int ctas = max_ctas < 1 ? 1 : max_ctas;
  // Communicating launches are bounded by the barrier slots of the pad; the local one may fill the GPU
  // (one row per CTA at a time, eight resident CTAs per SM hide the three dependent passes over a row).
  const int cap = algo == kNormLocal ? 148 * 8 : kMaxCommBlocks;
  if (ctas > cap) ctas = cap;
  if (ctas > rows) ctas = rows < 1 ? 1 : rows;
  if (a.dtype == kF16) return dispatch_ppt<__half>(algo, ctx, ctas, a, stream);
  return dispatch_ppt<__nv_bfloat16>(algo, ctx, ctas, a, stream);
}

}  // namespace oob
