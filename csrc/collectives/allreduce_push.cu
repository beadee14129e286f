// Small-message all-reduce in one kernel with ONE rank barrier: every rank PUSHES its (unregistered) input into slot
// `rank` of a registered staging area on all ranks (multimem.st through the switch, or peer stores), the blocks of
// all ranks meet once, and every rank then sums the `world` pieces from its OWN memory in rank order (fp32) and
// writes the result to a local output.
//
// Compared with the pull kernels of collectives.cu (barrier -> remote loads -> barrier, preceded by a copy of the
// input into registered memory) this takes the copy kernel, one barrier and the remote round trip of the loads off
// the critical path: what remains is one NVLink traversal for the data with the flag right behind it.  It moves
// (world - 1) x the message per rank, so it is for messages up to a few hundred KiB (decode-step all-reduces).
//
// What lets the closing barrier go: the staging area holds TWO sets of pieces and consecutive calls alternate between
// them.  Which set a call uses is decided on the device (a call counter in the rank's signal pad, bumped by the block
// that finishes last), so the alternation also holds when a captured CUDA graph is replayed or when graphs captured
// at different times follow one another.  A rank that starts call k + 2 (same set as call k) has passed the barrier of
// call k + 1, which every rank enters only after it has finished reading the pieces of call k.  The staging area is
// used by this kernel only; results go wherever the caller wants them (local stores).
//
// Capability parity: the reference's fast one-shot all-reduce (src/comm/fast_multi_gpu_allreduce_sm90.cu:155-257)
// is also a push (cp.reduce.async.bulk of the own chunk into every peer, element-wise atomics in the storage dtype,
// three grid barriers and two rendezvous); here the reduction is a local fp32 sum in rank order after one barrier.
#include <cuda_runtime.h>

#include "../device/reduce.cuh"
#include "../device/sync.cuh"
#include "collectives.h"

namespace oob {
namespace {

constexpr int kPushThreads = 512;

// Block b of every rank owns the same stripe of the message (whole 16-byte packs; the last block also takes the
// elements that do not fill a pack), so one barrier between the blocks of equal index is all the ordering needed,
// whatever the alignment of each rank's own input and output (a rank whose local pointers are not 16-byte aligned
// moves its elements one by one; the pieces in the staging area are always aligned).
template <typename T, int OP, int NR, bool MC>
__global__ void __launch_bounds__(kPushThreads)
    allreduce_push_kernel(CommCtx ctx_param, PeerPtrs staging, const char* in_local, size_t in_emu_stride, char* out_local,
                          size_t out_emu_stride, size_t count, size_t piece_bytes) {
  const CommCtx ctx = resolve_ctx(ctx_param);
  const int world = ctx.world, rank = ctx.rank;
  constexpr size_t E = PackTraits<T>::kElems;
  const char* src = in_local + in_emu_stride * blockIdx.y;
  char* dst = out_local + out_emu_stride * blockIdx.y;
  const bool src_vec = (reinterpret_cast<uintptr_t>(src) & 15) == 0;
  const bool dst_vec = (reinterpret_cast<uintptr_t>(dst) & 15) == 0;
  const size_t packs = count / E;
  const size_t per = (packs + gridDim.x - 1) / gridDim.x;
  const size_t p0 = min(packs, per * blockIdx.x), p1 = min(packs, p0 + per);
  const bool has_tail = blockIdx.x == gridDim.x - 1;
  const size_t tail0 = packs * E;
  // Set of pieces of this call: every block reads the counter before any block of this launch can bump it (the bump
  // needs all blocks to have finished), and all ranks have made the same number of calls.
  __shared__ uint32_t s_set;
  if (threadIdx.x == 0) s_set = ptx::ld_relaxed_sys(call_epoch_ptr(ctx, kPushCallSlot)) & 1u;
  __syncthreads();
  const size_t set_off = size_t(s_set) * size_t(world) * piece_bytes;
  const size_t my_piece = set_off + size_t(rank) * piece_bytes;

  // ---- push this block's stripe of the input into piece `rank` of every rank's staging area ----------------------
  for (size_t p = p0 + threadIdx.x; p < p1; p += kPushThreads) {
    uint4 v;
    if (src_vec) {
      v = ptx::ld_nc_v4(src + p * 16);
    } else {
      T* e = reinterpret_cast<T*>(&v);
#pragma unroll
      for (int i = 0; i < int(E); ++i) e[i] = *reinterpret_cast<const T*>(src + (p * E + i) * sizeof(T));
    }
    if constexpr (MC) {
      ptx::multimem_st_v4(static_cast<char*>(staging.mc) + my_piece + p * 16, v);
    } else if constexpr (NR > 0) {
#pragma unroll
      for (int r = 0; r < NR; ++r) ptx::st_v4(static_cast<char*>(staging.p[(rank + r) % NR]) + my_piece + p * 16, v);
    } else {
      for (int r = 0; r < world; ++r) ptx::st_v4(static_cast<char*>(staging.p[(rank + r) % world]) + my_piece + p * 16, v);
    }
  }
  if (has_tail) {
    for (size_t e = tail0 + threadIdx.x; e < count; e += kPushThreads) {
      const T v = *reinterpret_cast<const T*>(src + e * sizeof(T));
      for (int r = 0; r < world; ++r) st_elem<T>(static_cast<char*>(staging.p[r]) + my_piece + e * sizeof(T), v);
    }
  }

  // ---- the one barrier: block b of every rank has pushed its stripe ------------------------------------------------
  if (!rank_barrier(ctx, blockIdx.x, 40)) return;

  // ---- sum the pieces from LOCAL memory, rank order, fp32 ---------------------------------------------------------
  // Through the switch this rank's own piece comes back over NVLink as well; nothing orders that copy before the
  // loads below (the rank's own flag is a plain local store), so the own contribution is taken from the input.
  // The pieces were written by other GPUs during this kernel: they are read with coherent loads (never through the
  // read-only path).
  const char* mine = static_cast<const char*>(staging.p[rank]) + set_off;
  for (size_t p = p0 + threadIdx.x; p < p1; p += kPushThreads) {
    float acc[E];
    uint4 own;
    if (MC) {
      if (src_vec) {
        own = ptx::ld_nc_v4(src + p * 16);
      } else {
        T* e = reinterpret_cast<T*>(&own);
#pragma unroll
        for (int i = 0; i < int(E); ++i) e[i] = *reinterpret_cast<const T*>(src + (p * E + i) * sizeof(T));
      }
    }
    if constexpr (NR > 0) {
      uint4 v[NR];
#pragma unroll
      for (int r = 0; r < NR; ++r) v[r] = ptx::ld_relaxed_sys_v4(mine + size_t(r) * piece_bytes + p * 16);
      if (MC) {
#pragma unroll
        for (int r = 0; r < NR; ++r)
          if (r == rank) v[r] = own;
      }
      PackTraits<T>::unpack(v[0], acc);
#pragma unroll
      for (int r = 1; r < NR; ++r) {
        float f[E];
        PackTraits<T>::unpack(v[r], f);
#pragma unroll
        for (int i = 0; i < int(E); ++i) acc[i] = combine<OP>(acc[i], f[i]);
      }
    } else {
      PackTraits<T>::unpack((MC && rank == 0) ? own : ptx::ld_relaxed_sys_v4(mine + p * 16), acc);
      for (int r = 1; r < world; ++r) {
        float f[E];
        PackTraits<T>::unpack((MC && r == rank) ? own : ptx::ld_relaxed_sys_v4(mine + size_t(r) * piece_bytes + p * 16), f);
#pragma unroll
        for (int i = 0; i < int(E); ++i) acc[i] = combine<OP>(acc[i], f[i]);
      }
    }
    const uint4 o = PackTraits<T>::pack(acc);
    if (dst_vec) {
      ptx::st_v4(dst + p * 16, o);
    } else {
      const T* e = reinterpret_cast<const T*>(&o);
#pragma unroll
      for (int i = 0; i < int(E); ++i) st_elem<T>(dst + (p * E + i) * sizeof(T), e[i]);
    }
  }
  if (has_tail) {
    for (size_t e = tail0 + threadIdx.x; e < count; e += kPushThreads) {
      float acc = PackTraits<T>::to_float(ld_elem_sys<T>(mine + e * sizeof(T)));
      for (int r = 1; r < world; ++r)
        acc = combine<OP>(acc, PackTraits<T>::to_float(ld_elem_sys<T>(mine + size_t(r) * piece_bytes + e * sizeof(T))));
      st_elem<T>(dst + e * sizeof(T), PackTraits<T>::from_float(acc));
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

template <typename K, typename... Args>
cudaError_t launch_push(K kernel, const CommCtx& ctx, int ctas, cudaStream_t stream, Args... args) {
  if (ctx.emu_table != nullptr) {
    dim3 grid(ctas, ctx.world);
    CommCtx c = ctx;
    void* argv[] = {(void*)&c, (void*)&args...};
    return cudaLaunchCooperativeKernel((const void*)kernel, grid, dim3(kPushThreads), argv, 0, stream);
  }
  kernel<<<dim3(ctas, 1), kPushThreads, 0, stream>>>(ctx, args...);
  return cudaGetLastError();
}

template <typename T, int OP, int NR>
cudaError_t push_dispatch_mc(const CommCtx& ctx, bool mc, const PeerPtrs& st, const char* in, size_t in_stride, char* out,
                             size_t out_stride, size_t count, size_t piece, int ctas, cudaStream_t stream) {
  if (mc) return launch_push(allreduce_push_kernel<T, OP, NR, true>, ctx, ctas, stream, st, in, in_stride, out, out_stride, count, piece);
  return launch_push(allreduce_push_kernel<T, OP, NR, false>, ctx, ctas, stream, st, in, in_stride, out, out_stride, count, piece);
}

template <typename T, int OP>
cudaError_t push_dispatch(const CommCtx& ctx, bool mc, const PeerPtrs& st, const char* in, size_t in_stride, char* out,
                          size_t out_stride, size_t count, size_t piece, int ctas, cudaStream_t stream) {
  switch (ctx.world) {
    case 2:
      return push_dispatch_mc<T, OP, 2>(ctx, mc, st, in, in_stride, out, out_stride, count, piece, ctas, stream);
    case 4:
      return push_dispatch_mc<T, OP, 4>(ctx, mc, st, in, in_stride, out, out_stride, count, piece, ctas, stream);
    case 8:
      return push_dispatch_mc<T, OP, 8>(ctx, mc, st, in, in_stride, out, out_stride, count, piece, ctas, stream);
    default:
      return push_dispatch_mc<T, OP, 0>(ctx, mc, st, in, in_stride, out, out_stride, count, piece, ctas, stream);
  }
}

template <typename T>
cudaError_t push_dispatch_op(int op, const CommCtx& ctx, bool mc, const PeerPtrs& st, const char* in, size_t in_stride,
                             char* out, size_t out_stride, size_t count, size_t piece, int ctas, cudaStream_t stream) {
  switch (op) {
    case kSum:
      return push_dispatch<T, kSum>(ctx, mc, st, in, in_stride, out, out_stride, count, piece, ctas, stream);
    case kMin:
      return push_dispatch<T, kMin>(ctx, mc, st, in, in_stride, out, out_stride, count, piece, ctas, stream);
    case kMax:
      return push_dispatch<T, kMax>(ctx, mc, st, in, in_stride, out, out_stride, count, piece, ctas, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace

// `piece_bytes` (a multiple of 16, at least the message size) is the distance between the ranks' pieces in the staging
// area, which holds two sets of world * piece_bytes.
cudaError_t launch_allreduce_push(const CommCtx& ctx, int dtype, int op, bool use_mc, const PeerPtrs& staging,
                                  size_t piece_bytes, const void* in_local, size_t in_emu_stride, void* out_local,
                                  size_t out_emu_stride, size_t count, int max_ctas, cudaStream_t stream) {
  if (count == 0 || (piece_bytes & 15) != 0) return cudaErrorInvalidValue;
  const size_t esize = dtype == kF32 ? 4 : 2;
  if (count * esize > piece_bytes) return cudaErrorInvalidValue;
  if (use_mc && staging.mc == nullptr) return cudaErrorInvalidValue;
  size_t need = (count * esize / 16 + kPushThreads - 1) / kPushThreads;
  if (need < 1) need = 1;
  int ctas = max_ctas < 1 ? 8 : max_ctas;
  if (ctas > kMaxCommBlocks) ctas = kMaxCommBlocks;
  if (static_cast<size_t>(ctas) > need) ctas = static_cast<int>(need);
  const char* in = static_cast<const char*>(in_local);
  char* out = static_cast<char*>(out_local);
  switch (dtype) {
    case kF16:
      return push_dispatch_op<__half>(op, ctx, use_mc, staging, in, in_emu_stride, out, out_emu_stride, count, piece_bytes, ctas, stream);
    case kBF16:
      return push_dispatch_op<__nv_bfloat16>(op, ctx, use_mc, staging, in, in_emu_stride, out, out_emu_stride, count, piece_bytes,
                                             ctas, stream);
    case kF32:
      return push_dispatch_op<float>(op, ctx, use_mc, staging, in, in_emu_stride, out, out_emu_stride, count, piece_bytes, ctas, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace oob
