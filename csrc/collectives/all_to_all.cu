// All-to-all over peer memory: every rank holds `world` chunks of `count_per_peer` elements and sends chunk j to
// rank j, which stores it as chunk (sender) of its output.  The building block of expert-parallel dispatch /
// combine.
//
// One kernel: barrier between the ranks' blocks (every output buffer is free to be overwritten), then each rank
// PUSHES its chunks with 128-bit stores, eight loads in flight per thread, peers visited in ring order starting
// with the rank's own chunk so that no two ranks hammer the same destination at the same time; barrier (all chunks
// have landed and are visible).  Bytes opaque: any 16-bit or 32-bit dtype.
//
// Capability parity: the reference has no all-to-all of its own, only an NCCL grouped send/recv baseline
// (src/baseline_impl.cu:178-267); this kernel has no counterpart there.
#include <cuda_runtime.h>

#include "../device/reduce.cuh"
#include "../device/sync.cuh"
#include "collectives.h"

namespace oob {
namespace {

constexpr int kA2aThreads = 512;
constexpr int kA2aUnroll = 8;

__global__ void __launch_bounds__(kA2aThreads) all_to_all_kernel(CommCtx ctx_param, PeerPtrs out, const char* src_local,
                                                                 size_t src_emu_stride, size_t chunk_bytes) {
  const CommCtx ctx = resolve_ctx(ctx_param);
  const int world = ctx.world, rank = ctx.rank;
  if (!rank_barrier(ctx, blockIdx.x, 35)) return;
  const char* src = src_local + src_emu_stride * blockIdx.y;
  const bool vec_ok = (chunk_bytes & 15) == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0;
  const size_t packs = vec_ok ? chunk_bytes / 16 : 0;
  const size_t per = (packs + gridDim.x - 1) / gridDim.x;  // contiguous stripe of every chunk for this block
  const size_t p_begin = min(packs, per * blockIdx.x), p_end = min(packs, p_begin + per);
  for (int i = 0; i < world; ++i) {
    const int peer = (rank + i) % world;
    const char* s = src + size_t(peer) * chunk_bytes;                                  // chunk destined to `peer`
    char* d = static_cast<char*>(out.p[peer]) + size_t(rank) * chunk_bytes;           // slot `rank` of its output
    for (size_t pb = p_begin + threadIdx.x; pb < p_end; pb += size_t(kA2aThreads) * kA2aUnroll) {
      uint4 v[kA2aUnroll];
#pragma unroll
      for (int u = 0; u < kA2aUnroll; ++u) {
        const size_t p = pb + size_t(u) * kA2aThreads;
        v[u] = ptx::ld_nc_v4(s + (p < p_end ? p : pb) * 16);  // past the stripe: re-read, result unused
      }
#pragma unroll
      for (int u = 0; u < kA2aUnroll; ++u) {
        const size_t p = pb + size_t(u) * kA2aThreads;
        if (p < p_end) ptx::st_v4(d + p * 16, v[u]);
      }
    }
    if (!vec_ok) {
      // Bytes that do not form aligned 16-byte packs: 2-byte units (chunk sizes are multiples of the element size).
      for (size_t b = (size_t(blockIdx.x) * kA2aThreads + threadIdx.x) * 2; b < chunk_bytes;
           b += size_t(gridDim.x) * kA2aThreads * 2)
        *reinterpret_cast<unsigned short*>(d + b) = *reinterpret_cast<const unsigned short*>(s + b);
    }
  }
  rank_barrier(ctx, blockIdx.x, 36);
}

}  // namespace

cudaError_t launch_all_to_all(const CommCtx& ctx, const PeerPtrs& out, const void* src_local, size_t src_emu_stride,
                              size_t chunk_bytes, int max_ctas, cudaStream_t stream) {
  if (chunk_bytes == 0 || (chunk_bytes & 1)) return cudaErrorInvalidValue;
  size_t need = (chunk_bytes / 16 + kA2aThreads - 1) / kA2aThreads;
  if (need < 1) need = 1;
  int ctas = max_ctas < 1 ? 16 : max_ctas;
  if (ctas > kMaxCommBlocks) ctas = kMaxCommBlocks;
  if (static_cast<size_t>(ctas) > need) ctas = static_cast<int>(need);
  const char* src = static_cast<const char*>(src_local);
  if (ctx.emu_table != nullptr) {
    dim3 grid(ctas, ctx.world);
    CommCtx c = ctx;
    PeerPtrs o = out;
    void* argv[] = {(void*)&c, (void*)&o, (void*)&src, (void*)&src_emu_stride, (void*)&chunk_bytes};
    return cudaLaunchCooperativeKernel((const void*)all_to_all_kernel, grid, dim3(kA2aThreads), argv, 0, stream);
  }
  all_to_all_kernel<<<dim3(ctas, 1), kA2aThreads, 0, stream>>>(ctx, out, src, src_emu_stride, chunk_bytes);
  return cudaGetLastError();
}

}  // namespace oob
