// Host-callable launchers of the collective kernels (internal C++ interface;
// the exported C ABI is csrc/api/oob.h).
#pragma once
#include <cuda_runtime.h>
#include <cstddef>
#include "../device/comm_ctx.h"

namespace oob {

enum ArAlgo : int { kArOneShotP2P = 0, kArTwoShotP2P = 1, kArTwoShotNvls = 2, kArOneShotNvls = 3 };
enum RsAlgo : int { kRsP2P = 0, kRsNvls = 1 };
enum AgAlgo : int { kAgPushP2P = 0, kAgPushNvls = 1, kAgPullP2P = 2 };

// `out_local` (+ emu stride) is used by the one-shot algorithms; `out` (a
// registered buffer) by the two-shot ones.  `count` is in elements.
cudaError_t launch_allreduce(const CommCtx& ctx, int dtype, int op, int algo, const PeerPtrs& in, const PeerPtrs& out,
                             void* out_local, size_t out_local_emu_stride, size_t count, int max_ctas,
                             cudaStream_t stream);

cudaError_t launch_reduce_scatter(const CommCtx& ctx, int dtype, int op, int algo, const PeerPtrs& in,
                                  void* out_local, size_t out_local_emu_stride, size_t count, int max_ctas,
                                  cudaStream_t stream);

cudaError_t launch_all_gather(const CommCtx& ctx, int dtype, int algo, const PeerPtrs& out, const void* src_local,
                              size_t src_local_emu_stride, void* dst_local, size_t dst_local_emu_stride,
                              size_t count, int max_ctas, cudaStream_t stream);

// One-barrier push all-reduce for small messages (allreduce_push.cu): `in_local` / `out_local` are ordinary device
// memory; `staging` is a registered area of world * piece_bytes that must come from a ring of two or more areas used
// round robin.  `use_mc`: push with multimem.st through the switch.
cudaError_t launch_allreduce_push(const CommCtx& ctx, int dtype, int op, bool use_mc, const PeerPtrs& staging,
                                  size_t piece_bytes, const void* in_local, size_t in_emu_stride, void* out_local,
                                  size_t out_emu_stride, size_t count, int max_ctas, cudaStream_t stream);

// Flag-in-data all-reduce without a barrier for messages up to a few tens of KiB (allreduce_ll.cu).  The staging area
// (two sets of world * piece_bytes, piece_bytes >= 8 bytes per 32-bit word of the message) must be zeroed once before
// its first use and written by this kernel only.
cudaError_t launch_allreduce_ll(const CommCtx& ctx, int dtype, int op, bool use_mc, const PeerPtrs& staging,
                                size_t piece_bytes, const void* in_local, size_t in_emu_stride, void* out_local,
                                size_t out_emu_stride, size_t count, int max_ctas, cudaStream_t stream);

// Rank r's chunk j (chunk_bytes each, `src_local` holds `world` of them) lands as chunk r of rank j's registered
// `out` buffer (all_to_all.cu).
cudaError_t launch_all_to_all(const CommCtx& ctx, const PeerPtrs& out, const void* src_local, size_t src_emu_stride,
                              size_t chunk_bytes, int max_ctas, cudaStream_t stream);

// Residual-add + RMSNorm, stand-alone and fused into the all-reduce /
// reduce-scatter (see fused_norm.cu).
enum NormAlgo : int {
  kNormLocal = 0,         // no communication: y = rmsnorm(x + residual)
  kNormArOneShot = 1,     // every rank reduces all rows itself, then normalises (small token counts)
  kNormArTwoShot = 2,     // rank r reduces + normalises its row shard and pushes y / new residual to all ranks
  kNormArTwoShotNvls = 3, // same with multimem.ld_reduce / multimem.st
  kNormRs = 4,            // reduce-scatter by rows + residual + norm; outputs stay local (sequence-parallel form)
  kNormRsNvls = 5,
  kNormArPush = 6,        // decode sizes: every rank pushes its rows to all ranks, ONE rank barrier, every rank sums the
                          // pieces locally and normalises every row (staging area as for the push all-reduce)
  kNormArPushNvls = 7,    // same, pushed with multimem.st
  kNormArLl = 8,          // the smallest messages: rows travel as 8-byte cells of data + call number, no barrier at all
                          // (staging area, cell format and call counter of allreduce_ll.cu)
};

// Call-epoch words of the signal pad shared by the push kernels (allreduce_push.cu, fused_norm.cu): the number of push
// calls this rank has made (its parity selects the set of pieces a call uses) and the blocks of the running call
// that have finished.
constexpr int kPushCallSlot = 0;
constexpr int kPushDoneSlot = 1;
// The same pair of words for the flag-in-data all-reduce (allreduce_ll.cu), whose call number is also the flag value.
constexpr int kLlCallSlot = 2;
constexpr int kLlDoneSlot = 3;

struct NormArgs {
  int dtype;              // kF16 / kBF16
  int rows, hidden;       // x is [rows, hidden] on every rank
  float eps;
  PeerPtrs x;             // partial sums (registered); for kNormLocal only x.p[rank] is read
  const void* residual;   // [rows, hidden] local (full) for AR algos; [rows_of_rank, hidden] for RS; may be null
  size_t residual_emu_stride;
  const void* weight;     // [hidden]
  PeerPtrs y;             // normalised output: pushed to all ranks by two-shot algos
  void* y_local;          // used by local / one-shot / RS algos
  size_t y_local_emu_stride;
  PeerPtrs res_out;       // x_sum + residual, same placement rule as y (p[rank]==nullptr to skip)
  void* res_out_local;
  size_t res_out_local_emu_stride;
  PeerPtrs staging;       // push algorithms: two sets of world * piece_bytes (registered)
  size_t piece_bytes;     // >= rows * hidden * sizeof(T), a multiple of 16
};

cudaError_t launch_fused_norm(const CommCtx& ctx, int algo, const NormArgs& args, int max_ctas, cudaStream_t stream);

}  // namespace oob
