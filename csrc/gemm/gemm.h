// Host interface of the tcgen05 GEMM family (plain, GEMM->all-reduce,
// GEMM->reduce-scatter+residual+RMSNorm, all-gather->GEMM).
#pragma once
#include <cuda_runtime.h>
#include <cstddef>
#include <cstdint>
#include "../device/comm_ctx.h"

namespace oob {

enum GemmMode : int {
  kGemmPlain = 0,   // C = A * B^T
  kGemmAr = 1,      // C_all_ranks = sum_r A_r * B_r^T               (row-parallel linear)
  kGemmRsNorm = 2,  // rows of rank: y = rmsnorm(sum_r A_r B_r^T + residual) * w
  kGemmAg = 3,      // C = allgather_rows(A_shard) * B^T             (column-parallel linear)
};

constexpr int kTileM = 128;
constexpr int kTileN = 256;
constexpr int kTileK = 64;
constexpr int kTileBytes = kTileM * kTileN * 2;  // one 16-bit output tile

// Layout of one CTA's trace record (GemmArgs::trace).
enum TraceSlot : int {
  kTraceStart = 0,       // kernel entry
  kTraceGemmDone = 1,    // GEMM CTAs: all tiles computed and stored / pushed
  kTraceFirstReady = 2,  // communication role: first work item became ready; GEMM CTAs of the two-SM fused kernel:
                         // the last tile has left the epilogue (its publication may still be under way)
  kTraceCommDone = 3,    // communication role: last work item finished (before the final rank barrier)
  kTraceEnd = 4,         // after the final rank barrier
  kTraceItems = 5,       // communication work items this CTA processed
  kTraceWaitNs = 6,      // total time this CTA spent waiting for arrival counters
  kTraceRole = 7,        // 0 = GEMM CTA, 1 = dedicated communication CTA
  kTraceWords = 8
};

// All matrices are 16-bit (fp16 or bf16), A is [M, K] row-major with leading
// dimension lda, B is [N, K] row-major (the layout of a torch Linear weight)
// with leading dimension ldb, C is [M, N] row-major.
struct GemmArgs {
  int mode;
  int fmt;  // 0 = fp16, 1 = bf16
  int M, N, K;
  const void* A;
  int lda;
  const void* B;
  int ldb;
  void* C;  // plain / AG modes: local output
  int ldc;
  size_t a_emu_stride, b_emu_stride, c_emu_stride;  // single-GPU emulation: per-rank byte strides of A, B, C

  int comm_ctas;  // CTAs reserved for the communication role (fused modes)
  int max_ctas;   // 0 = one CTA per SM
  int use_nvls;   // fused modes: 0 = peer loads/stores even when a multicast alias exists
  int no_join;    // fused AR / RS: 1 = only the comm_ctas CTAs reduce (GEMM CTAs exit when out of tiles)
  // Optional device-side trace: kTraceWords 64-bit words per CTA (globaltimer nanoseconds at fixed points of
  // the kernel and a few counts), written when non-null.  See TraceSlot.
  unsigned long long* trace;

  // Plain mode: K split over `splits` CTAs per tile (0 = choose from the shape, 1 = off).  The fp32 partials
  // and their arrival counters live in splitk_ws (nullptr = the library's own workspace, grown on demand).
  int splits;
  void* splitk_ws;
  // Split-K: 1 = the kernel only writes its partial tiles and a reduction kernel launched right after sums them
  // (set by launch_gemm; callers ask through splitk_reduce: 0 / 1 = second kernel, -1 = sum inside the GEMM kernel).
  int splitk_defer;
  int splitk_reduce;
  // Plain mode, split problems only: an elementwise op applied by the kernel that sums the splits (see
  // splitk_epilogues.cuh).  epilogue_args is a HOST pointer to the op's argument block.
  // Plain mode, M <= 4: 1 = the CUDA-core streaming kernel (gemv.cu); 0 = by shape (M = 1, and M = 2 with a small
  // weight matrix; OOB_GEMM_GEMV=1 widens that to every M <= 4, =0 switches it off); -1 = never.
  int gemv;
  int epilogue;               // 0 = none, 1 = SwiGLU (oob_gemm_epilogue_swiglu_t), 2 = RoPE + KV write (oob_rope_args_t)
  const void* epilogue_args;
  // 0 = the two-SM kernel (256x256 tiles on CTA pairs) when the shape suits it, 1 = always when possible,
  // -1 = never (the one-SM kernel with 128x256 tiles).  Applies to the plain GEMM and to the fused modes.
  int pair;
  // Two-SM kernel, plain and AG modes: stream-K tail (the last wave and the remainder are cut along K so that no
  // pair idles; partial accumulators meet in a library-owned workspace).  0 = when it pays for the shape, 1 = whenever
  // the tile count leaves a remainder, -1 = never.
  int stream_k;
  // Two-SM kernel, every mode: optional tile-order record.  Two 64-bit words per 128-row half of every 256x256 tile,
  // indexed 2 * (tile's number in the schedule) + (CTA of the pair): [0] globaltimer nanoseconds at which the half
  // was complete in this GPU's memory (fused AR / RS: when it was published to the rank that reduces it),
  // [1] = pair << 32 | index of the tile in that pair's own sequence.  Sorting by [0] gives the completion order.
  unsigned long long* order;
  // Plain mode, M <= 128: 1 = the weight-streaming kernel (gemm_skinny.cu), 0 / -1 = the tiled kernels (0 follows
  // OOB_GEMM_SKINNY=1 for M <= 16).
  int skinny;

  // Fused modes
  PeerPtrs partial;     // AR / RS: per-owner staging of partial tiles, registered; see oob_gemm_partial_bytes
  const void* push_maps; // AR / RS: device array of `world` tensor maps, one over each rank's staging buffer
                        // seen as [slices * 128, 256]; filled in by launch_gemm
  PeerPtrs c_sym;       // AR: output [M, N] in every rank's registered memory
  int counter_base;     // first general counter of the pad used by this op
  // RS + norm tail (rows of this rank only; M / world must be a multiple of 128)
  const void* residual; // [M/world, N] or null
  const void* weight;   // [N] or null (null: no normalisation, y = sum + residual)
  float eps;
  void* y_local;        // [M/world, N]
  void* res_out_local;  // [M/world, N] or null
  size_t rs_emu_stride; // emulation stride of residual / y_local / res_out_local
  // AG: A is this rank's [M/world, K] shard; gathered copy lives in a_full
  PeerPtrs a_full;      // [M, K] registered on every rank
};

// Launches on `stream`.  Returns cudaErrorInvalidValue for unsupported shapes
// (K % 8, N % 8, leading dimensions not multiples of 8 elements, ...).
cudaError_t launch_gemm(const CommCtx& ctx, const GemmArgs& args, cudaStream_t stream);

// Argument checks shared by every entry point.
cudaError_t validate_gemm(const CommCtx& ctx, const GemmArgs& args);

// Number of general counters a fused op needs from counter_base on.
int gemm_counters_needed(int mode, int M, int N, int world);

// Split count the plain GEMM picks for a shape on `sms` SMs (1 = no split).
int gemm_auto_splits(int M, int N, int K, int sms);

// Split-K workspace: bytes a plain GEMM needs (0 = not split), and an ahead-of-time reservation on the current device
// (see oob_gemm_reserve_workspace in the C API).
size_t gemm_splitk_bytes(int M, int N, int K, int max_ctas, int splits);
cudaError_t gemm_reserve_splitk(size_t bytes);
cudaError_t gemm_pair_reserve_workspace();

// Split count launch_gemm uses for a plain GEMM given the caller's `splits` (0 = by shape) and CTA budget.
int gemm_plan_splits(int M, int N, int K, int max_ctas, int splits);

}  // namespace oob
