// Split-K GEMM whose workspace is a fixed array inside the library image, for callers that cannot allocate
// device memory when they call (see csrc/api/oob_noalloc.h for who they are and for the contract).  The kernel
// is the plain-mode kernel of gemm_kernel.cuh; only the origin of the workspace differs from oob_gemm().
#include <mutex>
#include <string>

#include "../api/oob.h"
#include "../api/oob_noalloc.h"
#include "../runtime/errors.h"
#include "gemm_kernel.cuh"

namespace oob {
namespace {

using namespace gemm_detail;

// Arrival counters (fixed-size block, as the kernel expects) followed by the fp32 partial tiles.  In host code
// this name is only a handle for cudaGetSymbolAddress: it is not a device address and must never be passed to
// a kernel as such.
static __device__ __align__(256) unsigned char g_static_ws[kSplitkCounterBytes + OOB_SPLITK_STATIC_BYTES];

std::mutex g_mu;
void* g_ws_addr[64] = {};  // device address of g_static_ws per device ordinal, looked up once

// First call on a device (with that device current): resolve the array's device address.
cudaError_t static_workspace(int dev, void** out) {
  std::lock_guard<std::mutex> g(g_mu);
  void*& slot = g_ws_addr[dev & 63];
  if (slot == nullptr) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_static_ws);
    if (e != cudaSuccess) return e;
    slot = p;
  }
  *out = slot;
  return cudaSuccess;
}

uint64_t partial_need(int M, int N, int splits) {
  const uint64_t tiles = uint64_t((M + kTileM - 1) / kTileM) * ((N + kTileN - 1) / kTileN);
  return tiles * uint64_t(splits) * (uint64_t(kTileM) * kTileN * 4);
}

}  // namespace
}  // namespace oob

extern "C" uint64_t oob_gemm_splitk_static_need(int M, int N, int K, int splits) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  return oob::partial_need(M, N, oob::gemm_detail::normalize_splits(K, splits));
}

extern "C" int oob_gemm_splitk_static(int dtype, int M, int N, int K, const void* A, int lda, const void* B, int ldb,
                                      void* C, int ldc, int splits, int max_ctas, void* stream) {
  using namespace oob;
  using namespace oob::gemm_detail;
  if (dtype != OOB_F16 && dtype != OOB_BF16) return set_error(OOB_ERR_INVALID, "GEMM dtype must be fp16 or bf16");
  GemmArgs a{};
  a.mode = kGemmPlain;
  a.fmt = dtype == OOB_BF16 ? 1 : 0;
  a.M = M;
  a.N = N;
  a.K = K;
  a.A = A;
  a.lda = lda;
  a.B = B;
  a.ldb = ldb;
  a.C = C;
  a.ldc = ldc;
  a.max_ctas = max_ctas;
  CommCtx ctx{};
  ctx.world = 1;
  ctx.rank = 0;
  ctx.timeout_ns = 2000000000ull;
  if (validate_gemm(ctx, a) != cudaSuccess)
    return set_error(OOB_ERR_INVALID, "unsupported GEMM arguments (K and leading dimensions must be multiples of 8, "
                                      "pointers 16-byte aligned)");
  a.splits = normalize_splits(K, splits);
  const uint64_t tiles = uint64_t((M + kTileM - 1) / kTileM) * ((N + kTileN - 1) / kTileN);
  const uint64_t need = partial_need(M, N, a.splits);
  if (need > OOB_SPLITK_STATIC_BYTES || tiles > kSplitkMaxTiles)
    return set_error(OOB_ERR_NOMEM, "problem needs " + std::to_string(need) + " bytes of split-K partial tiles, the "
                                    "built-in array holds " + std::to_string(uint64_t(OOB_SPLITK_STATIC_BYTES)) +
                                    "; use fewer splits or oob_gemm()");
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  void* ws = nullptr;
  e = static_workspace(dev, &ws);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(split-K array)");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (a.splits > 1) {
    // The array keeps whatever the previous call left: the counters this call uses must start at zero.
    e = cudaMemsetAsync(ws, 0, tiles * 4 * sizeof(uint32_t), s);
    if (e != cudaSuccess) return cuda_fail(e, "clearing split-K counters");
    a.splitk_ws = ws;
  }
  // Tensor maps are encoded on the host for every call (no cache: nothing is kept, nothing is allocated).
  e = a.fmt == 1 ? launch_mode<__nv_bfloat16, kGemmPlain>(ctx, a, s, encode_tmap_2d, nullptr)
                 : launch_mode<__half, kGemmPlain>(ctx, a, s, encode_tmap_2d, nullptr);
  if (e != cudaSuccess) return cuda_fail(e, "split-K GEMM launch");
  return OOB_OK;
}
