// Host entry of the tcgen05 GEMM family: argument checks, tensor-map cache, the library-owned split-K
// workspace, and dispatch to the kernels of gemm_kernel.cuh.
#include <cstdlib>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "../runtime/driver_api.h"
#include "gemm_kernel.cuh"
#include "gemm_pair.h"
#include "splitk_epilogues.cuh"

namespace oob {

// gemv.cu
bool gemv_supported(const GemmArgs& a);
cudaError_t launch_gemv(const GemmArgs& a, int sms, cudaStream_t stream);
// gemm_skinny.cu
bool gemm_skinny_supported(const GemmArgs& a);
cudaError_t launch_gemm_skinny(const GemmArgs& a, DeviceStatus* status, cudaStream_t stream, gemm_detail::TmapFn make_tmap);

namespace {

using namespace gemm_detail;

struct MapKey {
  const void* p;
  uint64_t rows, cols, ld;
  uint32_t box_rows;
  bool operator==(const MapKey& o) const {
    return p == o.p && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.p);
    h = h * 1000003u ^ k.rows;
    h = h * 1000003u ^ k.cols;
    h = h * 1000003u ^ k.ld;
    h = h * 1000003u ^ k.box_rows;
    return h;
  }
};

// Encoding a tensor map costs a few microseconds of host time; weights and registered buffers keep their
// addresses, so the encoded maps are cached by (pointer, shape).
bool make_tmap_cached(CUtensorMap* out, const void* p, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  const MapKey key{p, rows, cols, ld, box_rows};
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return true;
    }
  }
  if (!encode_tmap_2d(out, p, rows, cols, ld, box_rows)) return false;
  std::lock_guard<std::mutex> g(mu);
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return true;
}

// Library-owned scratch.  One split-K workspace per device, shared by every launch on that device: GEMMs that use it
// (split problems, the weight-streaming kernel) must not overlap on the GPU, i.e. they run on one stream or are
// ordered by events; the same holds for the stream-K workspace of the two-SM kernel.  A workspace that has been handed
// out is never freed or moved (a CUDA graph captured earlier keeps launching with its address): when a larger one is
// needed a new block is allocated and the old one stays alive.  Nothing can be allocated while the stream is being
// captured: the caller reserves beforehand (gemm_reserve_splitk / oob_gemm_reserve_workspace).
struct SplitkBlock {
  void* ptr = nullptr;
  size_t bytes = 0;
};
struct DeviceScratch {
  SplitkBlock splitk;          // current block
  std::vector<void*> retired;  // outgrown blocks, kept alive for launches in flight and captured graphs
  CUtensorMap* emu_maps = nullptr;
};
DeviceScratch g_scratch[64];
std::mutex g_scratch_mu;

// Caller holds g_scratch_mu.  `stream` orders the clearing of the arrival counters before the launch that follows
// (null: cleared synchronously).
cudaError_t grow_splitk(DeviceScratch& s, size_t need, cudaStream_t stream, bool sync_clear) {
  const size_t cap = need + (need >> 2);
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, cap);
  if (e != cudaSuccess) return e;
  e = sync_clear ? cudaMemset(p, 0, kSplitkCounterBytes) : cudaMemsetAsync(p, 0, kSplitkCounterBytes, stream);
  if (e != cudaSuccess) {
    cudaFree(p);
    return e;
  }
  if (s.splitk.ptr) s.retired.push_back(s.splitk.ptr);
  s.splitk.ptr = p;
  s.splitk.bytes = cap;
  return cudaSuccess;
}

cudaError_t ensure_splitk(int dev, size_t need, cudaStream_t stream, void** out) {
  std::lock_guard<std::mutex> g(g_scratch_mu);
  DeviceScratch& s = g_scratch[dev & 63];
  if (s.splitk.bytes < need) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (stream != nullptr && cudaStreamIsCapturing(stream, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone)
      return cudaErrorStreamCaptureUnsupported;  // cannot allocate now; see oob_gemm_reserve_workspace
    (void)cudaGetLastError();
    cudaError_t e = grow_splitk(s, need, stream, false);
    if (e != cudaSuccess) return e;
  }
  *out = s.splitk.ptr;
  return cudaSuccess;
}

// Tensor maps over every rank's staging buffer (for the epilogue's bulk tensor stores), kept on the device and
// cached by the buffer they describe.
struct PushKey {
  const void* p[kMaxRanks];  // every rank's buffer as mapped here: a map is only valid for exactly these addresses
  uint64_t rows;
  int world;
  bool operator==(const PushKey& o) const {
    if (rows != o.rows || world != o.world) return false;
    for (int r = 0; r < world; ++r)
      if (p[r] != o.p[r]) return false;
    return true;
  }
};
struct PushKeyHash {
  size_t operator()(const PushKey& k) const {
    size_t h = k.rows * 1000003u ^ size_t(k.world);
    for (int r = 0; r < k.world; ++r) h = h * 1000003u ^ reinterpret_cast<size_t>(k.p[r]);
    return h;
  }
};
std::unordered_map<PushKey, CUtensorMap*, PushKeyHash> g_push_maps;

cudaError_t ensure_push_maps(const CommCtx& ctx, const GemmArgs& a, const void** out) {
  const uint64_t tiles = uint64_t((a.M + kTileM - 1) / kTileM) * ((a.N + kTileN - 1) / kTileN);
  const uint64_t rows = (tiles + kMaxRanks) * kTileM;  // capacity promised by oob_gemm_partial_bytes
  PushKey key{};
  for (int r = 0; r < ctx.world; ++r) key.p[r] = a.partial.p[r];
  key.rows = rows;
  key.world = ctx.world;
  std::lock_guard<std::mutex> g(g_scratch_mu);
  auto it = g_push_maps.find(key);
  if (it != g_push_maps.end()) {
    *out = it->second;
    return cudaSuccess;
  }
  CUtensorMap host[kMaxRanks];
  for (int r = 0; r < ctx.world; ++r)
    if (!encode_tmap_2d(&host[r], a.partial.p[r], rows, kTileN, kTileN, 32)) return cudaErrorInvalidValue;
  CUtensorMap* dev_maps = nullptr;
  cudaError_t e = cudaMalloc(&dev_maps, sizeof(CUtensorMap) * kMaxRanks);
  if (e != cudaSuccess) return e;
  e = cudaMemcpy(dev_maps, host, sizeof(CUtensorMap) * ctx.world, cudaMemcpyHostToDevice);
  if (e != cudaSuccess) return e;
  g_push_maps.emplace(key, dev_maps);
  *out = dev_maps;
  return cudaSuccess;
}

cudaError_t ensure_emu_maps(int dev, CUtensorMap** out) {
  std::lock_guard<std::mutex> g(g_scratch_mu);
  DeviceScratch& s = g_scratch[dev & 63];
  if (s.emu_maps == nullptr) {
    cudaError_t e = cudaMalloc(&s.emu_maps, sizeof(CUtensorMap) * 3 * kMaxRanks);
    if (e != cudaSuccess) return e;
  }
  *out = s.emu_maps;
  return cudaSuccess;
}

template <typename T>
cudaError_t launch_fmt(const CommCtx& ctx, const GemmArgs& a, cudaStream_t stream, CUtensorMap* emu_maps) {
  switch (a.mode) {
    case kGemmPlain:
      return launch_mode<T, kGemmPlain>(ctx, a, stream, make_tmap_cached, emu_maps);
    case kGemmAr:
      return launch_mode<T, kGemmAr>(ctx, a, stream, make_tmap_cached, emu_maps);
    case kGemmRsNorm:
      return launch_mode<T, kGemmRsNorm>(ctx, a, stream, make_tmap_cached, emu_maps);
    case kGemmAg:
      return launch_mode<T, kGemmAg>(ctx, a, stream, make_tmap_cached, emu_maps);
  }
  return cudaErrorInvalidValue;
}

}  // namespace

cudaError_t gemm_library_workspace(size_t bytes, cudaStream_t stream, void** out) {
  int dev = 0;
  cudaGetDevice(&dev);
  return ensure_splitk(dev, bytes, stream, out);
}

cudaError_t gemm_reserve_splitk(size_t bytes) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  std::lock_guard<std::mutex> g(g_scratch_mu);
  DeviceScratch& s = g_scratch[dev & 63];
  if (bytes == 0 || s.splitk.bytes >= bytes) return cudaSuccess;
  return grow_splitk(s, bytes, nullptr, true);
}

size_t gemm_splitk_bytes(int M, int N, int K, int max_ctas, int splits) {
  const int s = gemm_plan_splits(M, N, K, max_ctas, splits);
  return s > 1 ? gemm_detail::splitk_workspace_bytes(M, N, s) : 0;
}

bool encode_tmap_2d(CUtensorMap* out, const void* p, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
  const DriverApi* drv = driver_api();
  if (drv == nullptr || drv->cuTensorMapEncodeTiled == nullptr) return false;
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {ld * 2};
  cuuint32_t box[2] = {kTileK, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = drv->cuTensorMapEncodeTiled(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(p), gdim, gstride,
                                           box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

int gemm_counters_needed(int mode, int M, int N, int world) {
  const int tiles_m = (M + kTileM - 1) / kTileM, tiles_n = (N + kTileN - 1) / kTileN;
  switch (mode) {
    case kGemmAr: {
      // one-SM kernel: per-tile arrivals + ticket; two-SM kernel: arrivals + finished work items per owned 128x256
      // half tile
      const int one_sm = (tiles_m * tiles_n + world - 1) / world + 1;
      const int pair = 2 * ((2 * ((M + 2 * kTileM - 1) / (2 * kTileM)) * tiles_n + world - 1) / world) + 1;  // + ticket
      return one_sm > pair ? one_sm : pair;
    }
    case kGemmRsNorm:
      return 2 * ((M / world + kTileM - 1) / kTileM) + 1;  // arrivals + finished items per row block + ticket
    case kGemmAg:
      return tiles_m + 1;  // chunk flags + finished GEMM CTAs
  }
  return 0;
}

int gemm_auto_splits(int M, int N, int K, int sms) {
  const int tiles = ((M + kTileM - 1) / kTileM) * ((N + kTileN - 1) / kTileN);
  if (tiles * 2 > sms || K < 4 * kTileK) return 1;
  int s = sms / tiles;
  if (s > 8) s = 8;
  // Keep at least four K blocks (256 elements) per split so that the pipeline still fills.
  const int num_kb = (K + kTileK - 1) / kTileK;
  if (s > num_kb / 4) s = num_kb / 4;
  return gemm_detail::normalize_splits(K, s);
}

int gemm_plan_splits(int M, int N, int K, int max_ctas, int splits) {
  if (splits == 0) splits = gemm_auto_splits(M, N, K, max_ctas > 0 ? max_ctas : gemm_detail::sm_count());
  splits = gemm_detail::normalize_splits(K, splits);
  const size_t tiles = size_t((M + kTileM - 1) / kTileM) * ((N + kTileN - 1) / kTileN);
  if (tiles > gemm_detail::kSplitkMaxTiles) splits = 1;
  return splits;
}

cudaError_t validate_gemm(const CommCtx& ctx, const GemmArgs& a) {
  if (a.M <= 0 || a.N <= 0 || a.K <= 0) return cudaErrorInvalidValue;
  if (a.K % 8 != 0 || a.lda % 8 != 0 || a.ldb % 8 != 0) return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(a.A) & 15) || (reinterpret_cast<uintptr_t>(a.B) & 15)) return cudaErrorInvalidValue;
  if (a.mode != kGemmPlain) {
    if (a.N % 8 != 0) return cudaErrorInvalidValue;
    if (gemm_counters_needed(a.mode, a.M, a.N, ctx.world) + a.counter_base > kNumCounters - 1)
      return cudaErrorInvalidValue;
  }
  if (a.mode == kGemmRsNorm || a.mode == kGemmAg) {
    if (a.M % ctx.world != 0 || (a.M / ctx.world) % kTileM != 0) return cudaErrorInvalidValue;
    if (a.mode == kGemmRsNorm && a.N > 6 * gemm_detail::kThreadsFused * 8) return cudaErrorInvalidValue;
    if (a.mode == kGemmAg && ctx.world < 2) return cudaErrorInvalidValue;
  }
  if (a.mode == kGemmPlain || a.mode == kGemmAg) {
    if (reinterpret_cast<uintptr_t>(a.C) & 15) return cudaErrorInvalidValue;
  }
  return cudaSuccess;
}

cudaError_t launch_gemm(const CommCtx& ctx, const GemmArgs& args, cudaStream_t stream) {
  cudaError_t e = validate_gemm(ctx, args);
  if (e != cudaSuccess) return e;
  GemmArgs a = args;
  int dev = 0;
  cudaGetDevice(&dev);
  if (a.mode == kGemmPlain) {
    // One to four rows: the CUDA-core streaming kernel.  By argument, or when the call leaves the choice open: for one
    // row always, for two rows when the weight matrix is small (N x K up to 12 M elements), which is where it measured
    // faster than the tensor-core paths on B200 (M = 1: 6.1 / 8.6 / 13.9 us against 10.6 / 14.3 / 17.2 us for
    // 8192 x 1024, 1280 x 8192, 8192 x 3584; M = 2 on the two smaller ones: 8.0 / 11.7 against 10.4 / 14.3 us; from
    // M = 4 on it loses everywhere).  OOB_GEMM_GEMV=0 switches the rule off, =1 widens it to every M <= 4.
    static const int gemv_env = [] {
      const char* v = getenv("OOB_GEMM_GEMV");
      return v == nullptr ? -1 : (v[0] == '1' ? 1 : 0);
    }();
    const bool gemv_by_shape =
        gemv_env != 0 && (a.M == 1 || (a.M == 2 && static_cast<long long>(a.N) * a.K <= 12ll * 1000 * 1000));
    if (a.epilogue == 0 && gemv_supported(a) && ctx.emu_table == nullptr && a.c_emu_stride == 0 && a.splitk_ws == nullptr &&
        (a.gemv > 0 || (a.gemv == 0 && a.splits == 0 && a.skinny <= 0 && (gemv_env == 1 || gemv_by_shape))))
      return launch_gemv(a, a.max_ctas > 0 ? a.max_ctas : sm_count(), stream);
    // The weight-streaming kernel (stream-K over 128-row weight tiles) is opt-in: measured on B200, inside a replayed
    // decode step it is 2 - 12 % slower at M <= 16 than the 128x256 split-K tiles followed by the reduction kernel,
    // and far slower from M = 32 on (every CTA re-reads its share of the activations, which then rivals the weight
    // traffic).  OOB_GEMM_SKINNY=1 makes it the default for M <= 16.
    static const bool skinny_env_on = [] {
      const char* v = getenv("OOB_GEMM_SKINNY");
      return v != nullptr && v[0] == '1';
    }();
    if (a.epilogue == 0 && gemm_skinny_supported(a) && ctx.emu_table == nullptr && a.c_emu_stride == 0 && a.splitk_ws == nullptr &&
        (a.skinny > 0 || (a.skinny == 0 && a.splits == 0 && a.M <= 16 && skinny_env_on)))
      return launch_gemm_skinny(a, ctx.status, stream, make_tmap_cached);
    const int splits = gemm_plan_splits(a.M, a.N, a.K, a.max_ctas, a.splits);
    a.splits = splits;
    if (a.epilogue != 0) {
      // The epilogue lives in the kernel that sums the splits: the problem has to be one that is split.
      if (splits <= 1 || ctx.emu_table != nullptr || a.c_emu_stride != 0 || a.epilogue_args == nullptr || a.epilogue > 2)
        return cudaErrorInvalidValue;
    }
    if (splits > 1 && a.splitk_ws == nullptr) {
      e = ensure_splitk(dev, splitk_workspace_bytes(a.M, a.N, splits), stream, &a.splitk_ws);
      if (e != cudaSuccess) return e;
    }
    // The sum over the splits is left to a second, grid-wide kernel.  In the GEMM kernel that sum is done by the
    // one warp that arrives last for a 32-row quadrant, a chain of (rows / 8) x splits L2 round trips behind a
    // fence and an atomic; measured inside a replayed decode step the second kernel wins at every M (batch 1: 92.6
    // -> 86.0 us per layer, batch 16: 113.8 -> 91.1, batch 64: 160.6 -> 109.8).  OOB_SPLITK_REDUCE_MIN_M raises the
    // row count from which it is used.  Both paths add the splits in the same order: bit-identical results.
    static const int splitk_reduce_min_rows = [] {
      const char* v = getenv("OOB_SPLITK_REDUCE_MIN_M");
      return v != nullptr && atoi(v) > 0 ? atoi(v) : 1;
    }();
    a.splitk_defer = 0;
    if (splits > 1 && ctx.emu_table == nullptr && a.c_emu_stride == 0 &&
        (a.epilogue != 0 || a.splitk_reduce > 0 || (a.splitk_reduce == 0 && a.M >= splitk_reduce_min_rows)))
      a.splitk_defer = 1;
    // Large problems go to the two-SM kernel: same tile count per SM, two thirds of the operand traffic.
    const bool pair_ok = splits == 1 && ctx.emu_table == nullptr && a.c_emu_stride == 0 && (a.max_ctas == 0 || a.max_ctas >= 2);
    static const bool pair_env_off = [] {
      const char* v = getenv("OOB_GEMM_PAIR");
      return v != nullptr && v[0] == '0';
    }();
    const bool pair_auto = a.M > kTileM && !pair_env_off;
    if (pair_ok && (a.pair > 0 || (a.pair == 0 && pair_auto))) {
      e = launch_gemm_pair(ctx, a, stream, make_tmap_cached, nullptr);
      if (e != cudaErrorNotSupported) return e;
      cudaGetLastError();
    }
  } else {
    a.splits = 1;
    // Fused modes on CTA pairs: same mainloop as the plain two-SM kernel, communication in clusters of the same
    // launch.  pair = 0 follows OOB_FUSED_PAIR (default on).
    static const bool fused_pair_env_off = [] {
      const char* v = getenv("OOB_FUSED_PAIR");
      return v != nullptr && v[0] == '0';
    }();
    if ((a.pair > 0 || (a.pair == 0 && !fused_pair_env_off)) && gemm_pair_supported(ctx, a)) {
      CUtensorMap* emu_maps = nullptr;
      if (ctx.emu_table != nullptr) {
        e = ensure_emu_maps(dev, &emu_maps);
        if (e != cudaSuccess) return e;
      }
      e = launch_gemm_pair(ctx, a, stream, make_tmap_cached, emu_maps);
      if (e != cudaErrorNotSupported) return e;
      cudaGetLastError();
    }
  }
  if (a.mode == kGemmAr || a.mode == kGemmRsNorm) {
    e = ensure_push_maps(ctx, a, &a.push_maps);
    if (e != cudaSuccess) return e;
  }
  CUtensorMap* emu_maps = nullptr;
  if (ctx.emu_table != nullptr) {
    e = ensure_emu_maps(dev, &emu_maps);
    if (e != cudaSuccess) return e;
  }
  e = a.fmt == 1 ? launch_fmt<__nv_bfloat16>(ctx, a, stream, emu_maps) : launch_fmt<__half>(ctx, a, stream, emu_maps);
  if (e != cudaSuccess || a.mode != kGemmPlain || !a.splitk_defer) return e;
  if (a.epilogue == 1) {
    const int F = static_cast<const oob_gemm_epilogue_swiglu_t*>(a.epilogue_args)->F;
    return a.fmt == 1 ? launch_splitk_reduce_swiglu<__nv_bfloat16>(a, F, stream) : launch_splitk_reduce_swiglu<__half>(a, F, stream);
  }
  if (a.epilogue == 2) {
    const oob_rope_args_t& r = *static_cast<const oob_rope_args_t*>(a.epilogue_args);
    return a.fmt == 1 ? launch_splitk_reduce_rope_kv<__nv_bfloat16>(a, r, stream) : launch_splitk_reduce_rope_kv<__half>(a, r, stream);
  }
  return a.fmt == 1 ? launch_splitk_reduce<__nv_bfloat16>(a, stream) : launch_splitk_reduce<__half>(a, stream);
}

}  // namespace oob
