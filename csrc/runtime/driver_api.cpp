#include "driver_api.h"
#include <cuda_runtime.h>
#include <mutex>

namespace oob {
namespace {

template <typename F>
bool load(F& fn, const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr) {
    (void)cudaGetLastError();
    fn = nullptr;
    return false;
  }
  fn = reinterpret_cast<F>(p);
  return true;
}

}  // namespace

const DriverApi* driver_api() {
  static DriverApi api{};
  static bool ok = false;
  static std::once_flag once;
  std::call_once(once, [] {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
      (void)cudaGetLastError();
      return;
    }
    cudaFree(nullptr);  // make sure a primary context exists
    bool all = true;
    all &= load(api.cuTensorMapEncodeTiled, "cuTensorMapEncodeTiled");
    all &= load(api.cuMemCreate, "cuMemCreate");
    all &= load(api.cuMemRelease, "cuMemRelease");
    all &= load(api.cuMemAddressReserve, "cuMemAddressReserve");
    all &= load(api.cuMemAddressFree, "cuMemAddressFree");
    all &= load(api.cuMemMap, "cuMemMap");
    all &= load(api.cuMemUnmap, "cuMemUnmap");
    all &= load(api.cuMemSetAccess, "cuMemSetAccess");
    all &= load(api.cuMemGetAllocationGranularity, "cuMemGetAllocationGranularity");
    all &= load(api.cuMemExportToShareableHandle, "cuMemExportToShareableHandle");
    all &= load(api.cuMemImportFromShareableHandle, "cuMemImportFromShareableHandle");
    all &= load(api.cuMemGetAddressRange, "cuMemGetAddressRange");
    all &= load(api.cuDeviceGet, "cuDeviceGet");
    all &= load(api.cuDeviceGetAttribute, "cuDeviceGetAttribute");
    all &= load(api.cuGetErrorString, "cuGetErrorString");
    // Multicast entry points may be missing on old drivers: optional.
    load(api.cuMulticastCreate, "cuMulticastCreate");
    load(api.cuMulticastAddDevice, "cuMulticastAddDevice");
    load(api.cuMulticastBindMem, "cuMulticastBindMem");
    load(api.cuMulticastUnbind, "cuMulticastUnbind");
    load(api.cuMulticastGetGranularity, "cuMulticastGetGranularity");
    ok = all;
  });
  return ok ? &api : nullptr;
}

}  // namespace oob
