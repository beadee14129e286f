// Thread-local "last error" used by every C ABI entry point.
#pragma once
#include <cuda_runtime.h>
#include <string>

namespace oob {
int set_error(int code, const std::string& msg);
int cuda_fail(cudaError_t e, const char* what);
}  // namespace oob
