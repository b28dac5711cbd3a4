#pragma once
#include "common.cuh"
namespace yb {
inline bool gemv_preferred(int64_t, int, int) { return false; }
inline int launch_gemv_forward(const void*, const int64_t*, const void*, int, const void*, const void*, const void*,
                               const void*, void*, int64_t, int, int, int, int64_t, void*, float*, cudaStream_t) {
  return YAMOE_ERR_UNSUPPORTED;
}
}
