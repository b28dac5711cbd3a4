// placeholder until the tcgen05 kernels land
#pragma once
#include "simt_gemm.cuh"
namespace yb {
inline bool umma_available() { return false; }
template <int MODE, class Epi>
inline int launch_umma_gemm(const GemmArgs&, const Epi&, int64_t, int64_t, cudaStream_t) { return YAMOE_ERR_UNSUPPORTED; }
}
