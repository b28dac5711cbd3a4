// CUDA-core grouped GEMM with fp32 accumulation: the fp32 path of the library and the
// always-available path every tcgen05 kernel is validated against.
//
// One kernel, three operand arrangements (all on the padded, expert-sorted row layout):
//   kFwd    C[row, n] = sum_k A[row, k] * W[e][k][n]     (A rows K-contiguous, W N-contiguous)
//           reference: csrc/batch_mm.cu:27-30 as called at csrc/moe.cpp:161,184
//   kDgrad  C[row, n] = sum_k A[row, k] * W[e][n][k]     (W K-contiguous: multiplication by W^T)
//           reference: csrc/experts_backward.cu:278-280, :309-310
//   kWgrad  C[e][m, n] = sum_{rows r of expert e} A[r, m] * B[r, n]
//           reference: csrc/experts_backward.cu:281-282, :311
// 64x64 output tile, 16-deep k slices, 256 threads, 4x4 accumulators per thread.
#pragma once
#include "common.cuh"
#include "epilogues.cuh"

namespace yb {

enum GemmMode { kFwd = 0, kDgrad = 1, kWgrad = 2 };

struct GemmArgs {
  const void* A; int64_t lda;
  const void* B; int64_t ldb; int64_t b_expert_stride;
  int M;   // kWgrad: rows of the per-expert output
  int N;   // output columns
  int K;   // kFwd/kDgrad: reduction length
  int E;
  const int32_t* tile_expert;
  const int32_t* pad_off;
  const int32_t* header;
  const int32_t* pair_expert = nullptr;   // tile-pair tables (256-row tcgen05 kernel only)
  const int32_t* pair_off = nullptr;
  const int32_t* counts = nullptr;        // rows present per expert (swapped-operand tcgen05 kernel only)
  // tcgen05 kFwd only: A is the UN-permuted source [gather_src_rows, K]; row r of the padded layout
  // is source row gather_rows[r] (negative = padding), fetched by TMA gather
  const int32_t* gather_rows = nullptr;
  int64_t gather_src_rows = 0;
};

constexpr int kSimtBM = 64, kSimtBN = 64, kSimtBK = 16, kSimtThreads = 256;

template <typename T, int MODE, class Epi>
__global__ void __launch_bounds__(kSimtThreads)
simt_gemm_kernel(GemmArgs g, Epi epi) {
  __shared__ __align__(16) float As[kSimtBK][kSimtBM + 4];
  __shared__ __align__(16) float Bs[kSimtBK][kSimtBN + 4];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int n0 = blockIdx.x * kSimtBN;
  int e, row0, k_begin, k_end, m_limit;
  if constexpr (MODE == kWgrad) {
    e = blockIdx.z;
    row0 = blockIdx.y * kSimtBM;            // m0 within the expert's output
    k_begin = g.pad_off[e];
    k_end = g.pad_off[e + 1];
    m_limit = g.M;
  } else {
    row0 = blockIdx.y * kSimtBM;            // padded row
    if (row0 >= g.header[kHdrRowsUsed]) return;
    e = g.tile_expert[row0 / kTileM];
    k_begin = 0;
    k_end = g.K;
    m_limit = row0 + kSimtBM;
  }
  const T* __restrict__ A = reinterpret_cast<const T*>(g.A);
  const T* __restrict__ B = reinterpret_cast<const T*>(g.B) + (MODE == kWgrad ? 0 : (size_t)e * g.b_expert_stride);
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = k_begin; k0 < k_end; k0 += kSimtBK) {
    // ---- A tile -> As[k][m]
    if constexpr (MODE == kWgrad) {
      const int k = tid >> 4, mq = (tid & 15) * 4;
      const bool kin = (k0 + k) < k_end;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int m = row0 + mq + i;
        As[k][mq + i] = (kin && m < m_limit) ? DT<T>::ld(A + (size_t)(k0 + k) * g.lda + m) : 0.f;
      }
    } else {
      const int m = tid >> 2, kq = (tid & 3) * 4;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int k = k0 + kq + i;
        As[kq + i][m] = (k < k_end) ? DT<T>::ld(A + (size_t)(row0 + m) * g.lda + k) : 0.f;
      }
    }
    // ---- B tile -> Bs[k][n]
    if constexpr (MODE == kDgrad) {
      const int n = tid >> 2, kq = (tid & 3) * 4;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int k = k0 + kq + i;
        Bs[kq + i][n] = (k < k_end && (n0 + n) < g.N) ? DT<T>::ld(B + (size_t)(n0 + n) * g.ldb + k) : 0.f;
      }
    } else {
      const int k = tid >> 4, nq = (tid & 15) * 4;
      const bool kin = (k0 + k) < k_end;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int n = n0 + nq + i;
        Bs[k][nq + i] = (kin && n < g.N) ? DT<T>::ld(B + (size_t)(k0 + k) * g.ldb + n) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kSimtBK; ++kk) {
      const float4 a4 = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
      const float4 b4 = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
      const float a[4] = {a4.x, a4.y, a4.z, a4.w};
      const float b[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
  const int n = n0 + tx * 4;
  if (n >= g.N) return;
#pragma unroll
  for (int i = 0; i < 4; ++i) epi.template apply<4>(e, row0 + ty * 4 + i, n, acc[i]);
}

template <typename T, int MODE, class Epi>
inline void launch_simt_gemm(const GemmArgs& g, const Epi& epi, int64_t max_rows, cudaStream_t stream) {
  dim3 grid;
  grid.x = (unsigned)ceil_div(g.N, kSimtBN);
  if (MODE == kWgrad) {
    grid.y = (unsigned)ceil_div(g.M, kSimtBM);
    grid.z = (unsigned)g.E;
  } else {
    grid.y = (unsigned)ceil_div(max_rows, kSimtBM);
    grid.z = 1;
  }
  simt_gemm_kernel<T, MODE, Epi><<<grid, kSimtThreads, 0, stream>>>(g, epi);
}

}  // namespace yb
