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
// 128x128 or 64x128 output tile, 16-deep k slices, 256 threads, 8x8 or 4x8 accumulators per thread.
#pragma once
#include "common.cuh"
#include "epilogues.cuh"

namespace yb {

enum GemmMode { kFwd = 0, kDgrad = 1, kWgrad = 2 };

// Optional gate of a row-tiled tcgen05 GEMM that is launched while the kernel that fills its A rows
// is still running (programmatic dependent launch): the kernel starts only once *prep has reached
// prep_target (tables complete), and loads the A rows of group e only once arrived[e] >= needed[e].
// Both waits poll local memory, are bounded by wait_ns and record a device status when they give up.
struct GemmGate {
  const int32_t* prep = nullptr;
  int prep_target = 0;
  const int32_t* arrived = nullptr;
  const int32_t* needed = nullptr;
  unsigned long long wait_ns = 0;
};

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
  const int32_t* counts = nullptr;        // rows present per expert: lets the CUDA-core kernel skip all-padding tiles
  // tcgen05 kFwd only: A is the UN-permuted source [gather_src_rows, K]; row r of the padded layout
  // is source row gather_rows[r] (negative = padding), fetched by TMA gather
  const int32_t* gather_rows = nullptr;
  int64_t gather_src_rows = 0;
  // row-tiled arrangements without tables (tile_expert == nullptr): one group (expert 0) owns the
  // a_rows rows of A; rows at and beyond a_rows read as zeros
  int64_t a_rows = 0;
  GemmGate gate;                          // tcgen05 kFwd only
};

constexpr int kSimtBN = 128, kSimtBK = 16, kSimtThreads = 256;

// NL consecutive elements of a row as fp32 (16-byte loads when `vec`); zeros when `ok` is false.
// `p` must be 16-byte aligned when `vec` is set.
template <typename T, int NL>
__device__ __forceinline__ void simt_load(const T* __restrict__ p, bool ok, bool vec, float (&v)[NL]) {
  if (!ok) {
#pragma unroll
    for (int i = 0; i < NL; ++i) v[i] = 0.f;
  } else if (vec) {
    load_vec<T, NL>(p, v);
  } else {
#pragma unroll
    for (int i = 0; i < NL; ++i) v[i] = DT<T>::ld(p + i);
  }
}

// BM x 128 x 16 tiles (BM = 128 or 64), 256 threads, (BM/16) x 8 accumulators per thread in 4-wide
// groups 64 apart, so shared-memory reads are conflict-free 16-byte loads; the next k-tile is fetched
// into registers while the current one is multiplied (two shared-memory buffers, one barrier per
// k-tile).  BM = 64 is for problems with few rows per expert: a 64-row tile that lies entirely in
// an expert's padding skips its main loop.  K, N and the row strides are multiples of 8 on every
// path that reaches this kernel.
template <typename T, int MODE, int BM, class Epi>
__global__ void __launch_bounds__(kSimtThreads, 2)
simt_gemm_kernel(GemmArgs g, Epi epi) {
  constexpr int RT = BM / 16;              // rows per thread = elements of A fetched per thread
  __shared__ __align__(16) float As[2][kSimtBK][BM + 4];
  __shared__ __align__(16) float Bs[2][kSimtBK][kSimtBN + 4];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int n0 = blockIdx.x * kSimtBN;
  int e, row0, k_begin, k_end, m_limit;
  if constexpr (MODE == kWgrad) {
    e = blockIdx.z;
    row0 = blockIdx.y * BM;                 // m0 within the expert's output
    k_begin = g.pad_off[e];
    k_end = g.pad_off[e + 1];
    m_limit = g.M;
  } else {
    row0 = blockIdx.y * BM;                 // padded row
    if (g.tile_expert == nullptr) {
      if (row0 >= g.a_rows) return;
      e = 0;
    } else {
      if (row0 >= g.header[kHdrRowsUsed]) return;
      e = g.tile_expert[row0 / kTileM];
    }
    k_begin = 0;
    k_end = g.K;
    m_limit = row0 + BM;
    if (g.counts != nullptr) {              // nothing but padding in this tile: zeros, no main loop
      const int begin = g.pad_off[e];
      const int have = min(g.counts[e], g.pad_off[e + 1] - begin);
      if (row0 - begin >= have) k_end = 0;
    }
  }
  const T* __restrict__ A = reinterpret_cast<const T*>(g.A);
  const T* __restrict__ B = reinterpret_cast<const T*>(g.B) + (MODE == kWgrad ? 0 : (size_t)e * g.b_expert_stride);
  constexpr int kAlign = 16 / (int)sizeof(T);
  const bool vec_a = (g.lda % kAlign) == 0 && (reinterpret_cast<uintptr_t>(A) & 15) == 0 && RT % kAlign == 0;
  const bool vec_b = (g.ldb % kAlign) == 0 && (reinterpret_cast<uintptr_t>(B) & 15) == 0;

  // which elements of each operand tile this thread fetches
  //   A contiguous along k (rows x k):  RT elements at row tid / (16/RT), k offset (tid % (16/RT)) * RT
  //   A contiguous along m (wgrad):     RT elements at k = tid / 16, m offset (tid % 16) * RT
  //   B contiguous along k (dgrad):     8 elements at n = tid / 2, k offset (tid % 2) * 8
  //   B contiguous along n:             8 elements at k = tid / 16, n offset (tid % 16) * 8
  constexpr int TPR = 16 / RT;
  const int ak_row = tid / TPR, ak_k = (tid % TPR) * RT;
  const int am_k = tid >> 4, am_m = (tid & 15) * RT;
  const int bk_n = tid >> 1, bk_k = (tid & 1) * 8;
  const int bn_k = tid >> 4, bn_n = (tid & 15) * 8;
  float ra[RT], rb[8];
  auto fetch = [&](int k0) {
    if constexpr (MODE == kWgrad) {
      const int k = k0 + am_k, m = row0 + am_m;
      simt_load<T, RT>(A + (size_t)k * g.lda + m, k < k_end && m < m_limit, vec_a, ra);
    } else {
      const int k = k0 + ak_k;
      simt_load<T, RT>(A + (size_t)(row0 + ak_row) * g.lda + k, k < k_end && (g.a_rows == 0 || row0 + ak_row < g.a_rows),
                       vec_a, ra);
    }
    if constexpr (MODE == kDgrad) {
      const int k = k0 + bk_k, n = n0 + bk_n;
      simt_load<T, 8>(B + (size_t)n * g.ldb + k, k < k_end && n < g.N, vec_b, rb);
    } else {
      const int k = k0 + bn_k, n = n0 + bn_n;
      simt_load<T, 8>(B + (size_t)k * g.ldb + n, k < k_end && n < g.N, vec_b, rb);
    }
  };
  auto stage = [&](int buf) {
    if constexpr (MODE == kWgrad) {
#pragma unroll
      for (int i = 0; i < RT; i += 4)
        *reinterpret_cast<float4*>(&As[buf][am_k][am_m + i]) = make_float4(ra[i], ra[i + 1], ra[i + 2], ra[i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < RT; ++i) As[buf][ak_k + i][ak_row] = ra[i];
    }
    if constexpr (MODE == kDgrad) {
#pragma unroll
      for (int i = 0; i < 8; ++i) Bs[buf][bk_k + i][bk_n] = rb[i];
    } else {
      *reinterpret_cast<float4*>(&Bs[buf][bn_k][bn_n]) = make_float4(rb[0], rb[1], rb[2], rb[3]);
      *reinterpret_cast<float4*>(&Bs[buf][bn_k][bn_n + 4]) = make_float4(rb[4], rb[5], rb[6], rb[7]);
    }
  };

  float acc[RT][8];
#pragma unroll
  for (int i = 0; i < RT; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  int buf = 0;
  if (k_begin < k_end) {
    fetch(k_begin);
    stage(0);
  }
  __syncthreads();
  for (int k0 = k_begin; k0 < k_end; k0 += kSimtBK) {
    const bool more = k0 + kSimtBK < k_end;
    if (more) fetch(k0 + kSimtBK);
#pragma unroll
    for (int kk = 0; kk < kSimtBK; ++kk) {
      float a[RT], b[8];
#pragma unroll
      for (int h = 0; h < RT / 4; ++h) {
        const float4 q = *reinterpret_cast<const float4*>(&As[buf][kk][h * 64 + ty * 4]);
        a[4 * h] = q.x; a[4 * h + 1] = q.y; a[4 * h + 2] = q.z; a[4 * h + 3] = q.w;
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float4 q = *reinterpret_cast<const float4*>(&Bs[buf][kk][h * 64 + tx * 4]);
        b[4 * h] = q.x; b[4 * h + 1] = q.y; b[4 * h + 2] = q.z; b[4 * h + 3] = q.w;
      }
#pragma unroll
      for (int i = 0; i < RT; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    if (more) stage(buf ^ 1);
    __syncthreads();
    buf ^= 1;
  }
#pragma unroll
  for (int i = 0; i < RT; ++i) {
    const int row = row0 + (i >> 2) * 64 + ty * 4 + (i & 3);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int n = n0 + h * 64 + tx * 4;
      if (n >= g.N) continue;
      const float v[4] = {acc[i][4 * h], acc[i][4 * h + 1], acc[i][4 * h + 2], acc[i][4 * h + 3]};
      epi.template apply<4>(e, row, n, v);
    }
  }
}

template <typename T, int MODE, class Epi>
inline void launch_simt_gemm(const GemmArgs& g, const Epi& epi, int64_t max_rows, cudaStream_t stream) {
  dim3 grid;
  grid.x = (unsigned)ceil_div(g.N, kSimtBN);
  if (MODE == kWgrad) {
    grid.y = (unsigned)ceil_div(g.M, 128);
    grid.z = (unsigned)g.E;
    simt_gemm_kernel<T, MODE, 128, Epi><<<grid, kSimtThreads, 0, stream>>>(g, epi);
    return;
  }
  grid.z = 1;
  // few rows per expert (the padded bound max_rows includes 128 spare rows per expert): 64-row tiles
  if (g.counts != nullptr && max_rows < (int64_t)640 * g.E) {
    grid.y = (unsigned)ceil_div(max_rows, 64);
    simt_gemm_kernel<T, MODE, 64, Epi><<<grid, kSimtThreads, 0, stream>>>(g, epi);
  } else {
    grid.y = (unsigned)ceil_div(max_rows, 128);
    simt_gemm_kernel<T, MODE, 128, Epi><<<grid, kSimtThreads, 0, stream>>>(g, epi);
  }
}

}  // namespace yb
