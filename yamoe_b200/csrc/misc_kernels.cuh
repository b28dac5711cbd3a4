// Memory-bound helper kernels around the grouped GEMMs: row gathers into the padded,
// expert-sorted layout, the fp32 -> storage cast of the combined output, bias-gradient column
// sums and the placement of routing-weight gradients.
#pragma once
#include "common.cuh"
#include "epilogues.cuh"

namespace yb {

constexpr int kRowWarps = 8;  // rows per CTA in the warp-per-row kernels

// dst[row, 0:H] = src[row_token[row], :], zeros for padding rows.  One warp per row, 16-byte
// accesses.  reference: csrc/gather.cu:6-66 (which writes a padded [E,C,H] buffer instead).
// Rows of dst are dst_ld elements apart; when dst_ld > H the columns behind the copy get
// (1, 0, 0, ...) for token rows and zeros for padding rows: a weight-gradient GEMM that takes dst as
// its transposed operand then yields, in output row H, the column sums of its other operand
// (the bias gradient, reference: csrc/experts_backward.cu:308).
template <typename T>
__global__ void __launch_bounds__(kRowWarps * 32)
gather_rows_kernel(const T* __restrict__ src, T* __restrict__ dst, const int32_t* __restrict__ row_token,
                   const int32_t* __restrict__ header, int H, int dst_ld) {
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x * kRowWarps + (threadIdx.x >> 5);
  if (row >= header[kHdrRowsUsed]) return;
  const int lane = threadIdx.x & 31;
  const int tok = row_token[row];
  const int nvec = H * (int)sizeof(T) / 16;
  uint4* d = reinterpret_cast<uint4*>(dst + (size_t)row * dst_ld);
  if (tok < 0) {
    for (int i = lane; i < nvec; i += 32) d[i] = make_uint4(0, 0, 0, 0);
  } else {
    const uint4* s = reinterpret_cast<const uint4*>(src + (size_t)tok * H);
    for (int i = lane; i < nvec; i += 32) d[i] = __ldg(s + i);
  }
  for (int j = H + lane; j < dst_ld; j += 32) DT<T>::st(dst + (size_t)row * dst_ld + j, (j == H && tok >= 0) ? 1.f : 0.f);
}

// Backward gather: gys[row, :] = grad_y[token, :] where grad_y is grad_out, or the sum of its K
// slot slices (reference: csrc/experts_backward.cu:224-228); also seeds the routing-weight
// gradient of the row with <grad_y[token], b_down[e]>, the bias part of <grad_y, y_e>
// (reference: csrc/experts_backward.cu:83-88).
template <typename T>
__global__ void __launch_bounds__(kRowWarps * 32)
gather_grad_kernel(const T* __restrict__ grad_out, int slots, const T* __restrict__ down_bias,
                   T* __restrict__ gys, float* __restrict__ gw_row, const int32_t* __restrict__ row_token,
                   const int32_t* __restrict__ tile_expert, const int32_t* __restrict__ header, int H) {
  const int row = blockIdx.x * kRowWarps + (threadIdx.x >> 5);
  if (row >= header[kHdrRowsUsed]) return;
  const int lane = threadIdx.x & 31;
  const int tok = row_token[row];
  constexpr int VE = 16 / (int)sizeof(T);
  const int nvec = H / VE;
  T* d = gys + (size_t)row * H;
  if (tok < 0) {
    for (int i = lane; i < nvec; i += 32) reinterpret_cast<uint4*>(d)[i] = make_uint4(0, 0, 0, 0);
    if (lane == 0) gw_row[row] = 0.f;
    return;
  }
  const int e = tile_expert[row / kTileM];
  const T* b = down_bias + (size_t)e * H;
  float dot = 0.f;
  for (int i = lane; i < nvec; i += 32) {
    float g[VE], bb[VE];
    load_vec<T, VE>(grad_out + ((size_t)tok * slots) * H + (size_t)i * VE, g);
    for (int s = 1; s < slots; ++s) {
      float g2[VE];
      load_vec<T, VE>(grad_out + ((size_t)tok * slots + s) * H + (size_t)i * VE, g2);
#pragma unroll
      for (int j = 0; j < VE; ++j) g[j] += g2[j];
    }
    store_vec<T, VE>(d + (size_t)i * VE, g);
    load_vec<T, VE>(b + (size_t)i * VE, bb);
#pragma unroll
    for (int j = 0; j < VE; ++j) dot += g[j] * bb[j];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
  if (lane == 0) gw_row[row] = dot;
}

// out[i] = (T) acc[i]
template <typename T>
__global__ void cast_kernel(const float* __restrict__ acc, T* __restrict__ out, int64_t n_vec4) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n_vec4; i += stride) {
    float4 q = __ldg(reinterpret_cast<const float4*>(acc) + i);
    const float v[4] = {q.x, q.y, q.z, q.w};
    store_vec<T, 4>(out + i * 4, v);
  }
}

// dst[e, n] = sum over the kept rows r of expert e of  w_r * src[r, n]   (WEIGHTED)
//                                                  or       src[r, n]
// reference: csrc/experts_backward.cu:277 (down bias), :308 (gate_up bias).  fp32 accumulation.
// grid (ceil(N / (32 * elements per 16 bytes)), E); empty experts get exact zeros.
template <typename T, bool WEIGHTED>
__global__ void __launch_bounds__(256)
colsum_kernel(const T* __restrict__ src, const float* __restrict__ row_weight,
              const int32_t* __restrict__ pad_off, const int32_t* __restrict__ counts, int64_t capacity,
              T* __restrict__ dst, int N) {
  // 256 columns per CTA: a lane owns VE adjacent columns (one 16-byte load), the 8 warps take
  // every 8th row, partial sums meet in shared memory.
  constexpr int VE = 16 / (int)sizeof(T);
  constexpr int CPB = 32 * VE;                 // columns per CTA
  __shared__ float part[8][CPB];
  const int e = blockIdx.y;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int n = blockIdx.x * CPB + lane * VE;
  const int r0 = pad_off[e];
  const int c = counts[e];
  const int kept = (int64_t)c < capacity ? c : (int)capacity;
  float acc[VE];
#pragma unroll
  for (int j = 0; j < VE; ++j) acc[j] = 0.f;
  if (n < N) {
    int r = w;
    for (; r + 24 < kept; r += 32) {           // four rows in flight per warp
      float v[4][VE];
#pragma unroll
      for (int u = 0; u < 4; ++u) load_vec<T, VE>(src + (size_t)(r0 + r + 8 * u) * N + n, v[u]);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float wgt = WEIGHTED ? row_weight[r0 + r + 8 * u] : 1.0f;
#pragma unroll
        for (int j = 0; j < VE; ++j) acc[j] = fmaf(wgt, v[u][j], acc[j]);
      }
    }
    for (; r < kept; r += 8) {
      float v[VE];
      load_vec<T, VE>(src + (size_t)(r0 + r) * N + n, v);
      const float wgt = WEIGHTED ? row_weight[r0 + r] : 1.0f;
#pragma unroll
      for (int j = 0; j < VE; ++j) acc[j] = fmaf(wgt, v[j], acc[j]);
    }
  }
#pragma unroll
  for (int j = 0; j < VE; ++j) part[w][lane * VE + j] = acc[j];
  __syncthreads();
  for (int col = threadIdx.x; col < CPB; col += 256) {
    if (blockIdx.x * CPB + col >= N) continue;
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) s += part[k][col];
    DT<T>::st(dst + (size_t)e * N + blockIdx.x * CPB + col, s);
  }
}

// d_routing[t, e] (dense) or d_routing[t, slot] = gw_row[row] for every kept row.
// reference: csrc/experts_backward.cu:266-274 (placement), with the sort permutation applied once.
template <typename T>
__global__ void routing_grad_kernel(const float* __restrict__ gw_row, const int32_t* __restrict__ row_token,
                                    const int32_t* __restrict__ row_flat, const int32_t* __restrict__ tile_expert,
                                    const int32_t* __restrict__ header, T* __restrict__ d_routing,
                                    int routing_cols, int E) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= header[kHdrRowsUsed]) return;
  const int tok = row_token[row];
  if (tok < 0) return;
  const size_t idx = (routing_cols == E) ? (size_t)tok * E + tile_expert[row / kTileM] : (size_t)row_flat[row];
  DT<T>::st(d_routing + idx, gw_row[row]);
}

// out[t, :] = sum over the kept slots k of y[flat_row[t*K + k], :]   (rows already weighted).
// Second half of the combine (reference: csrc/scatter.cu:67-108): fp32 accumulation in slot
// order, one rounding, every output element written exactly once (no zero-fill, no atomics).
template <typename T>
__global__ void __launch_bounds__(kRowWarps * 32)
combine_padded_kernel(const T* __restrict__ y, const int32_t* __restrict__ flat_row, T* __restrict__ out,
                      int64_t Tn, int H, int K) {
  pdl_wait();
  const int64_t t = (int64_t)blockIdx.x * kRowWarps + (threadIdx.x >> 5);
  if (t >= Tn) return;
  const int lane = threadIdx.x & 31;
  constexpr int VE = 16 / (int)sizeof(T);
  const int nvec = H / VE;
  int32_t r[8];
  const int kk = K < 8 ? K : 8;
  for (int k = 0; k < kk; ++k) r[k] = flat_row[t * K + k];
  for (int i = lane; i < nvec; i += 32) {
    float acc[VE];
#pragma unroll
    for (int j = 0; j < VE; ++j) acc[j] = 0.f;
    for (int k = 0; k < K; ++k) {
      const int32_t row = k < 8 ? r[k] : flat_row[t * K + k];
      if (row < 0) continue;
      float v[VE];
      load_vec<T, VE>(y + (size_t)row * H + (size_t)i * VE, v);
#pragma unroll
      for (int j = 0; j < VE; ++j) acc[j] += v[j];
    }
    store_vec<T, VE>(out + (size_t)t * H + (size_t)i * VE, acc);
  }
}

// ---- expert-parallel helpers ---------------------------------------------------------------
// dst[j, :] = src[sorted_indices[j] / K, :]: rows in expert-sorted order, ready to be sent to
// the ranks that own the experts.  One warp per row, 16-byte accesses.
template <typename T>
__global__ void __launch_bounds__(kRowWarps * 32)
permute_rows_kernel(const T* __restrict__ src, const int32_t* __restrict__ sorted_indices, T* __restrict__ dst,
                    int64_t S, int H, int K, int64_t n_src) {
  const int64_t row = (int64_t)blockIdx.x * kRowWarps + (threadIdx.x >> 5);
  if (row >= S) return;
  const int lane = threadIdx.x & 31;
  const int flat = sorted_indices[row];
  const int nvec = H * (int)sizeof(T) / 16;
  uint4* d = reinterpret_cast<uint4*>(dst + (size_t)row * H);
  if (flat < 0 || flat / K >= n_src) {          // entry of a dropped assignment (-1): a zero row
    for (int i = lane; i < nvec; i += 32) d[i] = make_uint4(0, 0, 0, 0);
    return;
  }
  const uint4* s = reinterpret_cast<const uint4*>(src + (size_t)(flat / K) * H);
  for (int i = lane; i < nvec; i += 32) d[i] = __ldg(s + i);
}

// inv[sorted_indices[j]] = j; entries outside [0, n_flat) (the -1 tail left for dropped assignments) are skipped
__global__ void invert_perm_kernel(const int32_t* __restrict__ sorted_indices, int32_t* __restrict__ inv, int64_t S,
                                   int64_t n_flat) {
  const int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= S) return;
  const int32_t p = sorted_indices[j];
  if (p >= 0 && p < n_flat) inv[p] = (int32_t)j;
}

// out[t, :] = sum_k w[t, k] * rows[inv[t*K + k], :]   (fp32 accumulation, fixed order, one rounding).
// The weighted combine of csrc/scatter.cu:67-108 for rows that came back from the expert owners.
template <typename T>
__global__ void __launch_bounds__(kRowWarps * 32)
combine_rows_kernel(const T* __restrict__ rows, const int32_t* __restrict__ inv,
                    const int64_t* __restrict__ router_indices, const T* __restrict__ routing_weights,
                    int routing_cols, T* __restrict__ out, int64_t Tn, int H, int E, int K) {
  const int64_t t = (int64_t)blockIdx.x * kRowWarps + (threadIdx.x >> 5);
  if (t >= Tn) return;
  const int lane = threadIdx.x & 31;
  constexpr int VE = 16 / (int)sizeof(T);
  const int nvec = H / VE;
  for (int i = lane; i < nvec; i += 32) {
    float acc[VE];
#pragma unroll
    for (int j = 0; j < VE; ++j) acc[j] = 0.f;
    for (int k = 0; k < K; ++k) {
      const int32_t r = inv[t * K + k];
      if (r < 0) continue;
      const int col = (routing_cols == E) ? (int)router_indices[t * K + k] : k;
      const float w = DT<T>::ld(routing_weights + (size_t)t * routing_cols + col);
      float v[VE];
      load_vec<T, VE>(rows + (size_t)r * H + (size_t)i * VE, v);
#pragma unroll
      for (int j = 0; j < VE; ++j) acc[j] = fmaf(w, v[j], acc[j]);
    }
    store_vec<T, VE>(out + (size_t)t * H + (size_t)i * VE, acc);
  }
}

// ---- the reference's three small sub-operators on its padded [E, C, H] layout ------------------
// This library's own path never materialises [E, C, H]; these serve callers of the standalone ops.

// out[e, i, :] = x[indices[bins[e-1] + i] / top_k, :] for i < min(count_e, C), zeros otherwise.
// reference: csrc/gather.cu:7-66.  One warp per (e, i); VEC: 16-byte copies.
template <typename T, bool VEC>
__global__ void __launch_bounds__(kRowWarps * 32)
binned_gather_kernel(const T* __restrict__ x, const int32_t* __restrict__ indices, const int32_t* __restrict__ bins,
                     T* __restrict__ out, int64_t Tn, int H, int E, int C, int top_k) {
  const int64_t r = (int64_t)blockIdx.x * kRowWarps + (threadIdx.x >> 5);
  if (r >= (int64_t)E * C) return;
  const int lane = threadIdx.x & 31;
  const int e = (int)(r / C), i = (int)(r - (int64_t)e * C);
  const int start = e ? bins[e - 1] : 0;
  int64_t tok = -1;
  if (i < bins[e] - start) {
    tok = indices[start + i] / top_k;
    if (tok < 0 || tok >= Tn) tok = -1;
  }
  T* dst = out + (size_t)r * H;
  if constexpr (VEC) {
    const int nvec = H * (int)sizeof(T) / 16;
    uint4* d = reinterpret_cast<uint4*>(dst);
    if (tok < 0) {
      for (int v = lane; v < nvec; v += 32) d[v] = make_uint4(0, 0, 0, 0);
    } else {
      const uint4* sp = reinterpret_cast<const uint4*>(x + (size_t)tok * H);
      for (int v = lane; v < nvec; v += 32) d[v] = __ldg(sp + v);
    }
  } else {
    for (int h = lane; h < H; h += 32) DT<T>::st(dst + h, tok < 0 ? 0.f : DT<T>::ld(x + (size_t)tok * H + h));
  }
}

__device__ __forceinline__ void atomic_add_elem(float* p, float v) { atomicAdd(p, v); }
__device__ __forceinline__ void atomic_add_elem(__nv_bfloat16* p, float v) { atomicAdd(p, __float2bfloat16_rn(v)); }

// y[tok, :] += weights[start + i] * src[e, i, :] for i < min(count_e, C).
// reference: csrc/scatter.cu:67-108: the product is rounded to the storage type, then added
// atomically with one rounding per addition; the order of a token's K additions is not fixed
// there either.  One warp per (e, i).
template <typename T>
__global__ void __launch_bounds__(kRowWarps * 32)
binned_scatter_kernel(const T* __restrict__ src, const int32_t* __restrict__ indices,
                      const int32_t* __restrict__ bins, const T* __restrict__ weights, T* __restrict__ y,
                      int64_t Tn, int H, int E, int C, int top_k) {
  const int64_t r = (int64_t)blockIdx.x * kRowWarps + (threadIdx.x >> 5);
  if (r >= (int64_t)E * C) return;
  const int lane = threadIdx.x & 31;
  const int e = (int)(r / C), i = (int)(r - (int64_t)e * C);
  const int start = e ? bins[e - 1] : 0;
  if (i >= bins[e] - start) return;
  const int64_t tok = indices[start + i] / top_k;
  if (tok < 0 || tok >= Tn) return;
  const float scale = weights != nullptr ? DT<T>::ld(weights + start + i) : 1.0f;
  const T* sp = src + (size_t)r * H;
  T* yp = y + (size_t)tok * H;
  if constexpr (sizeof(T) == 2) {
    if ((H & 1) == 0 && (reinterpret_cast<uintptr_t>(yp) & 3) == 0 && (reinterpret_cast<uintptr_t>(sp) & 3) == 0) {
      for (int h = 2 * lane; h < H; h += 64) {
        const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(sp + h);
        atomicAdd(reinterpret_cast<__nv_bfloat162*>(yp + h),
                  __floats2bfloat162_rn(__low2float(v) * scale, __high2float(v) * scale));
      }
      return;
    }
  }
  for (int h = lane; h < H; h += 32) {
    float p = DT<T>::ld(sp + h) * scale;
    if constexpr (sizeof(T) == 2) p = __bfloat162float(__float2bfloat16_rn(p));
    atomic_add_elem(yp + h, p);
  }
}

// out[i] = in[idx[i]]    reference: csrc/index_select.cu:7-16
template <typename T>
__global__ void index_select_kernel(const T* __restrict__ in, const int32_t* __restrict__ idx, T* __restrict__ out,
                                    int64_t N) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < N) out[i] = in[(int64_t)idx[i]];
}

}  // namespace yb
