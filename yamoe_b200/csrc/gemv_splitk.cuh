// Decode path, second arrangement: split the REDUCTION dimension over CTAs so that every CTA
// streams whole, contiguous weight rows.
//
// The slab arrangement (gemv.cuh) gives a CTA a 64- or 128-column slab of one expert's matrix:
// 128/256-byte pieces at an 11.5 KB stride, which costs DRAM efficiency, and at T = 1 too few
// CTAs.  Here a CTA owns (touched expert, band of weight rows k0..k1): it reads rows that are
// fully contiguous in memory (all N columns), multiplies them with its band of the input rows and
// adds its partial result with vector fp32 reductions:
//   stage one  pre32[p, 0:2H] += x_t[k0:k1] . W_gu[e][k0:k1, :]            (p = t*K + slot)
//   stage two  out32[t, 0:H]  += w_p * ( glu(pre32[p] + b_gu[e])[k0:k1] . W_d[e][k0:k1, :] ), band 0
//              also adds w_p * b_d[e]; the GLU is applied while the band is staged
//   stage three rounds out32 to the bf16 output.
// pre32 must be zero on entry (one memset); stage one also zeroes out32 for stage two.  The
// number of bands is chosen so that about three CTAs per SM exist whatever the token count.
// Routing is rebuilt per CTA exactly as in gemv.cuh.
#pragma once
#include <cstring>

#include "gemv.cuh"

namespace yb {

constexpr int kSkMaxGroups = 3;     // column groups of 2048 (256 threads x 8) a thread may own: N <= 6144

struct GemvSkArgs {
  const __nv_bfloat16* hidden;      // [T, H]
  const int64_t* router_indices;    // [T, K]
  const __nv_bfloat16* routing_weights;
  int routing_cols;
  const __nv_bfloat16* W;           // stage one: gate_up [E,H,2H]; stage two: down [E,H,H]
  const __nv_bfloat16* bias_gu;     // [E, 2H]
  const __nv_bfloat16* bias_d;      // [E, H]
  float* pre32;                     // [S, 2H]
  float* out32;                     // [T, H]
  int S, E, K, H, T, bands;
  int64_t capacity;
};

// In-CTA routing shared by both stages: returns the expert served by slot blockIdx.x (or -1),
// fills rows[] with its assignments in stable order and returns their kept count.
__device__ __forceinline__ int gemv_sk_route(const GemvSkArgs& g, int32_t* cnt, int32_t* rows, int* s_warp,
                                             int* s_my_e, int& n_rows) {
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  for (int e = tid; e < g.E; e += kGemvThreads) cnt[e] = 0;
  if (tid == 0) *s_my_e = -1;
  __syncthreads();
  int my = -1;
  if (tid < g.S) {
    const int64_t v = g.router_indices[tid];
    if (v >= 0 && v < g.E) { my = (int)v; atomicAdd(&cnt[my], 1); }
  }
  __syncthreads();
  const int per = (g.E + kGemvThreads - 1) / kGemvThreads;
  const int e0 = tid * per;
  int local = 0;
  for (int i = 0; i < per; ++i) local += (e0 + i < g.E && cnt[e0 + i] > 0) ? 1 : 0;
  int incl = local;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  if (lane == 31) s_warp[w] = incl;
  __syncthreads();
  int base = 0;
  for (int i = 0; i < w; ++i) base += s_warp[i];
  int rank = base + incl - local;
  for (int i = 0; i < per; ++i) {
    if (e0 + i < g.E && cnt[e0 + i] > 0) {
      if (rank == (int)blockIdx.x) *s_my_e = e0 + i;
      ++rank;
    }
  }
  __syncthreads();
  const int e = *s_my_e;
  if (e < 0) return -1;
  const bool mine = (my == e);
  const unsigned bal = __ballot_sync(0xffffffffu, mine);
  __syncthreads();                       // s_warp is reused
  if (lane == 0) s_warp[w] = __popc(bal);
  __syncthreads();
  base = 0;
  for (int i = 0; i < w; ++i) base += s_warp[i];
  if (mine) rows[base + __popc(bal & ((1u << lane) - 1u))] = tid;
  __syncthreads();
  const int n_all = cnt[e];
  n_rows = (int64_t)n_all < g.capacity ? n_all : (int)g.capacity;
  return e;
}

// acc[m][g][j] += xs[m][kk] * W[k0+kk][(tid + 256 g) * 8 + j] over the band; four weight rows in flight.
template <int MT, int NG>
__device__ __forceinline__ void gemv_sk_accumulate(const __nv_bfloat16* __restrict__ wrow, int N, int nk,
                                                   const float* __restrict__ xs, int xs_pitch,
                                                   float (&acc)[kGemvMT][kSkMaxGroups][8]) {
  const int tid = threadIdx.x;
  bool ok[NG];
#pragma unroll
  for (int gq = 0; gq < NG; ++gq) ok[gq] = (tid + 256 * gq) * 8 < N;
  int kk = 0;
  for (; kk + 4 <= nk; kk += 4) {
    uint4 q[4][NG];
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int gq = 0; gq < NG; ++gq)
        q[u][gq] = ok[gq] ? __ldcs(reinterpret_cast<const uint4*>(wrow + (size_t)(kk + u) * N) + tid + 256 * gq)
                          : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float xv[MT];
#pragma unroll
      for (int m = 0; m < MT; ++m) xv[m] = xs[m * xs_pitch + kk + u];
#pragma unroll
      for (int gq = 0; gq < NG; ++gq) {
        float wv[8];
        unpack8(q[u][gq], wv);
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[m][gq][j] = fmaf(xv[m], wv[j], acc[m][gq][j]);
      }
    }
  }
  for (; kk < nk; ++kk) {
#pragma unroll
    for (int gq = 0; gq < NG; ++gq) {
      const uint4 q = ok[gq] ? __ldcs(reinterpret_cast<const uint4*>(wrow + (size_t)kk * N) + tid + 256 * gq)
                             : make_uint4(0, 0, 0, 0);
      float wv[8];
      unpack8(q, wv);
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const float xv = xs[m * xs_pitch + kk];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[m][gq][j] = fmaf(xv, wv[j], acc[m][gq][j]);
      }
    }
  }
}

template <int STAGE>
__global__ void __launch_bounds__(kGemvThreads)
gemv_sk_kernel(const GemvSkArgs g) {
  constexpr int NG = (STAGE == kGateUp) ? 3 : 2;        // column groups per thread (N <= 2048 * NG)
  extern __shared__ __align__(16) uint8_t sk_smem[];
  const int N = (STAGE == kGateUp) ? 2 * g.H : g.H;
  const int rb = (g.H + g.bands - 1) / g.bands;         // weight rows per band
  float* xs = reinterpret_cast<float*>(sk_smem);        // [MT][rb]
  int32_t* cnt = reinterpret_cast<int32_t*>(xs + kGemvMT * rb);
  int32_t* rows = cnt + g.E;
  __shared__ int s_warp[8];
  __shared__ int s_my_e;
  const int tid = threadIdx.x;
  if constexpr (STAGE == kGateUp) {
    // clear the accumulator of stage two (that launch starts after this one has finished)
    const size_t nthreads = (size_t)gridDim.x * gridDim.y * kGemvThreads;
    const size_t gtid = ((size_t)blockIdx.y * gridDim.x + blockIdx.x) * kGemvThreads + tid;
    const size_t nvec = (size_t)g.T * g.H / 4;
    for (size_t i = gtid; i < nvec; i += nthreads) reinterpret_cast<float4*>(g.out32)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  int n_rows = 0;
  const int e = gemv_sk_route(g, cnt, rows, s_warp, &s_my_e, n_rows);
  if (e < 0) return;
  const int k0 = blockIdx.y * rb;
  const int nk = min(rb, g.H - k0);
  if (nk <= 0) return;
  const __nv_bfloat16* wrow = g.W + ((size_t)e * g.H + k0) * N;

  for (int r0 = 0; r0 < n_rows; r0 += kGemvMT) {
    const int mt = min(kGemvMT, n_rows - r0);
    // stage this band of the input rows as fp32
    for (int i = tid; i < mt * nk; i += kGemvThreads) {
      const int m = i / nk, kk = i - m * nk;
      const int p = rows[r0 + m];
      float v;
      if constexpr (STAGE == kGateUp) {
        v = __bfloat162float(g.hidden[(size_t)(p / g.K) * g.H + k0 + kk]);
      } else {
        const float2 pr = __ldcg(reinterpret_cast<const float2*>(g.pre32 + (size_t)p * 2 * g.H) + k0 + kk);
        const float bg = __bfloat162float(g.bias_gu[(size_t)e * 2 * g.H + 2 * (k0 + kk)]);
        const float bu = __bfloat162float(g.bias_gu[(size_t)e * 2 * g.H + 2 * (k0 + kk) + 1]);
        v = __bfloat162float(__float2bfloat16_rn(glu_act(pr.x + bg, pr.y + bu)));   // same rounding as the GEMM path
      }
      xs[m * rb + kk] = v;
    }
    __syncthreads();
    float acc[kGemvMT][kSkMaxGroups][8];
#pragma unroll
    for (int m = 0; m < kGemvMT; ++m)
#pragma unroll
      for (int gq = 0; gq < kSkMaxGroups; ++gq)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[m][gq][j] = 0.f;
    if (mt == 1) gemv_sk_accumulate<1, NG>(wrow, N, nk, xs, rb, acc);
    else if (mt == 2) gemv_sk_accumulate<2, NG>(wrow, N, nk, xs, rb, acc);
    else if (mt == 3) gemv_sk_accumulate<3, NG>(wrow, N, nk, xs, rb, acc);
    else gemv_sk_accumulate<4, NG>(wrow, N, nk, xs, rb, acc);
    // partial results -> global fp32 accumulators
    for (int m = 0; m < mt; ++m) {
      const int p = rows[r0 + m];
      float scale = 1.f;
      float* dst;
      if constexpr (STAGE == kGateUp) {
        dst = g.pre32 + (size_t)p * N;
      } else {
        const int t = p / g.K;
        const int wc = (g.routing_cols == g.E) ? e : (p - t * g.K);
        scale = __bfloat162float(g.routing_weights[(size_t)t * g.routing_cols + wc]);
        dst = g.out32 + (size_t)t * N;
      }
#pragma unroll
      for (int gq = 0; gq < NG; ++gq) {
        const int col = (tid + 256 * gq) * 8;
        if (col >= N) continue;
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = acc[m][gq][j];
        if constexpr (STAGE == kDown) {
          if (blockIdx.y == 0) {
            float b[8];
            load_vec<__nv_bfloat16, 8>(g.bias_d + (size_t)e * N + col, b);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] += b[j];
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] *= scale;
        }
        red_add_vec<8>(dst + col, o);
      }
    }
    __syncthreads();
  }
}

}  // namespace yb

namespace yb {

// Which decode arrangement runs: YAMOE_B200_GEMV=slab|splitk overrides the default.
inline bool gemv_splitk_selected() {
  static int v = []() {
    const char* env = std::getenv("YAMOE_B200_GEMV");
    if (env && !std::strcmp(env, "slab")) return 0;
    if (env && !std::strcmp(env, "splitk")) return 1;
    return 1;
  }();
  return v != 0;
}

inline int gemv_sk_bands(int64_t S, int E, int H) {
  const int64_t slots = E < S ? E : S;
  int64_t bands = ceil_div(3 * 148, slots);
  const int64_t max_bands = H / 16 > 0 ? H / 16 : 1;
  if (bands > max_bands) bands = max_bands;
  if (bands < 1) bands = 1;
  return (int)bands;
}

// bf16 only.  pre32: S*2H floats, acc32: T*H floats (neither needs initialising).
inline int launch_gemv_splitk_forward(const void* hidden, const int64_t* ridx, const void* rw, int rcols,
                                      const void* wgu, const void* bgu, const void* wd, const void* bd, void* out,
                                      int64_t T, int H, int E, int K, int64_t cap, float* pre32, float* acc32,
                                      cudaStream_t st) {
  const int64_t S = T * K;
  if (S > kGemvMaxS || H % 8 != 0 || E > 1024 || 2 * H > 2048 * kSkMaxGroups) return YAMOE_ERR_UNSUPPORTED;
  using bf = __nv_bfloat16;
  GemvSkArgs g{reinterpret_cast<const bf*>(hidden), ridx, reinterpret_cast<const bf*>(rw), rcols,
               reinterpret_cast<const bf*>(wgu), reinterpret_cast<const bf*>(bgu), reinterpret_cast<const bf*>(bd),
               pre32, acc32, (int)S, E, K, H, (int)T, gemv_sk_bands(S, E, H), cap};
  const int rb = (int)ceil_div(H, g.bands);
  const size_t smem = (size_t)kGemvMT * rb * 4 + (size_t)E * 4 + kGemvMaxS * 4;
  static size_t configured = 0;
  if (smem > configured) {
    if (cudaFuncSetAttribute(gemv_sk_kernel<kGateUp>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
        cudaFuncSetAttribute(gemv_sk_kernel<kDown>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return YAMOE_ERR_UNSUPPORTED;
    configured = smem;
  }
  if (cudaMemsetAsync(pre32, 0, (size_t)S * 2 * H * sizeof(float), st) != cudaSuccess) return YAMOE_ERR_CUDA;
  const int slots = (int)(E < S ? E : S);
  dim3 grid((unsigned)slots, (unsigned)g.bands);
  {
    StageTimer tm(kStageGateUp, st);
    gemv_sk_kernel<kGateUp><<<grid, kGemvThreads, smem, st>>>(g);
  }
  GemvSkArgs g2 = g;
  g2.W = reinterpret_cast<const bf*>(wd);
  {
    StageTimer tm(kStageDown, st);
    gemv_sk_kernel<kDown><<<grid, kGemvThreads, smem, st>>>(g2);
  }
  const int64_t nv = T * H / 4;
  cast_kernel<bf><<<(unsigned)std::min<int64_t>(ceil_div(nv, 256), 148 * 8), 256, 0, st>>>(
      acc32, reinterpret_cast<bf*>(out), nv);
  return cudaGetLastError() == cudaSuccess ? YAMOE_OK : YAMOE_ERR_CUDA;
}

}  // namespace yb
