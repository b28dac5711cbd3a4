// Router tail of the MoE layer: top-k over the E router logits of a token, softmax over the k
// selected logits, and the dense [T, E] score row (zeros outside the selection), in one pass.
// Replaces the chain torch.topk -> softmax -> zeros_like().scatter_() of the reference layer
// (torch-ext/yamoe/layers.py:136-149; oracle torch-ext/yamoe/vendored/gpt_oss_mlp.py:127-139).
//
// launch_router_forward puts the router projection in front of it (torch-ext/yamoe/layers.py:126-131:
// logits = x W_r^T + b_r): for bf16 one tcgen05 GEMM whose epilogue holds a token's whole logit row in
// one thread and does the top-k, softmax and scatter there (EpiRouter: one kernel for the router);
// otherwise the CUDA-core GEMM writes the logits and router_topk_kernel follows.
//
// router_topk_kernel: one warp per token; each lane holds E/32 logits; k rounds of warp arg-max (ties resolve to the
// lower expert id); selected experts come out in descending logit order like torch.topk.
// The selection is total: NaN logits rank above everything (as torch.topk ranks them), -inf logits
// are still selectable once nothing larger is left, so every round picks a valid expert.
#pragma once
#include "common.cuh"
#include "epilogues.cuh"
#include "simt_gemm.cuh"
#include "umma_gemm.cuh"

namespace yb {

constexpr int kRouterMaxPerLane = 32;   // E <= 1024
constexpr int kRouterMaxK = 32;

template <typename T>
__global__ void __launch_bounds__(256)
router_topk_kernel(const T* __restrict__ logits, int64_t* __restrict__ indices, T* __restrict__ scores,
                   int64_t Tn, int E, int K) {
  const int64_t t = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t >= Tn) return;
  const int lane = threadIdx.x & 31;
  float v[kRouterMaxPerLane];
  const int per = (E + 31) / 32;
#pragma unroll
  for (int i = 0; i < kRouterMaxPerLane; ++i) {
    const int e = i * 32 + lane;
    v[i] = (i < per && e < E) ? DT<T>::ld(logits + t * E + e) : -INFINITY;
  }
  // zero the dense row
  for (int e = lane; e < E; e += 32) DT<T>::st(scores + t * E + e, 0.f);
  float sel_v = 0.f;      // lane k keeps the k-th selected logit
  int sel_e = 0;
  uint32_t taken = 0;     // bit i: this lane's i-th logit has been selected
  for (int k = 0; k < K; ++k) {
    float best = -INFINITY, best_raw = -INFINITY;    // ordering key (NaN -> +inf) and the logit itself
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kRouterMaxPerLane; ++i) {
      const int e = i * 32 + lane;
      const float key = (v[i] != v[i]) ? INFINITY : v[i];
      if (i < per && e < E && !((taken >> i) & 1u) && (best_e == 0x7fffffff || key > best)) {
        best = key; best_raw = v[i]; best_e = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const float orw = __shfl_xor_sync(0xffffffffu, best_raw, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (oe != 0x7fffffff && (best_e == 0x7fffffff || ov > best || (ov == best && oe < best_e))) {
        best = ov; best_raw = orw; best_e = oe;
      }
    }
    if (lane == k) { sel_v = best_raw; sel_e = best_e; }
    // remove the winner from its owner's candidates
    if (best_e != 0x7fffffff && (best_e & 31) == lane) taken |= 1u << (best_e >> 5);
  }
  // softmax over the K selected logits (lanes 0..K-1), in fp32
  const float mx = __shfl_sync(0xffffffffu, sel_v, 0);       // first selection is the maximum
  float ex = lane < K ? __expf(sel_v - mx) : 0.f;
  float sum = ex;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  __syncwarp();
  if (lane < K && sel_e < E) {
    indices[t * K + lane] = sel_e;
    DT<T>::st(scores + t * E + sel_e, ex / sum);
  }
}

// Order-preserving integer image of a logit: NaN ranks above everything (as torch.topk ranks it),
// -inf below every finite value but above kTakenKey.
constexpr int kTakenKey = INT32_MIN;
__device__ __forceinline__ int router_key(float v) {
  if (v != v) return INT32_MAX;
  const int b = __float_as_int(v);
  const int k = b >= 0 ? b : (b ^ 0x7fffffff);     // monotone in v; -0.0 just below +0.0
  return k == kTakenKey ? kTakenKey + 1 : k;
}

// Epilogue of the router GEMM (row-tiled, one group): a thread receives the NV-column chunks of its
// row one after the other, parks the biased logits (rounded to the storage type, like the output of
// the reference's F.linear) in its own row of `logits`, and after the last chunk selects the K
// largest, applies the softmax over them and writes indices and the dense score row.
template <typename T>
struct EpiRouter {
  const T* bias;             // [E] or null
  float* logits;             // [rows padded to the tile height, E] scratch
  int64_t* indices;          // [Tn, K]
  T* scores;                 // [Tn, E]
  int Tn, E, K;

  template <int NV>
  __device__ __forceinline__ void apply(int /*e*/, int row, int n0, const float (&v)[NV]) const {
    if (row >= Tn) return;
    float* mine = logits + (size_t)row * E;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      if (n0 + i < E) {
        float x = v[i] + (bias != nullptr ? DT<T>::ld(bias + n0 + i) : 0.f);
        if constexpr (sizeof(T) == 2) x = __bfloat162float(__float2bfloat16_rn(x));
        mine[n0 + i] = x;
      }
    }
    if (n0 + NV < E) return;                       // more chunks of this row follow (same thread)
    T* out = scores + (size_t)row * E;
    for (int e = 0; e < E; ++e) DT<T>::st(out + e, 0.f);
    float first = 0.f, sum = 0.f;
    float exv[kRouterMaxK];
    // pass 1: selection; a selected entry is overwritten by a NaN pattern that marks it as taken
    for (int k = 0; k < K; ++k) {
      int best_key = kTakenKey, best_e = -1;
      float best_v = 0.f;
      for (int e = 0; e < E; ++e) {
        const float x = mine[e];
        const int key = (__float_as_uint(x) == 0x7fc0dead) ? kTakenKey : router_key(x);
        if (key > best_key) { best_key = key; best_e = e; best_v = x; }     // ties: lower expert id stays
      }
      if (best_e < 0) break;                       // cannot happen while K <= E
      if (k == 0) first = best_v;                  // the first selection is the maximum
      const float ex = __expf(best_v - first);
      sum += ex;
      exv[k] = ex;
      indices[(size_t)row * K + k] = best_e;
      mine[best_e] = __uint_as_float(0x7fc0dead);
    }
    // pass 2: normalise the K selected entries
    for (int k = 0; k < K; ++k) DT<T>::st(out + indices[(size_t)row * K + k], exv[k] / sum);
  }
};

// Plain epilogue of the router GEMM for the two-kernel form: logits[row, n] = v + bias, storage type.
template <typename T>
struct EpiBiasRows {
  const T* bias;             // [N] or null
  T* C;                      // [rows, N]
  int rows, N;

  template <int NV>
  __device__ __forceinline__ void apply(int /*e*/, int row, int n0, const float (&v)[NV]) const {
    if (row >= rows) return;
#pragma unroll
    for (int i = 0; i < NV; ++i)
      if (n0 + i < N) DT<T>::st(C + (size_t)row * N + n0 + i, v[i] + (bias != nullptr ? DT<T>::ld(bias + n0 + i) : 0.f));
  }
};

template <typename T>
inline int launch_router_topk(const void* logits, int64_t* indices, void* scores, int64_t Tn, int E, int K,
                              cudaStream_t st) {
  router_topk_kernel<T><<<(unsigned)ceil_div(Tn, 8), 256, 0, st>>>(reinterpret_cast<const T*>(logits), indices,
                                                                 reinterpret_cast<T*>(scores), Tn, E, K);
  return cudaGetLastError() == cudaSuccess ? YAMOE_OK : YAMOE_ERR_CUDA;
}

// Scratch of launch_router_forward: a 64-byte header (device status) and one logit row per
// token, padded to the 128-row tile of the GEMM.
inline size_t router_workspace_bytes(int64_t Tn, int E) {
  return 256 + (size_t)round_up(Tn > 0 ? Tn : 1, kTileM) * E * sizeof(float);
}

template <typename T>
inline int launch_router_forward(const void* x, const void* w_router, const void* b_router, int64_t* indices,
                                 void* scores, int64_t Tn, int H, int E, int K, bool tcgen05_ok, void* ws,
                                 cudaStream_t st) {
  int32_t* header = reinterpret_cast<int32_t*>(ws);
  float* logits = reinterpret_cast<float*>(reinterpret_cast<char*>(ws) + 256);
  YB_CUDA_OK(cudaMemsetAsync(header, 0, 16 * sizeof(int32_t), st));
  const int64_t tiles = ceil_div(Tn, kTileM);
  // C[row, n] = sum_k x[row, k] * W_r[n, k]: the data-gradient arrangement with one group
  GemmArgs g{x, H, w_router, H, 0, 0, E, H, 1, nullptr, nullptr, header};
  g.a_rows = Tn;
  if constexpr (sizeof(T) == 2) {
    if (tcgen05_ok) {
      EpiRouter<T> epi{reinterpret_cast<const T*>(b_router), logits, indices, reinterpret_cast<T*>(scores), (int)Tn, E, K};
      return launch_umma_gemm<kDgrad>(g, epi, Tn, tiles, st);
    }
  }
  // two kernels: logits in the storage type, then top-k / softmax / scatter
  T* lg = reinterpret_cast<T*>(logits);
  EpiBiasRows<T> epi{reinterpret_cast<const T*>(b_router), lg, (int)Tn, E};
  launch_simt_gemm<T, kDgrad>(g, epi, tiles * kTileM, st);
  return launch_router_topk<T>(lg, indices, scores, Tn, E, K, st);
}

}  // namespace yb
