// Router tail of the MoE layer: top-k over the E router logits of a token, softmax over the k
// selected logits, and the dense [T, E] score row (zeros outside the selection), in one pass.
// Replaces the chain torch.topk -> softmax -> zeros_like().scatter_() of the reference layer
// (torch-ext/yamoe/layers.py:136-149; oracle torch-ext/yamoe/vendored/gpt_oss_mlp.py:127-139).
// One warp per token; each lane holds E/32 logits; k rounds of warp arg-max (ties resolve to the
// lower expert id); selected experts come out in descending logit order like torch.topk.
// The selection is total: NaN logits rank above everything (as torch.topk ranks them), -inf logits
// are still selectable once nothing larger is left, so every round picks a valid expert.
#pragma once
#include "common.cuh"

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

template <typename T>
inline int launch_router_topk(const void* logits, int64_t* indices, void* scores, int64_t Tn, int E, int K,
                              cudaStream_t st) {
  router_topk_kernel<T><<<(unsigned)ceil_div(Tn, 8), 256, 0, st>>>(reinterpret_cast<const T*>(logits), indices,
                                                                 reinterpret_cast<T*>(scores), Tn, E, K);
  return cudaGetLastError() == cudaSuccess ? YAMOE_OK : YAMOE_ERR_CUDA;
}

}  // namespace yb
