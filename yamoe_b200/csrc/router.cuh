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

// One warp: the K largest of one row of logits (generic pointer: global or shared memory), softmax
// over them in fp32, indices and the dense score row.  NaN ranks above everything; among equal
// values the lower expert id wins.
template <typename T>
__device__ __forceinline__ void router_select_row(const T* row_logits, int64_t* __restrict__ idx_row,
                                                  T* __restrict__ score_row, int E, int K, int lane) {
  float v[kRouterMaxPerLane];
  const int per = (E + 31) / 32;
#pragma unroll
  for (int i = 0; i < kRouterMaxPerLane; ++i) {
    const int e = i * 32 + lane;
    v[i] = (i < per && e < E) ? DT<T>::ld(row_logits + e) : -INFINITY;
  }
  // zero the dense row
  for (int e = lane; e < E; e += 32) DT<T>::st(score_row + e, 0.f);
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
    idx_row[lane] = sel_e;
    DT<T>::st(score_row + sel_e, ex / sum);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
router_topk_kernel(const T* __restrict__ logits, int64_t* __restrict__ indices, T* __restrict__ scores,
                   int64_t Tn, int E, int K) {
  const int64_t t = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t >= Tn) return;
  router_select_row<T>(logits + t * E, indices + t * K, scores + t * E, E, K, threadIdx.x & 31);
}

// Router for a handful of tokens (decode): CTA (t, g) computes the logits of token t for the eight
// experts 8g .. 8g+7, one warp per expert: a dot product over H read straight from the router
// weights, four 16-byte loads in flight per lane, fp32 accumulation, bias, rounding to the storage
// type like the output of the reference's F.linear.  The CTA that finishes last for a token (a
// ticket per token, zeroed before the launch) selects.  The 45 dependent k-blocks of the
// tensor-core kernel cost about 40 us whatever the number of rows; this form has T * E / 8 CTAs
// that each wait for a few loads.
constexpr int kRouterSmallMaxT = 64;

template <typename T>
__global__ void __launch_bounds__(256)
router_small_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ bias,
                    T* logits, int32_t* tickets, int64_t* __restrict__ indices, T* __restrict__ scores,
                    int H, int E, int K) {
  __shared__ int s_last;
  const int64_t t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int e = blockIdx.y * 8 + warp;
  constexpr int VE = 16 / (int)sizeof(T);
  const int nvec = H / VE;
  if (e < E) {
    const T* wr = w + (size_t)e * H;
    const T* xr = x + (size_t)t * H;
    float acc = 0.f;
    int i = lane;
    for (; i + 96 < nvec; i += 128) {
      float a[4][VE], b[4][VE];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        load_vec<T, VE>(wr + (size_t)(i + 32 * u) * VE, a[u]);
        load_vec<T, VE>(xr + (size_t)(i + 32 * u) * VE, b[u]);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int j = 0; j < VE; ++j) acc += a[u][j] * b[u][j];
    }
    for (; i < nvec; i += 32) {
      float a[VE], b[VE];
      load_vec<T, VE>(wr + (size_t)i * VE, a);
      load_vec<T, VE>(xr + (size_t)i * VE, b);
#pragma unroll
      for (int j = 0; j < VE; ++j) acc += a[j] * b[j];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) DT<T>::st(logits + t * E + e, acc + (bias != nullptr ? DT<T>::ld(bias + e) : 0.f));
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(tickets + t, 1) == (int)gridDim.y - 1;
  __syncthreads();
  if (s_last && warp == 0) {
    __threadfence();
    router_select_row<T>(logits + t * E, indices + t * K, scores + t * E, E, K, lane);
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

// Epilogue of the router GEMM (row-tiled, one group).  A thread receives the NV-column chunks of
// its row one after the other (ascending n0).  The logits of a chunk (biased, rounded to the
// storage type like the output of the reference's F.linear) and the K best entries so far stay in
// registers; between chunks the K best (value, expert) pairs rest in the thread's own slot of
// `state`.  After the last chunk the softmax over the K selected values goes out: indices, and the
// K non-zero entries of the dense score row (the row has been zero-filled before the launch).
// Rows with E <= NV (32 experts) never touch `state`.
constexpr int kRouterFusedMaxK = 8;

template <typename T>
struct EpiRouter {
  const T* bias;             // [E] or null
  float* state;              // [rows padded to the tile height, 2 * kRouterFusedMaxK] scratch
  int64_t* indices;          // [Tn, K]
  T* scores;                 // [Tn, E], zero-filled
  int Tn, E, K;

  template <int NV>
  __device__ __forceinline__ void apply(int /*e*/, int row, int n0, const float (&v)[NV]) const {
    static_assert(NV <= 32, "one bit per column of the chunk");
    if (row >= Tn) return;
    float x[NV];
    uint32_t taken_chunk = 0, taken_run = 0;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      float y = v[i] + ((bias != nullptr && n0 + i < E) ? DT<T>::ld(bias + n0 + i) : 0.f);
      if constexpr (sizeof(T) == 2) y = __bfloat162float(__float2bfloat16_rn(y));
      x[i] = y;
      if (n0 + i >= E) taken_chunk |= 1u << i;               // columns beyond E are never selected
    }
    // the K best of the earlier chunks (all of lower expert id than this chunk's)
    float rv[kRouterFusedMaxK];
    int re[kRouterFusedMaxK], rk[kRouterFusedMaxK];
    float* mine = state + (size_t)row * (2 * kRouterFusedMaxK);
#pragma unroll
    for (int j = 0; j < kRouterFusedMaxK; ++j) {
      const bool have = n0 > 0 && j < K;
      rv[j] = have ? mine[j] : 0.f;
      re[j] = have ? __float_as_int(mine[kRouterFusedMaxK + j]) : -1;
      rk[j] = have ? router_key(rv[j]) : kTakenKey;
    }
    // K selection passes over (earlier best, this chunk); a strictly greater key wins, so among
    // equal values the lower expert id stays (the earlier list is scanned first and is in order)
    float ov[kRouterFusedMaxK];
    int oe[kRouterFusedMaxK];
#pragma unroll
    for (int k = 0; k < kRouterFusedMaxK; ++k) {
      ov[k] = 0.f;
      oe[k] = -1;
      if (k < K) {
        int best_key = kTakenKey, best_e = -1, best_slot = -1;
        float best_v = 0.f;
#pragma unroll
        for (int j = 0; j < kRouterFusedMaxK; ++j)
          if (!((taken_run >> j) & 1u) && rk[j] > best_key) { best_key = rk[j]; best_e = re[j]; best_v = rv[j]; best_slot = j; }
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const int key = router_key(x[i]);
          if (!((taken_chunk >> i) & 1u) && key > best_key) { best_key = key; best_e = n0 + i; best_v = x[i]; best_slot = 32 + i; }
        }
        if (best_slot >= 32) taken_chunk |= 1u << (best_slot - 32);
        else if (best_slot >= 0) taken_run |= 1u << best_slot;
        ov[k] = best_v;
        oe[k] = best_e;
      }
    }
    if (n0 + NV < E) {                             // more chunks of this row follow (same thread)
#pragma unroll
      for (int k = 0; k < kRouterFusedMaxK; ++k)
        if (k < K) {
          mine[k] = ov[k];
          mine[kRouterFusedMaxK + k] = __int_as_float(oe[k]);
        }
      return;
    }
    // softmax over the selected values; the first selection is the maximum
    float ex[kRouterFusedMaxK], sum = 0.f;
#pragma unroll
    for (int k = 0; k < kRouterFusedMaxK; ++k) {
      ex[k] = k < K ? __expf(ov[k] - ov[0]) : 0.f;
      sum += ex[k];
    }
    T* out = scores + (size_t)row * E;
#pragma unroll
    for (int k = 0; k < kRouterFusedMaxK; ++k)
      if (k < K && oe[k] >= 0) {
        indices[(size_t)row * K + k] = oe[k];
        DT<T>::st(out + oe[k], ex[k] / sum);
      }
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

// Scratch of launch_router_forward: a header (device status), 64 tickets, and per token (padded
// to the 128-row tile of the GEMM) room for a logit row (two-kernel and few-token forms) or the
// selection state.
inline size_t router_workspace_bytes(int64_t Tn, int E) {
  return 512 + (size_t)round_up(Tn > 0 ? Tn : 1, kTileM) * (E > 2 * kRouterFusedMaxK ? E : 2 * kRouterFusedMaxK) * sizeof(float);
}

template <typename T>
inline int launch_router_forward(const void* x, const void* w_router, const void* b_router, int64_t* indices,
                                 void* scores, int64_t Tn, int H, int E, int K, bool tcgen05_ok, void* ws,
                                 cudaStream_t st) {
  int32_t* header = reinterpret_cast<int32_t*>(ws);
  int32_t* tickets = reinterpret_cast<int32_t*>(reinterpret_cast<char*>(ws) + 256);
  float* logits = reinterpret_cast<float*>(reinterpret_cast<char*>(ws) + 512);
  YB_CUDA_OK(cudaMemsetAsync(header, 0, 16 * sizeof(int32_t), st));
  if (Tn == 0) return YAMOE_OK;
  if (Tn <= kRouterSmallMaxT) {
    YB_CUDA_OK(cudaMemsetAsync(tickets, 0, kRouterSmallMaxT * sizeof(int32_t), st));
    router_small_kernel<T><<<dim3((unsigned)Tn, (unsigned)ceil_div(E, 8)), 256, 0, st>>>(
        reinterpret_cast<const T*>(x), reinterpret_cast<const T*>(w_router), reinterpret_cast<const T*>(b_router),
        reinterpret_cast<T*>(logits), tickets, indices, reinterpret_cast<T*>(scores), H, E, K);
    return cudaGetLastError() == cudaSuccess ? YAMOE_OK : YAMOE_ERR_CUDA;
  }
  const int64_t tiles = ceil_div(Tn, kTileM);
  // C[row, n] = sum_k x[row, k] * W_r[n, k]: the data-gradient arrangement with one group
  GemmArgs g{x, H, w_router, H, 0, 0, E, H, 1, nullptr, nullptr, header};
  g.a_rows = Tn;
  if constexpr (sizeof(T) == 2) {
    if (tcgen05_ok && K <= kRouterFusedMaxK) {
      YB_CUDA_OK(cudaMemsetAsync(scores, 0, (size_t)Tn * E * sizeof(T), st));
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
