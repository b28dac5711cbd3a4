// Routing: per-expert histogram, prefix sums and a stable counting sort of the S = T*K
// (token, slot) assignments, in two launches and without any device-wide spin wait.
//
// Replaces, bit for bit, what the reference computes with a CUB radix sort
// (csrc/sort.cu:17-59: ascending expert id, ties by ascending flat position) followed by
// bincount_cumsum (csrc/bincount_cumsum.cu:7-56: inclusive scan, slot E left at 0), the
// routing-weight gather (csrc/moe.cpp:199-203) and index_select (csrc/index_select.cu:7-16).
//
// Launch 1  route_count_kernel   one CTA per 2048 assignments: shared-memory histogram ->
//           block_counts[blk][e].  The CTA that takes the last ticket turns block_counts into
//           exclusive prefixes over blocks and derives counts, bins, the padded row offsets
//           and the tile -> expert table.
// Launch 2  route_place_kernel   same partition; every warp ranks its 256 assignments with
//           __match_any_sync ballots (stable within the warp), warps are chained through a
//           shared-memory prefix, blocks through block_counts; each assignment is written to
//           its sorted slot and to its row of the padded, expert-sorted layout.
#pragma once
#include "common.cuh"

namespace yb {

constexpr int kRouteThreads = 256;
constexpr int kRouteWarps = kRouteThreads / 32;
constexpr int kRouteRounds = 8;                                   // assignments per lane
constexpr int kRouteItems = kRouteThreads * kRouteRounds;         // assignments per CTA

__global__ void __launch_bounds__(kRouteThreads)
route_count_kernel(const int64_t* __restrict__ router_indices, int S, int E, int64_t capacity,
                   RouteTables rt, int nblk) {
  extern __shared__ int32_t smem_i[];
  int32_t* hist = smem_i;            // [E]
  int32_t* poff = smem_i + E;        // [E+1]
  int32_t* qoff = smem_i + 2 * E + 1;  // [E+1]
  __shared__ int is_last;
  const int tid = threadIdx.x;
  for (int e = tid; e < E; e += kRouteThreads) hist[e] = 0;
  __syncthreads();
  const int base = blockIdx.x * kRouteItems;
#pragma unroll
  for (int i = 0; i < kRouteRounds; ++i) {
    int j = base + i * kRouteThreads + tid;
    if (j < S) {
      int64_t e = router_indices[j];
      if (e >= 0 && e < E) atomicAdd(&hist[(int)e], 1);
    }
  }
  __syncthreads();
  for (int e = tid; e < E; e += kRouteThreads) rt.block_counts[(size_t)blockIdx.x * E + e] = hist[e];
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    int t = atomicAdd(&rt.header[kHdrTicket], 1);
    is_last = (t == nblk - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  for (int e = tid; e < E; e += kRouteThreads) {
    int run = 0;
    for (int b = 0; b < nblk; ++b) {
      volatile int32_t* p = rt.block_counts + (size_t)b * E + e;
      int c = *p;
      *p = run;
      run += c;
    }
    rt.counts[e] = run;
    hist[e] = run;
  }
  __syncthreads();
  if (tid == 0) {
    int cum = 0, rows = 0, dropped = 0, pairs = 0;
    for (int e = 0; e < E; ++e) {
      int c = hist[e];
      cum += c;
      rt.bins[e] = cum;
      int kept = (int64_t)c < capacity ? c : (int)capacity;
      dropped += c - kept;
      poff[e] = rows;
      rt.pad_off[e] = rows;
      qoff[e] = pairs;
      if (rt.pair_off != nullptr) rt.pair_off[e] = pairs;
      const int tiles = (kept + kTileM - 1) / kTileM;
      rows += tiles * kTileM;
      pairs += (tiles + 1) / 2;
    }
    poff[E] = rows;
    qoff[E] = pairs;
    if (rt.pair_off != nullptr) rt.pair_off[E] = pairs;
    rt.header[kHdrPairs] = pairs;
    rt.bins[E] = 0;
    rt.pad_off[E] = rows;
    rt.header[kHdrRowTiles] = rows / kTileM;
    rt.header[kHdrRowsUsed] = rows;
    rt.header[kHdrDropped] = dropped;
    rt.header[kHdrTicket] = 0;
  }
  __syncthreads();
  if (rt.tile_expert != nullptr) {
    for (int e = tid; e < E; e += kRouteThreads)
      for (int t = poff[e] / kTileM; t < poff[e + 1] / kTileM; ++t) rt.tile_expert[t] = e;
  }
  if (rt.pair_expert != nullptr) {
    for (int e = tid; e < E; e += kRouteThreads)
      for (int t = qoff[e]; t < qoff[e + 1]; ++t) rt.pair_expert[t] = e;
  }
}

template <typename T>
__global__ void __launch_bounds__(kRouteThreads)
route_place_kernel(const int64_t* __restrict__ router_indices, const T* __restrict__ routing_weights,
                   int routing_cols, int S, int E, int K, int64_t capacity, RouteTables rt) {
  extern __shared__ int32_t smem_i[];
  int32_t* wcnt = smem_i;  // [kRouteWarps][E]
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  for (int i = tid; i < kRouteWarps * E; i += kRouteThreads) wcnt[i] = 0;
  __syncthreads();
  const int base = blockIdx.x * kRouteItems + w * (32 * kRouteRounds);
  int ex[kRouteRounds];
#pragma unroll
  for (int i = 0; i < kRouteRounds; ++i) {
    int j = base + i * 32 + lane;
    int e = -1 - lane;  // unique negative key: never matches another lane
    if (j < S) {
      int64_t v = router_indices[j];
      if (v >= 0 && v < E) e = (int)v;
    }
    ex[i] = e;
  }
  int32_t* mine = wcnt + w * E;
#pragma unroll
  for (int i = 0; i < kRouteRounds; ++i) {
    unsigned mask = __match_any_sync(0xffffffffu, ex[i]);
    if (ex[i] >= 0 && (__ffs(mask) - 1) == lane) mine[ex[i]] += __popc(mask);
    __syncwarp();
  }
  __syncthreads();
  for (int e = tid; e < E; e += kRouteThreads) {
    int run = rt.block_counts[(size_t)blockIdx.x * E + e];
    for (int ww = 0; ww < kRouteWarps; ++ww) {
      int c = wcnt[ww * E + e];
      wcnt[ww * E + e] = run;
      run += c;
    }
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < kRouteRounds; ++i) {
    const int e = ex[i];
    unsigned mask = __match_any_sync(0xffffffffu, e);
    int pos = 0;
    if (e >= 0) pos = mine[e] + __popc(mask & ((1u << lane) - 1u));
    __syncwarp();
    if (e >= 0 && (__ffs(mask) - 1) == lane) mine[e] += __popc(mask);
    __syncwarp();
    if (e >= 0) {
      const int p = base + i * 32 + lane;
      const int start = e ? rt.bins[e - 1] : 0;
      rt.sorted_values[start + pos] = e;
      rt.sorted_indices[start + pos] = p;
      if (rt.flat_pos != nullptr) rt.flat_pos[p] = start + pos;
      if (rt.row_token != nullptr && (int64_t)pos < capacity) {
        const int r = rt.pad_off[e] + pos;
        const int t = p / K;
        rt.row_token[r] = t;
        rt.row_flat[r] = p;
        rt.flat_row[p] = r;
        const int col = (routing_cols == E) ? e : (p - t * K);
        rt.row_weight[r] = DT<T>::ld(routing_weights + (size_t)t * routing_cols + col);
      }
    }
  }
}

// Host-side launcher.  `rt` must point into zero-initialised header memory for the ticket
// (the caller memsets the header) and, when row tables are requested, row_token / row_flat
// must have been filled with -1.
template <typename T>
inline int launch_route(const int64_t* router_indices, const T* routing_weights, int routing_cols,
                        int64_t T_tokens, int E, int K, int64_t capacity, const RouteTables& rt,
                        cudaStream_t stream) {
  const int S = (int)(T_tokens * K);
  const int nblk = (int)ceil_div(S, kRouteItems);
  size_t smem1 = (size_t)(3 * E + 2) * sizeof(int32_t);
  size_t smem2 = (size_t)kRouteWarps * E * sizeof(int32_t);
  route_count_kernel<<<nblk, kRouteThreads, smem1, stream>>>(router_indices, S, E, capacity, rt, nblk);
  route_place_kernel<T><<<nblk, kRouteThreads, smem2, stream>>>(router_indices, routing_weights,
                                                               routing_cols, S, E, K, capacity, rt);
  return cudaGetLastError() == cudaSuccess ? YAMOE_OK : YAMOE_ERR_CUDA;
}

inline int route_blocks(int64_t S) { return (int)ceil_div(S, kRouteItems); }

}  // namespace yb
