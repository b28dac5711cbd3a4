// Expert parallelism over peer memory: the dispatch and combine exchanges as plain stores into
// the other GPUs' buffers (NVLink), with every offset derived on the device from the all-gathered
// [G, E] count matrix, so that a call needs no host round trip and no split sizes.
// The reference is single-GPU; there is no counterpart.
//
// Rank r owns experts [r*per, (r+1)*per) and a shard of the tokens.  Buffers that peers write
// into (symmetric allocations, one per rank, same size everywhere):
//   recv_x [max_rows, H]   rows of the experts this rank owns, already in the padded,
//                          expert-sorted layout the grouped GEMMs consume: expert le starts at
//                          pad_off[le]; inside it rows are ordered by source rank, then by the
//                          source's stable order (= global token order, which is what the
//                          capacity rule needs)
//   back_y [S_local, H]    result rows of this rank's assignments, in its own sorted order
//
//   ep_plan_kernel        count matrix -> where my rows start on each owner (dest_row), this
//                         rank's tile tables, and the (source, expert) segments for the way back
//   ep_rowtables_kernel   validity of every local row (padding and rows beyond the capacity)
//   ep_dispatch_kernel    hidden[token] -> recv_x of the owner, one warp per row, 16-byte stores
//   ep_return_kernel      y rows -> back_y of the source rank (zeros for dropped rows)
// The backward pass travels the same way: token rows and upstream-gradient rows with the row
// dispatch kernel, the routing weight of every assignment with ep_dispatch_weight_kernel; the
// input-gradient rows return through the dgrad GEMM's epilogue (EpiPeerRows without a bias) and
// the routing-weight gradients with ep_return_scalar_kernel.
// Peer loads are never used and nothing here waits on another GPU: the phases are separated by
// stream-ordered collectives issued by the host binding.
#pragma once
#include "common.cuh"
#include "misc_kernels.cuh"

namespace yb {

struct EpTables {
  RouteTables rt;          // tables of the LOCAL problem (per experts, padded rows)
  int32_t* dest_row;       // [E]      first row on the owner of expert e for rows sent by this rank
  int32_t* src_start;      // [G*per]  start of expert (r*per+le) in source s's sorted order
  int32_t* seg_row;        // [G*per]  first local row of the rows source s sent for local expert le
  int64_t* row_dest;       // [max_rows] address of the row's slot in its source rank's back buffer, 0 for padding
};

// One CTA.  counts_all[s*E + e] = assignments of source rank s to global expert e.
__global__ void __launch_bounds__(256)
ep_plan_kernel(const int32_t* __restrict__ counts_all, int G, int rank, int E, EpTables t) {
  extern __shared__ int32_t sm[];
  int32_t* tot = sm;               // [E] rows of expert e over all sources
  int32_t* before = sm + E;        // [E] rows of expert e from sources s < rank
  int32_t* poff = sm + 2 * E;      // [E] padded row offset of e inside its owner
  const int per = E / G, tid = threadIdx.x;
  for (int e = tid; e < E; e += 256) {
    int a = 0, b = 0;
    for (int s = 0; s < G; ++s) {
      const int c = counts_all[s * E + e];
      if (s < rank) b += c;
      a += c;
    }
    tot[e] = a;
    before[e] = b;
  }
  __syncthreads();
  if (tid < G) {                   // padded offsets inside owner `tid`
    int rows = 0;
    for (int le = 0; le < per; ++le) {
      const int e = tid * per + le;
      poff[e] = rows;
      rows += (tot[e] + kTileM - 1) / kTileM * kTileM;
    }
  }
  __syncthreads();
  for (int e = tid; e < E; e += 256) t.dest_row[e] = poff[e] + before[e];
  // return segments: for every source s and local expert le
  for (int i = tid; i < G * per; i += 256) {
    const int s = i / per, le = i - s * per, e = rank * per + le;
    int start = 0;
    for (int e2 = 0; e2 < e; ++e2) start += counts_all[s * E + e2];
    int row = poff[e];
    for (int s2 = 0; s2 < s; ++s2) row += counts_all[s2 * E + e];
    t.src_start[i] = start;
    t.seg_row[i] = row;
  }
  // local tile tables
  if (tid == 0) {
    int rows = 0, pairs = 0, cum = 0;
    for (int le = 0; le < per; ++le) {
      const int c = tot[rank * per + le];
      cum += c;
      t.rt.counts[le] = c;
      t.rt.bins[le] = cum;
      t.rt.pad_off[le] = rows;
      t.rt.pair_off[le] = pairs;
      const int tiles = (c + kTileM - 1) / kTileM;
      rows += tiles * kTileM;
      pairs += (tiles + 1) / 2;
    }
    t.rt.bins[per] = 0;
    t.rt.pad_off[per] = rows;
    t.rt.pair_off[per] = pairs;
    t.rt.header[kHdrRowTiles] = rows / kTileM;
    t.rt.header[kHdrRowsUsed] = rows;
    t.rt.header[kHdrPairs] = pairs;
    t.rt.header[kHdrDropped] = 0;
  }
  __syncthreads();
  for (int le = tid; le < per; le += 256) {
    const int e = rank * per + le;
    const int tiles = (tot[e] + kTileM - 1) / kTileM;
    const int t0 = poff[e] / kTileM;
    for (int k = 0; k < tiles; ++k) t.rt.tile_expert[t0 + k] = le;
  }
  __syncthreads();
  if (tid == 0) {                  // pair -> expert (serial: pair offsets are only in global memory)
    int pairs = 0;
    for (int le = 0; le < per; ++le) {
      const int tiles = (tot[rank * per + le] + kTileM - 1) / kTileM;
      for (int k = 0; k < (tiles + 1) / 2; ++k) t.rt.pair_expert[pairs++] = le;
    }
  }
}

// row_token[r] = r for kept rows, -1 for padding and for rows beyond the capacity; weight 1;
// row_dest[r] = where the row's result goes in the peer memory of the rank it came from.
__global__ void ep_rowtables_kernel(EpTables t, int64_t capacity, int64_t max_rows, void* const* peer_back,
                                    int G, int per, int64_t row_bytes) {
  const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= max_rows) return;
  int32_t tok = -1;
  int64_t dest = 0;
  if (r < t.rt.header[kHdrRowsUsed]) {
    const int le = t.rt.tile_expert[r / kTileM];
    const int64_t i = r - t.rt.pad_off[le];
    const int64_t c = t.rt.counts[le];
    if (i < (c < capacity ? c : capacity)) tok = (int32_t)r;
    if (i < c && peer_back != nullptr) {
      int s = 0;
      while (s + 1 < G && t.seg_row[(s + 1) * per + le] <= r) ++s;
      const int64_t dst_row = (int64_t)t.src_start[s * per + le] + (r - t.seg_row[s * per + le]);
      dest = reinterpret_cast<int64_t>(peer_back[s]) + dst_row * row_bytes;
    }
  }
  t.rt.row_token[r] = tok;
  t.rt.row_weight[r] = 1.0f;
  t.row_dest[r] = dest;
}

// Down-projection epilogue fused with the combine exchange: the bias-added result row goes
// straight into the back buffer of the rank that owns the token (a peer store over NVLink);
// rows dropped by the capacity send zeros, padding rows send nothing.
template <typename T>
struct EpiPeerRows {
  const T* bias;             // [per, N], or nullptr
  const int64_t* row_dest;
  const int32_t* row_token;
  int N;

  template <int NV>
  __device__ __forceinline__ void apply(int e, int row, int n0, const float (&v)[NV]) const {
    const int64_t dest = row_dest[row];
    if (dest == 0) return;
    float o[NV];
    if (row_token[row] < 0) {
#pragma unroll
      for (int i = 0; i < NV; ++i) o[i] = 0.f;
    } else if (bias != nullptr) {
      load_vec<T, NV>(bias + (size_t)e * N + n0, o);
#pragma unroll
      for (int i = 0; i < NV; ++i) o[i] += v[i];
    } else {
#pragma unroll
      for (int i = 0; i < NV; ++i) o[i] = v[i];
    }
    store_vec<T, NV>(reinterpret_cast<T*>(dest) + n0, o);
  }
};

// One warp per sorted assignment j: copies hidden[token] into the owner's recv_x.
template <typename T>
__global__ void __launch_bounds__(kRowWarps * 32)
ep_dispatch_kernel(const T* __restrict__ hidden, const int32_t* __restrict__ sorted_values,
                   const int32_t* __restrict__ sorted_indices, const int32_t* __restrict__ bins,
                   const int32_t* __restrict__ dest_row, void* const* __restrict__ peer_x, int64_t S, int H, int E,
                   int per, int K) {
  const int64_t j = (int64_t)blockIdx.x * kRowWarps + (threadIdx.x >> 5);
  if (j >= S || j >= bins[E - 1]) return;
  const int lane = threadIdx.x & 31;
  const int e = sorted_values[j];
  const int i = (int)j - (e ? bins[e - 1] : 0);
  const int tok = sorted_indices[j] / K;
  T* dst = reinterpret_cast<T*>(peer_x[e / per]) + (size_t)(dest_row[e] + i) * H;
  const uint4* s = reinterpret_cast<const uint4*>(hidden + (size_t)tok * H);
  uint4* d = reinterpret_cast<uint4*>(dst);
  const int nvec = H * (int)sizeof(T) / 16;
  for (int v = lane; v < nvec; v += 32) d[v] = __ldg(s + v);
}

// One warp per local row: sends y[row] back to the rank the row came from (zeros if dropped).
template <typename T>
__global__ void __launch_bounds__(kRowWarps * 32)
ep_return_kernel(const T* __restrict__ y, EpTables t, void* const* __restrict__ peer_back, int H, int G, int per) {
  const int64_t r = (int64_t)blockIdx.x * kRowWarps + (threadIdx.x >> 5);
  if (r >= t.rt.header[kHdrRowsUsed]) return;
  const int lane = threadIdx.x & 31;
  const int le = t.rt.tile_expert[r / kTileM];
  if (r - t.rt.pad_off[le] >= t.rt.counts[le]) return;          // padding
  int s = 0;
  while (s + 1 < G && t.seg_row[(s + 1) * per + le] <= r) ++s;   // source whose segment holds r
  const int64_t dst_row = (int64_t)t.src_start[s * per + le] + (r - t.seg_row[s * per + le]);
  uint4* d = reinterpret_cast<uint4*>(reinterpret_cast<T*>(peer_back[s]) + (size_t)dst_row * H);
  const int nvec = H * (int)sizeof(T) / 16;
  if (t.rt.row_token[r] < 0) {
    for (int v = lane; v < nvec; v += 32) d[v] = make_uint4(0, 0, 0, 0);
  } else {
    const uint4* src = reinterpret_cast<const uint4*>(y + (size_t)r * H);
    for (int v = lane; v < nvec; v += 32) d[v] = src[v];
  }
}

// One thread per sorted assignment j: its routing weight (fp32) goes to the owner's recv_w at
// the row its token row went to.  routing_cols == E: dense [T, E] weights, else [T, K].
template <typename T>
__global__ void ep_dispatch_weight_kernel(const T* __restrict__ routing_weights, int routing_cols,
                                          const int32_t* __restrict__ sorted_values,
                                          const int32_t* __restrict__ sorted_indices,
                                          const int32_t* __restrict__ bins, const int32_t* __restrict__ dest_row,
                                          void* const* __restrict__ peer_w, int64_t S, int E, int per, int K) {
  const int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= S || j >= bins[E - 1]) return;
  const int e = sorted_values[j];
  const int i = (int)j - (e ? bins[e - 1] : 0);
  const int flat = sorted_indices[j];
  const size_t idx = routing_cols == E ? (size_t)(flat / K) * E + e : (size_t)flat;
  reinterpret_cast<float*>(peer_w[e / per])[dest_row[e] + i] = DT<T>::ld(routing_weights + idx);
}

// row_weight[r] = received routing weight for kept rows, 0 for padding and dropped rows.
__global__ void ep_load_weights_kernel(EpTables t, const float* __restrict__ recv_w, int64_t max_rows) {
  const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= max_rows) return;
  t.rt.row_weight[r] = t.rt.row_token[r] >= 0 ? recv_w[r] : 0.f;
}

// One thread per local row: val[row] (fp32) goes back to the rank the row came from, at the
// position of the assignment in that rank's sorted order.  Padding rows send nothing.
__global__ void ep_return_scalar_kernel(const float* __restrict__ val, EpTables t,
                                        void* const* __restrict__ peer_back_w, int G, int per) {
  const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= t.rt.header[kHdrRowsUsed]) return;
  const int le = t.rt.tile_expert[r / kTileM];
  if (r - t.rt.pad_off[le] >= t.rt.counts[le]) return;
  int s = 0;
  while (s + 1 < G && t.seg_row[(s + 1) * per + le] <= r) ++s;
  const int64_t dst_row = (int64_t)t.src_start[s * per + le] + (r - t.seg_row[s * per + le]);
  reinterpret_cast<float*>(peer_back_w[s])[dst_row] = t.rt.row_token[r] >= 0 ? val[r] : 0.f;
}

}  // namespace yb
