// Expert parallelism over peer memory, without host-side collectives: token rows travel to the
// expert owners and result rows back as plain stores into the other GPUs' buffers (NVLink); every
// offset is derived on the device from the [G, E] matrix of per-rank counts, and the count exchange
// and the phase boundaries are flags in symmetric memory, so that one expert-parallel call is a
// fixed chain of kernels on one stream: no NCCL call, no host round trip, no split sizes.
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
// The backward pass travels the same way: token rows, upstream-gradient rows and one fp32 routing
// weight per row go out with the dispatch kernel; the input-gradient rows return through the last
// data-gradient GEMM's epilogue (EpiPeerRows without a bias) and the routing-weight gradients with
// ep_return_scalar_kernel.
//
// Every rank owns a control block that its peers may write (EpCtrl, layout below).  A call has an
// epoch number (a device counter in the rank's private state, incremented by the first kernel of
// the call).  Flags carry the epoch of the phase that completed:
//
//   ep_publish_kernel     clears my arrival counters, then my per-expert counts ->
//                         counts[epoch & 1][rank][:] of every peer and flag_counts[rank] = epoch there
//   ep_dispatch_kernel    waits until flag_counts[s] >= epoch for every source s (bounded), derives
//                         every offset from the [G, E] counts, writes this rank's tile and row
//                         tables (state[prep] counts the CTAs that are done with them), stores my
//                         rows into the owners' receive buffers -- after each row arrived[le] += 1
//                         on the owner, with release semantics -- and its last CTA sets
//                         flag_dispatch[rank] = epoch on every peer
//   gate_up GEMM          forward: launched with programmatic dependent launch, so it runs NEXT TO
//                         the dispatch kernel; it starts once state[prep] is complete and loads the
//                         rows of local expert le once arrived[le] has reached that expert's row
//                         count (both waits bounded).  Rows travel local-expert-index major, so
//                         expert 0 of every owner completes first: the transfer of the later
//                         experts overlaps the tensor-core work on the earlier ones.
//   ep_wait_kernel        backward (three row streams, no overlap): one warp waits for
//                         flag_dispatch[s] >= epoch from every source (bounded)
//   (further grouped GEMMs; the last one returns result rows to their sources from its epilogue,
//   in 128-byte pieces)
//   ep_signal_kernel      flag_return[rank] = epoch on every peer
//   ep_combine_kernel     waits for flag_return[o] >= epoch from every owner (bounded), then sums
//                         each token's K returned rows
//
// Only stores cross NVLink; every wait polls this GPU's own memory with ld.acquire.sys and gives
// up after `wait_ns`, recording a status word in the workspace header (the data of that call is
// then invalid, the GPU and all buffers stay usable).  A rank reuses a peer's buffer only after
// that peer told it, by the flags of the previous phase, that it is done reading: the receive
// buffers are written in call n+1 only after every owner signalled flag_return for call n, which
// it does after its last kernel that reads them; the back buffers only after the token owner
// signalled flag_dispatch for call n+1, which follows its combine of call n on its stream.
//
// Rows whose destination would fall outside the receive buffer are never stored: the plan checks
// every owner's padded row total against max_rows and, on overflow, marks the call invalid on
// every rank (all ranks see the same counts) so that nothing is stored or computed.
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

// Down-projection epilogue fused with the combine exchange: the bias-added result row goes
// straight into the back buffer of the rank that owns the token (a peer store over NVLink);
// rows dropped by the capacity send zeros, padding rows send nothing.  In the tcgen05 kernel the
// rows leave in 128-byte pieces (kStagedRows), which is what makes the NVLink stores efficient.
template <typename T>
struct EpiPeerRows {
  static constexpr bool kStagedRows = sizeof(T) == 2;
  static constexpr int kOutPerChunk = 32;
  const T* bias;             // [per, N], or nullptr
  const int64_t* row_dest;
  const int32_t* row_token;
  int N;

  __device__ __forceinline__ T* row_ptr(int row) const { return reinterpret_cast<T*>(row_dest[row]); }

  template <int NV>
  __device__ __forceinline__ void values(int e, int row, int n0, const float (&v)[NV], float (&o)[NV]) const {
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
  }

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

enum EpStatus {
  kStatusEpCountsTimeout = 4,
  kStatusEpDispatchTimeout = 5,
  kStatusEpReturnTimeout = 6,
  kStatusEpOverflow = 7,
};

// Layout (int32 words) of the control block peers write into.
struct EpCtrlLayout {
  int G, E;
  __host__ __device__ int counts(int parity, int src) const { return (parity * G + src) * E; }
  __host__ __device__ int flag_counts() const { return 2 * G * E; }
  __host__ __device__ int flag_dispatch() const { return 2 * G * E + 64 * ((G + 63) / 64); }
  __host__ __device__ int flag_return() const { return 2 * G * E + 2 * 64 * ((G + 63) / 64); }
  // arrived[le]: rows of local expert le that have landed in this rank's receive buffer in the
  // current call (every source adds 1 per row, with release semantics, after storing the row)
  __host__ __device__ int arrived() const { return 2 * G * E + 3 * 64 * ((G + 63) / 64); }
  __host__ __device__ int words() const { return arrived() + E; }
};

// Private per-rank state that lives across calls (zeroed once by the owner).
//   prep: CTAs of the dispatch kernel that have finished this rank's tile and row tables
enum EpStateSlot { kEpStateEpoch = 0, kEpStateTicket = 1, kEpStatePrep = 2 };

__device__ __forceinline__ int32_t ld_acquire_sys(const int32_t* p) {
  int32_t v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int32_t* p, int32_t v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint64_t ep_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Polls a flag in this GPU's memory until it reaches `epoch`; false when `limit_ns` ran out.
__device__ __forceinline__ bool ep_wait_flag(const int32_t* flag, int32_t epoch, uint64_t limit_ns) {
  const uint64_t t0 = ep_timer_ns();
  for (;;) {
    if (ld_acquire_sys(flag) - epoch >= 0) return true;
    if (ep_timer_ns() - t0 > limit_ns) return false;
    __nanosleep(64);
  }
}

// One CTA.  Starts a call: bumps the epoch, then tells every rank how many assignments this rank
// has for each expert.
__global__ void __launch_bounds__(256)
ep_publish_kernel(const int32_t* __restrict__ counts, int32_t* __restrict__ state, void* const* __restrict__ peer_ctrl,
                  EpCtrlLayout lay, int rank) {
  __shared__ int32_t s_epoch;
  if (threadIdx.x == 0) {
    s_epoch = state[kEpStateEpoch] + 1;
    state[kEpStateEpoch] = s_epoch;
    state[kEpStateTicket] = 0;
    state[kEpStatePrep] = 0;
  }
  // my arrival counters start the call at zero; no peer adds to them before it has seen the count
  // flag this kernel sets at its end
  for (int i = threadIdx.x; i < lay.E; i += blockDim.x)
    reinterpret_cast<int32_t*>(peer_ctrl[rank])[lay.arrived() + i] = 0;
  __syncthreads();
  const int32_t epoch = s_epoch;
  for (int i = threadIdx.x; i < lay.G * lay.E; i += blockDim.x) {
    const int g = i / lay.E, e = i - g * lay.E;
    reinterpret_cast<int32_t*>(peer_ctrl[g])[lay.counts(epoch & 1, rank) + e] = counts[e];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < lay.G)
    st_release_sys(reinterpret_cast<int32_t*>(peer_ctrl[threadIdx.x]) + lay.flag_counts() + rank, epoch);
}

struct EpDispatchArgs {
  const void* hidden;            // [T, H]
  const void* grad;              // [T, H] or null          (backward: upstream-gradient rows)
  const void* routing_weights;   // [T, routing_cols] or null (backward: one fp32 per row travels)
  int routing_cols;
  const int32_t* sorted_values;  // [S]
  const int32_t* sorted_indices; // [S]
  const int32_t* bins;           // [E+1]
  void* const* peer_x;           // [G] receive buffers for token rows
  void* const* peer_g;           // [G] receive buffers for gradient rows, or null
  void* const* peer_w;           // [G] receive buffers for routing weights, or null
  void* const* peer_back;        // [G] buffers the result rows return to (for row_dest)
  void* const* peer_ctrl;        // [G]
  const int32_t* ctrl;           // this rank's control block
  int32_t* state;
  int64_t max_rows, capacity, row_bytes;
  int S, H, E, G, rank, K;
  int signal_rows;               // add 1 to the owner's arrived[le] after every row (forward: the GEMM waits per expert)
  uint64_t wait_ns;
};

__device__ __forceinline__ void red_release_sys_add(int32_t* p, int32_t v) {
  asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// One warp copies a row of nvec 16-byte pieces, four loads in flight per lane.
__device__ __forceinline__ void ep_copy_row(const uint4* __restrict__ s, uint4* __restrict__ d, int nvec, int lane) {
  int v = lane;
  for (; v + 96 < nvec; v += 128) {
    const uint4 q0 = __ldg(s + v), q1 = __ldg(s + v + 32), q2 = __ldg(s + v + 64), q3 = __ldg(s + v + 96);
    d[v] = q0; d[v + 32] = q1; d[v + 64] = q2; d[v + 96] = q3;
  }
  for (; v < nvec; v += 32) d[v] = __ldg(s + v);
}

// Persistent grid, two CTAs per SM next to a GEMM CTA (64 registers per thread), four without one.
// Shared memory: 6*E + 2 int32.  Order of work in every CTA:
//   1. wait for every source's counts; derive the offsets (all CTAs, in shared memory)
//   2. this rank's tile tables (CTA 0) and its share of the row tables; state[prep] += 1
//   3. its share of this rank's rows -> their owners, local-expert index major: first the rows of
//      every owner's local expert 0, then of every owner's local expert 1, ...; inside one local
//      expert index the owners are visited starting behind this rank, so that at any moment every
//      owner receives from a different source.  An owner's experts therefore become complete in
//      the order in which its grouped GEMM works on them.
//   4. ticket; the last CTA sets flag_dispatch[rank] on every peer
template <typename T>
__global__ void __launch_bounds__(kRowWarps * 32, 4)
ep_dispatch_fused_kernel(const EpDispatchArgs a, EpTables t) {
  extern __shared__ int32_t sm[];
  int32_t* tot = sm;               // [E] rows of expert e over all sources
  int32_t* before = sm + a.E;      // [E] rows of expert e from sources s < rank
  int32_t* poff = sm + 2 * a.E;    // [E] padded row offset of e inside its owner
  int32_t* sstart = sm + 3 * a.E;  // [G*per] start of expert (rank*per+le) in source s's sorted order
  int32_t* segr = sm + 4 * a.E;    // [G*per] first local row of the rows source s sent for local expert le
  int32_t* xstart = sm + 5 * a.E;  // [E+1] start of every expert's rows in this rank's transfer order
  __shared__ int s_bad, s_last;
  pdl_trigger();                   // a dependent GEMM may become resident; it gates itself on state[prep] and arrived[]
#ifdef YB_PROF
  if (threadIdx.x == 0) atomicMin(&g_prof[10], (unsigned long long)ep_timer_ns());
#endif
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int E = a.E, G = a.G, per = E / G, rank = a.rank;
  const EpCtrlLayout lay{G, E};
  const int32_t epoch = a.state[kEpStateEpoch];
  if (tid == 0) s_bad = 0;
  __syncthreads();
  // ---- every source's counts for this call must have arrived ---------------------------------
  if (tid < G && !ep_wait_flag(a.ctrl + lay.flag_counts() + tid, epoch, a.wait_ns)) {
    s_bad = kStatusEpCountsTimeout;
  }
  __syncthreads();
  const int32_t* counts_all = a.ctrl + lay.counts(epoch & 1, 0);   // [G][E]
  if (s_bad == 0) {
    for (int e = tid; e < E; e += nthr) {
      int c_all = 0, c_before = 0;
      for (int s = 0; s < G; ++s) {
        const int c = max(__ldcg(counts_all + s * E + e), 0);
        if (s < rank) c_before += c;
        c_all += c;
      }
      tot[e] = c_all;
      before[e] = c_before;
    }
    __syncthreads();
    if (tid < G) {                  // padded offsets inside owner `tid`, checked against the buffer
      int64_t rows = 0;
      for (int le = 0; le < per; ++le) {
        const int e = tid * per + le;
        poff[e] = (int)rows;
        rows += (tot[e] + kTileM - 1) / kTileM * kTileM;
        if (rows > a.max_rows) { s_bad = kStatusEpOverflow; break; }
      }
    }
    // way back: where source s keeps the rows of my local expert le in its sorted order
    for (int s = tid; s < G; s += nthr) {
      int run = 0;
      for (int e = 0; e < (rank + 1) * per; ++e) {
        if (e >= rank * per) sstart[s * per + (e - rank * per)] = run;
        run += max(__ldcg(counts_all + s * E + e), 0);
      }
    }
    // my transfer order: position x = le * G + ((owner - rank - 1) mod G); exclusive scan of the
    // row counts in that order by warp 0 (each lane a run of consecutive positions).  The counts
    // sit in segr for the moment (it gets its own contents below).
    for (int x = tid; x < E; x += nthr) {
      const int le = x / G, owner = (rank + 1 + (x - le * G)) % G;
      const int e = owner * per + le;
      segr[x] = a.bins[e] - (e ? a.bins[e - 1] : 0);
    }
    __syncthreads();
    if (tid < 32) {
      const int chunk = (E + 31) / 32, x0 = min(tid * chunk, E), x1 = min(x0 + chunk, E);
      int sum = 0;
      for (int x = x0; x < x1; ++x) sum += segr[x];
      int incl = sum;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (tid >= o) incl += v;
      }
      int run = incl - sum;
      for (int x = x0; x < x1; ++x) {
        xstart[x] = run;
        run += segr[x];
      }
      if (tid == 31) xstart[E] = incl;
    }
    __syncthreads();
    // first local row of the rows source s sent for my local expert le
    for (int le = tid; le < per; le += nthr) {
      int row = poff[rank * per + le];
      for (int s = 0; s < G; ++s) {
        segr[s * per + le] = row;
        row += max(__ldcg(counts_all + s * E + rank * per + le), 0);
      }
    }
    __syncthreads();
  }
  const int bad = s_bad;
  // ---- CTA 0: this rank's own tile tables and the (source, expert) segments for the way back ----
  if (blockIdx.x == 0) {
    if (bad != 0) {
      if (tid == 0) {
        atomicMax(t.rt.header + kHdrStatus, bad);
        t.rt.header[kHdrRowTiles] = 0;
        t.rt.header[kHdrRowsUsed] = 0;
        t.rt.header[kHdrPairs] = 0;
        t.rt.header[kHdrDropped] = 0;
      }
      for (int le = tid; le <= per; le += nthr) {
        t.rt.pad_off[le] = 0;
        t.rt.pair_off[le] = 0;
        t.rt.bins[le] = 0;
        if (le < per) t.rt.counts[le] = 0;
      }
    } else {
      for (int i = tid; i < G * per; i += nthr) {
        t.src_start[i] = sstart[i];
        t.seg_row[i] = segr[i];
      }
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
          for (int k = 0; k < tiles; ++k) t.rt.tile_expert[rows / kTileM + k] = le;
          for (int k = 0; k < (tiles + 1) / 2; ++k) t.rt.pair_expert[pairs + k] = le;
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
    }
  }
  // ---- this CTA's share of the row tables: validity of every local row and where its result goes --
  // row_token[r] = r for kept rows, -1 for padding and for rows beyond the capacity; weight 1;
  // row_dest[r] = the row's slot in the back buffer of the rank it came from, 0 for padding.
  {
    const int me = rank * per;
    const int used = bad ? 0 : poff[me + per - 1] + (tot[me + per - 1] + kTileM - 1) / kTileM * kTileM;
    const int64_t chunk = (a.max_rows + gridDim.x - 1) / gridDim.x;
    const int64_t r_end = min((int64_t)(blockIdx.x + 1) * chunk, a.max_rows);
    for (int64_t r = (int64_t)blockIdx.x * chunk + tid; r < r_end; r += nthr) {
      int32_t tok = -1;
      int64_t dest = 0;
      if (r < used) {
        int lo = 0, hi = per - 1;                      // last local expert whose first row is <= r
        while (lo < hi) {
          const int mid = (lo + hi + 1) >> 1;
          if (poff[me + mid] <= r) lo = mid; else hi = mid - 1;
        }
        const int le = lo;
        const int64_t i = r - poff[me + le];
        const int64_t c = tot[me + le];
        if (i < (c < a.capacity ? c : a.capacity)) tok = (int32_t)r;
        if (i < c && a.peer_back != nullptr) {
          int sidx = 0;
          while (sidx + 1 < G && segr[(sidx + 1) * per + le] <= r) ++sidx;
          const int64_t dst_row = (int64_t)sstart[sidx * per + le] + (r - segr[sidx * per + le]);
          dest = reinterpret_cast<int64_t>(a.peer_back[sidx]) + dst_row * a.row_bytes;
        }
      }
      t.rt.row_token[r] = tok;
      t.rt.row_weight[r] = 1.0f;
      t.row_dest[r] = dest;
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) atomicAdd(a.state + kEpStatePrep, 1);
  }
  // ---- my rows -> their owners -------------------------------------------------------------------
  if (bad == 0) {
    const int warp = tid >> 5, lane = tid & 31;
    const int nvec = a.H * (int)sizeof(T) / 16;
    // A warp takes four consecutive transfer positions per trip: their stores are in flight
    // together, and rows of the same expert share one release.
    constexpr int kRowsPerTrip = 4;
    // Phase le = the rows of every owner's local expert le.  The phases are walked in order by all
    // warps, so the rows of phase le are (nearly) all on their way before those of phase le + 1
    // start: experts complete at their owners in the order the owners' GEMMs want them.  The warp
    // that takes the first rows of a phase rotates, so that small phases do not all land on the
    // same few SMs.
    const int nw = gridDim.x * kRowWarps, gw = blockIdx.x * kRowWarps + warp;
    for (int ph = 0; ph < per; ++ph) {
    const int p0 = xstart[ph * G], p1 = xstart[(ph + 1) * G];
    const int slot = (gw + ph * 251) % nw;
    for (int base = p0 + slot * kRowsPerTrip; base < p1; base += nw * kRowsPerTrip) {
      int sig_owner = -1, sig_le = 0, sig_n = 0;       // rows stored but not yet announced
      for (int jj = base; jj < min(base + kRowsPerTrip, p1); ++jj) {
        int lo = 0, hi = E - 1;                        // transfer position x with xstart[x] <= jj < xstart[x+1]
        while (lo < hi) {
          const int mid = (lo + hi + 1) >> 1;
          if (xstart[mid] <= jj) lo = mid; else hi = mid - 1;
        }
        const int le = lo / G, owner = (rank + 1 + (lo - le * G)) % G;
        const int e = owner * per + le;
        const int i = jj - xstart[lo];
        const int j = (e ? a.bins[e - 1] : 0) + i;     // position in my sorted order
        const int flat = a.sorted_indices[j];
        const int tok = flat / a.K;
        const int64_t drow = (int64_t)poff[e] + before[e] + i;
        if (drow >= a.max_rows) continue;        // cannot happen once the totals passed the check
        if (a.signal_rows && sig_n > 0 && (owner != sig_owner || le != sig_le)) {
          __syncwarp();
          if (lane == 0)
            red_release_sys_add(reinterpret_cast<int32_t*>(a.peer_ctrl[sig_owner]) + lay.arrived() + sig_le, sig_n);
          sig_n = 0;
        }
        ep_copy_row(reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(a.hidden) + (size_t)tok * a.H),
                    reinterpret_cast<uint4*>(reinterpret_cast<T*>(a.peer_x[owner]) + (size_t)drow * a.H), nvec, lane);
        if (a.grad != nullptr)
          ep_copy_row(reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(a.grad) + (size_t)tok * a.H),
                      reinterpret_cast<uint4*>(reinterpret_cast<T*>(a.peer_g[owner]) + (size_t)drow * a.H), nvec, lane);
        if (a.routing_weights != nullptr && lane == 0) {
          const size_t idx = a.routing_cols == E ? (size_t)tok * E + e : (size_t)flat;
          reinterpret_cast<float*>(a.peer_w[owner])[drow] =
              DT<T>::ld(reinterpret_cast<const T*>(a.routing_weights) + idx);
        }
        sig_owner = owner; sig_le = le; ++sig_n;
      }
      if (a.signal_rows && sig_n > 0) {
        // the rows are complete once every lane's stores are ordered before lane 0's release
        __syncwarp();
        if (lane == 0)
          red_release_sys_add(reinterpret_cast<int32_t*>(a.peer_ctrl[sig_owner]) + lay.arrived() + sig_le, sig_n);
      }
    }
    }
  }
#ifdef YB_PROF
  if (threadIdx.x == 0) atomicMax(&g_prof[11], (unsigned long long)ep_timer_ns());
#endif
  // ---- the last CTA tells every owner that this rank's rows are in place -----------------------
  __threadfence_system();
  __syncthreads();
  if (tid == 0) s_last = (atomicAdd(a.state + kEpStateTicket, 1) == (int)gridDim.x - 1);
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    if (tid < G)
      st_release_sys(reinterpret_cast<int32_t*>(a.peer_ctrl[tid]) + lay.flag_dispatch() + rank, epoch);
    if (tid == 0) a.state[kEpStateTicket] = 0;
  }
}

// One warp: lane s waits for `flags[s]` to reach the epoch of this call.
__global__ void ep_wait_kernel(const int32_t* __restrict__ flags, int G, const int32_t* __restrict__ state,
                               int32_t* __restrict__ header, int status_code, uint64_t wait_ns) {
  const int32_t epoch = state[kEpStateEpoch];
  for (int s = threadIdx.x; s < G; s += blockDim.x)
    if (!ep_wait_flag(flags + s, epoch, wait_ns)) atomicMax(header + kHdrStatus, status_code);
}

// One warp: everything this rank stored into its peers during the preceding kernels of the stream
// is made visible, then flag[rank] = epoch on every peer.
__global__ void ep_signal_kernel(void* const* __restrict__ peer_ctrl, int flag_word, int G, int rank,
                                 const int32_t* __restrict__ state) {
  const int32_t epoch = state[kEpStateEpoch];
  __threadfence_system();
  for (int g = threadIdx.x; g < G; g += blockDim.x)
    st_release_sys(reinterpret_cast<int32_t*>(peer_ctrl[g]) + flag_word + rank, epoch);
}

// out[t, :] = sum_k w[t, k] * back[flat_pos[t*K + k], :] once every owner's rows have come back.
// `back` was written by other GPUs while this kernel may already have been running: it is read
// with L1 bypassed.  UNIT: weights are 1 (the backward pass returns already-weighted rows).
template <typename T, bool UNIT>
__global__ void __launch_bounds__(kRowWarps * 32)
ep_combine_kernel(const T* __restrict__ back, const int32_t* __restrict__ flat_pos,
                  const int64_t* __restrict__ router_indices, const T* __restrict__ routing_weights,
                  int routing_cols, T* __restrict__ out, int64_t Tn, int H, int E, int K,
                  const int32_t* __restrict__ flags, int G, const int32_t* __restrict__ state,
                  int32_t* __restrict__ header, uint64_t wait_ns) {
  const int32_t epoch = state[kEpStateEpoch];
  if (threadIdx.x < G && !ep_wait_flag(flags + threadIdx.x, epoch, wait_ns))
    atomicMax(header + kHdrStatus, (int)kStatusEpReturnTimeout);
  __syncthreads();
  const int lane = threadIdx.x & 31;
  constexpr int VE = 16 / (int)sizeof(T);
  const int nvec = H / VE;
  for (int64_t t = (int64_t)blockIdx.x * kRowWarps + (threadIdx.x >> 5); t < Tn; t += (int64_t)gridDim.x * kRowWarps) {
    for (int i = lane; i < nvec; i += 32) {
      float acc[VE];
#pragma unroll
      for (int j = 0; j < VE; ++j) acc[j] = 0.f;
      for (int k = 0; k < K; ++k) {
        const int32_t r = flat_pos[t * K + k];
        if (r < 0) continue;
        float w = 1.0f;
        if constexpr (!UNIT) {
          const int col = (routing_cols == E) ? (int)router_indices[t * K + k] : k;
          w = DT<T>::ld(routing_weights + (size_t)t * routing_cols + col);
        }
        const uint4 q = __ldcg(reinterpret_cast<const uint4*>(back + (size_t)r * H) + i);
        float v[VE];
        if constexpr (sizeof(T) == 2) {
          const uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            v[2 * j] = __uint_as_float(u[j] << 16);
            v[2 * j + 1] = __uint_as_float(u[j] & 0xffff0000u);
          }
        } else {
          v[0] = __uint_as_float(q.x); v[1] = __uint_as_float(q.y);
          v[2] = __uint_as_float(q.z); v[3] = __uint_as_float(q.w);
        }
#pragma unroll
        for (int j = 0; j < VE; ++j) acc[j] = fmaf(w, v[j], acc[j]);
      }
      store_vec<T, VE>(out + (size_t)t * H + (size_t)i * VE, acc);
    }
  }
}

// d_routing[t, expert] (dense) or d_routing[t, slot] = returned routing-weight gradient of the
// assignment, 0 for assignments that were not routed.  `d_routing` must be zero-filled when dense.
template <typename T>
__global__ void ep_routing_grad_kernel(const float* __restrict__ back_w, const int32_t* __restrict__ flat_pos,
                                       const int64_t* __restrict__ router_indices, T* __restrict__ d_routing,
                                       int64_t S, int routing_cols, int E, int K) {
  const int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= S) return;
  const int32_t j = flat_pos[p];
  const float v = j >= 0 ? __ldcg(back_w + j) : 0.f;
  if (routing_cols == E) {
    const int64_t e = router_indices[p];
    if (e >= 0 && e < E && j >= 0) DT<T>::st(d_routing + (p / K) * E + e, v);
  } else {
    DT<T>::st(d_routing + p, v);
  }
}

}  // namespace yb
