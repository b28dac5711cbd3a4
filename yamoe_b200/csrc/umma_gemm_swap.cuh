// Row-tiled tcgen05 GEMMs with the operands swapped, on CTA pairs (cta_group::2): the weight slab
// feeds the M = 256 side of tcgen05.mma (128 output columns per CTA) and the token rows feed the
// N side.
//
// Why: the instruction costs N/2 clocks whatever M is, and N may be any multiple of 32 up to 256
// (16 with one CTA).  With the rows on the N side an expert with 530 rows is computed as 576 rows
// (three tiles of 192); with the rows on the M side (umma_gemm.cuh) the same expert costs
// 5 x 128 = 640 rows, and the pair kernel of umma_gemm_2cta.cuh even 768.  Per SM and 64-deep k-block a full tile moves
// 16 KB of weights and at most 16 KB of rows (half of the tile's rows; the pair shares them),
// against 48 KB in the one-CTA kernel.
//
// The padded, expert-sorted row layout is unchanged.  A work item is (expert, 256-column tile,
// row tile); an expert's rows are split evenly over as many row tiles as it has 256-row pairs
// (pair_off / pair_expert tables), each rounded up to 32 rows.
//
//   kFwd    C[r][n] = sum_k X[r][k] W[e][k][n]   A = W[e] MN-major (two 64-column boxes), B = X K-major
//   kDgrad  C[r][n] = sum_k X[r][k] W[e][n][k]   A = W[e] K-major (one 128-row box),      B = X K-major
//
// The accumulator is transposed in TMEM (lane = output column, TMEM column = row).  Each epilogue
// warp turns its 32 x 32 fragment around through a padded shared-memory tile, so that a thread
// again holds 32 consecutive columns of one row and the epilogue functors are those of the
// unswapped kernels.  The last row tile of an expert hands the padding rows behind it to the
// functor as zeros (every functor zero-fills or skips padding rows).
//
// Roles, signals across the pair, bounded waits and the abort path are those of
// umma_gemm_2cta.cuh; every CTA loads its own operands.
#pragma once
#include "umma_gemm_2cta.cuh"

namespace yb {

constexpr int kSwapBM = 128;                 // output columns per CTA (M side, 256 per pair)
constexpr int kSwapRows = 256;               // rows per row tile (N side, upper bound)
constexpr int kSwapWBytes = kSwapBM * 128;   // 16 KB
constexpr int kSwapXBytes = (kSwapRows / 2) * 128;   // this CTA's half of the rows, 16 KB
constexpr int kSwapStageBytes = kSwapWBytes + kSwapXBytes;
constexpr int kSwapStages = 6;
constexpr int kSwapSmemTotal = kSwapStages * kSwapStageBytes + 1024;

struct SwapParams {
  int N, K;
  const int32_t* pad_off;
  const int32_t* pair_off;
  const int32_t* pair_expert;
  const int32_t* counts;      // rows present per expert (clipped to the padded extent), or null
  int32_t* header;
};

struct SwapTile {
  int e;
  int row0;        // first row of the tile (padded layout)
  int nrows;      // rows the instruction computes (a multiple of 32)
  int n0;          // first output column of the pair
  int zero_end;    // last tile of the expert: end of the padded extent, else 0
};

template <int MODE, class Epi>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kU2Threads, 1)
umma_gemm_swap_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                      const SwapParams p, const Epi epi) {
  static_assert(MODE == kFwd || MODE == kDgrad, "row-tiled GEMMs only");
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kSwapStages];     // used in the leader CTA
  __shared__ __align__(8) uint64_t bar_empty[kSwapStages];    // per CTA
  __shared__ __align__(8) uint64_t bar_tmem_full[2];          // per CTA
  __shared__ __align__(8) uint64_t bar_tmem_empty[2];         // used in the leader CTA
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ float tbuf[4][32][33];          // one transposition tile per epilogue warp

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kSwapStages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 2);        // one arrive.expect_tx from each CTA's producer
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&bar_tmem_full[a]), 1);
      mbar_init(smem_u32(&bar_tmem_empty[a]), 256);  // epilogue threads of both CTAs
    }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_base_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // the peer's barriers exist before any remote signal is sent
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  // ---- tile walk (identical in every role): expert, then column tile, row tile fastest ----------
  const int NT = (p.N + 2 * kSwapBM - 1) / (2 * kSwapBM);
  const int total = p.header[kHdrPairs] * NT;
  const int kblocks = p.K / kUmmaBK;
  const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
  auto decode = [&](int id) {
    SwapTile t;
    const int u = id / NT;
    t.e = p.pair_expert[u];
    const int first = p.pair_off[t.e];
    const int cnt = p.pair_off[t.e + 1] - first;
    const int local = id - first * NT;
    const int nt = local / cnt;
    const int rt = local - nt * cnt;
    const int begin = p.pad_off[t.e];
    const int extent = p.pad_off[t.e + 1] - begin;
    int have = extent;
    if (p.counts != nullptr) have = max(min(p.counts[t.e], extent), 1);
    // cta_group::2 wants N in multiples of 32.  per_tile <= 256 because have <= 256 * cnt, and the
    // last tile is never empty because have > 256 * (cnt - 1).
    const int per_tile = (((have + cnt - 1) / cnt) + 31) & ~31;
    const int done = rt * per_tile;
    const int rows = max(min(per_tile, have - done), 0);
    t.row0 = begin + done;
    t.nrows = max((rows + 31) & ~31, 32);
    t.n0 = nt * 2 * kSwapBM;
    t.zero_end = (rt == cnt - 1) ? begin + extent : 0;
    return t;
  };

  if (warp == 0) {
    // =========================== TMA producer (both CTAs) ====================================
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int id = cluster_id; id < total && ok; id += n_clusters) {
        const SwapTile t = decode(id);
        const int half = t.nrows >> 1;
        const int my_row0 = t.row0 + (int)rank * half;
        const int my_n0 = t.n0 + (int)rank * kSwapBM;
        const int nbox = (half + 63) >> 6;
        const uint32_t bytes = (uint32_t)(kSwapWBytes + nbox * 8192);
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, &abort_flag)) {
            abort_flag = 1;
            atomicMax(p.header + kHdrStatus, (int)kStatusProducerTimeout);
            ok = false;
            break;
          }
          const uint32_t full = mapa_u32(smem_u32(&bar_full[stage]), 0);
          const uint32_t sa = smem_base + stage * kSwapStageBytes;
          const uint32_t sb = sa + kSwapWBytes;
          mbar_expect_tx_cluster(full, bytes);
          if constexpr (MODE == kFwd) {
            tma2_load_3d(sa, &tmW, my_n0, kb * kUmmaBK, t.e, full);
            tma2_load_3d(sa + 8192, &tmW, my_n0 + 64, kb * kUmmaBK, t.e, full);
          } else {
            tma2_load_3d(sa, &tmW, kb * kUmmaBK, my_n0, t.e, full);
          }
          for (int i = 0; i < nbox; ++i) tma2_load_2d(sb + i * 8192, &tmX, kb * kUmmaBK, my_row0 + i * 64, full);
          if (++stage == kSwapStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // =========================== MMA issuer (leader CTA only) ================================
    if (leader && lane == 0) {
      constexpr bool kAMn = (MODE == kFwd);
      constexpr uint32_t idesc_base = (1u << 4) | (1u << 7) | (1u << 10) | ((kAMn ? 1u : 0u) << 15) |
                                      ((uint32_t)((2 * kSwapBM) >> 4) << 24);
      constexpr uint32_t a_kstep = kAMn ? (16 * 128) >> 4 : 32 >> 4;
      constexpr uint32_t b_kstep = 32 >> 4;
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int id = cluster_id; id < total && ok; id += n_clusters) {
        const SwapTile t = decode(id);
        const uint32_t idesc = idesc_base | ((uint32_t)(t.nrows >> 3) << 17);
        if (!mbar_wait(smem_u32(&bar_tmem_empty[acc]), acc_phase ^ 1u, &abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kUmmaAccStride;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(smem_u32(&bar_full[stage]), phase, &abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_base + stage * kSwapStageBytes;
          const uint32_t sb = sa + kSwapWBytes;
          const uint64_t adesc = kAMn ? make_smem_desc(sa, 8192, 1024) : make_smem_desc(sa, 16, 1024);
          const uint64_t bdesc = make_smem_desc(sb, 16, 1024);
#pragma unroll
          for (int k = 0; k < kUmmaBK / 16; ++k)
            tc2_mma_bf16(d_tmem, adesc + (uint64_t)(k * a_kstep), bdesc + (uint64_t)(k * b_kstep), idesc,
                         (uint32_t)((kb | k) != 0));
          tc2_commit(smem_u32(&bar_empty[stage]));                 // free the stage in both CTAs
          tc2_commit(mapa_u32(smem_u32(&bar_empty[stage]), 1));
          if (++stage == kSwapStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc2_commit(smem_u32(&bar_tmem_full[acc]));
        tc2_commit(mapa_u32(smem_u32(&bar_tmem_full[acc]), 1));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
      if (!ok) {
        abort_flag = 1;
        atomicMax(p.header + kHdrStatus, (int)kStatusMmaTimeout);
      }
    }
    __syncwarp();
  } else {
    // =========================== epilogue (warps 2..5 of both CTAs) ==========================
    const int q = warp & 3;                    // TMEM lane quarter = 32 output columns
    float (*tb)[33] = tbuf[q];
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int id = cluster_id; id < total; id += n_clusters) {
      const SwapTile t = decode(id);
      const int ncol = t.n0 + (int)rank * kSwapBM + q * 32;   // first output column of this warp
      const bool live = ncol < p.N;
      if (!mbar_wait(smem_u32(&bar_tmem_full[acc]), acc_phase, &abort_flag)) {
        abort_flag = 1;
        atomicMax(p.header + kHdrStatus, (int)kStatusEpilogueTimeout);
        break;
      }
      tc_fence_after();
      const uint32_t t_lane = tmem_base + acc * kUmmaAccStride + ((uint32_t)(q * 32) << 16);
      const int nchunks = (t.nrows + 31) >> 5;  // chunks of 32 rows that hold computed values
      if (live) {
        uint32_t ra[32], rb[32];
        tc_ld_32x32_issue(t_lane, ra);
#pragma unroll 1
        for (int c = 0; c < nchunks; c += 2) {
          tc_ld_wait(ra);
          if (c + 1 < nchunks) tc_ld_32x32_issue(t_lane + (c + 1) * 32, rb);
          {
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) tb[lane][i] = __uint_as_float(ra[i]);
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = tb[j][lane];
            __syncwarp();
            if (c * 32 + lane < t.nrows) epi.template apply<32>(t.e, t.row0 + c * 32 + lane, ncol, v);
          }
          if (c + 1 < nchunks) {
            tc_ld_wait(rb);
            if (c + 2 < nchunks) tc_ld_32x32_issue(t_lane + (c + 2) * 32, ra);
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) tb[lane][i] = __uint_as_float(rb[i]);
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = tb[j][lane];
            __syncwarp();
            if ((c + 1) * 32 + lane < t.nrows) epi.template apply<32>(t.e, t.row0 + (c + 1) * 32 + lane, ncol, v);
          }
        }
      }
      tc_fence_before();
      mbar_arrive_cluster(mapa_u32(smem_u32(&bar_tmem_empty[acc]), 0));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
      if (live && t.zero_end != 0) {
        // padding rows behind the expert's last computed row
        float z[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) z[i] = 0.f;
        for (int r = t.row0 + t.nrows + lane; r < t.zero_end; r += 32) epi.template apply<32>(t.e, r, ncol, z);
      }
    }
  }

  // ---- teardown ---------------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (abort_flag != 0) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  cluster_sync_all();          // neither CTA releases shared memory or TMEM the pair may still use
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// 0 = rows on the M side (umma_gemm.cuh), 1 = swapped operands for the forward-shaped GEMMs,
// 2 = also for the data-gradient GEMMs.  YAMOE_B200_SWAP overrides.  Off by default: measured on
// B200 (T=4096, H=2880, E=32, K=4) the gate_up GEMM takes 550 us swapped against 460 us; the stage
// hand-off across the CTA pair costs about 0.35 us per k-block, more than the padding it saves.
inline int umma_swap_level() {
  static int v = []() {
    const char* env = std::getenv("YAMOE_B200_SWAP");
    return env ? std::atoi(env) : 0;
  }();
  return v;
}

template <int MODE, class Epi>
inline int launch_umma_gemm_swap(const GemmArgs& g, const Epi& epi, int64_t max_rows, int64_t max_tiles,
                                 cudaStream_t stream) {
  if (!umma_available()) return YAMOE_ERR_UNSUPPORTED;
  CUtensorMap tmW, tmX;
  bool ok = true;
  const uint64_t dx[2] = {(uint64_t)g.K, (uint64_t)max_rows}, sx[1] = {(uint64_t)g.lda * 2};
  const uint32_t bx[2] = {64, 64};
  ok = ok && make_map(&tmX, g.A, 2, dx, sx, bx);
  const uint64_t sw[2] = {(uint64_t)g.ldb * 2, (uint64_t)g.b_expert_stride * 2};
  if (MODE == kFwd) {
    const uint64_t dw[3] = {(uint64_t)g.N, (uint64_t)g.K, (uint64_t)g.E};
    const uint32_t bw[3] = {64, 64, 1};
    ok = ok && make_map(&tmW, g.B, 3, dw, sw, bw);
  } else {
    const uint64_t dw[3] = {(uint64_t)g.K, (uint64_t)g.N, (uint64_t)g.E};
    const uint32_t bw[3] = {64, (uint32_t)kSwapBM, 1};
    ok = ok && make_map(&tmW, g.B, 3, dw, sw, bw);
  }
  if (!ok) return YAMOE_ERR_CUDA;
  auto kern = umma_gemm_swap_kernel<MODE, Epi>;
  static bool attr_done = false;   // per template instantiation
  if (!attr_done) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSwapSmemTotal) != cudaSuccess)
      return YAMOE_ERR_CUDA;
    attr_done = true;
  }
  SwapParams p{g.N, g.K, g.pad_off, g.pair_off, g.pair_expert, g.counts, const_cast<int32_t*>(g.header)};
  const int NT = (int)ceil_div(g.N, 2 * kSwapBM);
  const int grid = (int)std::min<int64_t>(2 * max_tiles * NT, umma_sm_count()) & ~1;
  if (grid <= 0) return YAMOE_OK;
  kern<<<grid, kU2Threads, kSwapSmemTotal, stream>>>(tmW, tmX, p, epi);
  return cudaGetLastError() == cudaSuccess ? YAMOE_OK : YAMOE_ERR_CUDA;
}

// Row-tiled GEMMs: swapped-operand pair kernel, pair kernel or one-CTA kernel.
template <int MODE, class Epi>
inline int launch_umma(const GemmArgs& g, const Epi& epi, int64_t max_rows, int64_t max_tiles, cudaStream_t stream) {
  if constexpr (MODE != kWgrad) {
    const bool pairs = g.pair_expert != nullptr && g.pair_off != nullptr && g.gather_rows == nullptr;
    if (pairs && umma_swap_level() >= (MODE == kFwd ? 1 : 2))
      return launch_umma_gemm_swap<MODE>(g, epi, max_rows, max_tiles, stream);
    if (pairs && umma_2cta_enabled()) return launch_umma_gemm_2cta<MODE>(g, epi, max_rows, max_tiles, stream);
  }
  return launch_umma_gemm<MODE>(g, epi, max_rows, max_tiles, stream);
}

}  // namespace yb
