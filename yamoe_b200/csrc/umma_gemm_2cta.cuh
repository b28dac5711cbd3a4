// Two-CTA (cta_group::2) variant of the tcgen05 grouped GEMM for the row-tiled arrangements
// (forward and data gradients).
//
// A cluster of two CTAs computes a 256 x 256 tile: each CTA stages its own 128 rows of A and
// HALF of the B tile (128 columns); one tcgen05.mma.cta_group::2 issued by the leader CTA
// multiplies the pair's 256 rows by all 256 columns, each SM accumulating its own 128 rows in its
// own TMEM.  Per SM and 64-deep k-block that is 32 KB of TMA traffic instead of the 48 KB of the
// one-CTA kernel.  No TMA multicast is used anywhere: each CTA loads its own operands and only
// the completion signals cross the pair.
//
// Signals:  both producers post their transaction bytes on the LEADER's full barrier
// (cp.async.bulk.tensor ... .cta_group::2 with the leader's barrier address); the leader's MMA
// thread frees a stage / publishes an accumulator with ONE tcgen05.commit to its own barrier, and
// the leader thread that waits on that barrier anyway (its producer lane for a stage, a lane of
// its first epilogue warp for an accumulator) passes the news on with a plain remote
// mbarrier.arrive.  (A second commit aimed at the peer's barrier measured about 45 clocks of
// tensor-pipe time per k-block.)  The 2 x 128 epilogue threads of the pair arrive on the leader's
// accumulator-empty barrier.  Work items are (expert, column tile, pair of row
// tiles); an expert with an odd number of row tiles ends with a pair whose second half is
// computed on stale operands and discarded.  Every wait is bounded as in umma_gemm.cuh.
#pragma once
#include "umma_gemm.cuh"

namespace yb {

constexpr int kU2Threads = 192;
constexpr int kU2BN = 256;                 // columns of the pair's tile
constexpr int kU2ABytes = 128 * 128;       // 128 rows x 64 bf16
constexpr int kU2BBytes = 128 * 128;       // this CTA's 128 columns x 64 bf16
constexpr int kU2StageBytes = kU2ABytes + kU2BBytes;
constexpr int kU2Stages = 6;
constexpr int kU2Smem = kU2Stages * kU2StageBytes + 1024;

__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t bar_cluster_addr, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(bar_cluster_addr), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void tma2_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma2_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2,
                                             uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tc2_commit(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
               : "memory");
}
__device__ __forceinline__ void tc2_mma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8, %9, %10, %11, %12}, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u),
        "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}

struct Umma2Params {
  int N, K, E;
  const int32_t* pair_expert;
  const int32_t* pair_off;
  const int32_t* pad_off;
  int32_t* header;
};

template <int MODE, class Epi>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kU2Threads, 1)
umma_gemm_2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const Umma2Params p, const Epi epi) {
  static_assert(MODE == kFwd || MODE == kDgrad, "row-tiled arrangements only");
  constexpr int BN = kU2BN;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kU2Stages];       // used in the leader CTA
  __shared__ __align__(8) uint64_t bar_empty[kU2Stages];      // per CTA
  __shared__ __align__(8) uint64_t bar_tmem_full[2];          // per CTA
  __shared__ __align__(8) uint64_t bar_tmem_empty[2];         // used in the leader CTA
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int32_t s_pad[kUmmaMaxExperts + 1];    // copy of pad_off[0..E]
  __shared__ int32_t s_pair[kUmmaMaxExperts + 1];   // copy of pair_off[0..E]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kU2Stages; ++s) {
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
  // Tile look-up off the critical path, as in the one-CTA kernel: offset tables in shared memory,
  // the expert of a work item fetched one item ahead.
  const bool tab_in_smem = p.E <= kUmmaMaxExperts;
  if (tab_in_smem) {
    for (int i = threadIdx.x; i <= p.E; i += kU2Threads) {
      s_pad[i] = p.pad_off[i];
      s_pair[i] = p.pair_off[i];
    }
    __syncthreads();
  }
  const int32_t* pad = tab_in_smem ? s_pad : p.pad_off;
  const int32_t* pair = tab_in_smem ? s_pair : p.pair_off;

  const int NT = (p.N + BN - 1) / BN;
  const int total = p.header[kHdrPairs] * NT;
  const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
  auto expert_of = [&](int id) -> int { return id < total ? __ldg(p.pair_expert + id / NT) : 0; };
  auto decode = [&](int id, int e_hint, int& e, int& row0, bool& has1, int& n0) {
    e = e_hint;
    const int first = pair[e];
    const int cnt = pair[e + 1] - first;
    const int local = id - first * NT;
    const int nt = local / cnt;
    const int pl = local - nt * cnt;
    const int p0 = pad[e];
    const int tiles = (pad[e + 1] - p0) / kTileM;
    row0 = p0 + pl * 256;
    has1 = 2 * pl + 1 < tiles;
    n0 = nt * BN;
  };
  const int kblocks = p.K / kUmmaBK;

  if (warp == 0) {
    // =========================== TMA producer (both CTAs) ====================================
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      long long prof_empty = 0;
      (void)prof_empty;
      int fills = 0;                       // k-blocks issued so far (saturating use: compared with the ring size)
      int e_next = expert_of(cluster_id);
      for (int id = cluster_id; id < total && ok; id += n_clusters) {
        int e, row0, n0;
        bool has1;
        decode(id, e_next, e, row0, has1, n0);
        e_next = expert_of(id + n_clusters);
        const bool load_a = leader || has1;
        // The last column tile may be narrower (a multiple of 64 columns): the pair then multiplies by
        // ncols columns and each CTA stages half of them.  MN-major B (forward) comes in 64-column
        // boxes, so a half of 32 columns still loads one box and uses its first 32 columns; the
        // K-major B of the data gradients is one box of 128 rows whatever the half is.
        const int ncols = min(BN, p.N - n0);
        const int half = ncols >> 1;
        const int bboxes = MODE == kFwd ? (half + 63) >> 6 : 2;
        const uint32_t bytes = (load_a ? kU2ABytes : 0) + bboxes * 8192;
        const int my_row0 = row0 + (int)rank * 128;
        const int my_n0 = n0 + (int)rank * half;
        for (int kb = 0; kb < kblocks; ++kb) {
          YB_PROF_T0
          if (!mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, &abort_flag)) {
            abort_flag = 1;
            atomicMax(p.header + kHdrStatus, (int)kStatusProducerTimeout);
            ok = false;
            break;
          }
          YB_PROF_ADD(prof_empty)
          // the leader's barrier was released by the MMA thread's commit: tell the peer's producer.
          // (Not during the first trip round the ring, where every stage is free from the start and
          // the waits on both sides pass without any arrival.)
          if (leader && fills >= kU2Stages) mbar_arrive_cluster(mapa_u32(smem_u32(&bar_empty[stage]), 1));
          if (fills < kU2Stages) ++fills;
          const uint32_t full = mapa_u32(smem_u32(&bar_full[stage]), 0);
          const uint32_t sa = smem_base + stage * kU2StageBytes;
          const uint32_t sb = sa + kU2ABytes;
          mbar_expect_tx_cluster(full, bytes);
          if (load_a) tma2_load_2d(sa, &tmA, kb * kUmmaBK, my_row0, full);
          if constexpr (MODE == kFwd) {
            tma2_load_3d(sb, &tmB, my_n0, kb * kUmmaBK, e, full);
            if (bboxes > 1) tma2_load_3d(sb + 8192, &tmB, my_n0 + 64, kb * kUmmaBK, e, full);
          } else {
            tma2_load_3d(sb, &tmB, kb * kUmmaBK, my_n0, e, full);
          }
          if (++stage == kU2Stages) { stage = 0; phase ^= 1u; }
        }
      }
      YB_PROF_FLUSH(leader ? 0 : 1, prof_empty)
    }
    __syncwarp();
  } else if (warp == 1) {
    // =========================== MMA issuer (leader CTA only) ================================
    if (leader && lane == 0) {
      constexpr bool kBMn = (MODE == kFwd);
      // instruction descriptor without its N field (bits 17..22 = N / 8), which depends on the tile
      constexpr uint32_t idesc_base = (1u << 4) | (1u << 7) | (1u << 10) | ((kBMn ? 1u : 0u) << 16) |
                                      ((uint32_t)(256 >> 4) << 24);
      constexpr uint32_t a_kstep = 32 >> 4;
      constexpr uint32_t b_kstep = kBMn ? (16 * 128) >> 4 : 32 >> 4;
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      long long prof_full = 0, prof_tmem = 0, prof_all = 0;
      (void)prof_full; (void)prof_tmem; (void)prof_all;
#ifdef YB_PROF
      const long long prof_begin = clock64();
#endif
      int e_next = expert_of(cluster_id);
      for (int id = cluster_id; id < total && ok; id += n_clusters) {
        int e, row0, n0;
        bool has1;
        decode(id, e_next, e, row0, has1, n0);
        e_next = expert_of(id + n_clusters);
        const uint32_t idesc = idesc_base | ((uint32_t)(min(BN, p.N - n0) >> 3) << 17);
        {
          YB_PROF_T0
          if (!mbar_wait(smem_u32(&bar_tmem_empty[acc]), acc_phase ^ 1u, &abort_flag)) { ok = false; break; }
          YB_PROF_ADD(prof_tmem)
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kUmmaAccStride;
        for (int kb = 0; kb < kblocks; ++kb) {
          {
            YB_PROF_T0
            if (!mbar_wait(smem_u32(&bar_full[stage]), phase, &abort_flag)) { ok = false; break; }
            YB_PROF_ADD(prof_full)
          }
          tc_fence_after();
          const uint32_t sa = smem_base + stage * kU2StageBytes;
          const uint32_t sb = sa + kU2ABytes;
          const uint64_t adesc = make_smem_desc(sa, 16, 1024);
          const uint64_t bdesc = kBMn ? make_smem_desc(sb, 8192, 1024) : make_smem_desc(sb, 16, 1024);
#pragma unroll
          for (int k = 0; k < kUmmaBK / 16; ++k)
            tc2_mma_bf16(d_tmem, adesc + (uint64_t)(k * a_kstep), bdesc + (uint64_t)(k * b_kstep), idesc,
                         (uint32_t)((kb | k) != 0));
          tc2_commit(smem_u32(&bar_empty[stage]));     // frees the stage here; the producer forwards it
          if (++stage == kU2Stages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc2_commit(smem_u32(&bar_tmem_full[acc]));     // the leader's epilogue forwards it to the peer
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
      if (!ok) {
        abort_flag = 1;
        atomicMax(p.header + kHdrStatus, (int)kStatusMmaTimeout);
      }
#ifdef YB_PROF
      prof_all = clock64() - prof_begin;
#endif
      YB_PROF_FLUSH(2, prof_full)
      YB_PROF_FLUSH(3, prof_tmem)
      YB_PROF_FLUSH(4, prof_all)
    }
    __syncwarp();
  } else {
    // =========================== epilogue (warps 2..5 of both CTAs) ==========================
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    int e_next = expert_of(cluster_id);
    for (int id = cluster_id; id < total; id += n_clusters) {
      int e, row0, n0;
      bool has1;
      decode(id, e_next, e, row0, has1, n0);
      e_next = expert_of(id + n_clusters);
      const int row = row0 + (int)rank * 128 + q * 32 + lane;
      if (!mbar_wait(smem_u32(&bar_tmem_full[acc]), acc_phase, &abort_flag)) {
        abort_flag = 1;
        atomicMax(p.header + kHdrStatus, (int)kStatusEpilogueTimeout);
        break;
      }
      // the accumulator is complete in both CTAs: one lane of the leader tells the peer's epilogue
      if (leader && warp == 2 && lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&bar_tmem_full[acc]), 1));
      tc_fence_after();
      if (leader || has1) {
        const uint32_t t_row = tmem_base + acc * kUmmaAccStride + ((uint32_t)(q * 32) << 16);
        const int nchunks = min(BN / 32, (p.N - n0 + 31) / 32);
        uint32_t ra[32], rb[32];
        tc_ld_32x32_issue(t_row, ra);
#pragma unroll 1
        for (int c = 0; c < nchunks; c += 2) {
          tc_ld_wait(ra);
          if (c + 1 < nchunks) tc_ld_32x32_issue(t_row + (c + 1) * 32, rb);
          {
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(ra[i]);
            epi.template apply<32>(e, row, n0 + c * 32, v);
          }
          if (c + 1 < nchunks) {
            tc_ld_wait(rb);
            if (c + 2 < nchunks) tc_ld_32x32_issue(t_row + (c + 2) * 32, ra);
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(rb[i]);
            epi.template apply<32>(e, row, n0 + (c + 1) * 32, v);
          }
        }
      }
      tc_fence_before();
      mbar_arrive_cluster(mapa_u32(smem_u32(&bar_tmem_empty[acc]), 0));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
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

// Off by default: measured on B200 the pair kernel is 7-12 % slower than the one-CTA kernel at
// every token count tried (the extra row padding of 256-row pairs and the cross-CTA signalling
// cost more than the halved B traffic saves).  YAMOE_B200_2CTA=1 selects it.
inline bool umma_2cta_enabled() {
  static int on = []() {
    const char* env = std::getenv("YAMOE_B200_2CTA");
    return env ? std::atoi(env) : 0;
  }();
  return on != 0;
}

template <int MODE, class Epi>
inline int launch_umma_gemm_2cta(const GemmArgs& g, const Epi& epi, int64_t max_rows, int64_t max_tiles,
                                 cudaStream_t stream) {
  if (!umma_available()) return YAMOE_ERR_UNSUPPORTED;
  CUtensorMap tmA, tmB;
  bool ok = true;
  const uint64_t da[2] = {(uint64_t)g.K, (uint64_t)max_rows}, sa[1] = {(uint64_t)g.lda * 2};
  const uint32_t ba[2] = {64, 128};
  ok = ok && make_map(&tmA, g.A, 2, da, sa, ba);
  if (MODE == kFwd) {
    const uint64_t db[3] = {(uint64_t)g.N, (uint64_t)g.K, (uint64_t)g.E};
    const uint64_t sb[2] = {(uint64_t)g.ldb * 2, (uint64_t)g.b_expert_stride * 2};
    const uint32_t bb[3] = {64, 64, 1};
    ok = ok && make_map(&tmB, g.B, 3, db, sb, bb);
  } else {
    const uint64_t db[3] = {(uint64_t)g.K, (uint64_t)g.N, (uint64_t)g.E};
    const uint64_t sb[2] = {(uint64_t)g.ldb * 2, (uint64_t)g.b_expert_stride * 2};
    const uint32_t bb[3] = {64, 128, 1};
    ok = ok && make_map(&tmB, g.B, 3, db, sb, bb);
  }
  if (!ok) return YAMOE_ERR_CUDA;
  auto kern = umma_gemm_2cta_kernel<MODE, Epi>;
  static PerDevice<int> attr_done;   // per template instantiation and device
  const int dev = current_device_index();
  if (!attr_done.get(dev)) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kU2Smem) != cudaSuccess)
      return YAMOE_ERR_CUDA;
    attr_done.set(dev, 1);
  }
  Umma2Params p{g.N, g.K, g.E, g.pair_expert, g.pair_off, g.pad_off, const_cast<int32_t*>(g.header)};
  const int NT = (int)ceil_div(g.N, kU2BN);
  const int64_t total_max = max_tiles * NT;                       // upper bound on tile pairs x column tiles
  int grid = (int)std::min<int64_t>(2 * total_max, umma_sm_count()) & ~1;
  if (grid <= 0) return YAMOE_OK;
  kern<<<grid, kU2Threads, kU2Smem, stream>>>(tmA, tmB, p, epi);
  return cudaGetLastError() == cudaSuccess ? YAMOE_OK : YAMOE_ERR_CUDA;
}

// Row-tiled GEMMs: pair kernel (when selected and the tile-pair tables exist) or one-CTA kernel.
template <int MODE, class Epi>
inline int launch_umma(const GemmArgs& g, const Epi& epi, int64_t max_rows, int64_t max_tiles, cudaStream_t stream) {
  if constexpr (MODE != kWgrad) {
    const bool pairs = g.pair_expert != nullptr && g.pair_off != nullptr && g.gather_rows == nullptr;
    if (pairs && umma_2cta_enabled()) return launch_umma_gemm_2cta<MODE>(g, epi, max_rows, max_tiles, stream);
  }
  return launch_umma_gemm<MODE>(g, epi, max_rows, max_tiles, stream);
}

}  // namespace yb
