// tcgen05 / TMEM / TMA grouped GEMM for bf16 operands with fp32 accumulation (sm_100a).
//
// One persistent, warp-specialised kernel serves the five GEMMs of the expert forward and
// backward passes (the reference runs them as padded cuBLAS bmm calls: csrc/batch_mm.cu:27-30,
// csrc/experts_backward.cu:181,198,279-282,309-311).  Arrangements (see simt_gemm.cuh):
//   kFwd    A rows K-major (TMA 2D),           B = W[e][k][n]  MN-major (TMA 4D, blocked by 64 columns)
//   kDgrad  A rows K-major (TMA 2D),           B = W[e][n][k]  K-major  (TMA 3D)
//   kWgrad  A = act[r][m] MN-major (TMA 3D),   B = grad[r][n]  MN-major (TMA 3D), k = rows of e
// The 128-byte swizzle limits a box to 64 columns of an MN-major operand.  Such an operand is
// therefore described as (64 columns, rows, column block[, expert]): a box of 64 x 64 x BN/64
// brings a whole stage with ONE copy and lands as BN/64 consecutive 8 KB boxes, exactly what
// separate copies would have produced.  The single producer thread sits on the stage round trip,
// and one copy instead of four took the gate_up GEMM of the 20B forward from 501 to 457 us.
// Operands whose width (or row pitch, for the weight gradient) is not a multiple of 64 fall back
// to one copy per box.
//
// CTA = 6 warps: warp 0 issues TMA loads into a 4-stage shared-memory ring (128-byte swizzle,
// 48 KB per stage at BN = 256), warp 1 allocates TMEM and issues tcgen05.mma (128 x BN x 16 per
// instruction, one elected thread), warps 2..5 drain the fp32 accumulator from TMEM with tcgen05.ld and run the epilogue
// functor.  Two accumulators (2 x 256 TMEM columns) let the epilogue of tile i overlap the
// main loop of tile i+1.  Tiles are walked expert by expert with the row tile varying fastest,
// so the CTAs running at any moment share one expert's weight slab in L2.
//
// Tile look-up is kept off the critical path: the padded row offsets of all experts sit in
// shared memory, and the one table entry a tile still needs from global memory (its expert) is
// fetched one tile ahead, so that no role stalls on a dependent global load between two tiles.
// The last column tile of a matrix whose width is not a multiple of BN is issued with a narrower
// instruction (N = remaining columns); columns past the edge are zero-filled by the copy (or,
// with one copy per box, not loaded at all).
//
// Every mbarrier wait is bounded: after kWaitLimitNs the waiting role raises an abort flag,
// all roles leave their loops, the CTA frees its TMEM, records a status code in the workspace
// header and returns.
#pragma once
#include <cuda.h>

#include <cstdlib>
#include <mutex>
#include <type_traits>

#include "common.cuh"
#include "epilogues.cuh"
#include "simt_gemm.cuh"

namespace yb {

constexpr int kUmmaBM = 128;
constexpr int kUmmaBK = 64;            // 64 bf16 = one 128-byte swizzle row
constexpr int kUmmaThreads = 192;          // TMA producer, MMA issuer, four epilogue warps
constexpr int kUmmaGatherThreads = 128;    // four more warps that gather the A rows when the gather is fused
constexpr int kUmmaAccStride = 256;    // TMEM columns between the two accumulators
constexpr int kUmmaMaxExperts = 1024;  // padded row offsets of up to this many experts are cached in shared memory
constexpr uint64_t kWaitLimitNs = 2000000000ull;

// Optional wait-time accounting for pipeline studies (compile with -DYB_PROF): every role adds the
// SM clocks it spent inside bounded waits to g_prof[slot]; yamoe_b200_prof_read returns and clears them.
#ifdef YB_PROF
__device__ unsigned long long g_prof[16];
#define YB_PROF_T0 const long long _pt0 = clock64();
#define YB_PROF_ADD(var) var += clock64() - _pt0;
#define YB_PROF_FLUSH(slot, var) atomicAdd(&g_prof[slot], (unsigned long long)(var));
#else
#define YB_PROF_T0
#define YB_PROF_ADD(var)
#define YB_PROF_FLUSH(slot, var)
#endif

enum DeviceStatus { kStatusOk = 0, kStatusProducerTimeout = 1, kStatusMmaTimeout = 2, kStatusEpilogueTimeout = 3,
                    kStatusGateTimeout = 5 };   // 5: rows that another GPU was to deliver did not arrive in time

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait on an mbarrier phase.  Returns false when the wait was abandoned.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          uint64_t limit_ns = kWaitLimitNs) {
  uint64_t t0 = 0;
  for (uint32_t it = 0;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 255u) == 255u) {
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      if (*abort_flag != 0 || now - t0 > limit_ns) return false;
    }
  }
}

// Test aid: one thread waits, with the given limit, on a barrier that nothing ever arrives at,
// and records what the grouped GEMM's roles record when a wait gives up.  No TMA, no TMEM.
__global__ void mbar_wait_probe_kernel(int32_t* header, uint64_t limit_ns) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (!mbar_wait(smem_u32(&bar), 0, &abort_flag, limit_ns)) {
      abort_flag = 1;
      atomicMax(header + kHdrStatus, (int)kStatusProducerTimeout);
    }
  }
  __syncthreads();
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
// 16-byte asynchronous copy global -> shared (L2 only); src_bytes = 0 writes zeros instead.
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
// makes this thread's completed generic-proxy writes to shared memory visible to the async proxy (tcgen05.mma)
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}
// Issues the TMEM load of 32 columns for this thread's lane; the registers are valid only after
// tc_ld_wait().
__device__ __forceinline__ void tc_ld_32x32_issue(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
// Waits for the outstanding TMEM loads.  The registers are passed through the statement so that
// the compiler cannot schedule any use of them before the wait.
__device__ __forceinline__ void tc_ld_wait(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
                 "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
                 "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
               :: "memory");
}

// Shared-memory matrix descriptor (tcgen05 format): start address, leading / stride byte
// offsets in 16-byte units, descriptor version 1, 128-byte swizzle.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;   // descriptor version (Blackwell)
  d |= (uint64_t)2 << 61;   // SWIZZLE_128B
  return d;
}

// Epilogue functors that declare `static constexpr bool kStagedRows = true` get their output rows
// written in 128-byte pieces: a warp parks two 32-column chunks of its 32 rows in shared memory
// (bf16), then stores them so that eight lanes cover 128 contiguous bytes of one row.  Plain
// functors store 16 bytes per lane to 32 different rows per instruction, which local memory
// tolerates (L2 merges the pieces) but which wastes most of every NVLink packet when the row lives
// in another GPU's memory.  Such a functor provides, besides apply():
//   kOutPerChunk                                    32, or 16 for a functor that turns column pairs into one value
//   T* row_ptr(int row) const                       start of the output row, or nullptr to skip it
//   values<32>(e, row, n0, v, o) const              o[0 .. kOutPerChunk) = the outputs of accumulator columns n0 .. n0+31
// Functors that read a tile-shaped operand of their own in the epilogue (EpiGluBackward reads the
// stored pre-activations) may declare `prefetch_tile(row, n0, ncols)`: the epilogue calls it for
// its row before it waits for the accumulator, so that those lines are on their way to L2/L1
// while the main loop of the tile is still running.
template <class E, class = void>
struct epi_prefetches : std::false_type {};
template <class E>
struct epi_prefetches<E, std::enable_if_t<E::kPrefetchTile>> : std::true_type {};

// Forward epilogues that declare `static constexpr bool kMayGather = true` also get the kernel
// instantiation whose extra warps gather the A rows (one more kernel per such functor).
template <class E, class = void>
struct epi_gathers : std::false_type {};
template <class E>
struct epi_gathers<E, std::enable_if_t<E::kMayGather>> : std::true_type {};

template <class E, class = void>
struct epi_staged : std::false_type {};
template <class E>
struct epi_staged<E, std::enable_if_t<E::kStagedRows>> : std::true_type {};
constexpr int kStagePitch = 144;    // bytes per parked row: 64 bf16 + 16 bytes against bank conflicts

struct UmmaParams {
  int M, N, K, E;           // as GemmArgs
  const int32_t* tile_expert;   // null: one group (expert 0) owns all `uniform_tiles` row tiles, no tables
  const int32_t* pad_off;
  int uniform_tiles;
  int32_t* header;
  const int32_t* gather_rows;   // kFwd: source row of every padded row (gather fused into the A operand), or null
  const void* gather_src;       //       the un-permuted source rows [*, gather_ld]
  int64_t gather_ld;
  GemmGate gate;                // see GemmGate
  // MN-major operands whose width is a multiple of 64 are described as (64 columns, rows, column
  // block[, expert]) so that ONE copy brings all the 64-column boxes of a stage (box 64 x 64 x BN/64):
  // the producer thread issues two copies per k-block instead of five (forward) or six (weight
  // gradient), and the last box lands earlier
  int a_wide, b_wide;
};

template <int BN>
struct UmmaSmem {
  static constexpr int kABytes = kUmmaBM * 128;
  static constexpr int kBBytes = BN * 128;
  static constexpr int kStageBytes = kABytes + kBBytes;
#ifdef YB_STAGES
  static constexpr int kStages = YB_STAGES;                         // timing experiments only
#else
  static constexpr int kStages = (227 * 1024 - 8192) / kStageBytes;  // 6 / 5 / 4 stages for BN 128 / 192 / 256
#endif
  static constexpr int kTotal = kStages * kStageBytes + 1024;       // + slack for 1024-byte alignment
};

// GATHER (kFwd only): the kernel is launched with four more warps that fetch the A rows themselves
// (see "A-row gather" below); without it the kernel has six warps and no trace of that role.
template <int MODE, int BN, class Epi, bool GATHER = false>
__global__ void __launch_bounds__(kUmmaThreads + (GATHER ? kUmmaGatherThreads : 0), 1)
umma_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const UmmaParams p, const Epi epi) {
  using SM = UmmaSmem<BN>;
  constexpr int kUmmaStages = SM::kStages;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kUmmaStages];
  __shared__ __align__(8) uint64_t bar_empty[kUmmaStages];
  __shared__ __align__(8) uint64_t bar_tmem_full[2];
  __shared__ __align__(8) uint64_t bar_tmem_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int32_t s_pad[kUmmaMaxExperts + 1];   // copy of pad_off[0..E]
  constexpr bool kStaged = epi_staged<Epi>::value;
  __shared__ __align__(16) uint8_t s_out[kStaged ? 4 * 32 * kStagePitch : 16];   // parked output rows, per epilogue warp

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;

  // Gather fused into the A operand: four extra warps copy the tile's rows straight from the
  // un-permuted source into the swizzled A stage (cp.async), the TMA producer loads only B, and a
  // stage is full after the producer's arrival plus one per gather warp.
  constexpr bool gather = GATHER && MODE == kFwd;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kUmmaStages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), gather ? 1 + kUmmaGatherThreads / 32 : 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&bar_tmem_full[a]), 1);
      mbar_init(smem_u32(&bar_tmem_empty[a]), 128);
    }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_base_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  // Set-up is done: let the next kernel on the stream begin its own set-up, then wait until the
  // previous kernel has completed before touching anything it produced.
  pdl_trigger();
  const bool gated = p.gate.prep != nullptr;
#ifdef YB_PROF
  if (gated && threadIdx.x == 0) atomicMin(&g_prof[8], (unsigned long long)global_timer_ns());
#endif
  if (!gated) {
    pdl_wait();
  } else {
    // launched next to the kernel that fills the tables and the A rows: no wait for its completion,
    // only for the tables (bounded); a time-out leaves this kernel without work
    if (threadIdx.x == 0) {
      const uint64_t t0 = global_timer_ns();
      int ready = 1;
      for (;;) {
        int v;
        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p.gate.prep) : "memory");
        if (v >= p.gate.prep_target) break;
        if (global_timer_ns() - t0 > p.gate.wait_ns) { ready = 0; break; }
        __nanosleep(200);
      }
      if (!ready) {
        abort_flag = 1;
        atomicMax(p.header + kHdrStatus, (int)kStatusGateTimeout);
      }
    }
    __syncthreads();
  }
  const bool uniform = p.tile_expert == nullptr && MODE != kWgrad;
  const bool pad_in_smem = uniform || p.E <= kUmmaMaxExperts;
  if (pad_in_smem) {
    if (uniform) {
      if (threadIdx.x == 0) { s_pad[0] = 0; s_pad[1] = p.uniform_tiles * kTileM; }
    } else {
      for (int i = threadIdx.x; i <= p.E; i += blockDim.x) s_pad[i] = p.pad_off[i];
    }
    __syncthreads();
  }
  const int32_t* pad = pad_in_smem ? s_pad : p.pad_off;

  // ---- tile walk (identical in every role) ---------------------------------------------------
  const int NT = (p.N + BN - 1) / BN;
  int total;
  int MT = 0;
  if constexpr (MODE == kWgrad) {
    MT = (p.M + kUmmaBM - 1) / kUmmaBM;
    total = p.E * MT * NT;
  } else {
    total = (uniform ? p.uniform_tiles : p.header[kHdrRowTiles]) * NT;
  }
  if (gated && abort_flag != 0) total = 0;
  // Expert of tile `id` for the row-tiled arrangements: the only part of a tile's description
  // that comes from global memory.  Every role asks for it one tile ahead.
  auto expert_of = [&](int id) -> int {
    if constexpr (MODE == kWgrad) return 0;
    if (uniform) return 0;
    return id < total ? __ldg(p.tile_expert + id / NT) : 0;
  };
  auto decode = [&](int id, int e_hint, int& e, int& row0, int& n0, int& kb_begin_row, int& kblocks) {
    if constexpr (MODE == kWgrad) {
      e = id / (MT * NT);
      const int rem = id - e * (MT * NT);
      const int nt = rem / MT;
      row0 = (rem - nt * MT) * kUmmaBM;
      n0 = nt * BN;
      kb_begin_row = pad[e];
      kblocks = (pad[e + 1] - kb_begin_row) / kUmmaBK;
    } else {
      e = e_hint;
      const int p0 = pad[e];
      const int first = p0 / kTileM;
      const int cnt = (pad[e + 1] - p0) / kTileM;
      const int local = id - first * NT;
      const int nt = local / cnt;
      row0 = (first + (local - nt * cnt)) * kUmmaBM;
      n0 = nt * BN;
      kb_begin_row = 0;
      kblocks = p.K / kUmmaBK;
    }
  };

  if (warp == 0) {
    // =========================== TMA producer ================================================
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      long long prof_empty = 0;
      (void)prof_empty;
      int gate_done = -1;                  // last group whose rows are known to have arrived
      int e_next = expert_of(blockIdx.x);
      for (int id = blockIdx.x; id < total && ok; id += gridDim.x) {
        int e, row0, n0, krow, kblocks;
        decode(id, e_next, e, row0, n0, krow, kblocks);
        e_next = expert_of(id + gridDim.x);      // consumed after this tile's k loop
        // MN-major B arrives as 64-column boxes: the last column tile asks only for those it has.
        // (The K-major B of the data gradients is one box of BN rows; rows past N read as zeros.)
        const int nboxes = MODE == kDgrad ? BN / 64 : (min(BN, p.N - n0) + 63) >> 6;
        const uint32_t stage_tx = (gather ? 0 : SM::kABytes) + (p.b_wide ? BN / 64 : nboxes) * 8192;
        if (MODE == kFwd && p.gate.arrived != nullptr && e != gate_done) {
          // the A rows of this group come from other GPUs: all of them must have landed
          const int need = p.gate.needed[e];
          const uint64_t t0 = global_timer_ns();
          for (;;) {
            int v;
            asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p.gate.arrived + e) : "memory");
            if (v >= need) break;
            if (abort_flag != 0 || global_timer_ns() - t0 > p.gate.wait_ns) { ok = false; break; }
            __nanosleep(100);
          }
          if (!ok) {
            abort_flag = 1;
            atomicMax(p.header + kHdrStatus, (int)kStatusGateTimeout);
            break;
          }
          asm volatile("fence.proxy.async.global;" ::: "memory");   // the TMA loads below read what those stores wrote
#ifdef YB_PROF
          if (gate_done < 0) atomicMax(&g_prof[9], (unsigned long long)global_timer_ns());
          atomicMax(&g_prof[12], (unsigned long long)global_timer_ns());
#endif
          gate_done = e;
        }
        for (int kb = 0; kb < kblocks; ++kb) {
          YB_PROF_T0
          if (!mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, &abort_flag)) {
            abort_flag = 1;
            atomicMax(p.header + kHdrStatus, (int)kStatusProducerTimeout);
            ok = false;
            break;
          }
          YB_PROF_ADD(prof_empty)
          const uint32_t full = smem_u32(&bar_full[stage]);
          const uint32_t sa = smem_base + stage * SM::kStageBytes;
          const uint32_t sb = sa + SM::kABytes;
          mbar_expect_tx(full, stage_tx);
          if constexpr (MODE == kWgrad) {
            const int r = krow + kb * kUmmaBK;
            if (p.a_wide) {
              tma_load_3d(sa, &tmA, 0, r, row0 >> 6, full);
            } else {
#pragma unroll
              for (int i = 0; i < kUmmaBM / 64; ++i) tma_load_2d(sa + i * 8192, &tmA, row0 + i * 64, r, full);
            }
            if (p.b_wide) {
              tma_load_3d(sb, &tmB, 0, r, n0 >> 6, full);
            } else {
#pragma unroll
              for (int i = 0; i < BN / 64; ++i)
                if (i < nboxes) tma_load_2d(sb + i * 8192, &tmB, n0 + i * 64, r, full);
            }
          } else {
            if (!gather) tma_load_2d(sa, &tmA, kb * kUmmaBK, row0, full);
            if constexpr (MODE == kFwd) {
              if (p.b_wide) {
                tma_load_4d(sb, &tmB, 0, kb * kUmmaBK, n0 >> 6, e, full);
              } else {
#pragma unroll
                for (int i = 0; i < BN / 64; ++i)
                  if (i < nboxes) tma_load_3d(sb + i * 8192, &tmB, n0 + i * 64, kb * kUmmaBK, e, full);
              }
            } else {
              tma_load_3d(sb, &tmB, kb * kUmmaBK, n0, e, full);
            }
          }
          if (++stage == kUmmaStages) { stage = 0; phase ^= 1u; }
        }
      }
      YB_PROF_FLUSH(0, prof_empty)
    }
    __syncwarp();
  } else if (warp == 1) {
    // =========================== MMA issuer ==================================================
    if (lane == 0) {
      constexpr bool kAMn = (MODE == kWgrad);
      constexpr bool kBMn = (MODE != kDgrad);
      // instruction descriptor without its N field (bits 17..22 = N / 8), which depends on the tile
      constexpr uint32_t idesc_base = (1u << 4) | (1u << 7) | (1u << 10) | ((kAMn ? 1u : 0u) << 15) |
                                      ((kBMn ? 1u : 0u) << 16) | ((uint32_t)(kUmmaBM >> 4) << 24);
      constexpr uint32_t a_kstep = kAMn ? (16 * 128) >> 4 : 32 >> 4;   // descriptor units of 16 bytes
      constexpr uint32_t b_kstep = kBMn ? (16 * 128) >> 4 : 32 >> 4;
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      long long prof_full = 0, prof_tmem = 0, prof_all = 0;
      (void)prof_full; (void)prof_tmem; (void)prof_all;
#ifdef YB_PROF
      const long long prof_begin = clock64();
#endif
      int e_next = expert_of(blockIdx.x);
      for (int id = blockIdx.x; id < total && ok; id += gridDim.x) {
        int e, row0, n0, krow, kblocks;
        decode(id, e_next, e, row0, n0, krow, kblocks);
        e_next = expert_of(id + gridDim.x);
        if (kblocks == 0) continue;
        // columns this tile really has, rounded up to the instruction's granularity of 16
        const uint32_t ncols = (uint32_t)(min(BN, p.N - n0) + 15) & ~15u;
        const uint32_t idesc = idesc_base | ((ncols >> 3) << 17);
        {
          YB_PROF_T0
          if (!mbar_wait(smem_u32(&bar_tmem_empty[acc]), acc_phase ^ 1u, &abort_flag)) {
            abort_flag = 1;
            atomicMax(p.header + kHdrStatus, (int)kStatusMmaTimeout);
            break;
          }
          YB_PROF_ADD(prof_tmem)
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kUmmaAccStride;
        for (int kb = 0; kb < kblocks; ++kb) {
          {
            YB_PROF_T0
            if (!mbar_wait(smem_u32(&bar_full[stage]), phase, &abort_flag)) {
              abort_flag = 1;
              atomicMax(p.header + kHdrStatus, (int)kStatusMmaTimeout);
              ok = false;
              break;
            }
            YB_PROF_ADD(prof_full)
          }
          tc_fence_after();
          const uint32_t sa = smem_base + stage * SM::kStageBytes;
          const uint32_t sb = sa + SM::kABytes;
          const uint64_t adesc = kAMn ? make_smem_desc(sa, 8192, 1024) : make_smem_desc(sa, 16, 1024);
          const uint64_t bdesc = kBMn ? make_smem_desc(sb, 8192, 1024) : make_smem_desc(sb, 16, 1024);
#pragma unroll
          for (int k = 0; k < kUmmaBK / 16; ++k)
            tc_mma_bf16(d_tmem, adesc + (uint64_t)(k * a_kstep), bdesc + (uint64_t)(k * b_kstep), idesc,
                        (uint32_t)((kb | k) != 0));
          tc_commit(smem_u32(&bar_empty[stage]));
          if (++stage == kUmmaStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc_commit(smem_u32(&bar_tmem_full[acc]));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
#ifdef YB_PROF
      prof_all = clock64() - prof_begin;
#endif
      YB_PROF_FLUSH(2, prof_full)
      YB_PROF_FLUSH(3, prof_tmem)
      YB_PROF_FLUSH(4, prof_all)
    }
    __syncwarp();
  } else if (gather && warp >= kUmmaThreads / 32) {
    // =========================== A-row gather (warps 6..9, only launched when gathering) ========
    // Warp g copies rows 32g .. 32g+31 of the tile: eight lanes cover the 128 bytes one row
    // contributes to a 64-deep k-block, so an instruction fetches four full 128-byte lines.  The
    // 16-byte piece c of row r lands at piece (c ^ (r & 7)) of that row: the 128-byte swizzle
    // the MMA's descriptor expects (what a tiled TMA load would have produced).  Copies are
    // asynchronous; three k-blocks are kept in flight per warp, and a k-block is announced on the
    // stage's full barrier once its copies have completed and a proxy fence has made them visible
    // to the tensor core.
    if constexpr (gather) {
      {
        constexpr int kInFlight = 3;
        const int gw = warp - kUmmaThreads / 32;
        const int piece = lane & 7, sub = lane >> 3;
        const char* src = reinterpret_cast<const char*>(p.gather_src);
        const size_t row_bytes = (size_t)p.gather_ld * 2;
        int stage = 0, arr_stage = 0, pending = 0;
        uint32_t phase = 0;
        bool ok = true;
        int e_next = expert_of(blockIdx.x);
        for (int id = blockIdx.x; id < total && ok; id += gridDim.x) {
          int e, row0, n0, krow, kblocks;
          decode(id, e_next, e, row0, n0, krow, kblocks);
          e_next = expert_of(id + gridDim.x);
          int tok[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) tok[i] = __ldg(p.gather_rows + row0 + gw * 32 + i * 4 + sub);
          for (int kb = 0; kb < kblocks; ++kb) {
            int good = 1;
            if (lane == 0) good = mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, &abort_flag) ? 1 : 0;
            good = __shfl_sync(0xffffffffu, good, 0);
            if (!good) {
              if (lane == 0) {
                abort_flag = 1;
                atomicMax(p.header + kHdrStatus, (int)kStatusProducerTimeout);
              }
              ok = false;
              break;
            }
            const uint32_t sa = smem_base + stage * SM::kStageBytes;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int r = gw * 32 + i * 4 + sub;
              const bool real = tok[i] >= 0;                       // padding rows are written as zeros
              cp_async_16(sa + r * 128 + ((piece ^ (r & 7)) << 4),
                          src + (real ? (size_t)tok[i] * row_bytes + (size_t)kb * 128 + piece * 16 : 0), real ? 16u : 0u);
            }
            cp_async_commit();
            if (++pending == kInFlight) {
              cp_async_wait<kInFlight - 1>();
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) mbar_arrive(smem_u32(&bar_full[arr_stage]));
              if (++arr_stage == kUmmaStages) arr_stage = 0;
              --pending;
            }
            if (++stage == kUmmaStages) { stage = 0; phase ^= 1u; }
          }
        }
        cp_async_wait<0>();                 // nothing of this warp is in flight past this point
        fence_proxy_async_smem();
        __syncwarp();
        if (ok && lane == 0)
          for (; pending > 0; --pending) {
            mbar_arrive(smem_u32(&bar_full[arr_stage]));
            if (++arr_stage == kUmmaStages) arr_stage = 0;
          }
      }
    }
    __syncwarp();
  } else {
    // =========================== epilogue (warps 2..5) =======================================
    const int q = warp & 3;                    // TMEM lane quarter this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    int e_next = expert_of(blockIdx.x);
    for (int id = blockIdx.x; id < total; id += gridDim.x) {
      int e, row0, n0, krow, kblocks;
      decode(id, e_next, e, row0, n0, krow, kblocks);
      e_next = expert_of(id + gridDim.x);
      const int row = row0 + q * 32 + lane;
      if (kblocks == 0) {
        float z[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) z[i] = 0.f;
        for (int c = 0; c < BN / 32; ++c)
          if (n0 + c * 32 < p.N) epi.template apply<32>(e, row, n0 + c * 32, z);
        continue;
      }
      if constexpr (epi_prefetches<Epi>::value) epi.prefetch_tile(row, n0, min(BN, p.N - n0));
      if (!mbar_wait(smem_u32(&bar_tmem_full[acc]), acc_phase, &abort_flag)) {
        abort_flag = 1;
        atomicMax(p.header + kHdrStatus, (int)kStatusEpilogueTimeout);
        break;
      }
      tc_fence_after();
      const uint32_t t_row = tmem_base + acc * kUmmaAccStride + ((uint32_t)(q * 32) << 16);
      // two register buffers: the TMEM load of chunk c+1 is in flight while chunk c is processed
      const int nchunks = min(BN / 32, (p.N - n0 + 31) / 32);
      uint32_t ra[32], rb[32];
      tc_ld_32x32_issue(t_row, ra);
      if constexpr (kStaged) {
        constexpr int OUT = Epi::kOutPerChunk;                            // output columns per 32-column chunk
        constexpr int CPP = 64 / OUT;                                     // chunks that fill a parked 128-byte row
        constexpr int DIV = 32 / OUT;                                     // accumulator columns per output column
        uint8_t* mine = s_out + (q * 32 + lane) * kStagePitch;            // this thread's parked row
        const unsigned long long my_dst = reinterpret_cast<unsigned long long>(epi.row_ptr(row));
        const int piece = lane & 7, sub = lane >> 3;                      // 16-byte piece of a row, row within a group of 4
        const int n_out = p.N / DIV;
        auto park = [&](const uint32_t (&r)[32], int c) {
          float v[32], o[OUT];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
          epi.template values<32>(e, row, n0 + c * 32, v, o);
          uint4* dst = reinterpret_cast<uint4*>(mine + (c % CPP) * OUT * 2);
#pragma unroll
          for (int i = 0; i < OUT / 8; ++i)
            dst[i] = make_uint4(pack_bf16x2(o[8 * i], o[8 * i + 1]), pack_bf16x2(o[8 * i + 2], o[8 * i + 3]),
                                pack_bf16x2(o[8 * i + 4], o[8 * i + 5]), pack_bf16x2(o[8 * i + 6], o[8 * i + 7]));
        };
        auto flush = [&](int c_last) {                                    // parked chunks end with chunk c_last
          __syncwarp();
          const int col0 = (n0 + (c_last - c_last % CPP) * 32) / DIV;     // first output column of the parked piece
          const int ncol = min((c_last % CPP + 1) * OUT, n_out - col0);   // columns parked and present
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r = i * 4 + sub;                                    // row of the warp's 32
            const unsigned lo = __shfl_sync(0xffffffffu, (unsigned)(my_dst & 0xffffffffull), r);
            const unsigned hi = __shfl_sync(0xffffffffu, (unsigned)(my_dst >> 32), r);
            const unsigned long long dst = ((unsigned long long)hi << 32) | lo;
            if (dst != 0 && piece * 8 < ncol) {
              const uint4 val = *reinterpret_cast<const uint4*>(s_out + (q * 32 + r) * kStagePitch + piece * 16);
              *reinterpret_cast<uint4*>(dst + (size_t)(col0 + piece * 8) * 2) = val;
            }
          }
          __syncwarp();
        };
#pragma unroll 1
        for (int c = 0; c < nchunks; c += 2) {
          tc_ld_wait(ra);
          if (c + 1 < nchunks) tc_ld_32x32_issue(t_row + (c + 1) * 32, rb);
          park(ra, c);
          if (c % CPP == CPP - 1 || c + 1 == nchunks) flush(c);
          if (c + 1 < nchunks) {
            tc_ld_wait(rb);
            if (c + 2 < nchunks) tc_ld_32x32_issue(t_row + (c + 2) * 32, ra);
            park(rb, c + 1);
            if ((c + 1) % CPP == CPP - 1 || c + 2 == nchunks) flush(c + 1);
          }
        }
      } else {
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
      mbar_arrive(smem_u32(&bar_tmem_empty[acc]));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  // ---- teardown ---------------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (abort_flag != 0) {
    // give copies that may still be in flight time to land before the shared memory is released
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
  // A gated kernel ran next to its predecessor; it ends only once that kernel has ended, so that
  // "this kernel is complete" keeps implying "everything before it on the stream is complete".
  if (gated) pdl_wait();
}

// ---------------------------------------------------------------------------------------------
// Host side: tensor maps and launch
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  return fn;
}

// The tcgen05 kernels need the driver's tensor-map encoder and a device of compute capability 10.x
// (the library is built for sm_100a only, but the check keeps the answer honest per device).
inline bool umma_available() {
  if (encode_tiled_fn() == nullptr) return false;
  static PerDevice<int> major_plus_1;
  const int dev = current_device_index();
  int m = major_plus_1.get(dev);
  if (m == 0) {
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) major = 0;
    m = major + 1;
    major_plus_1.set(dev, m);
  }
  return m - 1 == 10;
}

// bf16 tensor map with 128-byte swizzle; dims / box innermost first, strides in bytes for dims 1...
// Encoding a map is a driver call that costs some tens of microseconds of host time; the same
// (pointer, shape, box) comes back call after call (weights, persistent buffers, workspaces that the
// caching allocator hands out again), so the last maps are kept in a small table.
struct TensorMapKey {
  const void* base;
  int rank;
  uint64_t dims[4], strides[3];
  uint32_t box[4];
  bool operator==(const TensorMapKey& o) const {
    if (base != o.base || rank != o.rank) return false;
    for (int i = 0; i < rank; ++i)
      if (dims[i] != o.dims[i] || box[i] != o.box[i]) return false;
    for (int i = 0; i + 1 < rank; ++i)
      if (strides[i] != o.strides[i]) return false;
    return true;
  }
};

inline bool make_map(CUtensorMap* m, const void* base, int rank, const uint64_t* dims, const uint64_t* strides,
                     const uint32_t* box) {
  constexpr int kSlots = 32;
  static TensorMapKey keys[kSlots];
  static CUtensorMap maps[kSlots];
  static int used = 0, next = 0;
  static std::mutex mu;
  TensorMapKey key{};
  key.base = base;
  key.rank = rank;
  for (int i = 0; i < rank; ++i) { key.dims[i] = dims[i]; key.box[i] = box[i]; }
  for (int i = 0; i + 1 < rank; ++i) key.strides[i] = strides[i];
  {
    std::lock_guard<std::mutex> lock(mu);
    for (int i = 0; i < used; ++i)
      if (keys[i] == key) { *m = maps[i]; return true; }
  }
  cuuint64_t gd[4];
  cuuint64_t gs[3];
  cuuint32_t bx[4], es[4] = {1, 1, 1, 1};
  for (int i = 0; i < rank; ++i) { gd[i] = dims[i]; bx[i] = box[i]; }
  for (int i = 0; i + 1 < rank; ++i) gs[i] = strides[i];
  CUresult r = encode_tiled_fn()(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), gd,
                                 gs, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  std::lock_guard<std::mutex> lock(mu);
  const int slot = used < kSlots ? used++ : (next = (next + 1) % kSlots);
  keys[slot] = key;
  maps[slot] = *m;
  return true;
}

inline int umma_sm_count() {
  static PerDevice<int> count;
  const int dev = current_device_index();
  int n = count.get(dev);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    count.set(dev, n);
  }
  return n;
}

// Output-tile width of the tcgen05 GEMMs (128, 192 or 256 columns); YAMOE_B200_BN overrides.
inline int umma_tile_n() {
  static int bn = []() {
    const char* env = std::getenv("YAMOE_B200_BN");
    int v = env ? std::atoi(env) : 0;
    return (v == 128 || v == 192 || v == 256) ? v : 256;
  }();
  return bn;
}

template <int MODE, int BN, class Epi, bool GATHER>
inline int launch_umma_kernel(const GemmArgs& g, const Epi& epi, const CUtensorMap& tmA, const CUtensorMap& tmB,
                              int64_t max_tiles, bool a_wide, bool b_wide, cudaStream_t stream);

template <int MODE, int BN, class Epi>
inline int launch_umma_gemm_bn(const GemmArgs& g, const Epi& epi, int64_t max_rows, int64_t max_tiles,
                               cudaStream_t stream) {
  if (!umma_available()) return YAMOE_ERR_UNSUPPORTED;
  CUtensorMap tmA, tmB;
  bool ok = true;
  const bool gather = MODE == kFwd && g.gather_rows != nullptr;
  // one copy per operand and k-block where the MN-major operand's width allows the blocked view
  // (YAMOE_B200_WIDE_TMA=0 keeps one copy per 64-column box)
  static const bool wide_on = []() {
    const char* env = std::getenv("YAMOE_B200_WIDE_TMA");
    return env == nullptr || std::atoi(env) != 0;
  }();
  // (weight gradient: the operands' row pitch decides - columns between the width and the pitch
  // exist in memory, and whatever they hold only reaches output rows / columns that are not stored)
  const bool a_wide = wide_on && MODE == kWgrad && g.lda % 64 == 0 && g.M <= g.lda;
  const bool b_wide = wide_on && (MODE == kWgrad ? (g.ldb % 64 == 0 && g.N <= g.ldb) : (MODE == kFwd && g.N % 64 == 0));
  if (MODE == kWgrad) {
    const uint32_t ba[2] = {64, 64};
    if (a_wide) {
      const uint64_t da[3] = {64, (uint64_t)max_rows, (uint64_t)g.lda / 64}, sa[2] = {(uint64_t)g.lda * 2, 128};
      const uint32_t bw[3] = {64, 64, kUmmaBM / 64};
      ok = ok && make_map(&tmA, g.A, 3, da, sa, bw);
    } else {
      const uint64_t da[2] = {(uint64_t)g.M, (uint64_t)max_rows}, sa[1] = {(uint64_t)g.lda * 2};
      ok = ok && make_map(&tmA, g.A, 2, da, sa, ba);
    }
    if (b_wide) {
      const uint64_t db[3] = {64, (uint64_t)max_rows, (uint64_t)g.ldb / 64}, sb[2] = {(uint64_t)g.ldb * 2, 128};
      const uint32_t bw[3] = {64, 64, BN / 64};
      ok = ok && make_map(&tmB, g.B, 3, db, sb, bw);
    } else {
      const uint64_t db[2] = {(uint64_t)g.N, (uint64_t)max_rows}, sb[1] = {(uint64_t)g.ldb * 2};
      ok = ok && make_map(&tmB, g.B, 2, db, sb, ba);
    }
  } else {
    const uint64_t da[2] = {(uint64_t)g.K, (uint64_t)max_rows};
    const uint64_t sa[1] = {(uint64_t)g.lda * 2};
    const uint32_t ba[2] = {64, 128u};
    // with the gather fused, A is read by the gather warps: no map of it is needed
    if (!gather) ok = ok && make_map(&tmA, g.A, 2, da, sa, ba);
    if (MODE == kFwd && b_wide) {
      const uint64_t db[4] = {64, (uint64_t)g.K, (uint64_t)g.N / 64, (uint64_t)g.E};
      const uint64_t sb[3] = {(uint64_t)g.ldb * 2, 128, (uint64_t)g.b_expert_stride * 2};
      const uint32_t bb[4] = {64, 64, BN / 64, 1};
      ok = ok && make_map(&tmB, g.B, 4, db, sb, bb);
    } else if (MODE == kFwd) {
      const uint64_t db[3] = {(uint64_t)g.N, (uint64_t)g.K, (uint64_t)g.E};
      const uint64_t sb[2] = {(uint64_t)g.ldb * 2, (uint64_t)g.b_expert_stride * 2};
      const uint32_t bb[3] = {64, 64, 1};
      ok = ok && make_map(&tmB, g.B, 3, db, sb, bb);
    } else {
      const uint64_t db[3] = {(uint64_t)g.K, (uint64_t)g.N, (uint64_t)g.E};
      const uint64_t sb[2] = {(uint64_t)g.ldb * 2, (uint64_t)g.b_expert_stride * 2};
      const uint32_t bb[3] = {64, (uint32_t)BN, 1};
      ok = ok && make_map(&tmB, g.B, 3, db, sb, bb);
    }
  }
  if (!ok) return YAMOE_ERR_CUDA;
  if (gather) tmA = tmB;              // placeholder for the unused kernel parameter
  if constexpr (MODE == kFwd && epi_gathers<Epi>::value) {
    if (gather) return launch_umma_kernel<MODE, BN, Epi, true>(g, epi, tmA, tmB, max_tiles, a_wide, b_wide, stream);
  } else {
    if (gather) return YAMOE_ERR_UNSUPPORTED;     // no gathering instantiation for this epilogue
  }
  return launch_umma_kernel<MODE, BN, Epi, false>(g, epi, tmA, tmB, max_tiles, a_wide, b_wide, stream);
}

template <int MODE, int BN, class Epi, bool GATHER>
inline int launch_umma_kernel(const GemmArgs& g, const Epi& epi, const CUtensorMap& tmA, const CUtensorMap& tmB,
                              int64_t max_tiles, bool a_wide, bool b_wide, cudaStream_t stream) {
  using SM = UmmaSmem<BN>;
  constexpr bool gather = GATHER;
  auto kern = umma_gemm_kernel<MODE, BN, Epi, GATHER>;
  static PerDevice<int> attr_done;   // per template instantiation and device
  const int dev = current_device_index();
  if (!attr_done.get(dev)) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::kTotal) != cudaSuccess)
      return YAMOE_ERR_CUDA;
    attr_done.set(dev, 1);
  }
  UmmaParams p{g.M, g.N, g.K, g.E, g.tile_expert, g.pad_off, (int)max_tiles, const_cast<int32_t*>(g.header),
               gather ? g.gather_rows : nullptr, g.A, g.lda, g.gate, a_wide ? 1 : 0, b_wide ? 1 : 0};
  const int NT = (int)ceil_div(g.N, BN);
  int64_t total_max = MODE == kWgrad ? (int64_t)g.E * ceil_div(g.M, kUmmaBM) * NT : max_tiles * NT;
  int grid = (int)std::min<int64_t>(total_max, umma_sm_count());
  if (grid <= 0) return YAMOE_OK;
  // a gated GEMM is meant to start while its predecessor on the stream still runs
  const int threads = kUmmaThreads + (gather ? kUmmaGatherThreads : 0);
  if (launch_pdl_opt(g.gate.prep != nullptr, kern, dim3(grid), dim3(threads), SM::kTotal, stream, tmA, tmB, p, epi) !=
      cudaSuccess)
    return YAMOE_ERR_CUDA;
  return cudaGetLastError() == cudaSuccess ? YAMOE_OK : YAMOE_ERR_CUDA;
}

template <int MODE, class Epi>
inline int launch_umma_gemm(const GemmArgs& g, const Epi& epi, int64_t max_rows, int64_t max_tiles,
                            cudaStream_t stream) {
  switch (umma_tile_n()) {
    case 128: return launch_umma_gemm_bn<MODE, 128>(g, epi, max_rows, max_tiles, stream);
    case 192: return launch_umma_gemm_bn<MODE, 192>(g, epi, max_rows, max_tiles, stream);
    default: return launch_umma_gemm_bn<MODE, 256>(g, epi, max_rows, max_tiles, stream);
  }
}

}  // namespace yb
