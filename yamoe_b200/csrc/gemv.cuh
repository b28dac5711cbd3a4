// Decode path: weight-streaming GEMV kernels for token counts so small (T*K <= 256) that the
// expert forward is bound by reading the weights of the experts that are hit, once, from HBM.
// The reference has no such path: it runs the same padded bmm over all E experts
// (csrc/moe.cpp:161,184), reading every expert's weights whether it is used or not.
//
// Exactly two launches, no routing launch, no memset and no cast launch:
//   gemv_kernel<kGateUp>  act[p, j]  = glu(x_t . W_gu[e][:, 2j] + b, x_t . W_gu[e][:, 2j+1] + b);
//                         also zeroes the fp32 combine buffer and the slab counters for stage two
//   gemv_kernel<kDown>    out32[t,:] += w_p * (act[p,:] . W_d[e] + b_d[e]); the last CTA to finish a
//                         column slab (ticket counter, no waiting) rounds that slab to bf16 output;
//                         with few experts hit, 2 or 4 CTAs (gridDim.z) split the reduction
//                         dimension of a slab and meet in the same fp32 buffer
// p = t*K + slot is the flat assignment index.  Grid = (touched-expert slot, column slab).  Every
// CTA rebuilds the (<= 256 entry) routing in shared memory: histogram, ascending list of touched
// experts, and the stable row list of its own expert, honouring the capacity
// (csrc/gather.cu:18-26).  Each thread streams 16-byte (8 x bf16) pieces of weight rows, 8 loads
// in flight, the 8 warps split the reduction dimension, partial sums meet in shared memory.
#pragma once
#include <cstdlib>

#include "common.cuh"
#include "epilogues.cuh"
#include "misc_kernels.cuh"

namespace yb {

constexpr int kGemvThreads = 256;
constexpr int kGemvMaxS = 256;     // assignments the in-CTA routing handles
constexpr int kGemvMT = 4;         // rows of one expert processed per weight pass
enum GemvStage { kGateUp = 0, kDown = 1 };

struct GemvArgs {
  const __nv_bfloat16* x;          // kGateUp: hidden [T,H]; kDown: act [S,H]
  const int64_t* router_indices;   // [T,K]
  const __nv_bfloat16* routing_weights;
  int routing_cols;
  const __nv_bfloat16* W;          // [E, Kdim, N]
  const __nv_bfloat16* bias;       // [E, N]
  __nv_bfloat16* act;              // kGateUp output [S, N/2]
  float* out32;                    // fp32 combine buffer [T, H]: zeroed by kGateUp, reduced into by kDown
  __nv_bfloat16* out;              // kDown: final output [T, N]
  int32_t* slab_done;              // [ceil(H/64)] per-slab completion counters: zeroed by kGateUp
  int S, E, K, Kdim, N, T, H;
  int64_t capacity;
};

__device__ __forceinline__ void unpack8(const uint4& q, float (&w)[8]) {
  const uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    w[2 * j] = __uint_as_float(u[j] << 16);
    w[2 * j + 1] = __uint_as_float(u[j] & 0xffff0000u);
  }
}

// Streams the CTA's weight slab once for MT rows held in shared memory.
template <int NB, int MT>
__device__ __forceinline__ void gemv_accumulate(const __nv_bfloat16* __restrict__ wp, int N, int Kdim,
                                                const __nv_bfloat16* __restrict__ xs, bool col_ok,
                                                float (&acc)[kGemvMT][8]) {
  constexpr int LPR = NB / 8;            // lanes per weight row
  constexpr int RPW = 32 / LPR;          // weight rows per warp load
  constexpr int RPI = 8 * RPW;           // weight rows per CTA iteration
  constexpr int UN = 8;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int rp = lane / LPR;
  int k = w * RPW + rp;
  for (; k + (UN - 1) * RPI < Kdim; k += UN * RPI) {
    uint4 q[UN];
#pragma unroll
    for (int u = 0; u < UN; ++u)
      q[u] = col_ok ? __ldcs(reinterpret_cast<const uint4*>(wp + (size_t)(k + u * RPI) * N)) : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      float wv[8];
      unpack8(q[u], wv);
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const float xv = __bfloat162float(xs[m * Kdim + k + u * RPI]);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[m][j] = fmaf(xv, wv[j], acc[m][j]);
      }
    }
  }
  for (; k < Kdim; k += RPI) {
    const uint4 q = col_ok ? __ldcs(reinterpret_cast<const uint4*>(wp + (size_t)k * N)) : make_uint4(0, 0, 0, 0);
    float wv[8];
    unpack8(q, wv);
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      const float xv = __bfloat162float(xs[m * Kdim + k]);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[m][j] = fmaf(xv, wv[j], acc[m][j]);
    }
  }
}

template <int STAGE, int NB>
__global__ void __launch_bounds__(kGemvThreads, 3)
gemv_kernel(const GemvArgs g) {
  constexpr int LPR = NB / 8, RPW = 32 / LPR, NPART = 8 * RPW;
  extern __shared__ __align__(16) uint8_t gemv_smem[];
  // layout: xs [MT][Kdim] bf16 | red [NPART][MT][NB] f32 | cnt [E] i32 | s_e [256] i32 | rows [256] i32
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(gemv_smem);
  float* red = reinterpret_cast<float*>(gemv_smem + (((size_t)kGemvMT * g.Kdim * 2 + 15) & ~size_t(15)));
  int32_t* cnt = reinterpret_cast<int32_t*>(red + NPART * kGemvMT * NB);
  int32_t* s_e = cnt + g.E;
  int32_t* rows = s_e + kGemvMaxS;
  __shared__ int s_warp[8];
  __shared__ int s_my_e, s_touched;

  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  if constexpr (STAGE == kGateUp) pdl_trigger();   // stage two may set up its routing while this kernel streams
  if constexpr (STAGE == kGateUp) {
    // every CTA of the grid (also those that find no expert below) clears a share of the buffers
    // the second launch accumulates into; that launch starts only after this one has finished
    const size_t nthreads = (size_t)gridDim.x * gridDim.y * kGemvThreads;
    const size_t gtid = ((size_t)blockIdx.y * gridDim.x + blockIdx.x) * kGemvThreads + tid;
    const size_t nvec = (size_t)g.T * g.H / 4;
    for (size_t i = gtid; i < nvec; i += nthreads) reinterpret_cast<float4*>(g.out32)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    const int nslab = (g.H + 63) / 64;
    if (gtid < (size_t)nslab) g.slab_done[gtid] = 0;
  }
  // ---- routing, rebuilt per CTA ---------------------------------------------------------------
  int e;
  if (g.S <= 32) {
    // At most one assignment per lane: warp 0 sorts with ballots, no shared-memory histogram and
    // a single barrier.  (At T = 1 the set-up of a CTA is a visible share of its 10 us of streaming.)
    if (w == 0) {
      int my = -1;
      if (lane < g.S) {
        const int64_t v = g.router_indices[lane];
        if (v >= 0 && v < g.E) my = (int)v;
      }
      const unsigned valid = __ballot_sync(0xffffffffu, my >= 0);
      const unsigned same = __match_any_sync(0xffffffffu, my);
      const bool first = my >= 0 && (__ffs(same) - 1) == lane;     // first assignment of its expert
      // rank of my expert among the touched ones, ascending
      int rank = 0;
      for (int o = 0; o < 32; ++o) {
        const int oe = __shfl_sync(0xffffffffu, my, o);
        const int of = __shfl_sync(0xffffffffu, (int)first, o);
        if (of && oe < my) ++rank;
      }
      const unsigned firsts = __ballot_sync(0xffffffffu, first);
      const unsigned pick = __ballot_sync(0xffffffffu, first && rank == (int)blockIdx.x);
      int mine_e = -1;
      if (pick) mine_e = __shfl_sync(0xffffffffu, my, __ffs(pick) - 1);
      const unsigned members = __ballot_sync(0xffffffffu, my >= 0 && my == mine_e) & valid;
      if (my >= 0 && my == mine_e) rows[__popc(members & ((1u << lane) - 1u))] = lane;   // stable: ascending p
      if (lane == 0) {
        s_my_e = mine_e;
        s_touched = __popc(firsts);
        s_warp[0] = __popc(members);
      }
    }
    __syncthreads();
    e = s_my_e;
    if (e < 0) return;                    // fewer touched experts than grid slots
  } else {
  for (int ee = tid; ee < g.E; ee += kGemvThreads) cnt[ee] = 0;
  if (tid == 0) { s_my_e = -1; s_touched = 0; }
  __syncthreads();
  int my = -1;
  if (tid < g.S) {
    const int64_t v = g.router_indices[tid];
    if (v >= 0 && v < g.E) { my = (int)v; atomicAdd(&cnt[my], 1); }
  }
  s_e[tid] = my;
  __syncthreads();
  {
    // rank of every touched expert in ascending order; the CTA serves the blockIdx.x-th one
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
        if (rank == (int)blockIdx.x) s_my_e = e0 + i;
        ++rank;
      }
    }
    if (tid == kGemvThreads - 1) s_touched = rank;   // last thread ends on the total
    __syncthreads();
  }
  e = s_my_e;
  if (e < 0) return;                      // fewer touched experts than grid slots
  {
    // stable list of this expert's assignments
    const bool mine = (my == e);
    const unsigned bal = __ballot_sync(0xffffffffu, mine);
    if (lane == 0) s_warp[w] = __popc(bal);
    __syncthreads();
    int base = 0;
    for (int i = 0; i < w; ++i) base += s_warp[i];
    if (mine) rows[base + __popc(bal & ((1u << lane) - 1u))] = tid;
    __syncthreads();
  }
  }
  const int n_all = g.S <= 32 ? s_warp[0] : cnt[e];
  const int n_rows = (int64_t)n_all < g.capacity ? n_all : (int)g.capacity;
  const int n0 = blockIdx.y * NB;
  const int cg = lane % LPR;
  const int n = n0 + cg * 8;
  const bool col_ok = n < g.N;
  // reduction range of this CTA: gridDim.z CTAs share one (expert, column slab) and meet in out32
  int k0 = 0, klen = g.Kdim;
  if (STAGE == kDown && gridDim.z > 1) {          // 32-bit arithmetic, down stage only
    const unsigned parts = gridDim.z;
    const unsigned kchunk = (((unsigned)g.Kdim + parts - 1u) / parts + 63u) & ~63u;
    k0 = (int)min(blockIdx.z * kchunk, (unsigned)g.Kdim);
    klen = min((int)kchunk, g.Kdim - k0);
  }
  const __nv_bfloat16* wp = g.W + ((size_t)e * g.Kdim + k0) * g.N + n;
  // everything above read only the caller's inputs; below come act / out32 / slab counters
  if constexpr (STAGE == kDown) pdl_wait();
  const int part = w * RPW + lane / LPR;

  for (int r0 = 0; r0 < n_rows; r0 += kGemvMT) {
    const int mt = min(kGemvMT, n_rows - r0);
    // stage the input rows (bf16) in shared memory
    const int vec_per_row = klen / 8;
    for (int i = tid; i < mt * vec_per_row; i += kGemvThreads) {
      const int m = i / vec_per_row, c = i - m * vec_per_row;
      const int p = rows[r0 + m];
      const size_t src_row = (STAGE == kGateUp) ? (size_t)(p / g.K) : (size_t)p;
      reinterpret_cast<uint4*>(xs + (size_t)m * klen)[c] =
          __ldg(reinterpret_cast<const uint4*>(g.x + src_row * g.Kdim + k0) + c);
    }
    __syncthreads();
    float acc[kGemvMT][8];
#pragma unroll
    for (int m = 0; m < kGemvMT; ++m)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[m][j] = 0.f;
    if (mt == 1) gemv_accumulate<NB, 1>(wp, g.N, klen, xs, col_ok, acc);
    else if (mt == 2) gemv_accumulate<NB, 2>(wp, g.N, klen, xs, col_ok, acc);
    else if (mt == 3) gemv_accumulate<NB, 3>(wp, g.N, klen, xs, col_ok, acc);
    else gemv_accumulate<NB, 4>(wp, g.N, klen, xs, col_ok, acc);
    // partial sums -> shared memory: red[part][m][col]
    for (int m = 0; m < mt; ++m) {
      float* dst = red + ((size_t)part * kGemvMT + m) * NB + cg * 8;
      *reinterpret_cast<float4*>(dst) = make_float4(acc[m][0], acc[m][1], acc[m][2], acc[m][3]);
      *reinterpret_cast<float4*>(dst + 4) = make_float4(acc[m][4], acc[m][5], acc[m][6], acc[m][7]);
    }
    __syncthreads();
    if constexpr (STAGE == kGateUp) {
      // thread -> (row m, column pair j): NB/2 pairs per row
      for (int i = tid; i < mt * (NB / 2); i += kGemvThreads) {
        const int m = i / (NB / 2), j = i - m * (NB / 2);
        const int col = n0 + 2 * j;
        if (col >= g.N) continue;
        float sg = 0.f, su = 0.f;
#pragma unroll 4
        for (int pp = 0; pp < NPART; ++pp) {
          const float2 v = *reinterpret_cast<const float2*>(red + ((size_t)pp * kGemvMT + m) * NB + 2 * j);
          sg += v.x; su += v.y;
        }
        sg += __bfloat162float(g.bias[(size_t)e * g.N + col]);
        su += __bfloat162float(g.bias[(size_t)e * g.N + col + 1]);
        const int p = rows[r0 + m];
        g.act[(size_t)p * (g.N / 2) + col / 2] = __float2bfloat16_rn(glu_act(sg, su));
      }
    } else {
      for (int i = tid; i < mt * NB; i += kGemvThreads) {
        const int m = i / NB, j = i - m * NB;
        const int col = n0 + j;
        if (col >= g.N) continue;
        float s = 0.f;
#pragma unroll 4
        for (int pp = 0; pp < NPART; ++pp) s += red[((size_t)pp * kGemvMT + m) * NB + j];
        if (blockIdx.z == 0) s += __bfloat162float(g.bias[(size_t)e * g.N + col]);
        const int p = rows[r0 + m];
        const int t = p / g.K;
        const int wc = (g.routing_cols == g.E) ? e : (p - t * g.K);
        const float wgt = __bfloat162float(g.routing_weights[(size_t)t * g.routing_cols + wc]);
        atomicAdd(g.out32 + (size_t)t * g.N + col, wgt * s);
      }
    }
    __syncthreads();
  }
  if constexpr (STAGE == kDown) {
    // Column slab finished by this CTA; whoever completes the slab last converts it.
    __shared__ int s_last;
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = (atomicAdd(g.slab_done + blockIdx.y, 1) == s_touched * (int)gridDim.z - 1);
    __syncthreads();
    if (s_last) {
      __threadfence();
      const int width = min(NB, g.N - n0);
      for (int i = tid; i < g.T * (width / 2); i += kGemvThreads) {
        const int t = i / (width / 2), j = (i - t * (width / 2)) * 2;
        const float2 v = __ldcg(reinterpret_cast<const float2*>(g.out32 + (size_t)t * g.N + n0 + j));
        *reinterpret_cast<uint32_t*>(g.out + (size_t)t * g.N + n0 + j) = pack_bf16x2(v.x, v.y);
      }
    }
  }
}

// Column-slab width of the gate_up stage: narrow slabs when few experts are hit, so that the grid
// still covers every SM at least twice.  YAMOE_B200_GEMV_NB overrides (64 or 128).
inline int gemv_gate_up_slab(int64_t S, int E, int N) {
  static int forced = []() {
    const char* env = std::getenv("YAMOE_B200_GEMV_NB");
    const int v = env ? std::atoi(env) : 0;
    return (v == 64 || v == 128) ? v : 0;
  }();
  if (forced) return forced;
  const int64_t slots = E < S ? E : S;
  return slots * ceil_div(N, 128) < 4 * 148 ? 64 : 128;
}

// Number of CTAs that share the reduction dimension of one (expert, column slab) in the down
// stage.  With few experts hit, one CTA per slab leaves the grid (slots x 45 slabs) too coarse to
// balance over 148 SMs: 180 CTAs at T = 1 put two slabs on some SMs and one on others.
// YAMOE_B200_GEMV_KS overrides (1, 2 or 4).
inline int gemv_down_ksplit(int64_t S, int E, int N) {
  static int forced = []() {
    const char* env = std::getenv("YAMOE_B200_GEMV_KS");
    const int v = env ? std::atoi(env) : 0;
    return (v == 1 || v == 2 || v == 4) ? v : 0;
  }();
  if (forced) return forced;
  const int64_t ctas = (E < S ? E : S) * ceil_div(N, 64);
  return ctas <= 2 * 148 ? 2 : 1;     // measured: 53.6 / 55.0 / 55.6 us with 2 / 1 / 4 parts at T = 1; no gain beyond
}

inline bool gemv_preferred(int64_t T, int E, int K) {
  const int64_t S = T * K;
  return S <= kGemvMaxS && S <= 4 * (int64_t)E;   // at most ~4 rows per expert on average
}

template <int STAGE, int NB>
inline int launch_gemv_stage(const GemvArgs& g, cudaStream_t st, int ksplit = 1) {
  constexpr int NPART = 8 * (32 / (NB / 8));
  size_t smem = (((size_t)kGemvMT * g.Kdim * 2 + 15) & ~size_t(15)) + (size_t)NPART * kGemvMT * NB * 4 +
                (size_t)g.E * 4 + 2 * kGemvMaxS * 4;
  auto kern = gemv_kernel<STAGE, NB>;
  static PerDevice<size_t> configured;   // per template instantiation and device
  const int dev = current_device_index();
  if (smem > configured.get(dev)) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return YAMOE_ERR_UNSUPPORTED;
    configured.set(dev, smem);
  }
  const int slots = g.E < g.S ? g.E : g.S;
  dim3 grid((unsigned)slots, (unsigned)ceil_div(g.N, NB), (unsigned)(STAGE == kDown ? ksplit : 1));
  if (STAGE == kDown) {
    if (launch_pdl_opt(true, kern, grid, dim3(kGemvThreads), smem, st, g) != cudaSuccess) return YAMOE_ERR_CUDA;
  } else {
    kern<<<grid, kGemvThreads, smem, st>>>(g);
  }
  return cudaGetLastError() == cudaSuccess ? YAMOE_OK : YAMOE_ERR_CUDA;
}

// bf16 only.  `act` must hold S*H elements, `acc32` T*H floats, `slab_done` ceil(H/64) ints;
// none of them needs initialising.
inline int launch_gemv_forward(const void* hidden, const int64_t* ridx, const void* rw, int rcols, const void* wgu,
                               const void* bgu, const void* wd, const void* bd, void* out, int64_t T, int H, int E,
                               int K, int64_t cap, void* act, float* acc32, int32_t* slab_done, cudaStream_t st) {
  const int64_t S = T * K;
  if (S > kGemvMaxS || H % 8 != 0 || E > 1024) return YAMOE_ERR_UNSUPPORTED;
  using bf = __nv_bfloat16;
  GemvArgs g1{reinterpret_cast<const bf*>(hidden), ridx, reinterpret_cast<const bf*>(rw), rcols,
              reinterpret_cast<const bf*>(wgu), reinterpret_cast<const bf*>(bgu), reinterpret_cast<bf*>(act),
              acc32, nullptr, slab_done, (int)S, E, K, H, 2 * H, (int)T, H, cap};
  GemvArgs g2{reinterpret_cast<const bf*>(act), ridx, reinterpret_cast<const bf*>(rw), rcols,
              reinterpret_cast<const bf*>(wd), reinterpret_cast<const bf*>(bd), nullptr, acc32,
              reinterpret_cast<bf*>(out), slab_done, (int)S, E, K, H, H, (int)T, H, cap};
  int rc;
  {
    StageTimer tm(kStageGateUp, st);
    rc = gemv_gate_up_slab(S, E, 2 * H) == 64 ? launch_gemv_stage<kGateUp, 64>(g1, st)
                                              : launch_gemv_stage<kGateUp, 128>(g1, st);
  }
  if (rc) return rc;
  {
    StageTimer tm(kStageDown, st);
    static const int down_nb = []() {
      const char* env = std::getenv("YAMOE_B200_GEMV_DOWN_NB");
      return env ? std::atoi(env) : 0;
    }();
    // 128-column slabs pay only when they still give every SM about eight CTAs (T = 64: 1006 us
    // against 1018 us; T = 16: 465 us against 457 us)
    const bool wide = down_nb ? down_nb == 128 : (E < S ? E : S) * ceil_div(H, 128) >= 8 * 148;
    rc = wide ? launch_gemv_stage<kDown, 128>(g2, st, 1)
              : launch_gemv_stage<kDown, 64>(g2, st, gemv_down_ksplit(S, E, H));
  }
  return rc;
}

}  // namespace yb
