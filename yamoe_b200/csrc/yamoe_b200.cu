// C ABI of the yamoe_b200 library: argument checks, workspace carving and the sequencing of
// the routing, gather, grouped-GEMM and reduction kernels for the expert forward and backward
// passes.  Takes the place of the reference's orchestration in csrc/moe.cpp:45-223 and
// csrc/experts_backward.cu:126-341; none of that code allocates here — all scratch lives in
// the caller's workspace — and nothing synchronises with the host.
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include <type_traits>

#include "common.cuh"
#include "epilogues.cuh"
#include "misc_kernels.cuh"
#include "routing.cuh"
#include "simt_gemm.cuh"
#include "umma_gemm.cuh"
#include "umma_gemm_2cta.cuh"
#include "gemv.cuh"
#include "ep_fused.cuh"
#include "router.cuh"

namespace yb {

static std::atomic<int> g_path{-1};

static int current_path() {
  int p = g_path.load();
  if (p >= 0) return p;
  const char* env = std::getenv("YAMOE_B200_PATH");
  p = YAMOE_PATH_AUTO;
  if (env != nullptr) {
    if (!std::strcmp(env, "simt")) p = YAMOE_PATH_SIMT;
    else if (!std::strcmp(env, "tcgen05")) p = YAMOE_PATH_TCGEN05;
    else if (!std::strcmp(env, "gemv")) p = YAMOE_PATH_GEMV;
  }
  g_path.store(p);
  return p;
}

// Bump allocator over the caller's workspace; with base == nullptr it only measures.
struct Bump {
  char* base;
  size_t off = 0;
  explicit Bump(void* b) : base(reinterpret_cast<char*>(b)) {}
  template <typename U>
  U* take(size_t n) {
    off = (off + 255) & ~size_t(255);
    U* p = base ? reinterpret_cast<U*>(base + off) : nullptr;
    off += n * sizeof(U);
    return p;
  }
};

struct Plan {
  RouteTables rt;
  int64_t S, max_rows, max_tiles;
  size_t esize;
  // forward
  void* xs = nullptr;      // [max_rows, H]   gathered hidden rows
  void* act = nullptr;     // [max_rows, H]   GLU output
  void* yrows = nullptr;   // [max_rows, H]   weighted down-projection rows (bf16 two-step combine)
  float* acc32 = nullptr;  // [T, H]          fp32 combine target when the output is bf16
  int32_t* slab_done = nullptr;  // [ceil(H/64)] completion counters of the decode path
  // backward
  void* gys = nullptr;     // [max_rows, H]   gathered grad_y rows
  void* pre = nullptr;     // [max_rows, 2H]  biased pre-activations
  void* actw = nullptr;    // [max_rows, H]   routing weight * activation
  void* gpre = nullptr;    // [max_rows, 2H]  gradient of the pre-activations
  float* gw_row = nullptr; // [max_rows]
  size_t bytes = 0;
  size_t row_tables_bytes = 0;
};

static void carve_tables(Bump& b, Plan& p, int64_t T, int E, int K, bool rows) {
  p.S = T * K;
  p.max_tiles = max_row_tiles(p.S, E);
  p.max_rows = p.max_tiles * kTileM;
  p.rt.header = b.take<int32_t>(16);
  p.rt.counts = b.take<int32_t>(E);
  p.rt.bins = b.take<int32_t>(E + 1);
  p.rt.pad_off = b.take<int32_t>(E + 1);
  p.rt.block_counts = b.take<int32_t>((size_t)route_blocks(p.S) * E);
  p.rt.tile_expert = b.take<int32_t>(p.max_tiles);
  p.rt.pair_off = b.take<int32_t>(E + 1);
  p.rt.pair_expert = b.take<int32_t>(p.max_tiles);
  p.rt.sorted_values = b.take<int32_t>(p.S);
  p.rt.sorted_indices = b.take<int32_t>(p.S);
  if (rows) {
    // row_token, row_flat and flat_row are adjacent so that one memset marks every row as padding
    // and every assignment as dropped
    p.rt.row_token = b.take<int32_t>(2 * (size_t)p.max_rows + (size_t)p.S);
    p.rt.row_flat = p.rt.row_token ? p.rt.row_token + p.max_rows : nullptr;
    p.rt.flat_row = p.rt.row_token ? p.rt.row_token + 2 * p.max_rows : nullptr;
    p.row_tables_bytes = (2 * (size_t)p.max_rows + (size_t)p.S) * sizeof(int32_t);
    p.rt.row_weight = b.take<float>(p.max_rows);
  } else {
    p.rt.row_token = p.rt.row_flat = p.rt.flat_row = nullptr;
    p.rt.row_weight = nullptr;
  }
}

static Plan plan_forward(void* ws, int64_t T, int H, int E, int K, int dtype) {
  Plan p;
  Bump b(ws);
  p.esize = dtype == YAMOE_BF16 ? 2 : 4;
  carve_tables(b, p, T, E, K, true);
  p.xs = b.take<char>((size_t)p.max_rows * H * p.esize);
  p.act = b.take<char>((size_t)p.max_rows * H * p.esize);
  if (dtype == YAMOE_BF16) {
    // decode path: fp32 accumulator [T,H]; grouped-GEMM path: weighted rows [max_rows,H].
    // They are never live together, the larger one sizes the region.
    const size_t a = (size_t)T * H * sizeof(float), y = (size_t)p.max_rows * H * p.esize;
    char* region = b.take<char>(a > y ? a : y);
    p.acc32 = reinterpret_cast<float*>(region);
    p.yrows = region;
  }
  p.slab_done = b.take<int32_t>((size_t)ceil_div(H, 64));
  p.bytes = b.off + 256;
  return p;
}

// Extra columns behind the H real ones in the backward layout of xs and actw: the first carries
// 1 (xs) or the routing weight (actw) so that the weight-gradient GEMMs also produce the bias
// gradients.  64 of them keep every bf16 row a multiple of 128 bytes long: rows that straddle
// 128-byte lines cost the TMA loads of the GEMMs that read these buffers extra L2 sectors
// (measured: + 0.2 ms on the T = 8192 backward with 8 columns).
constexpr int kBiasCols = 64;

static Plan plan_backward(void* ws, int64_t T, int H, int E, int K, int dtype) {
  Plan p;
  Bump b(ws);
  p.esize = dtype == YAMOE_BF16 ? 2 : 4;
  carve_tables(b, p, T, E, K, true);
  p.xs = b.take<char>((size_t)p.max_rows * (H + kBiasCols) * p.esize);
  p.gys = b.take<char>((size_t)p.max_rows * H * p.esize);
  p.pre = b.take<char>((size_t)p.max_rows * 2 * H * p.esize);
  p.actw = b.take<char>((size_t)p.max_rows * (H + kBiasCols) * p.esize);
  p.gpre = b.take<char>((size_t)p.max_rows * 2 * H * p.esize);
  p.gw_row = b.take<float>(p.max_rows);
  if (dtype == YAMOE_BF16) p.acc32 = b.take<float>((size_t)T * H);
  p.bytes = b.off + 256;
  return p;
}

static int check_common(int64_t T, int H, int E, int K, int dtype) {
  if (dtype != YAMOE_F32 && dtype != YAMOE_BF16) return YAMOE_ERR_DTYPE;
  if (T < 0 || H <= 0 || E <= 0 || K <= 0) return YAMOE_ERR_BAD_ARG;
  if (H % 8 != 0) return YAMOE_ERR_BAD_ARG;
  if (E > 1024) return YAMOE_ERR_UNSUPPORTED;
  if (T * K >= (int64_t)1 << 30) return YAMOE_ERR_UNSUPPORTED;
  return YAMOE_OK;
}

static int prepare_routing(const Plan& p, cudaStream_t st) {
  YB_CUDA_OK(cudaMemsetAsync(p.rt.header, 0, 16 * sizeof(int32_t), st));
  if (p.rt.row_token) YB_CUDA_OK(cudaMemsetAsync(p.rt.row_token, 0xFF, p.row_tables_bytes, st));
  return YAMOE_OK;
}

// YAMOE_B200_FUSED_GATHER=1 lets the gate_up GEMM of the forward fetch its A rows straight from
// hidden_states (four extra warps per CTA copy them into the swizzled A stage with cp.async), so
// that the permuted activations are never written to global memory.  Off by default: the GEMM fed
// that way measures 518 us against 457 us for the TMA-fed one, more than the 27 us gather kernel
// it saves (0.841 against 0.814 ms per forward at T = 4096).
static bool fused_gather_enabled() {
  static int on = []() {
    const char* env = std::getenv("YAMOE_B200_FUSED_GATHER");
    return env ? std::atoi(env) : 0;
  }();
  return on != 0;
}

static bool use_tcgen05(int path, int dtype, int H) {
  if (dtype != YAMOE_BF16 || !umma_available()) return false;
  if (H % 64 != 0) return false;
  return path == YAMOE_PATH_AUTO || path == YAMOE_PATH_TCGEN05;
}

template <typename T>
static int forward_impl(const void* hidden, const int64_t* ridx, const void* rw, int rcols, const void* wgu,
                        const void* bgu, const void* wd, const void* bd, void* out, int64_t Tn, int H, int E,
                        int K, int64_t cap, int dtype, void* ws, cudaStream_t st) {
  Plan p = plan_forward(ws, Tn, H, E, K, dtype);
  const int path = current_path();
  float* acc = p.acc32 ? p.acc32 : reinterpret_cast<float*>(out);
  if (Tn == 0) return YAMOE_OK;

  if (dtype == YAMOE_BF16 && (path == YAMOE_PATH_GEMV || (path == YAMOE_PATH_AUTO && gemv_preferred(Tn, E, K)))) {
    int rc = launch_gemv_forward(hidden, ridx, rw, rcols, wgu, bgu, wd, bd, out, Tn, H, E, K, cap, p.act, acc,
                                 p.slab_done, st);
    if (rc != YAMOE_ERR_UNSUPPORTED) return rc;
  }
  const bool tc = use_tcgen05(path, dtype, H);
  if (!tc) YB_CUDA_OK(cudaMemsetAsync(acc, 0, (size_t)Tn * H * sizeof(float), st));

  int rc = prepare_routing(p, st);
  if (rc) return rc;
  {
    StageTimer tm(kStageRoute, st);
    rc = launch_route<T>(ridx, reinterpret_cast<const T*>(rw), rcols, Tn, E, K, cap, p.rt, st);
  }
  if (rc) return rc;
  // With the gather fused the gate_up GEMM reads its A rows from hidden_states itself; otherwise
  // gather_rows_kernel materialises the permuted copy first.
  const bool fused_gather = tc && fused_gather_enabled() && !umma_2cta_enabled();
  const unsigned row_blocks = (unsigned)ceil_div(p.max_rows, kRowWarps);
  if (!fused_gather) {
    StageTimer tm(kStageGather, st);
    if (launch_pdl(gather_rows_kernel<T>, dim3(row_blocks), dim3(kRowWarps * 32), 0, st,
                   reinterpret_cast<const T*>(hidden), reinterpret_cast<T*>(p.xs),
                   (const int32_t*)p.rt.row_token, (const int32_t*)p.rt.header, H, H) != cudaSuccess)
      return YAMOE_ERR_CUDA;
  }
  EpiGluAct<T> glu{reinterpret_cast<const T*>(bgu), reinterpret_cast<T*>(p.act), p.rt.row_token, H};
  EpiScatterAdd<T, true, true> comb{reinterpret_cast<const T*>(bd), acc, p.rt.row_token, p.rt.row_weight, H};
  GemmArgs g1{p.xs, H, wgu, 2 * (int64_t)H, (int64_t)H * 2 * H, 0, 2 * H, H, E,
              p.rt.tile_expert, p.rt.pad_off, p.rt.header};
  g1.pair_expert = p.rt.pair_expert; g1.pair_off = p.rt.pair_off; g1.counts = p.rt.counts;
  GemmArgs g2{p.act, H, wd, H, (int64_t)H * H, 0, H, H, E, p.rt.tile_expert, p.rt.pad_off, p.rt.header};
  g2.pair_expert = p.rt.pair_expert; g2.pair_off = p.rt.pair_off; g2.counts = p.rt.counts;
  if (fused_gather) {
    g1.A = hidden;
    g1.gather_rows = p.rt.row_token;
    g1.gather_src_rows = Tn;
  }
  if (tc) {
    if constexpr (sizeof(T) == 2) {
      {
        StageTimer tm(kStageGateUp, st);
        rc = launch_umma<kFwd>(g1, glu, p.max_rows, p.max_tiles, st);
      }
      if (rc) return rc;
      // two-step combine: weighted rows out of the GEMM epilogue, then one gather-sum pass
      EpiWeightedRows<T> wrows{reinterpret_cast<const T*>(bd), reinterpret_cast<T*>(p.yrows), p.rt.row_token,
                               p.rt.row_weight, H};
      {
        StageTimer tm(kStageDown, st);
        rc = launch_umma<kFwd>(g2, wrows, p.max_rows, p.max_tiles, st);
      }
      if (rc) return rc;
      StageTimer tm(kStageCombine, st);
      if (launch_pdl(combine_padded_kernel<T>, dim3((unsigned)ceil_div(Tn, kRowWarps)), dim3(kRowWarps * 32), 0, st,
                     reinterpret_cast<const T*>(p.yrows), (const int32_t*)p.rt.flat_row, reinterpret_cast<T*>(out),
                     Tn, H, K) != cudaSuccess)
        return YAMOE_ERR_CUDA;
      return cudaGetLastError() == cudaSuccess ? YAMOE_OK : YAMOE_ERR_CUDA;
    }
  } else {
    {
      StageTimer tm(kStageGateUp, st);
      launch_simt_gemm<T, kFwd>(g1, glu, p.max_rows, st);
    }
    {
      StageTimer tm(kStageDown, st);
      launch_simt_gemm<T, kFwd>(g2, comb, p.max_rows, st);
    }
  }
  if (p.acc32) {
    const int64_t nv = Tn * H / 4;
    cast_kernel<T><<<(unsigned)std::min<int64_t>(ceil_div(nv, 256), 148 * 8), 256, 0, st>>>(
        p.acc32, reinterpret_cast<T*>(out), nv);
  }
  return cudaGetLastError() == cudaSuccess ? YAMOE_OK : YAMOE_ERR_CUDA;
}

// Forward pass that leaves what the backward pass needs in a workspace with the BACKWARD layout:
// routing tables, xs, pre (biased pre-activations) and actw (weight * activation).  The
// activation itself and the weighted output rows only live until the call returns; they borrow
// the regions the backward pass later uses for gpre and gys.
template <typename T>
static int forward_train_impl(const void* hidden, const int64_t* ridx, const void* rw, int rcols, const void* wgu,
                              const void* bgu, const void* wd, const void* bd, void* out, int64_t Tn, int H, int E,
                              int K, int64_t cap, int dtype, void* ws, cudaStream_t st) {
  Plan p = plan_backward(ws, Tn, H, E, K, dtype);
  if (Tn == 0) return YAMOE_OK;
  int rc = prepare_routing(p, st);
  if (rc) return rc;
  rc = launch_route<T>(ridx, reinterpret_cast<const T*>(rw), rcols, Tn, E, K, cap, p.rt, st);
  if (rc) return rc;
  const unsigned row_blocks = (unsigned)ceil_div(p.max_rows, kRowWarps);
  const int Hp = H + kBiasCols;
  gather_rows_kernel<T><<<row_blocks, kRowWarps * 32, 0, st>>>(reinterpret_cast<const T*>(hidden),
                                                              reinterpret_cast<T*>(p.xs), p.rt.row_token,
                                                              p.rt.header, H, Hp);
  T* act = reinterpret_cast<T*>(p.gpre);
  T* yrows = reinterpret_cast<T*>(p.gys);
  EpiGlu<T> glu{reinterpret_cast<const T*>(bgu), act, reinterpret_cast<T*>(p.actw), reinterpret_cast<T*>(p.pre),
                p.rt.row_token, p.rt.row_weight, H, Hp};
  EpiWeightedRows<T> wrows{reinterpret_cast<const T*>(bd), yrows, p.rt.row_token, p.rt.row_weight, H};
  GemmArgs g1{p.xs, Hp, wgu, 2 * (int64_t)H, (int64_t)H * 2 * H, 0, 2 * H, H, E,
              p.rt.tile_expert, p.rt.pad_off, p.rt.header};
  g1.pair_expert = p.rt.pair_expert; g1.pair_off = p.rt.pair_off; g1.counts = p.rt.counts;
  GemmArgs g2{act, H, wd, H, (int64_t)H * H, 0, H, H, E, p.rt.tile_expert, p.rt.pad_off, p.rt.header};
  g2.pair_expert = p.rt.pair_expert; g2.pair_off = p.rt.pair_off; g2.counts = p.rt.counts;
  if (use_tcgen05(current_path(), dtype, H)) {
    if constexpr (sizeof(T) == 2) {
      if ((rc = launch_umma<kFwd>(g1, glu, p.max_rows, p.max_tiles, st))) return rc;
      if ((rc = launch_umma<kFwd>(g2, wrows, p.max_rows, p.max_tiles, st))) return rc;
    }
  } else {
    launch_simt_gemm<T, kFwd>(g1, glu, p.max_rows, st);
    launch_simt_gemm<T, kFwd>(g2, wrows, p.max_rows, st);
  }
  combine_padded_kernel<T><<<(unsigned)ceil_div(Tn, kRowWarps), kRowWarps * 32, 0, st>>>(
      yrows, p.rt.flat_row, reinterpret_cast<T*>(out), Tn, H, K);
  return cudaGetLastError() == cudaSuccess ? YAMOE_OK : YAMOE_ERR_CUDA;
}

template <typename T>
static int backward_impl(const void* grad_out, int per_slot, const void* hidden, const int64_t* ridx,
                         const void* rw, int rcols, const void* wgu, const void* bgu, const void* wd,
                         const void* bd, void* d_hidden, void* d_routing, void* d_wgu, void* d_bgu, void* d_wd,
                         void* d_bd, int64_t Tn, int H, int E, int K, int64_t cap, int dtype, void* ws,
                         cudaStream_t st, bool saved = false) {
  // saved: the workspace already holds the routing tables, xs, pre and actw of the forward pass
  // (forward_train_impl); routing, the token gather and the gate_up recompute are skipped.
  Plan p = plan_backward(ws, Tn, H, E, K, dtype);
  const int path = current_path();
  const size_t es = sizeof(T);
  float* acc = p.acc32 ? p.acc32 : reinterpret_cast<float*>(d_hidden);
  YB_CUDA_OK(cudaMemsetAsync(acc, 0, (size_t)Tn * H * sizeof(float), st));
  YB_CUDA_OK(cudaMemsetAsync(d_routing, 0, (size_t)Tn * rcols * es, st));
  if (Tn == 0) {
    YB_CUDA_OK(cudaMemsetAsync(d_wgu, 0, (size_t)E * H * 2 * H * es, st));
    YB_CUDA_OK(cudaMemsetAsync(d_bgu, 0, (size_t)E * 2 * H * es, st));
    YB_CUDA_OK(cudaMemsetAsync(d_wd, 0, (size_t)E * H * H * es, st));
    YB_CUDA_OK(cudaMemsetAsync(d_bd, 0, (size_t)E * H * es, st));
    return YAMOE_OK;
  }
  int rc = YAMOE_OK;
  const int Hp = H + kBiasCols;     // row pitch of xs and actw (see kBiasCols)
  const unsigned row_blocks = (unsigned)ceil_div(p.max_rows, kRowWarps);
  if (!saved) {
    rc = prepare_routing(p, st);
    if (rc) return rc;
    rc = launch_route<T>(ridx, reinterpret_cast<const T*>(rw), rcols, Tn, E, K, cap, p.rt, st);
    if (rc) return rc;
    gather_rows_kernel<T><<<row_blocks, kRowWarps * 32, 0, st>>>(reinterpret_cast<const T*>(hidden),
                                                                reinterpret_cast<T*>(p.xs), p.rt.row_token,
                                                                p.rt.header, H, Hp);
  }
  gather_grad_kernel<T><<<row_blocks, kRowWarps * 32, 0, st>>>(
      reinterpret_cast<const T*>(grad_out), per_slot ? K : 1, reinterpret_cast<const T*>(bd),
      reinterpret_cast<T*>(p.gys), p.gw_row, p.rt.row_token, p.rt.tile_expert, p.rt.header, H);

  // 1. recompute: pre = xs W_gu + b_gu,  actw = w * glu(pre)
  EpiGlu<T> glu{reinterpret_cast<const T*>(bgu), nullptr, reinterpret_cast<T*>(p.actw),
                reinterpret_cast<T*>(p.pre), p.rt.row_token, p.rt.row_weight, H, Hp};
  GemmArgs g1{p.xs, Hp, wgu, 2 * (int64_t)H, (int64_t)H * 2 * H, 0, 2 * H, H, E,
              p.rt.tile_expert, p.rt.pad_off, p.rt.header};
  g1.pair_expert = p.rt.pair_expert; g1.pair_off = p.rt.pair_off; g1.counts = p.rt.counts;
  // 2. gI' = gys W_d^T; fused GLU backward -> gpre, routing-weight gradient -> gw_row
  EpiGluBackward<T> glub{reinterpret_cast<const T*>(p.pre), reinterpret_cast<T*>(p.gpre), p.gw_row,
                         p.rt.row_token, p.rt.row_weight, H};
  GemmArgs g2{p.gys, H, wd, H, (int64_t)H * H, 0, H, H, E, p.rt.tile_expert, p.rt.pad_off, p.rt.header};
  g2.pair_expert = p.rt.pair_expert; g2.pair_off = p.rt.pair_off; g2.counts = p.rt.counts;
  // 3. dW_d[e] = actw_e^T gys_e; the column of routing weights behind actw adds db_d[e] as output row H
  EpiStoreBias<T> st_wd{reinterpret_cast<T*>(d_wd), reinterpret_cast<T*>(d_bd), H, H};
  GemmArgs g3{p.actw, Hp, p.gys, H, 0, H + 1, H, 0, E, p.rt.tile_expert, p.rt.pad_off, p.rt.header};
  g3.pair_expert = p.rt.pair_expert; g3.pair_off = p.rt.pair_off; g3.counts = p.rt.counts;
  // 4. dHidden[token] += gpre W_gu^T
  EpiScatterAdd<T, false, false> sc_dh{nullptr, acc, p.rt.row_token, p.rt.row_weight, H};
  GemmArgs g4{p.gpre, 2 * (int64_t)H, wgu, 2 * (int64_t)H, (int64_t)H * 2 * H, 0, H, 2 * H, E,
              p.rt.tile_expert, p.rt.pad_off, p.rt.header};
  g4.pair_expert = p.rt.pair_expert; g4.pair_off = p.rt.pair_off; g4.counts = p.rt.counts;
  // 5. dW_gu[e] = xs_e^T gpre_e; the column of ones behind xs adds db_gu[e] as output row H
  EpiStoreBias<T> st_wgu{reinterpret_cast<T*>(d_wgu), reinterpret_cast<T*>(d_bgu), H, 2 * H};
  GemmArgs g5{p.xs, Hp, p.gpre, 2 * (int64_t)H, 0, H + 1, 2 * H, 0, E, p.rt.tile_expert, p.rt.pad_off, p.rt.header};
  g5.pair_expert = p.rt.pair_expert; g5.pair_off = p.rt.pair_off; g5.counts = p.rt.counts;

  if (use_tcgen05(path, dtype, H)) {
    if constexpr (sizeof(T) == 2) {
      if (!saved && (rc = launch_umma<kFwd>(g1, glu, p.max_rows, p.max_tiles, st))) return rc;
      if ((rc = launch_umma<kDgrad>(g2, glub, p.max_rows, p.max_tiles, st))) return rc;
      if ((rc = launch_umma<kWgrad>(g3, st_wd, p.max_rows, p.max_tiles, st))) return rc;
      if ((rc = launch_umma<kDgrad>(g4, sc_dh, p.max_rows, p.max_tiles, st))) return rc;
      if ((rc = launch_umma<kWgrad>(g5, st_wgu, p.max_rows, p.max_tiles, st))) return rc;
    }
  } else {
    if (!saved) launch_simt_gemm<T, kFwd>(g1, glu, p.max_rows, st);
    launch_simt_gemm<T, kDgrad>(g2, glub, p.max_rows, st);
    launch_simt_gemm<T, kWgrad>(g3, st_wd, p.max_rows, st);
    launch_simt_gemm<T, kDgrad>(g4, sc_dh, p.max_rows, st);
    launch_simt_gemm<T, kWgrad>(g5, st_wgu, p.max_rows, st);
  }
  // routing-weight gradients (the bias gradients came out of the weight-gradient GEMMs)
  routing_grad_kernel<T><<<(unsigned)ceil_div(p.max_rows, 256), 256, 0, st>>>(
      p.gw_row, p.rt.row_token, p.rt.row_flat, p.rt.tile_expert, p.rt.header, reinterpret_cast<T*>(d_routing),
      rcols, E);
  if (p.acc32) {
    const int64_t nv = Tn * H / 4;
    cast_kernel<T><<<(unsigned)std::min<int64_t>(ceil_div(nv, 256), 148 * 8), 256, 0, st>>>(
        p.acc32, reinterpret_cast<T*>(d_hidden), nv);
  }
  return cudaGetLastError() == cudaSuccess ? YAMOE_OK : YAMOE_ERR_CUDA;
}

// Uniform layout for the batched-matmul sub-operator: expert e owns rows [e*C, (e+1)*C).
__global__ void uniform_tables_kernel(RouteTables rt, int E, int C) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i <= E) rt.pad_off[i] = i * C;
  if (i < E) rt.counts[i] = C;
  const int tiles = C / kTileM, pairs = (tiles + 1) / 2;
  if (i < E * tiles) rt.tile_expert[i] = i / tiles;
  if (i <= E) rt.pair_off[i] = i * pairs;
  if (i < E * pairs) rt.pair_expert[i] = i / pairs;
  if (i == 0) {
    rt.header[kHdrRowTiles] = E * tiles;
    rt.header[kHdrRowsUsed] = E * C;
    rt.header[kHdrPairs] = E * pairs;
  }
}

template <typename T>
static int batch_mm_impl(const void* x, const void* w, void* out, int E, int C, int M, int N, int K, int mode,
                         void* ws, cudaStream_t st) {
  Plan p;
  Bump b(ws);
  carve_tables(b, p, (int64_t)E * C, E, 1, false);
  const int path = current_path();
  YB_CUDA_OK(cudaMemsetAsync(p.rt.header, 0, 16 * sizeof(int32_t), st));
  const int nt = E * (C / kTileM) + E + 1;
  uniform_tables_kernel<<<(unsigned)ceil_div(nt, 256), 256, 0, st>>>(p.rt, E, C);
  const int64_t rows = (int64_t)E * C;
  const bool tc = sizeof(T) == 2 && umma_available() && path != YAMOE_PATH_SIMT;
  int rc = YAMOE_OK;
  if (mode == kWgrad) {
    EpiStore<T> epi{reinterpret_cast<T*>(out), M, N};
    GemmArgs g{x, M, w, N, 0, M, N, 0, E, p.rt.tile_expert, p.rt.pad_off, p.rt.header};
      g.pair_expert = p.rt.pair_expert; g.pair_off = p.rt.pair_off;
    if (tc) { if constexpr (sizeof(T) == 2) rc = launch_umma<kWgrad>(g, epi, rows, rows / kTileM, st); }
    else launch_simt_gemm<T, kWgrad>(g, epi, rows, st);
  } else {
    EpiStoreRows<T> epi{reinterpret_cast<T*>(out), N};
    if (mode == kFwd) {
      GemmArgs g{x, K, w, N, (int64_t)K * N, 0, N, K, E, p.rt.tile_expert, p.rt.pad_off, p.rt.header};
      g.pair_expert = p.rt.pair_expert; g.pair_off = p.rt.pair_off;
      if (tc) { if constexpr (sizeof(T) == 2) rc = launch_umma<kFwd>(g, epi, rows, rows / kTileM, st); }
      else launch_simt_gemm<T, kFwd>(g, epi, rows, st);
    } else {
      GemmArgs g{x, K, w, K, (int64_t)K * N, 0, N, K, E, p.rt.tile_expert, p.rt.pad_off, p.rt.header};
      g.pair_expert = p.rt.pair_expert; g.pair_off = p.rt.pair_off;
      if (tc) { if constexpr (sizeof(T) == 2) rc = launch_umma<kDgrad>(g, epi, rows, rows / kTileM, st); }
      else launch_simt_gemm<T, kDgrad>(g, epi, rows, st);
    }
  }
  if (rc) return rc;
  return cudaGetLastError() == cudaSuccess ? YAMOE_OK : YAMOE_ERR_CUDA;
}

// ---- expert parallelism over peer memory ---------------------------------------------------
struct EpPlan {
  EpTables t;
  void* act = nullptr;     // [max_rows, H]
  // backward only (the tables and `act` above sit at the same offsets in both layouts)
  void* gys = nullptr;     // [max_rows, H]   upstream-gradient rows, zero where not kept
  void* pre = nullptr;     // [max_rows, 2H]
  void* gpre = nullptr;    // [max_rows, 2H]
  float* gw_row = nullptr; // [max_rows]
  size_t bytes = 0;
};

static EpPlan plan_ep(void* ws, int64_t max_rows, int H, int E, int G, int dtype, bool backward = false) {
  EpPlan p;
  Bump b(ws);
  const int per = E / G;
  const int64_t max_tiles = max_rows / kTileM;
  RouteTables& rt = p.t.rt;
  rt = RouteTables{};
  rt.header = b.take<int32_t>(16);
  rt.counts = b.take<int32_t>(per);
  rt.bins = b.take<int32_t>(per + 1);
  rt.pad_off = b.take<int32_t>(per + 1);
  rt.pair_off = b.take<int32_t>(per + 1);
  rt.tile_expert = b.take<int32_t>(max_tiles);
  rt.pair_expert = b.take<int32_t>(max_tiles);
  rt.row_token = b.take<int32_t>(max_rows);
  rt.row_weight = b.take<float>(max_rows);
  p.t.dest_row = b.take<int32_t>(E);
  p.t.src_start = b.take<int32_t>((size_t)G * per);
  p.t.seg_row = b.take<int32_t>((size_t)G * per);
  p.t.row_dest = b.take<int64_t>(max_rows);
  const size_t es = dtype == YAMOE_BF16 ? 2 : 4;
  p.act = b.take<char>((size_t)max_rows * H * es);
  if (backward) {
    p.gys = b.take<char>((size_t)max_rows * H * es);
    p.pre = b.take<char>((size_t)max_rows * 2 * H * es);
    p.gpre = b.take<char>((size_t)max_rows * 2 * H * es);
    p.gw_row = b.take<float>(max_rows);
  }
  p.bytes = b.off + 256;
  return p;
}

static int check_ep(int64_t max_rows, int H, int E, int G, int rank, int dtype) {
  if (dtype != YAMOE_F32 && dtype != YAMOE_BF16) return YAMOE_ERR_DTYPE;
  if (H <= 0 || H % 8 != 0 || E <= 0 || G <= 0 || G > 256 || E % G != 0 || rank < 0 || rank >= G) return YAMOE_ERR_BAD_ARG;
  if (max_rows <= 0 || max_rows % kTileM != 0 || E > 1024) return YAMOE_ERR_BAD_ARG;
  return YAMOE_OK;
}

template <typename T>
static int ep_local_forward_impl(const void* recv_x, const void* wgu, const void* bgu, const void* wd,
                                 const void* bd, void* yrows, int64_t max_rows, int H, int per, int dtype,
                                 const EpPlan& p, cudaStream_t st, const GemmGate& gate = GemmGate{}) {
  const RouteTables& rt = p.t.rt;
  const int64_t max_tiles = max_rows / kTileM;
  EpiGluAct<T> glu{reinterpret_cast<const T*>(bgu), reinterpret_cast<T*>(p.act), rt.row_token, H};
  EpiWeightedRows<T> wrows{reinterpret_cast<const T*>(bd), reinterpret_cast<T*>(yrows), rt.row_token,
                           rt.row_weight, H};
  EpiPeerRows<T> prows{reinterpret_cast<const T*>(bd), p.t.row_dest, rt.row_token, H};
  const bool fused = yrows == nullptr;     // results go straight to the source ranks
  GemmArgs g1{recv_x, H, wgu, 2 * (int64_t)H, (int64_t)H * 2 * H, 0, 2 * H, H, per, rt.tile_expert, rt.pad_off,
              rt.header};
  g1.pair_expert = rt.pair_expert; g1.pair_off = rt.pair_off; g1.counts = rt.counts;
  g1.gate = gate;
  GemmArgs g2{p.act, H, wd, H, (int64_t)H * H, 0, H, H, per, rt.tile_expert, rt.pad_off, rt.header};
  g2.pair_expert = rt.pair_expert; g2.pair_off = rt.pair_off; g2.counts = rt.counts;
  int rc = YAMOE_OK;
  if (use_tcgen05(current_path(), dtype, H)) {
    if constexpr (sizeof(T) == 2) {
      {
        StageTimer tm(kStageGateUp, st);
        // the gate is a feature of the one-CTA kernel
        rc = gate.prep != nullptr ? launch_umma_gemm<kFwd>(g1, glu, max_rows, max_tiles, st)
                                  : launch_umma<kFwd>(g1, glu, max_rows, max_tiles, st);
      }
      if (rc) return rc;
      StageTimer tm(kStageDown, st);
      rc = fused ? launch_umma<kFwd>(g2, prows, max_rows, max_tiles, st)
                 : launch_umma<kFwd>(g2, wrows, max_rows, max_tiles, st);
      if (rc) return rc;
    }
  } else {
    launch_simt_gemm<T, kFwd>(g1, glu, max_rows, st);
    if (fused) launch_simt_gemm<T, kFwd>(g2, prows, max_rows, st);
    else launch_simt_gemm<T, kFwd>(g2, wrows, max_rows, st);
  }
  return cudaGetLastError() == cudaSuccess ? YAMOE_OK : YAMOE_ERR_CUDA;
}

// Backward of the local problem on the rows peers stored here: recv_x (token rows), recv_g
// (upstream-gradient rows) and recv_w (routing weights), all in the padded layout of the plan.
// Input-gradient rows leave through the last dgrad GEMM's epilogue into the source ranks' buffers
// (row_dest of the plan), routing-weight gradients through ep_return_scalar_kernel.
template <typename T>
static int ep_local_backward_impl(const void* recv_x, const void* recv_g, const float* recv_w, const void* wgu,
                                  const void* bgu, const void* wd, const void* bd, void* d_wgu, void* d_bgu,
                                  void* d_wd, void* d_bd, void* const* peer_back_w, int64_t cap, int64_t max_rows,
                                  int H, int per, int G, int dtype, const EpPlan& p, cudaStream_t st,
                                  const GemmGate& gate = GemmGate{}) {
  const RouteTables& rt = p.t.rt;
  const int64_t max_tiles = max_rows / kTileM;
  auto with_pairs = [&](GemmArgs g) { g.pair_expert = rt.pair_expert; g.pair_off = rt.pair_off; g.counts = rt.counts; return g; };
  // p.act receives the activations times the routing weight; the weights are taken from the
  // receive buffer itself (row_weight is filled from it only after this GEMM)
  EpiGlu<T> glu{reinterpret_cast<const T*>(bgu), nullptr, reinterpret_cast<T*>(p.act), reinterpret_cast<T*>(p.pre),
                rt.row_token, recv_w, H, 0};
  GemmArgs g1 = with_pairs(GemmArgs{recv_x, H, wgu, 2 * (int64_t)H, (int64_t)H * 2 * H, 0, 2 * H, H, per,
                                    rt.tile_expert, rt.pad_off, rt.header});
  g1.gate = gate;
  EpiGluBackward<T> glub{reinterpret_cast<const T*>(p.pre), reinterpret_cast<T*>(p.gpre), p.gw_row, rt.row_token,
                         rt.row_weight, H};
  const GemmArgs g2 = with_pairs(GemmArgs{p.gys, H, wd, H, (int64_t)H * H, 0, H, H, per, rt.tile_expert, rt.pad_off,
                                          rt.header});
  EpiStore<T> st_wd{reinterpret_cast<T*>(d_wd), H, H};
  const GemmArgs g3 = with_pairs(GemmArgs{p.act, H, p.gys, H, 0, H, H, 0, per, rt.tile_expert, rt.pad_off,
                                          rt.header});
  EpiPeerRows<T> prows{nullptr, p.t.row_dest, rt.row_token, H};
  const GemmArgs g4 = with_pairs(GemmArgs{p.gpre, 2 * (int64_t)H, wgu, 2 * (int64_t)H, (int64_t)H * 2 * H, 0, H,
                                          2 * H, per, rt.tile_expert, rt.pad_off, rt.header});
  EpiStore<T> st_wgu{reinterpret_cast<T*>(d_wgu), H, 2 * H};
  const GemmArgs g5 = with_pairs(GemmArgs{recv_x, H, p.gpre, 2 * (int64_t)H, 0, H, 2 * H, 0, per, rt.tile_expert,
                                          rt.pad_off, rt.header});
  int rc = YAMOE_OK;
  const bool tc = use_tcgen05(current_path(), dtype, H);
  // The recomputed gate_up GEMM needs only the token rows: it goes first, and with a gate it runs
  // next to the dispatch kernel, waiting for each expert's rows by itself.  When it has finished,
  // every row of this rank (token, gradient, weight) has arrived.
  if (tc) {
    if constexpr (sizeof(T) == 2) {
      if ((rc = launch_umma<kFwd>(g1, glu, max_rows, max_tiles, st))) return rc;
    }
  } else {
    launch_simt_gemm<T, kFwd>(g1, glu, max_rows, st);
  }
  ep_load_weights_kernel<<<(unsigned)ceil_div(max_rows, 256), 256, 0, st>>>(p.t, recv_w, max_rows);
  gather_grad_kernel<T><<<(unsigned)ceil_div(max_rows, kRowWarps), kRowWarps * 32, 0, st>>>(
      reinterpret_cast<const T*>(recv_g), 1, reinterpret_cast<const T*>(bd), reinterpret_cast<T*>(p.gys), p.gw_row,
      rt.row_token, rt.tile_expert, rt.header, H);
  if (tc) {
    if constexpr (sizeof(T) == 2) {
      if ((rc = launch_umma<kDgrad>(g2, glub, max_rows, max_tiles, st))) return rc;
      if ((rc = launch_umma<kWgrad>(g3, st_wd, max_rows, max_tiles, st))) return rc;
      if ((rc = launch_umma<kDgrad>(g4, prows, max_rows, max_tiles, st))) return rc;
      if ((rc = launch_umma<kWgrad>(g5, st_wgu, max_rows, max_tiles, st))) return rc;
    }
  } else {
    launch_simt_gemm<T, kDgrad>(g2, glub, max_rows, st);
    launch_simt_gemm<T, kWgrad>(g3, st_wd, max_rows, st);
    launch_simt_gemm<T, kDgrad>(g4, prows, max_rows, st);
    launch_simt_gemm<T, kWgrad>(g5, st_wgu, max_rows, st);
  }
  colsum_kernel<T, true><<<dim3((unsigned)ceil_div(H, 512 / (int)sizeof(T)), per), 256, 0, st>>>(
      reinterpret_cast<const T*>(p.gys), rt.row_weight, rt.pad_off, rt.counts, cap, reinterpret_cast<T*>(d_bd), H);
  colsum_kernel<T, false><<<dim3((unsigned)ceil_div(2 * H, 512 / (int)sizeof(T)), per), 256, 0, st>>>(
      reinterpret_cast<const T*>(p.gpre), rt.row_weight, rt.pad_off, rt.counts, cap, reinterpret_cast<T*>(d_bgu),
      2 * H);
  ep_return_scalar_kernel<<<(unsigned)ceil_div(max_rows, 256), 256, 0, st>>>(p.gw_row, p.t, peer_back_w, G, per);
  return cudaGetLastError() == cudaSuccess ? YAMOE_OK : YAMOE_ERR_CUDA;
}


// ---- expert parallelism as one chain of kernels (flags in symmetric memory) ----------------------
// Workspace of a whole expert-parallel call: the plan / activation region of plan_ep first (so the
// status word sits at the start of the workspace), then the tables of the local sort.
struct EpCallPlan {
  EpPlan ep;
  RouteTables rt;          // local sort of this rank's assignments (no row tables)
  size_t bytes = 0;
};

static EpCallPlan plan_ep_call(void* ws, const yamoe_ep_ctx_t& c, int64_t T, bool backward) {
  EpCallPlan p;
  p.ep = plan_ep(ws, c.max_rows, c.H, c.E, c.G, c.dtype, backward);
  Bump b(ws);
  b.off = p.ep.bytes;
  const int64_t S = T * c.K;
  p.rt.header = b.take<int32_t>(16);
  p.rt.counts = b.take<int32_t>(c.E);
  p.rt.bins = b.take<int32_t>(c.E + 1);
  p.rt.pad_off = b.take<int32_t>(c.E + 1);
  p.rt.block_counts = b.take<int32_t>((size_t)route_blocks(S > 0 ? S : 1) * c.E);
  p.rt.sorted_values = b.take<int32_t>(S > 0 ? S : 1);
  p.rt.sorted_indices = b.take<int32_t>(S > 0 ? S : 1);
  p.rt.flat_pos = b.take<int32_t>(S > 0 ? S : 1);
  p.bytes = b.off + 256;
  return p;
}

static int check_ep_ctx(const yamoe_ep_ctx_t* c, bool backward) {
  if (!c) return YAMOE_ERR_BAD_ARG;
  int rc = check_ep(c->max_rows, c->H, c->E, c->G, c->rank, c->dtype);
  if (rc) return rc;
  if (c->K <= 0 || c->back_rows <= 0) return YAMOE_ERR_BAD_ARG;
  if (!c->peer_recv_x || !c->peer_back || !c->peer_ctrl || !c->recv_x || !c->back || !c->ctrl || !c->state)
    return YAMOE_ERR_BAD_ARG;
  if (backward && (!c->peer_recv_g || !c->peer_recv_w || !c->peer_back_w || !c->recv_g || !c->recv_w || !c->back_w))
    return YAMOE_ERR_BAD_ARG;
  return YAMOE_OK;
}

// Steps shared by the forward and the backward call, up to the point where every row this rank's
// experts need has arrived: local sort, count exchange, dispatch, row tables, wait.
// With `gate` (forward on the tcgen05 path) the prologue ends with the dispatch kernel still
// running: *gate is filled in for the gate_up GEMM, which is launched next to it and waits for each
// expert's rows by itself.  Otherwise the prologue ends with the wait for all sources.
template <typename T>
static int ep_call_prologue(const yamoe_ep_ctx_t& c, const EpCallPlan& p, const void* hidden, const void* grad,
                            const int64_t* ridx, const void* rw, int rcols, int64_t Tn, int64_t cap,
                            void* const* peer_back, cudaStream_t st, GemmGate* gate = nullptr) {
  const int64_t S = Tn * c.K;
  const uint64_t wait_ns = c.wait_ns ? c.wait_ns : kWaitLimitNs;
  const EpCtrlLayout lay{c.G, c.E};
  YB_CUDA_OK(cudaMemsetAsync(p.ep.t.rt.header, 0, 16 * sizeof(int32_t), st));
  YB_CUDA_OK(cudaMemsetAsync(p.rt.header, 0, 16 * sizeof(int32_t), st));
  if (S > 0) {
    YB_CUDA_OK(cudaMemsetAsync(p.rt.flat_pos, 0xFF, (size_t)S * sizeof(int32_t), st));
    int rc = launch_route<float>(ridx, nullptr, c.E, S, c.E, 1, (int64_t)1 << 40, p.rt, st);
    if (rc) return rc;
  } else {
    YB_CUDA_OK(cudaMemsetAsync(p.rt.counts, 0, (size_t)c.E * sizeof(int32_t), st));
    YB_CUDA_OK(cudaMemsetAsync(p.rt.bins, 0, (size_t)(c.E + 1) * sizeof(int32_t), st));
  }
  ep_publish_kernel<<<1, 256, 0, st>>>(p.rt.counts, reinterpret_cast<int32_t*>(c.state), c.peer_ctrl, lay, c.rank);
  EpDispatchArgs a{};
  a.hidden = hidden;
  a.grad = grad;
  a.routing_weights = grad ? rw : nullptr;
  a.routing_cols = rcols;
  a.sorted_values = p.rt.sorted_values;
  a.sorted_indices = p.rt.sorted_indices;
  a.bins = p.rt.bins;
  a.peer_x = c.peer_recv_x;
  a.peer_g = c.peer_recv_g;
  a.peer_w = c.peer_recv_w;
  a.peer_back = peer_back;
  a.peer_ctrl = c.peer_ctrl;
  a.ctrl = reinterpret_cast<const int32_t*>(c.ctrl);
  a.state = reinterpret_cast<int32_t*>(c.state);
  a.max_rows = c.max_rows;
  a.capacity = cap;
  a.row_bytes = (int64_t)c.H * sizeof(T);
  a.S = (int)S; a.H = c.H; a.E = c.E; a.G = c.G; a.rank = c.rank; a.K = c.K;
  a.signal_rows = gate != nullptr ? 1 : 0;
  a.wait_ns = wait_ns;
  // Alone the kernel fills the GPU (four CTAs per SM).  Next to the gated GEMM it runs with one CTA
  // on every second SM (YAMOE_B200_EP_DISPATCH_CTAS overrides the number): that many warps still
  // saturate NVLink, they take little from the GEMM, and - what matters most - few enough rows are
  // in flight at a time that the experts really complete in phase order; with hundreds of CTAs
  // every phase is issued at once and the first expert is complete only when nearly all are.
  // Measured on 2 GPUs, weak-scaled forward: 0.925 ms with 296 CTAs, 0.879 with 148, 0.869 with 74,
  // 0.881 with 37, 1.12 with 18; 0.927 without overlap.  The kernel asks for the same (maximal)
  // shared-memory carve-out as the GEMM: CTAs of kernels with different carve-outs do not share an SM.
  static const int grid_cap_env = []() {
    const char* env = std::getenv("YAMOE_B200_EP_DISPATCH_CTAS");
    return env != nullptr ? std::atoi(env) : 0;
  }();
  const int64_t grid_cap = gate == nullptr      ? (int64_t)umma_sm_count() * 4
                           : grid_cap_env > 0 ? grid_cap_env
                                              : std::max(1, umma_sm_count() / 2);
  const int grid = (int)std::max<int64_t>(
      1, std::min<int64_t>(std::max<int64_t>(ceil_div(S, kRowWarps * 4), ceil_div(c.max_rows, 4096)), grid_cap));
  {
    static PerDevice<int> carveout_set;    // per template instantiation and device
    const int dev = current_device_index();
    if (!carveout_set.get(dev)) {
      cudaFuncSetAttribute(ep_dispatch_fused_kernel<T>, cudaFuncAttributePreferredSharedMemoryCarveout,
                           (int)cudaSharedmemCarveoutMaxShared);
      carveout_set.set(dev, 1);
    }
  }
  ep_dispatch_fused_kernel<T><<<grid, kRowWarps * 32, (size_t)(6 * c.E + 2) * sizeof(int32_t), st>>>(a, p.ep.t);
  if (gate != nullptr) {
    gate->prep = reinterpret_cast<const int32_t*>(c.state) + kEpStatePrep;
    gate->prep_target = grid;
    gate->arrived = reinterpret_cast<const int32_t*>(c.ctrl) + lay.arrived();
    gate->needed = p.ep.t.rt.counts;
    gate->wait_ns = wait_ns;
  } else {
    ep_wait_kernel<<<1, 32, 0, st>>>(reinterpret_cast<const int32_t*>(c.ctrl) + lay.flag_dispatch(), c.G,
                                     reinterpret_cast<const int32_t*>(c.state), p.ep.t.rt.header,
                                     (int)kStatusEpDispatchTimeout, wait_ns);
  }
  return cudaGetLastError() == cudaSuccess ? YAMOE_OK : YAMOE_ERR_CUDA;
}

// The gate_up GEMM (the recomputed one in the backward pass) overlaps the dispatch when it is the
// tcgen05 kernel; YAMOE_B200_EP_OVERLAP=0 keeps the two apart (dispatch, wait for all sources,
// then the GEMMs).
static bool ep_overlap_enabled() {
  static const bool on = []() {
    const char* env = std::getenv("YAMOE_B200_EP_OVERLAP");
    return env == nullptr || std::atoi(env) != 0;
  }();
  return on;
}

template <typename T>
static int ep_forward_impl(const yamoe_ep_ctx_t& c, const void* hidden, const int64_t* ridx, const void* rw,
                           int rcols, const void* wgu, const void* bgu, const void* wd, const void* bd, void* out,
                           int64_t Tn, int64_t cap, void* ws, cudaStream_t st) {
  const EpCallPlan p = plan_ep_call(ws, c, Tn, false);
  const EpCtrlLayout lay{c.G, c.E};
  const uint64_t wait_ns = c.wait_ns ? c.wait_ns : kWaitLimitNs;
  int rc;
  const bool overlap = ep_overlap_enabled() && sizeof(T) == 2 && use_tcgen05(current_path(), c.dtype, c.H);
  GemmGate gate;
  {
    StageTimer tm(kStageEpDispatch, st);
    rc = ep_call_prologue<T>(c, p, hidden, nullptr, ridx, rw, rcols, Tn, cap, c.peer_back, st,
                             overlap ? &gate : nullptr);
  }
  if (rc) return rc;
  // gate_up + GLU + down on the received rows; the down GEMM's epilogue stores every result row
  // into the back buffer of the rank that owns the token
  rc = ep_local_forward_impl<T>(c.recv_x, wgu, bgu, wd, bd, nullptr, c.max_rows, c.H, c.E / c.G, c.dtype, p.ep, st,
                                gate);
  if (rc) return rc;
  StageTimer tm(kStageEpCombine, st);
  ep_signal_kernel<<<1, 32, 0, st>>>(c.peer_ctrl, lay.flag_return(), c.G, c.rank,
                                     reinterpret_cast<const int32_t*>(c.state));
  const int grid = (int)std::max<int64_t>(1, std::min<int64_t>(ceil_div(Tn, kRowWarps), (int64_t)umma_sm_count() * 8));
  ep_combine_kernel<T, false><<<grid, kRowWarps * 32, 0, st>>>(
      reinterpret_cast<const T*>(c.back), p.rt.flat_pos, ridx, reinterpret_cast<const T*>(rw), rcols,
      reinterpret_cast<T*>(out), Tn, c.H, c.E, c.K, reinterpret_cast<const int32_t*>(c.ctrl) + lay.flag_return(), c.G,
      reinterpret_cast<const int32_t*>(c.state), p.ep.t.rt.header, wait_ns);
  return cudaGetLastError() == cudaSuccess ? YAMOE_OK : YAMOE_ERR_CUDA;
}

template <typename T>
static int ep_backward_impl(const yamoe_ep_ctx_t& c, const void* grad_out, const void* hidden, const int64_t* ridx,
                            const void* rw, int rcols, const void* wgu, const void* bgu, const void* wd,
                            const void* bd, void* d_hidden, void* d_routing, void* d_wgu, void* d_bgu, void* d_wd,
                            void* d_bd, int64_t Tn, int64_t cap, void* ws, cudaStream_t st) {
  const EpCallPlan p = plan_ep_call(ws, c, Tn, true);
  const EpCtrlLayout lay{c.G, c.E};
  const uint64_t wait_ns = c.wait_ns ? c.wait_ns : kWaitLimitNs;
  const int64_t S = Tn * c.K;
  const bool overlap = ep_overlap_enabled() && sizeof(T) == 2 && use_tcgen05(current_path(), c.dtype, c.H);
  GemmGate gate;
  int rc = ep_call_prologue<T>(c, p, hidden, grad_out, ridx, rw, rcols, Tn, cap, c.peer_back, st,
                               overlap ? &gate : nullptr);
  if (rc) return rc;
  rc = ep_local_backward_impl<T>(c.recv_x, c.recv_g, reinterpret_cast<const float*>(c.recv_w), wgu, bgu, wd, bd,
                                 d_wgu, d_bgu, d_wd, d_bd, c.peer_back_w, cap, c.max_rows, c.H, c.E / c.G, c.G,
                                 c.dtype, p.ep, st, gate);
  if (rc) return rc;
  ep_signal_kernel<<<1, 32, 0, st>>>(c.peer_ctrl, lay.flag_return(), c.G, c.rank,
                                     reinterpret_cast<const int32_t*>(c.state));
  const int grid = (int)std::max<int64_t>(1, std::min<int64_t>(ceil_div(Tn, kRowWarps), (int64_t)umma_sm_count() * 8));
  ep_combine_kernel<T, true><<<grid, kRowWarps * 32, 0, st>>>(
      reinterpret_cast<const T*>(c.back), p.rt.flat_pos, ridx, nullptr, rcols, reinterpret_cast<T*>(d_hidden), Tn,
      c.H, c.E, c.K, reinterpret_cast<const int32_t*>(c.ctrl) + lay.flag_return(), c.G,
      reinterpret_cast<const int32_t*>(c.state), p.ep.t.rt.header, wait_ns);
  if (rcols == c.E) YB_CUDA_OK(cudaMemsetAsync(d_routing, 0, (size_t)Tn * rcols * sizeof(T), st));
  if (S > 0)
    ep_routing_grad_kernel<T><<<(unsigned)ceil_div(S, 256), 256, 0, st>>>(
        reinterpret_cast<const float*>(c.back_w), p.rt.flat_pos, ridx, reinterpret_cast<T*>(d_routing), S, rcols, c.E,
        c.K);
  return cudaGetLastError() == cudaSuccess ? YAMOE_OK : YAMOE_ERR_CUDA;
}

// ---- routing without a caller workspace -------------------------------------------------
// Scratch for yamoe_b200_route_static.  It is part of the library image: every GPU that loads the
// library keeps these bytes reserved until the process exits.  All calls on one device share it.
constexpr size_t kStaticScratchBytes = 1u << 20;
static __device__ __align__(256) unsigned char g_route_static_scratch[kStaticScratchBytes];

constexpr int kMaxStaticDevices = 64;
static void* g_static_scratch_addr[kMaxStaticDevices] = {};
static std::mutex g_static_scratch_mutex;

// Device address of the static scratch on the current device.  In host code the array's name
// is only a handle, so the address is asked for once per device and remembered.
static int static_scratch_address(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxStaticDevices) return YAMOE_ERR_CUDA;
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_route_static_scratch) != cudaSuccess || p == nullptr) return YAMOE_ERR_CUDA;
    g_static_scratch_addr[dev] = p;
  }
  *out = g_static_scratch_addr[dev];
  return YAMOE_OK;
}

// Scratch the routing kernels need besides their outputs; with base == nullptr it only measures.
static size_t carve_static_route(void* base, RouteTables& rt, int64_t S, int E) {
  Bump b(base);
  rt.header = b.take<int32_t>(16);
  rt.counts = b.take<int32_t>(E);
  rt.pad_off = b.take<int32_t>(E + 1);
  rt.block_counts = b.take<int32_t>((size_t)route_blocks(S) * E);
  return b.off;
}

}  // namespace yb

using namespace yb;

extern "C" {

int yamoe_b200_version(void) { return 100; }

const char* yamoe_b200_status_string(int s) {
  switch (s) {
    case YAMOE_OK: return "ok";
    case YAMOE_ERR_BAD_ARG: return "bad argument";
    case YAMOE_ERR_WORKSPACE: return "workspace null, misaligned or too small";
    case YAMOE_ERR_DTYPE: return "unsupported dtype";
    case YAMOE_ERR_CUDA: return "CUDA call failed";
    case YAMOE_ERR_UNSUPPORTED: return "unsupported configuration";
    case YAMOE_ERR_DEVICE_TIMEOUT: return "bounded device-side wait gave up";
    case YAMOE_ERR_STATIC_SCRATCH: return "request needs more than the 1 MiB static scratch of yamoe_b200_route_static";
    default: return "unknown status";
  }
}

int yamoe_b200_set_path(int path) {
  int prev = current_path();
  if (path >= YAMOE_PATH_AUTO && path <= YAMOE_PATH_GEMV) g_path.store(path);
  return prev;
}

int yamoe_b200_set_stage_events(void* start_event, void* stop_event, int stage) {
  if (stage < kStageNone || stage > kStageLast) return YAMOE_ERR_BAD_ARG;
  if (stage != kStageNone && (!start_event || !stop_event)) return YAMOE_ERR_BAD_ARG;
  g_events.stage.store(kStageNone);
  g_events.start.store(start_event);
  g_events.stop.store(stop_event);
  g_events.stage.store(stage);
  return YAMOE_OK;
}

size_t yamoe_b200_route_workspace_bytes(int64_t T, int E, int K) {
  if (T < 0 || E <= 0 || K <= 0) return 0;
  Plan p;
  Bump b(nullptr);
  carve_tables(b, p, T, E, K, false);
  return b.off + 256;
}

int yamoe_b200_route(const int64_t* router_indices, int32_t* sorted_values, int32_t* sorted_indices,
                     int32_t* bins, int32_t* counts, int64_t T, int E, int K, void* workspace,
                     size_t workspace_bytes, void* stream) {
  int rc = check_common(T, 8, E, K, YAMOE_F32);
  if (rc) return rc;
  if (!router_indices || !sorted_values || !sorted_indices || !bins) return YAMOE_ERR_BAD_ARG;
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255) ||
      workspace_bytes < yamoe_b200_route_workspace_bytes(T, E, K))
    return YAMOE_ERR_WORKSPACE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  Plan p;
  Bump b(workspace);
  carve_tables(b, p, T, E, K, false);
  p.rt.sorted_values = sorted_values;
  p.rt.sorted_indices = sorted_indices;
  p.rt.bins = bins;
  if (counts) p.rt.counts = counts;
  p.rt.tile_expert = nullptr;
  p.rt.pair_expert = nullptr;
  YB_CUDA_OK(cudaMemsetAsync(p.rt.header, 0, 16 * sizeof(int32_t), st));
  if (T == 0) {
    YB_CUDA_OK(cudaMemsetAsync(bins, 0, (size_t)(E + 1) * sizeof(int32_t), st));
    if (counts) YB_CUDA_OK(cudaMemsetAsync(counts, 0, (size_t)E * sizeof(int32_t), st));
    return YAMOE_OK;
  }
  // ids outside [0, E) are dropped: the entries behind the last kept one read -1
  YB_CUDA_OK(cudaMemsetAsync(sorted_values, 0xFF, (size_t)T * K * sizeof(int32_t), st));
  YB_CUDA_OK(cudaMemsetAsync(sorted_indices, 0xFF, (size_t)T * K * sizeof(int32_t), st));
  return launch_route<float>(router_indices, nullptr, E, T, E, K, (int64_t)1 << 40, p.rt, st);
}

size_t yamoe_b200_route_static_scratch_needed(int64_t T, int E, int K) {
  if (T < 0 || E <= 0 || K <= 0) return 0;
  RouteTables rt;
  return carve_static_route(nullptr, rt, T * K, E);
}

int yamoe_b200_route_static(const int64_t* router_indices, int32_t* sorted_values, int32_t* sorted_indices,
                            int32_t* bins, int32_t* counts, int64_t T, int E, int K, void* stream) {
  int rc = check_common(T, 8, E, K, YAMOE_F32);
  if (rc) return rc;
  if (!router_indices || !sorted_values || !sorted_indices || !bins) return YAMOE_ERR_BAD_ARG;
  RouteTables rt{};
  if (carve_static_route(nullptr, rt, T * K, E) > kStaticScratchBytes) return YAMOE_ERR_STATIC_SCRATCH;
  void* scratch = nullptr;
  rc = static_scratch_address(&scratch);
  if (rc) return rc;
  carve_static_route(scratch, rt, T * K, E);
  rt.sorted_values = sorted_values;
  rt.sorted_indices = sorted_indices;
  rt.bins = bins;
  if (counts) rt.counts = counts;
  rt.tile_expert = nullptr;
  rt.row_token = rt.row_flat = nullptr;
  rt.row_weight = nullptr;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // the ticket counter and status words must start at zero; the array keeps the last call's contents
  YB_CUDA_OK(cudaMemsetAsync(rt.header, 0, 16 * sizeof(int32_t), st));
  if (T == 0) {
    YB_CUDA_OK(cudaMemsetAsync(bins, 0, (size_t)(E + 1) * sizeof(int32_t), st));
    if (counts) YB_CUDA_OK(cudaMemsetAsync(counts, 0, (size_t)E * sizeof(int32_t), st));
    return YAMOE_OK;
  }
  YB_CUDA_OK(cudaMemsetAsync(sorted_values, 0xFF, (size_t)T * K * sizeof(int32_t), st));
  YB_CUDA_OK(cudaMemsetAsync(sorted_indices, 0xFF, (size_t)T * K * sizeof(int32_t), st));
  return launch_route<float>(router_indices, nullptr, E, T, E, K, (int64_t)1 << 40, rt, st);
}

size_t yamoe_b200_forward_workspace_bytes(int64_t T, int H, int E, int K, int dtype) {
  if (check_common(T, H, E, K, dtype)) return 0;
  return plan_forward(nullptr, T, H, E, K, dtype).bytes;
}

int yamoe_b200_experts_forward(const void* hidden_states, const int64_t* router_indices,
                               const void* routing_weights, int routing_cols, const void* gate_up_proj,
                               const void* gate_up_proj_bias, const void* down_proj, const void* down_proj_bias,
                               void* out, int64_t T, int H, int E, int K, int64_t expert_capacity, int dtype,
                               void* workspace, size_t workspace_bytes, void* stream) {
  int rc = check_common(T, H, E, K, dtype);
  if (rc) return rc;
  if (routing_cols != E && routing_cols != K) return YAMOE_ERR_BAD_ARG;
  if (expert_capacity < 0) return YAMOE_ERR_BAD_ARG;
  if (T > 0 && (!hidden_states || !router_indices || !routing_weights || !out)) return YAMOE_ERR_BAD_ARG;
  if (!gate_up_proj || !gate_up_proj_bias || !down_proj || !down_proj_bias) return YAMOE_ERR_BAD_ARG;
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255) ||
      workspace_bytes < yamoe_b200_forward_workspace_bytes(T, H, E, K, dtype))
    return YAMOE_ERR_WORKSPACE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == YAMOE_BF16)
    return forward_impl<__nv_bfloat16>(hidden_states, router_indices, routing_weights, routing_cols, gate_up_proj,
                                       gate_up_proj_bias, down_proj, down_proj_bias, out, T, H, E, K,
                                       expert_capacity, dtype, workspace, st);
  return forward_impl<float>(hidden_states, router_indices, routing_weights, routing_cols, gate_up_proj,
                             gate_up_proj_bias, down_proj, down_proj_bias, out, T, H, E, K, expert_capacity,
                             dtype, workspace, st);
}

size_t yamoe_b200_backward_workspace_bytes(int64_t T, int H, int E, int K, int dtype) {
  if (check_common(T, H, E, K, dtype)) return 0;
  return plan_backward(nullptr, T, H, E, K, dtype).bytes;
}

int yamoe_b200_experts_backward(const void* grad_out, int grad_out_per_slot, const void* hidden_states,
                                const int64_t* router_indices, const void* routing_weights, int routing_cols,
                                const void* gate_up_proj, const void* gate_up_proj_bias, const void* down_proj,
                                const void* down_proj_bias, void* d_hidden, void* d_routing, void* d_gate_up_proj,
                                void* d_gate_up_proj_bias, void* d_down_proj, void* d_down_proj_bias, int64_t T,
                                int H, int E, int K, int64_t expert_capacity, int dtype, void* workspace,
                                size_t workspace_bytes, void* stream) {
  int rc = check_common(T, H, E, K, dtype);
  if (rc) return rc;
  if (routing_cols != E && routing_cols != K) return YAMOE_ERR_BAD_ARG;
  if (expert_capacity < 0) return YAMOE_ERR_BAD_ARG;
  if (T > 0 && (!grad_out || !hidden_states || !router_indices || !routing_weights || !d_hidden || !d_routing))
    return YAMOE_ERR_BAD_ARG;
  if (!gate_up_proj || !gate_up_proj_bias || !down_proj || !down_proj_bias || !d_gate_up_proj ||
      !d_gate_up_proj_bias || !d_down_proj || !d_down_proj_bias)
    return YAMOE_ERR_BAD_ARG;
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255) ||
      workspace_bytes < yamoe_b200_backward_workspace_bytes(T, H, E, K, dtype))
    return YAMOE_ERR_WORKSPACE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == YAMOE_BF16)
    return backward_impl<__nv_bfloat16>(grad_out, grad_out_per_slot, hidden_states, router_indices,
                                        routing_weights, routing_cols, gate_up_proj, gate_up_proj_bias, down_proj,
                                        down_proj_bias, d_hidden, d_routing, d_gate_up_proj, d_gate_up_proj_bias,
                                        d_down_proj, d_down_proj_bias, T, H, E, K, expert_capacity, dtype,
                                        workspace, st);
  return backward_impl<float>(grad_out, grad_out_per_slot, hidden_states, router_indices, routing_weights,
                              routing_cols, gate_up_proj, gate_up_proj_bias, down_proj, down_proj_bias, d_hidden,
                              d_routing, d_gate_up_proj, d_gate_up_proj_bias, d_down_proj, d_down_proj_bias, T, H,
                              E, K, expert_capacity, dtype, workspace, st);
}

size_t yamoe_b200_batch_mm_workspace_bytes(int E, int C) {
  if (E <= 0 || C <= 0) return 0;
  Plan p;
  Bump b(nullptr);
  carve_tables(b, p, (int64_t)E * C, E, 1, false);
  return b.off + 256;
}

int yamoe_b200_batch_mm(const void* x, const void* weights, void* out, int E, int C, int M, int N, int K,
                        int mode, int dtype, void* workspace, size_t workspace_bytes, void* stream) {
  if (dtype != YAMOE_F32 && dtype != YAMOE_BF16) return YAMOE_ERR_DTYPE;
  if (!x || !weights || !out || E <= 0 || C <= 0 || N <= 0 || mode < 0 || mode > 2) return YAMOE_ERR_BAD_ARG;
  if (mode == kWgrad ? (M <= 0) : (K <= 0)) return YAMOE_ERR_BAD_ARG;
  if (C % kTileM != 0 || N % 64 != 0 || (mode == kWgrad ? M % 64 != 0 : K % 64 != 0)) return YAMOE_ERR_UNSUPPORTED;
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255) ||
      workspace_bytes < yamoe_b200_batch_mm_workspace_bytes(E, C))
    return YAMOE_ERR_WORKSPACE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == YAMOE_BF16) return batch_mm_impl<__nv_bfloat16>(x, weights, out, E, C, M, N, K, mode, workspace, st);
  return batch_mm_impl<float>(x, weights, out, E, C, M, N, K, mode, workspace, st);
}

int yamoe_b200_permute_rows(const void* src, int64_t n_src, const int32_t* sorted_indices, void* dst, int64_t S, int H,
                            int K, int dtype, void* stream) {
  if (dtype != YAMOE_F32 && dtype != YAMOE_BF16) return YAMOE_ERR_DTYPE;
  if (S < 0 || H <= 0 || H % 8 != 0 || K <= 0 || n_src < 0) return YAMOE_ERR_BAD_ARG;
  if (S == 0) return YAMOE_OK;
  if (!src || !sorted_indices || !dst) return YAMOE_ERR_BAD_ARG;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const unsigned blocks = (unsigned)ceil_div(S, kRowWarps);
  if (dtype == YAMOE_BF16)
    permute_rows_kernel<__nv_bfloat16><<<blocks, kRowWarps * 32, 0, st>>>(
        reinterpret_cast<const __nv_bfloat16*>(src), sorted_indices, reinterpret_cast<__nv_bfloat16*>(dst), S, H, K,
        n_src);
  else
    permute_rows_kernel<float><<<blocks, kRowWarps * 32, 0, st>>>(
        reinterpret_cast<const float*>(src), sorted_indices, reinterpret_cast<float*>(dst), S, H, K, n_src);
  return cudaGetLastError() == cudaSuccess ? YAMOE_OK : YAMOE_ERR_CUDA;
}

int yamoe_b200_combine_rows(const void* rows, const int32_t* sorted_indices, int64_t n_sorted,
                            const int64_t* router_indices, const void* routing_weights, int routing_cols, void* out,
                            int64_t T, int H, int E, int K, int dtype, void* workspace, size_t workspace_bytes,
                            void* stream) {
  if (dtype != YAMOE_F32 && dtype != YAMOE_BF16) return YAMOE_ERR_DTYPE;
  if (T < 0 || H <= 0 || H % 8 != 0 || K <= 0 || E <= 0 || n_sorted < 0 || n_sorted > T * K) return YAMOE_ERR_BAD_ARG;
  if (routing_cols != E && routing_cols != K) return YAMOE_ERR_BAD_ARG;
  if (T == 0) return YAMOE_OK;
  if (!rows || !sorted_indices || !router_indices || !routing_weights || !out) return YAMOE_ERR_BAD_ARG;
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255) || workspace_bytes < (size_t)T * K * sizeof(int32_t))
    return YAMOE_ERR_WORKSPACE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int32_t* inv = reinterpret_cast<int32_t*>(workspace);
  YB_CUDA_OK(cudaMemsetAsync(inv, 0xFF, (size_t)T * K * sizeof(int32_t), st));
  if (n_sorted > 0)
    invert_perm_kernel<<<(unsigned)ceil_div(n_sorted, 256), 256, 0, st>>>(sorted_indices, inv, n_sorted, T * K);
  const unsigned blocks = (unsigned)ceil_div(T, kRowWarps);
  if (dtype == YAMOE_BF16)
    combine_rows_kernel<__nv_bfloat16><<<blocks, kRowWarps * 32, 0, st>>>(
        reinterpret_cast<const __nv_bfloat16*>(rows), inv, router_indices,
        reinterpret_cast<const __nv_bfloat16*>(routing_weights), routing_cols, reinterpret_cast<__nv_bfloat16*>(out),
        T, H, E, K);
  else
    combine_rows_kernel<float><<<blocks, kRowWarps * 32, 0, st>>>(
        reinterpret_cast<const float*>(rows), inv, router_indices, reinterpret_cast<const float*>(routing_weights),
        routing_cols, reinterpret_cast<float*>(out), T, H, E, K);
  return cudaGetLastError() == cudaSuccess ? YAMOE_OK : YAMOE_ERR_CUDA;
}

size_t yamoe_b200_ep_ctrl_bytes(int G, int E) {
  if (G <= 0 || E <= 0) return 0;
  return (size_t)EpCtrlLayout{G, E}.words() * sizeof(int32_t);
}

size_t yamoe_b200_ep_call_workspace_bytes(const yamoe_ep_ctx_t* ctx, int64_t T, int backward) {
  if (check_ep_ctx(ctx, false) || T < 0) return 0;
  return plan_ep_call(nullptr, *ctx, T, backward != 0).bytes;
}

int yamoe_b200_ep_forward(const yamoe_ep_ctx_t* ctx, const void* hidden_states, const int64_t* router_indices,
                          const void* routing_weights, int routing_cols, const void* gate_up_proj,
                          const void* gate_up_proj_bias, const void* down_proj, const void* down_proj_bias,
                          void* out, int64_t T, int64_t expert_capacity, void* workspace, size_t workspace_bytes,
                          void* stream) {
  int rc = check_ep_ctx(ctx, false);
  if (rc) return rc;
  if (T < 0 || expert_capacity < 0 || T * ctx->K > ctx->back_rows) return YAMOE_ERR_BAD_ARG;
  if (routing_cols != ctx->E && routing_cols != ctx->K) return YAMOE_ERR_BAD_ARG;
  if (T > 0 && (!hidden_states || !router_indices || !routing_weights || !out)) return YAMOE_ERR_BAD_ARG;
  if (!gate_up_proj || !gate_up_proj_bias || !down_proj || !down_proj_bias) return YAMOE_ERR_BAD_ARG;
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255) ||
      workspace_bytes < yamoe_b200_ep_call_workspace_bytes(ctx, T, 0))
    return YAMOE_ERR_WORKSPACE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (ctx->dtype == YAMOE_BF16)
    return ep_forward_impl<__nv_bfloat16>(*ctx, hidden_states, router_indices, routing_weights, routing_cols,
                                          gate_up_proj, gate_up_proj_bias, down_proj, down_proj_bias, out, T,
                                          expert_capacity, workspace, st);
  return ep_forward_impl<float>(*ctx, hidden_states, router_indices, routing_weights, routing_cols, gate_up_proj,
                                gate_up_proj_bias, down_proj, down_proj_bias, out, T, expert_capacity, workspace, st);
}

int yamoe_b200_ep_backward(const yamoe_ep_ctx_t* ctx, const void* grad_out, const void* hidden_states,
                           const int64_t* router_indices, const void* routing_weights, int routing_cols,
                           const void* gate_up_proj, const void* gate_up_proj_bias, const void* down_proj,
                           const void* down_proj_bias, void* d_hidden, void* d_routing, void* d_gate_up_proj,
                           void* d_gate_up_proj_bias, void* d_down_proj, void* d_down_proj_bias, int64_t T,
                           int64_t expert_capacity, void* workspace, size_t workspace_bytes, void* stream) {
  int rc = check_ep_ctx(ctx, true);
  if (rc) return rc;
  if (T < 0 || expert_capacity < 0 || T * ctx->K > ctx->back_rows) return YAMOE_ERR_BAD_ARG;
  if (routing_cols != ctx->E && routing_cols != ctx->K) return YAMOE_ERR_BAD_ARG;
  if (T > 0 && (!grad_out || !hidden_states || !router_indices || !routing_weights || !d_hidden || !d_routing))
    return YAMOE_ERR_BAD_ARG;
  if (!gate_up_proj || !gate_up_proj_bias || !down_proj || !down_proj_bias || !d_gate_up_proj ||
      !d_gate_up_proj_bias || !d_down_proj || !d_down_proj_bias)
    return YAMOE_ERR_BAD_ARG;
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255) ||
      workspace_bytes < yamoe_b200_ep_call_workspace_bytes(ctx, T, 1))
    return YAMOE_ERR_WORKSPACE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (ctx->dtype == YAMOE_BF16)
    return ep_backward_impl<__nv_bfloat16>(*ctx, grad_out, hidden_states, router_indices, routing_weights,
                                           routing_cols, gate_up_proj, gate_up_proj_bias, down_proj, down_proj_bias,
                                           d_hidden, d_routing, d_gate_up_proj, d_gate_up_proj_bias, d_down_proj,
                                           d_down_proj_bias, T, expert_capacity, workspace, st);
  return ep_backward_impl<float>(*ctx, grad_out, hidden_states, router_indices, routing_weights, routing_cols,
                                 gate_up_proj, gate_up_proj_bias, down_proj, down_proj_bias, d_hidden, d_routing,
                                 d_gate_up_proj, d_gate_up_proj_bias, d_down_proj, d_down_proj_bias, T,
                                 expert_capacity, workspace, st);
}

int yamoe_b200_ep_wait_probe(const int32_t* flags, int G, int32_t epoch, uint64_t wait_ns, int32_t* state,
                             int32_t* header, void* stream) {
  if (!flags || !state || !header || G <= 0 || G > 256) return YAMOE_ERR_BAD_ARG;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  YB_CUDA_OK(cudaMemcpyAsync(state + kEpStateEpoch, &epoch, sizeof(int32_t), cudaMemcpyHostToDevice, st));
  YB_CUDA_OK(cudaMemsetAsync(header, 0, 16 * sizeof(int32_t), st));
  ep_wait_kernel<<<1, 32, 0, st>>>(flags, G, state, header, (int)kStatusEpDispatchTimeout, wait_ns ? wait_ns : 1000000ull);
  return cudaGetLastError() == cudaSuccess ? YAMOE_OK : YAMOE_ERR_CUDA;
}

int yamoe_b200_router_topk(const void* router_logits, int64_t* router_indices, void* router_scores, int64_t T, int E,
                           int K, int dtype, void* stream) {
  if (dtype != YAMOE_F32 && dtype != YAMOE_BF16) return YAMOE_ERR_DTYPE;
  if (T < 0 || E <= 0 || K <= 0 || K > E || K > kRouterMaxK || E > 32 * kRouterMaxPerLane) return YAMOE_ERR_BAD_ARG;
  if (T == 0) return YAMOE_OK;
  if (!router_logits || !router_indices || !router_scores) return YAMOE_ERR_BAD_ARG;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == YAMOE_BF16) return launch_router_topk<__nv_bfloat16>(router_logits, router_indices, router_scores, T, E, K, st);
  return launch_router_topk<float>(router_logits, router_indices, router_scores, T, E, K, st);
}

size_t yamoe_b200_router_workspace_bytes(int64_t T, int E) {
  if (T < 0 || E <= 0) return 0;
  return router_workspace_bytes(T, E);
}

int yamoe_b200_router_forward(const void* hidden_states, const void* router_weight, const void* router_bias,
                              int64_t* router_indices, void* router_scores, int64_t T, int H, int E, int K, int dtype,
                              void* workspace, size_t workspace_bytes, void* stream) {
  if (dtype != YAMOE_F32 && dtype != YAMOE_BF16) return YAMOE_ERR_DTYPE;
  if (T < 0 || H <= 0 || H % 8 != 0 || E <= 0 || K <= 0 || K > E || K > kRouterMaxK || E > 32 * kRouterMaxPerLane)
    return YAMOE_ERR_BAD_ARG;
  if (T == 0) return YAMOE_OK;
  if (!hidden_states || !router_weight || !router_indices || !router_scores) return YAMOE_ERR_BAD_ARG;
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255) || workspace_bytes < router_workspace_bytes(T, E))
    return YAMOE_ERR_WORKSPACE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const bool tc = use_tcgen05(current_path(), dtype, H) && E <= 256;
  if (dtype == YAMOE_BF16)
    return launch_router_forward<__nv_bfloat16>(hidden_states, router_weight, router_bias, router_indices,
                                                router_scores, T, H, E, K, tc, workspace, st);
  return launch_router_forward<float>(hidden_states, router_weight, router_bias, router_indices, router_scores, T, H, E,
                                      K, false, workspace, st);
}

int yamoe_b200_experts_forward_saving(const void* hidden_states, const int64_t* router_indices,
                                      const void* routing_weights, int routing_cols, const void* gate_up_proj,
                                      const void* gate_up_proj_bias, const void* down_proj,
                                      const void* down_proj_bias, void* out, int64_t T, int H, int E, int K,
                                      int64_t expert_capacity, int dtype, void* saved, size_t saved_bytes,
                                      void* stream) {
  int rc = check_common(T, H, E, K, dtype);
  if (rc) return rc;
  if (routing_cols != E && routing_cols != K) return YAMOE_ERR_BAD_ARG;
  if (expert_capacity < 0) return YAMOE_ERR_BAD_ARG;
  if (T > 0 && (!hidden_states || !router_indices || !routing_weights || !out)) return YAMOE_ERR_BAD_ARG;
  if (!gate_up_proj || !gate_up_proj_bias || !down_proj || !down_proj_bias) return YAMOE_ERR_BAD_ARG;
  if (!saved || (reinterpret_cast<uintptr_t>(saved) & 255) ||
      saved_bytes < yamoe_b200_backward_workspace_bytes(T, H, E, K, dtype))
    return YAMOE_ERR_WORKSPACE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == YAMOE_BF16)
    return forward_train_impl<__nv_bfloat16>(hidden_states, router_indices, routing_weights, routing_cols,
                                             gate_up_proj, gate_up_proj_bias, down_proj, down_proj_bias, out, T, H, E,
                                             K, expert_capacity, dtype, saved, st);
  return forward_train_impl<float>(hidden_states, router_indices, routing_weights, routing_cols, gate_up_proj,
                                   gate_up_proj_bias, down_proj, down_proj_bias, out, T, H, E, K, expert_capacity,
                                   dtype, saved, st);
}

int yamoe_b200_experts_backward_saved(const void* grad_out, int grad_out_per_slot, const void* routing_weights,
                                      int routing_cols, const void* gate_up_proj, const void* down_proj,
                                      const void* down_proj_bias, void* d_hidden, void* d_routing,
                                      void* d_gate_up_proj, void* d_gate_up_proj_bias, void* d_down_proj,
                                      void* d_down_proj_bias, int64_t T, int H, int E, int K, int64_t expert_capacity,
                                      int dtype, void* saved, size_t saved_bytes, void* stream) {
  int rc = check_common(T, H, E, K, dtype);
  if (rc) return rc;
  if (routing_cols != E && routing_cols != K) return YAMOE_ERR_BAD_ARG;
  if (T > 0 && (!grad_out || !routing_weights || !d_hidden || !d_routing)) return YAMOE_ERR_BAD_ARG;
  if (!gate_up_proj || !down_proj || !down_proj_bias || !d_gate_up_proj || !d_gate_up_proj_bias || !d_down_proj ||
      !d_down_proj_bias)
    return YAMOE_ERR_BAD_ARG;
  if (!saved || (reinterpret_cast<uintptr_t>(saved) & 255) ||
      saved_bytes < yamoe_b200_backward_workspace_bytes(T, H, E, K, dtype))
    return YAMOE_ERR_WORKSPACE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == YAMOE_BF16)
    return backward_impl<__nv_bfloat16>(grad_out, grad_out_per_slot, nullptr, nullptr, routing_weights, routing_cols,
                                        gate_up_proj, nullptr, down_proj, down_proj_bias, d_hidden, d_routing,
                                        d_gate_up_proj, d_gate_up_proj_bias, d_down_proj, d_down_proj_bias, T, H, E, K,
                                        expert_capacity, dtype, saved, st, true);
  return backward_impl<float>(grad_out, grad_out_per_slot, nullptr, nullptr, routing_weights, routing_cols,
                              gate_up_proj, nullptr, down_proj, down_proj_bias, d_hidden, d_routing, d_gate_up_proj,
                              d_gate_up_proj_bias, d_down_proj, d_down_proj_bias, T, H, E, K, expert_capacity, dtype,
                              saved, st, true);
}

int yamoe_b200_binned_gather(const void* x, const int32_t* indices, const int32_t* bins, void* out, int64_t T, int H,
                             int E, int64_t C, int top_k, int dtype, void* stream) {
  if (dtype != YAMOE_F32 && dtype != YAMOE_BF16) return YAMOE_ERR_DTYPE;
  if (T < 0 || H <= 0 || E <= 0 || C < 0 || top_k <= 0 || (int64_t)E * C >= ((int64_t)1 << 31) || C >= ((int64_t)1 << 31))
    return YAMOE_ERR_BAD_ARG;
  if (C == 0) return YAMOE_OK;
  if (!x || !indices || !bins || !out) return YAMOE_ERR_BAD_ARG;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const size_t es = dtype == YAMOE_BF16 ? 2 : 4;
  const bool vec = (H * es) % 16 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  const unsigned blocks = (unsigned)ceil_div((int64_t)E * C, kRowWarps);
  auto launch = [&](auto tag, auto vtag) {
    using T_ = decltype(tag);
    binned_gather_kernel<T_, decltype(vtag)::value><<<blocks, kRowWarps * 32, 0, st>>>(
        reinterpret_cast<const T_*>(x), indices, bins, reinterpret_cast<T_*>(out), T, H, E, (int)C, top_k);
  };
  if (dtype == YAMOE_BF16) {
    if (vec) launch(__nv_bfloat16{}, std::true_type{}); else launch(__nv_bfloat16{}, std::false_type{});
  } else {
    if (vec) launch(float{}, std::true_type{}); else launch(float{}, std::false_type{});
  }
  return cudaGetLastError() == cudaSuccess ? YAMOE_OK : YAMOE_ERR_CUDA;
}

int yamoe_b200_binned_scatter(const void* src, const int32_t* indices, const int32_t* bins, const void* weights,
                              void* y, int64_t T, int H, int E, int64_t C, int top_k, int dtype, void* stream) {
  if (dtype != YAMOE_F32 && dtype != YAMOE_BF16) return YAMOE_ERR_DTYPE;
  if (T < 0 || H <= 0 || E <= 0 || C < 0 || top_k <= 0 || (int64_t)E * C >= ((int64_t)1 << 31) || C >= ((int64_t)1 << 31))
    return YAMOE_ERR_BAD_ARG;
  if (C == 0 || T == 0) return YAMOE_OK;
  if (!src || !indices || !bins || !y) return YAMOE_ERR_BAD_ARG;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const unsigned blocks = (unsigned)ceil_div((int64_t)E * C, kRowWarps);
  if (dtype == YAMOE_BF16)
    binned_scatter_kernel<__nv_bfloat16><<<blocks, kRowWarps * 32, 0, st>>>(
        reinterpret_cast<const __nv_bfloat16*>(src), indices, bins, reinterpret_cast<const __nv_bfloat16*>(weights),
        reinterpret_cast<__nv_bfloat16*>(y), T, H, E, (int)C, top_k);
  else
    binned_scatter_kernel<float><<<blocks, kRowWarps * 32, 0, st>>>(
        reinterpret_cast<const float*>(src), indices, bins, reinterpret_cast<const float*>(weights),
        reinterpret_cast<float*>(y), T, H, E, (int)C, top_k);
  return cudaGetLastError() == cudaSuccess ? YAMOE_OK : YAMOE_ERR_CUDA;
}

int yamoe_b200_index_select(void* out, const void* in, const int32_t* idx, int64_t N, int dtype, void* stream) {
  if (dtype != YAMOE_F32 && dtype != YAMOE_BF16) return YAMOE_ERR_DTYPE;
  if (N < 0) return YAMOE_ERR_BAD_ARG;
  if (N == 0) return YAMOE_OK;
  if (!out || !in || !idx) return YAMOE_ERR_BAD_ARG;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const unsigned blocks = (unsigned)ceil_div(N, 256);
  if (dtype == YAMOE_BF16)
    index_select_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(in), idx,
                                                               reinterpret_cast<__nv_bfloat16*>(out), N);
  else
    index_select_kernel<float><<<blocks, 256, 0, st>>>(reinterpret_cast<const float*>(in), idx,
                                                       reinterpret_cast<float*>(out), N);
  return cudaGetLastError() == cudaSuccess ? YAMOE_OK : YAMOE_ERR_CUDA;
}

#ifdef YB_PROF
int yamoe_b200_prof_read(unsigned long long* out16) {
  unsigned long long zero[16] = {};
  zero[8] = zero[10] = ~0ull;          // slots that hold a minimum
  if (cudaDeviceSynchronize() != cudaSuccess) return YAMOE_ERR_CUDA;
  if (cudaMemcpyFromSymbol(out16, g_prof, sizeof(zero)) != cudaSuccess) return YAMOE_ERR_CUDA;
  if (cudaMemcpyToSymbol(g_prof, zero, sizeof(zero)) != cudaSuccess) return YAMOE_ERR_CUDA;
  return YAMOE_OK;
}
#endif

int yamoe_b200_mbar_wait_probe(void* workspace, uint64_t limit_ns, void* stream) {
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255)) return YAMOE_ERR_WORKSPACE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  YB_CUDA_OK(cudaMemsetAsync(workspace, 0, 16 * sizeof(int32_t), st));
  mbar_wait_probe_kernel<<<1, 32, 0, st>>>(reinterpret_cast<int32_t*>(workspace), limit_ns ? limit_ns : 1000000ull);
  return cudaGetLastError() == cudaSuccess ? YAMOE_OK : YAMOE_ERR_CUDA;
}

int yamoe_b200_device_status(const void* workspace, void* stream, int32_t* status_out) {
  if (!workspace || !status_out) return YAMOE_ERR_BAD_ARG;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int32_t* header = reinterpret_cast<const int32_t*>(workspace);
  YB_CUDA_OK(cudaMemcpyAsync(status_out, header + kHdrStatus, sizeof(int32_t), cudaMemcpyDeviceToHost, st));
  YB_CUDA_OK(cudaStreamSynchronize(st));
  return YAMOE_OK;
}

}  // extern "C"
