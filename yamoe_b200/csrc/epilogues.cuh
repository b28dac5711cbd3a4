// Epilogue functors shared by the SIMT and the tcgen05 grouped GEMMs.  A GEMM hands each
// functor a run of NV consecutive fp32 accumulator columns of one output row:
//
//     epi.template apply<NV>(expert, row, n0, v)       // v[i] = C[row][n0 + i]
//
// "row" is a row of the padded, expert-sorted layout for the row-tiled GEMMs (forward and
// data gradients) and a row of the per-expert output matrix for the weight-gradient GEMMs.
// n0 is a multiple of NV; NV is 4 (SIMT) or 32 (tcgen05).
#pragma once
#include "common.cuh"

namespace yb {

// ---- small vector load / store helpers (fp32 <-> storage dtype) ------------------------------
template <typename T, int N>
__device__ __forceinline__ void load_vec(const T* __restrict__ src, float (&out)[N]) {
  if constexpr (sizeof(T) == 4) {
    if constexpr (N % 4 == 0) {
#pragma unroll
      for (int i = 0; i < N / 4; ++i) {
        float4 q = __ldg(reinterpret_cast<const float4*>(src) + i);
        out[4 * i] = q.x; out[4 * i + 1] = q.y; out[4 * i + 2] = q.z; out[4 * i + 3] = q.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < N; ++i) out[i] = __ldg(reinterpret_cast<const float*>(src) + i);
    }
  } else {
    if constexpr (N % 8 == 0) {
#pragma unroll
      for (int i = 0; i < N / 8; ++i) {
        uint4 q = __ldg(reinterpret_cast<const uint4*>(src) + i);
        const uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          out[8 * i + 2 * j] = __uint_as_float(u[j] << 16);
          out[8 * i + 2 * j + 1] = __uint_as_float(u[j] & 0xffff0000u);
        }
      }
    } else if constexpr (N % 2 == 0) {
#pragma unroll
      for (int i = 0; i < N / 2; ++i) {
        uint32_t u = __ldg(reinterpret_cast<const uint32_t*>(src) + i);
        out[2 * i] = __uint_as_float(u << 16);
        out[2 * i + 1] = __uint_as_float(u & 0xffff0000u);
      }
    } else {
#pragma unroll
      for (int i = 0; i < N; ++i) out[i] = DT<T>::ld(src + i);
    }
  }
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&p);
}

template <typename T, int N>
__device__ __forceinline__ void store_vec(T* __restrict__ dst, const float (&v)[N]) {
  if constexpr (sizeof(T) == 4) {
    if constexpr (N % 4 == 0) {
#pragma unroll
      for (int i = 0; i < N / 4; ++i)
        reinterpret_cast<float4*>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    } else if constexpr (N % 2 == 0) {
#pragma unroll
      for (int i = 0; i < N / 2; ++i) reinterpret_cast<float2*>(dst)[i] = make_float2(v[2 * i], v[2 * i + 1]);
    } else {
#pragma unroll
      for (int i = 0; i < N; ++i) reinterpret_cast<float*>(dst)[i] = v[i];
    }
  } else {
    if constexpr (N % 8 == 0) {
#pragma unroll
      for (int i = 0; i < N / 8; ++i)
        reinterpret_cast<uint4*>(dst)[i] =
            make_uint4(pack_bf16x2(v[8 * i], v[8 * i + 1]), pack_bf16x2(v[8 * i + 2], v[8 * i + 3]),
                       pack_bf16x2(v[8 * i + 4], v[8 * i + 5]), pack_bf16x2(v[8 * i + 6], v[8 * i + 7]));
    } else if constexpr (N % 4 == 0) {
#pragma unroll
      for (int i = 0; i < N / 4; ++i)
        reinterpret_cast<uint2*>(dst)[i] =
            make_uint2(pack_bf16x2(v[4 * i], v[4 * i + 1]), pack_bf16x2(v[4 * i + 2], v[4 * i + 3]));
    } else if constexpr (N % 2 == 0) {
#pragma unroll
      for (int i = 0; i < N / 2; ++i) reinterpret_cast<uint32_t*>(dst)[i] = pack_bf16x2(v[2 * i], v[2 * i + 1]);
    } else {
#pragma unroll
      for (int i = 0; i < N; ++i) DT<T>::st(dst + i, v[i]);
    }
  }
}

// fp32 reduction into global memory, 16 bytes per instruction (red.global.add.v4.f32).
template <int N>
__device__ __forceinline__ void red_add_vec(float* __restrict__ dst, const float (&v)[N]) {
  static_assert(N % 4 == 0, "vector reduction works on groups of 4 floats");
#pragma unroll
  for (int i = 0; i < N / 4; ++i)
    atomicAdd(reinterpret_cast<float4*>(dst) + i, make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]));
}

// ---- gate_up epilogue: + bias, clamped SwiGLU on interleaved column pairs --------------------
// reference: csrc/moe.cpp:163-180.  Emits NV/2 activation columns per call.  Padding rows are
// written as exact zeros so that weight-gradient GEMMs may run over whole padded segments.
// Optional outputs for the backward recompute: `pre` (biased pre-activations, [rows,2H]) and
// `actw` (activation times routing weight).  Rows of actw are actw_ld >= H elements apart; the
// columns behind the H activations receive (w_row, 0, 0, ...), so that the weight-gradient GEMM
// whose transposed operand is actw also produces the down-projection bias gradient
// sum_r w_r * grad_y[r] in its output row H (reference: csrc/experts_backward.cu:277).
template <typename T>
struct EpiGlu {
  const T* bias;             // [E, 2H]
  T* act;                    // [rows, H]   (may be null when only actw/pre are wanted)
  T* actw;                   // [rows, actw_ld]   or null
  T* pre;                    // [rows, 2H]  or null
  const int32_t* row_token;
  const float* row_weight;
  int H;                     // activation columns (= N/2)
  int actw_ld;               // row pitch of actw (0 = H)

  template <int NV>
  __device__ __forceinline__ void apply(int e, int row, int n0, const float (&v)[NV]) const {
    static_assert(NV % 2 == 0, "gate/up pairs");
    float a[NV / 2], p[NV];
    const bool pad = row_token[row] < 0;
    if (pad) {
#pragma unroll
      for (int i = 0; i < NV; ++i) p[i] = 0.f;
#pragma unroll
      for (int i = 0; i < NV / 2; ++i) a[i] = 0.f;
    } else {
      float b[NV];
      load_vec<T, NV>(bias + (size_t)e * 2 * H + n0, b);
#pragma unroll
      for (int i = 0; i < NV; ++i) p[i] = v[i] + b[i];
      if (pre != nullptr) {
        // the backward pass re-derives the activation from the stored (rounded) pre-activations
        float q[NV];
        store_vec<T, NV>(pre + (size_t)row * 2 * H + n0, p);
        if constexpr (sizeof(T) == 2) {
#pragma unroll
          for (int i = 0; i < NV; ++i) q[i] = __bfloat162float(__float2bfloat16_rn(p[i]));
#pragma unroll
          for (int i = 0; i < NV; ++i) p[i] = q[i];
        }
      }
#pragma unroll
      for (int i = 0; i < NV / 2; ++i) a[i] = glu_act(p[2 * i], p[2 * i + 1]);
    }
    if (pad && pre != nullptr) store_vec<T, NV>(pre + (size_t)row * 2 * H + n0, p);
    if (act != nullptr) store_vec<T, NV / 2>(act + (size_t)row * H + n0 / 2, a);
    if (actw != nullptr) {
      // read past L1: on the expert-parallel path the weights are stored by other GPUs while this
      // kernel is already resident
      const float w = pad ? 0.f : __ldcg(row_weight + row);
      const int ld = actw_ld > 0 ? actw_ld : H;
#pragma unroll
      for (int i = 0; i < NV / 2; ++i) a[i] *= w;
      store_vec<T, NV / 2>(actw + (size_t)row * ld + n0 / 2, a);
      if (n0 == 0) {
        // (ld - H) is a multiple of 8 and rows are 16-byte aligned: eight columns per store
        float x[8] = {w, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int j = H; j < ld; j += 8) {
          store_vec<T, 8>(actw + (size_t)row * ld + j, x);
          x[0] = 0.f;
        }
      }
    }
  }
};

// ---- gate_up epilogue of the forward pass proper: only the activation is written ---------------
// Same arithmetic as EpiGlu.  It can leave the tcgen05 kernel in 128-byte pieces (kStagedRows), but
// for rows in local memory that measured slower (516 us against 465 us for the gate_up GEMM at
// T = 4096), so it is off.
template <typename T>
struct EpiGluAct {
  static constexpr bool kMayGather = true;     // the forward's gate_up GEMM may gather its A rows itself
  static constexpr bool kStagedRows = false;
  static constexpr int kOutPerChunk = 16;
  const T* bias;             // [E, 2H]
  T* act;                    // [rows, H]
  const int32_t* row_token;
  int H;

  // every row is written: padding rows as exact zeros (see EpiGlu)
  __device__ __forceinline__ T* row_ptr(int row) const { return act + (size_t)row * H; }

  template <int NV>
  __device__ __forceinline__ void values(int e, int row, int n0, const float (&v)[NV], float (&o)[NV / 2]) const {
    if (row_token[row] < 0) {
#pragma unroll
      for (int i = 0; i < NV / 2; ++i) o[i] = 0.f;
      return;
    }
    float b[NV];
    load_vec<T, NV>(bias + (size_t)e * 2 * H + n0, b);
#pragma unroll
    for (int i = 0; i < NV / 2; ++i) o[i] = glu_act(v[2 * i] + b[2 * i], v[2 * i + 1] + b[2 * i + 1]);
  }

  template <int NV>
  __device__ __forceinline__ void apply(int e, int row, int n0, const float (&v)[NV]) const {
    float a[NV / 2];
    values<NV>(e, row, n0, v, a);
    store_vec<T, NV / 2>(act + (size_t)row * H + n0 / 2, a);
  }
};

// ---- scatter-add epilogue: dst[token] += scale * (v + bias) ----------------------------------
// Forward combine (reference: csrc/moe.cpp:187 and csrc/scatter.cu:67-108) with BIAS=WEIGHT=true;
// data-gradient scatter into dHidden (reference: csrc/experts_backward.cu:92-124) with both false.
// Accumulates in fp32 with vector reductions; the order of the K additions per token is not fixed.
template <typename T, bool BIAS, bool WEIGHT>
struct EpiScatterAdd {
  const T* bias;             // [E, N] or null
  float* dst;                // [T, N] fp32
  const int32_t* row_token;
  const float* row_weight;
  int N;

  template <int NV>
  __device__ __forceinline__ void apply(int e, int row, int n0, const float (&v)[NV]) const {
    const int tok = row_token[row];
    if (tok < 0) return;
    float o[NV];
    if constexpr (BIAS) {
      load_vec<T, NV>(bias + (size_t)e * N + n0, o);
#pragma unroll
      for (int i = 0; i < NV; ++i) o[i] += v[i];
    } else {
#pragma unroll
      for (int i = 0; i < NV; ++i) o[i] = v[i];
    }
    if constexpr (WEIGHT) {
      const float w = row_weight[row];
#pragma unroll
      for (int i = 0; i < NV; ++i) o[i] *= w;
    }
    red_add_vec<NV>(dst + (size_t)tok * N + n0, o);
  }
};

// ---- data gradient of the down projection fused with the GLU backward -----------------------
// v = (grad_y[token] . W_d^T)[j0..j0+NV)  (not yet scaled by the routing weight).
// reference: csrc/experts_backward.cu:79-88 (routing-weight gradient), :285-305 (GLU backward).
// Adds sum_j v[j]*act[j] to gw_row[row], then writes the interleaved gradient of the
// pre-activations, scaled by the routing weight, to g_pre[row, 2*j0 .. 2*j0+2NV).
template <typename T>
struct EpiGluBackward {
  static constexpr bool kPrefetchTile = true;
  const T* pre;              // [rows, 2H] biased pre-activations from the recompute
  T* g_pre;                  // [rows, 2H]
  float* gw_row;             // [rows]
  const int32_t* row_token;
  const float* row_weight;
  int H;

  // the 2*ncols pre-activations this row's epilogue will read for output columns n0 .. n0+ncols
  __device__ __forceinline__ void prefetch_tile(int row, int n0, int ncols) const {
    if (row_token[row] < 0) return;
    const char* p = reinterpret_cast<const char*>(pre + (size_t)row * 2 * H + 2 * n0);
    for (int b = 0; b < 2 * ncols * (int)sizeof(T); b += 128)
      asm volatile("prefetch.global.L2 [%0];" ::"l"(p + b));
  }

  template <int NV>
  __device__ __forceinline__ void apply(int /*e*/, int row, int n0, const float (&v)[NV]) const {
    float out[2 * NV];
    if (row_token[row] < 0) {
#pragma unroll
      for (int i = 0; i < 2 * NV; ++i) out[i] = 0.f;
    } else {
      float p[2 * NV];
      load_vec<T, 2 * NV>(pre + (size_t)row * 2 * H + 2 * n0, p);
      const float w = row_weight[row];
      float dot = 0.f;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const float pg = p[2 * i], pu = p[2 * i + 1];
        const float gc = fminf(pg, kLimit);
        const float uc = fminf(fmaxf(pu, -kLimit), kLimit);
        const float s = __fdividef(1.0f, 1.0f + __expf(-kAlpha * gc));
        const float gate_act = gc * s;
        dot += v[i] * (uc + 1.0f) * gate_act;
        const float gi = w * v[i];
        float gu = gi * gate_act;
        float gg = gi * (uc + 1.0f) * (s + gc * s * (1.0f - s) * kAlpha);
        if (pg > kLimit) gg = 0.f;
        if (pu > kLimit || pu < -kLimit) gu = 0.f;
        out[2 * i] = gg;
        out[2 * i + 1] = gu;
      }
      atomicAdd(gw_row + row, dot);
    }
    store_vec<T, 2 * NV>(g_pre + (size_t)row * 2 * H + 2 * n0, out);
  }
};

// ---- plain store of a per-expert output matrix (weight gradients) ----------------------------
// reference: csrc/experts_backward.cu:281-282, :311.  Rows beyond M are skipped.
template <typename T>
struct EpiStore {
  T* C;                      // [E, M, N]
  int M, N;

  template <int NV>
  __device__ __forceinline__ void apply(int e, int row, int n0, const float (&v)[NV]) const {
    if (row >= M) return;
    store_vec<T, NV>(C + ((size_t)e * M + row) * N + n0, v);
  }
};

// ---- weight gradient with the bias gradient riding along ------------------------------------
// The transposed operand of the GEMM carries one extra column (see gather_rows_kernel / EpiGlu),
// so output row M holds the bias gradient: rows < M go to C, row M to bias_out, later rows nowhere.
template <typename T>
struct EpiStoreBias {
  T* C;                      // [E, M, N]
  T* bias_out;               // [E, N]
  int M, N;

  template <int NV>
  __device__ __forceinline__ void apply(int e, int row, int n0, const float (&v)[NV]) const {
    if (row < M) store_vec<T, NV>(C + ((size_t)e * M + row) * N + n0, v);
    else if (row == M) store_vec<T, NV>(bias_out + (size_t)e * N + n0, v);
  }
};

// ---- down-projection epilogue for the two-step combine: y[row] = w_row * (v + bias) ------------
// reference: csrc/moe.cpp:187 and the per-row scaling of csrc/scatter.cu:98-106.  The K rows of a
// token are summed afterwards by combine_padded_kernel; padding rows are never read and are skipped.
template <typename T>
struct EpiWeightedRows {
  // Parking the rows in shared memory and storing 128-byte pieces (kStagedRows, see umma_gemm.cuh)
  // pays when the rows cross NVLink; for local rows it measured slower (down GEMM 272 us against
  // 258 us at T = 4096), because L2 merges the 16-byte pieces anyway and the epilogue gets longer.
  static constexpr bool kStagedRows = false;
  static constexpr int kOutPerChunk = 32;
  const T* bias;             // [E, N]
  T* y;                      // [rows, N]
  const int32_t* row_token;
  const float* row_weight;
  int N;

  __device__ __forceinline__ T* row_ptr(int row) const { return row_token[row] < 0 ? nullptr : y + (size_t)row * N; }

  template <int NV>
  __device__ __forceinline__ void values(int e, int row, int n0, const float (&v)[NV], float (&o)[NV]) const {
    if (row_token[row] < 0) {
#pragma unroll
      for (int i = 0; i < NV; ++i) o[i] = 0.f;
      return;
    }
    load_vec<T, NV>(bias + (size_t)e * N + n0, o);
    const float w = row_weight[row];
#pragma unroll
    for (int i = 0; i < NV; ++i) o[i] = w * (o[i] + v[i]);
  }

  template <int NV>
  __device__ __forceinline__ void apply(int e, int row, int n0, const float (&v)[NV]) const {
    if (row_token[row] < 0) return;
    float o[NV];
    load_vec<T, NV>(bias + (size_t)e * N + n0, o);
    const float w = row_weight[row];
#pragma unroll
    for (int i = 0; i < NV; ++i) o[i] = w * (o[i] + v[i]);
    store_vec<T, NV>(y + (size_t)row * N + n0, o);
  }
};

// ---- plain store of row-tiled output C[row, n0..] (batched matmul sub-operator) --------------
template <typename T>
struct EpiStoreRows {
  T* C;                      // [rows, N]
  int N;

  template <int NV>
  __device__ __forceinline__ void apply(int /*e*/, int row, int n0, const float (&v)[NV]) const {
    store_vec<T, NV>(C + (size_t)row * N + n0, v);
  }
};

}  // namespace yb
