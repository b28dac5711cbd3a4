// Shared definitions for the yamoe_b200 kernels: status codes, dtype traits, small helpers.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>
#include <stdint.h>

#include <atomic>
#include <cstdlib>
#include <utility>

#include "../../include/yamoe_b200.h"

namespace yb {

constexpr int kTileM = 128;          // row padding granularity of the expert-sorted buffers
constexpr float kAlpha = 1.702f;     // reference: csrc/moe.cpp:179
constexpr float kLimit = 7.0f;       // reference: csrc/moe.cpp:175

#define YB_CUDA_OK(expr)                                  \
  do {                                                    \
    cudaError_t _e = (expr);                              \
    if (_e != cudaSuccess) return YAMOE_ERR_CUDA;         \
  } while (0)

template <typename T> struct DT;
template <> struct DT<float> {
  static __device__ __forceinline__ float ld(const float* p) { return *p; }
  static __device__ __forceinline__ void st(float* p, float v) { *p = v; }
};
template <> struct DT<__nv_bfloat16> {
  static __device__ __forceinline__ float ld(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void st(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};

__host__ __device__ inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }
__host__ __device__ inline int64_t ceil_div(int64_t x, int64_t m) { return (x + m - 1) / m; }

// Upper bound on the number of kTileM-row tiles the padded, expert-sorted layout can use:
// every expert rounds its kept rows up to a multiple of kTileM.
inline int64_t max_row_tiles(int64_t S, int E) {
  int64_t ne = E < S ? E : S;
  return ceil_div(S, kTileM) + ne;
}

// Clamped SwiGLU of one (gate, up) pre-activation pair.  reference: csrc/moe.cpp:167-180.
__device__ __forceinline__ float glu_act(float g, float u) {
  g = fminf(g, kLimit);
  u = fminf(fmaxf(u, -kLimit), kLimit);
  const float s = __fdividef(1.0f, 1.0f + __expf(-kAlpha * g));
  return (u + 1.0f) * (g * s);
}

// ---- thread-block cluster helpers ---------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of `addr` (a shared::cta address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t smem_addr_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ float ld_shared_cluster_f32(uint32_t cluster_addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr) : "memory");
  return v;
}

// ---- programmatic dependent launch -----------------------------------------------------------
// A kernel launched with launch_pdl may start while its predecessor on the stream is still
// draining; it must execute pdl_wait() before touching any memory the predecessor writes or
// reads.  A predecessor calls pdl_trigger() as early as it likes: the dependent's CTAs then
// become resident as soon as SMs free up, and their set-up overlaps the predecessor's tail.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Measured on B200: between the two decode GEMV kernels it saves about 2 us per call (T = 1: 52.0 us
// against 53.8 us as a CUDA-graph replay), so that pair uses it by default; between the kernels of
// the grouped-GEMM forward it did not help (0.843 ms with, 0.814 ms without) and stays off.
// YAMOE_B200_PDL=1 turns it on everywhere, YAMOE_B200_PDL=0 off everywhere.
inline int pdl_setting() {
  static int v = []() {
    const char* env = std::getenv("YAMOE_B200_PDL");
    return env ? (std::atoi(env) != 0 ? 1 : 0) : -1;
  }();
  return v;
}
inline bool pdl_enabled(bool default_on = false) {
  const int v = pdl_setting();
  return v < 0 ? default_on : v != 0;
}

// Function attributes and device properties belong to one device; a process may drive several.
constexpr int kMaxDevices = 64;
inline int current_device_index() {
  int dev = 0;
  return cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < kMaxDevices ? dev : 0;
}
// A value remembered per device (for instance the dynamic shared memory a kernel was configured
// for); zero-initialised, so "0" has to mean "not set yet".
template <typename V>
struct PerDevice {
  std::atomic<V> v[kMaxDevices] = {};
  V get(int dev) const { return v[dev].load(std::memory_order_acquire); }
  void set(int dev, V x) { v[dev].store(x, std::memory_order_release); }
};

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_opt(bool default_on, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                  cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled(default_on) ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...);
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args&&... args) {
  return launch_pdl_opt(false, kern, grid, block, smem, st, std::forward<Args>(args)...);
}

// Routing tables kept at the head of every workspace (all int32 unless noted).
struct RouteTables {
  int32_t* header = nullptr;       // [16]: 0 ticket, 1 n_row_tiles, 2 rows_used, 3 dropped, 4 device status, 5 tile pairs
  int32_t* counts = nullptr;       // [E]
  int32_t* bins = nullptr;         // [E+1] inclusive prefix sums, bins[E] = 0
  int32_t* pad_off = nullptr;      // [E+1] first padded row of each expert, pad_off[E] = rows_used
  int32_t* block_counts = nullptr; // [nblk*E] per-block histogram, then exclusive prefix over blocks
  int32_t* tile_expert = nullptr;  // [max_row_tiles] expert owning each kTileM-row tile
  int32_t* pair_off = nullptr;     // [E+1] prefix sum of ceil(row tiles of e / 2): pairs of row tiles per expert
  int32_t* pair_expert = nullptr;  // [max_row_tiles] expert owning each pair of row tiles
  int32_t* sorted_values = nullptr;   // [S]
  int32_t* sorted_indices = nullptr;  // [S]
  int32_t* row_token = nullptr;    // [max_rows] token of each padded row, -1 for padding
  int32_t* row_flat = nullptr;     // [max_rows] flat position p = t*K + slot, -1 for padding
  float* row_weight = nullptr;     // [max_rows] routing weight of the row
  int32_t* flat_row = nullptr;     // [S] padded row of assignment p = t*K + slot, -1 when dropped
  int32_t* flat_pos = nullptr;     // [S] optional: position of assignment p in the sorted order (inverse of
                                   //     sorted_indices); the caller pre-fills it with -1
};

enum HeaderSlot { kHdrTicket = 0, kHdrRowTiles = 1, kHdrRowsUsed = 2, kHdrDropped = 3, kHdrStatus = 4, kHdrPairs = 5 };

// Optional CUDA-event bracket around one stage of the forward / backward sequence, for
// benchmarks that need the device time of a single kernel inside a full call.
struct StageEvents {
  std::atomic<int> stage{0};
  std::atomic<void*> start{nullptr}, stop{nullptr};
};
inline StageEvents g_events;
enum Stage { kStageNone = 0, kStageGateUp = 1, kStageDown = 2, kStageRoute = 3, kStageGather = 4,
             kStageEpDispatch = 5, kStageEpCombine = 6, kStageCombine = 7, kStageLast = 7 };

inline const char* stage_name(int stage) {
  static const char* const names[] = {"yamoe_b200", "yamoe_b200:gate_up", "yamoe_b200:down", "yamoe_b200:route",
                                      "yamoe_b200:gather", "yamoe_b200:ep_dispatch", "yamoe_b200:ep_combine",
                                      "yamoe_b200:combine"};
  return names[stage >= 0 && stage <= kStageLast ? stage : 0];
}

// Brackets the launches of one stage: an NVTX range on the host thread (a no-op unless a profiler
// that listens to NVTX is attached) and, when the stage was selected with
// yamoe_b200_set_stage_events, the caller's two events on the stream.
struct StageTimer {
  bool on;
  cudaStream_t st;
  StageTimer(int stage, cudaStream_t s) : on(g_events.stage.load() == stage && g_events.start.load()), st(s) {
    nvtxRangePushA(stage_name(stage));
    if (on) cudaEventRecord(reinterpret_cast<cudaEvent_t>(g_events.start.load()), st);
  }
  ~StageTimer() {
    if (on) cudaEventRecord(reinterpret_cast<cudaEvent_t>(g_events.stop.load()), st);
    nvtxRangePop();
  }
};

}  // namespace yb
