/*
 * yamoe_b200 — C ABI of the B200 (sm_100a) expert forward / backward library.
 *
 * Plain pointers and sizes only: no torch types cross this boundary.  Every pointer is a
 * device pointer unless stated otherwise.  The library never allocates or frees device
 * memory (all scratch comes from the caller-provided workspace, 256-byte aligned), never
 * keeps a pointer after a call returns, performs no host/device synchronisation and
 * enqueues all work on the stream it is given.
 *
 * Every entry point returns YAMOE_OK (0) or a negative yamoe_status_t.
 *
 * The comments cite the interface of the reference project (drbh/yamoe) that each entry
 * point replaces, as path:line within that project.
 */
#ifndef YAMOE_B200_H_
#define YAMOE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  YAMOE_OK = 0,
  YAMOE_ERR_BAD_ARG = -1,        /* null pointer, non-positive size, H not a multiple of 8, ... */
  YAMOE_ERR_WORKSPACE = -2,      /* workspace pointer null / misaligned / too small          */
  YAMOE_ERR_DTYPE = -3,          /* dtype is not YAMOE_F32 or YAMOE_BF16                      */
  YAMOE_ERR_CUDA = -4,           /* a CUDA runtime / driver call failed (launch, tensor map)  */
  YAMOE_ERR_UNSUPPORTED = -5,    /* valid request this build cannot serve                     */
  YAMOE_ERR_DEVICE_TIMEOUT = -6, /* a bounded device-side wait gave up (see device status)    */
  YAMOE_ERR_STATIC_SCRATCH = -7  /* yamoe_b200_route_static: request exceeds its fixed scratch */
} yamoe_status_t;

typedef enum { YAMOE_F32 = 0, YAMOE_BF16 = 1 } yamoe_dtype_t;

/* Path selection for the GEMMs.  AUTO picks tcgen05 for bf16 when shapes allow, the GEMV path
 * for decode-sized bf16 token counts, and the SIMT path otherwise (fp32 always). */
typedef enum {
  YAMOE_PATH_AUTO = 0,
  YAMOE_PATH_SIMT = 1,     /* CUDA-core FFMA grouped GEMM, fp32 accumulate (any dtype)     */
  YAMOE_PATH_TCGEN05 = 2,  /* tcgen05 / TMEM / TMA grouped GEMM (bf16 only)                */
  YAMOE_PATH_GEMV = 3      /* weight-streaming GEMV path for small token counts (bf16)     */
} yamoe_path_t;

/* Library version (major*10000 + minor*100 + patch). */
int yamoe_b200_version(void);

/* Human-readable name of a status code; never NULL. */
const char *yamoe_b200_status_string(int status);

/* Process-wide path override used by tests and the benchmark; returns the previous value. */
int yamoe_b200_set_path(int path);

/* Profiling aid, process-wide and not thread-safe: while `stage` is non-zero, every forward call
 * records `start_event` / `stop_event` (cudaEvent_t) on its stream immediately before / after
 * the kernels of that stage: 1 gate_up GEMM, 2 down GEMM, 3 routing, 4 row gather, 5 the
 * expert-parallel call up to the arrival of all rows (local sort, count exchange, dispatch, wait),
 * 6 its end (return signal, wait for all owners, combine), 7 the combine of the single-GPU forward;
 * 0 disables.  The same stages are NVTX ranges ("yamoe_b200:<stage>") on the calling thread. */
int yamoe_b200_set_stage_events(void *start_event, void *stop_event, int stage);

/* ---------------------------------------------------------------------------------------------
 * Routing: stable sort of the S = T*K (token, slot) assignments by expert id, per-expert
 * histogram and inclusive prefix sum.  Replaces sort_cuda (csrc/sort.cu:61-91) and
 * bincount_cumsum_cuda (csrc/bincount_cumsum.cu:58-98) as used at csrc/moe.cpp:141-144.
 *
 *   router_indices  int64 [T*K]        expert id of assignment p = t*K + slot
 *   sorted_values   int32 [T*K]  out   expert ids in ascending order
 *   sorted_indices  int32 [T*K]  out   flat position p of each sorted entry (ties: ascending p)
 *   bins            int32 [E+1]  out   bins[e] = number of assignments with id <= e; bins[E] = 0
 *   counts          int32 [E]    out   per-expert histogram (may be NULL)
 * Bit-exact and deterministic.  Ids outside [0,E) are dropped from all outputs: the kept entries
 * come first and the remaining entries of sorted_values / sorted_indices read -1.
 * ------------------------------------------------------------------------------------------- */
size_t yamoe_b200_route_workspace_bytes(int64_t T, int E, int K);
int yamoe_b200_route(const int64_t *router_indices, int32_t *sorted_values, int32_t *sorted_indices,
                     int32_t *bins, int32_t *counts, int64_t T, int E, int K,
                     void *workspace, size_t workspace_bytes, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Routing for callers that cannot hand over a workspace.  This entry point has no counterpart in
 * the reference project.
 *
 * Same inputs, outputs and results as yamoe_b200_route, but it takes no workspace: the few
 * hundred KB the routing kernels need besides their outputs (a ticket/status header, the padded
 * offsets and the per-block histograms) live in a fixed 1 MiB array inside the library image.  It
 * is meant for hosts that must not touch an allocator at the point of the call: a serving loop
 * whose memory pool is frozen after start-up, a plugin interface that only passes input and output
 * buffers, a runtime that forbids cudaMalloc on its worker threads.  The call itself performs no
 * cudaMalloc / cudaFree and uses no allocating library routine.
 *
 * Limits and rules:
 *   - yamoe_b200_route_static_scratch_needed(T, E, K) must not exceed 1 MiB (1 048 576 bytes),
 *     roughly ceil(T*K/2048) * E * 4 bytes; larger requests fail with YAMOE_ERR_STATIC_SCRATCH
 *     and launch nothing.  E <= 1024 as everywhere else.
 *   - The array exists once per GPU and costs 1 MiB of device memory on every GPU that loads the
 *     library, until the process exits.
 *   - The first call on each device looks up the array's device address (with that device
 *     current) and caches it; make that first call outside of any stream capture.
 *   - All calls on a device share the array and it keeps the previous call's contents; the part
 *     that must start at zero is cleared on `stream` at the start of every call.  Two calls whose
 *     GPU work can overlap (different streams without ordering) race on it: serialise them.
 * ------------------------------------------------------------------------------------------- */
size_t yamoe_b200_route_static_scratch_needed(int64_t T, int E, int K);
int yamoe_b200_route_static(const int64_t *router_indices, int32_t *sorted_values, int32_t *sorted_indices,
                            int32_t *bins, int32_t *counts, int64_t T, int E, int K, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Expert forward.  Replaces experts_cuda (csrc/moe.cpp:45-223; schema
 * torch-ext/torch_binding.cpp:58-69).
 *
 *   hidden_states     dtype [T,H]
 *   router_indices    int64 [T,K]
 *   routing_weights   dtype [T,routing_cols], routing_cols == E (dense) or == K (per slot)
 *   gate_up_proj      dtype [E,H,2H]   gate = even columns, up = odd columns
 *   gate_up_proj_bias dtype [E,2H]
 *   down_proj         dtype [E,H,H]
 *   down_proj_bias    dtype [E,H]
 *   out               dtype [T,H]      fully overwritten
 *   expert_capacity   rows kept per expert: the first min(n_e, capacity) assignments of expert e
 *                     in stable sorted order (csrc/gather.cu:18-26, csrc/scatter.cu:78-96)
 * ------------------------------------------------------------------------------------------- */
size_t yamoe_b200_forward_workspace_bytes(int64_t T, int H, int E, int K, int dtype);
int yamoe_b200_experts_forward(const void *hidden_states, const int64_t *router_indices,
                               const void *routing_weights, int routing_cols,
                               const void *gate_up_proj, const void *gate_up_proj_bias,
                               const void *down_proj, const void *down_proj_bias, void *out,
                               int64_t T, int H, int E, int K, int64_t expert_capacity, int dtype,
                               void *workspace, size_t workspace_bytes, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Expert backward.  Replaces experts_backward_cuda (csrc/experts_backward.cu:126-341; schema
 * torch-ext/torch_binding.cpp:71-83).  Gradients are written in the order the reference
 * returns them (csrc/experts_backward.cu:340); every output is fully overwritten.
 *
 *   grad_out          dtype, T*H elements, or T*K*H elements (grad_out_per_slot != 0) that are
 *                     summed over K first (csrc/experts_backward.cu:224-228)
 *   d_hidden          dtype [T,H]
 *   d_routing         dtype [T,routing_cols]; zero outside selected, kept entries.  The value is
 *                     the autograd gradient <grad_out[t], y_e[t]>; the reference applies the sort
 *                     permutation twice here (csrc/experts_backward.cu:261-264) and is not followed.
 *   d_gate_up_proj    dtype [E,H,2H];  d_gate_up_proj_bias dtype [E,2H]
 *   d_down_proj       dtype [E,H,H];   d_down_proj_bias    dtype [E,H]
 * ------------------------------------------------------------------------------------------- */
size_t yamoe_b200_backward_workspace_bytes(int64_t T, int H, int E, int K, int dtype);
int yamoe_b200_experts_backward(const void *grad_out, int grad_out_per_slot,
                                const void *hidden_states, const int64_t *router_indices,
                                const void *routing_weights, int routing_cols,
                                const void *gate_up_proj, const void *gate_up_proj_bias,
                                const void *down_proj, const void *down_proj_bias,
                                void *d_hidden, void *d_routing, void *d_gate_up_proj,
                                void *d_gate_up_proj_bias, void *d_down_proj, void *d_down_proj_bias,
                                int64_t T, int H, int E, int K, int64_t expert_capacity, int dtype,
                                void *workspace, size_t workspace_bytes, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Batched per-expert matmul on a uniform layout (expert e owns rows [e*C, (e+1)*C) of x).
 * Replaces batch_mm (csrc/batch_mm.cu:7-31; schema torch-ext/torch_binding.cpp:50-56), and
 * unlike it honours the transposed-weight flag.  `mode`:
 *   0  out[e] [C,N] = x[e] [C,K] @ weights[e] [K,N]
 *   1  out[e] [C,N] = x[e] [C,K] @ weights[e]^T,  weights [E,N,K]          (trans_b)
 *   2  out[e] [M,N] = x[e]^T @ weights[e],  x [E,C,M], weights [E,C,N]     (weight gradient)
 * C must be a multiple of 128 and N, K (M for mode 2) multiples of 64.  fp32 accumulation,
 * output in `dtype`.
 * ------------------------------------------------------------------------------------------- */
size_t yamoe_b200_batch_mm_workspace_bytes(int E, int C);
int yamoe_b200_batch_mm(const void *x, const void *weights, void *out, int E, int C, int M, int N, int K,
                        int mode, int dtype, void *workspace, size_t workspace_bytes, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Expert-parallel helpers (no counterpart in the reference, which is single-GPU).  Around an
 * all-to-all exchange of rows between the ranks that own tokens and the ranks that own experts:
 *   permute_rows   dst[j,:] = src[sorted_indices[j] / K, :]          rows in expert-sorted order
 *   combine_rows   out[t,:] = sum_k w[t,k] * rows[pos(t*K+k), :]      pos = inverse of sorted_indices
 * `sorted_indices` is the output of yamoe_b200_route (n_sorted entries; assignments missing from
 * it contribute nothing; entries that are negative or not below n_src*K -- the -1 tail that route
 * leaves for dropped ids -- give a zero row in permute_rows and are skipped by combine_rows).
 * `src` has n_src rows.  combine_rows needs a workspace of T*K*4 bytes and accumulates in fp32
 * in slot order, so it is deterministic.  The weights come from routing_weights[t, expert] when
 * routing_cols == E and from routing_weights[t, k] when routing_cols == K, as in the forward op.
 * ------------------------------------------------------------------------------------------- */
int yamoe_b200_permute_rows(const void *src, int64_t n_src, const int32_t *sorted_indices, void *dst, int64_t S,
                            int H, int K, int dtype, void *stream);
int yamoe_b200_combine_rows(const void *rows, const int32_t *sorted_indices, int64_t n_sorted,
                            const int64_t *router_indices, const void *routing_weights, int routing_cols,
                            void *out, int64_t T, int H, int E, int K, int dtype, void *workspace,
                            size_t workspace_bytes, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Expert parallelism as ONE call per rank (no counterpart in the reference, which is single-GPU).
 * G ranks, rank r owns experts [r*E/G, (r+1)*E/G) and a shard of the tokens.  Token rows travel to
 * the expert owners and result rows back as peer stores over NVLink; every offset is derived on
 * the device from the per-rank expert counts, and the count exchange and the phase boundaries are
 * flags in peer-writable memory instead of host-issued collectives: a call enqueues a fixed chain
 * of kernels on `stream` and nothing else -- no NCCL call, no host synchronisation, no split
 * sizes.  Kernels only STORE to peer memory; every wait polls local memory.
 *
 * Buffers (each allocated by every rank with the same size and made peer-accessible; the
 * peer_* members are DEVICE arrays of G pointers, index = rank, own buffer included):
 *   recv_x [max_rows, H] dtype   rows received for this rank's experts (padded expert-sorted layout)
 *   back   [back_rows, H] dtype  result rows of this rank's own assignments, in its sorted order
 *   ctrl   yamoe_b200_ep_ctrl_bytes(G, E) bytes, zeroed once before the first call on any rank
 *   recv_g [max_rows, H] dtype, recv_w [max_rows] fp32, back_w [back_rows] fp32   (backward only)
 * `state` is 256 bytes of this rank's private device memory, zeroed once; it holds the call
 * counter (epoch) that the flags carry.  All ranks must make the same sequence of calls.
 * max_rows must be a multiple of 128 and at least (assignments of all ranks that can land on one
 * rank) + 128 * E/G; a call whose rows would not fit stores nothing and reports device status 7.
 *
 * Every device-side wait (for the counts, for the dispatched rows, for the returned rows) polls
 * this GPU's own memory and gives up after `wait_ns` nanoseconds (0 = 2 s): the call then leaves
 * device status 4, 5 or 6 in the workspace header (yamoe_b200_device_status), its outputs are
 * invalid, and the GPU and all buffers stay usable.
 * Received receive-buffer padding rows must hold finite values for the backward pass: zero
 * recv_x and recv_g once before the first call.
 * ------------------------------------------------------------------------------------------- */
typedef struct {
  int32_t G, rank, E, K, H, dtype;
  int64_t max_rows;   /* rows of recv_x / recv_g / recv_w */
  int64_t back_rows;  /* rows of back / back_w; every call needs T*K <= back_rows */
  void *const *peer_recv_x, *const *peer_recv_g, *const *peer_recv_w;
  void *const *peer_back, *const *peer_back_w, *const *peer_ctrl;
  void *recv_x, *recv_g, *recv_w, *back, *back_w, *ctrl; /* this rank's own buffers */
  void *state;
  uint64_t wait_ns;
} yamoe_ep_ctx_t;

size_t yamoe_b200_ep_ctrl_bytes(int G, int E);
size_t yamoe_b200_ep_call_workspace_bytes(const yamoe_ep_ctx_t *ctx, int64_t T, int backward);
/* out [T,H] = this rank's token shard through all E experts; arguments as yamoe_b200_experts_forward
 * with the four weight tensors holding this rank's E/G experts only. */
int yamoe_b200_ep_forward(const yamoe_ep_ctx_t *ctx, const void *hidden_states, const int64_t *router_indices,
                          const void *routing_weights, int routing_cols, const void *gate_up_proj,
                          const void *gate_up_proj_bias, const void *down_proj, const void *down_proj_bias,
                          void *out, int64_t T, int64_t expert_capacity, void *workspace, size_t workspace_bytes,
                          void *stream);
/* Gradients as yamoe_b200_experts_backward (grad_out [T,H]); weight and bias gradients cover this
 * rank's E/G experts and stay here (experts are not replicated, so nothing is all-reduced). */
int yamoe_b200_ep_backward(const yamoe_ep_ctx_t *ctx, const void *grad_out, const void *hidden_states,
                           const int64_t *router_indices, const void *routing_weights, int routing_cols,
                           const void *gate_up_proj, const void *gate_up_proj_bias, const void *down_proj,
                           const void *down_proj_bias, void *d_hidden, void *d_routing, void *d_gate_up_proj,
                           void *d_gate_up_proj_bias, void *d_down_proj, void *d_down_proj_bias, int64_t T,
                           int64_t expert_capacity, void *workspace, size_t workspace_bytes, void *stream);
/* Test aid for the give-up path: sets the epoch in `state` to `epoch`, clears `header` (16 int32) and
 * runs the one-warp wait of the expert-parallel path on `flags[0..G)` with the given limit (0 = 1 ms).
 * header[4] is 5 afterwards if some flag never reached `epoch`, else 0.  One GPU, no peer involved. */
int yamoe_b200_ep_wait_probe(const int32_t *flags, int G, int32_t epoch, uint64_t wait_ns, int32_t *state,
                             int32_t *header, void *stream);

/* ---------------------------------------------------------------------------------------------
 * The reference's three small sub-operators on its padded [E, C, H] layout.  The expert op of this
 * library never builds that layout; these are for callers of the standalone operators.
 *   binned_gather   replaces gather_cuda        (csrc/gather.cu:68-109, torch-ext/torch_binding.cpp:9-17)
 *                   out[e, i, :] = x[indices[bins[e-1] + i] / top_k, :] for i < min(count_e, C), else 0
 *   binned_scatter  replaces scatter_cuda       (csrc/scatter.cu:110-147, torch_binding.cpp:19-29)
 *                   y[tok, :] += weights[bins[e-1] + i] * src[e, i, :]; weights may be NULL (= 1);
 *                   y is accumulated into, atomically, as in the reference
 *   index_select    replaces index_select_out_cuda (csrc/index_select.cu:18-52, torch_binding.cpp:44-48)
 *                   out[i] = in[idx[i]]
 * indices: int32 [S] flat (token, slot) positions in expert-sorted order; bins: int32 [E] inclusive
 * prefix sums of the per-expert counts.
 * ------------------------------------------------------------------------------------------- */
int yamoe_b200_binned_gather(const void *x, const int32_t *indices, const int32_t *bins, void *out, int64_t T,
                             int H, int E, int64_t C, int top_k, int dtype, void *stream);
int yamoe_b200_binned_scatter(const void *src, const int32_t *indices, const int32_t *bins, const void *weights,
                              void *y, int64_t T, int H, int E, int64_t C, int top_k, int dtype, void *stream);
int yamoe_b200_index_select(void *out, const void *in, const int32_t *idx, int64_t N, int dtype, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Router tail of the layer that calls the expert op.  Replaces the top-k / softmax / scatter
 * chain of Yamoe.forward (torch-ext/yamoe/layers.py:136-149):
 *   router_indices [T,K] int64  = experts of the K largest logits, descending
 *   router_scores  [T,E] dtype  = softmax over those K logits at the selected columns, 0 elsewhere
 * E <= 1024, K <= 32.  Ties between equal logits go to the lower expert id.
 * ------------------------------------------------------------------------------------------- */
int yamoe_b200_router_topk(const void *router_logits, int64_t *router_indices, void *router_scores, int64_t T,
                           int E, int K, int dtype, void *stream);

/* Whole router of the layer in front of the expert op, replacing the chain
 * F.linear -> topk -> softmax -> zeros_like().scatter_() of Yamoe.forward
 * (torch-ext/yamoe/layers.py:126-149; oracle torch-ext/yamoe/vendored/gpt_oss_mlp.py:119-139):
 *   logits = hidden_states [T,H] @ router_weight [E,H]^T + router_bias [E]   (rounded to `dtype`)
 * followed by what yamoe_b200_router_topk does.  ONE kernel in two cases: up to 64 tokens (either
 * dtype; a warp per (token, expert) dot product, the CTA finishing a token last selects), and bf16
 * with H a multiple of 64, E <= 256 and K <= 8 (a tcgen05 GEMM whose epilogue does the top-k,
 * softmax and scatter).  Otherwise a GEMM and the top-k kernel run back to back.  router_bias may
 * be NULL.  The workspace (256-byte aligned, yamoe_b200_router_workspace_bytes) holds a status
 * header, per-token tickets and the logits or the selection state. */
size_t yamoe_b200_router_workspace_bytes(int64_t T, int E);
int yamoe_b200_router_forward(const void *hidden_states, const void *router_weight, const void *router_bias,
                              int64_t *router_indices, void *router_scores, int64_t T, int H, int E, int K,
                              int dtype, void *workspace, size_t workspace_bytes, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Training pair that keeps activations instead of recomputing them (the reference's autograd
 * wrapper saves only the seven inputs and recomputes the whole forward in backward,
 * torch-ext/yamoe/layers.py:38-46, csrc/experts_backward.cu:176-199).
 *   yamoe_b200_experts_forward_saving   same result as yamoe_b200_experts_forward; `saved` (sized by
 *       yamoe_b200_backward_workspace_bytes, 256-byte aligned) receives the routing tables, the
 *       gathered rows, the biased pre-activations and the weighted activations
 *   yamoe_b200_experts_backward_saved   same gradients as yamoe_b200_experts_backward, reading them
 *       from `saved` instead of running routing, gather and the gate_up GEMM again.  `saved` must
 *       be untouched since the matching forward call with the same T, H, E, K, capacity and dtype;
 *       it is also the scratch of this call and is consumed by it.
 * ------------------------------------------------------------------------------------------- */
int yamoe_b200_experts_forward_saving(const void *hidden_states, const int64_t *router_indices,
                                      const void *routing_weights, int routing_cols, const void *gate_up_proj,
                                      const void *gate_up_proj_bias, const void *down_proj,
                                      const void *down_proj_bias, void *out, int64_t T, int H, int E, int K,
                                      int64_t expert_capacity, int dtype, void *saved, size_t saved_bytes,
                                      void *stream);
int yamoe_b200_experts_backward_saved(const void *grad_out, int grad_out_per_slot, const void *routing_weights,
                                      int routing_cols, const void *gate_up_proj, const void *down_proj,
                                      const void *down_proj_bias, void *d_hidden, void *d_routing,
                                      void *d_gate_up_proj, void *d_gate_up_proj_bias, void *d_down_proj,
                                      void *d_down_proj_bias, int64_t T, int H, int E, int K, int64_t expert_capacity,
                                      int dtype, void *saved, size_t saved_bytes, void *stream);

/* Device status word of the last forward/backward call that used `workspace`: 0 when every
 * bounded device-side wait completed, otherwise a code naming the wait that gave up.  Reads
 * 4 bytes from the device with cudaMemcpyAsync on `stream` and synchronises that stream. */
int yamoe_b200_device_status(const void *workspace, void *stream, int32_t *status_out);

/* Test aid for the give-up path of the grouped GEMM's pipeline waits: clears the 64-byte header at
 * the start of `workspace` (256-byte aligned, >= 64 bytes) and runs one thread that waits, for at most
 * `limit_ns` nanoseconds (0 = 1 ms), on a shared-memory barrier nothing arrives at, using the same
 * bounded wait as the GEMM kernels.  yamoe_b200_device_status on `workspace` then returns 1. */
int yamoe_b200_mbar_wait_probe(void *workspace, uint64_t limit_ns, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* YAMOE_B200_H_ */
