// Thin torch binding over the C ABI: the operators `yamoe_b200::experts` and
// `yamoe_b200::experts_backward` with the reference's schemas
// (torch-ext/torch_binding.cpp:58-83), implemented as argument checks, output / workspace
// allocation through torch, and one call into libyamoe_b200.so with raw pointers and torch's
// current stream.  Takes the place of torch-ext/torch_binding.cpp + csrc/moe.cpp:45-136 of the
// reference; the preconditions and their messages follow csrc/moe.cpp:58-96.
//
// Built separately from the CUDA library (host compiler only) and loaded with
// torch.ops.load_library; when it is absent the same operators are registered from Python
// (yamoe_b200/ops.py), which costs some tens of microseconds more per call.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <cstdlib>
#include <vector>

#include "../../include/yamoe_b200.h"

namespace {

struct Shape {
  int64_t T;
  int H, E, K, dtype;
};

Shape validate(const at::Tensor& hidden_states, const at::Tensor& router_indices, const at::Tensor& routing_weights,
               const at::Tensor& gate_up_proj, const at::Tensor& gate_up_proj_bias, const at::Tensor& down_proj,
               const at::Tensor& down_proj_bias, int64_t num_experts, int64_t top_k) {
  const at::Tensor* tensors[] = {&hidden_states, &router_indices, &routing_weights, &gate_up_proj,
                                 &gate_up_proj_bias, &down_proj, &down_proj_bias};
  const char* names[] = {"hidden_states", "router_indices", "routing_weights", "gate_up_proj",
                         "gate_up_proj_bias", "down_proj", "down_proj_bias"};
  for (int i = 0; i < 7; ++i) TORCH_CHECK(tensors[i]->is_cuda(), names[i], " must be on CUDA");
  TORCH_CHECK(hidden_states.dim() == 2, "hidden_states must be 2D [T, H]");
  TORCH_CHECK(router_indices.dim() == 2, "router_indices must be 2D [T, K]");
  TORCH_CHECK(routing_weights.dim() == 2, "routing_weights must be 2D [T, K]");
  TORCH_CHECK(gate_up_proj.dim() == 3, "gate_up_proj must be 3D [E, H, 2*H]");
  TORCH_CHECK(gate_up_proj_bias.dim() == 2, "gate_up_proj_bias must be 2D [E, 2*H]");
  TORCH_CHECK(down_proj.dim() == 3, "down_proj must be 3D [E, H, H]");
  TORCH_CHECK(down_proj_bias.dim() == 2, "down_proj_bias must be 2D [E, H]");
  const int64_t T = hidden_states.size(0), H = hidden_states.size(1), E = num_experts, K = top_k;
  TORCH_CHECK(router_indices.size(0) == T && router_indices.size(1) == K, "router_indices must be [T, K]");
  TORCH_CHECK(routing_weights.size(0) == T && (routing_weights.size(1) == K || routing_weights.size(1) == E),
              "routing_weights must be [T, K] or [T, E]");
  TORCH_CHECK(gate_up_proj.size(0) == E && gate_up_proj.size(1) == H && gate_up_proj.size(2) == 2 * H,
              "gate_up_proj must be [E, H, 2*H]");
  TORCH_CHECK(gate_up_proj_bias.size(0) == E && gate_up_proj_bias.size(1) == 2 * H,
              "gate_up_proj_bias must be [E, 2*H]");
  TORCH_CHECK(down_proj.size(0) == E && down_proj.size(1) == H && down_proj.size(2) == H, "down_proj must be [E, H, H]");
  TORCH_CHECK(down_proj_bias.size(0) == E && down_proj_bias.size(1) == H, "down_proj_bias must be [E, H]");
  const auto dt = hidden_states.scalar_type();
  TORCH_CHECK(dt == at::kFloat || dt == at::kBFloat16, "yamoe_b200 supports float32 and bfloat16, got ", dt);
  for (int i = 2; i < 7; ++i)
    TORCH_CHECK(tensors[i]->scalar_type() == dt, names[i], " must have the dtype of hidden_states (", dt, "), got ",
                tensors[i]->scalar_type());
  TORCH_CHECK(router_indices.scalar_type() == at::kLong || router_indices.scalar_type() == at::kInt,
              "router_indices must be int64");
  return Shape{T, (int)H, (int)E, (int)K, dt == at::kBFloat16 ? YAMOE_BF16 : YAMOE_F32};
}

void check(int status, const char* what) {
  TORCH_CHECK(status == YAMOE_OK, "yamoe_b200: ", what, " failed: ", yamoe_b200_status_string(status), " (status ",
              status, ")");
}

// YAMOE_B200_CHECK_STATUS=1: read the device status word after the call (one stream synchronisation)
void check_device_status(const at::Tensor& ws, cudaStream_t st, const char* what) {
  static const bool on = []() {
    const char* env = std::getenv("YAMOE_B200_CHECK_STATUS");
    return env != nullptr && env[0] != '\0' && !(env[0] == '0' && env[1] == '\0');
  }();
  if (!on) return;
  int32_t status = 0;
  check(yamoe_b200_device_status(ws.data_ptr(), st, &status), what);
  TORCH_CHECK(status == 0, "yamoe_b200: ", what, " failed: ", yamoe_b200_status_string(YAMOE_ERR_DEVICE_TIMEOUT),
              " (device status ", status, ")");
}

at::Tensor workspace(size_t nbytes, const at::Tensor& like) {
  return at::empty({(int64_t)(nbytes > 256 ? nbytes : 256)}, like.options().dtype(at::kByte));
}

at::Tensor experts_cuda(const at::Tensor& hidden_states, const at::Tensor& router_indices,
                        const at::Tensor& routing_weights, const at::Tensor& gate_up_proj,
                        const at::Tensor& gate_up_proj_bias, const at::Tensor& down_proj,
                        const at::Tensor& down_proj_bias, int64_t expert_capacity, int64_t num_experts,
                        int64_t top_k) {
  const Shape s = validate(hidden_states, router_indices, routing_weights, gate_up_proj, gate_up_proj_bias, down_proj,
                           down_proj_bias, num_experts, top_k);
  const c10::cuda::CUDAGuard guard(hidden_states.device());
  const at::Tensor hs = hidden_states.contiguous(), ri = router_indices.to(at::kLong).contiguous(),
                   rw = routing_weights.contiguous(), wgu = gate_up_proj.contiguous(),
                   bgu = gate_up_proj_bias.contiguous(), wd = down_proj.contiguous(), bd = down_proj_bias.contiguous();
  at::Tensor out = at::empty_like(hs);
  const size_t nbytes = yamoe_b200_forward_workspace_bytes(s.T, s.H, s.E, s.K, s.dtype);
  TORCH_CHECK(nbytes > 0, "yamoe_b200: unsupported shape (H must be a positive multiple of 8, E <= 1024)");
  const at::Tensor ws = workspace(nbytes, hs);
  cudaStream_t st = at::cuda::getCurrentCUDAStream().stream();
  check(yamoe_b200_experts_forward(hs.data_ptr(), ri.data_ptr<int64_t>(), rw.data_ptr(), (int)rw.size(1),
                                   wgu.data_ptr(), bgu.data_ptr(), wd.data_ptr(), bd.data_ptr(), out.data_ptr(), s.T,
                                   s.H, s.E, s.K, expert_capacity, s.dtype, ws.data_ptr(), (size_t)ws.numel(), st),
        "experts");
  check_device_status(ws, st, "experts");
  return out;
}

std::vector<at::Tensor> experts_backward_cuda(const at::Tensor& grad_out, const at::Tensor& hidden_states,
                                              const at::Tensor& router_indices, const at::Tensor& routing_weights,
                                              const at::Tensor& gate_up_proj, const at::Tensor& gate_up_proj_bias,
                                              const at::Tensor& down_proj, const at::Tensor& down_proj_bias,
                                              int64_t expert_capacity, int64_t num_experts, int64_t top_k) {
  TORCH_CHECK(grad_out.is_cuda(), "grad_out must be CUDA");
  const Shape s = validate(hidden_states, router_indices, routing_weights, gate_up_proj, gate_up_proj_bias, down_proj,
                           down_proj_bias, num_experts, top_k);
  TORCH_CHECK(grad_out.numel() == s.T * s.H || grad_out.numel() == s.T * s.K * s.H,
              "grad_out numel must be T*H or T*K*H");
  TORCH_CHECK(grad_out.scalar_type() == hidden_states.scalar_type(), "grad_out must have the dtype of hidden_states");
  const int per_slot = (grad_out.numel() == s.T * s.K * s.H && s.K != 1) ? 1 : 0;
  const c10::cuda::CUDAGuard guard(hidden_states.device());
  const at::Tensor go = grad_out.contiguous(), hs = hidden_states.contiguous(),
                   ri = router_indices.to(at::kLong).contiguous(), rw = routing_weights.contiguous(),
                   wgu = gate_up_proj.contiguous(), bgu = gate_up_proj_bias.contiguous(), wd = down_proj.contiguous(),
                   bd = down_proj_bias.contiguous();
  at::Tensor d_hidden = at::empty_like(hs), d_routing = at::empty_like(rw), d_wgu = at::empty_like(wgu),
             d_bgu = at::empty_like(bgu), d_wd = at::empty_like(wd), d_bd = at::empty_like(bd);
  const size_t nbytes = yamoe_b200_backward_workspace_bytes(s.T, s.H, s.E, s.K, s.dtype);
  TORCH_CHECK(nbytes > 0, "yamoe_b200: unsupported shape (H must be a positive multiple of 8, E <= 1024)");
  const at::Tensor ws = workspace(nbytes, hs);
  cudaStream_t st = at::cuda::getCurrentCUDAStream().stream();
  check(yamoe_b200_experts_backward(go.data_ptr(), per_slot, hs.data_ptr(), ri.data_ptr<int64_t>(), rw.data_ptr(),
                                    (int)rw.size(1), wgu.data_ptr(), bgu.data_ptr(), wd.data_ptr(), bd.data_ptr(),
                                    d_hidden.data_ptr(), d_routing.data_ptr(), d_wgu.data_ptr(), d_bgu.data_ptr(),
                                    d_wd.data_ptr(), d_bd.data_ptr(), s.T, s.H, s.E, s.K, expert_capacity, s.dtype,
                                    ws.data_ptr(), (size_t)ws.numel(), st),
        "experts_backward");
  check_device_status(ws, st, "experts_backward");
  return std::vector<at::Tensor>{d_hidden, d_routing, d_wgu, d_bgu, d_wd, d_bd};
}

}  // namespace

TORCH_LIBRARY_FRAGMENT(yamoe_b200, m) {
  m.def(
      "experts(Tensor hidden_states, Tensor router_indices, Tensor routing_weights, Tensor gate_up_proj, "
      "Tensor gate_up_proj_bias, Tensor down_proj, Tensor down_proj_bias, int expert_capacity, "
      "int num_experts, int top_k) -> Tensor");
  m.def(
      "experts_backward(Tensor grad_out, Tensor hidden_states, Tensor router_indices, Tensor routing_weights, "
      "Tensor gate_up_proj, Tensor gate_up_proj_bias, Tensor down_proj, Tensor down_proj_bias, "
      "int expert_capacity, int num_experts, int top_k) -> Tensor[]");
}

TORCH_LIBRARY_IMPL(yamoe_b200, CUDA, m) {
  m.impl("experts", &experts_cuda);
  m.impl("experts_backward", &experts_backward_cuda);
}
