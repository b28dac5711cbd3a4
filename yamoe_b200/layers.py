"""Autograd glue for the expert op: saves the seven inputs in forward and calls
`experts_backward` in backward, returning gradients in the op's argument order.
reference: torch-ext/yamoe/layers.py:6-100 (`_ExpertsFn`)."""
from __future__ import annotations

import torch

from . import ops


class _ExpertsFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden_flat, router_indices, routing_weights_dense, gate_up_proj, gate_up_proj_bias,
                down_proj, down_proj_bias, expert_capacity, num_experts, top_k, enable_router_grads):
        out = ops.experts(hidden_flat, router_indices, routing_weights_dense, gate_up_proj, gate_up_proj_bias,
                          down_proj, down_proj_bias, expert_capacity, num_experts, top_k)
        ctx.expert_capacity, ctx.num_experts, ctx.top_k = expert_capacity, num_experts, top_k
        ctx.enable_router_grads = bool(enable_router_grads)
        ctx.save_for_backward(hidden_flat, router_indices, routing_weights_dense, gate_up_proj,
                              gate_up_proj_bias, down_proj, down_proj_bias)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        saved = ctx.saved_tensors
        d_hidden, d_routing, d_wgu, d_bgu, d_wd, d_bd = ops.experts_backward(
            grad_output, *saved, ctx.expert_capacity, ctx.num_experts, ctx.top_k)
        return (d_hidden, None, d_routing if ctx.enable_router_grads else None, d_wgu, d_bgu, d_wd, d_bd,
                None, None, None, None)


class _ExpertsSavedFn(torch.autograd.Function):
    """Like `_ExpertsFn`, but the forward keeps the routing tables, gathered rows, pre-activations
    and weighted activations (about 12*S*H bytes in bf16), and the backward skips routing, the
    gather and the gate_up recompute: 12 instead of 16 S*H^2 of GEMM work."""

    @staticmethod
    def forward(ctx, hidden_flat, router_indices, routing_weights, gate_up_proj, gate_up_proj_bias,
                down_proj, down_proj_bias, expert_capacity, num_experts, top_k, enable_router_grads):
        out, saved = ops.experts_forward_saving(hidden_flat, router_indices, routing_weights, gate_up_proj,
                                                gate_up_proj_bias, down_proj, down_proj_bias, expert_capacity,
                                                num_experts, top_k)
        ctx.expert_capacity, ctx.num_experts, ctx.top_k = expert_capacity, num_experts, top_k
        ctx.enable_router_grads = bool(enable_router_grads)
        ctx.save_for_backward(saved, routing_weights, gate_up_proj, down_proj, down_proj_bias)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        saved, routing_weights, gate_up_proj, down_proj, down_proj_bias = ctx.saved_tensors
        d_hidden, d_routing, d_wgu, d_bgu, d_wd, d_bd = ops.experts_backward_saved(
            grad_output, saved, routing_weights, gate_up_proj, down_proj, down_proj_bias, ctx.expert_capacity,
            ctx.num_experts, ctx.top_k)
        return (d_hidden, None, d_routing if ctx.enable_router_grads else None, d_wgu, d_bgu, d_wd, d_bd,
                None, None, None, None)


def experts_autograd(hidden_flat, router_indices, routing_weights, gate_up_proj, gate_up_proj_bias, down_proj,
                     down_proj_bias, expert_capacity, num_experts, top_k, enable_router_grads=True,
                     save_activations=False):
    """Differentiable `experts`: forward through the CUDA op, backward through `experts_backward`
    (recomputing the forward, like the reference) or, with `save_activations`, through the pair
    that keeps the forward's intermediates.  A backward pass can run once per forward."""
    fn = _ExpertsSavedFn if save_activations else _ExpertsFn
    return fn.apply(hidden_flat, router_indices, routing_weights, gate_up_proj, gate_up_proj_bias,
                    down_proj, down_proj_bias, expert_capacity, num_experts, top_k, enable_router_grads)


def ceil_div(a, b):
    return (a + b - 1) // b


class Yamoe(torch.nn.Module):
    """Drop-in `forward` for a GPT-OSS MoE block (an object with `router.weight`, `router.bias`,
    `experts.gate_up_proj`, `experts.gate_up_proj_bias`, `experts.down_proj`,
    `experts.down_proj_bias`, and optionally `num_experts`, `top_k`), returning
    `(output [B,S,H], router_scores [T,E])` like the reference layer
    (torch-ext/yamoe/layers.py:103-218; oracle torch-ext/yamoe/vendored/gpt_oss_mlp.py:142-159).

    Differences from the reference layer, on purpose:
    * `expert_capacity` defaults to the reference's `ceil(T*K/E)` (layers.py:162), which drops
      assignments of over-subscribed experts; set the attribute `expert_capacity` (for example to
      the token count) for a run that never drops and therefore matches `GptOssMLP`.
    * gradients are not switched off: when autograd is recording, the router runs in PyTorch and
      the experts go through `_ExpertsFn`, so router and expert weights receive gradients.  Without
      autograd the whole router (projection, top-k, softmax, scatter) runs in the library: one
      tcgen05 kernel for bf16.
    """
    can_torch_compile: bool = False

    def forward(self, hidden_states: torch.Tensor):
        batch, seq, hidden = hidden_states.shape
        T = batch * seq
        E = getattr(self, "num_experts", self.router.weight.shape[0])
        K = getattr(self, "top_k", 4)
        x = hidden_states.reshape(T, hidden)
        needs_grad = torch.is_grad_enabled() and (
            x.requires_grad or self.router.weight.requires_grad or self.experts.gate_up_proj.requires_grad)
        if needs_grad:
            logits = torch.nn.functional.linear(x, self.router.weight, self.router.bias)
            top_v, router_indices = torch.topk(logits, K, dim=-1)
            top_w = torch.nn.functional.softmax(top_v, dim=-1, dtype=top_v.dtype)
            router_scores = torch.zeros_like(logits).scatter(1, router_indices, top_w)
        else:
            # router projection, top-k, softmax and scatter in the library (one kernel for bf16)
            router_indices, router_scores = ops.router_forward(x, self.router.weight, self.router.bias, K)
        cap = getattr(self, "expert_capacity", None)
        if cap is None:
            cap = ceil_div(T * K, E)
        gate_up = self.experts.gate_up_proj[:, :, : 2 * hidden]
        gate_up_bias = self.experts.gate_up_proj_bias[:, : 2 * hidden]
        down = self.experts.down_proj[:, :hidden, :]
        down_bias = self.experts.down_proj_bias
        if needs_grad:
            out = _ExpertsFn.apply(x, router_indices, router_scores, gate_up, gate_up_bias, down, down_bias,
                                   int(cap), E, K, True)
        else:
            out = ops.experts(x, router_indices, router_scores, gate_up, gate_up_bias, down, down_bias, int(cap), E, K)
        return out.view(batch, seq, hidden), router_scores
