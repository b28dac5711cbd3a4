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


def experts_autograd(hidden_flat, router_indices, routing_weights, gate_up_proj, gate_up_proj_bias, down_proj,
                     down_proj_bias, expert_capacity, num_experts, top_k, enable_router_grads=True):
    """Differentiable `experts`: forward through the CUDA op, backward through `experts_backward`."""
    return _ExpertsFn.apply(hidden_flat, router_indices, routing_weights, gate_up_proj, gate_up_proj_bias,
                            down_proj, down_proj_bias, expert_capacity, num_experts, top_k, enable_router_grads)
