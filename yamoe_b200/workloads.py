"""Seeded synthetic inputs for the expert op, with the shapes and value distributions of the
reference's own benchmark scripts (readme_example.py:14-45, perf_plot.py:29-39).  Shared by the
tests and the benchmark; plain torch on a CPU generator so that every machine gets the same
tensors."""
from __future__ import annotations

import torch



def make_routing(T, E, K, gen, expert_bias=None):
    """softmax over E logits, top-K without renormalisation, dense scatter
    (readme_example.py:27-36)."""
    logits = torch.randn(T, E, generator=gen)
    if expert_bias is not None:
        logits = logits + expert_bias
    probs = torch.softmax(logits, dim=-1)
    weights, indices = torch.topk(probs, K, dim=-1)
    dense = torch.zeros(T, E)
    dense.scatter_(1, indices, weights)
    return indices.contiguous(), dense


def make_inputs(T, H, E, K, seed=42, weight_std=0.02, bias_std=0.02, dtype=torch.float32,
                skew=False, with_grad=False, weights_on=None):
    """Generation order: logits, hidden, gate_up, gate_up_bias, down, down_bias, (grad_out).

    With `weights_on="cuda"` the four weight tensors are drawn on that device from a device
    generator with the same seed (for the 120B-shaped workloads whose 6.4 GB of weights are too
    slow to draw on the host); routing and activations still come from the CPU generator."""
    gen = torch.Generator().manual_seed(seed)
    bias = None
    if skew:
        bias = -1.2 * torch.log(torch.arange(E, dtype=torch.float32) + 1.0)
    indices, dense = make_routing(T, E, K, gen, bias)
    hidden = torch.randn(T, H, generator=gen)
    if weights_on is not None:
        dgen = torch.Generator(device=weights_on).manual_seed(seed)

        def draw(*shape, std):
            out = torch.empty(*shape, dtype=dtype, device=weights_on)
            for e in range(shape[0]):       # per expert: bounds the fp32 temporary
                out[e] = (torch.randn(*shape[1:], generator=dgen, device=weights_on) * std).to(dtype)
            return out
        out = dict(hidden_states=hidden.to(dtype), router_indices=indices, routing_weights=dense.to(dtype),
                   gate_up_proj=draw(E, H, 2 * H, std=weight_std), gate_up_proj_bias=draw(E, 2 * H, std=bias_std),
                   down_proj=draw(E, H, H, std=weight_std), down_proj_bias=draw(E, H, std=bias_std))
        if with_grad:
            out["grad_out"] = torch.randn(T, H, generator=gen).to(dtype)
        return out
    wgu = torch.randn(E, H, 2 * H, generator=gen) * weight_std
    bgu = torch.randn(E, 2 * H, generator=gen) * bias_std
    wd = torch.randn(E, H, H, generator=gen) * weight_std
    bd = torch.randn(E, H, generator=gen) * bias_std
    out = dict(hidden_states=hidden.to(dtype), router_indices=indices,
               routing_weights=dense.to(dtype), gate_up_proj=wgu.to(dtype),
               gate_up_proj_bias=bgu.to(dtype), down_proj=wd.to(dtype),
               down_proj_bias=bd.to(dtype))
    if with_grad:
        out["grad_out"] = torch.randn(T, H, generator=gen).to(dtype)
    return out


def make_readme_inputs(batch=2, seq=256, H=2880, E=8, K=2, seed=42):
    """The README workload (readme_example.py:15-45) at a chosen batch size: N(0,1)
    weights, zero biases, fp32."""
    torch.manual_seed(seed)
    logits = torch.randn(batch, seq, E)
    probs = torch.softmax(logits, dim=-1)
    weights, indices = torch.topk(probs, K, dim=-1)
    T = batch * seq
    dense = torch.zeros(T, E, dtype=weights.dtype)
    fi, fw = indices.reshape(-1, K), weights.reshape(-1, K)
    dense[torch.arange(T).unsqueeze(1).expand(-1, K), fi] = fw
    hidden = torch.randn(batch, seq, H)
    wgu = torch.randn(E, H, 2 * H)
    bgu = torch.zeros(E, 2 * H)
    wd = torch.randn(E, H, H)
    bd = torch.zeros(E, H)
    return dict(hidden_states=hidden.view(T, H), router_indices=fi.contiguous(),
                routing_weights=dense, gate_up_proj=wgu, gate_up_proj_bias=bgu,
                down_proj=wd, down_proj_bias=bd)


