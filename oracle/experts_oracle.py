"""CPU oracle for the yamoe expert forward / backward path.  TEST INFRASTRUCTURE ONLY.

This module is a CPU restatement (torch CPU tensors, fp32 or fp64 arithmetic) of the
algorithm the reference implements for `yamoe.experts` and `yamoe.experts_backward`.
It is the checker for the CUDA path: only the test-suite, the smoke check and the
CPU-baseline leg of the benchmark may import it.  The shipped package never does.

Parity pin: every function here is compared against the reference's own pure-PyTorch
implementations (`reference.py::GptOssExperts` in both branches, its twin
`vendored/gpt_oss_mlp.py`, and `vendored/yamoe_ref.py::binned_experts_ref`), imported by
file path, by `tests/golden/make_golden.py`; the resulting input/output vectors are
committed under `tests/golden/` and re-checked by the CPU test-suite.  The reference
itself ships no golden vectors or tests for this path.

Reference lines each function follows (paths are within the reference project):

* routing        csrc/sort.cu:17-59 (stable radix sort of expert ids, payload = iota),
                 csrc/bincount_cumsum.cu:7-56,72 (inclusive scan, slot E stays 0),
                 torch-ext/yamoe/vendored/yamoe_ref.py:38-43
* forward        csrc/moe.cpp:138-222; csrc/gather.cu:18-26 and csrc/scatter.cu:78-96
                 (capacity drop); build/torch28-cxx11-cu129-x86_64-linux/yamoe/reference.py:38-59
* backward       csrc/experts_backward.cu:176-340 with the routing-gradient placement of
                 autograd (the reference applies the sort permutation twice at :261-264).
"""
from __future__ import annotations

import torch

ALPHA = 1.702  # csrc/moe.cpp:179, reference.py:15
LIMIT = 7.0    # csrc/moe.cpp:175, reference.py:16


def route_oracle(router_indices: torch.Tensor, num_experts: int):
    """Stable sort of the flattened (token, slot) assignments by expert id.

    Returns (sorted_values int32 [S], sorted_indices int32 [S], counts int32 [E],
    bins int32 [E+1]) with `bins[e]` the inclusive prefix sum and `bins[E] == 0`
    (csrc/bincount_cumsum.cu:51-53,72; csrc/moe.cpp:122-124).  Ties keep ascending flat
    position p = t*K + slot, the order a stable LSD radix sort yields (csrc/sort.cu:30).
    """
    flat = router_indices.reshape(-1).to(torch.int64)
    sorted_values, sorted_indices = torch.sort(flat, stable=True)
    counts = torch.bincount(flat.clamp(0, num_experts - 1), minlength=num_experts)
    bins = torch.zeros(num_experts + 1, dtype=torch.int64)
    bins[:num_experts] = torch.cumsum(counts, 0)
    return (sorted_values.to(torch.int32), sorted_indices.to(torch.int32),
            counts.to(torch.int32), bins.to(torch.int32))


def _selected(routing_weights, router_indices, num_experts):
    """[T,K] weights of the chosen experts: a dense [T,E] input is gathered
    (csrc/moe.cpp:199-203), a [T,K] input is used as it is
    (csrc/experts_backward.cu:204-205)."""
    K = router_indices.shape[1]
    if routing_weights.shape[1] == num_experts:
        return torch.gather(routing_weights, 1, router_indices.to(torch.int64))
    assert routing_weights.shape[1] == K
    return routing_weights


def glu(pre: torch.Tensor) -> torch.Tensor:
    """Clamped SwiGLU on interleaved columns (csrc/moe.cpp:167-180, reference.py:51-55)."""
    g = pre[..., 0::2].clamp(max=LIMIT)
    u = pre[..., 1::2].clamp(min=-LIMIT, max=LIMIT)
    return (u + 1) * (g * torch.sigmoid(g * ALPHA))


def kept_rows(router_indices: torch.Tensor, num_experts: int, capacity: int):
    """For every expert the flat positions it keeps: the first min(n_e, C) of its segment
    in stable sorted order (csrc/gather.cu:18-26)."""
    _, sorted_indices, _, bins = route_oracle(router_indices, num_experts)
    out, start = [], 0
    for e in range(num_experts):
        end = int(bins[e])
        out.append(sorted_indices[start:min(end, start + capacity)].to(torch.int64))
        start = end
    return out


def experts_forward_oracle(hidden_states, router_indices, routing_weights, gate_up_proj,
                           gate_up_proj_bias, down_proj, down_proj_bias, expert_capacity,
                           num_experts, top_k, compute_dtype=torch.float32):
    """out[t] = sum over the kept slots (t,k) of w[t,k] * (glu(x_t W_gu[e] + b_gu[e]) W_d[e] + b_d[e]).

    Inputs are promoted to `compute_dtype`; the result is returned in `compute_dtype`.
    """
    cd = compute_dtype
    T, H = hidden_states.shape
    x = hidden_states.to(cd)
    w_sel = _selected(routing_weights, router_indices, num_experts).to(cd).reshape(-1)
    out = torch.zeros(T, H, dtype=cd)
    for e, flat_pos in enumerate(kept_rows(router_indices, num_experts, expert_capacity)):
        if flat_pos.numel() == 0:
            continue
        tok = flat_pos // top_k
        pre = x[tok] @ gate_up_proj[e].to(cd) + gate_up_proj_bias[e].to(cd)
        y = glu(pre) @ down_proj[e].to(cd) + down_proj_bias[e].to(cd)
        out.index_add_(0, tok, y * w_sel[flat_pos, None])
    return out


def experts_backward_oracle(grad_out, hidden_states, router_indices, routing_weights,
                            gate_up_proj, gate_up_proj_bias, down_proj, down_proj_bias,
                            expert_capacity, num_experts, top_k, compute_dtype=torch.float32):
    """Hand-derived gradients in the order the reference returns them
    (csrc/experts_backward.cu:340): dHidden, dRouting, dWgu, dbgu, dWd, dbd.

    `grad_out` holds T*H elements, or T*K*H which are summed over K first (:224-228).
    dRouting has the shape of `routing_weights`; only selected, kept entries are non-zero.
    Clamp gradients pass at equality (:296-299).
    """
    cd = compute_dtype
    T, H = hidden_states.shape
    E, K = num_experts, top_k
    x = hidden_states.to(cd)
    gy = grad_out.to(cd).reshape(T, -1, H).sum(1) if grad_out.numel() == T * K * H and K != 1 \
        else grad_out.to(cd).reshape(T, H)
    dense = routing_weights.shape[1] == E
    w_sel = _selected(routing_weights, router_indices, E).to(cd).reshape(-1)
    d_hidden = torch.zeros(T, H, dtype=cd)
    d_sel = torch.zeros(T * K, dtype=cd)
    d_wgu = torch.zeros(gate_up_proj.shape, dtype=cd)
    d_bgu = torch.zeros(gate_up_proj_bias.shape, dtype=cd)
    d_wd = torch.zeros(down_proj.shape, dtype=cd)
    d_bd = torch.zeros(down_proj_bias.shape, dtype=cd)
    for e, flat_pos in enumerate(kept_rows(router_indices, E, expert_capacity)):
        if flat_pos.numel() == 0:
            continue
        tok = flat_pos // K
        xe = x[tok]
        wgu, wd = gate_up_proj[e].to(cd), down_proj[e].to(cd)
        pre = xe @ wgu + gate_up_proj_bias[e].to(cd)
        pg, pu = pre[:, 0::2], pre[:, 1::2]
        gc, uc = pg.clamp(max=LIMIT), pu.clamp(min=-LIMIT, max=LIMIT)
        sig = torch.sigmoid(gc * ALPHA)
        gate_act = gc * sig
        act = (uc + 1) * gate_act
        y = act @ wd + down_proj_bias[e].to(cd)
        g_e = gy[tok] * w_sel[flat_pos, None]                      # :79-81
        d_sel[flat_pos] = (gy[tok] * y).sum(1)                     # :83-88
        d_bd[e] = g_e.sum(0)                                       # :277
        g_i = g_e @ wd.t()                                         # :278-280
        d_wd[e] = act.t() @ g_e                                    # :281-282
        g_u = g_i * gate_act                                       # :285
        g_g = g_i * (uc + 1) * (sig + gc * sig * (1 - sig) * ALPHA)  # :286-293
        g_g = torch.where(pg > LIMIT, torch.zeros_like(g_g), g_g)  # :296-297
        g_u = torch.where((pu > LIMIT) | (pu < -LIMIT), torch.zeros_like(g_u), g_u)  # :298-299
        g_pre = torch.stack([g_g, g_u], dim=-1).reshape(pre.shape)  # :302-305
        d_bgu[e] = g_pre.sum(0)                                    # :308
        d_hidden.index_add_(0, tok, g_pre @ wgu.t())               # :309-310, :115-123
        d_wgu[e] = xe.t() @ g_pre                                  # :311
    if dense:
        d_routing = torch.zeros(T, E, dtype=cd)
        d_routing.scatter_add_(1, router_indices.to(torch.int64), d_sel.view(T, K))  # :266-271
    else:
        d_routing = d_sel.view(T, K)
    return d_hidden, d_routing, d_wgu, d_bgu, d_wd, d_bd


# Seeded synthetic workloads live in the package (they are inputs, not a checker) and are
# re-exported here for the tests.
from yamoe_b200.workloads import make_inputs, make_readme_inputs, make_routing  # noqa: E402,F401


def binned_gather_oracle(x, indices, bins, num_experts, capacity, top_k):
    """out[e, i] = x[indices[bins[e-1] + i] // top_k] for i < min(count_e, capacity), zeros elsewhere
    (csrc/gather.cu:17-62; torch-ext/yamoe/vendored/yamoe_ref.py:4-15)."""
    T, H = x.shape
    out = torch.zeros(num_experts, capacity, H, dtype=x.dtype)
    for e in range(num_experts):
        start = int(bins[e - 1]) if e else 0
        n = min(int(bins[e]) - start, capacity)
        if n > 0:
            tok = indices[start:start + n].long() // top_k
            ok = (tok >= 0) & (tok < T)
            out[e, :n][ok] = x[tok[ok]]
    return out


def binned_scatter_oracle(src, indices, bins, weights_sorted, y, top_k, compute_dtype=torch.float64):
    """y[tok] += weights_sorted[bins[e-1] + i] * src[e, i] for i < min(count_e, capacity)
    (csrc/scatter.cu:67-108).  `weights_sorted` is indexed by sorted position, as in the CUDA
    operator; yamoe_ref.py:18-35 indexes the un-sorted weights by flat position, which is the same
    value.  Accumulates in `compute_dtype` and returns a new tensor of y's dtype."""
    E, C, H = src.shape
    T = y.shape[0]
    acc = y.to(compute_dtype).clone()
    for e in range(E):
        start = int(bins[e - 1]) if e else 0
        n = min(int(bins[e]) - start, C)
        for i in range(n):
            tok = int(indices[start + i]) // top_k
            if 0 <= tok < T:
                w = 1.0 if weights_sorted is None else weights_sorted[start + i].to(compute_dtype)
                acc[tok] += w * src[e, i].to(compute_dtype)
    return acc.to(y.dtype)


def router_oracle(hidden, router_weight, router_bias, top_k):
    """Router of the layer that feeds the expert op (torch-ext/yamoe/vendored/gpt_oss_mlp.py:127-139,
    torch-ext/yamoe/layers.py:126-149): logits = x W^T + b, top-k on the logits, softmax over the k
    selected logits, dense [T,E] scores.  Returns (router_scores, router_indices)."""
    logits = torch.nn.functional.linear(hidden, router_weight, router_bias)
    top_v, idx = torch.topk(logits, top_k, dim=-1)
    top_w = torch.softmax(top_v, dim=-1)
    return torch.zeros_like(logits).scatter_(1, idx, top_w), idx


def check_close(x, ref, rtol, name="", rel_l2=None):
    """|x - ref| <= rtol*|ref| + rtol*max|ref| elementwise (and optionally a rel-L2 bound).
    Returns (max_violation_ratio, rel_l2) and raises AssertionError on failure."""
    x, ref = x.double(), ref.double()
    scale = ref.abs().max().item()
    bound = rtol * ref.abs() + rtol * scale
    err = (x - ref).abs()
    ratio = (err / bound.clamp_min(1e-300)).max().item() if ref.numel() else 0.0
    l2 = ((x - ref).norm() / ref.norm().clamp_min(1e-300)).item() if ref.numel() else 0.0
    if scale == 0.0:
        assert err.max().item() == 0.0 if ref.numel() else True, f"{name}: expected exact zeros"
        return 0.0, 0.0
    assert ratio <= 1.0, f"{name}: max |err|/bound = {ratio:.3f} (rel-L2 {l2:.3e})"
    if rel_l2 is not None:
        assert l2 <= rel_l2, f"{name}: rel-L2 {l2:.3e} > {rel_l2:.1e}"
    return ratio, l2


def reference_forward_from(path: str):
    """Wraps the reference project's own `GptOssExperts` (its reference.py, loaded from `path`) in
    the signature of `experts_forward_oracle`, running the sparse (training) branch
    (reference.py:38-59).  The reference has no expert capacity: the wrapper is only valid when the
    capacity drops nothing, which holds for every benchmark workload."""
    import importlib.util
    import types
    spec = importlib.util.spec_from_file_location("yamoe_reference_py", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)

    def forward(hidden_states, router_indices, routing_weights, gate_up_proj, gate_up_proj_bias, down_proj,
                down_proj_bias, expert_capacity, num_experts, top_k, compute_dtype=torch.float32):
        T, H = hidden_states.shape
        cfg = types.SimpleNamespace(intermediate_size=H, num_local_experts=num_experts, hidden_size=H)
        m = mod.GptOssExperts(cfg)
        for name, t in (("gate_up_proj", gate_up_proj), ("gate_up_proj_bias", gate_up_proj_bias),
                        ("down_proj", down_proj), ("down_proj_bias", down_proj_bias)):
            getattr(m, name).data = t.to(compute_dtype)
        m.train()
        dense = routing_weights
        if dense.shape[1] != num_experts:
            dense = torch.zeros(T, num_experts, dtype=routing_weights.dtype)
            dense.scatter_(1, router_indices.to(torch.int64), routing_weights)
        with torch.no_grad():
            out = m(hidden_states.to(compute_dtype).view(1, T, H), router_indices=router_indices.to(torch.int64),
                    routing_weights=dense.to(compute_dtype))
        return out.view(T, H)

    return forward
