"""torch operators `yamoe_b200::experts` / `experts_backward` / `sort` / `bincount_cumsum` /
`gather` / `scatter` / `index_select_out` / `batch_mm`
with the schemas of the reference binding (torch-ext/torch_binding.cpp:9-83),
implemented as thin calls into the C ABI: validate, allocate the output and one workspace
tensor with torch, pass raw pointers and torch's current stream.
"""
from __future__ import annotations

import os

import torch

from . import _lib

_DT = {torch.float32: _lib.YAMOE_F32, torch.bfloat16: _lib.YAMOE_BF16}



def _load_cpp_binding() -> bool:
    """`experts` and `experts_backward` come from the C++ binding (csrc/torch_binding.cpp, built as
    libyamoe_b200_torch.so next to the CUDA library) when it is there: same schemas, same checks, a
    dispatch that costs a few microseconds instead of some tens.  YAMOE_B200_PY_BINDING=1 keeps the
    Python registration below (used by the tests that compare the two)."""
    if os.environ.get("YAMOE_B200_PY_BINDING", "0") not in ("", "0"):
        return False
    if os.environ.get("YAMOE_B200_LIB"):
        return False                 # the binding is linked against the default build of the library
    from .build import BINDING_PATH
    if not os.path.exists(BINDING_PATH):
        return False
    _lib.lib()                       # the CUDA library must be loaded first (and must exist)
    torch.ops.load_library(BINDING_PATH)
    return True


CPP_BINDING = _load_cpp_binding()

if not CPP_BINDING:
    torch.library.define(
        "yamoe_b200::experts",
        "(Tensor hidden_states, Tensor router_indices, Tensor routing_weights, Tensor gate_up_proj, "
        "Tensor gate_up_proj_bias, Tensor down_proj, Tensor down_proj_bias, int expert_capacity, "
        "int num_experts, int top_k) -> Tensor")
    torch.library.define(
        "yamoe_b200::experts_backward",
        "(Tensor grad_out, Tensor hidden_states, Tensor router_indices, Tensor routing_weights, "
        "Tensor gate_up_proj, Tensor gate_up_proj_bias, Tensor down_proj, Tensor down_proj_bias, "
        "int expert_capacity, int num_experts, int top_k) -> Tensor[]")
torch.library.define("yamoe_b200::sort", "(Tensor x, int end_bit, Tensor(a!) x_out, Tensor(b!) iota_out) -> ()")
torch.library.define("yamoe_b200::batch_mm",
                     "(Tensor x, Tensor weights, Tensor batch_sizes, Tensor(a!) output, bool trans_b=False) -> Tensor")
torch.library.define("yamoe_b200::bincount_cumsum", "(Tensor input, Tensor(a!) output, int minlength) -> ()")
torch.library.define("yamoe_b200::gather",
                     "(Tensor x, Tensor indices, Tensor bins, Tensor(a!) output, int E, int C, int top_k) -> ()")
torch.library.define("yamoe_b200::scatter",
                     "(Tensor src, Tensor indices, Tensor bins, Tensor weights, Tensor(a!) y, int T, int E, int C, "
                     "int top_k) -> ()")
torch.library.define("yamoe_b200::index_select_out", "(Tensor(a!) out, Tensor input, Tensor idx_int32) -> Tensor(a!)")


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _workspace(nbytes: int, device) -> torch.Tensor:
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)


def _check_device_status(ws: torch.Tensor, what: str) -> None:
    """With YAMOE_B200_CHECK_STATUS=1 every expert call is followed by a read of the device status
    word of its workspace (one stream synchronisation): a bounded wait inside a kernel that gave up
    then raises instead of returning partly written outputs.  Off by default (no host sync)."""
    if os.environ.get("YAMOE_B200_CHECK_STATUS", "0") not in ("", "0"):
        _lib.check_device_status(ws.data_ptr(), _stream(), what)


def _validate(hidden_states, router_indices, routing_weights, gate_up_proj, gate_up_proj_bias, down_proj,
              down_proj_bias, num_experts, top_k):
    """Same preconditions, in the same order, as csrc/moe.cpp:58-96."""
    names = ["hidden_states", "router_indices", "routing_weights", "gate_up_proj", "gate_up_proj_bias",
             "down_proj", "down_proj_bias"]
    tensors = [hidden_states, router_indices, routing_weights, gate_up_proj, gate_up_proj_bias, down_proj,
               down_proj_bias]
    for n, t in zip(names, tensors):
        _require(t.is_cuda, f"{n} must be on CUDA")
    _require(hidden_states.dim() == 2, "hidden_states must be 2D [T, H]")
    _require(router_indices.dim() == 2, "router_indices must be 2D [T, K]")
    _require(routing_weights.dim() == 2, "routing_weights must be 2D [T, K]")
    _require(gate_up_proj.dim() == 3, "gate_up_proj must be 3D [E, H, 2*H]")
    _require(gate_up_proj_bias.dim() == 2, "gate_up_proj_bias must be 2D [E, 2*H]")
    _require(down_proj.dim() == 3, "down_proj must be 3D [E, H, H]")
    _require(down_proj_bias.dim() == 2, "down_proj_bias must be 2D [E, H]")
    T, H = hidden_states.shape
    E, K = int(num_experts), int(top_k)
    _require(tuple(router_indices.shape) == (T, K), "router_indices must be [T, K]")
    _require(routing_weights.shape[0] == T and routing_weights.shape[1] in (K, E),
             "routing_weights must be [T, K] or [T, E]")
    _require(tuple(gate_up_proj.shape) == (E, H, 2 * H), "gate_up_proj must be [E, H, 2*H]")
    _require(tuple(gate_up_proj_bias.shape) == (E, 2 * H), "gate_up_proj_bias must be [E, 2*H]")
    _require(tuple(down_proj.shape) == (E, H, H), "down_proj must be [E, H, H]")
    _require(tuple(down_proj_bias.shape) == (E, H), "down_proj_bias must be [E, H]")
    dt = hidden_states.dtype
    _require(dt in _DT, f"yamoe_b200 supports float32 and bfloat16, got {dt}")
    for n, t in zip(names[2:], tensors[2:]):
        _require(t.dtype == dt, f"{n} must have the dtype of hidden_states ({dt}), got {t.dtype}")
    _require(router_indices.dtype in (torch.int64, torch.int32), "router_indices must be int64")
    return T, H, E, K


def _impl_unless_cpp(name):
    """Registers the Python implementation of an operator unless the C++ binding already has one."""
    def deco(fn):
        return fn if CPP_BINDING else torch.library.impl(name, "CUDA")(fn)
    return deco


@_impl_unless_cpp("yamoe_b200::experts")
def _experts_cuda(hidden_states, router_indices, routing_weights, gate_up_proj, gate_up_proj_bias, down_proj,
                  down_proj_bias, expert_capacity, num_experts, top_k):
    T, H, E, K = _validate(hidden_states, router_indices, routing_weights, gate_up_proj, gate_up_proj_bias,
                           down_proj, down_proj_bias, num_experts, top_k)
    L = _lib.lib()
    with torch.cuda.device(hidden_states.device):
        hs = hidden_states.contiguous()
        ri = router_indices.to(torch.int64).contiguous()
        rw = routing_weights.contiguous()
        wgu, bgu = gate_up_proj.contiguous(), gate_up_proj_bias.contiguous()
        wd, bd = down_proj.contiguous(), down_proj_bias.contiguous()
        out = torch.empty_like(hs)
        dt = _DT[hs.dtype]
        nbytes = L.yamoe_b200_forward_workspace_bytes(T, H, E, K, dt)
        _require(nbytes > 0, "yamoe_b200: unsupported shape (H must be a positive multiple of 8, E <= 1024)")
        ws = _workspace(nbytes, hs.device)
        st = L.yamoe_b200_experts_forward(hs.data_ptr(), ri.data_ptr(), rw.data_ptr(), rw.shape[1], wgu.data_ptr(),
                                          bgu.data_ptr(), wd.data_ptr(), bd.data_ptr(), out.data_ptr(), T, H, E, K,
                                          int(expert_capacity), dt, ws.data_ptr(), ws.numel(), _stream())
        _lib.check(st, "experts")
        _check_device_status(ws, "experts")
    return out


@_impl_unless_cpp("yamoe_b200::experts_backward")
def _experts_backward_cuda(grad_out, hidden_states, router_indices, routing_weights, gate_up_proj,
                           gate_up_proj_bias, down_proj, down_proj_bias, expert_capacity, num_experts, top_k):
    _require(grad_out.is_cuda, "grad_out must be CUDA")
    T, H, E, K = _validate(hidden_states, router_indices, routing_weights, gate_up_proj, gate_up_proj_bias,
                           down_proj, down_proj_bias, num_experts, top_k)
    _require(grad_out.numel() in (T * H, T * K * H), "grad_out numel must be T*H or T*K*H")
    _require(grad_out.dtype == hidden_states.dtype, "grad_out must have the dtype of hidden_states")
    per_slot = int(grad_out.numel() == T * K * H and K != 1)
    L = _lib.lib()
    with torch.cuda.device(hidden_states.device):
        go = grad_out.contiguous()
        hs = hidden_states.contiguous()
        ri = router_indices.to(torch.int64).contiguous()
        rw = routing_weights.contiguous()
        wgu, bgu = gate_up_proj.contiguous(), gate_up_proj_bias.contiguous()
        wd, bd = down_proj.contiguous(), down_proj_bias.contiguous()
        d_hidden, d_routing = torch.empty_like(hs), torch.empty_like(rw)
        d_wgu, d_bgu = torch.empty_like(wgu), torch.empty_like(bgu)
        d_wd, d_bd = torch.empty_like(wd), torch.empty_like(bd)
        dt = _DT[hs.dtype]
        nbytes = L.yamoe_b200_backward_workspace_bytes(T, H, E, K, dt)
        _require(nbytes > 0, "yamoe_b200: unsupported shape (H must be a positive multiple of 8, E <= 1024)")
        ws = _workspace(nbytes, hs.device)
        st = L.yamoe_b200_experts_backward(go.data_ptr(), per_slot, hs.data_ptr(), ri.data_ptr(), rw.data_ptr(),
                                           rw.shape[1], wgu.data_ptr(), bgu.data_ptr(), wd.data_ptr(), bd.data_ptr(),
                                           d_hidden.data_ptr(), d_routing.data_ptr(), d_wgu.data_ptr(),
                                           d_bgu.data_ptr(), d_wd.data_ptr(), d_bd.data_ptr(), T, H, E, K,
                                           int(expert_capacity), dt, ws.data_ptr(), ws.numel(), _stream())
        _lib.check(st, "experts_backward")
        _check_device_status(ws, "experts_backward")
    return [d_hidden, d_routing, d_wgu, d_bgu, d_wd, d_bd]


def experts_forward_saving(hidden_states, router_indices, routing_weights, gate_up_proj, gate_up_proj_bias,
                           down_proj, down_proj_bias, expert_capacity, num_experts, top_k):
    """`experts` that also returns the buffer `experts_backward_saved` needs (routing tables,
    gathered rows, pre-activations, weighted activations), so that the backward pass does not
    recompute the gate_up GEMM.  Returns (out, saved)."""
    T, H, E, K = _validate(hidden_states, router_indices, routing_weights, gate_up_proj, gate_up_proj_bias,
                           down_proj, down_proj_bias, num_experts, top_k)
    L = _lib.lib()
    with torch.cuda.device(hidden_states.device):
        hs = hidden_states.contiguous()
        ri = router_indices.to(torch.int64).contiguous()
        rw = routing_weights.contiguous()
        wgu, bgu = gate_up_proj.contiguous(), gate_up_proj_bias.contiguous()
        wd, bd = down_proj.contiguous(), down_proj_bias.contiguous()
        out = torch.empty_like(hs)
        dt = _DT[hs.dtype]
        nbytes = L.yamoe_b200_backward_workspace_bytes(T, H, E, K, dt)
        _require(nbytes > 0, "yamoe_b200: unsupported shape (H must be a positive multiple of 8, E <= 1024)")
        saved = _workspace(nbytes, hs.device)
        st = L.yamoe_b200_experts_forward_saving(hs.data_ptr(), ri.data_ptr(), rw.data_ptr(), rw.shape[1],
                                                 wgu.data_ptr(), bgu.data_ptr(), wd.data_ptr(), bd.data_ptr(),
                                                 out.data_ptr(), T, H, E, K, int(expert_capacity), dt,
                                                 saved.data_ptr(), saved.numel(), _stream())
        _lib.check(st, "experts_forward_saving")
    return out, saved


def experts_backward_saved(grad_out, saved, routing_weights, gate_up_proj, down_proj, down_proj_bias,
                           expert_capacity, num_experts, top_k):
    """Gradients (same six tensors as `experts_backward`) from the buffer left by
    `experts_forward_saving`; the buffer is consumed."""
    T, H = grad_out.numel() // gate_up_proj.shape[1], gate_up_proj.shape[1]
    E, K = int(num_experts), int(top_k)
    per_slot = 0
    if grad_out.numel() == routing_weights.shape[0] * K * H and K != 1:
        per_slot, T = 1, routing_weights.shape[0]
    _require(grad_out.is_cuda and grad_out.dtype in _DT, "grad_out must be a CUDA float32/bfloat16 tensor")
    L = _lib.lib()
    with torch.cuda.device(grad_out.device):
        go = grad_out.contiguous()
        rw = routing_weights.contiguous()
        wgu, wd, bd = gate_up_proj.contiguous(), down_proj.contiguous(), down_proj_bias.contiguous()
        d_hidden = torch.empty(T, H, dtype=go.dtype, device=go.device)
        d_routing = torch.empty_like(rw)
        d_wgu = torch.empty_like(wgu)
        d_bgu = torch.empty(E, 2 * H, dtype=go.dtype, device=go.device)
        d_wd, d_bd = torch.empty_like(wd), torch.empty_like(bd)
        st = L.yamoe_b200_experts_backward_saved(go.data_ptr(), per_slot, rw.data_ptr(), rw.shape[1], wgu.data_ptr(),
                                                 wd.data_ptr(), bd.data_ptr(), d_hidden.data_ptr(), d_routing.data_ptr(),
                                                 d_wgu.data_ptr(), d_bgu.data_ptr(), d_wd.data_ptr(), d_bd.data_ptr(),
                                                 T, H, E, K, int(expert_capacity), _DT[go.dtype], saved.data_ptr(),
                                                 saved.numel(), _stream())
        _lib.check(st, "experts_backward_saved")
    return [d_hidden, d_routing, d_wgu, d_bgu, d_wd, d_bd]


def route(router_indices: torch.Tensor, num_experts: int):
    """Stable sort of the flattened assignments by expert id plus histogram and inclusive
    prefix sums: (sorted_values, sorted_indices, bins[E+1], counts[E]), all int32."""
    _require(router_indices.is_cuda, "router_indices must be on CUDA")
    flat = router_indices.to(torch.int64).contiguous().view(-1)
    S, E = flat.numel(), int(num_experts)
    L = _lib.lib()
    with torch.cuda.device(flat.device):
        opts = dict(dtype=torch.int32, device=flat.device)
        sv, si = torch.empty(S, **opts), torch.empty(S, **opts)
        bins, counts = torch.empty(E + 1, **opts), torch.empty(E, **opts)
        ws = _workspace(L.yamoe_b200_route_workspace_bytes(S, E, 1), flat.device)
        st = L.yamoe_b200_route(flat.data_ptr(), sv.data_ptr(), si.data_ptr(), bins.data_ptr(), counts.data_ptr(),
                                S, E, 1, ws.data_ptr(), ws.numel(), _stream())
        _lib.check(st, "route")
    return sv, si, bins, counts


@torch.library.impl("yamoe_b200::sort", "CUDA")
def _sort_cuda(x, end_bit, x_out, iota_out):
    """reference: csrc/sort.cu:61-91.  Keys must lie in [0, 2**end_bit) with 2**end_bit <= 1024
    or simply below 1024: the counting sort serves expert ids, not general integers."""
    _require(x.dim() == 1 and x_out.shape == x.shape and iota_out.shape == x.shape, "sort: shape mismatch")
    sv, si, _, _ = route(x, 1024 if end_bit >= 10 else (1 << max(int(end_bit), 0)))
    x_out.copy_(sv)
    iota_out.copy_(si)


@torch.library.impl("yamoe_b200::bincount_cumsum", "CUDA")
def _bincount_cumsum_cuda(input, output, minlength):
    """reference: csrc/bincount_cumsum.cu:58-98: output[e] = inclusive prefix sum, output[minlength:] = 0."""
    _, _, bins, _ = route(input, int(minlength))
    output.zero_()
    output[:minlength].copy_(bins[:minlength])


def _binned_checks(name, data, indices, bins, E):
    _require(data.is_cuda and indices.is_cuda and bins.is_cuda, f"{name}: CUDA tensors expected")
    _require(data.dtype in _DT, f"{name}: float32 or bfloat16 expected, got {data.dtype}")
    _require(indices.dtype == torch.int32 and bins.dtype == torch.int32, f"{name}: indices and bins must be int32")
    _require(bins.numel() >= E, f"{name}: bins must hold E cumulative counts")
    _require(data.is_contiguous() and indices.is_contiguous() and bins.is_contiguous(),
             f"{name}: contiguous tensors expected")


@torch.library.impl("yamoe_b200::gather", "CUDA")
def _gather_cuda(x, indices, bins, output, E, C, top_k):
    """reference: csrc/gather.cu:68-109.  output [E, C, H] is overwritten (zeros beyond each count)."""
    E, C = int(E), int(C)
    _binned_checks("gather", x, indices, bins, E)
    _require(x.dim() == 2, "gather: x must be [T, H]")
    T, H = x.shape
    _require(tuple(output.shape) == (E, C, H), "Output tensor must have shape [E, C, H]")
    _require(output.dtype == x.dtype and output.is_cuda and output.is_contiguous(),
             "gather: output must be a contiguous CUDA tensor of x's dtype")
    with torch.cuda.device(x.device):
        st = _lib.lib().yamoe_b200_binned_gather(x.data_ptr(), indices.data_ptr(), bins.data_ptr(), output.data_ptr(),
                                                 T, H, E, C, int(top_k), _DT[x.dtype], _stream())
        _lib.check(st, "gather")


@torch.library.impl("yamoe_b200::scatter", "CUDA")
def _scatter_cuda(src, indices, bins, weights, y, T, E, C, top_k):
    """reference: csrc/scatter.cu:110-147.  y [T, H] is accumulated into; `weights` [S] are in
    expert-sorted order (an empty tensor means no scaling)."""
    T, E, C = int(T), int(E), int(C)
    _binned_checks("scatter", src, indices, bins, E)
    _require(src.dim() == 3 and src.shape[0] == E and src.shape[1] == C, "scatter: src must be [E, C, H]")
    H = src.shape[2]
    _require(y.is_cuda and y.is_contiguous() and y.dtype == src.dtype and y.dim() == 2 and y.shape[0] >= T
             and y.shape[1] == H, "scatter: y must be a contiguous [T, H] CUDA tensor of src's dtype")
    w_ptr = None
    if weights is not None and weights.numel() > 0:
        _require(weights.is_cuda and weights.dtype == src.dtype and weights.is_contiguous()
                 and weights.numel() >= indices.numel(), "scatter: weights must be [S] of src's dtype")
        w_ptr = weights.data_ptr()
    with torch.cuda.device(src.device):
        st = _lib.lib().yamoe_b200_binned_scatter(src.data_ptr(), indices.data_ptr(), bins.data_ptr(), w_ptr,
                                                  y.data_ptr(), T, H, E, C, int(top_k), _DT[src.dtype], _stream())
        _lib.check(st, "scatter")


@torch.library.impl("yamoe_b200::index_select_out", "CUDA")
def _index_select_out_cuda(out, input, idx_int32):
    """reference: csrc/index_select.cu:18-52: out[i] = input[idx[i]] over flat, contiguous tensors."""
    _require(input.is_cuda and idx_int32.is_cuda and out.is_cuda, "cuda only")
    _require(idx_int32.dtype == torch.int32, "idx must be int32")
    _require(input.is_contiguous() and idx_int32.is_contiguous() and out.is_contiguous(), "contiguous required")
    _require(input.dtype in _DT and out.dtype == input.dtype, "index_select_out: float32 or bfloat16 expected")
    _require(out.numel() >= idx_int32.numel(), "index_select_out: out is too small")
    with torch.cuda.device(input.device):
        st = _lib.lib().yamoe_b200_index_select(out.data_ptr(), input.data_ptr(), idx_int32.data_ptr(),
                                                idx_int32.numel(), _DT[input.dtype], _stream())
        _lib.check(st, "index_select_out")
    return out


def _batch_mm_raw(x, weights, out, mode):
    E, C = x.shape[0], x.shape[1]
    M = x.shape[2] if mode == 2 else 0
    K = 0 if mode == 2 else x.shape[2]
    N = out.shape[2]
    L = _lib.lib()
    with torch.cuda.device(x.device):
        ws = _workspace(L.yamoe_b200_batch_mm_workspace_bytes(E, C), x.device)
        st = L.yamoe_b200_batch_mm(x.data_ptr(), weights.data_ptr(), out.data_ptr(), E, C, M, N, K, mode,
                                   _DT[x.dtype], ws.data_ptr(), ws.numel(), _stream())
        _lib.check(st, "batch_mm")
    return out


@torch.library.impl("yamoe_b200::batch_mm", "CUDA")
def _batch_mm_cuda(x, weights, batch_sizes, output, trans_b=False):
    """reference: csrc/batch_mm.cu:7-31.  x [E,C,K]; weights [E,K,N] or, with trans_b, [E,N,K];
    output [E,C,N].  `batch_sizes` is accepted and ignored, as in the reference."""
    _require(x.dim() == 3 and weights.dim() == 3 and output.dim() == 3, "batch_mm: 3D tensors expected")
    _require(x.dtype in _DT and weights.dtype == x.dtype and output.dtype == x.dtype, "batch_mm: dtype mismatch")
    _require(x.is_contiguous() and weights.is_contiguous() and output.is_contiguous(), "batch_mm: contiguous tensors expected")
    return _batch_mm_raw(x, weights, output, 1 if trans_b else 0)


def batch_mm_wgrad(x, y):
    """out[e] = x[e]^T @ y[e] for x [E,C,M], y [E,C,N]: the weight-gradient arrangement."""
    out = torch.empty(x.shape[0], x.shape[2], y.shape[2], dtype=x.dtype, device=x.device)
    return _batch_mm_raw(x.contiguous(), y.contiguous(), out, 2)


def permute_rows(src: torch.Tensor, sorted_indices: torch.Tensor, top_k: int) -> torch.Tensor:
    """rows[j] = src[sorted_indices[j] // top_k]: token rows in expert-sorted order."""
    _require(src.is_cuda and src.dim() == 2 and src.dtype in _DT, "permute_rows: 2D CUDA float32/bfloat16 expected")
    src, si = src.contiguous(), sorted_indices.contiguous()
    out = torch.empty(si.numel(), src.shape[1], dtype=src.dtype, device=src.device)
    with torch.cuda.device(src.device):
        st = _lib.lib().yamoe_b200_permute_rows(src.data_ptr(), src.shape[0], si.data_ptr(), out.data_ptr(),
                                                si.numel(), src.shape[1], int(top_k), _DT[src.dtype], _stream())
        _lib.check(st, "permute_rows")
    return out


def combine_rows(rows: torch.Tensor, sorted_indices: torch.Tensor, router_indices: torch.Tensor,
                 routing_weights: torch.Tensor, num_experts: int) -> torch.Tensor:
    """out[t] = sum_k w[t,k] * rows[position of assignment (t,k) in sorted_indices]."""
    T, K = router_indices.shape
    H = rows.shape[1]
    rows, si = rows.contiguous(), sorted_indices.contiguous()
    ri, rw = router_indices.to(torch.int64).contiguous(), routing_weights.contiguous()
    _require(rows.dtype in _DT and rw.dtype == rows.dtype, "combine_rows: dtype mismatch")
    out = torch.empty(T, H, dtype=rows.dtype, device=rows.device)
    with torch.cuda.device(rows.device):
        ws = _workspace(T * K * 4, rows.device)
        st = _lib.lib().yamoe_b200_combine_rows(rows.data_ptr(), si.data_ptr(), si.numel(), ri.data_ptr(),
                                                rw.data_ptr(), rw.shape[1], out.data_ptr(), T, H, int(num_experts), K,
                                                _DT[rows.dtype], ws.data_ptr(), ws.numel(), _stream())
        _lib.check(st, "combine_rows")
    return out


def router_topk(router_logits: torch.Tensor, top_k: int):
    """(router_indices [T,K] int64, router_scores [T,E]) from router logits [T,E]: top-k, softmax
    over the k selected logits, dense scatter, in one kernel (torch-ext/yamoe/layers.py:136-149)."""
    _require(router_logits.is_cuda and router_logits.dim() == 2 and router_logits.dtype in _DT,
             "router_topk: 2D CUDA float32/bfloat16 logits expected")
    logits = router_logits.contiguous()
    T, E = logits.shape
    idx = torch.empty(T, int(top_k), dtype=torch.int64, device=logits.device)
    scores = torch.empty_like(logits)
    with torch.cuda.device(logits.device):
        st = _lib.lib().yamoe_b200_router_topk(logits.data_ptr(), idx.data_ptr(), scores.data_ptr(), T, E, int(top_k),
                                               _DT[logits.dtype], _stream())
        _lib.check(st, "router_topk")
    return idx, scores


def router_forward(hidden_states: torch.Tensor, router_weight: torch.Tensor, router_bias, top_k: int):
    """(router_indices [T,K] int64, router_scores [T,E]) straight from the layer input: router
    projection, top-k, softmax over the k selected logits and dense scatter
    (torch-ext/yamoe/layers.py:126-149).  One kernel for bf16 (tcgen05 GEMM with the top-k in its
    epilogue); the CUDA-core GEMM plus the top-k kernel otherwise."""
    _require(hidden_states.is_cuda and hidden_states.dim() == 2 and hidden_states.dtype in _DT,
             "router_forward: 2D CUDA float32/bfloat16 hidden_states expected")
    _require(router_weight.dim() == 2 and router_weight.shape[1] == hidden_states.shape[1]
             and router_weight.dtype == hidden_states.dtype, "router_forward: router weight must be [E, H] of the same dtype")
    x, w = hidden_states.contiguous(), router_weight.contiguous()
    b = router_bias.contiguous() if router_bias is not None else None
    _require(b is None or (b.dtype == x.dtype and b.numel() == w.shape[0]), "router_forward: bias must be [E] of the same dtype")
    T, H = x.shape
    E = w.shape[0]
    idx = torch.empty(T, int(top_k), dtype=torch.int64, device=x.device)
    scores = torch.empty(T, E, dtype=x.dtype, device=x.device)
    L = _lib.lib()
    with torch.cuda.device(x.device):
        ws = _workspace(L.yamoe_b200_router_workspace_bytes(T, E), x.device)
        st = L.yamoe_b200_router_forward(x.data_ptr(), w.data_ptr(), b.data_ptr() if b is not None else None,
                                         idx.data_ptr(), scores.data_ptr(), T, H, E, int(top_k), _DT[x.dtype],
                                         ws.data_ptr(), ws.numel(), _stream())
        _lib.check(st, "router_forward")
        _check_device_status(ws, "router_forward")
    return idx, scores


experts = torch.ops.yamoe_b200.experts
batch_mm = torch.ops.yamoe_b200.batch_mm
experts_backward = torch.ops.yamoe_b200.experts_backward
sort = torch.ops.yamoe_b200.sort
gather = torch.ops.yamoe_b200.gather
scatter = torch.ops.yamoe_b200.scatter
index_select_out = torch.ops.yamoe_b200.index_select_out
bincount_cumsum = torch.ops.yamoe_b200.bincount_cumsum
