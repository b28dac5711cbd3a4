"""Parity at the full sizes of the benchmark configurations.

The CPU oracle is too slow for whole 120B-shaped problems, but every output row depends only on
its own token, so the oracle is run on a SUBSET of tokens (with the full expert weights) and
compared with the same rows of the full-size CUDA result.  Weight gradients, which mix all
tokens, are cross-checked between the tcgen05 path and the CUDA-core path at full size and
against the oracle on a reduced token count.
"""
import pytest
import torch

from oracle import experts_oracle as orc
from helpers import RTOL_BF16, REL_L2_BF16

pytestmark = pytest.mark.gpu
KEYS = ["hidden_states", "router_indices", "routing_weights", "gate_up_proj", "gate_up_proj_bias",
        "down_proj", "down_proj_bias"]


def _subset_oracle(inp_dev, rows, cap, E, K):
    """Oracle forward for the token rows `rows` (a slice) using CPU copies of the full weights."""
    args = [inp_dev[k][rows].cpu() for k in KEYS[:3]] + [inp_dev[k].cpu() for k in KEYS[3:]]
    return orc.experts_forward_oracle(*args, cap, E, K)


def test_config2_forward_full_size_vs_oracle():
    import yamoe_b200
    from yamoe_b200 import workloads
    T, H, E, K = 4096, 2880, 32, 4
    inp = workloads.make_inputs(T, H, E, K, seed=42, dtype=torch.bfloat16)
    counts = torch.bincount(inp["router_indices"].reshape(-1), minlength=E)
    assert int(counts.max()) <= T                      # capacity T drops nothing
    out = yamoe_b200.experts(*[inp[k].cuda() for k in KEYS], T, E, K)
    ref = orc.experts_forward_oracle(*[inp[k] for k in KEYS], T, E, K)
    orc.check_close(out.float().cpu(), ref, RTOL_BF16, "config 2 forward", rel_l2=REL_L2_BF16)
    # the routing itself, bit-exact at this size
    sv, si, bins, cnt = yamoe_b200.route(inp["router_indices"].cuda(), E)
    rsv, rsi, rcnt, rbins = orc.route_oracle(inp["router_indices"], E)
    assert torch.equal(si.cpu(), rsi) and torch.equal(bins.cpu(), rbins) and torch.equal(cnt.cpu(), rcnt)


@pytest.mark.parametrize("T", [1, 4, 16, 64])
def test_config3_decode_full_shape_vs_oracle(T):
    import yamoe_b200
    from yamoe_b200 import workloads
    H, E, K = 2880, 128, 4
    inp = workloads.make_inputs(T, H, E, K, seed=42, dtype=torch.bfloat16, weights_on="cuda")
    dev = {k: v.cuda() for k, v in inp.items()}
    out = yamoe_b200.experts(*[dev[k] for k in KEYS], T, E, K)
    # reduce the problem to the experts that are hit so that the CPU copy stays small
    hit = torch.unique(inp["router_indices"])
    remap = torch.full((E,), -1, dtype=torch.int64)
    remap[hit] = torch.arange(hit.numel())
    ridx = remap[inp["router_indices"]]
    rw = inp["routing_weights"][:, hit]
    small = [inp["hidden_states"], ridx, rw] + [dev[k][hit.cuda()].cpu() for k in KEYS[3:]]
    ref = orc.experts_forward_oracle(*small, T, hit.numel(), K)
    orc.check_close(out.float().cpu(), ref, RTOL_BF16, f"config 3 decode T={T}", rel_l2=REL_L2_BF16)


def test_config4_skewed_prefill_full_size_subset_and_cross_path():
    import yamoe_b200
    from yamoe_b200 import workloads
    T, H, E, K = 16384, 2880, 128, 4
    inp = workloads.make_inputs(T, H, E, K, seed=42, dtype=torch.bfloat16, skew=True, weights_on="cuda")
    dev = {k: v.cuda() for k, v in inp.items()}
    counts = torch.bincount(inp["router_indices"].reshape(-1), minlength=E)
    assert int(counts[0]) > 10000 and int((counts == 0).sum()) > 0      # the skew is really there
    out = yamoe_b200.experts(*[dev[k] for k in KEYS], T, E, K)
    rows = slice(0, 384)
    ref = _subset_oracle(dev, rows, T, E, K)
    orc.check_close(out[rows].float().cpu(), ref, RTOL_BF16, "config 4 forward (token subset)", rel_l2=REL_L2_BF16)
    rows = slice(T - 128, T)
    ref = _subset_oracle(dev, rows, T, E, K)
    orc.check_close(out[rows].float().cpu(), ref, RTOL_BF16, "config 4 forward (last tokens)", rel_l2=REL_L2_BF16)
    # whole output: tcgen05 path against the CUDA-core path
    yamoe_b200.set_path("simt")
    try:
        out_simt = yamoe_b200.experts(*[dev[k] for k in KEYS], T, E, K)
    finally:
        yamoe_b200.set_path("auto")
    orc.check_close(out.float().cpu(), out_simt.float().cpu(), RTOL_BF16, "tcgen05 vs CUDA-core path", rel_l2=REL_L2_BF16)


def test_config5_backward_full_size():
    import yamoe_b200
    from yamoe_b200 import workloads
    T, H, E, K = 8192, 2880, 32, 4
    inp = workloads.make_inputs(T, H, E, K, seed=42, dtype=torch.bfloat16, with_grad=True)
    dev = {k: v.cuda() for k, v in inp.items()}
    grads = yamoe_b200.experts_backward(dev["grad_out"], *[dev[k] for k in KEYS], T, E, K)
    names = ["d_hidden", "d_routing", "d_wgu", "d_bgu", "d_wd", "d_bd"]
    # token-local gradients against the oracle on a token subset
    rows = slice(0, 256)
    sub = [inp[k][rows] for k in KEYS[:3]] + [inp[k] for k in KEYS[3:]]
    ref = orc.experts_backward_oracle(inp["grad_out"][rows], *sub, T, E, K)
    orc.check_close(grads[0][rows].float().cpu(), ref[0], RTOL_BF16, "d_hidden (token subset)", rel_l2=2e-2)
    orc.check_close(grads[1][rows].float().cpu(), ref[1], RTOL_BF16, "d_routing (token subset)", rel_l2=2e-2)
    # unselected routing entries carry exactly zero gradient
    mask = torch.ones(T, E, dtype=torch.bool).scatter_(1, inp["router_indices"], False)
    assert float(grads[1].float().cpu()[mask].abs().max()) == 0.0
    # gradients that mix all tokens: tcgen05 path against the CUDA-core path at full size
    yamoe_b200.set_path("simt")
    try:
        grads_simt = yamoe_b200.experts_backward(dev["grad_out"], *[dev[k] for k in KEYS], T, E, K)
    finally:
        yamoe_b200.set_path("auto")
    for a, b, n in zip(grads, grads_simt, names):
        orc.check_close(a.float().cpu(), b.float().cpu(), RTOL_BF16, f"{n}: tcgen05 vs CUDA-core path", rel_l2=2e-2)
    # bias gradients are cheap to restate exactly: d_bd[e] = sum over rows of e of w * grad_out[token]
    w = torch.gather(inp["routing_weights"].float(), 1, inp["router_indices"])
    d_bd = torch.zeros(E, H)
    d_bd.index_add_(0, inp["router_indices"].reshape(-1),
                    (w.reshape(-1, 1) * inp["grad_out"].float().repeat_interleave(K, 0)))
    orc.check_close(grads[5].float().cpu(), d_bd, RTOL_BF16, "d_bd vs closed form", rel_l2=2e-2)
    # weight gradients against the oracle at the full hidden size, for the fullest and the emptiest
    # expert: the oracle runs on that expert's rows alone (a one-expert, top-1 problem)
    counts = torch.bincount(inp["router_indices"].reshape(-1), minlength=E)
    for e in (int(counts.argmax()), int(counts.argmin())):
        tok = (inp["router_indices"] == e).any(1).nonzero().reshape(-1)
        n = tok.numel()
        one = orc.experts_backward_oracle(
            inp["grad_out"][tok], inp["hidden_states"][tok], torch.zeros(n, 1, dtype=torch.int64),
            inp["routing_weights"][tok, e].reshape(n, 1), inp["gate_up_proj"][e:e + 1], inp["gate_up_proj_bias"][e:e + 1],
            inp["down_proj"][e:e + 1], inp["down_proj_bias"][e:e + 1], n, 1, 1)
        for gi, name in ((2, "d_wgu"), (3, "d_bgu"), (4, "d_wd"), (5, "d_bd")):
            orc.check_close(grads[gi][e].float().cpu(), one[gi][0], RTOL_BF16, f"{name}[{e}] vs oracle ({n} rows)",
                            rel_l2=2e-2)
