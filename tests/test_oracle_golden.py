"""The CPU oracle against the golden vectors generated from the reference's own PyTorch
code (tests/golden/make_golden.py).  No GPU needed."""
import pytest
import torch

from oracle import experts_oracle as orc
from helpers import SMALL_CASES, golden_inputs, load_golden


@pytest.mark.parametrize("name", SMALL_CASES)
def test_routing_matches_golden(name):
    g = load_golden(name)
    T, H, E, K = g["dims"].tolist()
    sv, si, counts, bins = orc.route_oracle(g["router_indices"], E)
    assert torch.equal(sv, g["sorted_values"])
    assert torch.equal(si, g["sorted_indices"])
    assert torch.equal(bins, g["bins"])
    assert bins[E] == 0 and bins[E - 1] == T * K


@pytest.mark.parametrize("name", SMALL_CASES)
def test_forward_matches_reference_branches(name):
    g = load_golden(name)
    T, H, E, K = g["dims"].tolist()
    out = orc.experts_forward_oracle(*golden_inputs(g), T, E, K)
    orc.check_close(out, g["out_train"], 1e-5, "train branch")
    orc.check_close(out, g["out_eval"], 1e-4, "eval branch")
    out64 = orc.experts_forward_oracle(*golden_inputs(g), T, E, K, compute_dtype=torch.float64)
    orc.check_close(out64, g["out_train"], 1e-5, "fp64 oracle")


@pytest.mark.parametrize("name", SMALL_CASES)
def test_capacity_drop_matches_binned_reference(name):
    g = load_golden(name)
    T, H, E, K = g["dims"].tolist()
    out = orc.experts_forward_oracle(*golden_inputs(g), int(g["cap_small"]), E, K)
    orc.check_close(out, g["out_drop"], 1e-5, "capacity drop")
    # the drop really removes something in these cases
    assert (g["out_drop"] - g["out_train"]).abs().max() > 1e-3


@pytest.mark.parametrize("name", SMALL_CASES)
def test_backward_matches_autograd(name):
    g = load_golden(name)
    T, H, E, K = g["dims"].tolist()
    grads = orc.experts_backward_oracle(g["grad_out"], *golden_inputs(g), T, E, K)
    for got, key in zip(grads, ["d_hidden", "d_routing", "d_wgu", "d_bgu", "d_wd", "d_bd"]):
        orc.check_close(got, g[key], 2e-5, key)


def test_backward_topk_shaped_inputs():
    """[T,K] routing weights and [T,K,H] grad_out (csrc/experts_backward.cu:204-205,224-228)."""
    g = load_golden("small_a")
    T, H, E, K = g["dims"].tolist()
    inp = golden_inputs(g)
    sel = torch.gather(g["routing_weights"], 1, g["router_indices"])
    gk = g["grad_out"].unsqueeze(1).repeat(1, K, 1) / K
    inp_k = list(inp)
    inp_k[2] = sel
    grads = orc.experts_backward_oracle(gk, *inp_k, T, E, K)
    orc.check_close(grads[0], g["d_hidden"], 2e-5, "d_hidden")
    d_sel = torch.gather(g["d_routing"], 1, g["router_indices"])
    orc.check_close(grads[1], d_sel, 2e-5, "d_routing[T,K]")


def test_readme_workload_digest():
    g = load_golden("readme_digest")
    inp = orc.make_readme_inputs(batch=2)
    assert torch.equal(inp["hidden_states"][0, :8], g["hidden_head"]), "seeded inputs changed"
    sv, si, counts, bins = orc.route_oracle(inp["router_indices"], 8)
    assert torch.equal(counts, g["counts"]) and torch.equal(bins, g["bins"])
    assert torch.equal(si[:64], g["sorted_indices_head"])
    assert int(counts.max()) <= 256          # capacity 256 drops nothing in this workload
    out = orc.experts_forward_oracle(inp["hidden_states"], inp["router_indices"], inp["routing_weights"],
                                     inp["gate_up_proj"], inp["gate_up_proj_bias"], inp["down_proj"],
                                     inp["down_proj_bias"], 256, 8, 2)
    scale = g["absmax"]
    assert (out[::16, ::45] - g["sub_train"]).abs().max() <= 1e-4 * scale
    assert (out[::16, ::45] - g["sub_eval"]).abs().max() <= 1e-4 * scale
    assert (out.double().sum(1) - g["rowsum_train"]).abs().max() <= 1e-4 * scale * 54


@pytest.mark.parametrize("cap", [37, 5])
def test_binned_gather_scatter_oracles_match_reference(cap):
    """binned_gather / binned_scatter of the reference's yamoe_ref.py (full and dropping capacity)."""
    g = load_golden("subops_small")
    T, H, E, K = g["dims"].tolist()
    si, bins = g["sorted_indices"], g["bins"]
    out = orc.binned_gather_oracle(g["hidden_states"], si, bins, E, cap, K)
    assert torch.equal(out, g[f"gather_c{cap}"])
    sel = torch.gather(g["routing_weights"], 1, g["router_indices"]).reshape(-1)
    w_sorted = sel[si.long()]
    src = g[f"src_c{cap}"]
    y = orc.binned_scatter_oracle(src, si, bins, w_sorted, torch.zeros(T, H), K)
    orc.check_close(y, g[f"scatter_c{cap}"], 1e-6, "binned_scatter")
    y1 = orc.binned_scatter_oracle(src, si, bins, None, torch.zeros(T, H), K)
    orc.check_close(y1, g[f"scatter_plain_c{cap}"], 1e-6, "binned_scatter without weights")


@pytest.mark.parametrize("name", SMALL_CASES)
def test_backward_under_dropping_capacity_matches_autograd(name):
    """Gradients through the reference's binned_experts_ref with a capacity that drops rows:
    dropped assignments contribute no gradient anywhere."""
    g, d = load_golden(name), load_golden("drop_grads")
    T, H, E, K = g["dims"].tolist()
    cap = int(d[f"{name}_cap"])
    assert cap == int(g["cap_small"])
    grads = orc.experts_backward_oracle(g["grad_out"], *golden_inputs(g), cap, E, K)
    for got, key in zip(grads, ["d_hidden", "d_routing", "d_wgu", "d_bgu", "d_wd", "d_bd"]):
        orc.check_close(got, d[f"{name}_{key}"], 2e-5, key + " (dropping capacity)")
    # the drop really changes the gradients
    assert (d[f"{name}_d_hidden"] - g["d_hidden"]).abs().max() > 1e-3
