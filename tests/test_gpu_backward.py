"""Backward parity of `experts_backward` (through the C ABI) against autograd through the
reference's training branch (golden vectors) and against the CPU oracle."""
import pytest
import torch

from oracle import experts_oracle as orc
from helpers import RTOL_BF16, RTOL_F32, SMALL_CASES, golden_inputs, load_golden

pytestmark = pytest.mark.gpu
GRADS = ["d_hidden", "d_routing", "d_wgu", "d_bgu", "d_wd", "d_bd"]


def run_backward(grad_out, inp, capacity, E, K, path="auto"):
    import yamoe_b200
    yamoe_b200.set_path(path)
    try:
        outs = yamoe_b200.experts_backward(grad_out.cuda(), *[t.cuda() for t in inp], capacity, E, K)
        torch.cuda.synchronize()
    finally:
        yamoe_b200.set_path("auto")
    return [o.cpu() for o in outs]


@pytest.mark.parametrize("name", SMALL_CASES)
def test_backward_fp32_golden(name):
    g = load_golden(name)
    T, H, E, K = g["dims"].tolist()
    grads = run_backward(g["grad_out"], golden_inputs(g), T, E, K)
    for got, key in zip(grads, GRADS):
        orc.check_close(got, g[key], RTOL_F32, key)


@pytest.mark.parametrize("name", SMALL_CASES)
def test_backward_fp32_golden_dropping_capacity(name):
    """Against autograd through the reference's binned_experts_ref with a capacity that drops rows."""
    g, d = load_golden(name), load_golden("drop_grads")
    T, H, E, K = g["dims"].tolist()
    grads = run_backward(g["grad_out"], golden_inputs(g), int(d[f"{name}_cap"]), E, K)
    for got, key in zip(grads, GRADS):
        orc.check_close(got, d[f"{name}_{key}"], RTOL_F32, key + " (dropping capacity)")


def test_backward_capacity_drop_and_slot_shapes():
    g = load_golden("small_c")
    T, H, E, K = g["dims"].tolist()
    cap = int(g["cap_small"])
    inp = golden_inputs(g)
    ref = orc.experts_backward_oracle(g["grad_out"], *inp, cap, E, K)
    got = run_backward(g["grad_out"], inp, cap, E, K)
    for a, b, key in zip(got, ref, GRADS):
        orc.check_close(a, b, RTOL_F32, key + " (capacity drop)")
    # [T,K] routing weights and [T,K,H] grad_out
    inp_k = list(inp)
    inp_k[2] = torch.gather(g["routing_weights"], 1, g["router_indices"])
    gk = (g["grad_out"].unsqueeze(1).repeat(1, K, 1) / K).contiguous()
    ref = orc.experts_backward_oracle(gk, *inp_k, T, E, K)
    got = run_backward(gk, inp_k, T, E, K)
    assert got[1].shape == (T, K)
    for a, b, key in zip(got, ref, GRADS):
        orc.check_close(a, b, RTOL_F32, key + " (per-slot shapes)")


@pytest.mark.parametrize("path", ["simt", "auto"])
@pytest.mark.parametrize("T,H,E,K", [(96, 64, 4, 2), (512, 128, 8, 2), (1024, 256, 32, 4)])
def test_backward_bf16(path, T, H, E, K):
    inp = orc.make_inputs(T, H, E, K, seed=T + 1, weight_std=1.6 / (H ** 0.5), bias_std=0.2, dtype=torch.bfloat16,
                          with_grad=True)
    keys = ["hidden_states", "router_indices", "routing_weights", "gate_up_proj", "gate_up_proj_bias",
            "down_proj", "down_proj_bias"]
    args = [inp[k] for k in keys]
    ref = orc.experts_backward_oracle(inp["grad_out"], *args, T, E, K)
    got = run_backward(inp["grad_out"], args, T, E, K, path=path)
    for a, b, key in zip(got, ref, GRADS):
        assert a.dtype == torch.bfloat16
        orc.check_close(a.float(), b, RTOL_BF16, f"{key} bf16 ({path})", rel_l2=2e-2)


def test_autograd_function_end_to_end():
    import yamoe_b200
    g = load_golden("small_b")
    T, H, E, K = g["dims"].tolist()
    inp = [t.cuda() for t in golden_inputs(g)]
    for i in (0, 2, 3, 4, 5, 6):
        inp[i].requires_grad_(True)
    out = yamoe_b200.experts_autograd(*inp, T, E, K, True)
    (out * g["grad_out"].cuda()).sum().backward()
    orc.check_close(out.detach().cpu(), g["out_train"], RTOL_F32, "forward")
    for i, key in zip((0, 2, 3, 4, 5, 6), GRADS):
        orc.check_close(inp[i].grad.cpu(), g[key], RTOL_F32, key)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_saved_activation_pair_matches_recompute(dtype):
    """forward_saving + backward_saved give the output and gradients of experts + experts_backward."""
    import yamoe_b200
    T, H, E, K = 700, 256, 8, 2
    inp = orc.make_inputs(T, H, E, K, seed=21, weight_std=0.1, bias_std=0.2, dtype=dtype, with_grad=True)
    keys = ["hidden_states", "router_indices", "routing_weights", "gate_up_proj", "gate_up_proj_bias",
            "down_proj", "down_proj_bias"]
    for cap in (T, 120):
        dev = [inp[k].cuda() for k in keys]
        for i in (0, 2, 3, 4, 5, 6):
            dev[i].requires_grad_(True)
        out = yamoe_b200.experts_autograd(*dev, cap, E, K, True, save_activations=True)
        (out.float() * inp["grad_out"].cuda().float()).sum().backward()
        ref_out = orc.experts_forward_oracle(*[inp[k] for k in keys], cap, E, K)
        ref_g = orc.experts_backward_oracle(inp["grad_out"], *[inp[k] for k in keys], cap, E, K)
        tol = RTOL_F32 if dtype == torch.float32 else RTOL_BF16
        orc.check_close(out.detach().float().cpu(), ref_out, tol, f"saved-mode forward (capacity {cap})")
        for i, r, name in zip((0, 2, 3, 4, 5, 6), ref_g, GRADS):
            orc.check_close(dev[i].grad.float().cpu(), r, tol, f"saved-mode {name} (capacity {cap})",
                            rel_l2=None if dtype == torch.float32 else 2e-2)
