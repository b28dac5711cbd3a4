"""Forward parity of the CUDA op (called through the C ABI) against the golden vectors and the
CPU oracle."""
import pytest
import torch

from oracle import experts_oracle as orc
from helpers import RTOL_BF16, RTOL_F32, REL_L2_BF16, SMALL_CASES, golden_inputs, load_golden

pytestmark = pytest.mark.gpu


def run_experts(inp, capacity, E, K, path="auto", dtype=None):
    import yamoe_b200
    yamoe_b200.set_path(path)
    try:
        args = [t.cuda() if dtype is None or not t.is_floating_point() else t.to(dtype).cuda() for t in inp]
        out = yamoe_b200.experts(*args, capacity, E, K)
        torch.cuda.synchronize()
    finally:
        yamoe_b200.set_path("auto")
    return out.cpu()


@pytest.mark.parametrize("name", SMALL_CASES)
def test_forward_fp32_golden(name):
    g = load_golden(name)
    T, H, E, K = g["dims"].tolist()
    out = run_experts(golden_inputs(g), T, E, K)
    orc.check_close(out, g["out_train"], RTOL_F32, "fp32 forward vs reference training branch")
    orc.check_close(out, g["out_eval"], RTOL_F32, "fp32 forward vs reference eval branch")


@pytest.mark.parametrize("name", SMALL_CASES)
def test_forward_capacity_drop(name):
    g = load_golden(name)
    T, H, E, K = g["dims"].tolist()
    out = run_experts(golden_inputs(g), int(g["cap_small"]), E, K)
    orc.check_close(out, g["out_drop"], RTOL_F32, "capacity drop vs binned reference")


def test_forward_topk_shaped_weights():
    g = load_golden("small_a")
    T, H, E, K = g["dims"].tolist()
    inp = golden_inputs(g)
    inp[2] = torch.gather(g["routing_weights"], 1, g["router_indices"])
    out = run_experts(inp, T, E, K)
    orc.check_close(out, g["out_train"], RTOL_F32, "per-slot routing weights")


def test_forward_zero_capacity_and_empty():
    g = load_golden("small_a")
    T, H, E, K = g["dims"].tolist()
    out = run_experts(golden_inputs(g), 0, E, K)
    assert out.abs().max() == 0
    inp = [t[:0] if i < 3 else t for i, t in enumerate(golden_inputs(g))]
    assert run_experts(inp, 4, E, K).shape == (0, H)


def test_forward_readme_workload_fp32():
    """T=512, H=2880, E=8, K=2, N(0,1) weights: the clamps fire constantly, outputs reach ~5e3."""
    inp = orc.make_readme_inputs(batch=2)
    keys = ["hidden_states", "router_indices", "routing_weights", "gate_up_proj", "gate_up_proj_bias",
            "down_proj", "down_proj_bias"]
    out = run_experts([inp[k] for k in keys], 256, 8, 2)
    g = load_golden("readme_digest")
    scale = g["absmax"]
    assert (out[::16, ::45] - g["sub_train"]).abs().max() <= RTOL_F32 * scale
    ref = orc.experts_forward_oracle(*[inp[k] for k in keys], 256, 8, 2)
    orc.check_close(out, ref, RTOL_F32, "README workload vs oracle")


@pytest.mark.parametrize("path", ["simt", "auto"])
@pytest.mark.parametrize("T,H,E,K", [(96, 64, 4, 2), (300, 128, 8, 2), (1024, 256, 32, 4)])
def test_forward_bf16(path, T, H, E, K):
    inp = orc.make_inputs(T, H, E, K, seed=T, weight_std=0.2 / (H ** 0.5) * 8, bias_std=0.2, dtype=torch.bfloat16)
    keys = ["hidden_states", "router_indices", "routing_weights", "gate_up_proj", "gate_up_proj_bias",
            "down_proj", "down_proj_bias"]
    args = [inp[k] for k in keys]
    out = run_experts(args, T, E, K, path=path)
    assert out.dtype == torch.bfloat16
    ref = orc.experts_forward_oracle(*args, T, E, K)     # fp32 arithmetic on the bf16-rounded inputs
    orc.check_close(out.float(), ref, RTOL_BF16, f"bf16 forward ({path})", rel_l2=REL_L2_BF16)


def test_validation_errors():
    import yamoe_b200
    g = load_golden("small_a")
    T, H, E, K = g["dims"].tolist()
    inp = [t.cuda() for t in golden_inputs(g)]
    with pytest.raises(RuntimeError, match="hidden_states must be 2D"):
        yamoe_b200.experts(inp[0].view(1, T, H), *inp[1:], T, E, K)
    with pytest.raises(RuntimeError, match="routing_weights must be"):
        yamoe_b200.experts(inp[0], inp[1], inp[2][:, :3], *inp[3:], T, E, K)
    with pytest.raises(RuntimeError, match="must be on CUDA"):
        yamoe_b200.experts(inp[0].cpu(), *inp[1:], T, E, K)


@pytest.mark.parametrize("dtype,cos,rel", [(torch.float32, 0.999999, 1e-5), (torch.bfloat16, 0.9999, 1e-2)])
def test_compare_table_metrics(dtype, cos, rel, capsys):
    """The metric table of the reference's compare_example.py, op against oracle."""
    import compare_table
    r = compare_table.compare(256, 256, 8, 2, dtype, iters=2)
    compare_table.print_table(r)
    text = capsys.readouterr().out
    assert "Cosine Similarity" in text and "Max Abs Diff" in text
    assert r["cosine"] > cos and r["rel_l2"] < rel
