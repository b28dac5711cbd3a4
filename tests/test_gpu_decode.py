"""Decode-sized token counts: the weight-streaming GEMV path against the CPU oracle, and against
the grouped-GEMM path on the same inputs."""
import pytest
import torch

from oracle import experts_oracle as orc
from helpers import RTOL_BF16, REL_L2_BF16
from test_gpu_forward import run_experts

pytestmark = pytest.mark.gpu
KEYS = ["hidden_states", "router_indices", "routing_weights", "gate_up_proj", "gate_up_proj_bias",
        "down_proj", "down_proj_bias"]


@pytest.mark.parametrize("T", [1, 4, 16, 64])
def test_decode_gemv_120b_like(T):
    H, E, K = 512, 128, 4
    inp = orc.make_inputs(T, H, E, K, seed=42 + T, weight_std=0.05, bias_std=0.1, dtype=torch.bfloat16)
    args = [inp[k] for k in KEYS]
    ref = orc.experts_forward_oracle(*args, T, E, K)
    out = run_experts(args, T, E, K, path="gemv")
    orc.check_close(out.float(), ref, RTOL_BF16, f"gemv T={T}", rel_l2=REL_L2_BF16)
    auto = run_experts(args, T, E, K, path="auto")          # auto picks the GEMV path here
    assert torch.equal(auto, out) or (auto.float() - out.float()).abs().max() <= 2e-2 * ref.abs().max()


@pytest.mark.parametrize("T,H,E,K,cap", [(3, 64, 5, 2, 3), (7, 136, 4, 1, 2), (40, 64, 2, 2, 64), (9, 2880, 6, 3, 9),
                                          (128, 64, 8, 2, 128), (32, 64, 1, 1, 32)])
def test_decode_gemv_shapes_and_capacity(T, H, E, K, cap):
    inp = orc.make_inputs(T, H, E, K, seed=T * 7 + H, weight_std=1.0 / (H ** 0.5), bias_std=0.2,
                          dtype=torch.bfloat16)
    args = [inp[k] for k in KEYS]
    ref = orc.experts_forward_oracle(*args, cap, E, K)
    out = run_experts(args, cap, E, K, path="gemv")
    orc.check_close(out.float(), ref, RTOL_BF16, "gemv", rel_l2=REL_L2_BF16)


def test_decode_gemv_topk_weights():
    T, H, E, K = 5, 64, 16, 4
    inp = orc.make_inputs(T, H, E, K, seed=3, weight_std=0.1, bias_std=0.2, dtype=torch.bfloat16)
    args = [inp[k] for k in KEYS]
    ref = orc.experts_forward_oracle(*args, T, E, K)
    args[2] = torch.gather(inp["routing_weights"], 1, inp["router_indices"])
    out = run_experts(args, T, E, K, path="gemv")
    orc.check_close(out.float(), ref, RTOL_BF16, "gemv per-slot weights", rel_l2=REL_L2_BF16)
