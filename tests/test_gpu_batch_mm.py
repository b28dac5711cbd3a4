"""The grouped-GEMM kernels in isolation (batched matmul sub-operator) against torch fp32
matmuls of the same bf16-rounded operands, for each operand arrangement and both GEMM paths."""
import pytest
import torch

from oracle import experts_oracle as orc

pytestmark = pytest.mark.gpu


def _rand(shape, seed, dtype):
    return (torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * 0.25).to(dtype)


@pytest.mark.parametrize("path", ["simt", "auto"])
@pytest.mark.parametrize("E,C,K,N", [(1, 128, 64, 64), (2, 128, 128, 192), (3, 256, 320, 448), (4, 128, 64, 576)])
@pytest.mark.parametrize("trans_b", [False, True])
def test_batch_mm_rows(path, E, C, K, N, trans_b):
    import yamoe_b200
    x = _rand((E, C, K), 1, torch.bfloat16)
    w = _rand((E, N, K) if trans_b else (E, K, N), 2, torch.bfloat16)
    out = torch.empty(E, C, N, dtype=torch.bfloat16, device="cuda")
    yamoe_b200.set_path(path)
    try:
        yamoe_b200.batch_mm(x.cuda(), w.cuda(), torch.empty(0, device="cuda"), out, trans_b)
        torch.cuda.synchronize()
    finally:
        yamoe_b200.set_path("auto")
    ref = torch.bmm(x.float(), w.float().transpose(1, 2) if trans_b else w.float())
    orc.check_close(out.float().cpu(), ref, 1e-2, f"batch_mm trans_b={trans_b} {path}")


@pytest.mark.parametrize("path", ["simt", "auto"])
@pytest.mark.parametrize("E,C,M,N", [(1, 128, 64, 64), (2, 256, 128, 192), (3, 128, 320, 448)])
def test_batch_mm_wgrad(path, E, C, M, N):
    import yamoe_b200
    x = _rand((E, C, M), 3, torch.bfloat16)
    y = _rand((E, C, N), 4, torch.bfloat16)
    yamoe_b200.set_path(path)
    try:
        out = yamoe_b200.batch_mm_wgrad(x.cuda(), y.cuda())
        torch.cuda.synchronize()
    finally:
        yamoe_b200.set_path("auto")
    ref = torch.bmm(x.float().transpose(1, 2), y.float())
    orc.check_close(out.float().cpu(), ref, 1e-2, f"batch_mm wgrad {path}")


def test_batch_mm_fp32():
    import yamoe_b200
    x = _rand((2, 128, 64), 5, torch.float32)
    w = _rand((2, 64, 128), 6, torch.float32)
    out = torch.empty(2, 128, 128, device="cuda")
    yamoe_b200.batch_mm(x.cuda(), w.cuda(), torch.empty(0, device="cuda"), out, False)
    orc.check_close(out.cpu(), torch.bmm(x, w), 1e-5, "batch_mm fp32")


@pytest.mark.parametrize("switch", ["YAMOE_B200_2CTA=1", "YAMOE_B200_FUSED_GATHER=1", "YAMOE_B200_WIDE_TMA=0"])
def test_opt_in_kernel_variants_in_subprocess(switch):
    """The cta_group::2 GEMM, the forward with the gather fused into the gate_up GEMM (instead of the
    separate gather kernel) and the GEMMs with one TMA copy per 64-column box (instead of one per
    operand) are selected by environment variables read once per process."""
    import os
    import subprocess
    import sys
    code = (
        "import torch, yamoe_b200\n"
        "from yamoe_b200 import workloads\n"
        "from oracle import experts_oracle as orc\n"
        "g = torch.Generator().manual_seed(0)\n"
        "x = (torch.randn(3, 384, 320, generator=g) * 0.25).bfloat16(); w = (torch.randn(3, 320, 448, generator=g) * 0.25).bfloat16()\n"
        "out = torch.empty(3, 384, 448, dtype=torch.bfloat16, device='cuda')\n"
        "yamoe_b200.batch_mm(x.cuda(), w.cuda(), torch.empty(0, device='cuda'), out, False)\n"
        "orc.check_close(out.float().cpu(), torch.bmm(x.float(), w.float()), 1e-2, 'two-CTA batch_mm')\n"
        "wt = w.transpose(1, 2).contiguous()\n"
        "yamoe_b200.batch_mm(x.cuda(), wt.cuda(), torch.empty(0, device='cuda'), out, True)\n"
        "orc.check_close(out.float().cpu(), torch.bmm(x.float(), w.float()), 1e-2, 'two-CTA batch_mm trans_b')\n"
        "keys = ['hidden_states','router_indices','routing_weights','gate_up_proj','gate_up_proj_bias','down_proj','down_proj_bias']\n"
        "inp = workloads.make_inputs(700, 256, 8, 2, seed=4, weight_std=0.1, bias_std=0.2, dtype=torch.bfloat16)\n"
        "o = yamoe_b200.experts(*[inp[k].cuda() for k in keys], 700, 8, 2)\n"
        "ref = orc.experts_forward_oracle(*[inp[k] for k in keys], 700, 8, 2)\n"
        "orc.check_close(o.float().cpu(), ref, 2e-2, 'two-CTA forward', rel_l2=1e-2)\n"
        "inp = workloads.make_inputs(300, 128, 4, 2, seed=5, weight_std=0.1, bias_std=0.2, dtype=torch.bfloat16, with_grad=True)\n"
        "got = yamoe_b200.experts_backward(inp['grad_out'].cuda(), *[inp[k].cuda() for k in keys], 100, 4, 2)\n"
        "ref = orc.experts_backward_oracle(inp['grad_out'], *[inp[k] for k in keys], 100, 4, 2)\n"
        "for g, r, n in zip(got, ref, ['d_hidden', 'd_routing', 'd_wgu', 'd_bgu', 'd_wd', 'd_bd']):\n"
        "    orc.check_close(g.float().cpu(), r, 2e-2, 'variant backward ' + n, rel_l2=2e-2)\n"
        "print('ok')\n")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=root)
    name, _, value = switch.partition("=")
    env[name] = value
    res = subprocess.run([sys.executable, "-c", code], env=env, cwd=root, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and "ok" in res.stdout, res.stdout[-2000:] + res.stderr[-2000:]
