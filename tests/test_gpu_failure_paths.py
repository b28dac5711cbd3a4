"""Failure paths of the CUDA library, exercised without faulting or hanging the GPU: a bounded
device-side wait that runs out, expert ids outside [0, E) through the whole operator, and the
opt-in device-status check of the operator binding."""
import ctypes

import pytest
import torch

from helpers import INPUT_KEYS
from oracle import experts_oracle as orc

pytestmark = pytest.mark.gpu


def test_bounded_mbarrier_wait_gives_up():
    """The pipeline wait of the grouped GEMM on a barrier nothing arrives at, limit 1 ms: the kernel
    must return, leave status 1 in the workspace header, and the GPU must stay usable."""
    from yamoe_b200 import _lib
    L = _lib.lib()
    ws = torch.zeros(256, dtype=torch.uint8, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(L.yamoe_b200_mbar_wait_probe(ws.data_ptr(), 1_000_000, st), "mbar_wait_probe")
    out = ctypes.c_int32(-1)
    _lib.check(L.yamoe_b200_device_status(ws.data_ptr(), st, ctypes.byref(out)), "device_status")
    assert out.value == 1
    with pytest.raises(RuntimeError, match="bounded device-side wait"):
        _lib.check_device_status(ws.data_ptr(), st, "probe")
    assert float((torch.ones(4, device="cuda") + 1).sum()) == 8.0


def test_status_check_passes_on_a_normal_call(monkeypatch):
    """YAMOE_B200_CHECK_STATUS=1: the binding reads the device status after the call; a normal call
    (tcgen05 path, bf16) reports 0 and returns the same result as without the check."""
    import yamoe_b200
    inp = orc.make_inputs(384, 128, 8, 2, seed=5, weight_std=0.1, bias_std=0.1, dtype=torch.bfloat16, with_grad=True)
    dev = [inp[k].cuda() for k in INPUT_KEYS]
    plain = yamoe_b200.experts(*dev, 384, 8, 2)
    monkeypatch.setenv("YAMOE_B200_CHECK_STATUS", "1")
    checked = yamoe_b200.experts(*dev, 384, 8, 2)
    grads = yamoe_b200.experts_backward(inp["grad_out"].cuda(), *dev, 384, 8, 2)
    assert torch.equal(plain, checked) and len(grads) == 6


@pytest.mark.parametrize("dtype,rtol", [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)])
def test_out_of_range_expert_ids_are_dropped(dtype, rtol):
    """Ids -1 and E (the reference's histogram ignores them, csrc/bincount_cumsum.cu:34): the
    assignment contributes nothing to the output and gets zero gradient; everything else equals the
    oracle run with those assignments given weight 0."""
    import yamoe_b200
    T, H, E, K = 200, 128, 8, 2
    inp = orc.make_inputs(T, H, E, K, seed=21, weight_std=0.1, bias_std=0.1, dtype=dtype, with_grad=True)
    ri = inp["router_indices"].clone()
    w_slots = torch.gather(inp["routing_weights"], 1, ri).contiguous()      # [T, K] per-slot weights
    bad = torch.zeros(T, K, dtype=torch.bool)
    bad[3, 0] = bad[17, 1] = bad[100, 0] = bad[100, 1] = True               # token 100 loses both slots
    ri_bad = ri.clone()
    ri_bad[3, 0], ri_bad[17, 1], ri_bad[100, 0], ri_bad[100, 1] = -1, E, E + 5, -7
    weights = [inp[k] for k in INPUT_KEYS[3:]]
    dev_w = [w.cuda() for w in weights]
    out = yamoe_b200.experts(inp["hidden_states"].cuda(), ri_bad.cuda(), w_slots.cuda(), *dev_w, T, E, K)
    grads = yamoe_b200.experts_backward(inp["grad_out"].cuda(), inp["hidden_states"].cuda(), ri_bad.cuda(),
                                        w_slots.cuda(), *dev_w, T, E, K)
    torch.cuda.synchronize()
    # oracle: the same assignments kept on a valid expert with weight 0 (large capacity: order is irrelevant)
    w_zero = w_slots.clone()
    w_zero[bad] = 0
    ref = orc.experts_forward_oracle(inp["hidden_states"], ri, w_zero, *weights, T * K, E, K)
    orc.check_close(out.float().cpu(), ref, rtol, "forward with out-of-range ids", rel_l2=1e-2 if dtype != torch.float32 else None)
    assert float(out[100].float().abs().max()) == 0.0
    ref_g = orc.experts_backward_oracle(inp["grad_out"], inp["hidden_states"], ri, w_zero, *weights, T * K, E, K)
    names = ["d_hidden", "d_routing", "d_wgu", "d_bgu", "d_wd", "d_bd"]
    for g, r, name in zip(grads, ref_g, names):
        g = g.float().cpu()
        if name == "d_routing":
            assert float(g[bad].abs().max()) == 0.0              # dropped assignments: zero gradient
            g, r = g.clone(), r.clone()
            g[bad] = 0
            r[bad] = 0
        orc.check_close(g, r, rtol, f"{name} with out-of-range ids", rel_l2=2e-2 if dtype != torch.float32 else None)


def test_route_marks_dropped_tail_and_helpers_skip_it():
    """yamoe_b200.route leaves -1 behind the kept entries; permute_rows / combine_rows given the
    whole arrays must neither read nor write out of bounds and must ignore the tail."""
    import yamoe_b200
    from yamoe_b200 import ops
    T, H, E, K = 64, 64, 8, 2
    inp = orc.make_inputs(T, H, E, K, seed=4, dtype=torch.float32)
    ri = inp["router_indices"].clone()
    ri[5, 1], ri[9, 0] = E, -1
    sv, si, bins, counts = yamoe_b200.route(ri.cuda(), E)
    n_kept = int(bins[E - 1])
    assert n_kept == T * K - 2
    assert (si[n_kept:] == -1).all() and (sv[n_kept:] == -1).all()
    x = inp["hidden_states"].cuda()
    rows = ops.permute_rows(x, si, K)
    assert torch.equal(rows[:n_kept], x[si[:n_kept].long() // K])
    assert float(rows[n_kept:].abs().max()) == 0.0
    w_slots = torch.gather(inp["routing_weights"], 1, inp["router_indices"]).cuda()
    out = ops.combine_rows(rows, si, ri.cuda(), w_slots, E)
    w_eff = w_slots.clone()
    w_eff[5, 1] = 0
    w_eff[9, 0] = 0
    ref = w_eff.sum(1, keepdim=True) * x
    assert (out - ref).abs().max() <= 1e-5 * ref.abs().max()
