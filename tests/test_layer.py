"""The layer front-end (router + experts): oracle against the golden vectors of the reference's
GptOssMLP on CPU; the CUDA `Yamoe` module and the fused router kernel on GPU."""
import types

import pytest
import torch

from oracle import experts_oracle as orc
from helpers import load_golden


def _golden_layer():
    g = load_golden("mlp_small")
    T, H, E, K = g["dims"].tolist()
    return g, T, H, E, K


def test_router_and_layer_oracle_match_reference_mlp():
    g, T, H, E, K = _golden_layer()
    x = g["x"].reshape(T, H)
    scores, idx = orc.router_oracle(x, g["router_weight"], g["router_bias"], K)
    orc.check_close(scores, g["scores"], 1e-5, "router scores")
    out = orc.experts_forward_oracle(x, idx, scores, g["gate_up_proj"], g["gate_up_proj_bias"], g["down_proj"],
                                     g["down_proj_bias"], T, E, K)
    orc.check_close(out, g["out"].reshape(T, H), 1e-5, "layer output")


def _module(g, E, K, dtype=torch.float32, capacity=None):
    import yamoe_b200
    m = yamoe_b200.Yamoe()
    m.router = types.SimpleNamespace(weight=g["router_weight"].to(dtype).cuda(), bias=g["router_bias"].to(dtype).cuda())
    m.experts = types.SimpleNamespace(**{k: g[k].to(dtype).cuda() for k in
                                         ["gate_up_proj", "gate_up_proj_bias", "down_proj", "down_proj_bias"]})
    m.num_experts, m.top_k = E, K
    if capacity is not None:
        m.expert_capacity = capacity
    return m


@pytest.mark.gpu
def test_router_topk_kernel():
    import yamoe_b200
    for T, E, K, dtype in ((48, 8, 2, torch.float32), (1000, 32, 4, torch.float32), (257, 128, 4, torch.bfloat16),
                           (5, 1024, 8, torch.float32), (3, 5, 5, torch.float32)):
        logits = torch.randn(T, E, generator=torch.Generator().manual_seed(T)).to(dtype)
        idx, scores = yamoe_b200.router_topk(logits.cuda(), K)
        top_v, ref_idx = torch.topk(logits.float(), K, dim=-1)
        ref_scores = torch.zeros(T, E).scatter_(1, ref_idx, torch.softmax(top_v, -1))
        if dtype == torch.float32:
            assert torch.equal(idx.cpu(), ref_idx)
        else:   # bf16 logits can tie; compare the selected values instead of the ids
            assert torch.equal(torch.gather(logits.float(), 1, idx.cpu()), top_v)
        tol = 1e-6 if dtype == torch.float32 else 1e-2
        # compare the K score values per row (ids may differ where bf16 logits tie)
        got_sorted = scores.float().cpu().sort(dim=1, descending=True).values[:, :K]
        ref_sorted = ref_scores.sort(dim=1, descending=True).values[:, :K]
        assert (got_sorted - ref_sorted).abs().max() <= tol
        assert (torch.gather(scores.float().cpu(), 1, idx.cpu()) > 0).all()
        assert int((scores != 0).sum(1).max()) <= K


@pytest.mark.gpu
def test_router_forward_matches_linear_topk_softmax():
    """Router projection + top-k + softmax + scatter in the library against the reference layer's
    chain (torch-ext/yamoe/layers.py:126-149) in torch: fp32 through the CUDA-core GEMM and the top-k
    kernel, bf16 through the single tcgen05 kernel (H a multiple of 64, K <= 8; one and four column
    chunks per row), through the two-kernel form (H = 72, or K = 12), and both types through the
    one-CTA-per-token kernel (T <= 64)."""
    import yamoe_b200
    for T, H, E, K, dtype in ((300, 256, 32, 4, torch.float32), (1, 128, 8, 2, torch.float32),
                              (1000, 2880, 32, 4, torch.bfloat16), (130, 256, 128, 4, torch.bfloat16),
                              (5, 128, 48, 3, torch.bfloat16), (64, 72, 16, 2, torch.bfloat16),
                              (200, 72, 16, 2, torch.bfloat16), (200, 256, 64, 12, torch.bfloat16),
                              (4, 2880, 128, 4, torch.bfloat16), (129, 128, 40, 8, torch.bfloat16)):
        gen = torch.Generator().manual_seed(T + E)
        x = torch.randn(T, H, generator=gen).to(dtype)
        w = (torch.randn(E, H, generator=gen) / H ** 0.5).to(dtype)
        b = (torch.randn(E, generator=gen) * 0.1).to(dtype)
        idx, scores = yamoe_b200.router_forward(x.cuda(), w.cuda(), b.cuda(), K)
        idx, scores = idx.cpu(), scores.float().cpu()
        logits = torch.nn.functional.linear(x.cuda(), w.cuda(), b.cuda()).float().cpu()     # same dtype rounding
        top_v, ref_idx = torch.topk(logits, K, dim=-1)
        assert ((idx >= 0) & (idx < E)).all()
        if dtype == torch.float32:
            # selections agree wherever the k-th and (k+1)-th logits are not within rounding of each other
            sorted_v = logits.sort(dim=1, descending=True).values
            clear = (sorted_v[:, K - 1] - sorted_v[:, K]) > 1e-5 if E > K else torch.ones(T, dtype=torch.bool)
            assert torch.equal(idx[clear].sort(1).values, ref_idx[clear].sort(1).values)
            tol = 2e-5
        else:
            # bf16 logits tie often and the accumulation order differs from cuBLAS by an ulp here and
            # there: compare the selected logit values and the scores, not the ids
            got_v = torch.gather(logits, 1, idx)
            assert (got_v.sort(1, descending=True).values - top_v).abs().max() <= 2e-2 * logits.abs().max()
            tol = 2e-2
        ref_scores = torch.zeros(T, E).scatter_(1, ref_idx, torch.softmax(top_v, -1))
        got_sorted = scores.sort(dim=1, descending=True).values[:, :K]
        ref_sorted = ref_scores.sort(dim=1, descending=True).values[:, :K]
        assert (got_sorted - ref_sorted).abs().max() <= tol, (T, H, E, K, dtype)
        assert int((scores != 0).sum(1).max()) <= K
        assert ((scores.sum(1) - 1).abs() <= 2e-2).all()


@pytest.mark.gpu
def test_router_topk_non_finite_logits():
    """NaN rows and rows with fewer than K finite logits: every selected id must be a valid expert
    and nothing may be written outside the [T, E] score row, as with torch.topk."""
    import yamoe_b200
    T, E, K = 6, 16, 4
    logits = torch.randn(T, E, generator=torch.Generator().manual_seed(1))
    logits[0] = float("nan")                       # a whole NaN row
    logits[1, 3] = float("nan")                    # one NaN: ranks first, as in torch.topk
    logits[2] = float("-inf"); logits[2, 5] = 1.0; logits[2, 9] = 0.5      # two finite logits, K = 4
    logits[3] = float("-inf")                      # nothing finite at all
    guard = torch.full((T * E + 64,), 7.0, device="cuda")
    scores_buf = guard[:T * E].view(T, E)
    from yamoe_b200 import _lib
    idx = torch.full((T, K), -5, dtype=torch.int64, device="cuda")
    _lib.check(_lib.lib().yamoe_b200_router_topk(logits.cuda().data_ptr(), idx.data_ptr(), scores_buf.data_ptr(), T, E, K,
                                                 _lib.YAMOE_F32, torch.cuda.current_stream().cuda_stream), "router_topk")
    torch.cuda.synchronize()
    idx = idx.cpu()
    assert ((idx >= 0) & (idx < E)).all(), idx
    assert (guard[T * E:] == 7.0).all()            # nothing stored past the score rows
    for t in range(T):
        assert len(set(idx[t].tolist())) == K      # K distinct experts per row
    assert idx[1, 0] == 3
    assert set(idx[2, :2].tolist()) == {5, 9}
    ref_v, ref_i = torch.topk(logits[4:], K, dim=-1)
    assert torch.equal(idx[4:], ref_i)
    ref = torch.zeros(2, E).scatter_(1, ref_i, torch.softmax(ref_v, -1))
    assert (scores_buf[4:].cpu() - ref).abs().max() <= 1e-6
    s2 = scores_buf[2].cpu()
    assert abs(float(s2[5]) - float(torch.softmax(torch.tensor([1.0, 0.5]), 0)[0])) <= 1e-6
    assert torch.isnan(scores_buf[0].cpu()[idx[0]]).all()


@pytest.mark.gpu
def test_router_forward_non_finite_inputs():
    """NaN and infinite activations through the fused router kernels (few-token form, tensor-core
    form with one and with four column chunks): K distinct valid experts per row, finite rows
    untouched by their neighbours, nothing written outside the outputs."""
    import yamoe_b200
    for T, H, E, K in ((8, 128, 16, 4), (200, 128, 32, 4), (200, 128, 128, 4)):
        gen = torch.Generator().manual_seed(T + E)
        x = torch.randn(T, H, generator=gen).bfloat16()
        w = (torch.randn(E, H, generator=gen) / H ** 0.5).bfloat16()
        b = (torch.randn(E, generator=gen) * 0.1).bfloat16()
        x[0] = float("nan")                        # every logit of the row is NaN
        x[1, 7] = float("inf")                     # logits are +inf, -inf or NaN depending on the weight's sign
        idx, scores = yamoe_b200.router_forward(x.cuda(), w.cuda(), b.cuda(), K)
        torch.cuda.synchronize()
        idx, scores = idx.cpu(), scores.float().cpu()
        assert ((idx >= 0) & (idx < E)).all(), (T, E, idx[:2])
        for t in range(T):
            assert len(set(idx[t].tolist())) == K, (T, E, t, idx[t])
        clean = torch.ones(T, dtype=torch.bool); clean[:2] = False
        assert torch.isfinite(scores[clean]).all()
        assert ((scores[clean].sum(1) - 1).abs() <= 2e-2).all()
        assert int((scores[clean] != 0).sum(1).max()) <= K
        logits = torch.nn.functional.linear(x[clean].cuda(), w.cuda(), b.cuda()).float().cpu()
        top_v = torch.topk(logits, K, dim=-1).values
        got_v = torch.gather(logits, 1, idx[clean])
        assert (got_v.sort(1, descending=True).values - top_v).abs().max() <= 2e-2 * logits.abs().max()


@pytest.mark.gpu
def test_yamoe_module_matches_reference_mlp():
    g, T, H, E, K = _golden_layer()
    m = _module(g, E, K, capacity=T)
    with torch.no_grad():
        out, scores = m(g["x"].cuda())
    orc.check_close(scores.cpu(), g["scores"], 1e-5, "router scores")
    orc.check_close(out.cpu(), g["out"], 1e-4, "layer output vs GptOssMLP")


@pytest.mark.gpu
def test_yamoe_module_default_capacity_and_grads():
    g, T, H, E, K = _golden_layer()
    x = g["x"].reshape(T, H)
    scores, idx = orc.router_oracle(x, g["router_weight"], g["router_bias"], K)
    cap = -(-T * K // E)                                   # reference formula, layers.py:162
    ref = orc.experts_forward_oracle(x, idx, scores, g["gate_up_proj"], g["gate_up_proj_bias"], g["down_proj"],
                                     g["down_proj_bias"], cap, E, K)
    m = _module(g, E, K)
    with torch.no_grad():
        out, _ = m(g["x"].cuda())
    orc.check_close(out.cpu().reshape(T, H), ref, 1e-4, "default capacity (drops)")
    # with autograd recording, gradients reach the input, the router and the experts
    m = _module(g, E, K, capacity=T)
    for t in (m.router.weight, m.router.bias, m.experts.gate_up_proj, m.experts.down_proj):
        t.requires_grad_(True)
    xin = g["x"].cuda().requires_grad_(True)
    out, _ = m(xin)
    out.square().sum().backward()
    # reference gradients by autograd through the oracle on CPU
    xr = g["x"].clone().requires_grad_(True)
    rw_, rb_ = g["router_weight"].clone().requires_grad_(True), g["router_bias"].clone().requires_grad_(True)
    sc, ix = orc.router_oracle(xr.reshape(T, H), rw_, rb_, K)
    wgu = g["gate_up_proj"].clone().requires_grad_(True)
    o = torch.zeros(T, H)
    sel = torch.gather(sc, 1, ix)
    for k in range(K):
        e = ix[:, k]
        pre = torch.einsum("th,thn->tn", xr.reshape(T, H), wgu[e]) + g["gate_up_proj_bias"][e]
        y = torch.einsum("th,thn->tn", orc.glu(pre), g["down_proj"][e]) + g["down_proj_bias"][e]
        o = o + sel[:, k:k + 1] * y
    o.square().sum().backward()
    orc.check_close(xin.grad.cpu(), xr.grad, 1e-3, "d input")
    orc.check_close(m.router.weight.grad.cpu(), rw_.grad, 1e-3, "d router weight")
    orc.check_close(m.experts.gate_up_proj.grad.cpu(), wgu.grad, 1e-3, "d gate_up_proj")
