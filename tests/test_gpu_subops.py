"""The reference's small sub-operators on its padded [E, C, H] layout (`gather`, `scatter`,
`index_select_out`, schemas of torch-ext/torch_binding.cpp:9-48) against the CPU oracle and the
golden vectors made from yamoe_ref.py."""
import pytest
import torch

from oracle import experts_oracle as orc
from helpers import load_golden

pytestmark = pytest.mark.gpu


def _routing(T, E, K, seed):
    g = torch.Generator().manual_seed(seed)
    ri = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)])
    sv, si, counts, bins = orc.route_oracle(ri, E)
    return ri, si.to(torch.int32), bins[:E].to(torch.int32)


@pytest.mark.parametrize("cap", [37, 5])
def test_gather_scatter_match_golden(cap):
    import yamoe_b200
    g = load_golden("subops_small")
    T, H, E, K = g["dims"].tolist()
    si, bins = g["sorted_indices"].to(torch.int32).cuda(), g["bins"][:E].to(torch.int32).cuda()
    out = torch.full((E, cap, H), 7.0, device="cuda")
    yamoe_b200.gather(g["hidden_states"].cuda(), si, bins, out, E, cap, K)
    assert torch.equal(out.cpu(), g[f"gather_c{cap}"])
    sel = torch.gather(g["routing_weights"], 1, g["router_indices"]).reshape(-1)
    w_sorted = sel[g["sorted_indices"].long()].contiguous().cuda()
    y = torch.zeros(T, H, device="cuda")
    yamoe_b200.scatter(g[f"src_c{cap}"].cuda(), si, bins, w_sorted, y, T, E, cap, K)
    orc.check_close(y.cpu(), g[f"scatter_c{cap}"], 1e-5, "scatter vs yamoe_ref")
    y = torch.ones(T, H, device="cuda")           # accumulates into y; an empty weight tensor = no scaling
    yamoe_b200.scatter(g[f"src_c{cap}"].cuda(), si, bins, torch.empty(0, device="cuda"), y, T, E, cap, K)
    orc.check_close(y.cpu() - 1.0, g[f"scatter_plain_c{cap}"], 1e-5, "scatter without weights")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H,E,K,cap", [(300, 256, 8, 2, 64), (129, 36, 5, 3, 200), (64, 7, 4, 1, 3), (1, 8, 4, 2, 1)])
def test_gather_scatter_match_oracle(dtype, T, H, E, K, cap):
    """Vector and scalar paths (H = 36 and 7 are not multiples of the 16-byte vector), experts with no
    rows, capacity below and above the counts."""
    import yamoe_b200
    ri, si, bins = _routing(T, E, K, seed=T + H)
    gen = torch.Generator().manual_seed(1)
    x = torch.randn(T, H, generator=gen).to(dtype)
    out = torch.empty(E, cap, H, dtype=dtype, device="cuda")
    yamoe_b200.gather(x.cuda(), si.cuda(), bins.cuda(), out, E, cap, K)
    assert torch.equal(out.cpu(), orc.binned_gather_oracle(x, si, bins, E, cap, K))
    src = torch.randn(E, cap, H, generator=gen).to(dtype)
    w = torch.rand(T * K, generator=gen).to(dtype)
    y0 = torch.randn(T, H, generator=gen).to(dtype)
    y = y0.clone().cuda()
    yamoe_b200.scatter(src.cuda(), si.cuda(), bins.cuda(), w.cuda(), y, T, E, cap, K)
    ref = orc.binned_scatter_oracle(src, si, bins, w, y0, K)
    tol = 1e-5 if dtype == torch.float32 else 2e-2     # bf16: one rounding per addition, as in the reference
    orc.check_close(y.float().cpu(), ref.float(), tol, "scatter")


def test_scatter_single_slot_is_bit_exact_in_bf16():
    """With one addition per output element the rounding sequence is the reference's: product
    rounded to bf16, then one bf16 addition."""
    import yamoe_b200
    T, H, E, K, cap = 200, 64, 8, 1, 200
    ri, si, bins = _routing(T, E, K, seed=3)
    gen = torch.Generator().manual_seed(2)
    src = torch.randn(E, cap, H, generator=gen).bfloat16()
    w = torch.rand(T, generator=gen).bfloat16()
    y0 = torch.randn(T, H, generator=gen).bfloat16()
    y = y0.clone().cuda()
    yamoe_b200.scatter(src.cuda(), si.cuda(), bins.cuda(), w.cuda(), y, T, E, cap, K)
    ref = y0.clone()
    for e in range(E):
        start = int(bins[e - 1]) if e else 0
        for i in range(min(int(bins[e]) - start, cap)):
            tok = int(si[start + i]) // K
            ref[tok] = (ref[tok].float() + (src[e, i] * w[start + i]).float()).bfloat16()
    assert torch.equal(y.cpu(), ref)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_index_select_out(dtype):
    import yamoe_b200
    gen = torch.Generator().manual_seed(5)
    src = torch.randn(1000, generator=gen).to(dtype)
    idx = torch.randint(0, 1000, (4097,), generator=gen, dtype=torch.int32)
    out = torch.empty(4097, dtype=dtype, device="cuda")
    res = yamoe_b200.index_select_out(out, src.cuda(), idx.cuda())
    assert res.data_ptr() == out.data_ptr()
    assert torch.equal(out.cpu(), src[idx.long()])
    empty = torch.empty(0, dtype=dtype, device="cuda")
    yamoe_b200.index_select_out(empty, src.cuda(), torch.empty(0, dtype=torch.int32, device="cuda"))


def test_subop_argument_errors():
    import yamoe_b200
    x = torch.zeros(4, 8, device="cuda")
    si = torch.zeros(4, dtype=torch.int32, device="cuda")
    bins = torch.tensor([4, 4], dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match=r"\[E, C, H\]"):
        yamoe_b200.gather(x, si, bins, torch.empty(2, 3, 9, device="cuda"), 2, 3, 1)
    with pytest.raises(RuntimeError, match="int32"):
        yamoe_b200.gather(x, si.long(), bins, torch.empty(2, 3, 8, device="cuda"), 2, 3, 1)
    with pytest.raises(RuntimeError, match="idx must be int32"):
        yamoe_b200.index_select_out(torch.empty(4, device="cuda"), x.view(-1), si.long())
