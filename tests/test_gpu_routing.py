"""Routing kernels against the CPU oracle: bit-exact sorted order, histogram and prefix sums."""
import pytest
import torch

from oracle import experts_oracle as orc
from helpers import SMALL_CASES, load_golden

pytestmark = pytest.mark.gpu


def _check(idx, E):
    import yamoe_b200
    sv, si, bins, counts = yamoe_b200.route(idx.cuda(), E)
    rsv, rsi, rcounts, rbins = orc.route_oracle(idx, E)
    assert torch.equal(sv.cpu(), rsv)
    assert torch.equal(si.cpu(), rsi)
    assert torch.equal(bins.cpu(), rbins)
    assert torch.equal(counts.cpu(), rcounts)


@pytest.mark.parametrize("name", SMALL_CASES)
def test_route_golden(name):
    g = load_golden(name)
    T, H, E, K = g["dims"].tolist()
    _check(g["router_indices"], E)


@pytest.mark.parametrize("T,E,K", [(1, 1, 1), (1, 128, 4), (5, 3, 2), (37, 2, 1), (64, 128, 4), (513, 8, 2),
                                   (4096, 32, 4), (16384, 128, 4), (1000, 1024, 3), (2049, 5, 1)])
def test_route_random(T, E, K):
    gen = torch.Generator().manual_seed(T * 131 + E)
    idx = torch.stack([torch.randperm(E, generator=gen)[:K] for _ in range(T)]) if E >= K and T <= 600 \
        else torch.randint(0, E, (T, K), generator=gen)
    _check(idx, E)


def test_route_skewed_and_empty_experts():
    gen = torch.Generator().manual_seed(7)
    idx = torch.randint(0, 4, (3000, 2), generator=gen) * 5      # only experts 0,5,10,15 are hit
    _check(idx, 32)
    _check(torch.full((5000, 1), 17, dtype=torch.int64), 32)      # one expert takes everything


def test_route_is_deterministic():
    import yamoe_b200
    idx = torch.randint(0, 128, (16384, 4), generator=torch.Generator().manual_seed(3)).cuda()
    a = yamoe_b200.route(idx, 128)
    for _ in range(5):
        b = yamoe_b200.route(idx, 128)
        assert all(torch.equal(x, y) for x, y in zip(a, b))


def test_sort_and_bincount_cumsum_ops():
    """The sub-operators keep the reference's calling convention (torch-ext/torch_binding.cpp:31-42)."""
    import yamoe_b200
    x = torch.randint(0, 32, (16384,), dtype=torch.int32, generator=torch.Generator().manual_seed(1)).cuda()
    x_out, iota = torch.empty_like(x), torch.empty_like(x)
    yamoe_b200.sort(x, 32, x_out, iota)
    rv, ri = torch.sort(x.cpu().long(), stable=True)
    assert torch.equal(x_out.cpu().long(), rv) and torch.equal(iota.cpu().long(), ri)
    bins = torch.empty(33, dtype=torch.int32, device="cuda")
    yamoe_b200.bincount_cumsum(x_out, bins, 32)
    ref = torch.cumsum(torch.bincount(x.cpu().long(), minlength=32), 0)
    assert torch.equal(bins[:32].cpu().long(), ref) and int(bins[32]) == 0
