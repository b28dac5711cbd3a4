"""`yamoe_b200_route_static`: routing for hosts that cannot provide (or allocate) a workspace.

Some integrations only ever hand the library input and output buffers: their device memory pool is
sized once at start-up and nothing may call an allocator afterwards.  For them the library keeps
the routing scratch in a fixed 1 MiB array of its own.  This test drives that entry point through
the C ABI and checks that it returns exactly what the workspace-taking `yamoe_b200_route` returns,
on two consecutive calls (the scratch array keeps the first call's contents, so the second call
proves the per-call clearing), and that an oversized request is refused without launching.

The file name sorts last on purpose: a run that stops at the first failure has then already
executed every other test.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _route_workspace(L, idx, E):
    S = idx.numel()
    opts = dict(dtype=torch.int32, device="cuda")
    sv, si = torch.empty(S, **opts), torch.empty(S, **opts)
    bins, counts = torch.empty(E + 1, **opts), torch.empty(E, **opts)
    n = L.yamoe_b200_route_workspace_bytes(S, E, 1)
    ws = torch.empty(n, dtype=torch.uint8, device="cuda")
    st = L.yamoe_b200_route(idx.data_ptr(), sv.data_ptr(), si.data_ptr(), bins.data_ptr(), counts.data_ptr(),
                            S, E, 1, ws.data_ptr(), n, torch.cuda.current_stream().cuda_stream)
    assert st == 0
    return sv, si, bins, counts


def _route_static(L, idx, E):
    S = idx.numel()
    opts = dict(dtype=torch.int32, device="cuda")
    sv, si = torch.full((S,), -7, **opts), torch.full((S,), -7, **opts)
    bins, counts = torch.full((E + 1,), -7, **opts), torch.full((E,), -7, **opts)
    st = L.yamoe_b200_route_static(idx.data_ptr(), sv.data_ptr(), si.data_ptr(), bins.data_ptr(),
                                   counts.data_ptr(), S, E, 1, torch.cuda.current_stream().cuda_stream)
    assert st == 0, L.yamoe_b200_status_string(st)
    return sv, si, bins, counts


def test_route_static_matches_route_on_two_calls_in_a_row():
    from yamoe_b200 import _lib
    L = _lib.lib()
    gen = torch.Generator().manual_seed(5)
    first = torch.randint(0, 128, (16384 * 4,), generator=gen).cuda()       # 32 blocks, 128 experts
    second = torch.randint(0, 7, (5000,), generator=gen).cuda()             # different size and E
    for idx, E in ((first, 128), (second, 7)):
        want = _route_workspace(L, idx, E)
        got = _route_static(L, idx, E)
        torch.cuda.synchronize()
        for w, g, name in zip(want, got, ["sorted_values", "sorted_indices", "bins", "counts"]):
            assert torch.equal(w, g), f"{name} differs from yamoe_b200_route"
    # and once more with the first input: leftovers of the smaller call must not leak in
    want, got = _route_workspace(L, first, 128), _route_static(L, first, 128)
    torch.cuda.synchronize()
    assert all(torch.equal(w, g) for w, g in zip(want, got))


def test_route_static_refuses_requests_beyond_its_scratch():
    from yamoe_b200 import _lib
    L = _lib.lib()
    T, E = 4 * 1024 * 1024, 1024                       # 2048 blocks * 1024 experts * 4 B = 8 MiB
    assert L.yamoe_b200_route_static_scratch_needed(T, E, 1) > (1 << 20)
    dummy = torch.zeros(8, dtype=torch.int64, device="cuda")
    out = torch.zeros(2048, dtype=torch.int32, device="cuda")
    st = L.yamoe_b200_route_static(dummy.data_ptr(), out.data_ptr(), out.data_ptr(), out.data_ptr(), None,
                                   T, E, 1, torch.cuda.current_stream().cuda_stream)
    assert st == -7
    assert b"static scratch" in L.yamoe_b200_status_string(st)
    torch.cuda.synchronize()
    assert int(out.abs().sum()) == 0                   # nothing was launched
