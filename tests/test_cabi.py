"""The C-ABI library loads and exports every symbol include/yamoe_b200.h declares; argument
checks that need no GPU."""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from yamoe_b200 import build
    build.build()
    from yamoe_b200 import _lib
    return _lib.lib()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "yamoe_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(yamoe_b200_\w+)\s*\(", text)))


def test_header_symbols_exported(lib):
    from yamoe_b200 import _lib
    names = declared_symbols()
    assert len(names) >= 9
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == names


def test_version_and_status_strings(lib):
    assert lib.yamoe_b200_version() >= 100
    assert lib.yamoe_b200_status_string(0) == b"ok"
    assert b"workspace" in lib.yamoe_b200_status_string(-2)


def test_workspace_sizes(lib):
    assert lib.yamoe_b200_forward_workspace_bytes(4096, 2880, 32, 4, 1) > 2 * 16384 * 2880 * 2
    assert lib.yamoe_b200_backward_workspace_bytes(4096, 2880, 32, 4, 1) > \
        lib.yamoe_b200_forward_workspace_bytes(4096, 2880, 32, 4, 1)
    assert lib.yamoe_b200_forward_workspace_bytes(16, 2881, 8, 2, 1) == 0      # H % 8 != 0
    assert lib.yamoe_b200_forward_workspace_bytes(16, 64, 8, 2, 7) == 0        # bad dtype
    assert lib.yamoe_b200_route_workspace_bytes(0, 8, 2) > 0


def test_argument_checks_without_gpu(lib):
    # all rejected before any CUDA call is made
    assert lib.yamoe_b200_experts_forward(None, None, None, 8, None, None, None, None, None, 16, 64, 8, 2, 16, 0,
                                          None, 0, None) == -1
    assert lib.yamoe_b200_experts_forward(1, 1, 1, 5, 1, 1, 1, 1, 1, 16, 64, 8, 2, 16, 0, 256, 1 << 30, None) == -1
    assert lib.yamoe_b200_experts_forward(1, 1, 1, 8, 1, 1, 1, 1, 1, 16, 64, 8, 2, 16, 0, 256, 16, None) == -2
    assert lib.yamoe_b200_experts_forward(1, 1, 1, 8, 1, 1, 1, 1, 1, 16, 64, 8, 2, 16, 3, 256, 1 << 30, None) == -3
    assert lib.yamoe_b200_experts_forward(1, 1, 1, 8, 1, 1, 1, 1, 1, 16, 64, 8, 2, 16, 0, 100, 1 << 30, None) == -2
    assert lib.yamoe_b200_route(None, None, None, None, None, 4, 8, 2, None, 0, None) == -1


def test_ops_fail_loudly_without_cuda():
    import torch
    import yamoe_b200
    if torch.cuda.is_available():
        pytest.skip("CUDA present")
    x = torch.zeros(4, 8)
    with pytest.raises((RuntimeError, NotImplementedError)):
        yamoe_b200.experts(x, torch.zeros(4, 1, dtype=torch.int64), x[:, :2], torch.zeros(2, 8, 16),
                           torch.zeros(2, 16), torch.zeros(2, 8, 8), torch.zeros(2, 8), 4, 2, 1)
