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


def test_cpp_binding_is_built_and_registered(lib):
    """The C++ torch binding (csrc/torch_binding.cpp) is what registers `experts` and
    `experts_backward` when it has been built; its schemas are the reference's."""
    import torch
    from yamoe_b200 import build, ops
    assert os.path.exists(build.BINDING_PATH)
    assert ops.CPP_BINDING
    schema = str(torch.ops.yamoe_b200.experts.default._schema)
    assert "Tensor hidden_states, Tensor router_indices, Tensor routing_weights, Tensor gate_up_proj" in schema
    assert "int expert_capacity, int num_experts, int top_k) -> Tensor" in schema
    assert str(torch.ops.yamoe_b200.experts_backward.default._schema).endswith("-> Tensor[]")


@pytest.mark.gpu
def test_python_and_cpp_bindings_agree():
    """The same call through the Python registration of the operators (a child process with
    YAMOE_B200_PY_BINDING=1) and through the C++ binding: bit-identical outputs, same error text."""
    import subprocess
    import sys
    code = r'''
import sys, torch
sys.path.insert(0, %r)
import yamoe_b200
from yamoe_b200 import ops
from oracle import experts_oracle as orc
inp = orc.make_inputs(300, 128, 8, 2, seed=3, weight_std=0.1, bias_std=0.1, dtype=torch.bfloat16, with_grad=True)
keys = ["hidden_states", "router_indices", "routing_weights", "gate_up_proj", "gate_up_proj_bias", "down_proj", "down_proj_bias"]
dev = [inp[k].cuda() for k in keys]
out = yamoe_b200.experts(*dev, 300, 8, 2)
g = yamoe_b200.experts_backward(inp["grad_out"].cuda(), *dev, 300, 8, 2)
try:
    yamoe_b200.experts(dev[0], dev[1], dev[2], dev[3][:, :, :-2], *dev[4:], 300, 8, 2)
    msg = "no error"
except RuntimeError as exc:
    msg = str(exc).splitlines()[0]
torch.save({"cpp": ops.CPP_BINDING, "out": out.cpu(), "g": [t.cpu() for t in g], "msg": msg}, sys.argv[1])
''' % ROOT
    import tempfile
    import torch
    res = {}
    with tempfile.TemporaryDirectory() as tmp:
        for name, env in (("py", {"YAMOE_B200_PY_BINDING": "1"}), ("cpp", {"YAMOE_B200_PY_BINDING": "0"})):
            path = os.path.join(tmp, name + ".pt")
            subprocess.run([sys.executable, "-c", code, path], check=True, env=dict(os.environ, **env), timeout=300)
            res[name] = torch.load(path)
    assert res["cpp"]["cpp"] and not res["py"]["cpp"]
    assert torch.equal(res["py"]["out"], res["cpp"]["out"])
    # gradients accumulate with fp32 atomics whose order is not fixed: equal up to rounding
    for a, b in zip(res["py"]["g"], res["cpp"]["g"]):
        assert (a.float() - b.float()).abs().max() <= 2e-2 * b.float().abs().max() + 1e-6
    assert "gate_up_proj must be [E, H, 2*H]" in res["py"]["msg"] and "gate_up_proj must be [E, H, 2*H]" in res["cpp"]["msg"]
