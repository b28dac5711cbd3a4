"""Build recipe, output in-tree: libyamoe_b200.so (one nvcc invocation for sm_100a: all kernels and
the C ABI) and libyamoe_b200_torch.so (host compiler only: the C++ torch binding of `experts` and
`experts_backward` over that C ABI).

    python -m yamoe_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libyamoe_b200.so")
BINDING_PATH = os.path.join(PKG_DIR, "libyamoe_b200_torch.so")
BINDING_SRC = os.path.join(CSRC, "torch_binding.cpp")
SOURCES = ["yamoe_b200.cu"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-shared", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-ldl"]


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else (shutil.which("nvcc") or "nvcc")


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f != "torch_binding.cpp"]
    deps.append(os.path.join(os.path.dirname(PKG_DIR), "include", "yamoe_b200.h"))
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build_binding(force: bool = False, verbose: bool = False) -> str:
    """Compile the C++ torch binding against the installed torch (no CUDA code in it)."""
    header = os.path.join(os.path.dirname(PKG_DIR), "include", "yamoe_b200.h")
    if not force and os.path.exists(BINDING_PATH) and all(
            os.path.getmtime(BINDING_PATH) >= os.path.getmtime(d) for d in (BINDING_SRC, header, LIB_PATH)):
        return BINDING_PATH
    import torch
    from torch.utils import cpp_extension as ce
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    tlib = ce.library_paths()[0]
    cmd = [shutil.which("g++") or "g++", "-O2", "-std=c++17", "-shared", "-fPIC",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    cmd += [f"-I{p}" for p in ce.include_paths()] + [f"-I{os.path.join(cuda_home, 'include')}"]
    cmd += ["-o", BINDING_PATH, BINDING_SRC, f"-L{PKG_DIR}", "-l:libyamoe_b200.so", f"-L{tlib}", "-lc10", "-lc10_cuda",
            "-ltorch_cpu", "-ltorch_cuda", "-ltorch", f"-L{os.path.join(cuda_home, 'lib64')}", "-lcudart",
            "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{tlib}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("g++ failed building libyamoe_b200_torch.so:\n" + res.stderr[-4000:])
    return BINDING_PATH


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if it is missing or older than its sources; return its path."""
    path = _build_cuda(force, verbose)
    build_binding(force, verbose)
    return path


def _build_cuda(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return LIB_PATH
    cmd = [_nvcc(), *NVCC_FLAGS]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", LIB_PATH, *[os.path.join(CSRC, s) for s in SOURCES]]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libyamoe_b200.so:\n" + res.stderr[-4000:])
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
