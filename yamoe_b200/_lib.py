"""ctypes view of the C ABI declared in include/yamoe_b200.h.

The shared library must exist in-tree (built by `python -m yamoe_b200.build` or
`__graft_entry__.build()`); there is no fallback of any kind: a missing library raises.
"""
from __future__ import annotations

import ctypes
import os

from .build import LIB_PATH as _DEFAULT_LIB

# YAMOE_B200_LIB points at an alternative build of the same library (profiling experiments)
LIB_PATH = os.environ.get("YAMOE_B200_LIB") or _DEFAULT_LIB

c_void_p, c_int, c_int64, c_size_t = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_size_t

YAMOE_F32, YAMOE_BF16 = 0, 1


class EpCtx(ctypes.Structure):
    """yamoe_ep_ctx_t of include/yamoe_b200.h."""
    _fields_ = ([(n, ctypes.c_int32) for n in ("G", "rank", "E", "K", "H", "dtype")] +
                [("max_rows", ctypes.c_int64), ("back_rows", ctypes.c_int64)] +
                [(n, ctypes.c_void_p) for n in ("peer_recv_x", "peer_recv_g", "peer_recv_w", "peer_back",
                                                "peer_back_w", "peer_ctrl", "recv_x", "recv_g", "recv_w", "back",
                                                "back_w", "ctrl", "state")] +
                [("wait_ns", ctypes.c_uint64)])


_ctx_p = ctypes.POINTER(EpCtx)
PATH_AUTO, PATH_SIMT, PATH_TCGEN05, PATH_GEMV = 0, 1, 2, 3

# name -> (restype, argtypes); mirrors include/yamoe_b200.h one to one
SIGNATURES = {
    "yamoe_b200_version": (c_int, []),
    "yamoe_b200_status_string": (ctypes.c_char_p, [c_int]),
    "yamoe_b200_set_path": (c_int, [c_int]),
    "yamoe_b200_set_stage_events": (c_int, [c_void_p, c_void_p, c_int]),
    "yamoe_b200_route_workspace_bytes": (c_size_t, [c_int64, c_int, c_int]),
    "yamoe_b200_route": (c_int, [c_void_p] * 5 + [c_int64, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "yamoe_b200_route_static_scratch_needed": (c_size_t, [c_int64, c_int, c_int]),
    "yamoe_b200_route_static": (c_int, [c_void_p] * 5 + [c_int64, c_int, c_int, c_void_p]),
    "yamoe_b200_forward_workspace_bytes": (c_size_t, [c_int64, c_int, c_int, c_int, c_int]),
    "yamoe_b200_experts_forward": (c_int, [c_void_p, c_void_p, c_void_p, c_int] + [c_void_p] * 5 +
                                   [c_int64, c_int, c_int, c_int, c_int64, c_int, c_void_p, c_size_t, c_void_p]),
    "yamoe_b200_backward_workspace_bytes": (c_size_t, [c_int64, c_int, c_int, c_int, c_int]),
    "yamoe_b200_experts_backward": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int] +
                                    [c_void_p] * 10 +
                                    [c_int64, c_int, c_int, c_int, c_int64, c_int, c_void_p, c_size_t, c_void_p]),
    "yamoe_b200_batch_mm_workspace_bytes": (c_size_t, [c_int, c_int]),
    "yamoe_b200_batch_mm": (c_int, [c_void_p, c_void_p, c_void_p] + [c_int] * 7 + [c_void_p, c_size_t, c_void_p]),
    "yamoe_b200_permute_rows": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p]),
    "yamoe_b200_combine_rows": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_int64,
                                        c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "yamoe_b200_ep_ctrl_bytes": (c_size_t, [c_int, c_int]),
    "yamoe_b200_ep_call_workspace_bytes": (c_size_t, [_ctx_p, c_int64, c_int]),
    "yamoe_b200_ep_forward": (c_int, [_ctx_p, c_void_p, c_void_p, c_void_p, c_int] + [c_void_p] * 5 +
                              [c_int64, c_int64, c_void_p, c_size_t, c_void_p]),
    "yamoe_b200_ep_backward": (c_int, [_ctx_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int] + [c_void_p] * 10 +
                               [c_int64, c_int64, c_void_p, c_size_t, c_void_p]),
    "yamoe_b200_ep_wait_probe": (c_int, [c_void_p, c_int, ctypes.c_int32, ctypes.c_uint64, c_void_p, c_void_p,
                                         c_void_p]),
    "yamoe_b200_binned_gather": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int64, c_int,
                                         c_int, c_void_p]),
    "yamoe_b200_binned_scatter": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int,
                                          c_int64, c_int, c_int, c_void_p]),
    "yamoe_b200_index_select": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p]),
    "yamoe_b200_router_topk": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p]),
    "yamoe_b200_router_workspace_bytes": (c_size_t, [c_int64, c_int]),
    "yamoe_b200_router_forward": (c_int, [c_void_p] * 5 + [c_int64, c_int, c_int, c_int, c_int, c_void_p, c_size_t,
                                                           c_void_p]),
    "yamoe_b200_experts_forward_saving": (c_int, [c_void_p, c_void_p, c_void_p, c_int] + [c_void_p] * 5 +
                                          [c_int64, c_int, c_int, c_int, c_int64, c_int, c_void_p, c_size_t, c_void_p]),
    "yamoe_b200_experts_backward_saved": (c_int, [c_void_p, c_int, c_void_p, c_int] + [c_void_p] * 9 +
                                          [c_int64, c_int, c_int, c_int, c_int64, c_int, c_void_p, c_size_t, c_void_p]),
    "yamoe_b200_mbar_wait_probe": (c_int, [c_void_p, ctypes.c_uint64, c_void_p]),
    "yamoe_b200_device_status": (c_int, [c_void_p, c_void_p, ctypes.POINTER(ctypes.c_int32)]),
}

_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m yamoe_b200.build`. "
                "yamoe_b200 has no CPU or PyTorch fallback.")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check_device_status(workspace_ptr: int, stream: int, what: str) -> None:
    """Reads the device status word at the head of a workspace (synchronises the stream) and raises
    when a bounded device-side wait gave up during the call that used it."""
    out = ctypes.c_int32(0)
    check(lib().yamoe_b200_device_status(workspace_ptr, stream, ctypes.byref(out)), what + " (status read)")
    if out.value != 0:
        msg = lib().yamoe_b200_status_string(-6).decode()
        raise RuntimeError(f"yamoe_b200: {what} failed: {msg} (device status {out.value})")


def check(status: int, what: str) -> None:
    if status != 0:
        msg = lib().yamoe_b200_status_string(status).decode()
        raise RuntimeError(f"yamoe_b200: {what} failed: {msg} (status {status})")
