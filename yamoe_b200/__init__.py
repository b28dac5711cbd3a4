"""yamoe_b200: the expert forward/backward op of drbh/yamoe as hand-written sm_100a CUDA behind
the reference's operator interface (torch-ext/yamoe/__init__.py:6-12)."""
from . import _lib
from .layers import Yamoe, _ExpertsFn, experts_autograd
from .ops import (batch_mm, batch_mm_wgrad, bincount_cumsum, experts, experts_backward, gather, index_select_out,
                  route, router_forward, router_topk, scatter, sort)


def set_path(name: str) -> str:
    """Select the GEMM path: "auto", "simt", "tcgen05" or "gemv".  Returns the previous one."""
    names = ["auto", "simt", "tcgen05", "gemv"]
    prev = _lib.lib().yamoe_b200_set_path(names.index(name))
    return names[prev]


__all__ = ["experts", "experts_backward", "sort", "bincount_cumsum", "gather", "scatter", "index_select_out", "route",
           "batch_mm", "batch_mm_wgrad", "experts_autograd", "Yamoe", "router_topk", "router_forward", "_ExpertsFn", "set_path"]
