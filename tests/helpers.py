"""Shared helpers for the tests: golden loading and tolerance rules."""
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
SMALL_CASES = ["small_a", "small_b", "small_c", "small_d"]
INPUT_KEYS = ["hidden_states", "router_indices", "routing_weights", "gate_up_proj",
              "gate_up_proj_bias", "down_proj", "down_proj_bias"]

# Tolerances: |x - ref| <= rtol*|ref| + rtol*max|ref|, plus a rel-L2 bound for bf16.
RTOL_F32 = 1e-4
RTOL_BF16 = 2e-2
REL_L2_BF16 = 1e-2


def load_golden(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    return {k: torch.from_numpy(z[k]) if z[k].ndim else z[k].item() for k in z.files}


def golden_inputs(g):
    return [g[k] for k in INPUT_KEYS]
