"""Metric table of the reference's compare_example.py (:195-327) for this library: the CUDA op
against the CPU oracle on the same seeded inputs.  Rows: sum / min / max / L2 norm / std of both
outputs, time and peak device memory of the op, then MSE, MAE, cosine similarity, relative L2 error
and maximum absolute difference.

    python tests/compare_table.py [--tokens 512 --hidden 2880 --experts 8 --top-k 2 --dtype float32]

Test infrastructure: it imports the oracle, so it lives with the tests.
"""
import argparse
import os
import sys
import time

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from oracle import experts_oracle as orc  # noqa: E402

KEYS = ["hidden_states", "router_indices", "routing_weights", "gate_up_proj", "gate_up_proj_bias", "down_proj",
        "down_proj_bias"]


def compare(T, H, E, K, dtype, seed=42, iters=5):
    import yamoe_b200
    inp = orc.make_inputs(T, H, E, K, seed=seed, dtype=dtype)
    dev = [inp[k].cuda() for k in KEYS]
    for _ in range(3):
        yamoe_b200.experts(*dev, T, E, K)
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    base = torch.cuda.memory_allocated()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        out = yamoe_b200.experts(*dev, T, E, K)
    b.record()
    torch.cuda.synchronize()
    kernel_ms = a.elapsed_time(b) / iters
    kernel_mb = (torch.cuda.max_memory_allocated() - base) / 2**20
    t0 = time.perf_counter()
    ref = orc.experts_forward_oracle(*[inp[k] for k in KEYS], T, E, K)
    ref_ms = (time.perf_counter() - t0) * 1e3
    got = out.float().cpu()
    ref = ref.float()
    diff = got - ref
    return {
        "kernel": got, "reference": ref, "kernel_ms": kernel_ms, "reference_ms": ref_ms, "kernel_mb": kernel_mb,
        "mse": diff.pow(2).mean().item(), "mae": diff.abs().mean().item(),
        "cosine": torch.nn.functional.cosine_similarity(got.view(1, -1), ref.view(1, -1)).item(),
        "rel_l2": (diff.norm() / ref.norm()).item(), "max_abs": diff.abs().max().item(),
    }


def print_table(r):
    k, ref = r["kernel"], r["reference"]
    line = "=" * 78
    print(line)
    print(f"{'METRIC':<20} {'KERNEL (B200)':<18} {'ORACLE (CPU)':<18} {'SPEEDUP':<12}")
    print(line)
    for name, fn in (("Sum", torch.sum), ("Min", torch.min), ("Max", torch.max), ("Norm (L2)", torch.norm),
                     ("Std", torch.std)):
        print(f"{name:<20} {fn(k).item():<18.4f} {fn(ref).item():<18.4f} {'N/A':<12}")
    print("-" * 78)
    print(f"{'Time (ms)':<20} {r['kernel_ms']:<18.3f} {r['reference_ms']:<18.3f} "
          f"{r['reference_ms'] / r['kernel_ms']:<.2f}x")
    print(f"{'Memory (MB)':<20} {r['kernel_mb']:<18.2f} {'-':<18}")
    print("-" * 78)
    print("SIMILARITY METRICS (KERNEL vs ORACLE)")
    for name, key, fmt in (("MSE", "mse", "e"), ("MAE", "mae", "e"), ("Cosine Similarity", "cosine", "f"),
                           ("Relative Error", "rel_l2", "e"), ("Max Abs Diff", "max_abs", "e")):
        print(f"{name:<20} {r[key]:<20.6{fmt}}")
    print("-" * 78)
    print(f"{'INDEX':<6} {'KERNEL':<14} {'ORACLE':<14} {'DIFF':<14}")
    for i in range(10):
        a, b = k.view(-1)[i].item(), ref.view(-1)[i].item()
        print(f"{i:<6} {a:<14.6f} {b:<14.6f} {a - b:<14.6f}")
    print(line)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=512)
    ap.add_argument("--hidden", type=int, default=2880)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--top-k", type=int, default=2)
    ap.add_argument("--dtype", default="float32", choices=["float32", "bfloat16"])
    args = ap.parse_args()
    print_table(compare(args.tokens, args.hidden, args.experts, args.top_k, getattr(torch, args.dtype)))
