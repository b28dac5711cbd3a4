"""Time / peak-memory sweep of the expert forward over the shapes the reference's own benchmark
walks (perf_plot.py:29-39: six (seq_len, hidden, experts, top_k) configurations x batch sizes
1..64), with the reference's protocol (perf_plot.py:109-146): 5 warm-up calls, then the mean of 10
calls each followed by a device synchronisation, wall clock; peak allocated memory over those calls.

    python -m yamoe_b200.perf_sweep [--markdown out.md] [--dtype bf16|fp32] [--max-batch 64]

Differences from the reference script, stated because they change what is measured: tensors are
bfloat16 (the reference sweeps float16, which this library does not implement); the 8th argument
is passed as the reference passes it (`seq_len`, perf_plot.py:118), which for these routings drops
assignments of over-subscribed experts, and a second column gives the time with a capacity that
never drops (`T`).  A CUDA-event time of the same calls is reported beside the wall-clock mean.
"""
from __future__ import annotations

import argparse
import time

import torch

CONFIGS = [
    dict(seq_len=512, hidden_dim=2880, num_experts=32, top_k=4),
    dict(seq_len=1024, hidden_dim=2880, num_experts=32, top_k=4),
    dict(seq_len=512, hidden_dim=1024, num_experts=32, top_k=4),
    dict(seq_len=512, hidden_dim=2880, num_experts=16, top_k=2),
    dict(seq_len=2048, hidden_dim=1024, num_experts=16, top_k=2),
    dict(seq_len=768, hidden_dim=2048, num_experts=64, top_k=8),
]
BATCH_SIZES = [1, 2, 4, 8, 16, 32, 64]


def make_case(batch, seq_len, hidden_dim, num_experts, top_k, dtype, gen):
    """Inputs as perf_plot.py:60-105 builds them: N(0,1) logits -> softmax -> top-k without
    renormalisation, N(0,1) activations and weights, biases of ones."""
    T = batch * seq_len
    logits = torch.randn(T, num_experts, generator=gen)
    probs = torch.softmax(logits, dim=-1)
    w, idx = torch.topk(probs, top_k, dim=-1)
    dense = torch.zeros(T, num_experts).scatter_(1, idx, w)
    dev = "cuda"
    dgen = torch.Generator(device=dev).manual_seed(0)
    return dict(
        hidden=torch.randn(T, hidden_dim, generator=dgen, device=dev).to(dtype),
        idx=idx.to(dev), dense=dense.to(dev).to(dtype),
        wgu=torch.randn(num_experts, hidden_dim, 2 * hidden_dim, generator=dgen, device=dev).to(dtype),
        bgu=torch.ones(num_experts, 2 * hidden_dim, device=dev, dtype=dtype),
        wd=torch.randn(num_experts, hidden_dim, hidden_dim, generator=dgen, device=dev).to(dtype),
        bd=torch.ones(num_experts, hidden_dim, device=dev, dtype=dtype))


def time_case(c, capacity, num_experts, top_k):
    import yamoe_b200
    args = (c["hidden"], c["idx"], c["dense"], c["wgu"], c["bgu"], c["wd"], c["bd"], capacity, num_experts, top_k)
    for _ in range(5):
        yamoe_b200.experts(*args)
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    wall = []
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dev_ms = 0.0
    for _ in range(10):
        t0 = time.perf_counter()
        ev0.record()
        yamoe_b200.experts(*args)
        ev1.record()
        torch.cuda.synchronize()
        wall.append((time.perf_counter() - t0) * 1e3)
        dev_ms += ev0.elapsed_time(ev1)
    return sum(wall) / len(wall), dev_ms / 10, torch.cuda.max_memory_allocated() / 2 ** 20


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--markdown", default=None)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp32"])
    ap.add_argument("--max-batch", type=int, default=64)
    a = ap.parse_args()
    dtype = torch.bfloat16 if a.dtype == "bf16" else torch.float32
    gen = torch.Generator().manual_seed(0)
    lines = ["| seq_len | hidden | experts | top_k | batch | tokens | ms (wall, capacity=seq_len) | ms (CUDA events) | "
             "ms (CUDA events, capacity=T) | M tokens/s (capacity=T) | peak MB |", "|" + "---|" * 11]
    for cfg in CONFIGS:
        for b in [x for x in BATCH_SIZES if x <= a.max_batch]:
            T = b * cfg["seq_len"]
            try:
                c = make_case(b, dtype=dtype, gen=gen, **cfg)
                wall, dev_ms, mem = time_case(c, cfg["seq_len"], cfg["num_experts"], cfg["top_k"])
                _, dev_full, _ = time_case(c, T, cfg["num_experts"], cfg["top_k"])
                row = (f"| {cfg['seq_len']} | {cfg['hidden_dim']} | {cfg['num_experts']} | {cfg['top_k']} | {b} | {T} | "
                       f"{wall:.3f} | {dev_ms:.3f} | {dev_full:.3f} | {T / dev_full / 1e3:.2f} | {mem:.0f} |")
            except RuntimeError as exc:      # out of memory: report and go on, as the reference does
                if "out of memory" not in str(exc).lower():
                    raise
                row = f"| {cfg['seq_len']} | {cfg['hidden_dim']} | {cfg['num_experts']} | {cfg['top_k']} | {b} | {T} | OOM | | | | |"
            finally:
                c = None
                torch.cuda.empty_cache()
            print(row, flush=True)
            lines.append(row)
    if a.markdown:
        with open(a.markdown, "w") as f:
            f.write("\n".join(lines) + "\n")


if __name__ == "__main__":
    main()
