"""Benchmark of the expert forward path (and, by flag, its other workloads) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Prints ONE JSON line.  A "step" is one call of `yamoe_b200.experts` on one batch of seeded
synthetic input.  The default workload is the GPT-OSS-20B-shaped expert layer forward: 4096
tokens, hidden 2880, 32 experts, top-4, bf16 (weights and biases N(0, 0.02), activations N(0, 1),
softmax/top-4 routing without renormalisation).

* `value`      tokens/s with all inputs resident in HBM, timed with CUDA events over K steps,
               barrier + synchronize on both sides, max over ranks.
* `e2e`        the same metric through the public op with HOST inputs: every step copies the step's
               inputs (hidden_states, router_indices, routing_weights) from pinned host memory to
               the device and reads the [T, H] result back, inside the timed region.  Expert
               weights are model state and stay resident.
* `roofline`   gate_up grouped GEMM (the dominant kernel): algorithmic 4*S*H^2 FLOP per launch
               divided by its mean device time, bracketed by CUDA events inside each timed step.
* `cpu_baseline`  the CPU port of the reference's PyTorch implementation, timed on this box's host
               cores on a bounded sample (rank 0, N=1 only).
* `--impl reference`  times that CPU implementation with all host threads on the same workload.

With N > 1 (torchrun) every rank runs the same workload on its own tokens with a full replica of
the experts: tokens are independent units, so there is no data-path collective (weak scaling).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

KEYS = ["hidden_states", "router_indices", "routing_weights", "gate_up_proj", "gate_up_proj_bias",
        "down_proj", "down_proj_bias"]

WORKLOADS = {
    # name: (T, H, E, K, mode)
    "gptoss20b_fwd_t4096": dict(T=4096, H=2880, E=32, K=4, mode="fwd"),
    "gptoss20b_bwd_t8192": dict(T=8192, H=2880, E=32, K=4, mode="bwd"),
    "gptoss120b_decode_t1": dict(T=1, H=2880, E=128, K=4, mode="fwd"),
    "gptoss120b_decode_t4": dict(T=4, H=2880, E=128, K=4, mode="fwd"),
    "gptoss120b_decode_t16": dict(T=16, H=2880, E=128, K=4, mode="fwd"),
    "gptoss120b_decode_t64": dict(T=64, H=2880, E=128, K=4, mode="fwd"),
    # expert-parallel when launched on N > 1 GPUs: tokens sharded by rows, experts contiguously
    "gptoss120b_prefill_t16384": dict(T=16384, H=2880, E=128, K=4, mode="fwd", skew=True, ep=True),
    "gptoss20b_fwd_t8192_ep": dict(T=8192, H=2880, E=32, K=4, mode="fwd", ep=True),
    "gptoss20b_bwd_t8192_ep": dict(T=8192, H=2880, E=32, K=4, mode="bwd", ep=True),
    # forward + backward through autograd: recomputing the forward (as the reference does) / keeping activations
    "gptoss20b_train_t8192": dict(T=8192, H=2880, E=32, K=4, mode="train"),
    "gptoss20b_train_saved_t8192": dict(T=8192, H=2880, E=32, K=4, mode="train", saved=True),
    "readme_fp32_t512": dict(T=512, H=2880, E=8, K=2, mode="fwd", fp32=True),
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(bf16_tflops=d["bf16_tflops"], hbm_gbs=d["hbm_gbs"], source="measured")
    return dict(bf16_tflops=1590.0, hbm_gbs=6650.0, source="fallback")


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc = index, None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["no samples"])
        return dict(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))


def make_workload(name, weights_on=None):
    import torch
    from yamoe_b200 import workloads
    w = WORKLOADS[name]
    dtype = torch.float32 if w.get("fp32") else torch.bfloat16
    if name == "readme_fp32_t512":
        inp = workloads.make_readme_inputs(batch=2)
    else:
        big = w["E"] * w["H"] * w["H"] * 3 > 2 ** 31          # 120B-shaped: draw the weights on the device
        inp = workloads.make_inputs(w["T"], w["H"], w["E"], w["K"], seed=42, dtype=dtype,
                                    skew=w.get("skew", False), with_grad=(w["mode"] in ("bwd", "train")),
                                    weights_on=weights_on if big else None)
    return w, inp, dtype


def cpu_reference_time(w, inp, dtype, limit_s=20.0, threads=None):
    """Times the CPU port of the reference forward (sparse per-expert loop) in the workload's
    dtype.  Returns (tokens_per_s, cores, sample description)."""
    import torch
    from oracle import experts_oracle as orc
    if threads:
        torch.set_num_threads(threads)
    cores = torch.get_num_threads()
    T, E, K = w["T"], w["E"], w["K"]
    args = [inp[k] for k in KEYS]
    cap = 256 if w.get("fp32") else T

    def run():
        t0 = time.perf_counter()
        with torch.no_grad():
            if w["mode"] in ("bwd", "train"):
                orc.experts_backward_oracle(inp["grad_out"], *args, cap, E, K, compute_dtype=dtype)
            if w["mode"] in ("fwd", "train"):
                orc.experts_forward_oracle(*args, cap, E, K, compute_dtype=dtype)
        return time.perf_counter() - t0

    first = run()                               # warm-up, also sizes the sample
    reps = max(1, min(3, int(limit_s / max(first, 1e-3)) - 1))
    best = min([run() for _ in range(reps)] + ([first] if reps == 1 and first > limit_s / 2 else []))
    return T / best, cores, f"full workload ({T} tokens), best of {reps} after 1 warm-up, {dtype}, {cores} threads"


def run_reference(args):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w, inp, dtype = make_workload(args.workload, weights_on="cuda" if torch.cuda.is_available() else "cpu")
    inp = {k: v.cpu() for k, v in inp.items()}
    torch.set_num_threads(os.cpu_count() or 1)
    T = w["T"]
    args_list = [inp[k] for k in KEYS]
    from oracle import experts_oracle as orc
    cap = 256 if w.get("fp32") else T

    def step():
        with torch.no_grad():
            if w["mode"] in ("bwd", "train"):
                orc.experts_backward_oracle(inp["grad_out"], *args_list, cap, w["E"], w["K"], compute_dtype=dtype)
            if w["mode"] in ("fwd", "train"):
                orc.experts_forward_oracle(*args_list, cap, w["E"], w["K"], compute_dtype=dtype)

    steps, warm = max(1, min(args.steps, 5)), max(1, min(args.warmup, 1))
    for _ in range(warm):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    cores = torch.get_num_threads()
    val = T / dt
    line = {
        "impl": "reference", "metric": "moe_layer_tokens_per_s", "value": val, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warm, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if dtype == torch.bfloat16 else "f32",
        "data": "synthetic (seeded, shapes of the reference's own benchmarks)",
        "config": {"workload": args.workload, "tokens": T, "hidden": w["H"], "experts": w["E"], "top_k": w["K"],
                   "pass": w["mode"]},
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": f"full workload ({T} tokens) per step, {steps} steps, CPU port of the "
                                   f"reference's PyTorch experts (sparse branch), {cores} threads"},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def place_near_gpu(local_rank):
    """Pins this process to the CPUs of the GPU's NUMA node (when the allowed CPU set holds any), so
    that the pinned host buffers allocated afterwards are local to the GPU's PCIe root.  Returns a
    small record for the JSON line.  Host-to-device copies from the far socket run at about half
    the rate."""
    info = {"numa_node": None, "cpus_before": len(os.sched_getaffinity(0)), "cpus_after": None}
    info["_allowed"] = os.sched_getaffinity(0)
    try:
        import torch
        props = torch.cuda.get_device_properties(local_rank)
        if hasattr(props, "pci_bus_id"):
            bus = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        else:
            import pynvml
            pynvml.nvmlInit()
            bus = pynvml.nvmlDeviceGetPciInfo(pynvml.nvmlDeviceGetHandleByIndex(local_rank)).busId
            bus = (bus.decode() if isinstance(bus, bytes) else bus).lower()
            if len(bus.split(":")[0]) == 8:
                bus = bus[4:]
        base = f"/sys/bus/pci/devices/{bus}/"
        info["numa_node"] = int(open(base + "numa_node").read())
        local = set()
        for part in open(base + "local_cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            local.update(range(int(lo), int(hi or lo) + 1))
        want = local & os.sched_getaffinity(0)
        if want:
            os.sched_setaffinity(0, want)
    except Exception as exc:   # no NVML, no sysfs, odd bus id: leave the placement alone
        info["note"] = type(exc).__name__
    info["cpus_after"] = len(os.sched_getaffinity(0))
    return info


def copy_bandwidth(torch, nbytes=64 << 20):
    """Pinned host <-> device copy rates (GB/s), each direction alone: context for `e2e`."""
    h = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    d = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    out = {}
    for name, fn in (("h2d_gbs", lambda: d.copy_(h, non_blocking=True)), ("d2h_gbs", lambda: h.copy_(d, non_blocking=True))):
        fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(5):
            fn()
        b.record()
        torch.cuda.synchronize()
        out[name] = round(5 * nbytes / (a.elapsed_time(b) * 1e-3) / 1e9, 1)
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist
    import yamoe_b200
    from yamoe_b200 import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; yamoe_b200 has no CPU fallback")
    torch.cuda.set_device(local_rank)
    host_place = place_near_gpu(local_rank)
    allowed_cpus = host_place.pop("_allowed")
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    w, inp, dtype = make_workload(args.workload, weights_on="cuda")
    T, H, E, K = w["T"], w["H"], w["E"], w["K"]
    cap = 256 if w.get("fp32") else T
    dev = [inp[k].cuda() for k in KEYS]
    decode = T * K <= 256
    distinct = int(torch.unique(inp["router_indices"]).numel())
    weight_bytes = float(sum(dev[i].numel() * dev[i].element_size() for i in (3, 4, 5, 6)))
    flush_buf = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda") if decode else None
    flush_read = torch.zeros(64 * 1024 * 1024, dtype=torch.float32, device="cuda") if decode else None
    grad_out = inp["grad_out"].cuda() if w["mode"] in ("bwd", "train") else None
    if w["mode"] == "train":
        for i in (0, 2, 3, 4, 5, 6):
            dev[i].requires_grad_(True)
    L = _lib.lib()
    use_ep = bool(w.get("ep")) and world > 1
    if use_ep:
        from yamoe_b200 import ep
        T_total = T
        lo, hi = rank * (T // world), (rank + 1) * (T // world)
        local_w = ep.shard_expert_weights(*dev[3:], rank, world)
        inp = {k: (v[lo:hi] if k in KEYS[:3] + ["grad_out"] else v) for k, v in inp.items()}
        if grad_out is not None:
            grad_out = grad_out[lo:hi].contiguous()
        dev = [dev[i][lo:hi].contiguous() for i in range(3)] + list(local_w)
        torch.cuda.empty_cache()
        T = hi - lo
        ep_stats = {}
        peer_ctx = None
        if args.ep_mode in ("peer", "peer-fused") and w["mode"] in ("fwd", "bwd"):
            peer_ctx = ep.PeerExpertParallel(H, E, K, max_tokens_total=T_total, max_tokens_local=T, dtype=dtype,
                                             fused_return=(args.ep_mode == "peer-fused"),
                                             backward=(w["mode"] == "bwd"))

    def step():
        if use_ep and w["mode"] == "bwd":
            if peer_ctx is not None:
                return peer_ctx.backward(grad_out, *dev, cap)
            return ep.ep_experts_backward(grad_out, *dev, cap, E, K)
        if use_ep and peer_ctx is not None:
            return peer_ctx.forward(*dev, cap)
        if use_ep:
            return ep.ep_experts(*dev, cap, E, K, stats=ep_stats)
        if w["mode"] == "bwd":
            return yamoe_b200.experts_backward(grad_out, *dev, cap, E, K)
        if w["mode"] == "train":
            for i in (0, 2, 3, 4, 5, 6):
                dev[i].grad = None
            out = yamoe_b200.experts_autograd(*dev, cap, E, K, True, save_activations=bool(w.get("saved")))
            out.backward(grad_out)
            return dev[0].grad
        return yamoe_b200.experts(*dev, cap, E, K)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    sync_all()

    # ---- device-resident timing, with the gate_up GEMM bracketed by its own events ------------
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    for a, b in pairs:
        a.record(); b.record()           # forces creation of the underlying cudaEvent_t
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    sampler.start()
    t_start, t_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    if decode:
        # Touched weights (0.2 - 5.8 GB) are comparable to the 126 MB L2 at T=1: flush it between
        # steps and time every step by itself.  A call is ~50 us of GPU work but more than that of
        # Python dispatch, so the whole-call time is taken from a CUDA-graph replay of the same call
        # (the op issues only kernel launches); the gate_up kernel time comes from a second,
        # ungraphed pass with the stage events.
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            graph_out = step()
        sync_all()
        step_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in pairs]
        for s0, s1 in step_ev:
            flush_buf.fill_(1)             # 256 MB written: evicts the workload from the 126 MB L2 ...
            flush_read.sum()               # ... then 256 MB read: pushes the dirty lines out, so the timed
                                           # step does not pay for their write-back
            s0.record()
            graph.replay()
            s1.record()
        sync_all()
        ms_total = sum(s0.elapsed_time(s1) for s0, s1 in step_ev)
        for a, b in pairs:
            flush_buf.fill_(1)
            flush_read.sum()
            L.yamoe_b200_set_stage_events(a.cuda_event, b.cuda_event, 1)
            step()
        sync_all()
    else:
        t_start.record()
        for a, b in pairs:
            L.yamoe_b200_set_stage_events(a.cuda_event, b.cuda_event, 1)
            step()
        t_stop.record()
        sync_all()
        ms_total = t_start.elapsed_time(t_stop)
    L.yamoe_b200_set_stage_events(None, None, 0)
    gemm_ms = [a.elapsed_time(b) for a, b in pairs] if w["mode"] == "fwd" else []
    t = torch.tensor([ms_total], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = t.item() / args.steps
    value = world * T / (ms_step * 1e-3)

    # ---- end to end: host inputs in, host result out, every step -------------------------------
    host_in = [inp[k].pin_memory() for k in KEYS[:3]]
    host_out = torch.empty(T, H, dtype=dtype).pin_memory()
    host_go = inp["grad_out"].pin_memory() if w["mode"] in ("bwd", "train") else None
    h2d = sum(x.numel() * x.element_size() for x in host_in) + (host_go.numel() * host_go.element_size() if host_go is not None else 0)
    d2h = host_out.numel() * host_out.element_size()

    # Three streams pipeline consecutive steps: while step i computes, step i+1's inputs come in and
    # step i-1's result goes out (PCIe is full duplex).  Every step still copies its own inputs from
    # pinned host memory and its own result back; expert-parallel steps stay on one stream because
    # their collectives must be issued in the same order on every rank.
    pipelined = not use_ep
    cur = torch.cuda.current_stream()
    s_in, s_out = (torch.cuda.Stream(), torch.cuda.Stream()) if pipelined else (cur, cur)
    host_outs = [host_out, torch.empty_like(host_out).pin_memory()]
    in_ready = [torch.cuda.Event() for _ in range(2)]
    comp_done = [torch.cuda.Event() for _ in range(2)]
    out_done = [torch.cuda.Event() for _ in range(2)]
    keep = [None, None]
    dev_in = [[torch.empty_like(x, device="cuda") for x in host_in] for _ in range(2)]
    dev_go = [torch.empty_like(host_go, device="cuda") if host_go is not None else None for _ in range(2)]

    def run_op(a, g):
        if w["mode"] == "train":
            x = a[0].detach().requires_grad_(True)
            out = yamoe_b200.experts_autograd(x, a[1], a[2], *dev[3:], cap, E, K, False,
                                              save_activations=bool(w.get("saved")))
            out.backward(g)
            return x.grad
        if w["mode"] == "bwd":
            if use_ep:
                outs = (peer_ctx.backward(g, *a, *dev[3:], cap) if peer_ctx is not None
                        else ep.ep_experts_backward(g, *a, *dev[3:], cap, E, K))
            else:
                outs = yamoe_b200.experts_backward(g, *a, *dev[3:], cap, E, K)
            return outs[0]
        if use_ep:
            return peer_ctx.forward(*a, *dev[3:], cap) if peer_ctx is not None else ep.ep_experts(*a, *dev[3:], cap, E, K)
        return yamoe_b200.experts(*a, *dev[3:], cap, E, K)

    def e2e_step(i):
        b = i % 2
        with torch.cuda.stream(s_in):
            s_in.wait_event(comp_done[b])                 # device input buffers of step i-2 are free
            a, g = dev_in[b], dev_go[b]
            for d_, h_ in zip(a, host_in):
                d_.copy_(h_, non_blocking=True)
            if g is not None:
                g.copy_(host_go, non_blocking=True)
            in_ready[b].record(s_in)
        cur.wait_event(in_ready[b])
        out = run_op(a, g)
        comp_done[b].record(cur)
        with torch.cuda.stream(s_out):
            s_out.wait_event(comp_done[b])
            s_out.wait_event(out_done[b])                  # host buffer of step i-2 has been written
            host_outs[b].copy_(out, non_blocking=True)
            out_done[b].record(s_out)
        out.record_stream(s_out)
        keep[b] = out

    # Forward workloads on one GPU replay each step as a CUDA graph (host->device copies, the op
    # called through the public API, device->host copy): the host then issues one launch per step and
    # cannot fall behind the GPU.  Three graphs with their own buffers take turns on three streams,
    # so consecutive steps overlap as in the eager pipeline.  Anything else keeps the eager pipeline.
    graphs = None
    if pipelined and w["mode"] == "fwd" and not args.eager_e2e:
        try:
            graphs = []
            g_streams = [s_in, s_out, torch.cuda.Stream()]
            g_in = dev_in + [[torch.empty_like(x, device="cuda") for x in host_in]]
            g_out = host_outs + [torch.empty_like(host_out).pin_memory()]
            for b in range(3):
                gph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gph):
                    for d_, h_ in zip(g_in[b], host_in):
                        d_.copy_(h_, non_blocking=True)
                    g_out[b].copy_(run_op(g_in[b], None), non_blocking=True)
                graphs.append(gph)
        except Exception as exc:           # capture not possible here: time the eager pipeline
            sys.stderr.write(f"bench.py: CUDA-graph capture of the end-to-end step failed ({exc!r}); eager pipeline\n")
            graphs = None
            torch.cuda.synchronize()

    def graph_step(i):
        with torch.cuda.stream(g_streams[i % 3]):
            graphs[i % 3].replay()

    step_fn = graph_step if graphs is not None else e2e_step
    for i in range(min(args.warmup, 3) if graphs is None else 6):
        step_fn(i)
    sync_all()
    e_start, e_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_start.record()
    s_in.wait_event(e_start)
    s_out.wait_event(e_start)
    if graphs is not None:
        g_streams[2].wait_event(e_start)
    for i in range(args.steps):
        step_fn(i)
    cur.wait_stream(s_in)
    cur.wait_stream(s_out)
    if graphs is not None:
        cur.wait_stream(g_streams[2])
    e_stop.record()
    sync_all()
    clocks = sampler.stop()
    te = torch.tensor([e_start.elapsed_time(e_stop)], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_value = world * T / (te.item() / args.steps * 1e-3)

    if rank == 0:
        peaks = measured_peaks()
        if use_ep and peer_ctx is not None:
            per = E // world
            ep_stats["rows_received"] = int(peer_ctx.counts_all[:, rank * per:(rank + 1) * per].sum().item())
        S = ep_stats.get("rows_received", T * K) if use_ep else T * K      # rows this rank's GEMMs process
        line = {
            "metric": "moe_layer_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong" if use_ep else "weak", "vs_baseline": None,
            "dtype": "bf16" if dtype == torch.bfloat16 else "f32",
            "data": "synthetic (seeded, shapes of the reference's own benchmarks)",
            "config": {"workload": args.workload, "tokens": T, "hidden": H, "experts": E, "top_k": K,
                       "pass": w["mode"], "expert_capacity": cap,
                       "parallelism": (f"ep{world} (tokens sharded by rows, experts sharded contiguously, "
                                       + (f"dispatch + combine as NVLink peer stores [{args.ep_mode}], offsets on device, no host sync)"
                                          if use_ep and peer_ctx is not None else
                                          "NCCL all-to-all dispatch + combine; rank-0 rows sent/received "
                                          f"{ep_stats.get('rows_sent')}/{ep_stats.get('rows_received')})")) if use_ep else
                                      f"dp{world} (token shards, replicated experts, no collective)",
                       "l2": ("L2 flushed (256 MB write, then 256 MB read to drain the dirty lines) between steps; each step is a CUDA-graph replay of the op call timed by its own events" if decode
                              else f"expert weights ({weight_bytes / 1e9:.1f} GB) exceed the 126 MB L2; no flush")},
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "pipeline": ("every step is one CUDA-graph replay of (host->device copies, op, device->host copy); "
                                 "three such graphs take turns on three streams, so consecutive steps overlap"
                                 if graphs is not None else
                                 "host->device copy, op and device->host copy of consecutive steps overlap on three streams"
                                 if pipelined else "one stream, copies and op in sequence"),
                    "host": dict(host_place, **copy_bandwidth(torch))},
            "gpu_launches": args.steps * (2 if decode else {"fwd": 6, "bwd": 14, "train": 20}[w["mode"]]),
            "clocks": clocks,
            "achieved_tflops_whole_op": {"fwd": 6, "bwd": 16, "train": 22}[w["mode"]] * S * H * H / (ms_step * 1e-3) / 1e12,
        }
        if gemm_ms and decode:
            mean_ms = sum(gemm_ms) / len(gemm_ms)
            kbytes = distinct * (H * 2 * H * 2 + 2 * H * 2)          # gate_up weights + bias of the touched experts
            achieved = kbytes / (mean_ms * 1e-3) / 1e9
            line["roofline"] = {"bound": "hbm", "kernel": "gemv_kernel<gate_up + bias + clamped SwiGLU>",
                                "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                "frac": achieved / peaks["hbm_gbs"], "traffic": None, "kernel_ms": mean_ms,
                                "peak_source": peaks["source"] + " (copy bandwidth)",
                                "frac_of_nominal_8000": achieved / 8000.0, "distinct_experts": distinct,
                                "whole_op_gbs": distinct * 49783680 / (ms_step * 1e-3) / 1e9}
        elif gemm_ms and dtype == torch.float32:
            # fp32 runs on the CUDA cores (FFMA): no measured peak exists for that pipe, so the
            # fraction is against the nominal 148 SMs x 128 FMA x 2 x 1.965 GHz
            mean_ms = sum(gemm_ms) / len(gemm_ms)
            achieved = 4.0 * S * H * H / (mean_ms * 1e-3) / 1e12
            ffma_peak = 148 * 128 * 2 * 1.965e9 / 1e12
            line["roofline"] = {"bound": "tensor", "kernel": "simt_gemm_kernel<gate_up + bias + clamped SwiGLU> (fp32 FFMA)",
                                "achieved": achieved, "peak": ffma_peak, "unit": "TFLOP/s", "frac": achieved / ffma_peak,
                                "traffic": None, "kernel_ms": mean_ms,
                                "peak_source": "nominal fp32 FFMA rate (CUDA cores; the tensor pipe is not used in fp32)"}
        elif gemm_ms:
            mean_ms = sum(gemm_ms) / len(gemm_ms)
            achieved = 4.0 * S * H * H / (mean_ms * 1e-3) / 1e12
            line["roofline"] = {"bound": "tensor", "kernel": "umma_gemm_kernel<gate_up + bias + clamped SwiGLU>",
                                "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                                "frac": achieved / peaks["bf16_tflops"],
                                "traffic": args.traffic if args.workload == "gptoss20b_fwd_t4096" else None,
                                "kernel_ms": mean_ms, "peak_source": peaks["source"] + " (burst bf16 matmul)",
                                "frac_of_nominal_2250": achieved / 2250.0}
        if world == 1 and not args.no_cpu_baseline:
            os.sched_setaffinity(0, allowed_cpus)      # the CPU baseline may use every core again
            v, cores, sample = cpu_reference_time(w, {k: t.cpu() for k, t in inp.items()}, dtype)
            line["cpu_baseline"] = {"value": v, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gptoss20b_fwd_t4096", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--eager-e2e", action="store_true",
                    help="time the end-to-end leg with eager calls on three streams instead of CUDA-graph replays")
    ap.add_argument("--ep-mode", default="peer", choices=["peer", "peer-fused", "nccl"],
                    help="exchange used by the expert-parallel workloads on N > 1 GPUs")
    ap.add_argument("--traffic", type=float, default=1.268e9,
                    help="DRAM bytes per launch of the dominant kernel from an ncu capture (see profiles/)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
