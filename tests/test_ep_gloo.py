"""Expert-parallel exchange logic on CPU ranks (gloo, world size 2 and 4): the split arithmetic,
row ordering and capacity semantics of yamoe_b200.ep with stand-in compute, against the
single-process oracle on the concatenated tokens."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
KEYS = ["hidden_states", "router_indices", "routing_weights", "gate_up_proj", "gate_up_proj_bias",
        "down_proj", "down_proj_bias"]


def cpu_backend():
    """Torch-CPU stand-ins with the semantics of the CUDA kernels (tests only)."""
    from oracle import experts_oracle as orc
    from yamoe_b200 import ep

    def route(idx, E):
        sv, si, counts, bins = orc.route_oracle(idx, E)
        return sv, si, bins, counts

    def permute_rows(src, si, K):
        return src[(si.long() // K)]

    def experts(*a):
        return orc.experts_forward_oracle(*a).to(a[0].dtype)

    def combine_rows(rows, si, ridx, rw, E):
        T, K = ridx.shape
        inv = torch.full((T * K,), -1, dtype=torch.long)
        inv[si.long()] = torch.arange(si.numel())
        w = torch.gather(rw, 1, ridx) if rw.shape[1] == E else rw
        out = torch.zeros(T, rows.shape[1], dtype=torch.float64)
        for k in range(K):
            pos = inv[torch.arange(T) * K + k]
            ok = pos >= 0
            out[ok] += w[ok, k, None].double() * rows[pos[ok]].double()
        return out.to(rows.dtype)

    def experts_backward(*a):
        return [g.to(a[1].dtype) for g in orc.experts_backward_oracle(*a)]

    return ep.Backend(route=route, permute_rows=permute_rows, experts=experts, combine_rows=combine_rows,
                      experts_backward=experts_backward)


def _worker(rank, world, port, T, H, E, K, cap, skew, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from yamoe_b200 import ep, workloads
        inp = workloads.make_inputs(T, H, E, K, seed=5, weight_std=0.3, bias_std=0.3, skew=skew, with_grad=True)
        lo, hi = rank * (T // world), (rank + 1) * (T // world)
        local_w = ep.shard_expert_weights(*[inp[k] for k in KEYS[3:]], rank, world)
        stats = {}
        out = ep.ep_experts(inp["hidden_states"][lo:hi], inp["router_indices"][lo:hi], inp["routing_weights"][lo:hi],
                            *local_w, cap, E, K, backend=cpu_backend(), stats=stats)
        grads = ep.ep_experts_backward(inp["grad_out"][lo:hi], inp["hidden_states"][lo:hi],
                                       inp["router_indices"][lo:hi], inp["routing_weights"][lo:hi], *local_w, cap, E, K,
                                       backend=cpu_backend())
        stats["grads"] = grads
        q.put((rank, out, stats))
        dist.barrier()
    except Exception as exc:  # surface the failure instead of letting the parent time out
        q.put((rank, repr(exc), None))
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,T,H,E,K,cap,skew", [(2, 24, 16, 4, 2, 24, False), (2, 40, 16, 8, 3, 5, True),
                                                    (4, 32, 8, 8, 2, 32, True)])
def test_ep_matches_single_process(world, T, H, E, K, cap, skew):
    from oracle import experts_oracle as orc
    from yamoe_b200 import workloads
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() + world * 7 + T) % 2000
    procs = [ctx.Process(target=_worker, args=(r, world, port, T, H, E, K, cap, skew, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    failed = [r for r in results if r[2] is None]
    if failed:
        for p in procs:
            p.terminate()
        pytest.fail(f"rank {failed[0][0]} failed: {failed[0][1]}")
    results.sort(key=lambda x: x[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    inp = workloads.make_inputs(T, H, E, K, seed=5, weight_std=0.3, bias_std=0.3, skew=skew, with_grad=True)
    ref = orc.experts_forward_oracle(*[inp[k] for k in KEYS], cap, E, K)
    got = torch.cat([r[1] for r in results])
    orc.check_close(got, ref, 1e-5, "expert-parallel vs single process")
    # backward: token-sharded gradients concatenate over ranks, expert-sharded ones over experts
    ref_g = orc.experts_backward_oracle(inp["grad_out"], *[inp[k] for k in KEYS], cap, E, K)
    for i, name in enumerate(["d_hidden", "d_routing", "d_wgu", "d_bgu", "d_wd", "d_bd"]):
        got_g = torch.cat([r[2]["grads"][i] for r in results])
        orc.check_close(got_g, ref_g[i], 2e-5, f"expert-parallel {name}")
    # conservation: every row sent is received by exactly one rank
    assert sum(r[2]["rows_sent"] for r in results) == sum(r[2]["rows_received"] for r in results) == T * K
    if cap < T:
        full = orc.experts_forward_oracle(*[inp[k] for k in KEYS], T, E, K)
        assert (full - ref).abs().max() > 1e-4        # the capacity really drops rows in this case


def test_expert_range_and_sharding():
    from yamoe_b200 import ep
    assert ep.expert_range(3, 8, 128) == (48, 64)
    with pytest.raises(ValueError):
        ep.expert_range(0, 3, 128)
    w = torch.arange(8 * 2 * 4).view(8, 2, 4).float()
    shard = ep.shard_expert_weights(w, w[:, 0], w[:, :, :2], w[:, 0, :2], 1, 4)
    assert shard[0].shape == (2, 2, 4) and torch.equal(shard[0], w[2:4])


def _leaver_worker(rank, world, port, q):
    """Rank `world - 1` leaves between two calls (no collective in flight); the others must get an
    error from their next exchange instead of waiting for ever."""
    import datetime
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    from yamoe_b200 import ep, workloads
    T, H, E, K = 24, 16, 6, 2
    inp = workloads.make_inputs(T, H, E, K, seed=5, weight_std=0.3, bias_std=0.3)
    lo, hi = rank * (T // world), (rank + 1) * (T // world)
    local_w = ep.shard_expert_weights(*[inp[k] for k in KEYS[3:]], rank, world)
    args = (inp["hidden_states"][lo:hi], inp["router_indices"][lo:hi], inp["routing_weights"][lo:hi], *local_w, T, E, K)
    first = ep.ep_experts(*args, backend=cpu_backend())
    dist.barrier()                      # the step is complete on every rank
    if rank == world - 1:
        q.put((rank, "left", first))
        dist.destroy_process_group()
        return
    try:
        ep.ep_experts(*args, backend=cpu_backend())
        q.put((rank, "completed", None))
    except Exception as exc:            # the expected outcome: a clean error on the surviving ranks
        q.put((rank, "error", type(exc).__name__))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_rank_leaving_between_steps_gives_a_clean_error():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    world = 3
    port = 29500 + (os.getpid() + 977) % 2000
    procs = [ctx.Process(target=_leaver_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted((q.get(timeout=120) for _ in range(world)), key=lambda x: x[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode is not None, "a surviving rank is still waiting"
    assert results[world - 1][1] == "left"
    for r in results[:world - 1]:
        assert r[1] == "error", f"rank {r[0]} {r[1]} although a peer had left"
