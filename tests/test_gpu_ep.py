"""Expert parallelism on real GPUs (2 ranks, NCCL): the expert-parallel result must equal the
single-GPU op on the concatenated tokens.  Skipped when fewer than two GPUs are visible."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
KEYS = ["hidden_states", "router_indices", "routing_weights", "gate_up_proj", "gate_up_proj_bias",
        "down_proj", "down_proj_bias"]


def _worker(rank, world, port, T, H, E, K, cap, skew, q):
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import yamoe_b200
        from yamoe_b200 import ep, workloads
        inp = workloads.make_inputs(T, H, E, K, seed=9, weight_std=0.05, bias_std=0.1, dtype=torch.bfloat16, skew=skew,
                                    with_grad=True)
        lo, hi = rank * (T // world), (rank + 1) * (T // world)
        local_w = ep.shard_expert_weights(*[inp[k].cuda() for k in KEYS[3:]], rank, world)
        out = ep.ep_experts(inp["hidden_states"][lo:hi].cuda(), inp["router_indices"][lo:hi].cuda(),
                            inp["routing_weights"][lo:hi].cuda(), *local_w, cap, E, K)
        single = yamoe_b200.experts(*[inp[k].cuda() for k in KEYS], cap, E, K)[lo:hi]
        grads = ep.ep_experts_backward(inp["grad_out"][lo:hi].cuda(), inp["hidden_states"][lo:hi].cuda(),
                                       inp["router_indices"][lo:hi].cuda(), inp["routing_weights"][lo:hi].cuda(),
                                       *local_w, cap, E, K)
        torch.cuda.synchronize()
        q.put((rank, out.float().cpu(), (single.float().cpu(), [g.float().cpu() for g in grads])))
        dist.barrier()
    except Exception as exc:
        q.put((rank, repr(exc), None))
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("T,H,E,K,cap,skew", [(512, 256, 8, 2, 512, False), (1024, 128, 16, 4, 100, True)])
def test_ep_two_gpus_matches_single_gpu(T, H, E, K, cap, skew):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    from oracle import experts_oracle as orc
    from yamoe_b200 import workloads
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + (os.getpid() + T) % 1000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, T, H, E, K, cap, skew, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(2)]
    bad = [r for r in results if r[2] is None]
    if bad:
        for p in procs:
            p.terminate()
        pytest.fail(f"rank {bad[0][0]}: {bad[0][1]}")
    for p in procs:
        p.join(timeout=60)
    results.sort(key=lambda x: x[0])
    got = torch.cat([r[1] for r in results])
    single = torch.cat([r[2][0] for r in results])
    inp = workloads.make_inputs(T, H, E, K, seed=9, weight_std=0.05, bias_std=0.1, dtype=torch.bfloat16, skew=skew,
                                with_grad=True)
    ref = orc.experts_forward_oracle(*[inp[k] for k in KEYS], cap, E, K)
    orc.check_close(got, ref, 2e-2, "expert-parallel vs oracle", rel_l2=1e-2)
    orc.check_close(got, single, 2e-2, "expert-parallel vs single-GPU op", rel_l2=1e-2)
    ref_g = orc.experts_backward_oracle(inp["grad_out"], *[inp[k] for k in KEYS], cap, E, K)
    for i, name in enumerate(["d_hidden", "d_routing", "d_wgu", "d_bgu", "d_wd", "d_bd"]):
        got_g = torch.cat([r[2][1][i] for r in results])
        orc.check_close(got_g, ref_g[i], 2e-2, f"expert-parallel {name}", rel_l2=2e-2)


def test_permute_and_combine_rows_single_gpu():
    """The two expert-parallel helper kernels, without any exchange: permute, identity 'experts',
    combine must reproduce sum_k w[t,k] * x[t]."""
    import yamoe_b200
    from yamoe_b200 import ops, workloads
    T, H, E, K = 300, 128, 16, 4
    for dtype, tol in ((torch.float32, 1e-6), (torch.bfloat16, 1e-2)):
        inp = workloads.make_inputs(T, H, E, K, seed=2, dtype=dtype)
        x, ri, rw = inp["hidden_states"].cuda(), inp["router_indices"].cuda(), inp["routing_weights"].cuda()
        sv, si, bins, counts = yamoe_b200.route(ri, E)
        rows = ops.permute_rows(x, si, K)
        assert torch.equal(rows, x[(si.long() // K)])
        out = ops.combine_rows(rows, si, ri, rw, E)
        wsum = torch.gather(rw.float(), 1, ri).sum(1, keepdim=True)
        ref = wsum * x.float()
        assert (out.float() - ref).abs().max() <= tol * ref.abs().max() + 1e-6
        # assignments missing from the sorted list contribute nothing
        half = ops.combine_rows(rows[: si.numel() // 2], si[: si.numel() // 2], ri, rw, E)
        assert half.float().abs().sum() < out.float().abs().sum()


def _peer_worker(rank, world, port, q):
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from yamoe_b200 import ep, workloads
        outs = []
        H, E, K = 256, 16, 4
        ctx = ep.PeerExpertParallel(H, E, K, max_tokens_total=1024, max_tokens_local=512, dtype=torch.bfloat16)
        # three calls in a row on the same buffers: full capacity, a dropping capacity, fewer tokens
        for T, cap, skew, seed in ((1024, 1024, False, 9), (1024, 100, True, 10), (512, 512, True, 11)):
            inp = workloads.make_inputs(T, H, E, K, seed=seed, weight_std=0.05, bias_std=0.1, dtype=torch.bfloat16,
                                        skew=skew)
            lo, hi = rank * (T // world), (rank + 1) * (T // world)
            local_w = ep.shard_expert_weights(*[inp[k].cuda() for k in KEYS[3:]], rank, world)
            out = ctx.forward(inp["hidden_states"][lo:hi].cuda(), inp["router_indices"][lo:hi].cuda(),
                              inp["routing_weights"][lo:hi].cuda(), *local_w, cap)
            torch.cuda.synchronize()
            assert ctx.status() == 0, f"device status {ctx.status()}"
            outs.append(out.float().cpu())
        # receive buffers too small for a skewed routing: every rank must report the overflow status
        # (nothing is stored past a buffer), and the same object must serve a fitting call afterwards
        small = ep.PeerExpertParallel(H, E, K, max_tokens_total=512, max_tokens_local=512, dtype=torch.bfloat16)
        inp = workloads.make_inputs(1024, H, E, K, seed=10, weight_std=0.05, bias_std=0.1, dtype=torch.bfloat16,
                                    skew=True)
        lo, hi = rank * 512, (rank + 1) * 512
        local_w = ep.shard_expert_weights(*[inp[k].cuda() for k in KEYS[3:]], rank, world)
        small.forward(inp["hidden_states"][lo:hi].cuda(), inp["router_indices"][lo:hi].cuda(),
                      inp["routing_weights"][lo:hi].cuda(), *local_w, 1024)
        torch.cuda.synchronize()
        assert small.status() == 7, f"expected the overflow status, got {small.status()}"
        out = small.forward(inp["hidden_states"][lo:lo + 128].cuda(), inp["router_indices"][lo:lo + 128].cuda(),
                            inp["routing_weights"][lo:lo + 128].cuda(), *local_w, 1024)
        torch.cuda.synchronize()
        assert small.status() == 0, f"device status {small.status()} after a fitting call"
        outs.append(out.float().cpu())
        q.put((rank, outs, True))
        dist.barrier()
    except Exception as exc:
        q.put((rank, repr(exc), None))
        raise
    finally:
        dist.destroy_process_group()


def test_peer_store_ep_two_gpus():
    """Dispatch and combine as peer stores with on-device offsets and flags (no host round trip, no
    collective); the down GEMM's epilogue itself performs the combine stores."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    from oracle import experts_oracle as orc
    from yamoe_b200 import workloads
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29800 + os.getpid() % 1000
    procs = [ctx.Process(target=_peer_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(2)]
    bad = [r for r in results if r[2] is None]
    if bad:
        for p in procs:
            p.terminate()
        pytest.fail(f"rank {bad[0][0]}: {bad[0][1]}")
    for p in procs:
        p.join(timeout=60)
    results.sort(key=lambda x: x[0])
    H, E, K = 256, 16, 4
    for i, (T, cap, skew, seed) in enumerate(((1024, 1024, False, 9), (1024, 100, True, 10), (512, 512, True, 11))):
        inp = workloads.make_inputs(T, H, E, K, seed=seed, weight_std=0.05, bias_std=0.1, dtype=torch.bfloat16, skew=skew)
        ref = orc.experts_forward_oracle(*[inp[k] for k in KEYS], cap, E, K)
        got = torch.cat([r[1][i] for r in results])
        orc.check_close(got, ref, 2e-2, f"peer-store expert parallel, call {i}", rel_l2=1e-2)
    # the call after the overflow: 128 tokens per rank of the skewed 1024-token case
    inp = workloads.make_inputs(1024, H, E, K, seed=10, weight_std=0.05, bias_std=0.1, dtype=torch.bfloat16, skew=True)
    sel = torch.cat([torch.arange(0, 128), torch.arange(512, 640)])
    ref = orc.experts_forward_oracle(inp["hidden_states"][sel], inp["router_indices"][sel],
                                     inp["routing_weights"][sel], *[inp[k] for k in KEYS[3:]], 1024, E, K)
    got = torch.cat([r[1][3] for r in results])
    orc.check_close(got, ref, 2e-2, "peer-store expert parallel after an overflowing call", rel_l2=1e-2)


PEER_BWD_CASES = ((1024, 1024, False, 9, True), (1024, 100, True, 10, False), (512, 512, True, 11, True))


def _peer_bwd_worker(rank, world, port, q):
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from yamoe_b200 import ep, workloads
        H, E, K = 256, 16, 4
        ctx = ep.PeerExpertParallel(H, E, K, max_tokens_total=1024, max_tokens_local=512, dtype=torch.bfloat16,
                                    backward=True)
        outs = []
        # forward and backward alternate on the same buffers; dense and [T, K] routing weights
        for T, cap, skew, seed, dense in PEER_BWD_CASES:
            inp = workloads.make_inputs(T, H, E, K, seed=seed, weight_std=0.05, bias_std=0.1, dtype=torch.bfloat16,
                                        skew=skew, with_grad=True)
            lo, hi = rank * (T // world), (rank + 1) * (T // world)
            local_w = ep.shard_expert_weights(*[inp[k].cuda() for k in KEYS[3:]], rank, world)
            ri = inp["router_indices"][lo:hi].cuda()
            rw = inp["routing_weights"][lo:hi].cuda()
            if not dense:
                rw = torch.gather(rw, 1, ri).contiguous()
            out = ctx.forward(inp["hidden_states"][lo:hi].cuda(), ri, rw, *local_w, cap)
            grads = ctx.backward(inp["grad_out"][lo:hi].cuda(), inp["hidden_states"][lo:hi].cuda(), ri, rw,
                                 *local_w, cap)
            torch.cuda.synchronize()
            assert ctx.status() == 0, f"device status {ctx.status()}"
            outs.append((out.float().cpu(), [g.float().cpu() for g in grads]))
        q.put((rank, outs, True))
        dist.barrier()
    except Exception as exc:
        q.put((rank, repr(exc), None))
        raise
    finally:
        dist.destroy_process_group()


def test_peer_store_ep_backward_two_gpus():
    """Backward over peer stores: token rows, gradient rows and routing weights go to the expert
    owners, input-gradient rows return through the data-gradient GEMM's epilogue."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    from oracle import experts_oracle as orc
    from yamoe_b200 import workloads
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29900 + os.getpid() % 1000
    procs = [ctx.Process(target=_peer_bwd_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(2)]
    bad = [r for r in results if r[2] is None]
    if bad:
        for p in procs:
            p.terminate()
        pytest.fail(f"rank {bad[0][0]}: {bad[0][1]}")
    for p in procs:
        p.join(timeout=60)
    results.sort(key=lambda x: x[0])
    H, E, K = 256, 16, 4
    for i, (T, cap, skew, seed, dense) in enumerate(PEER_BWD_CASES):
        inp = workloads.make_inputs(T, H, E, K, seed=seed, weight_std=0.05, bias_std=0.1, dtype=torch.bfloat16,
                                    skew=skew, with_grad=True)
        ref = orc.experts_forward_oracle(*[inp[k] for k in KEYS], cap, E, K)
        got = torch.cat([r[1][i][0] for r in results])
        orc.check_close(got, ref, 2e-2, f"peer-store forward, call {i}", rel_l2=1e-2)
        ref_g = list(orc.experts_backward_oracle(inp["grad_out"], *[inp[k] for k in KEYS], cap, E, K))
        if not dense:
            ref_g[1] = torch.gather(ref_g[1], 1, inp["router_indices"])
        for j, name in enumerate(["d_hidden", "d_routing", "d_wgu", "d_bgu", "d_wd", "d_bd"]):
            got_g = torch.cat([r[1][i][1][j] for r in results])
            orc.check_close(got_g, ref_g[j], 2e-2, f"peer-store backward {name}, call {i}", rel_l2=2e-2)


def test_bounded_wait_gives_up_on_one_gpu():
    """The one-warp wait of the expert-parallel path on flags nobody sets: with a 1 ms limit it must
    return the time-out status and leave the GPU usable; with the flags set it must report 0."""
    import ctypes
    from yamoe_b200 import _lib
    L = _lib.lib()
    G = 4
    flags = torch.zeros(G, dtype=torch.int32, device="cuda")
    state = torch.zeros(64, dtype=torch.int32, device="cuda")
    header = torch.zeros(16, dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(L.yamoe_b200_ep_wait_probe(flags.data_ptr(), G, 3, 1_000_000, state.data_ptr(), header.data_ptr(), st),
               "ep_wait_probe")
    torch.cuda.synchronize()
    assert int(header[4]) == 5 and int(state[0]) == 3
    flags.fill_(3)
    _lib.check(L.yamoe_b200_ep_wait_probe(flags.data_ptr(), G, 3, 1_000_000, state.data_ptr(), header.data_ptr(), st),
               "ep_wait_probe")
    torch.cuda.synchronize()
    assert int(header[4]) == 0
    assert float((torch.ones(8, device="cuda") * 2).sum()) == 16.0      # the context still works
