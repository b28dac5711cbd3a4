"""Expert-parallel forward: the experts of one layer sharded contiguously over the ranks of a
process group, tokens sharded by rows (data-parallel), one all-to-all each way.

The reference is single-GPU and has nothing like this; the result must equal the single-GPU op
(`yamoe_b200.experts`, hence `reference.py`) on the concatenated tokens with all experts.

Per call, on every rank r (G ranks, E experts, E/G local experts, T_r local tokens):

1. route      stable sort of the local (token, slot) assignments by global expert id -> counts[E]
2. counts     all_to_all of the [G, E/G] count matrix: every rank learns how many rows each peer
              sends for each of its local experts
3. dispatch   rows hidden[token] in expert-sorted order (permute_rows kernel), all_to_all with the
              split sizes of step 2
4. compute    the received rows are tokens of a local problem with top_k = 1: expert id = local
              expert, weight 1; one call of the expert op on the local weight shard.  Rows arrive
              source-major and the op's sort is stable, so the capacity keeps the first C
              assignments of an expert in global token order, exactly like the single-GPU op.
5. combine    all_to_all back, then out[t] = sum_k w[t,k] * row(t,k) (combine_rows kernel)

The split sizes of steps 3 and 5 live on the host because `all_to_all_single` wants them there:
one device-to-host copy of 2*G integers per call.

`Backend` bundles the compute steps so that the exchange logic can be exercised on CPU ranks
(gloo) with stand-in compute; the default backend is the CUDA library, and nothing else ships.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.distributed as dist


@dataclass
class Backend:
    route: Callable        # (router_indices [T,K], E) -> sorted_values, sorted_indices, bins, counts
    permute_rows: Callable  # (hidden [T,H], sorted_indices, K) -> rows [S,H]
    experts: Callable      # the expert op
    combine_rows: Callable  # (rows [S,H], sorted_indices, router_indices, routing_weights, E) -> [T,H]
    experts_backward: Optional[Callable] = None   # the backward op


def cuda_backend() -> Backend:
    from . import ops
    return Backend(route=ops.route, permute_rows=ops.permute_rows, experts=ops.experts,
                   combine_rows=ops.combine_rows, experts_backward=ops.experts_backward)


def expert_range(rank: int, world: int, num_experts: int):
    """Contiguous shard of experts owned by `rank`."""
    if num_experts % world != 0:
        raise ValueError(f"num_experts ({num_experts}) must be divisible by the group size ({world})")
    per = num_experts // world
    return rank * per, (rank + 1) * per


def shard_expert_weights(gate_up_proj, gate_up_proj_bias, down_proj, down_proj_bias, rank, world):
    """Slices the four [E, ...] tensors to this rank's contiguous expert shard."""
    lo, hi = expert_range(rank, world, gate_up_proj.shape[0])
    return (gate_up_proj[lo:hi].contiguous(), gate_up_proj_bias[lo:hi].contiguous(),
            down_proj[lo:hi].contiguous(), down_proj_bias[lo:hi].contiguous())


def exchange_plan(counts: torch.Tensor, world: int, group=None):
    """counts: int32/int64 [E] local histogram.  Returns (recv_counts [G, E/G] on the device,
    send_splits, recv_splits as Python lists)."""
    E = counts.numel()
    per = E // world
    send_counts = counts.to(torch.int64).view(world, per).contiguous()
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    both = torch.stack([send_counts.sum(1), recv_counts.sum(1)]).cpu()
    return recv_counts, both[0].tolist(), both[1].tolist()


def ep_experts(hidden_states, router_indices, routing_weights, gate_up_local, gate_up_bias_local, down_local,
               down_bias_local, expert_capacity: int, num_experts: int, top_k: int, group=None,
               backend: Optional[Backend] = None, stats: Optional[dict] = None):
    """Expert-parallel `experts`.  `hidden_states` [T_r, H], `router_indices` [T_r, K] (global expert
    ids) and `routing_weights` [T_r, E] or [T_r, K] are this rank's token shard; the four weight
    tensors are this rank's expert shard ([E/G, ...]).  Returns this rank's [T_r, H] output."""
    be = backend or cuda_backend()
    world = dist.get_world_size(group)
    E, K = int(num_experts), int(top_k)
    per = E // world
    if gate_up_local.shape[0] != per:
        raise RuntimeError(f"expected {per} local experts, got {gate_up_local.shape[0]}")
    H = hidden_states.shape[1]

    _, sorted_indices, _, counts = be.route(router_indices, E)
    recv_counts, send_splits, recv_splits = exchange_plan(counts, world, group)
    n_send, n_recv = sum(send_splits), sum(recv_splits)
    sorted_indices = sorted_indices[:n_send]

    rows = be.permute_rows(hidden_states, sorted_indices, K)
    recv = torch.empty(n_recv, H, dtype=rows.dtype, device=rows.device)
    dist.all_to_all_single(recv, rows, recv_splits, send_splits, group=group)

    # local problem: one "token" per received row, top_k = 1, weight 1
    local_ids = torch.repeat_interleave(
        torch.arange(per, device=recv.device).repeat(world), recv_counts.view(-1).to(recv.device),
        output_size=n_recv).view(n_recv, 1)
    ones = torch.ones(n_recv, 1, dtype=recv.dtype, device=recv.device)
    y = be.experts(recv, local_ids, ones, gate_up_local, gate_up_bias_local, down_local, down_bias_local,
                   int(expert_capacity), per, 1)

    back = torch.empty(n_send, H, dtype=y.dtype, device=y.device)
    dist.all_to_all_single(back, y, send_splits, recv_splits, group=group)
    out = be.combine_rows(back, sorted_indices, router_indices, routing_weights, E)
    if stats is not None:
        stats.update(rows_sent=n_send, rows_received=n_recv, send_splits=send_splits, recv_splits=recv_splits)
    return out


def ep_experts_backward(grad_out, hidden_states, router_indices, routing_weights, gate_up_local,
                        gate_up_bias_local, down_local, down_bias_local, expert_capacity: int, num_experts: int,
                        top_k: int, group=None, backend: Optional[Backend] = None):
    """Expert-parallel `experts_backward`.  Same sharding as `ep_experts`; `grad_out` is this rank's
    [T_r, H] slice.  The exchange mirrors the forward: token rows, their upstream-gradient rows and
    their routing weights travel to the expert owners, which run the backward op on a local problem
    with top_k = 1; per-row input gradients and routing-weight gradients travel back.  Weight and
    bias gradients stay with the expert owner (experts are not replicated, so no all-reduce).

    Returns (d_hidden [T_r,H], d_routing [T_r, cols], d_gate_up_local, d_gate_up_bias_local,
    d_down_local, d_down_bias_local)."""
    be = backend or cuda_backend()
    world = dist.get_world_size(group)
    E, K = int(num_experts), int(top_k)
    per = E // world
    T, H = hidden_states.shape
    dt, dev = hidden_states.dtype, hidden_states.device

    _, sorted_indices, _, counts = be.route(router_indices, E)
    recv_counts, send_splits, recv_splits = exchange_plan(counts, world, group)
    n_send, n_recv = sum(send_splits), sum(recv_splits)
    sorted_indices = sorted_indices[:n_send]
    si = sorted_indices.long()

    dense = routing_weights.shape[1] == E
    w_sel = torch.gather(routing_weights, 1, router_indices.to(torch.int64)) if dense else routing_weights
    rows_x = be.permute_rows(hidden_states, sorted_indices, K)
    rows_g = be.permute_rows(grad_out.reshape(T, H), sorted_indices, K)
    rows_w = w_sel.reshape(-1)[si].reshape(n_send, 1).contiguous()

    def exchange(t, out_rows, out_splits, in_splits):
        buf = torch.empty(out_rows, t.shape[1], dtype=t.dtype, device=t.device)
        dist.all_to_all_single(buf, t.contiguous(), out_splits, in_splits, group=group)
        return buf

    recv_x = exchange(rows_x, n_recv, recv_splits, send_splits)
    recv_g = exchange(rows_g, n_recv, recv_splits, send_splits)
    recv_w = exchange(rows_w, n_recv, recv_splits, send_splits)
    local_ids = torch.repeat_interleave(
        torch.arange(per, device=dev).repeat(world), recv_counts.view(-1).to(dev), output_size=n_recv).view(n_recv, 1)

    d_rows, d_w_rows, d_wgu, d_bgu, d_wd, d_bd = be.experts_backward(
        recv_g, recv_x, local_ids, recv_w, gate_up_local, gate_up_bias_local, down_local, down_bias_local,
        int(expert_capacity), per, 1)

    back_rows = exchange(d_rows, n_send, send_splits, recv_splits)
    back_w = exchange(d_w_rows.reshape(n_recv, 1), n_send, send_splits, recv_splits)

    ones = torch.ones(T, K, dtype=dt, device=dev)
    d_hidden = be.combine_rows(back_rows, sorted_indices, router_indices, ones, E)
    d_sel = torch.zeros(T * K, dtype=dt, device=dev)
    d_sel[si] = back_w.reshape(-1)
    if dense:
        d_routing = torch.zeros(T, E, dtype=dt, device=dev)
        d_routing.scatter_(1, router_indices.to(torch.int64), d_sel.view(T, K))
    else:
        d_routing = d_sel.view(T, K)
    return d_hidden, d_routing, d_wgu, d_bgu, d_wd, d_bd


class PeerExpertParallel:
    """Expert-parallel forward (and, with `backward=True`, backward) whose dispatch and combine are
    peer stores over NVLink.

    All offsets come from the all-gathered [G, E] count matrix on the device: a call makes no
    device-to-host copy and needs no split sizes.  Buffers that peers write into are symmetric
    allocations made once, sized for `max_tokens_total` tokens over all ranks (worst case: every
    assignment lands on one rank) and `max_tokens_local` tokens on this rank.

    Sequence per call (one stream): route -> all_gather(counts) -> plan -> dispatch (peer stores) ->
    barrier -> grouped GEMMs on the received rows, the down GEMM's epilogue storing each result row
    straight into the token owner's buffer (`fused_return`; otherwise a separate return kernel) ->
    barrier -> combine.
    The barriers are stream-ordered collectives; no kernel of this path waits on another GPU.
    """

    def __init__(self, hidden: int, num_experts: int, top_k: int, max_tokens_total: int, max_tokens_local: int,
                 dtype=torch.bfloat16, group=None, fused_return: bool = False, backward: bool = False):
        import torch.distributed._symmetric_memory as symm_mem
        self.fused_return = bool(fused_return)
        from . import _lib
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.H, self.E, self.K, self.dtype = int(hidden), int(num_experts), int(top_k), dtype
        if self.E % self.world:
            raise ValueError("num_experts must be divisible by the group size")
        self.per = self.E // self.world
        self.dt = _lib.YAMOE_BF16 if dtype == torch.bfloat16 else _lib.YAMOE_F32
        s_total = max_tokens_total * self.K
        self.max_rows = ((s_total + 127) // 128 + self.per) * 128
        self.s_local = max_tokens_local * self.K
        dev = torch.device("cuda", torch.cuda.current_device())
        self.recv = symm_mem.empty(self.max_rows, self.H, dtype=dtype, device=dev)
        self.back = symm_mem.empty(max(self.s_local, 1), self.H, dtype=dtype, device=dev)
        h_recv = symm_mem.rendezvous(self.recv, self.group)
        h_back = symm_mem.rendezvous(self.back, self.group)
        self.peer_recv = torch.tensor(list(h_recv.buffer_ptrs), dtype=torch.int64, device=dev)
        self.peer_back = torch.tensor(list(h_back.buffer_ptrs), dtype=torch.int64, device=dev)
        self._handles = [h_recv, h_back]
        self.L = _lib.lib()
        self.has_backward = bool(backward)
        if self.has_backward:
            # upstream-gradient rows and routing weights travel to the expert owners, routing-weight
            # gradients travel back: three more buffers that peers write into
            self.recv_g = symm_mem.empty(self.max_rows, self.H, dtype=dtype, device=dev)
            self.recv_w = symm_mem.empty(self.max_rows, dtype=torch.float32, device=dev)
            self.back_w = symm_mem.empty(max(self.s_local, 1), dtype=torch.float32, device=dev)
            hs_ = [symm_mem.rendezvous(t, self.group) for t in (self.recv_g, self.recv_w, self.back_w)]
            self.peer_recv_g, self.peer_recv_w, self.peer_back_w = (
                torch.tensor(list(h.buffer_ptrs), dtype=torch.int64, device=dev) for h in hs_)
            self._handles += hs_
        ws_bytes = self.L.yamoe_b200_ep_backward_workspace_bytes if self.has_backward \
            else self.L.yamoe_b200_ep_workspace_bytes
        nbytes = ws_bytes(self.max_rows, self.H, self.E, self.world, self.dt)
        if nbytes == 0:
            raise RuntimeError("yamoe_b200: unsupported expert-parallel configuration")
        self.ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        self.y_rows = torch.empty(self.max_rows, self.H, dtype=dtype, device=dev)
        self.counts_all = torch.empty(self.world, self.E, dtype=torch.int32, device=dev)
        self.flag = torch.zeros(1, dtype=torch.int32, device=dev)
        self._check = _lib.check
        # padding rows of the receive buffer enter the weight-gradient GEMMs as the k dimension
        # (times zero): they must hold finite values, so start from zeros before any peer writes
        self.recv.zero_()
        self._barrier()

    def _barrier(self):
        dist.all_reduce(self.flag, group=self.group)      # stream-ordered; orders the peer stores

    def forward(self, hidden_states, router_indices, routing_weights, gate_up_local, gate_up_bias_local,
                down_local, down_bias_local, expert_capacity: int):
        from . import ops
        T, K = router_indices.shape
        if T * K > self.s_local or K != self.K or hidden_states.shape[1] != self.H:
            raise RuntimeError("PeerExpertParallel: call exceeds the sizes the buffers were made for")
        L, st = self.L, torch.cuda.current_stream().cuda_stream
        hs = hidden_states.contiguous()
        sv, si, bins, counts = ops.route(router_indices, self.E)
        dist.all_gather_into_tensor(self.counts_all.view(-1), counts, group=self.group)
        self._check(L.yamoe_b200_ep_plan(self.counts_all.data_ptr(), self.world, self.rank, self.E,
                                         int(expert_capacity), self.peer_back.data_ptr(), self.max_rows, self.H,
                                         self.dt, self.ws.data_ptr(), self.ws.numel(), st), "ep_plan")
        self._check(L.yamoe_b200_ep_dispatch(hs.data_ptr(), sv.data_ptr(), si.data_ptr(), bins.data_ptr(), T * K,
                                             self.peer_recv.data_ptr(), self.max_rows, self.H, self.E, self.world, K,
                                             self.dt, self.ws.data_ptr(), st), "ep_dispatch")
        self._barrier()
        y_ptr = None if self.fused_return else self.y_rows.data_ptr()
        self._check(L.yamoe_b200_ep_local_forward(self.recv.data_ptr(), gate_up_local.data_ptr(),
                                                  gate_up_bias_local.data_ptr(), down_local.data_ptr(),
                                                  down_bias_local.data_ptr(), y_ptr, self.max_rows,
                                                  self.H, self.E, self.world, self.dt, self.ws.data_ptr(), st),
                    "ep_local_forward")
        if not self.fused_return:
            self._check(L.yamoe_b200_ep_return(self.y_rows.data_ptr(), self.peer_back.data_ptr(), self.max_rows,
                                               self.H, self.E, self.world, self.dt, self.ws.data_ptr(), st),
                        "ep_return")
        self._barrier()
        return ops.combine_rows(self.back[: T * K], si, router_indices, routing_weights, self.E)

    def backward(self, grad_out, hidden_states, router_indices, routing_weights, gate_up_local, gate_up_bias_local,
                 down_local, down_bias_local, expert_capacity: int):
        """Expert-parallel `experts_backward` over the same peer buffers (made with `backward=True`).
        Returns what `ep_experts_backward` returns: (d_hidden [T_r,H], d_routing [T_r, cols],
        d_gate_up_local, d_gate_up_bias_local, d_down_local, d_down_bias_local)."""
        from . import ops
        if not self.has_backward:
            raise RuntimeError("PeerExpertParallel: made without backward=True")
        T, K = router_indices.shape
        H, E = self.H, self.E
        if T * K > self.s_local or K != self.K or hidden_states.shape[1] != H:
            raise RuntimeError("PeerExpertParallel: call exceeds the sizes the buffers were made for")
        L, st = self.L, torch.cuda.current_stream().cuda_stream
        dt, dev = hidden_states.dtype, hidden_states.device
        hs = hidden_states.contiguous()
        go = grad_out.reshape(T, H).contiguous()
        rw = routing_weights.contiguous()
        rcols = rw.shape[1]
        sv, si, bins, counts = ops.route(router_indices, E)
        dist.all_gather_into_tensor(self.counts_all.view(-1), counts, group=self.group)
        ws, S = self.ws.data_ptr(), T * K
        self._check(L.yamoe_b200_ep_plan(self.counts_all.data_ptr(), self.world, self.rank, E, int(expert_capacity),
                                         self.peer_back.data_ptr(), self.max_rows, H, self.dt, ws, self.ws.numel(),
                                         st), "ep_plan")
        for src, peers in ((hs, self.peer_recv), (go, self.peer_recv_g)):
            self._check(L.yamoe_b200_ep_dispatch(src.data_ptr(), sv.data_ptr(), si.data_ptr(), bins.data_ptr(), S,
                                                 peers.data_ptr(), self.max_rows, H, E, self.world, K, self.dt, ws,
                                                 st), "ep_dispatch")
        self._check(L.yamoe_b200_ep_dispatch_weights(rw.data_ptr(), rcols, sv.data_ptr(), si.data_ptr(),
                                                     bins.data_ptr(), S, self.peer_recv_w.data_ptr(), self.max_rows,
                                                     H, E, self.world, K, self.dt, ws, st), "ep_dispatch_weights")
        self._barrier()
        d_wgu, d_bgu = torch.empty_like(gate_up_local), torch.empty_like(gate_up_bias_local)
        d_wd, d_bd = torch.empty_like(down_local), torch.empty_like(down_bias_local)
        self._check(L.yamoe_b200_ep_local_backward(
            self.recv.data_ptr(), self.recv_g.data_ptr(), self.recv_w.data_ptr(), gate_up_local.data_ptr(),
            gate_up_bias_local.data_ptr(), down_local.data_ptr(), down_bias_local.data_ptr(), d_wgu.data_ptr(),
            d_bgu.data_ptr(), d_wd.data_ptr(), d_bd.data_ptr(), self.peer_back_w.data_ptr(), int(expert_capacity),
            self.max_rows, H, E, self.world, self.dt, ws, self.ws.numel(), st), "ep_local_backward")
        self._barrier()
        n_sorted = si.numel()
        ones = torch.ones(T, K, dtype=dt, device=dev)
        d_hidden = ops.combine_rows(self.back[:S], si, router_indices, ones, E)
        d_sel = torch.zeros(S, dtype=dt, device=dev)
        d_sel[si.long()] = self.back_w[:n_sorted].to(dt)
        if rcols == E:
            d_routing = torch.zeros(T, E, dtype=dt, device=dev)
            d_routing.scatter_(1, router_indices.to(torch.int64), d_sel.view(T, K))
        else:
            d_routing = d_sel.view(T, K)
        return d_hidden, d_routing, d_wgu, d_bgu, d_wd, d_bd
