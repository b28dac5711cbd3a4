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
    peer stores over NVLink and whose phase boundaries are flags in symmetric memory.

    One call is ONE entry into the library (`yamoe_b200_ep_forward` / `yamoe_b200_ep_backward`): a
    fixed chain of kernels on the current stream, with no NCCL collective, no device-to-host copy
    and no split sizes.  Per call: local sort -> my per-expert counts to every rank (flag) ->
    dispatch kernel (waits for all counts, derives every offset on the device, stores my rows into
    the owners' GEMM input layout, flag) -> wait for all sources -> grouped GEMMs on the received
    rows, the last one storing each result row straight into the token owner's buffer from its
    epilogue (flag) -> combine kernel (waits for all owners).  Every wait is bounded
    (`wait_seconds`); `status()` reads the device status word of the last call.

    Buffers that peers write into are symmetric allocations made once, sized for
    `max_tokens_total` tokens over all ranks (worst case: every assignment lands on one rank) and
    `max_tokens_local` tokens on this rank.  Construction is collective (it ends with a barrier);
    afterwards all ranks must make the same sequence of forward / backward calls.
    """

    def __init__(self, hidden: int, num_experts: int, top_k: int, max_tokens_total: int, max_tokens_local: int,
                 dtype=torch.bfloat16, group=None, backward: bool = False, wait_seconds: float = 2.0):
        import ctypes
        import torch.distributed._symmetric_memory as symm_mem
        from . import _lib
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.H, self.E, self.K, self.dtype = int(hidden), int(num_experts), int(top_k), dtype
        if self.E % self.world:
            raise ValueError("num_experts must be divisible by the group size")
        if max_tokens_local > max_tokens_total:
            raise ValueError("max_tokens_local cannot exceed max_tokens_total")
        self.per = self.E // self.world
        self.dt = _lib.YAMOE_BF16 if dtype == torch.bfloat16 else _lib.YAMOE_F32
        s_total = int(max_tokens_total) * self.K
        self.max_rows = ((s_total + 127) // 128 + self.per) * 128
        self.s_local = max(int(max_tokens_local) * self.K, 1)
        self.t_local = int(max_tokens_local)
        dev = torch.device("cuda", torch.cuda.current_device())
        self.L = L = _lib.lib()
        self._check = _lib.check
        self.has_backward = bool(backward)

        def symmetric(shape, dt):
            t = symm_mem.empty(*shape, dtype=dt, device=dev)
            t.zero_()
            h = symm_mem.rendezvous(t, self.group)
            ptrs = torch.tensor(list(h.buffer_ptrs), dtype=torch.int64, device=dev)
            self._keep.append((t, h, ptrs))
            return t, ptrs

        self._keep = []
        # padding rows of the receive buffers enter the weight-gradient GEMMs as the k dimension
        # (times zero): they must hold finite values, hence the zero fill
        self.recv, p_recv = symmetric((self.max_rows, self.H), dtype)
        self.back, p_back = symmetric((self.s_local, self.H), dtype)
        ctrl_words = L.yamoe_b200_ep_ctrl_bytes(self.world, self.E) // 4
        self.ctrl, p_ctrl = symmetric((ctrl_words,), torch.int32)
        ctx = _lib.EpCtx(G=self.world, rank=self.rank, E=self.E, K=self.K, H=self.H, dtype=self.dt,
                         max_rows=self.max_rows, back_rows=self.s_local,
                         peer_recv_x=p_recv.data_ptr(), peer_back=p_back.data_ptr(), peer_ctrl=p_ctrl.data_ptr(),
                         recv_x=self.recv.data_ptr(), back=self.back.data_ptr(), ctrl=self.ctrl.data_ptr(),
                         wait_ns=int(wait_seconds * 1e9))
        if self.has_backward:
            # upstream-gradient rows and routing weights travel to the expert owners, routing-weight
            # gradients travel back: three more buffers that peers write into
            self.recv_g, p_recv_g = symmetric((self.max_rows, self.H), dtype)
            self.recv_w, p_recv_w = symmetric((self.max_rows,), torch.float32)
            self.back_w, p_back_w = symmetric((self.s_local,), torch.float32)
            ctx.peer_recv_g, ctx.peer_recv_w, ctx.peer_back_w = (p_recv_g.data_ptr(), p_recv_w.data_ptr(),
                                                                   p_back_w.data_ptr())
            ctx.recv_g, ctx.recv_w, ctx.back_w = self.recv_g.data_ptr(), self.recv_w.data_ptr(), self.back_w.data_ptr()
        self.state = torch.zeros(64, dtype=torch.int32, device=dev)
        ctx.state = self.state.data_ptr()
        self.ctx = ctx
        self._ctx_ref = ctypes.byref(ctx)
        nbytes = L.yamoe_b200_ep_call_workspace_bytes(self._ctx_ref, self.t_local, int(self.has_backward))
        if nbytes == 0:
            raise RuntimeError("yamoe_b200: unsupported expert-parallel configuration")
        self.ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        torch.cuda.synchronize()
        dist.barrier(group=self.group)       # every rank's control block is zero before anyone publishes

    def status(self) -> int:
        """Device status word of the last call (synchronises the current stream): 0 = every wait
        completed; 4 / 5 / 6 = the wait for counts / dispatched rows / returned rows gave up;
        7 = the rows routed to one rank exceed the receive buffers; 1-3 = a GEMM pipeline wait."""
        import ctypes
        out = ctypes.c_int32(0)
        self._check(self.L.yamoe_b200_device_status(self.ws.data_ptr(), torch.cuda.current_stream().cuda_stream,
                                                    ctypes.byref(out)), "device_status")
        return int(out.value)

    def _common(self, hidden_states, router_indices, routing_weights):
        T, K = router_indices.shape
        if T > self.t_local or K != self.K or hidden_states.shape[1] != self.H:
            raise RuntimeError("PeerExpertParallel: call exceeds the sizes the buffers were made for")
        if hidden_states.dtype != self.dtype or routing_weights.dtype != self.dtype:
            raise RuntimeError("PeerExpertParallel: dtype differs from the one the buffers were made for")
        rw = routing_weights.contiguous()
        if rw.shape[1] not in (self.K, self.E):
            raise RuntimeError("routing_weights must be [T, K] or [T, E]")
        return T, hidden_states.contiguous(), router_indices.to(torch.int64).contiguous(), rw

    def forward(self, hidden_states, router_indices, routing_weights, gate_up_local, gate_up_bias_local,
                down_local, down_bias_local, expert_capacity: int):
        T, hs, ri, rw = self._common(hidden_states, router_indices, routing_weights)
        if gate_up_local.shape[0] != self.per:
            raise RuntimeError(f"expected {self.per} local experts, got {gate_up_local.shape[0]}")
        out = torch.empty_like(hs)
        st = torch.cuda.current_stream().cuda_stream
        self._check(self.L.yamoe_b200_ep_forward(
            self._ctx_ref, hs.data_ptr(), ri.data_ptr(), rw.data_ptr(), rw.shape[1], gate_up_local.data_ptr(),
            gate_up_bias_local.data_ptr(), down_local.data_ptr(), down_bias_local.data_ptr(), out.data_ptr(), T,
            int(expert_capacity), self.ws.data_ptr(), self.ws.numel(), st), "ep_forward")
        return out

    def backward(self, grad_out, hidden_states, router_indices, routing_weights, gate_up_local, gate_up_bias_local,
                 down_local, down_bias_local, expert_capacity: int):
        """Expert-parallel `experts_backward` over the same peer buffers (made with `backward=True`).
        Returns what `ep_experts_backward` returns: (d_hidden [T_r,H], d_routing [T_r, cols],
        d_gate_up_local, d_gate_up_bias_local, d_down_local, d_down_bias_local)."""
        if not self.has_backward:
            raise RuntimeError("PeerExpertParallel: made without backward=True")
        T, hs, ri, rw = self._common(hidden_states, router_indices, routing_weights)
        go = grad_out.reshape(T, self.H).contiguous()
        d_hidden, d_routing = torch.empty_like(hs), torch.empty_like(rw)
        d_wgu, d_bgu = torch.empty_like(gate_up_local), torch.empty_like(gate_up_bias_local)
        d_wd, d_bd = torch.empty_like(down_local), torch.empty_like(down_bias_local)
        st = torch.cuda.current_stream().cuda_stream
        self._check(self.L.yamoe_b200_ep_backward(
            self._ctx_ref, go.data_ptr(), hs.data_ptr(), ri.data_ptr(), rw.data_ptr(), rw.shape[1],
            gate_up_local.data_ptr(), gate_up_bias_local.data_ptr(), down_local.data_ptr(), down_bias_local.data_ptr(),
            d_hidden.data_ptr(), d_routing.data_ptr(), d_wgu.data_ptr(), d_bgu.data_ptr(), d_wd.data_ptr(),
            d_bd.data_ptr(), T, int(expert_capacity), self.ws.data_ptr(), self.ws.numel(), st), "ep_backward")
        return d_hidden, d_routing, d_wgu, d_bgu, d_wd, d_bd
