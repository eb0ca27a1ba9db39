"""Expert-parallel MoE dispatch and combine: one exchange step each way.

popcorn has no distributed code at all (its `momoe` op is single-GPU,
src/popcorn/kernels/momoe.py:34-53); this module is the multi-GPU form of the
permute / unpermute path.  Layout: tokens are sharded across ranks (each rank
routes its own tokens), experts are sharded in contiguous blocks
(expert e lives on rank e // (experts / world)).

dispatch(x, logits) on every rank:
  1. route the local tokens and build the local stable permutation (CUDA kernels);
     local rows are sorted by expert, hence already grouped by destination rank;
  2. all-gather the per-expert counts (world x experts int32) -- the only
     host-visible metadata; it gives every rank its send and receive split sizes;
  3. permute the local rows into the send buffer (CUDA kernel);
  4. all-to-all of the rows with those split sizes (NCCL over NVLink);
  5. reorder what arrived, (source rank, expert, token), into (expert, source rank,
     token) with the gather kernel.  Source ranks own ascending token ranges, so
     this is exactly the global stable order (expert, global token id) that a
     single GPU would produce.

combine(expert_rows) mirrors it: inverse reorder, all-to-all back with the split
sizes swapped, weighted unpermute on the owner rank.

The per-rank compute steps come from `local_ops` (default: popcorn_b200.ops, the
CUDA kernels).  Tests of the exchange logic on CPU processes pass a namespace of
CPU functions with the same signatures and run it over the gloo backend.

exchange="p2p" (CUDA only) fuses each exchange into the kernel next to it and keeps the host out of the step.
Every rank owns symmetric buffers that all ranks map (torch symmetric memory over NVLink): `recv`, which the
ranks' permute kernels fill with ordinary stores straight from their token rows, already in the final
(expert, source rank, token) order; `out`, from which the token owners' unpermute kernels load the expert outputs
while they accumulate; and a small `meta` buffer of counts and flags.  A step is then: route, index, one kernel that
writes this rank's per-expert counts into every rank's meta buffer, waits (bounded) for everybody's and derives the
addressing on the device, the destinations kernel, the permute kernel, a flag rendezvous; and for the combine a flag
rendezvous and the unpermute kernel.  No bulk collective, no NCCL call, no staging buffer, no reorder pass and no
device-to-host copy: `Dispatched.rows` is the whole receive buffer and `expert_offsets` (a device tensor) says which
rows are in use, which is what the grouped expert GEMM reads.  A wait that runs out or a receive beyond the buffers'
capacity is recorded in a status word (`ExpertParallel.check()` reads it) instead of hanging or trapping.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch
import torch.distributed as dist
from torch import Tensor


def check_counts(counts_all: Tensor, rank: int) -> None:
    """The gathered [world, experts] count table must be usable before any row moves: a malformed table (a rank that
    posted garbage, a table of the wrong shape) is reported on the host instead of becoming a wild address."""
    if counts_all.dim() != 2 or counts_all.shape[0] == 0:
        raise ValueError(f"expected a [world, experts] count table, got shape {tuple(counts_all.shape)}")
    world, experts = counts_all.shape
    if experts % world != 0:
        raise ValueError(f"experts={experts} must be a multiple of the world size {world}")
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside the table's world size {world}")
    if counts_all.is_floating_point() or bool((counts_all < 0).any()):
        raise ValueError("per-expert counts must be non-negative integers")


def p2p_plan(counts_all: Tensor, rank: int) -> tuple[Tensor, list[int], Tensor]:
    """Addressing for the fused exchange, from the [world, experts] count table, as host arithmetic: the statement of
    what `b200_moe_ep_exchange` computes on the device (the step itself no longer runs this; the tests hold the kernel
    to it, and a host that already has the table can use it).

    Returns (dst_base int32 [experts], rows_per_rank, expert_offsets int32 [local_experts + 1]):
    dst_base[e] is the row in the buffer of e's owner at which THIS rank's rows for expert e start:
    the owner's buffer is expert-major, and inside an expert the source ranks follow in rank order;
    rows_per_rank[r] is how many rows rank r receives in total; expert_offsets delimit this rank's
    own experts inside its buffer."""
    check_counts(counts_all, rank)
    world, experts = counts_all.shape
    if experts % world != 0:
        raise ValueError(f"experts={experts} must be a multiple of the world size {world}")
    per_rank = experts // world
    c = counts_all.to(torch.int64)
    total = c.sum(0)  # rows per expert over all sources
    blocks = total.view(world, per_rank)
    expert_base = (torch.cumsum(blocks, 1) - blocks).view(-1)  # start of each expert inside its owner's buffer
    before_me = c[:rank].sum(0)  # rows of lower source ranks inside the expert
    dst_base = (expert_base + before_me).to(torch.int32)
    rows_per_rank = blocks.sum(1).tolist()
    expert_offsets = torch.zeros(per_rank + 1, dtype=torch.int64)
    expert_offsets[1:] = torch.cumsum(blocks[rank], 0)
    return dst_base, rows_per_rank, expert_offsets.to(torch.int32)


@dataclass
class Dispatched:
    """What dispatch() hands to the expert computation, plus what combine() needs later."""

    rows: Tensor            # [received, hidden], grouped by local expert, global stable order inside
                            # (exchange="p2p": the whole receive buffer; expert_offsets[-1] rows of it are in use)
    expert_offsets: Tensor  # int32 [local_experts + 1] into rows (host tensor; exchange="p2p": device tensor)
    weights: Tensor         # fp32 [local_tokens, top_k]
    pos: Tensor             # int32 [local_tokens, top_k] positions in this rank's send buffer
    send_counts: list[int]  # rows sent to each rank
    recv_counts: list[int]  # rows received from each rank
    reorder: Tensor | None  # int32 [received]: rows[p] = arrived[reorder[p]]  (exchange="nccl")
    counts_all: Tensor | None  # int32 [world, experts] (host tensor; None with exchange="p2p", whose counts stay on the device)
    dst_rank: Tensor | None = None  # int32 [local_tokens, top_k]: owner of each pair's expert   (exchange="p2p")
    dst_row: Tensor | None = None   # int32 [local_tokens, top_k]: row in the owner's buffer      (exchange="p2p")
    out_rows: Tensor | None = None  # the symmetric output buffer, rows as in `rows`: write expert results here
    info: Tensor | None = None      # int32 [4] on the device: rows received, rows sent to other ranks, largest receive, world


def exchange_plan(counts_all: Tensor, rank: int) -> tuple[list[int], list[int], Tensor, Tensor, Tensor]:
    """Split sizes and the reorder segments of `rank`, from the gathered counts (host arithmetic).

    counts_all: int [world, experts]; experts are owned in contiguous blocks.
    Returns (send_counts, recv_counts, segment_source_start, segment_length, expert_offsets):
    segments are listed in output order (local expert major, source rank minor); segment i covers
    arrived[segment_source_start[i] : +segment_length[i]]."""
    check_counts(counts_all, rank)
    world, experts = counts_all.shape
    if experts % world != 0:
        raise ValueError(f"experts={experts} must be a multiple of the world size {world}")
    per_rank = experts // world
    counts_all = counts_all.to(torch.int64)
    send_counts = counts_all[rank].view(world, per_rank).sum(1).tolist()
    mine = counts_all[:, rank * per_rank : (rank + 1) * per_rank]  # [source, local expert]
    recv_counts = mine.sum(1).tolist()
    recv_base = torch.zeros(world, dtype=torch.int64)
    recv_base[1:] = torch.cumsum(mine.sum(1), 0)[:-1]
    within = torch.cumsum(mine, 1) - mine  # start of each local expert inside its source block
    source_start = (recv_base[:, None] + within).t().contiguous().view(-1)  # (expert major, source minor)
    length = mine.t().contiguous().view(-1)
    expert_offsets = torch.zeros(per_rank + 1, dtype=torch.int64)
    expert_offsets[1:] = torch.cumsum(mine.sum(0), 0)
    return send_counts, recv_counts, source_start, length, expert_offsets.to(torch.int32)


def expand_segments(source_start: Tensor, length: Tensor, total: int, device: torch.device | str) -> Tensor:
    """int32 [total] index: the concatenation of arange(start, start + length) over the segments."""
    if total == 0:
        return torch.empty(0, dtype=torch.int32, device=device)
    out_start = torch.cumsum(length, 0) - length
    delta = (source_start - out_start).to(device)
    index = torch.repeat_interleave(delta, length.to(device), output_size=total) + torch.arange(total, device=device)
    return index.to(torch.int32)


class ExpertParallel:
    """Token-sharded routing with block-sharded experts over a torch.distributed group."""

    def __init__(self, experts: int, top_k: int, group: Any = None, local_ops: Any = None,
                 exchange: str = "nccl", capacity_rows: int | None = None) -> None:
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if experts % self.world != 0:
            raise ValueError(f"experts={experts} must be a multiple of the world size {self.world}")
        if exchange not in ("nccl", "p2p"):
            raise ValueError("exchange must be 'nccl' or 'p2p'")
        self.experts, self.top_k = experts, top_k
        self.local_experts = experts // self.world
        if local_ops is None:
            from popcorn_b200 import ops as local_ops
        self.ops = local_ops
        self.exchange = exchange
        self.capacity_rows = capacity_rows
        self._symmetric = None  # (recv, out, recv_ptrs, out_ptrs, capacity, hidden, dtype), built on first use
        self._meta_ptrs: list[int] = []
        self._status: Tensor | None = None  # int32 [2] on the device: first failure of a fused-exchange kernel
        self._epoch = 0

    # -- fused exchange over peer memory ------------------------------------------------------------

    def _buffers(self, x: Tensor):
        """The two symmetric row buffers, allocated and mapped on the first dispatch."""
        if self._symmetric is not None:
            recv, out, recv_ptrs, out_ptrs, capacity, hidden, dtype = self._symmetric
            if hidden != x.shape[1] or dtype != x.dtype:
                raise ValueError("ExpertParallel(exchange='p2p') was set up for another hidden size or dtype")
            return self._symmetric
        import os

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer loads/stores only
        import torch.distributed._symmetric_memory as symm_mem

        group = self.group if self.group is not None else dist.group.WORLD
        hidden = x.shape[1]
        # worst case: every pair of every rank is routed to one rank
        capacity = self.capacity_rows or x.shape[0] * self.top_k * self.world
        cap = torch.tensor([capacity], dtype=torch.int64, device=x.device)
        dist.all_reduce(cap, op=dist.ReduceOp.MAX, group=self.group)  # ranks must agree on the shape
        capacity = int(cap.item())
        recv = symm_mem.empty((capacity, hidden), dtype=x.dtype, device=x.device)
        out = symm_mem.empty((capacity, hidden), dtype=x.dtype, device=x.device)
        recv_handle = symm_mem.rendezvous(recv, group)
        out_handle = symm_mem.rendezvous(out, group)
        self._symmetric = (recv, out, [int(p) for p in recv_handle.buffer_ptrs], [int(p) for p in out_handle.buffer_ptrs],
                           capacity, hidden, x.dtype)
        meta = symm_mem.empty(self.ops.moe_ep_meta_bytes() // 4, dtype=torch.int32, device=x.device)
        meta.zero_()
        meta_handle = symm_mem.rendezvous(meta, group)
        self._meta, self._meta_ptrs = meta, [int(p) for p in meta_handle.buffer_ptrs]
        self._handles = (recv_handle, out_handle, meta_handle)  # keep the mappings alive
        self._status = torch.zeros(2, dtype=torch.int32, device=x.device)
        torch.cuda.synchronize(x.device)
        dist.barrier(group=self.group)  # every rank's flags are zero before anybody's first step
        return self._symmetric

    def check(self) -> None:
        """Raise if a kernel of the fused exchange gave up waiting for a peer or found a receive over the buffers'
        capacity since the last check (synchronises; call it where a step's result is consumed, not inside the step)."""
        if self._status is None:
            return
        code, detail = self._status.tolist()
        if code:
            self._status.zero_()
            reason = {1: f"the count exchange timed out waiting for rank {detail}", 2: f"a rendezvous timed out waiting for rank {detail}",
                      3: f"a rank would receive {detail} rows, over the exchange capacity of {self._symmetric[4]}"}.get(code, f"code {code}")
            raise RuntimeError(f"expert-parallel exchange failed on rank {self.rank}: {reason}")

    def _dispatch_p2p(self, x: Tensor, router_logits: Tensor) -> Dispatched:
        ops = self.ops
        recv, out, recv_ptrs, _, capacity, _, _ = self._buffers(x)
        indices, weights, counts, offsets, _, pos = ops.moe_route_index(router_logits, self.top_k, want_perm=False)
        self._epoch += 1
        # counts to every rank, everybody's counts back, the plan: one kernel, nothing leaves the device.  Waiting for
        # every rank's counts also orders the ranks: a rank writes them after its previous step's last read of `out`.
        dst_base, expert_offsets, info = ops.moe_ep_exchange(counts, self._meta_ptrs, self.rank, capacity, self._epoch, self._status)
        dst_rank, dst_row = ops.moe_ep_destinations(indices, pos, offsets, dst_base, self.local_experts)
        ops.moe_permute_multi(x, dst_rank, dst_row, recv_ptrs)  # rows go straight into their owners' memory
        ops.moe_ep_barrier(self._meta_ptrs, self.rank, 1, self._epoch, self._status)  # every rank's stores have landed
        return Dispatched(recv, expert_offsets, weights, pos, [], [], None, None, dst_rank, dst_row, out, info)

    def _combine_p2p(self, expert_rows: Tensor, state: Dispatched) -> Tensor:
        _, out, _, out_ptrs, _, hidden, dtype = self._symmetric
        if expert_rows.data_ptr() != out.data_ptr():
            out[: expert_rows.shape[0]].copy_(expert_rows)  # results computed elsewhere: stage them for the peers
        self.ops.moe_ep_barrier(self._meta_ptrs, self.rank, 2, self._epoch, self._status)  # every rank's expert outputs are complete
        return self.ops.moe_unpermute_multi(out_ptrs, state.dst_rank, state.dst_row, state.weights, hidden, dtype)

    def dispatch(self, x: Tensor, router_logits: Tensor, routing: tuple[Tensor, Tensor] | None = None) -> Dispatched:
        """Route, exchange, reorder.  `routing` = (indices, weights) computed by the caller replaces the routing step
        (training calls pass weights that carry a gradient path to the logits); exchange="nccl" only."""
        if self.exchange == "p2p":
            if routing is not None:
                raise ValueError("precomputed routing is only taken by exchange='nccl'")
            return self._dispatch_p2p(x, router_logits)
        ops = self.ops
        indices, weights = routing if routing is not None else ops.moe_route(router_logits, self.top_k)
        counts, _, _, pos = ops.moe_index(indices, self.experts)
        # metadata exchange: every rank's per-expert counts
        gathered = torch.empty(self.world * self.experts, dtype=torch.int32, device=counts.device)
        dist.all_gather_into_tensor(gathered, counts.contiguous(), group=self.group)
        counts_all = gathered.view(self.world, self.experts).cpu()
        send_counts, recv_counts, seg_start, seg_len, expert_offsets = exchange_plan(counts_all, self.rank)
        # local rows in (expert, token) order = grouped by destination rank
        send = ops.moe_scatter_rows(x, pos)
        arrived = torch.empty((sum(recv_counts), x.shape[1]), dtype=x.dtype, device=x.device)
        dist.all_to_all_single(arrived, send, recv_counts, send_counts, group=self.group)
        reorder = expand_segments(seg_start, seg_len, arrived.shape[0], x.device)
        rows = ops.moe_gather(arrived, reorder)
        return Dispatched(rows, expert_offsets, weights, pos, send_counts, recv_counts, reorder, counts_all)

    def _deliver(self, send: Tensor, state: Dispatched) -> Tensor:
        """Rows in this rank's send order -> the expert owners, in (expert, source rank, token) order (exchange="nccl")."""
        arrived = torch.empty((sum(state.recv_counts), send.shape[1]), dtype=send.dtype, device=send.device)
        dist.all_to_all_single(arrived, send, state.recv_counts, state.send_counts, group=self.group)
        return self.ops.moe_gather(arrived, state.reorder)

    def _return(self, expert_rows: Tensor, state: Dispatched) -> Tensor:
        """The mirror image: expert-major rows back to the ranks they came from, in those ranks' send order."""
        total = expert_rows.shape[0]
        inverse = torch.empty(total, dtype=torch.int32, device=expert_rows.device)
        inverse[state.reorder.long()] = torch.arange(total, dtype=torch.int32, device=expert_rows.device)
        outbound = self.ops.moe_gather(expert_rows, inverse)  # back to (source rank, expert, token)
        returned = torch.empty((sum(state.send_counts), expert_rows.shape[1]), dtype=expert_rows.dtype, device=expert_rows.device)
        dist.all_to_all_single(returned, outbound, state.send_counts, state.recv_counts, group=self.group)
        return returned

    def combine(self, expert_rows: Tensor, state: Dispatched) -> Tensor:
        if self.exchange == "p2p":
            return self._combine_p2p(expert_rows, state)
        return self.ops.moe_unpermute(self._return(expert_rows, state), state.weights, state.pos)

    # -- training calls (exchange="nccl"): the two exchanges are each other's transposes ------------------------------

    def rows_with_grad(self, x: Tensor, state: Dispatched) -> Tensor:
        """`state.rows` with a gradient path back to `x` (the tokens `state` was dispatched from): the gradient rows
        travel back through the combine exchange and are summed per token with unit weights."""
        self._require_nccl()
        return _DispatchedRows.apply(x, self, state)

    def combine_with_grad(self, expert_rows: Tensor, weights: Tensor, state: Dispatched) -> Tensor:
        """combine() with gradients for the expert rows (delivered through the dispatch exchange) and the gate weights."""
        self._require_nccl()
        return _CombinedRows.apply(expert_rows, weights, self, state)

    def _require_nccl(self) -> None:
        if self.exchange != "nccl":
            raise NotImplementedError("training calls go through exchange='nccl'; the fused peer-memory exchange is inference-only")

    def momoe(self, x: Tensor, router_logits: Tensor, gate_weight: Tensor, up_weight: Tensor, down_weight: Tensor) -> Tensor:
        """The whole expert-parallel MoE layer for this rank's tokens: dispatch, the SwiGLU expert MLPs of this rank's
        experts on the tensor cores, combine (momoe of src/popcorn/kernels/momoe.py:34-53, sharded).

        gate_weight / up_weight: [local_experts, hidden, intermediate], down_weight: [local_experts, intermediate, hidden]
        — this rank's contiguous block of experts.  With exchange="p2p" the down projection writes straight into the
        symmetric buffer the peers combine from."""
        if gate_weight.shape[0] != self.local_experts:
            raise ValueError(f"expected the weights of this rank's {self.local_experts} experts, got {gate_weight.shape[0]}")
        if torch.is_grad_enabled() and any(t.requires_grad for t in (x, router_logits, gate_weight, up_weight, down_weight)):
            return self._momoe_with_grad(x, router_logits, gate_weight, up_weight, down_weight)
        state = self.dispatch(x, router_logits)
        offsets = state.expert_offsets.to(x.device, non_blocking=True)
        # only the rows inside the segments are ever read again (by the down projection, then by the combine)
        hidden_act = self.ops.moe_grouped_gemm(state.rows, gate_weight, offsets, up_weight, zero_fill=False)
        expert_rows = self.ops.moe_grouped_gemm(hidden_act, down_weight, offsets, None, state.out_rows, zero_fill=False)
        return self.combine(expert_rows, state)

    def _momoe_with_grad(self, x: Tensor, router_logits: Tensor, gate_weight: Tensor, up_weight: Tensor, down_weight: Tensor) -> Tensor:
        """The same layer for a training call: gradients for the local tokens, their router logits and this rank's expert
        weights (which collect the contributions of every rank's tokens, since the rows were exchanged).  Every rank
        must call backward: the gradient rows cross the same two exchanges in the opposite direction."""
        from popcorn_b200 import autograd as differentiable

        self._require_nccl()
        indices, weights = differentiable.moe_route(router_logits.float(), self.top_k)
        state = self.dispatch(x.detach(), router_logits.detach(), routing=(indices, weights.detach()))
        rows = self.rows_with_grad(x, state)
        offsets = state.expert_offsets.to(x.device, non_blocking=True)
        hidden_act = differentiable.moe_grouped_gemm(rows, gate_weight, offsets, up_weight)
        expert_rows = differentiable.moe_grouped_gemm(hidden_act, down_weight, offsets)
        return self.combine_with_grad(expert_rows, weights, state)


class _DispatchedRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, ep: ExpertParallel, state: Dispatched) -> Tensor:
        ctx.ep, ctx.state = ep, state
        return state.rows.view_as(state.rows)

    @staticmethod
    def backward(ctx, grad_rows: Tensor):
        ep, state = ctx.ep, ctx.state
        with torch.no_grad():
            returned = ep._return(grad_rows.contiguous(), state)
            grad_x = ep.ops.moe_unpermute(returned, torch.ones_like(state.weights), state.pos)
        return grad_x, None, None


class _CombinedRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, expert_rows: Tensor, weights: Tensor, ep: ExpertParallel, state: Dispatched) -> Tensor:
        with torch.no_grad():
            returned = ep._return(expert_rows, state)
            y = ep.ops.moe_unpermute(returned, weights, state.pos)
        ctx.ep, ctx.state = ep, state
        ctx.save_for_backward(returned, weights)
        return y

    @staticmethod
    def backward(ctx, grad_y: Tensor):
        ep, state = ctx.ep, ctx.state
        returned, weights = ctx.saved_tensors
        with torch.no_grad():
            grad_returned, grad_weights = ep.ops.moe_unpermute_backward(grad_y.contiguous(), returned, weights, state.pos)
            grad_expert_rows = ep._deliver(grad_returned, state)
        return grad_expert_rows, grad_weights, None, None
