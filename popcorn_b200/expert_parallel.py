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
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch
import torch.distributed as dist
from torch import Tensor


@dataclass
class Dispatched:
    """What dispatch() hands to the expert computation, plus what combine() needs later."""

    rows: Tensor            # [received, hidden], grouped by local expert, global stable order inside
    expert_offsets: Tensor  # int32 [local_experts + 1] into rows (host tensor)
    weights: Tensor         # fp32 [local_tokens, top_k]
    pos: Tensor             # int32 [local_tokens, top_k] positions in this rank's send buffer
    send_counts: list[int]  # rows sent to each rank
    recv_counts: list[int]  # rows received from each rank
    reorder: Tensor         # int32 [received]: rows[p] = arrived[reorder[p]]
    counts_all: Tensor      # int32 [world, experts] (host tensor)


def exchange_plan(counts_all: Tensor, rank: int) -> tuple[list[int], list[int], Tensor, Tensor, Tensor]:
    """Split sizes and the reorder segments of `rank`, from the gathered counts (host arithmetic).

    counts_all: int [world, experts]; experts are owned in contiguous blocks.
    Returns (send_counts, recv_counts, segment_source_start, segment_length, expert_offsets):
    segments are listed in output order (local expert major, source rank minor); segment i covers
    arrived[segment_source_start[i] : +segment_length[i]]."""
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

    def __init__(self, experts: int, top_k: int, group: Any = None, local_ops: Any = None) -> None:
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if experts % self.world != 0:
            raise ValueError(f"experts={experts} must be a multiple of the world size {self.world}")
        self.experts, self.top_k = experts, top_k
        self.local_experts = experts // self.world
        if local_ops is None:
            from popcorn_b200 import ops as local_ops
        self.ops = local_ops

    def dispatch(self, x: Tensor, router_logits: Tensor) -> Dispatched:
        ops = self.ops
        indices, weights = ops.moe_route(router_logits, self.top_k)
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

    def combine(self, expert_rows: Tensor, state: Dispatched) -> Tensor:
        ops = self.ops
        total = expert_rows.shape[0]
        inverse = torch.empty(total, dtype=torch.int32, device=expert_rows.device)
        inverse[state.reorder.long()] = torch.arange(total, dtype=torch.int32, device=expert_rows.device)
        outbound = ops.moe_gather(expert_rows, inverse)  # back to (source rank, expert, token)
        returned = torch.empty((sum(state.send_counts), expert_rows.shape[1]), dtype=expert_rows.dtype, device=expert_rows.device)
        dist.all_to_all_single(returned, outbound, state.send_counts, state.recv_counts, group=self.group)
        return ops.moe_unpermute(returned, state.weights, state.pos)
