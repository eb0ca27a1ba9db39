"""The kernels of the fused expert-parallel exchange on ONE GPU: the ranks are emulated one after the other.

A rank's exchange kernel publishes its counts and flags before it waits, so a first pass with a budget of a few
microseconds leaves every rank's counts and flags in every (emulated) rank's meta buffer — each of those kernels
gives up its wait, which is the bounded-wait path under test — and a second pass finds all flags set and computes the
plans.  No kernel ever needs another kernel to run at the same time.  The multi-GPU form of the same checks is
tests/test_expert_parallel_gpu.py.
"""

import pytest
import torch

from oracle import reference_ops as oracle
from popcorn_b200 import ops
from popcorn_b200.expert_parallel import p2p_plan

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
SHORT = 20_000  # ns: a wait nobody answers gives up after this


def make_meta(world):
    words = ops.moe_ep_meta_bytes() // 4
    metas = [torch.zeros(words, dtype=torch.int32, device=DEV) for _ in range(world)]
    return metas, [m.data_ptr() for m in metas]


def publish_then_plan(counts, ptrs, capacity, epoch):
    """Pass 1 publishes (and times out), pass 2 plans; returns per-rank (dst_base, expert_offsets, info) and the statuses of pass 1."""
    world = len(counts)
    first = []
    for rank in range(world):
        status = torch.zeros(2, dtype=torch.int32, device=DEV)
        dst_base, _, _ = ops.moe_ep_exchange(counts[rank], ptrs, rank, capacity, epoch, status, budget_ns=SHORT)
        first.append((status.tolist(), dst_base.cpu()))
    plans = []
    for rank in range(world):
        status = torch.zeros(2, dtype=torch.int32, device=DEV)
        plan = ops.moe_ep_exchange(counts[rank], ptrs, rank, capacity, epoch, status, budget_ns=SHORT)
        assert status.tolist() == [0, 0], f"rank {rank}: {status.tolist()}"
        plans.append(plan)
    return plans, first


@pytest.mark.parametrize("world,experts", [(2, 16), (4, 64), (8, 64), (1, 8), (8, 1024)])
def test_exchange_plan_equals_the_host_plan_and_waits_are_bounded(world, experts):
    gen = torch.Generator().manual_seed(world * 1000 + experts)
    counts_all = torch.randint(0, 500, (world, experts), generator=gen, dtype=torch.int32)
    counts_all[0, 0] = 0  # an expert nobody on rank 0 picked
    _, ptrs = metas = make_meta(world)
    counts = [counts_all[r].to(DEV) for r in range(world)]
    plans, first = publish_then_plan(counts, ptrs, capacity=10**9, epoch=1)
    for rank, (status, dst_base) in enumerate(first):
        if rank < world - 1:  # somebody had not published yet: the wait ran out and says for whom
            assert status[0] == 1 and rank < status[1] < world, status
            assert bool((dst_base < 0).all()), "a failed exchange must make every destination negative"
        else:                 # the last rank finds everybody's counts
            assert status == [0, 0]
    for rank in range(world):
        dst_base, expert_offsets, info = (t.cpu() for t in plans[rank])
        want_base, rows_per_rank, want_offsets = p2p_plan(counts_all, rank)
        assert torch.equal(dst_base, want_base) and torch.equal(expert_offsets, want_offsets)
        per = experts // world
        sent_away = int(counts_all[rank].sum()) - int(counts_all[rank, rank * per:(rank + 1) * per].sum())
        assert info.tolist() == [rows_per_rank[rank], sent_away, max(rows_per_rank), world]
    del metas


def test_exchange_reports_a_receive_over_capacity():
    world, experts = 2, 8
    counts_all = torch.full((world, experts), 100, dtype=torch.int32)
    _, ptrs = metas = make_meta(world)
    counts = [counts_all[r].to(DEV) for r in range(world)]
    for rank in range(world):  # publish
        ops.moe_ep_exchange(counts[rank], ptrs, rank, 10**9, 1, torch.zeros(2, dtype=torch.int32, device=DEV), budget_ns=SHORT)
    status = torch.zeros(2, dtype=torch.int32, device=DEV)
    dst_base, expert_offsets, info = ops.moe_ep_exchange(counts[0], ptrs, 0, 799, 1, status, budget_ns=SHORT)  # each rank receives 800
    assert status.tolist() == [3, 800]
    assert bool((dst_base < 0).all()) and not bool(expert_offsets.any()) and info.tolist()[0] == 0
    del metas


def test_barrier_times_out_without_peers_and_passes_with_them():
    world = 4
    _, ptrs = metas = make_meta(world)
    statuses = []
    for rank in range(world):  # nobody else has arrived when rank 0 .. 2 wait; rank 3 finds everybody
        status = torch.zeros(2, dtype=torch.int32, device=DEV)
        ops.moe_ep_barrier(ptrs, rank, 1, 7, status, budget_ns=SHORT)
        statuses.append(status.tolist())
    assert [s[0] for s in statuses] == [2, 2, 2, 0] and all(rank < s[1] < world for rank, s in enumerate(statuses[:3]))
    for rank in range(world):  # everybody has arrived at epoch 7 now
        status = torch.zeros(2, dtype=torch.int32, device=DEV)
        ops.moe_ep_barrier(ptrs, rank, 1, 7, status, budget_ns=SHORT)
        assert status.tolist() == [0, 0]
    status = torch.zeros(2, dtype=torch.int32, device=DEV)  # a later epoch, another channel: nobody there yet
    ops.moe_ep_barrier(ptrs, 0, 2, 7, status, budget_ns=SHORT)
    assert status.tolist()[0] == 2
    with pytest.raises(Exception, match="channel"):
        ops.moe_ep_barrier(ptrs, 0, 0, 8, status)
    del metas


@pytest.mark.parametrize("world", [2, 4])
def test_emulated_ranks_dispatch_and_combine_like_one_gpu(world):
    """route -> index -> exchange (device plan) -> destinations -> permute into the owners' buffers, then the combine
    straight out of them: the buffers hold the single-GPU expert-major rows, and every token's result is bit-equal to
    the single-GPU chain."""
    tokens, hidden, experts, top_k = 1024, 512, 16, 4
    gen = torch.Generator().manual_seed(90 + world)
    x = torch.randn(tokens, hidden, generator=gen).to(torch.bfloat16)
    logits = torch.randn(tokens, experts, generator=gen)
    assert oracle.route_is_unambiguous(logits, top_k)
    per_tokens, per_experts = tokens // world, experts // world
    capacity = per_tokens * top_k * world
    recv = [torch.zeros(capacity, hidden, dtype=torch.bfloat16, device=DEV) for _ in range(world)]
    recv_ptrs = [b.data_ptr() for b in recv]
    _, ptrs = metas = make_meta(world)
    local = []
    for rank in range(world):
        xs, ls = x[rank * per_tokens:(rank + 1) * per_tokens].to(DEV), logits[rank * per_tokens:(rank + 1) * per_tokens].to(DEV)
        indices, weights = ops.moe_route(ls, top_k)
        counts, offsets, _, pos = ops.moe_index(indices, experts)
        local.append((xs, indices, weights, counts, offsets, pos))
    plans, _ = publish_then_plan([l[3] for l in local], ptrs, capacity, epoch=1)
    where = []
    for rank in range(world):
        xs, indices, _, _, offsets, pos = local[rank]
        dst_rank, dst_row = ops.moe_ep_destinations(indices, pos, offsets, plans[rank][0], per_experts)
        ops.moe_permute_multi(xs, dst_rank, dst_row, recv_ptrs)
        where.append((dst_rank, dst_row))
    want_indices, want_weights = oracle.moe_route(logits, top_k)
    rows, _, offsets, _, pos = oracle.moe_permute(x, want_indices, experts)
    for rank in range(world):
        lo, hi = int(offsets[rank * per_experts]), int(offsets[(rank + 1) * per_experts])
        expert_offsets, info = plans[rank][1].cpu(), plans[rank][2].cpu()
        assert int(info[0]) == hi - lo and torch.equal(expert_offsets, offsets[rank * per_experts:(rank + 1) * per_experts + 1] - lo)
        assert torch.equal(recv[rank][: hi - lo].cpu(), rows[lo:hi]), f"rank {rank}: received rows are not the single-GPU rows"
    single = ops.moe_unpermute(rows.to(DEV), ops.moe_route(logits.to(DEV), top_k)[1], pos.to(DEV)).cpu()
    for rank in range(world):
        y = ops.moe_unpermute_multi(recv_ptrs, where[rank][0], where[rank][1], local[rank][2], hidden, torch.bfloat16)
        assert torch.equal(y.cpu(), single[rank * per_tokens:(rank + 1) * per_tokens])
    del metas
