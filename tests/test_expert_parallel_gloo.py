"""Expert-parallel dispatch / combine over world_size-2 (and 4) gloo process groups on CPU.

The exchange logic (split sizes, all-to-all, reorder, inverse) is what is under
test; the per-rank compute steps are the CPU oracle's, injected through
`local_ops`.  The result must equal the single-process oracle bit for bit:
the concatenation of the ranks' expert-major rows is the global stable
permutation, and combine() returns what a single-process unpermute returns.
"""

import os
import socket
import types

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import reference_ops as oracle
from popcorn_b200.expert_parallel import ExpertParallel, exchange_plan, expand_segments, p2p_plan

CPU_OPS = types.SimpleNamespace(
    moe_route=oracle.moe_route, moe_index=oracle.moe_index, moe_scatter_rows=oracle.moe_scatter_rows,
    moe_gather=oracle.moe_gather, moe_unpermute=oracle.moe_unpermute,
)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs(tokens, hidden, experts, seed=11):
    gen = torch.Generator().manual_seed(seed)
    return torch.randn(tokens, hidden, generator=gen).to(torch.bfloat16), torch.randn(tokens, experts, generator=gen)


def _worker(rank, world, port, tokens, hidden, experts, top_k, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        x, logits = _inputs(tokens, hidden, experts)
        lo, hi = tokens * rank // world, tokens * (rank + 1) // world
        ep = ExpertParallel(experts, top_k, local_ops=CPU_OPS)
        state = ep.dispatch(x[lo:hi], logits[lo:hi])
        # "expert computation": scale every row by (1 + its global expert id / 8)
        scale = torch.ones(state.rows.shape[0])
        for e in range(ep.local_experts):
            a, b = int(state.expert_offsets[e]), int(state.expert_offsets[e + 1])
            scale[a:b] = 1 + (rank * ep.local_experts + e) / 8
        processed = (state.rows.float() * scale[:, None]).to(torch.bfloat16)
        y = ep.combine(processed, state)
        out[rank] = (state.rows, state.expert_offsets, y, state.send_counts, state.recv_counts)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,tokens,experts,top_k", [(2, 64, 8, 2), (2, 37, 4, 3), (4, 50, 8, 4), (2, 16, 2, 1)])
def test_dispatch_and_combine_equal_the_single_process_result(world, tokens, experts, top_k):
    hidden = 24
    manager = mp.Manager()
    out = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), tokens, hidden, experts, top_k, out), nprocs=world, join=True)

    x, logits = _inputs(tokens, hidden, experts)
    indices, weights = oracle.moe_route(logits, top_k)
    rows, counts, offsets, perm, pos = oracle.moe_permute(x, indices, experts)
    per_rank = experts // world
    for rank in range(world):
        got_rows, got_offsets, _, send_counts, recv_counts = out[rank]
        lo, hi = int(offsets[rank * per_rank]), int(offsets[(rank + 1) * per_rank])
        assert torch.equal(got_rows, rows[lo:hi]), f"rank {rank}: rows are not the global stable permutation"
        assert torch.equal(got_offsets, offsets[rank * per_rank : (rank + 1) * per_rank + 1] - lo)
        assert sum(recv_counts) == hi - lo
        assert sum(send_counts) == (tokens * (rank + 1) // world - tokens * rank // world) * top_k
    expert_of_row = torch.repeat_interleave(torch.arange(experts), counts.long())
    processed = (rows.float() * (1 + expert_of_row / 8)[:, None]).to(torch.bfloat16)
    want = oracle.moe_unpermute(processed, weights, pos)
    got = torch.cat([out[rank][2] for rank in range(world)])
    assert torch.equal(got, want)


def test_exchange_plan_small_example():
    # 2 ranks, 4 experts (2 per rank); counts_all[source, expert]
    counts_all = torch.tensor([[3, 0, 2, 1], [1, 4, 0, 2]], dtype=torch.int32)
    send, recv, start, length, offsets = exchange_plan(counts_all, rank=0)
    assert send == [3, 3] and recv == [3, 5]
    # arrived on rank 0: [src0: e0 x3, e1 x0 | src1: e0 x1, e1 x4]; output order: e0(src0, src1), e1(src0, src1)
    assert start.tolist() == [0, 3, 3, 4] and length.tolist() == [3, 1, 0, 4]
    assert offsets.tolist() == [0, 4, 8]
    assert expand_segments(start, length, 8, "cpu").tolist() == [0, 1, 2, 3, 4, 5, 6, 7]
    send, recv, start, length, offsets = exchange_plan(counts_all, rank=1)
    assert send == [5, 2] and recv == [3, 2]
    assert start.tolist() == [0, 3, 2, 3] and length.tolist() == [2, 0, 1, 2]
    assert expand_segments(start, length, 5, "cpu").tolist() == [0, 1, 2, 3, 4]
    with pytest.raises(ValueError):
        exchange_plan(torch.zeros(3, 4, dtype=torch.int32), 0)


def test_expand_segments_reorders():
    # rank 0 of 2 owns experts 0 and 1.  arrived = [src0: e0 e0 e1 | src1: e0 e1 e1]
    # -> output e0(src0 x2, src1 x1), e1(src0 x1, src1 x2)
    counts_all = torch.tensor([[2, 1, 5, 0], [1, 2, 0, 7]], dtype=torch.int32)
    _, recv, start, length, offsets = exchange_plan(counts_all, rank=0)
    assert recv == [3, 3]
    assert expand_segments(start, length, 6, "cpu").tolist() == [0, 1, 3, 2, 4, 5]
    assert offsets.tolist() == [0, 3, 6]


@pytest.mark.parametrize("world,tokens,experts,top_k", [(2, 64, 8, 2), (4, 51, 8, 3), (8, 200, 64, 8), (1, 30, 4, 2)])
def test_fused_exchange_addressing_emulated_on_cpu(world, tokens, experts, top_k):
    """All ranks' pushes, emulated in one process: every rank's buffer ends up in the global stable
    order, and pulling with the same addresses reproduces the single-process unpermute."""
    hidden = 16
    x, logits = _inputs(tokens, hidden, experts, seed=13)
    indices, weights = oracle.moe_route(logits, top_k)
    rows, counts, offsets, perm, pos = oracle.moe_permute(x, indices, experts)
    per_rank = experts // world
    bounds = [tokens * r // world for r in range(world + 1)]
    local = []
    for r in range(world):
        idx_r = indices[bounds[r] : bounds[r + 1]]
        counts_r, offsets_r, _, pos_r = oracle.moe_index(idx_r, experts)
        local.append((idx_r, counts_r, offsets_r, pos_r))
    counts_all = torch.stack([c for _, c, _, _ in local])
    buffers = [torch.full((tokens * top_k, hidden), float("nan"), dtype=torch.bfloat16) for _ in range(world)]
    addresses = []
    for r in range(world):
        idx_r, _, offsets_r, pos_r = local[r]
        dst_base, rows_per_rank, expert_offsets = p2p_plan(counts_all, r)
        dst_rank, dst_row = oracle.moe_ep_destinations(idx_r, pos_r, offsets_r, dst_base, per_rank)
        addresses.append((dst_rank, dst_row))
        xr = x[bounds[r] : bounds[r + 1]]
        for t in range(xr.shape[0]):
            for k in range(top_k):
                buffers[int(dst_rank[t, k])][int(dst_row[t, k])] = xr[t]
        lo = int(offsets[r * per_rank])
        assert torch.equal(expert_offsets, offsets[r * per_rank : (r + 1) * per_rank + 1] - lo)
        assert rows_per_rank == [int(offsets[(q + 1) * per_rank] - offsets[q * per_rank]) for q in range(world)]
    for r in range(world):
        lo, hi = int(offsets[r * per_rank]), int(offsets[(r + 1) * per_rank])
        assert torch.equal(buffers[r][: hi - lo], rows[lo:hi]), f"rank {r}: buffer is not in the global stable order"
    # pull: (rank, row) ascending is ascending expert, so the accumulation order is the oracle's
    want = oracle.moe_unpermute(rows, weights, pos)
    for r in range(world):
        dst_rank, dst_row = addresses[r]
        w_r = weights[bounds[r] : bounds[r + 1]]
        key = dst_rank.long() * (tokens * top_k) + dst_row.long()
        order = key.argsort(dim=1)
        acc = torch.zeros(dst_rank.shape[0], hidden)
        for k in range(top_k):
            sel = order[:, k]
            picked = torch.stack([buffers[int(dst_rank[t, sel[t]])][int(dst_row[t, sel[t]])] for t in range(dst_rank.shape[0])]) if dst_rank.shape[0] else torch.zeros(0, hidden)
            acc = acc + picked.float() * w_r.gather(1, sel[:, None])
        assert torch.equal(acc.to(torch.bfloat16), want[bounds[r] : bounds[r + 1]])


# ------------------------------------------------- failures, made on the host --

def test_malformed_count_tables_are_rejected_before_any_row_moves():
    good = torch.tensor([[3, 1, 0, 2], [0, 4, 1, 1]], dtype=torch.int32)
    exchange_plan(good, 0)
    p2p_plan(good, 1)
    for bad, rank in ((good[:, :3], 0),                      # experts not divisible by the world size
                      (good.clone().index_put_((torch.tensor(1), torch.tensor(2)), torch.tensor(-5, dtype=torch.int32)), 0),  # a negative count
                      (good, 2),                             # a rank outside the table
                      (good.float(), 0),                     # not integers
                      (good.view(-1), 0)):                   # not a table
        with pytest.raises(ValueError):
            exchange_plan(bad, rank)
        with pytest.raises(ValueError):
            p2p_plan(bad, rank)


def _absent_peer_worker(rank, world, port, out):
    import datetime

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    try:
        if rank == 1:
            out[rank] = "left before the step"  # between steps, nothing of its own in flight
            return
        x, logits = _inputs(32, 64, 4)
        ep = ExpertParallel(4, 2, local_ops=CPU_OPS)
        try:
            ep.dispatch(x[:16], logits[:16])
            out[rank] = "no error"
        except Exception as error:  # the count exchange cannot complete without the peer
            out[rank] = f"error: {type(error).__name__}"
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


@pytest.mark.timeout(120)
def test_a_rank_that_never_posts_its_counts_is_an_error_not_a_hang():
    """One rank leaves before the step; the other's count exchange ends with an error inside the group's timeout."""
    out = mp.Manager().dict()
    mp.spawn(_absent_peer_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    assert out[1] == "left before the step"
    assert out[0].startswith("error:"), out[0]


def _capacity_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        table = torch.tensor([[40, 0], [25, 1]], dtype=torch.int32)  # rank 0 would receive 65 rows
        _, rows_per_rank, _ = p2p_plan(table, rank)
        out[rank] = rows_per_rank
    finally:
        dist.destroy_process_group()


def test_every_rank_derives_the_same_receive_sizes():
    out = mp.Manager().dict()
    mp.spawn(_capacity_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    assert out[0] == out[1] == [65, 1]


def _cpu_unpermute_backward(grad_y, rows, weights, pos):
    """(grad_rows, grad_weights) by autograd through the oracle's combine: the CPU stand-in of the backward kernel."""
    rows_leaf, weights_leaf = rows.detach().clone().requires_grad_(), weights.detach().clone().requires_grad_()
    with torch.enable_grad():
        oracle.moe_unpermute(rows_leaf, weights_leaf, pos).backward(grad_y)
    return rows_leaf.grad, weights_leaf.grad


CPU_TRAINING_OPS = types.SimpleNamespace(**vars(CPU_OPS), moe_unpermute_backward=_cpu_unpermute_backward)


def _expert_scale(offsets, first_expert):
    scale = torch.ones(int(offsets[-1]))
    for e in range(len(offsets) - 1):
        scale[int(offsets[e]):int(offsets[e + 1])] = 1 + (first_expert + e) / 8
    return scale[:, None]


def _grad_worker(rank, world, port, tokens, hidden, experts, top_k, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        x, logits = _inputs(tokens, hidden, experts)
        grad_y, _ = _inputs(tokens, hidden, experts, seed=12)
        lo, hi = tokens * rank // world, tokens * (rank + 1) // world
        ep = ExpertParallel(experts, top_k, local_ops=CPU_TRAINING_OPS)
        mine = x[lo:hi].clone().requires_grad_()
        state = ep.dispatch(mine.detach(), logits[lo:hi])
        weights = state.weights.clone().requires_grad_()
        rows = ep.rows_with_grad(mine, state)
        processed = (rows.float() * _expert_scale(state.expert_offsets, rank * ep.local_experts)).to(torch.bfloat16)
        ep.combine_with_grad(processed, weights, state).backward(grad_y[lo:hi])
        out[rank] = (mine.grad, weights.grad)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,tokens,experts,top_k", [(2, 64, 8, 2), (2, 37, 4, 3), (4, 50, 8, 4), (2, 16, 2, 1)])
def test_gradients_cross_the_exchanges_in_reverse(world, tokens, experts, top_k):
    """rows_with_grad / combine_with_grad: each exchange's backward is the other exchange; token and gate-weight
    gradients equal autograd through the single-process chain."""
    hidden = 24
    out = mp.Manager().dict()
    mp.spawn(_grad_worker, args=(world, _free_port(), tokens, hidden, experts, top_k, out), nprocs=world, join=True)

    x, logits = _inputs(tokens, hidden, experts)
    grad_y, _ = _inputs(tokens, hidden, experts, seed=12)
    indices, weights = oracle.moe_route(logits, top_k)
    x_leaf, w_leaf = x.clone().requires_grad_(), weights.clone().requires_grad_()
    rows, _, offsets, _, pos = oracle.moe_permute(x_leaf, indices, experts)
    processed = (rows.float() * _expert_scale(offsets, 0)).to(torch.bfloat16)
    oracle.moe_unpermute(processed, w_leaf, pos).backward(grad_y)
    got_x = torch.cat([out[rank][0] for rank in range(world)])
    got_w = torch.cat([out[rank][1] for rank in range(world)])
    assert torch.equal(got_w, w_leaf.grad)
    # the distributed path sums a token's top_k gradient rows in fp32 and rounds once; torch's index_select backward
    # accumulates in bf16, which is the same number for up to two rows
    if top_k <= 2:
        assert torch.equal(got_x, x_leaf.grad)
    assert float((got_x.float() - x_leaf.grad.float()).abs().max()) <= 2e-2 * max(1.0, float(x_leaf.grad.abs().max()))


def test_training_calls_need_the_nccl_exchange():
    ep = ExpertParallel.__new__(ExpertParallel)
    ep.exchange = "p2p"
    with pytest.raises(NotImplementedError, match="inference-only"):
        ep._require_nccl()
