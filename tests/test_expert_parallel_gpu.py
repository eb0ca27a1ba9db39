"""Expert-parallel dispatch / combine with the CUDA kernels and NCCL on 2 GPUs (skipped with fewer)."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import reference_ops as oracle

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs(tokens, hidden, experts):
    gen = torch.Generator().manual_seed(21)
    return torch.randn(tokens, hidden, generator=gen).to(torch.bfloat16), torch.randn(tokens, experts, generator=gen)


def _worker(rank, world, port, tokens, hidden, experts, top_k, exchange, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    device = torch.device("cuda", rank)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        from popcorn_b200.expert_parallel import ExpertParallel

        x, logits = _inputs(tokens, hidden, experts)
        lo, hi = tokens * rank // world, tokens * (rank + 1) // world
        ep = ExpertParallel(experts, top_k, exchange=exchange)
        for _ in range(2):  # the second step reuses the exchange buffers
            state = ep.dispatch(x[lo:hi].to(device), logits[lo:hi].to(device))
            # exchange="p2p" hands out its whole receive buffer; expert_offsets[-1] rows of it are in use
            rows = state.rows[: int(state.expert_offsets[-1])].clone()
            processed = (state.rows.float() * 1.5).to(torch.bfloat16)
            y = ep.combine(processed, state)
        torch.cuda.synchronize(device)
        ep.check()
        out[rank] = (rows.cpu(), state.expert_offsets.cpu(), y.cpu())
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("exchange", ["nccl", "p2p"])
def test_dispatch_and_combine_on_two_gpus(exchange):
    world, tokens, hidden, experts, top_k = 2, 4096, 1024, 16, 4
    out = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), tokens, hidden, experts, top_k, exchange, out), nprocs=world, join=True)
    x, logits = _inputs(tokens, hidden, experts)
    assert oracle.route_is_unambiguous(logits, top_k)
    indices, weights = oracle.moe_route(logits, top_k)
    rows, counts, offsets, perm, pos = oracle.moe_permute(x, indices, experts)
    per_rank = experts // world
    for rank in range(world):
        got_rows, got_offsets, _ = out[rank]
        lo, hi = int(offsets[rank * per_rank]), int(offsets[(rank + 1) * per_rank])
        assert torch.equal(got_rows, rows[lo:hi])
        assert torch.equal(got_offsets, offsets[rank * per_rank : (rank + 1) * per_rank + 1] - lo)
    want = oracle.moe_unpermute((rows.float() * 1.5).to(torch.bfloat16), weights, pos)
    got = torch.cat([out[rank][2] for rank in range(world)])
    # the kernel's routing weights differ from the oracle's in the last fp32 bit
    assert float((got.float() - want.float()).abs().max()) <= 2e-2
    assert float((got == want).float().mean()) > 0.99


def _mlp_weights(experts, hidden, inter):
    gen = torch.Generator().manual_seed(22)
    make = lambda a, b: (torch.randn(experts, a, b, generator=gen) / a ** 0.5).to(torch.bfloat16)  # noqa: E731
    return make(hidden, inter), make(hidden, inter), make(inter, hidden)


def _layer_worker(rank, world, port, tokens, hidden, inter, experts, top_k, exchange, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    device = torch.device("cuda", rank)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        from popcorn_b200.expert_parallel import ExpertParallel

        x, logits = _inputs(tokens, hidden, experts)
        gate, up, down = _mlp_weights(experts, hidden, inter)
        lo, hi = tokens * rank // world, tokens * (rank + 1) // world
        per = experts // world
        mine = slice(rank * per, (rank + 1) * per)
        ep = ExpertParallel(experts, top_k, exchange=exchange)
        for _ in range(2):
            y = ep.momoe(x[lo:hi].to(device), logits[lo:hi].to(device), gate[mine].to(device), up[mine].to(device), down[mine].to(device))
        torch.cuda.synchronize(device)
        out[rank] = y.cpu()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("exchange", ["nccl", "p2p"])
def test_whole_moe_layer_on_two_gpus(exchange):
    """dispatch -> tensor-core expert MLPs on each rank's experts -> combine equals the single-device chain."""
    world, tokens, hidden, inter, experts, top_k = 2, 2048, 512, 256, 8, 2
    out = mp.Manager().dict()
    mp.spawn(_layer_worker, args=(world, _free_port(), tokens, hidden, inter, experts, top_k, exchange, out), nprocs=world, join=True)
    x, logits = _inputs(tokens, hidden, experts)
    gate, up, down = _mlp_weights(experts, hidden, inter)
    indices, weights = oracle.moe_route(logits, top_k)
    rows, _, offsets, _, pos = oracle.moe_permute(x, indices, experts)
    hidden_act = oracle.moe_grouped_gemm(rows, gate, offsets, up)
    want = oracle.moe_unpermute(oracle.moe_grouped_gemm(hidden_act, down, offsets), weights, pos)
    got = torch.cat([out[rank] for rank in range(world)])
    assert got.shape == want.shape
    assert float((got.float() - want.float()).abs().max()) <= 2e-2
    assert float((got == want).float().mean()) > 0.97


def _training_worker(rank, world, port, tokens, hidden, inter, experts, top_k, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    device = torch.device("cuda", rank)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        from popcorn_b200.expert_parallel import ExpertParallel

        x, logits = _inputs(tokens, hidden, experts)
        grad_y, _ = _inputs(tokens, hidden, experts)
        gate, up, down = _mlp_weights(experts, hidden, inter)
        lo, hi = tokens * rank // world, tokens * (rank + 1) // world
        per = experts // world
        mine = slice(rank * per, (rank + 1) * per)
        leaves = [t.to(device).requires_grad_() for t in (x[lo:hi], logits[lo:hi], gate[mine], up[mine], down[mine])]
        ep = ExpertParallel(experts, top_k, exchange="nccl")
        y = ep.momoe(*leaves)
        y.backward(grad_y[lo:hi].flip(0).to(device))
        torch.cuda.synchronize(device)
        out[rank] = (y.detach().cpu(), *[t.grad.cpu() for t in leaves])
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_whole_moe_layer_trains_on_two_gpus():
    """Gradients of the sharded layer (tokens, router logits, each rank's expert weights) equal the single-device
    `autograd.momoe` gradients: the rows reach the experts in the same global order, so even the weight gradients,
    contracted over rows that came from both ranks, are the same sums."""
    from popcorn_b200 import autograd as differentiable

    world, tokens, hidden, inter, experts, top_k = 2, 1024, 256, 128, 8, 2
    out = mp.Manager().dict()
    mp.spawn(_training_worker, args=(world, _free_port(), tokens, hidden, inter, experts, top_k, out), nprocs=world, join=True)
    x, logits = _inputs(tokens, hidden, experts)
    grad_y, _ = _inputs(tokens, hidden, experts)
    gate, up, down = _mlp_weights(experts, hidden, inter)
    half = tokens // world
    grad_y = torch.cat([grad_y[r * half:(r + 1) * half].flip(0) for r in range(world)])
    leaves = [t.cuda().requires_grad_() for t in (x, gate, up, down, logits)]
    y = differentiable.momoe(*leaves, top_k)
    y.backward(grad_y.cuda())
    want_x, want_gate, want_up, want_down, want_logits = (t.grad.cpu() for t in leaves)
    assert torch.equal(torch.cat([out[r][0] for r in range(world)]), y.detach().cpu())
    assert torch.equal(torch.cat([out[r][1] for r in range(world)]), want_x)
    assert torch.equal(torch.cat([out[r][2] for r in range(world)]), want_logits)
    assert torch.equal(torch.cat([out[r][3] for r in range(world)]), want_gate)
    assert torch.equal(torch.cat([out[r][4] for r in range(world)]), want_up)
    assert torch.equal(torch.cat([out[r][5] for r in range(world)]), want_down)
