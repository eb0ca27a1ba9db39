"""b200_moe_route_index (routing and the index as one call) and b200_moe_index's one-launch cooperative form against
the oracle and against the three-kernel chain it replaces."""

import pytest
import torch

from oracle import reference_ops as oracle
from popcorn_b200 import ops

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def seeded_logits(tokens, experts, top_k, dtype, seed):
    """Rows without equal values: torch.topk leaves the order of ties open.  fp32 rows are normal draws (checked); 16-bit
    rows are a random order of distinct multiples of 1/8, which both 16-bit formats hold exactly."""
    gen = torch.Generator().manual_seed(seed)
    if dtype != torch.float32:
        order = torch.rand(tokens, experts, generator=gen).argsort(dim=1)
        return ((order - experts // 2).float() / 8).to(dtype)
    for _ in range(20):
        logits = torch.randn(tokens, experts, generator=gen) * 2
        if tokens == 0 or oracle.route_is_unambiguous(logits, top_k):
            return logits
    raise AssertionError("no tie-free draw")


def assert_equals_oracle(got, logits, top_k, experts, what):
    indices, weights, counts, offsets, perm, pos = (t.cpu() for t in got)
    want_indices, want_weights = oracle.moe_route(logits, top_k)
    want_counts, want_offsets, want_perm, want_pos = oracle.moe_index(want_indices, experts)
    assert torch.equal(indices, want_indices), what + ": expert indices"
    assert float((weights - want_weights.float()).abs().max()) <= 1e-6 if logits.numel() else True, what + ": weights"
    assert torch.equal(counts, want_counts) and torch.equal(offsets, want_offsets), what + ": counts / offsets"
    assert torch.equal(perm, want_perm) and torch.equal(pos, want_pos), what + ": permutation"


@pytest.mark.parametrize("tokens,experts,top_k,dtype", [
    (1, 8, 2, torch.float32), (7, 16, 4, torch.float32), (64, 64, 8, torch.float32), (65, 64, 8, torch.bfloat16),
    (1000, 32, 1, torch.float32), (4097, 64, 6, torch.float16), (9473, 48, 8, torch.float32), (65536, 64, 8, torch.float32),
    (20000, 12, 3, torch.bfloat16), (300, 64, 8, torch.float32),
    (512, 128, 8, torch.float32), (512, 64, 12, torch.float32), (300, 512, 4, torch.float32),  # the warp-per-token routing; the index chain
])
def test_route_index_equals_the_oracle_and_the_two_calls(tokens, experts, top_k, dtype):
    logits = seeded_logits(tokens, experts, top_k, dtype, seed=tokens + experts)
    got = ops.moe_route_index(logits.to(DEV), top_k)
    assert_equals_oracle(got, logits, top_k, experts, f"{tokens}x{experts} top-{top_k}")
    indices, weights = ops.moe_route(logits.to(DEV), top_k)
    separate = (indices, weights, *ops.moe_index(indices, experts))
    for one, two in zip(got, separate):
        assert torch.equal(one, two), "the results differ from moe_route + moe_index"


def test_the_token_list_is_optional():
    tokens, experts, top_k = 5000, 64, 8
    logits = seeded_logits(tokens, experts, top_k, torch.float32, seed=8).to(DEV)
    full = ops.moe_route_index(logits, top_k)
    lean = ops.moe_route_index(logits, top_k, want_perm=False)
    assert lean[4] is None
    for i in (0, 1, 2, 3, 5):
        assert torch.equal(full[i], lean[i])


def test_route_index_reads_strided_logits():
    tokens, experts, top_k = 3000, 64, 8
    wide = torch.zeros(tokens, 96)
    wide[:, :experts] = seeded_logits(tokens, experts, top_k, torch.float32, seed=5)
    got = ops.moe_route_index(wide.to(DEV)[:, :experts], top_k)
    assert_equals_oracle(got, wide[:, :experts], top_k, experts, "strided logits")


@pytest.mark.parametrize("tokens,top_k,experts", [(0, 2, 8), (1, 1, 1), (5000, 8, 64), (777, 3, 200), (65536, 8, 256), (100, 2, 1024)])
def test_index_one_launch_equals_the_three_launches(tokens, top_k, experts, monkeypatch):
    gen = torch.Generator().manual_seed(tokens + experts)
    indices = torch.randint(0, experts, (tokens, top_k), generator=gen, dtype=torch.int32)
    if tokens:
        indices[0, 0] = -1          # a pair with no expert is left out
        indices[-1, -1] = experts   # and so is one out of range
    valid = ((indices >= 0) & (indices < experts))
    one = [t.cpu() for t in ops.moe_index(indices.to(DEV), experts)]
    monkeypatch.setenv("B200_INDEX_CHAIN", "1")
    chain = [t.cpu() for t in ops.moe_index(indices.to(DEV), experts)]
    monkeypatch.delenv("B200_INDEX_CHAIN")
    names = ("counts", "offsets", "perm", "pos")
    live_rows = int(valid.sum())
    for name, a, b in zip(names, one, chain):
        if name == "perm":  # rows past the last routed pair are never written
            a, b = a[:live_rows], b[:live_rows]
        assert torch.equal(a, b), name
    counts, offsets, perm, pos = one
    assert int(offsets[-1]) == live_rows and torch.equal(counts.long(), torch.bincount(indices[valid].long(), minlength=experts))
    assert bool((pos[~valid] == -1).all())
    order = pos[valid].long()
    assert torch.equal(torch.sort(order).values, torch.arange(live_rows))
    token_of_pair = torch.arange(tokens).unsqueeze(1).expand(tokens, top_k)[valid]
    assert torch.equal(perm[:live_rows][order].long(), token_of_pair)
    # stable: inside an expert the rows keep pair order
    expert_of_row = torch.empty(live_rows, dtype=torch.long)
    expert_of_row[order] = indices[valid].long()
    assert bool((expert_of_row[1:] >= expert_of_row[:-1]).all())
    pair_of_row = torch.empty(live_rows, dtype=torch.long)
    pair_of_row[order] = torch.nonzero(valid.reshape(-1)).squeeze(1)
    same = expert_of_row[1:] == expert_of_row[:-1]
    assert bool((pair_of_row[1:][same] > pair_of_row[:-1][same]).all())


def test_one_workspace_serves_many_calls_and_a_replayed_graph():
    """The grid rendezvous keeps a generation counter in the workspace: back-to-back calls on one workspace, and a
    captured launch replayed with new inputs, must each meet afresh (a stale flag would let CTAs run ahead and rank
    their pairs against incomplete counts)."""
    import ctypes
    from popcorn_b200 import _lib
    tokens, experts, top_k = 20000, 64, 8
    need = ctypes.c_size_t(0)
    _lib.call("b200_moe_index_scratch_bytes", tokens, top_k, experts, ctypes.byref(need))
    scratch = torch.randint(0, 255, (need.value,), dtype=torch.uint8, device=DEV)  # arbitrary contents to start from
    static_logits = torch.empty(tokens, experts, device=DEV)
    out = dict(
        indices=torch.empty(tokens, top_k, dtype=torch.int32, device=DEV), weights=torch.empty(tokens, top_k, device=DEV),
        counts=torch.empty(experts, dtype=torch.int32, device=DEV), offsets=torch.empty(experts + 1, dtype=torch.int32, device=DEV),
        perm=torch.empty(tokens * top_k, dtype=torch.int32, device=DEV), pos=torch.empty(tokens, top_k, dtype=torch.int32, device=DEV))

    def call():
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        _lib.call("b200_moe_route_index", static_logits.data_ptr(), out["indices"].data_ptr(), out["weights"].data_ptr(), tokens, experts,
                  top_k, experts, _lib.F32, out["counts"].data_ptr(), out["offsets"].data_ptr(), out["perm"].data_ptr(),
                  out["pos"].data_ptr(), scratch.data_ptr(), ctypes.c_size_t(need.value), stream)

    def check(seed):
        logits = seeded_logits(tokens, experts, top_k, torch.float32, seed)
        static_logits.copy_(logits.to(DEV))
        return logits

    for seed in (1, 2, 3):
        logits = check(seed)
        call()
        assert_equals_oracle([out[k] for k in ("indices", "weights", "counts", "offsets", "perm", "pos")], logits, top_k, experts, f"call {seed}")
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        call()  # warm-up on the capture stream
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            call()
    torch.cuda.current_stream().wait_stream(side)
    for seed in (11, 12, 13):
        logits = check(seed)
        graph.replay()
        torch.cuda.synchronize()
        assert_equals_oracle([out[k] for k in ("indices", "weights", "counts", "offsets", "perm", "pos")], logits, top_k, experts, f"replay {seed}")
