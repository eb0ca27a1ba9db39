"""The hot-path ops inside a CUDA graph: captured once, replayed on new input values.

The kernels are launched with cudaLaunchKernelEx on the caller's stream and allocate nothing themselves (outputs and
workspaces come from torch's caching allocator, which is capture-aware), so a launch-bound sequence of them can be
captured and replayed without the per-call host work.  Results of a replay must equal the eager results bit for bit.
"""

import pytest
import torch

from popcorn_b200 import _lib, ops
from tests.test_parity_gpu import BF16, gpu, randn

pytestmark = pytest.mark.gpu


def test_forward_path_replays_in_a_cuda_graph():
    tokens, hidden, experts, top_k, inter = 256, 512, 8, 2, 256
    x, r = gpu(randn(7000, tokens, hidden, dtype=BF16)), gpu(randn(7001, tokens, hidden, dtype=BF16))
    w = gpu((1 + 0.1 * randn(7002, hidden)).to(BF16))
    q = gpu(randn(7003, 2, 128, 4, 64, dtype=BF16))
    cos, sin = gpu(torch.cos(randn(7004, 128, 32))), gpu(torch.sin(randn(7004, 128, 32)))
    logits = gpu(randn(7005, tokens, experts))
    gate = gpu((randn(7006, experts, hidden, inter) / hidden ** 0.5).to(BF16))
    up = gpu((randn(7007, experts, hidden, inter) / hidden ** 0.5).to(BF16))
    down = gpu((randn(7008, experts, inter, hidden) / inter ** 0.5).to(BF16))

    def step():
        y, s = ops.add_rms_norm(x, r, w, 1e-5)
        rotated = ops.rotary_embedding(q, cos, sin)
        act = ops.swiglu(y[:, : hidden // 2], y[:, hidden // 2:])
        layer = ops.momoe(s.view(1, tokens, hidden), gate, up, down, logits.view(1, tokens, experts), top_k)
        return y, s, rotated, act, layer

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):  # warm-up outside the capture: library handles, function attributes, allocator pools
            step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()

    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = step()
    for seed in (7100, 7200):
        x.copy_(gpu(randn(seed, tokens, hidden, dtype=BF16)))
        logits.copy_(gpu(randn(seed + 1, tokens, experts)))
        graph.replay()
        torch.cuda.synchronize()
        replayed = [t.clone() for t in captured]
        eager = step()
        torch.cuda.synchronize()
        for name, a, b in zip(("y", "s", "rotary", "swiglu", "momoe"), replayed, eager):
            assert torch.equal(a, b), f"{name}: the graph replay differs from the eager call"
    assert _lib.wait_timeouts() == 0
