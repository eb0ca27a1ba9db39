"""b200_moe_index_static: the index build for callers that may not allocate.

Some hosts of this library cannot give it a workspace: a serving loop whose device
memory is laid out once at start-up and which must never call cudaMalloc again, or
a plugin boundary that passes tensors but no allocator.  For them the library
carries its own 1 MiB scratch array.  This test drives the entry point through the
C ABI exactly as such a host would (raw pointers, caller-owned outputs), twice in
a row so that the second call runs on whatever the first one left in the shared
array, and compares every output with b200_moe_index, which takes its workspace
from the caller.  The outputs are integers, so the comparison is exact.

The file name sorts last on purpose: in a run that stops at the first failure,
every other test has already been executed.
"""

import ctypes

import pytest
import torch

from popcorn_b200 import _lib, ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def routing(seed, tokens, top_k, experts):
    gen = torch.Generator().manual_seed(seed)
    return torch.rand(tokens, experts, generator=gen).topk(top_k, dim=1).indices.to(torch.int32)


def index_static(indices, experts):
    """Call the no-workspace entry point; every buffer it touches is allocated here, by the caller."""
    tokens, top_k = indices.shape
    counts = torch.full((experts,), -7, dtype=torch.int32, device=DEV)
    offsets = torch.full((experts + 1,), -7, dtype=torch.int32, device=DEV)
    perm = torch.full((tokens * top_k,), -7, dtype=torch.int32, device=DEV)
    pos = torch.full((tokens, top_k), -7, dtype=torch.int32, device=DEV)
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    stream = ctypes.c_void_p(torch.cuda.current_stream(torch.device(DEV)).cuda_stream)
    with torch.cuda.device(DEV):
        _lib.call("b200_moe_index_static", p(indices), tokens, top_k, experts, p(counts), p(offsets), p(perm), p(pos), stream)
    return counts, offsets, perm, pos


def test_static_index_matches_the_workspace_entry_point_twice_in_a_row():
    # two different problems back to back: the second finds the first one's histogram in the shared array
    for seed, tokens, top_k, experts in ((31, 20000, 8, 64), (32, 3001, 6, 60)):
        indices = routing(seed, tokens, top_k, experts).to(DEV)
        want = ops.moe_index(indices, experts)
        got = index_static(indices, experts)
        for name, g, w in zip(("counts", "offsets", "perm", "pos"), got, want):
            assert torch.equal(g, w), f"{name} differs from b200_moe_index ({tokens} tokens, {experts} experts)"
    # and the same problem again, unchanged result
    indices = routing(31, 20000, 8, 64).to(DEV)
    first = index_static(indices, 64)
    second = index_static(indices, 64)
    assert all(torch.equal(a, b) for a, b in zip(first, second))


def test_static_index_rejects_what_does_not_fit():
    limit = ctypes.c_size_t(0)
    _lib.call("b200_moe_index_static_max_bytes", ctypes.byref(limit))
    assert limit.value == 1 << 20
    experts, top_k = 1024, 8
    tokens = 2048 * 300 // top_k  # 300 blocks x 1024 experts x 4 bytes > 1 MiB
    fake = ctypes.c_void_p(4096)  # never dereferenced: the size check comes first
    with pytest.raises(_lib.B200Error) as err:
        _lib.call("b200_moe_index_static", fake, tokens, top_k, experts, fake, fake, fake, fake, ctypes.c_void_p(0))
    assert err.value.status_name == "B200_ERR_SCRATCH" and "b200_moe_index" in err.value.detail


def test_static_index_empty_input():
    counts, offsets, perm, pos = index_static(torch.empty((0, 4), dtype=torch.int32, device=DEV), 16)
    assert counts.tolist() == [0] * 16 and offsets.tolist() == [0] * 17 and perm.numel() == 0 and pos.numel() == 0
