"""CUDA kernels (through the C ABI) against the CPU oracle and the golden vectors.

Tolerances are the ones the backend is specified to: max-abs <= 2e-2 for 16-bit
inputs, <= 1e-5 for fp32 inputs, and exact equality for permutation indices,
expert counts, offsets and gathered rows.  For the element-wise ops the kernels
reproduce the reference's intermediate roundings, so beyond the max-abs bound
the tests also require that almost every element is bit-identical.
"""

import pytest
import torch

from oracle import reference_ops as oracle
from popcorn_b200 import kernels, ops, workloads
from tests.golden.golden_io import case_names, load_case

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
MAX_ABS = {torch.float32: 1e-5, torch.float16: 2e-2, torch.bfloat16: 2e-2}
BF16, F16, F32 = torch.bfloat16, torch.float16, torch.float32


def check(got, want, *, exact_fraction=0.999, what=""):
    """max-abs within the dtype's bound, and at least `exact_fraction` of elements bit-equal."""
    got = got.cpu()
    assert got.shape == want.shape and got.dtype == want.dtype, (what, got.shape, want.shape, got.dtype, want.dtype)
    if want.numel() == 0:
        return
    assert torch.isfinite(got.float()).all() or not torch.isfinite(want.float()).all(), f"{what}: non-finite output"
    diff = (got.double() - want.double()).abs()
    worst = float(diff.max())
    same = float((got == want).double().mean())
    assert worst <= MAX_ABS[want.dtype], f"{what}: max-abs {worst:.3e} exceeds {MAX_ABS[want.dtype]:.0e} ({int((diff > MAX_ABS[want.dtype]).sum())} elements)"
    # the intermediate roundings of a 16-bit dtype hide last-bit fp32 differences (another exp, another
    # summation order); in fp32 those differences are visible, so there only the max-abs bound applies
    if want.dtype != torch.float32:
        assert same >= exact_fraction, f"{what}: only {same:.6f} of elements are bit-identical"


def randn(seed, *shape, dtype=F32, scale=1.0):
    gen = torch.Generator().manual_seed(seed)
    return (scale * torch.randn(shape, generator=gen)).to(dtype)


def gpu(t):
    return None if t is None else t.to(DEV)


# ------------------------------------------------------------ golden cases --

@pytest.mark.parametrize("name", [n for n in case_names() if n.startswith("rms_norm")])
def test_golden_rms_norm(name):
    t, meta = load_case(name)
    check(ops.rms_norm(gpu(t["x"]), gpu(t["weight"]), gpu(t.get("bias")), meta["eps"]), t["y"], what=name)


@pytest.mark.parametrize("name", [n for n in case_names() if n.startswith("add_rms_norm")])
def test_golden_add_rms_norm(name):
    t, meta = load_case(name)
    y, s = ops.add_rms_norm(gpu(t["x"]), gpu(t["residual"]), gpu(t["weight"]), meta["eps"], meta["offset"])
    assert torch.equal(s.cpu(), t["s"]), f"{name}: residual stream differs"
    check(y, t["y"], what=name)


@pytest.mark.parametrize("name", [n for n in case_names() if n.startswith("rope")])
def test_golden_rotary(name):
    t, meta = load_case(name)
    y = ops.rotary_embedding(gpu(t["x"]), gpu(t["cos"]), gpu(t["sin"]), meta["interleaved"])
    assert torch.equal(y.cpu(), t["y"]), f"{name}: rotary output is not bit-identical"
    x = gpu(t["x"]).clone()
    assert ops.rotary_embedding_(x, gpu(t["cos"]), gpu(t["sin"]), meta["interleaved"]) is x
    assert torch.equal(x.cpu(), t["y"]), f"{name}: in-place rotary output is not bit-identical"


@pytest.mark.parametrize("name", [n for n in case_names() if n.startswith("pairedrope")])
def test_golden_paired_rope(name):
    t, _ = load_case(name)
    yq, yk = ops.rope(gpu(t["q"]), gpu(t["k"]), gpu(t["cos"]), gpu(t["sin"]))
    assert torch.equal(yq.cpu(), t["yq"]) and torch.equal(yk.cpu(), t["yk"]), f"{name}: paired rope is not bit-identical"


PAIRED_ROPE_CASES = [
    # batch, q_heads, k_heads, seq, head_dim, dtype, cos_batch
    (2, 32, 8, 64, 128, BF16, 1), (3, 5, 1, 33, 64, BF16, 3), (1, 4, 4, 100, 256, BF16, 1), (2, 3, 2, 9, 96, F16, 1),
    (2, 2, 1, 17, 32, F32, 2), (1, 3, 2, 7, 20, BF16, 1), (2, 2, 2, 5, 6, F32, 1), (1, 1, 1, 300, 16, BF16, 1),
]


@pytest.mark.parametrize("batch,hq,hk,seq,dim,dtype,cos_batch", PAIRED_ROPE_CASES)
def test_paired_rope_shapes(batch, hq, hk, seq, dim, dtype, cos_batch):
    q = randn(1400 + dim, batch, hq, seq, dim, dtype=dtype, scale=2.0)
    k = randn(1401 + dim, batch, hk, seq, dim, dtype=dtype, scale=2.0)
    cos = torch.cos(randn(1402, cos_batch, seq, dim)).to(dtype)  # second half NOT a copy of the first
    sin = torch.sin(randn(1403, cos_batch, seq, dim)).to(dtype)
    want_q, want_k = oracle.rope(q, k, cos, sin)
    got_q, got_k = ops.rope(gpu(q), gpu(k), gpu(cos), gpu(sin))
    assert torch.equal(got_q.cpu(), want_q) and torch.equal(got_k.cpu(), want_k)
    # (batch, seq, heads, head_dim) storage viewed as (batch, heads, seq, head_dim): strided input
    stored = gpu(q.transpose(1, 2).contiguous()).transpose(1, 2)
    got_q2, _ = ops.rope(stored, gpu(k), gpu(cos), gpu(sin))
    assert torch.equal(got_q2.cpu(), want_q)


@pytest.mark.parametrize("name", [n for n in case_names() if n.startswith("swiglu")])
def test_golden_swiglu(name):
    t, _ = load_case(name)
    g = gpu(t["gate_up"])
    cols = g.shape[1] // 2
    check(ops.swiglu(g[:, :cols], g[:, cols:]), t["y"], what=name)


@pytest.mark.parametrize("name", [n for n in case_names() if n.startswith("momoe")])
def test_golden_route_and_moe_chain(name):
    """Routing equals the reference's; route -> permute -> MLP -> unpermute reproduces momoe's output."""
    t, meta = load_case(name)
    top_k = meta["top_k"]
    logits = t["router_logits"].reshape(-1, t["router_logits"].shape[-1])
    experts = logits.shape[1]
    idx, w = ops.moe_route(gpu(logits), top_k)
    assert torch.equal(idx.cpu(), t["topk_indices"].reshape(-1, top_k))
    check(w, t["topk_weights"].reshape(-1, top_k), exact_fraction=0.0, what=name + " weights")
    x = t["x"].reshape(-1, t["x"].shape[-1])
    rows, counts, offsets, perm, pos = ops.moe_permute(gpu(x), idx, experts)
    out_rows = torch.empty_like(rows)
    for e in range(experts):
        lo, hi = int(offsets[e]), int(offsets[e + 1])
        chunk = rows[lo:hi]
        hidden_act = (chunk @ gpu(t["up_weight"][e])) * torch.nn.functional.silu(chunk @ gpu(t["gate_weight"][e]))
        out_rows[lo:hi] = hidden_act @ gpu(t["down_weight"][e])
    y = ops.moe_unpermute(out_rows, w, pos)
    torch.testing.assert_close(y.cpu().reshape(t["y"].shape), t["y"], rtol=2e-3, atol=2e-3)  # tf32-free fp32 matmuls on GPU


# ------------------------------------------------- seeded shapes vs oracle --

NORM_SHAPES = [
    # rows, cols, dtype  -- covers every (threads-per-row, items) bucket and the scalar path
    (1, 8, BF16), (3, 256, BF16), (5, 264, BF16), (9, 512, F16), (7, 1024, BF16), (4, 2048, BF16), (3, 4096, BF16),
    (2, 8192, BF16), (2, 16384, BF16), (2, 32768, BF16), (1, 65536, BF16), (1, 65544, BF16), (1, 131072, BF16),
    (1000, 128, F32), (33, 4096, F32), (6, 100, F32), (5, 33, BF16), (4, 1023, F16), (2, 12288, F32), (2, 40000, F32),
    # short rows: several rows per warp (8 and 16 lanes per row), ragged last group
    (1030, 128, BF16), (515, 64, BF16), (301, 16, F32), (77, 72, F16), (3, 24, BF16),
]


@pytest.mark.parametrize("rows,cols,dtype", NORM_SHAPES)
def test_rms_norm_shapes(rows, cols, dtype):
    x = randn(100 + cols, rows, cols, dtype=dtype)
    w = (1 + 0.1 * randn(101, cols)).to(dtype)
    b = randn(102, cols, dtype=dtype)
    for bias, eps in ((None, 1e-6), (b, 1e-5)):
        check(ops.rms_norm(gpu(x), gpu(w), gpu(bias), eps), oracle.rms_norm(x, w, bias, eps), exact_fraction=0.995, what=f"rms_norm {rows}x{cols} {dtype}")


@pytest.mark.parametrize("rows,cols,dtype", NORM_SHAPES)
def test_add_rms_norm_shapes(rows, cols, dtype):
    x = randn(200 + cols, rows, cols, dtype=dtype)
    r = randn(201 + cols, rows, cols, dtype=dtype)
    w = (1 + 0.1 * randn(202, cols)).to(dtype)
    for eps, offset in ((1e-6, 0.0), (1e-5, 1.0)):
        y, s = ops.add_rms_norm(gpu(x), gpu(r), gpu(w), eps, offset)
        want_y, want_s = oracle.add_rms_norm(x, r, w, eps, offset)
        assert torch.equal(s.cpu(), want_s)
        check(y, want_y, exact_fraction=0.995, what=f"add_rms_norm {rows}x{cols} {dtype}")


def test_norm_strided_and_batched_inputs():
    buf = randn(300, 6, 5, 512 + 64, dtype=BF16)
    x = buf[..., 32 : 32 + 512]  # leading dims collapse to one stride, rows start 64 bytes into each line
    w = (1 + 0.1 * randn(301, 512)).to(BF16)
    check(ops.rms_norm(gpu(buf)[..., 32 : 32 + 512], gpu(w)), oracle.rms_norm(x, w), exact_fraction=0.995)
    odd = buf[..., 1 : 1 + 512]  # 2-byte aligned only -> scalar kernel
    check(ops.rms_norm(gpu(buf)[..., 1 : 1 + 512], gpu(w)), oracle.rms_norm(odd, w), exact_fraction=0.995)
    y, s = ops.add_rms_norm(gpu(buf)[..., 32 : 32 + 512], gpu(buf)[..., 64 : 64 + 512], gpu(w), 1e-5, 0.0)
    want_y, want_s = oracle.add_rms_norm(x, buf[..., 64 : 64 + 512], w, 1e-5, 0.0)
    assert torch.equal(s.cpu(), want_s)
    check(y, want_y, exact_fraction=0.995)
    assert y.shape == (6, 5, 512)


def test_empty_inputs():
    w = torch.ones(64, dtype=BF16, device=DEV)
    x = torch.empty(0, 64, dtype=BF16, device=DEV)
    assert ops.rms_norm(x, w).shape == (0, 64)
    y, s = ops.add_rms_norm(x, x, w)
    assert y.shape == s.shape == (0, 64)
    assert ops.swiglu(x, x).shape == (0, 64)
    q = torch.empty(0, 4, 2, 16, dtype=BF16, device=DEV)
    cs = torch.ones(4, 8, device=DEV)
    assert ops.rotary_embedding(q, cs, cs).shape == q.shape
    idx, wts = ops.moe_route(torch.empty(0, 8, device=DEV), 2)
    assert idx.shape == wts.shape == (0, 2)
    rows, counts, offsets, perm, pos = ops.moe_permute(torch.empty(0, 64, dtype=BF16, device=DEV), idx, 8)
    assert rows.shape == (0, 64) and counts.tolist() == [0] * 8 and offsets.tolist() == [0] * 9
    assert ops.moe_unpermute(rows, wts, pos).shape == (0, 64)


SWIGLU_SHAPES = [(1, 8, BF16), (7, 136, BF16), (64, 14336, BF16), (5, 33, BF16), (3, 1000, F16), (129, 257, F32), (16, 4096, F32), (300, 16, BF16), (2, 100000, BF16)]


@pytest.mark.parametrize("rows,cols,dtype", SWIGLU_SHAPES)
def test_swiglu_shapes(rows, cols, dtype):
    gate_up = randn(400 + cols, rows, 2 * cols, dtype=dtype, scale=2.0)
    g = gpu(gate_up)
    check(ops.swiglu(g[:, :cols], g[:, cols:]), oracle.swiglu(gate_up[:, :cols], gate_up[:, cols:]), what=f"swiglu strided {rows}x{cols}")
    a, b = gate_up[:, :cols].contiguous(), gate_up[:, cols:].contiguous()
    check(ops.swiglu(gpu(a), gpu(b)), oracle.swiglu(a, b), what=f"swiglu contiguous {rows}x{cols}")


def test_swiglu_extreme_values():
    a = torch.tensor([[-200.0, -88.0, -20.0, -1e-3, -0.0, 0.0, 1e-3, 20.0, 88.0, 200.0, float("inf"), float("-inf"), 3e38, -3e38, 1e-40, 5.0]], dtype=F32)
    b = torch.tensor([[1.0, -2.0, 3.0, 1e10, 1.0, -1.0, 1e-10, 0.5, 2.0, 1.0, 1.0, 1.0, 1.0, 1.0, 1.0, float("inf")]], dtype=F32)
    for dtype in (F32, BF16, F16):
        got = ops.swiglu(gpu(a.to(dtype)), gpu(b.to(dtype))).cpu()
        want = oracle.swiglu(a.to(dtype), b.to(dtype))
        assert torch.equal(torch.isnan(got), torch.isnan(want))
        ok = ~torch.isnan(want)
        assert torch.allclose(got[ok].double(), want[ok].double(), rtol=2e-2 if dtype != F32 else 1e-6, atol=1e-30, equal_nan=True), (dtype, got, want)


ROPE_CASES = [
    # batch, seq, heads, head_dim, half, dtype, cs_dtype, interleaved
    (2, 33, 32, 128, 64, BF16, F32, False), (1, 17, 8, 128, 64, BF16, F32, False), (2, 9, 5, 64, 32, BF16, F32, False),
    (3, 7, 4, 256, 128, BF16, F32, False), (1, 9, 6, 96, 48, BF16, F32, False), (2, 5, 3, 128, 32, BF16, F32, False),
    (2, 8, 4, 64, 32, BF16, F32, True), (1, 6, 7, 96, 24, F16, F32, True), (2, 6, 2, 32, 16, F32, F32, False),
    (2, 6, 2, 32, 8, F32, F32, True), (2, 4, 2, 64, 32, F16, F16, False), (2, 4, 2, 64, 16, BF16, BF16, True),
    (1, 5, 3, 20, 5, BF16, F32, False), (1, 5, 3, 30, 7, F32, F32, True), (9, 3, 1, 16, 8, BF16, F32, False),
]


@pytest.mark.parametrize("batch,seq,heads,head_dim,half,dtype,cs_dtype,interleaved", ROPE_CASES)
def test_rotary_shapes(batch, seq, heads, head_dim, half, dtype, cs_dtype, interleaved):
    x = randn(500 + head_dim + half, batch, seq, heads, head_dim, dtype=dtype, scale=2.0)
    cos, sin = workloads.rope_tables(seq, half)
    cos, sin = cos.to(cs_dtype), sin.to(cs_dtype)
    want = oracle.rotary_embedding(x, cos, sin, interleaved)
    got = ops.rotary_embedding(gpu(x), gpu(cos), gpu(sin), interleaved)
    assert torch.equal(got.cpu(), want)
    inplace = gpu(x).clone()
    ops.rotary_embedding_(inplace, gpu(cos), gpu(sin), interleaved)
    assert torch.equal(inplace.cpu(), want)


def test_rotary_qk_views_of_a_fused_buffer():
    batch, seq, hq, hk, d = 2, 19, 8, 2, 128
    qkv = randn(600, batch, seq, hq + 2 * hk, d, dtype=BF16)
    cos, sin = workloads.rope_tables(seq, d // 2)
    want_q = oracle.rotary_embedding(qkv[:, :, :hq], cos, sin)
    want_k = oracle.rotary_embedding(qkv[:, :, hq : hq + hk], cos, sin)
    dev = gpu(qkv)
    q, k, v = dev[:, :, :hq], dev[:, :, hq : hq + hk], dev[:, :, hq + hk :]
    ops.rotary_embedding_qk_(q, k, gpu(cos), gpu(sin))
    assert torch.equal(q.cpu(), want_q) and torch.equal(k.cpu(), want_k)
    assert torch.equal(v.cpu(), qkv[:, :, hq + hk :])  # untouched neighbour
    assert torch.equal(ops.rotary_embedding(gpu(qkv)[:, :, :hq], gpu(cos), gpu(sin)).cpu(), want_q)  # strided source


ROUTE_CASES = [(64, 8, 1, F32), (100, 8, 2, F32), (257, 64, 8, F32), (64, 60, 6, F32), (50, 160, 8, F32), (40, 256, 8, F32),
               (30, 1000, 32, F32), (33, 16, 16, F32), (128, 64, 8, BF16), (128, 32, 4, F16), (7, 1, 1, F32), (9, 33, 5, F32)]


@pytest.mark.parametrize("tokens,experts,top_k,dtype", ROUTE_CASES)
def test_route(tokens, experts, top_k, dtype):
    logits = randn(700 + experts + top_k, tokens, experts, dtype=dtype)
    if dtype != F32:  # 16-bit logits collide often; keep rows whose top-(k+1) are distinct
        keep = torch.tensor([oracle.route_is_unambiguous(row[None], top_k) for row in logits])
        logits = logits[keep]
    assert oracle.route_is_unambiguous(logits, top_k)
    want_idx, want_w = oracle.moe_route(logits, top_k)
    idx, w = ops.moe_route(gpu(logits), top_k)
    assert torch.equal(idx.cpu(), want_idx)
    check(w, want_w.float(), exact_fraction=0.0, what="route weights")
    assert torch.allclose(w.sum(-1).cpu(), torch.ones(logits.shape[0]), atol=1e-6)


def test_route_ties_go_to_the_lower_expert():
    logits = torch.zeros(4, 8)
    logits[1, 5] = 1.0
    logits[2, :] = torch.tensor([0.0, 2.0, 2.0, 0.0, 2.0, 0.0, 0.0, 0.0])
    idx, w = ops.moe_route(gpu(logits), 3)
    assert idx.cpu().tolist() == [[0, 1, 2], [5, 0, 1], [1, 2, 4], [0, 1, 2]]
    assert torch.allclose(w[0].cpu(), torch.full((3,), 1 / 3))


INDEX_CASES = [(1, 1, 1), (5, 2, 8), (100, 4, 11), (257, 8, 64), (2048, 1, 3), (3000, 6, 60), (1025, 8, 1000), (4096, 2, 256), (20000, 8, 64), (700, 16, 16)]


def random_routing(seed, tokens, top_k, experts, skew=False):
    gen = torch.Generator().manual_seed(seed)
    scores = torch.rand(tokens, experts, generator=gen)
    if skew:  # most experts never chosen
        scores[:, experts // 4 :] -= 2.0
    return scores.topk(top_k, dim=1).indices.to(torch.int32)


@pytest.mark.parametrize("tokens,top_k,experts", INDEX_CASES)
def test_index_and_permute_are_bit_exact(tokens, top_k, experts):
    for skew in (False, True):
        if skew and experts // 4 < top_k:
            continue
        indices = random_routing(800 + tokens, tokens, top_k, experts, skew)
        x = randn(801 + tokens, tokens, 72, dtype=BF16)
        want_rows, want_counts, want_offsets, want_perm, want_pos = oracle.moe_permute(x, indices, experts)
        rows, counts, offsets, perm, pos = ops.moe_permute(gpu(x), gpu(indices), experts)
        assert torch.equal(counts.cpu(), want_counts)
        assert torch.equal(offsets.cpu(), want_offsets)
        assert torch.equal(perm.cpu(), want_perm)
        assert torch.equal(pos.cpu(), want_pos)
        assert torch.equal(rows.cpu(), want_rows)
        assert torch.equal(ops.moe_gather(gpu(x), perm).cpu(), want_rows)


@pytest.mark.parametrize("hidden,dtype", [(8, BF16), (72, BF16), (4096, BF16), (4100, BF16), (33, BF16), (31, F32), (256, F32), (1000, F16), (20000, BF16)])
def test_permute_gather_unpermute_widths(hidden, dtype):
    tokens, top_k, experts = 300, 4, 16
    x = randn(900 + hidden, tokens, hidden, dtype=dtype)
    logits = randn(901 + hidden, tokens, experts)
    want_idx, want_w = oracle.moe_route(logits, top_k)
    want_rows, _, _, want_perm, want_pos = oracle.moe_permute(x, want_idx, experts)
    idx, w = ops.moe_route(gpu(logits), top_k)
    rows, _, _, perm, pos = ops.moe_permute(gpu(x), idx, experts)
    assert torch.equal(rows.cpu(), want_rows) and torch.equal(pos.cpu(), want_pos)
    scaled = want_rows * torch.linspace(0.5, 1.5, want_rows.shape[0])[:, None].to(dtype)  # rows differ per slot
    want_y = oracle.moe_unpermute(scaled, want_w, want_pos)
    got_y = ops.moe_unpermute(gpu(scaled), gpu(want_w), gpu(want_pos))
    assert torch.equal(got_y.cpu(), want_y), "unpermute with the oracle's weights must be bit-identical"
    check(ops.moe_unpermute(gpu(scaled), w, pos), want_y, exact_fraction=0.99, what="unpermute with kernel-routed weights")


def test_unpermute_top1_is_the_identity():
    tokens, hidden = 500, 264
    x = randn(950, tokens, hidden, dtype=BF16)
    indices = random_routing(951, tokens, 1, 8)
    rows, _, _, _, pos = ops.moe_permute(gpu(x), gpu(indices), 8)
    ones = torch.ones(tokens, 1, device=DEV)
    assert torch.equal(ops.moe_unpermute(rows, ones, pos).cpu(), x)


def test_mirror_registry_dispatches_to_the_cuda_ops():
    x = gpu(randn(960, 16, 512, dtype=BF16))
    w = gpu((1 + 0.1 * randn(961, 512)).to(BF16))
    assert torch.equal(kernels.rms_norm(x, w, backend="b200"), ops.rms_norm(x, w))
    assert torch.equal(kernels.rms_norm(x, w), ops.rms_norm(x, w))
    with kernels.swiglu["b200"] as scoped:
        assert torch.equal(scoped(x, x), ops.swiglu(x, x))
    y, s = kernels.add_rms_norm["b200"](x, x, w, 1e-5)
    want_y, want_s = ops.add_rms_norm(x, x, w, 1e-5)
    assert torch.equal(y, want_y) and torch.equal(s, want_s)


def test_launches_are_counted_and_run_on_the_current_stream():
    from popcorn_b200 import _lib

    x = gpu(randn(970, 64, 1024, dtype=BF16))
    before = _lib.launch_count()
    side = torch.cuda.Stream(device=DEV)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        y = ops.swiglu(x, x)
    side.synchronize()
    assert _lib.launch_count() == before + 1
    assert torch.equal(y, ops.swiglu(x, x))


def test_host_tensor_pipeline_matches_the_device_op():
    from popcorn_b200 import host

    rows, cols = 3000, 1024  # not a multiple of the chunk size
    x = randn(980, rows, cols, dtype=BF16).pin_memory()
    r = randn(981, rows, cols, dtype=BF16).pin_memory()
    w = (1 + 0.1 * randn(982, cols)).to(BF16)
    y, s = host.add_rms_norm_host(x, r, w, 1e-5, 0.0, chunk_rows=512)
    want_y, want_s = ops.add_rms_norm(gpu(x), gpu(r), gpu(w), 1e-5, 0.0)
    assert not y.is_cuda and torch.equal(y, want_y.cpu()) and torch.equal(s, want_s.cpu())
    oy, os_ = oracle.add_rms_norm(x, r, w, 1e-5, 0.0)
    assert torch.equal(s, os_)
    check(y, oy, exact_fraction=0.995)
    # a second call into caller-provided buffers, one chunk larger than the input
    y2, s2 = torch.empty_like(y).pin_memory(), torch.empty_like(s).pin_memory()
    host.add_rms_norm_host(x, r, gpu(w), 1e-5, 0.0, y=y2, s=s2, chunk_rows=1 << 20)
    assert torch.equal(y2, y) and torch.equal(s2, s)


# ------------------------------------------- parameters that are not contiguous --
# Every parameter below is a strided view, so the op has to make contiguous copies of TWO operands for one
# launch; both copies must be alive (and distinct) when the kernel runs.

def strided(t):
    """The same values as `t`, stored with a gap after every element (last stride 2)."""
    wide = torch.empty(*t.shape[:-1], t.shape[-1] * 2, dtype=t.dtype, device=DEV)
    view = wide[..., ::2]
    view.copy_(t)
    assert not view.is_contiguous() or view.numel() <= 1
    return view


def test_strided_cos_and_sin():
    x = randn(2100, 2, 48, 4, 64, dtype=BF16, scale=2.0)
    cos, sin = torch.cos(randn(2101, 48, 32)), torch.sin(randn(2102, 48, 32))
    want = oracle.rotary_embedding(x, cos, sin)
    assert torch.equal(ops.rotary_embedding(gpu(x), strided(cos), strided(sin)).cpu(), want)
    q, k = gpu(x).clone(), gpu(x[:, :, :2]).clone()
    ops.rotary_embedding_qk_(q, k, strided(cos), strided(sin))
    assert torch.equal(q.cpu(), want) and torch.equal(k.cpu(), want[:, :, :2])
    # the paired op and the fused norm + rope: cos, sin (and both weights) strided at once
    qp, kp = randn(2103, 2, 4, 48, 64, dtype=BF16), randn(2104, 2, 2, 48, 64, dtype=BF16)
    cosp, sinp = torch.cos(randn(2105, 1, 48, 64)).to(BF16), torch.sin(randn(2106, 1, 48, 64)).to(BF16)
    want_q, want_k = oracle.rope(qp, kp, cosp, sinp)
    got_q, got_k = ops.rope(gpu(qp), gpu(kp), strided(cosp), strided(sinp))
    assert torch.equal(got_q.cpu(), want_q) and torch.equal(got_k.cpu(), want_k)
    wq, wk = 1 + 0.1 * randn(2107, 64), 1 + 0.1 * randn(2108, 64)
    want_q, want_k = oracle.qk_norm_rope(qp, kp, wq.to(BF16), wk.to(BF16), cosp, sinp, 1e-6)
    got_q, got_k = ops.qk_norm_rope(gpu(qp), gpu(kp), strided(wq.to(BF16)), strided(wk.to(BF16)), strided(cosp), strided(sinp), 1e-6)
    check(got_q, want_q, what="qk_norm_rope q, strided parameters")
    check(got_k, want_k, what="qk_norm_rope k, strided parameters")


@pytest.mark.parametrize("dtype", [BF16, F32])
def test_strided_weight_and_bias(dtype):
    x = randn(2110, 24, 1024, dtype=dtype)
    w, b = (1 + 0.1 * randn(2111, 1024)).to(dtype), (0.5 * randn(2112, 1024)).to(dtype)
    check(ops.rms_norm(gpu(x), strided(w), strided(b), 1e-6), oracle.rms_norm(x, w, b, 1e-6), what="rms_norm, strided weight and bias")
    check(ops.layer_norm(gpu(x), strided(w), strided(b), 1e-6), oracle.layer_norm(x, w, b, 1e-6), what="layer_norm, strided weight and bias")
    g = randn(2113, 24, 1024, dtype=dtype)
    check(ops.rms_norm_gated(gpu(x), gpu(g), strided(w), strided(b), "swish", 1e-6), oracle.rms_norm_gated(x, g, w, b, "swish", 1e-6),
          what="rms_norm_gated, strided weight and bias")


def test_gate_and_up_weights_sliced_from_one_tensor():
    experts, hidden, inter, rows_per = 4, 256, 128, 96
    both = (randn(2120, experts, hidden, 2 * inter) / hidden ** 0.5).to(BF16)
    rows = randn(2121, experts * rows_per, hidden, dtype=BF16)
    offsets = torch.arange(0, experts * rows_per + 1, rows_per, dtype=torch.int32)
    gate, up = both[..., :inter], both[..., inter:]
    want = oracle.moe_grouped_gemm(rows, gate.contiguous(), offsets, up.contiguous())
    fused = gpu(both)
    got = ops.moe_grouped_gemm(gpu(rows), fused[..., :inter], gpu(offsets), fused[..., inter:])
    excess = (got.cpu().float() - want.float()).abs() / want.float().abs().clamp(min=1.0)
    assert float(excess.max()) <= 2e-2, float(excess.max())


# ------------------------------------------------ index build against the reference's own kernel --

@pytest.mark.parametrize("name", [n for n in case_names() if n.startswith("moeindex_")])
def test_index_equals_the_references_own_kernel(name):
    """b200_moe_index against counts / cumsums / col_idx written by the reference's find_used_experts
    (src/popcorn/impls/momoe_tl.py:1126-1161) on the same routing; bit-exact."""
    import hashlib

    t, meta = load_case(name)
    if "topk_indices" in t:
        indices = gpu(t["topk_indices"])
    else:
        w = workloads.moe_bf16()
        indices, _ = ops.moe_route(gpu(w.inputs["router_logits"]), meta["top_k"])
        assert hashlib.sha256(indices.cpu().numpy().tobytes()).hexdigest() == meta["topk_indices_sha256"]
    counts, offsets, perm, pos = (r.cpu() for r in ops.moe_index(indices, meta["experts"]))
    assert torch.equal(counts, t["counts"]) and torch.equal(offsets, t["cumsums"])
    if "col_idx" in t:
        assert torch.equal(perm, t["col_idx"])
    else:
        edge = t["col_idx_head"].numel()
        assert torch.equal(perm[:edge], t["col_idx_head"]) and torch.equal(perm[-edge:], t["col_idx_tail"])
        assert hashlib.sha256(perm.numpy().tobytes()).hexdigest() == meta["col_idx_sha256"]
    # pos is the inverse map the reference does not materialise: it must invert perm
    tokens, top_k = pos.shape
    assert torch.equal(perm[pos.reshape(-1).long()], torch.arange(tokens, dtype=torch.int32).repeat_interleave(top_k))
