"""The rotary siblings behind the same ABI: the fused qk_norm_rope and llama4_rope.

Golden vectors come from the real popcorn code (qk_norm_rope: the reference defined in its kernel-writing
notebook; llama4_rope: the registered reference), seeded shapes are compared with the CPU oracle.
llama4_rope has no reduction, so it must be bit-identical; qk_norm_rope sums squares in another order than
the CPU, so it gets the norm kernels' bar (max-abs <= 2e-2 for 16-bit inputs, <= 1e-5 for fp32, and 99.9 %
of 16-bit elements bit-identical).
"""

import pytest
import torch

from oracle import reference_ops as oracle
from popcorn_b200 import kernels, ops
from tests.golden.golden_io import case_names, load_case
from tests.test_parity_gpu import BF16, F16, F32, check, gpu, randn

pytestmark = pytest.mark.gpu


def repeated_tables(seed, cos_batch, seq, dim, dtype):
    angle = randn(seed, cos_batch, seq, dim // 2)
    return torch.cos(angle).repeat(1, 1, 2).to(dtype), torch.sin(angle).repeat(1, 1, 2).to(dtype)


@pytest.mark.parametrize("name", [n for n in case_names() if n.startswith("qknormrope")])
def test_golden_qk_norm_rope(name):
    t, meta = load_case(name)
    yq, yk = ops.qk_norm_rope(gpu(t["q"]), gpu(t["k"]), gpu(t["q_weight"]), gpu(t["k_weight"]), gpu(t["cos"]), gpu(t["sin"]), meta["eps"])
    check(yq, t["yq"], what=name + " q")
    check(yk, t["yk"], what=name + " k")


QK_NORM_ROPE_CASES = [
    # batch, q_heads, k_heads, seq, head_dim, dtype, cos_batch
    (2, 32, 8, 64, 128, BF16, 1), (3, 5, 1, 33, 64, BF16, 3), (1, 4, 4, 100, 256, BF16, 1), (2, 3, 2, 9, 96, F16, 1),
    (2, 2, 1, 17, 32, F32, 2), (1, 3, 2, 7, 20, BF16, 1), (2, 2, 2, 5, 6, F32, 1), (1, 1, 1, 300, 16, BF16, 1),
    (1, 2, 1, 40, 512, BF16, 1), (1, 2, 2, 11, 1024, F16, 1), (2, 4, 0, 16, 128, BF16, 1), (1, 6, 2, 1, 128, F32, 1),
]


@pytest.mark.parametrize("batch,hq,hk,seq,dim,dtype,cos_batch", QK_NORM_ROPE_CASES)
def test_qk_norm_rope_shapes(batch, hq, hk, seq, dim, dtype, cos_batch):
    q = randn(3400 + dim, batch, hq, seq, dim, dtype=dtype, scale=2.0)
    k = randn(3401 + dim, batch, hk, seq, dim, dtype=dtype, scale=0.5)
    qw, kw = (1 + 0.1 * randn(3402, dim)).to(dtype), (1 + 0.1 * randn(3403, dim)).to(dtype)
    cos = torch.cos(randn(3404, cos_batch, seq, dim)).to(dtype)  # second half NOT a copy of the first
    sin = torch.sin(randn(3405, cos_batch, seq, dim)).to(dtype)
    for eps in (1e-6, 1e-5):
        want_q, want_k = oracle.qk_norm_rope(q, k, qw, kw, cos, sin, eps)
        got_q, got_k = ops.qk_norm_rope(gpu(q), gpu(k), gpu(qw), gpu(kw), gpu(cos), gpu(sin), eps)
        check(got_q, want_q, what=f"qk_norm_rope q {batch}x{hq}x{seq}x{dim}")
        check(got_k, want_k, what=f"qk_norm_rope k {batch}x{hk}x{seq}x{dim}")
    # (batch, seq, heads, head_dim) storage viewed as (batch, heads, seq, head_dim): strided input
    stored = gpu(q.transpose(1, 2).contiguous()).transpose(1, 2)
    got_q2, _ = ops.qk_norm_rope(stored, gpu(k), gpu(qw), gpu(kw), gpu(cos), gpu(sin), 1e-5)
    assert torch.equal(got_q2, got_q)


def test_qk_norm_rope_equals_the_unfused_pair_of_ops():
    """Fusing changes no rounding: rope(rms_norm(q), rms_norm(k)) through the separate kernels agrees."""
    q, k = randn(3500, 2, 8, 128, 128, dtype=BF16), randn(3501, 2, 2, 128, 128, dtype=BF16)
    qw, kw = randn(3502, 128, dtype=BF16), randn(3503, 128, dtype=BF16)
    cos, sin = repeated_tables(3504, 1, 128, 128, BF16)
    fused_q, fused_k = ops.qk_norm_rope(gpu(q), gpu(k), gpu(qw), gpu(kw), gpu(cos), gpu(sin), 1e-6)
    pair_q, pair_k = ops.rope(ops.rms_norm(gpu(q), gpu(qw), None, 1e-6), ops.rms_norm(gpu(k), gpu(kw), None, 1e-6), gpu(cos), gpu(sin))
    assert float((fused_q == pair_q).double().mean()) > 0.999 and float((fused_k == pair_k).double().mean()) > 0.999
    # relative bound: the weights here are N(0,1), so outputs reach beyond the range where 2e-2 is one 16-bit step
    for fused, pair in ((fused_q, pair_q), (fused_k, pair_k)):
        assert float(((fused.float() - pair.float()).abs() / (pair.float().abs() + 1)).max()) <= 2 ** -7


@pytest.mark.parametrize("name", [n for n in case_names() if n.startswith("llama4rope")])
def test_golden_llama4_rope(name):
    t, _ = load_case(name)
    yq, yk = ops.llama4_rope(gpu(t["q"]), gpu(t["k"]), gpu(t["freqs"]))
    assert torch.equal(yq.cpu(), t["yq"]) and torch.equal(yk.cpu(), t["yk"]), f"{name}: llama4 rope is not bit-identical"


LLAMA4_CASES = [
    # batch, seq, q_heads, k_heads, head_dim, dtype
    (2, 64, 32, 8, 128, BF16), (3, 33, 5, 1, 64, BF16), (1, 100, 4, 4, 256, BF16), (2, 9, 3, 2, 96, F16),
    (2, 17, 2, 1, 32, F32), (1, 7, 3, 2, 20, BF16), (2, 5, 2, 2, 6, F32), (1, 300, 1, 1, 16, BF16), (9, 40, 9, 3, 128, BF16),
    (1, 3, 2, 1, 4096, BF16), (2, 16, 4, 0, 128, F16),
]


@pytest.mark.parametrize("batch,seq,hq,hk,dim,dtype", LLAMA4_CASES)
def test_llama4_rope_shapes(batch, seq, hq, hk, dim, dtype):
    q = randn(3600 + dim, batch, seq, hq, dim, dtype=dtype, scale=2.0)
    k = randn(3601 + dim, batch, seq, hk, dim, dtype=dtype, scale=2.0)
    angle = randn(3602, seq, dim // 2)
    freqs = torch.stack((angle.cos(), angle.sin()), -1).to(dtype)
    want_q, want_k = oracle.llama4_rope(q, k, freqs)
    got_q, got_k = ops.llama4_rope(gpu(q), gpu(k), gpu(freqs))
    assert torch.equal(got_q.cpu(), want_q) and torch.equal(got_k.cpu(), want_k)
    # q and k as views into one fused qkv buffer: strided heads
    if hk > 0:
        qkv = gpu(torch.cat((q, k, k), dim=2))
        got_q2, got_k2 = ops.llama4_rope(qkv[:, :, :hq], qkv[:, :, hq:hq + hk], gpu(freqs))
        assert torch.equal(got_q2.cpu(), want_q) and torch.equal(got_k2.cpu(), want_k)


def test_rope_family_through_the_registry_and_errors():
    q, k = randn(3700, 1, 4, 2, 64, dtype=BF16), randn(3701, 1, 4, 1, 64, dtype=BF16)
    angle = randn(3702, 4, 32)
    freqs = torch.stack((angle.cos(), angle.sin()), -1).to(BF16)
    got = kernels.llama4_rope(gpu(q), gpu(k), gpu(freqs), backend="b200")
    assert torch.equal(got[0].cpu(), oracle.llama4_rope(q, k, freqs)[0])
    qh, kh = q.transpose(1, 2).contiguous(), k.transpose(1, 2).contiguous()
    w = randn(3703, 64, dtype=BF16)
    cos, sin = repeated_tables(3704, 1, 4, 64, BF16)
    got = kernels.qk_norm_rope(gpu(qh), gpu(kh), gpu(w), gpu(w), gpu(cos), gpu(sin), backend="b200")
    check(got[0], oracle.qk_norm_rope(qh, kh, w, w, cos, sin)[0], what="registry qk_norm_rope")
    with pytest.raises(ValueError):
        ops.llama4_rope(gpu(q), gpu(k), gpu(freqs[:3]))
    with pytest.raises(TypeError):
        ops.llama4_rope(gpu(q), gpu(k), gpu(freqs.float()))
    with pytest.raises(ValueError):
        ops.qk_norm_rope(gpu(qh), gpu(kh), gpu(w[:32]), gpu(w), gpu(cos), gpu(sin))
    with pytest.raises(ValueError):
        ops.qk_norm_rope(gpu(qh), gpu(kh), gpu(w), gpu(w), gpu(cos[:, :2]), gpu(sin[:, :2]))
    empty_q, empty_k = ops.llama4_rope(gpu(q[:0]), gpu(k[:0]), gpu(freqs))
    assert empty_q.shape == q[:0].shape and empty_k.shape == k[:0].shape
