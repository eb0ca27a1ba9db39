"""The gradients of the grouped expert GEMM (same tcgen05 kernel, other operand layouts) and trainable momoe.

dgrad reads the weights along their rows (K-major B operand), wgrad contracts over each expert's rows (MN-major A
operand, the last K slice of a segment padded with zeros by the tensor map).  Bounds as for the forward GEMM:
products exact, fp32 sums in another order than the CPU's, one rounding, so |diff| <= 2e-2 * max(1, |y|) for bf16
(2e-3 for fp16) with nearly all elements bit-identical.  Whole-layer gradients are compared with autograd through
the registered reference's formula evaluated in fp64 on the routed pairs.
"""

import pytest
import torch
import torch.nn.functional as F

from oracle import reference_ops as oracle
from popcorn_b200 import _lib, autograd, kernels, ops
from tests.test_grouped_gemm_gpu import CASES, close, make
from tests.test_parity_gpu import BF16, F16, gpu, randn

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("counts,k,n,dtype", CASES)
def test_gate_up_stores_both_projections(counts, k, n, dtype):
    rows, gate, up, offsets = make(counts, k, n, dtype, 5300 + k, pad=2)
    got = ops.moe_grouped_gemm_gate_up(gpu(rows), gpu(gate), gpu(up), gpu(offsets))
    close(got, oracle.moe_grouped_gemm_gate_up(rows, gate, up, offsets), f"gate|up {counts} k={k} n={n}")
    assert _lib.wait_timeouts() == 0


@pytest.mark.parametrize("counts,k,n,dtype", CASES)
def test_dgrad(counts, k, n, dtype):
    _, gate, up, offsets = make(counts, k, n, dtype, 5400 + k, pad=3)
    total = int(offsets[-1]) + 3
    grad, grad2 = randn(5401 + n, total, n, dtype=dtype), randn(5402 + n, total, n, dtype=dtype)
    got = ops.moe_grouped_gemm_dgrad(gpu(grad), gpu(gate), gpu(offsets))
    # |grad_rows| ~ sqrt(n / k): scale the comparison like the forward's O(1) outputs
    close(got, oracle.moe_grouped_gemm_dgrad(grad, gate, offsets), f"dgrad {counts} k={k} n={n}")
    assert not got[int(offsets[-1]):].any(), "rows outside every segment must stay zero"
    got = ops.moe_grouped_gemm_dgrad(gpu(grad), gpu(gate), gpu(offsets), gpu(grad2), gpu(up))
    close(got, oracle.moe_grouped_gemm_dgrad(grad, gate, offsets, grad2, up), f"dgrad, two branches {counts} k={k} n={n}")
    # the two gradients as column halves of one buffer (shared row stride)
    both = gpu(torch.cat((grad, grad2), dim=1))
    got2 = ops.moe_grouped_gemm_dgrad(both[:, :n], gpu(gate), gpu(offsets), both[:, n:], gpu(up))
    assert torch.equal(got2, got)
    assert _lib.wait_timeouts() == 0


WGRAD_CASES = CASES + [
    ([64, 64], 128, 256, BF16), ([1, 2, 3, 4, 5, 6, 7], 64, 64, BF16), ([127, 129, 63, 65, 191], 256, 256, BF16),
    ([2000, 0, 1], 136, 520, BF16), ([0, 0, 0], 64, 64, BF16), ([300] * 9, 384, 128, F16),
]


@pytest.mark.parametrize("counts,k,n,dtype", WGRAD_CASES)
def test_wgrad(counts, k, n, dtype):
    rows, _, _, offsets = make(counts, k, n, dtype, 5500 + k, pad=5)
    total = int(offsets[-1]) + 5
    # O(1) results: the contraction runs over up to thousands of rows
    grad = (randn(5501 + n, total, n, dtype=dtype) / max(counts + [1]) ** 0.5).to(dtype)
    got = ops.moe_grouped_gemm_wgrad(gpu(rows), gpu(grad), gpu(offsets))
    close(got, oracle.moe_grouped_gemm_wgrad(rows, grad, offsets), f"wgrad {counts} k={k} n={n}")
    assert _lib.wait_timeouts() == 0


def test_wgrad_ignores_rows_of_other_experts_even_when_they_are_not_finite():
    """The padding of a segment's last K slice comes from the tensor map's zero fill, never from the neighbour's rows."""
    counts = [70, 3, 129]
    rows, _, _, offsets = make(counts, 128, 256, BF16, 5600)
    grad = (randn(5601, rows.shape[0], 256, dtype=BF16) / 8).to(BF16)
    want = oracle.moe_grouped_gemm_wgrad(rows, grad, offsets)
    poisoned_rows, poisoned_grad = rows.clone(), grad.clone()
    poisoned_rows[70:73] = float("nan")
    poisoned_grad[70:73] = float("inf")
    got = ops.moe_grouped_gemm_wgrad(gpu(poisoned_rows), gpu(poisoned_grad), gpu(offsets)).cpu()
    close(got[0], want[0], "expert before the poisoned one")
    close(got[2], want[2], "expert after the poisoned one")
    assert not torch.isfinite(got[1].float()).any()
    # segments that leave rows unused at both ends and in the middle
    sparse = torch.tensor([2, 60, 60, 70], dtype=torch.int32)  # rows 70.. (the poisoned ones first) belong to nobody
    got = ops.moe_grouped_gemm_wgrad(gpu(poisoned_rows), gpu(poisoned_grad), gpu(sparse)).cpu()
    close(got, oracle.moe_grouped_gemm_wgrad(rows, grad, sparse), "segments around the poisoned rows", exact_fraction=0.97)


def test_backward_gemms_at_scale_against_torch():
    """Segments of thousands of rows, many tiles per CTA: compared with torch matmul per expert on the GPU."""
    counts = [2048, 1500, 0, 2600, 1900]
    rows, gate, up, offsets = make(counts, 1024, 768, BF16, 5700)
    grad = (randn(5701, rows.shape[0], 768, dtype=BF16) / 32).to(BF16)
    r, g, w, o = gpu(rows), gpu(grad), gpu(gate), gpu(offsets)
    dgrad, wgrad = ops.moe_grouped_gemm_dgrad(g, w, o), ops.moe_grouped_gemm_wgrad(r, g, o)
    bounds = offsets.tolist()
    for e in range(len(counts)):
        lo, hi = bounds[e], bounds[e + 1]
        want_d = (g[lo:hi].float() @ w[e].float().t()).to(BF16)
        want_w = (r[lo:hi].float().t() @ g[lo:hi].float()).to(BF16)
        close(dgrad[lo:hi], want_d.cpu(), f"dgrad expert {e}", exact_fraction=0.97)
        close(wgrad[e], want_w.cpu(), f"wgrad expert {e}", exact_fraction=0.97)
    assert _lib.wait_timeouts() == 0


def reference_layer(x, gate, up, down, logits, top_k, wide):
    """The registered reference's formula (src/popcorn/kernels/momoe.py:47-53) with `wide` as its upcast type."""
    probs = logits.to(wide).softmax(-1)
    picked, idx = probs.topk(top_k, dim=-1)
    dense = torch.zeros_like(probs).scatter(-1, idx, picked / picked.sum(-1, keepdim=True))
    x_wide = x.to(wide)
    hidden = torch.einsum("td,edh->teh", x_wide, up.to(wide)) * F.silu(torch.einsum("td,edh->teh", x_wide, gate.to(wide)))
    return torch.einsum("ted,te->td", torch.einsum("teh,ehd->ted", hidden, down.to(wide)), dense).to(x.dtype)


@pytest.mark.parametrize("tokens,hidden,inter,experts,top_k,dtype", [(96, 128, 256, 8, 2, BF16), (200, 64, 136, 4, 3, BF16), (64, 256, 128, 16, 4, F16)])
def test_momoe_trains(tokens, hidden, inter, experts, top_k, dtype):
    x = randn(5800, tokens, hidden, dtype=dtype)
    gate = (randn(5801, experts, hidden, inter) / hidden ** 0.5).to(dtype)
    up = (randn(5802, experts, hidden, inter) / hidden ** 0.5).to(dtype)
    down = (randn(5803, experts, inter, hidden) / inter ** 0.5).to(dtype)
    logits = randn(5804, tokens, experts)
    grad_y = randn(5805, tokens, hidden, dtype=dtype)

    exact = [t.double().requires_grad_() for t in (x, gate, up, down, logits)]
    reference_layer(*exact, top_k, torch.float64).backward(grad_y.double())
    half = [t.clone().requires_grad_() for t in (x, gate, up, down, logits)]  # the reference as registered: fp32 inside, 16-bit gradients
    reference_layer(*half, top_k, torch.float32).backward(grad_y)

    ours = [gpu(t).requires_grad_() for t in (x, gate, up, down, logits)]
    y = kernels.momoe(*ours, top_k, backend="b200")
    y.backward(gpu(grad_y))
    for name, mine, ref64, ref16 in zip(("x", "gate_weight", "up_weight", "down_weight", "router_logits"), ours, exact, half):
        assert mine.grad is not None and mine.grad.dtype == mine.dtype, name
        scale = float(ref64.grad.abs().max())
        err = float((mine.grad.cpu().double() - ref64.grad).abs().max()) / scale
        ref_err = float((ref16.grad.double() - ref64.grad).abs().max()) / scale
        # popcorn grades a gradient against fp64 with the reference's own error as the budget (bench/compare.py:243-277)
        # 16-bit intermediates (hidden activations, expert outputs) bound every gradient, the fp32 router logits' too
        assert err <= max(2.0 * ref_err, 2e-2), f"grad {name}: {err:.3e} vs the reference's {ref_err:.3e}"
    assert _lib.wait_timeouts() == 0


def test_grouped_gemm_trains_through_the_registry():
    rows, gate, up, offsets = make([40, 0, 90], 64, 128, BF16, 5900)
    grad = randn(5901, rows.shape[0], 128, dtype=BF16)
    r, w, u = gpu(rows).requires_grad_(), gpu(gate).requires_grad_(), gpu(up).requires_grad_()
    kernels.moe_grouped_gemm(r, w, gpu(offsets), backend="b200").backward(gpu(grad))
    close(r.grad, oracle.moe_grouped_gemm_dgrad(grad, gate, offsets), "registry dgrad")
    close(w.grad, oracle.moe_grouped_gemm_wgrad(rows, grad, offsets), "registry wgrad")
    r.grad = w.grad = None
    out = autograd.moe_grouped_gemm(r, w, gpu(offsets), u)
    out.backward(gpu(grad))
    both = oracle.moe_grouped_gemm_gate_up(rows, gate, up, offsets)
    a, b = both[:, :128].clone().requires_grad_(), both[:, 128:].clone().requires_grad_()
    (F.silu(a) * b).backward(grad)
    want_rows = oracle.moe_grouped_gemm_dgrad(a.grad, gate, offsets, b.grad, up)
    assert float((r.grad.cpu().float() - want_rows.float()).abs().max()) <= 2e-2 * max(1.0, float(want_rows.abs().max()))
    assert float((u.grad.cpu().float() - oracle.moe_grouped_gemm_wgrad(rows, b.grad, offsets).float()).abs().max()) <= 6e-2


def test_backward_gemm_errors():
    rows, gate, up, offsets = make([16], 64, 64, BF16, 6000)
    with pytest.raises(ValueError):
        ops.moe_grouped_gemm_dgrad(gpu(rows), gpu(gate), gpu(offsets), gpu(rows))  # second gradient without its weight
    with pytest.raises(TypeError):
        ops.moe_grouped_gemm_wgrad(gpu(rows.float()), gpu(rows.float()), gpu(offsets))
    with pytest.raises(ValueError):
        ops.moe_grouped_gemm_wgrad(gpu(rows), gpu(rows[:8]), gpu(offsets))
    empty = ops.moe_grouped_gemm_wgrad(gpu(rows[:0]), gpu(rows[:0]), gpu(torch.zeros(3, dtype=torch.int32)))
    assert empty.shape == (2, 64, 64) and not empty.any()
