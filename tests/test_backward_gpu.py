"""Backward kernels against autograd of the CPU oracle (which is autograd of the reference's own code).

Gradients are graded the way popcorn's harness grades them (src/popcorn/bench/compare.py:243-277,
src/popcorn/bench/model.py:66-71): error against an fp64 evaluation, accepted when it is within
max(2 x the error of the native-precision reference, floor x scale), floors fp32 2e-5, fp16 1e-3,
bf16 2e-2.  For the 16-bit dtypes the kernels follow autograd's intermediate roundings, so almost
every element must also be bit-identical to the native-precision oracle.
"""

import pytest
import torch

from oracle import reference_ops as oracle
from popcorn_b200 import autograd as diff, kernels, workloads
from tests.golden.golden_io import case_names, load_case

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
FLOOR = {torch.float32: 2e-5, torch.float16: 1e-3, torch.bfloat16: 2e-2}
NORM_BWD_SHAPES = [(5, 64, torch.float32), (33, 256, torch.bfloat16), (12, 1032, torch.bfloat16), (70, 1544, torch.float32), (64, 1024, torch.bfloat16), (40, 4096, torch.bfloat16), (300, 8192, torch.bfloat16),
                   (7, 16384, torch.bfloat16), (9, 100, torch.float32), (6, 33, torch.bfloat16), (3, 40000, torch.float32), (130, 2048, torch.float16), (600, 512, torch.float32),
                   (40, 3072, torch.bfloat16), (20, 5120, torch.bfloat16), (11, 6144, torch.float16)]


def randn(seed, *shape, dtype=torch.float32, scale=1.0):
    gen = torch.Generator().manual_seed(seed)
    return (scale * torch.randn(shape, generator=gen)).to(dtype)


def grade(mine, native, truth, dtype, what, exact_fraction=None):
    mine = mine.cpu()
    err = float((mine.double() - truth).abs().max())
    budget = float((native.double() - truth).abs().max())
    scale = max(1.0, float(truth.abs().max()))
    assert err <= max(2 * budget, FLOOR[dtype] * scale), f"{what}: err {err:.3e} > max(2*{budget:.3e}, {FLOOR[dtype]:.0e}*{scale:.1f})"
    if exact_fraction is not None:
        same = float((mine == native).double().mean())
        assert same >= exact_fraction, f"{what}: only {same:.5f} bit-identical to the native-precision oracle"


def oracle_grads(fn, inputs, grad_out, wide=False):
    leaves = [t.double().requires_grad_(True) if wide else t.clone().requires_grad_(True) for t in inputs]
    out = fn(*leaves)
    return torch.autograd.grad(out, leaves, grad_out.double() if wide else grad_out)


@pytest.mark.parametrize("rows,cols,dtype", [(7, 136, torch.bfloat16), (64, 14336, torch.bfloat16), (5, 33, torch.bfloat16),
                                              (33, 1000, torch.float16), (129, 257, torch.float32), (16, 4096, torch.float32)])
def test_swiglu_backward(rows, cols, dtype):
    gate_up = randn(1100 + cols, rows, 2 * cols, dtype=dtype, scale=2.0)
    g = randn(1101 + cols, rows, cols, dtype=dtype)
    a, b = gate_up[:, :cols], gate_up[:, cols:]
    dev = gate_up.to(DEV).requires_grad_(True)
    out = diff.swiglu(dev[:, :cols], dev[:, cols:])
    (grad,) = torch.autograd.grad(out, dev, g.to(DEV))
    native = oracle_grads(oracle.swiglu, (a, b), g)
    truth = oracle_grads(oracle.swiglu, (a, b), g, wide=True)
    exact = 0.999 if dtype != torch.float32 else None
    grade(grad[:, :cols], native[0], truth[0], dtype, "grad_a", exact)
    grade(grad[:, cols:], native[1], truth[1], dtype, "grad_b", exact)


def test_swiglu_backward_full_config_sample():
    w = workloads.swiglu_bf16(scale=1 / 16)
    gate_up, cols = w.inputs["gate_up"], w.args["cols"]
    g = randn(1150, gate_up.shape[0], cols, dtype=torch.bfloat16)
    dev = gate_up.to(DEV).requires_grad_(True)
    (grad,) = torch.autograd.grad(diff.swiglu(dev[:, :cols], dev[:, cols:]), dev, g.to(DEV))
    native = oracle_grads(oracle.swiglu, (gate_up[:, :cols], gate_up[:, cols:]), g)
    got = grad.cpu()
    for name, mine, want in (("grad_a", got[:, :cols], native[0]), ("grad_b", got[:, cols:], native[1])):
        differing = int((mine != want).sum())
        worst = float((mine.float() - want.float()).abs().max())
        print(f"\n[swiglu backward {name}] elements={want.numel()} not-bit-identical={differing} max-abs={worst:.3e}")
        assert differing <= want.numel() * 1e-3 and worst <= 2e-2 * max(1.0, float(want.float().abs().max()))


@pytest.mark.parametrize("shape,half,dtype,interleaved", [((2, 33, 8, 128), 64, torch.bfloat16, False), ((1, 9, 6, 96), 24, torch.bfloat16, True),
                                                          ((2, 6, 2, 32), 16, torch.float32, False), ((2, 5, 3, 64), 16, torch.float16, False)])
def test_rotary_backward(shape, half, dtype, interleaved):
    x = randn(1200 + half, *shape, dtype=dtype)
    g = randn(1201 + half, *shape, dtype=dtype)
    cos, sin = workloads.rope_tables(shape[1], half)
    dev = x.to(DEV).requires_grad_(True)
    out = diff.rotary_embedding(dev, cos.to(DEV), sin.to(DEV), interleaved)
    (grad,) = torch.autograd.grad(out, dev, g.to(DEV))
    fn = lambda t: oracle.rotary_embedding(t, cos.to(t.dtype) if t.dtype == torch.float64 else cos, sin.to(t.dtype) if t.dtype == torch.float64 else sin, interleaved)  # noqa: E731
    (native,) = oracle_grads(fn, (x,), g)
    (truth,) = oracle_grads(fn, (x,), g, wide=True)
    grade(grad, native, truth, dtype, "grad_x")


@pytest.mark.parametrize("rows,cols,dtype", [(7, 136, torch.bfloat16), (64, 14336, torch.bfloat16), (5, 33, torch.bfloat16),
                                              (33, 1000, torch.float16), (129, 257, torch.float32)])
def test_geglu_backward(rows, cols, dtype):
    gate_up = randn(1900 + cols, rows, 2 * cols, dtype=dtype, scale=2.0)
    g = randn(1901 + cols, rows, cols, dtype=dtype)
    a, b = gate_up[:, :cols], gate_up[:, cols:]
    dev = gate_up.to(DEV).requires_grad_(True)
    out = diff.geglu(dev[:, :cols], dev[:, cols:])
    (grad,) = torch.autograd.grad(out, dev, g.to(DEV))
    native = oracle_grads(oracle.geglu, (a, b), g)
    truth = oracle_grads(oracle.geglu, (a, b), g, wide=True)
    # like the forward op, the kernel evaluates gelu through 1 / (1 + exp(-2u)) instead of 1 + tanh(u): where the
    # reference cancels, results land on the neighbouring 16-bit value
    exact = 0.95 if dtype != torch.float32 else None
    grade(grad[:, :cols], native[0], truth[0], dtype, "grad_a", exact)
    grade(grad[:, cols:], native[1], truth[1], dtype, "grad_b", exact)


@pytest.mark.parametrize("batch,hq,hk,seq,dim,dtype", [(2, 8, 2, 33, 128, torch.bfloat16), (1, 3, 1, 9, 64, torch.float16), (2, 2, 2, 5, 16, torch.float32)])
def test_paired_rope_backward(batch, hq, hk, seq, dim, dtype):
    q, k = randn(2000 + dim, batch, hq, seq, dim, dtype=dtype), randn(2001 + dim, batch, hk, seq, dim, dtype=dtype)
    gq, gk = randn(2002 + dim, batch, hq, seq, dim, dtype=dtype), randn(2003 + dim, batch, hk, seq, dim, dtype=dtype)
    cos = torch.cos(randn(2004, 1, seq, dim)).to(dtype)  # halves NOT repeated: the general transpose
    sin = torch.sin(randn(2005, 1, seq, dim)).to(dtype)
    leaves = [t.to(DEV).requires_grad_(True) for t in (q, k)]
    outs = diff.rope(leaves[0], leaves[1], cos.to(DEV), sin.to(DEV))
    grads = torch.autograd.grad(outs, leaves, [gq.to(DEV), gk.to(DEV)])
    cpu = [t.clone().requires_grad_(True) for t in (q, k)]
    native = torch.autograd.grad(oracle.rope(cpu[0], cpu[1], cos, sin), cpu, [gq, gk])
    for mine, want in zip(grads, native):
        assert torch.equal(mine.cpu(), want), "paired rope backward is not bit-identical to autograd of the reference"


@pytest.mark.parametrize("batch,seq,hq,hk,dim,dtype", [(2, 33, 8, 2, 128, torch.bfloat16), (1, 9, 3, 1, 64, torch.float16), (2, 5, 2, 2, 16, torch.float32)])
def test_llama4_rope_backward(batch, seq, hq, hk, dim, dtype):
    q, k = randn(2100 + dim, batch, seq, hq, dim, dtype=dtype), randn(2101 + dim, batch, seq, hk, dim, dtype=dtype)
    gq, gk = randn(2102 + dim, batch, seq, hq, dim, dtype=dtype), randn(2103 + dim, batch, seq, hk, dim, dtype=dtype)
    angle = randn(2104, seq, dim // 2)
    freqs = torch.stack((angle.cos(), angle.sin()), -1).to(dtype)
    leaves = [t.to(DEV).requires_grad_(True) for t in (q, k)]
    outs = diff.llama4_rope(leaves[0], leaves[1], freqs.to(DEV))
    grads = torch.autograd.grad(outs, leaves, [gq.to(DEV), gk.to(DEV)])
    cpu = [t.clone().requires_grad_(True) for t in (q, k)]
    native = torch.autograd.grad(oracle.llama4_rope(cpu[0], cpu[1], freqs), cpu, [gq, gk])
    for mine, want in zip(grads, native):
        assert torch.equal(mine.cpu(), want), "llama4 rope backward is not bit-identical to autograd of the reference"


@pytest.mark.parametrize("batch,hq,hk,seq,dim,dtype", [(2, 8, 2, 33, 128, torch.bfloat16), (1, 3, 1, 70, 64, torch.float16), (2, 2, 2, 5, 16, torch.float32),
                                                         (1, 2, 1, 9, 20, torch.bfloat16), (1, 4, 0, 40, 256, torch.bfloat16)])
def test_qk_norm_rope_backward(batch, hq, hk, seq, dim, dtype):
    q, k = randn(2200 + dim, batch, hq, seq, dim, dtype=dtype), randn(2201 + dim, batch, hk, seq, dim, dtype=dtype, scale=0.5)
    qw, kw = (1 + 0.1 * randn(2202, dim)).to(dtype), (1 + 0.1 * randn(2203, dim)).to(dtype)
    gq, gk = randn(2204 + dim, batch, hq, seq, dim, dtype=dtype), randn(2205 + dim, batch, hk, seq, dim, dtype=dtype)
    angle = randn(2206, 1, seq, dim // 2)
    cos, sin = torch.cos(angle).repeat(1, 1, 2).to(dtype), torch.sin(angle).repeat(1, 1, 2).to(dtype)
    leaves = [t.to(DEV).requires_grad_(True) for t in (q, k, qw, kw)]
    outs = diff.qk_norm_rope(*leaves, cos.to(DEV), sin.to(DEV), 1e-6)
    grads = torch.autograd.grad(outs, leaves, [gq.to(DEV), gk.to(DEV)], allow_unused=True)

    def reference(wide):
        cast = (lambda t: t.double()) if wide else (lambda t: t.clone())
        ls = [cast(t).requires_grad_(True) for t in (q, k, qw, kw)]
        out = oracle.qk_norm_rope(*ls, cast(cos), cast(sin), 1e-6)
        return torch.autograd.grad(out, ls, [cast(gq), cast(gk)], allow_unused=True)

    native, truth = reference(False), reference(True)
    for name, mine, nat, tru in zip(("grad_q", "grad_k", "grad_q_weight", "grad_k_weight"), grads, native, truth):
        if tru is None or tru.numel() == 0 or (hk == 0 and "k" in name.split("_")[1]):
            continue
        grade(mine, nat, tru, dtype, f"{name} {batch}x{hq}/{hk}x{seq}x{dim}")


@pytest.mark.parametrize("rows,cols,dtype", [(33, 256, torch.bfloat16), (40, 4096, torch.bfloat16), (9, 100, torch.float32), (6, 33, torch.bfloat16), (130, 2048, torch.float16)])
@pytest.mark.parametrize("with_bias", [False, True])
@pytest.mark.parametrize("activation", ["swish", "sigmoid"])
def test_rms_norm_gated_backward(rows, cols, dtype, with_bias, activation):
    x, gate = randn(2300 + cols, rows, cols, dtype=dtype), randn(2301 + cols, rows, cols, dtype=dtype, scale=2.0)
    w = (1 + 0.1 * randn(2302, cols)).to(dtype)
    b = randn(2303, cols, dtype=dtype) if with_bias else None
    grad = randn(2304 + cols, rows, cols, dtype=dtype)
    tensors = (x, gate, w, b) if with_bias else (x, gate, w)
    leaves = [t.to(DEV).requires_grad_(True) for t in tensors]
    y = diff.rms_norm_gated(leaves[0], leaves[1], leaves[2], leaves[3] if with_bias else None, activation, 1e-5)
    grads = torch.autograd.grad(y, leaves, grad.to(DEV))
    fn = (lambda x_, g_, w_, b_: oracle.rms_norm_gated(x_, g_, w_, b_, activation, 1e-5)) if with_bias else (lambda x_, g_, w_: oracle.rms_norm_gated(x_, g_, w_, None, activation, 1e-5))
    native = oracle_grads(fn, tensors, grad)
    truth = oracle_grads(fn, tensors, grad, wide=True)
    for name, mine, nat, tru in zip(("grad_x", "grad_gate", "grad_weight", "grad_bias"), grads, native, truth):
        grade(mine, nat, tru, dtype, f"{name} {rows}x{cols}")
    with pytest.raises(ValueError):
        diff.rms_norm_gated(leaves[0], leaves[1], leaves[2], None, "tanh", 1e-5)


@pytest.mark.parametrize("rows,cols,dtype", NORM_BWD_SHAPES)
def test_l2_norm_backward(rows, cols, dtype):
    x = randn(2400 + cols, rows, cols, dtype=dtype)
    g = randn(2401 + cols, rows, cols, dtype=dtype)
    dev = x.to(DEV).requires_grad_(True)
    (mine,) = torch.autograd.grad(diff.l2_norm(dev, 1e-6), dev, g.to(DEV))
    fn = lambda x_: oracle.l2_norm(x_, 1e-6)  # noqa: E731
    (native,) = oracle_grads(fn, (x,), g)
    (truth,) = oracle_grads(fn, (x,), g, wide=True)
    grade(mine, native, truth, dtype, f"l2_norm grad_x {rows}x{cols}")


@pytest.mark.parametrize("rows,cols,dtype", NORM_BWD_SHAPES)
@pytest.mark.parametrize("with_bias", [False, True])
def test_layer_norm_backward(rows, cols, dtype, with_bias):
    x = (randn(2500 + cols, rows, cols) + 0.3).to(dtype)
    w = (1 + 0.1 * randn(2501, cols)).to(dtype)
    b = randn(2502, cols, dtype=dtype) if with_bias else None
    g = randn(2503 + cols, rows, cols, dtype=dtype)
    tensors = (x, w, b) if with_bias else (x, w)
    leaves = [t.to(DEV).requires_grad_(True) for t in tensors]
    y = diff.layer_norm(leaves[0], leaves[1], leaves[2] if with_bias else None, 1e-5)
    grads = torch.autograd.grad(y, leaves, g.to(DEV))
    fn = (lambda x_, w_, b_: oracle.layer_norm(x_, w_, b_, 1e-5)) if with_bias else (lambda x_, w_: oracle.layer_norm(x_, w_, None, 1e-5))
    native = oracle_grads(fn, tensors, g)
    truth = oracle_grads(fn, tensors, g, wide=True)
    for name, mine, nat, tru in zip(("grad_x", "grad_weight", "grad_bias"), grads, native, truth):
        grade(mine, nat, tru, dtype, f"layer_norm {name} {rows}x{cols}")


@pytest.mark.parametrize("tokens,hidden,experts,top_k,dtype", [(64, 256, 8, 2, torch.bfloat16), (37, 72, 4, 3, torch.float16), (50, 33, 8, 4, torch.bfloat16),
                                                             (16, 64, 2, 1, torch.float32), (300, 4096, 64, 8, torch.bfloat16)])
def test_moe_steps_backward(tokens, hidden, experts, top_k, dtype):
    """route -> permute -> (an elementwise stand-in for the expert MLPs) -> unpermute, differentiated end to end."""
    x = randn(2600 + hidden, tokens, hidden, dtype=dtype)
    logits = randn(2601 + hidden, tokens, experts)
    grad = randn(2602 + hidden, tokens, hidden, dtype=dtype)
    assert oracle.route_is_unambiguous(logits, top_k)

    def chain(route, permute, unpermute, x_, logits_):
        indices, weights = route(logits_, top_k)
        rows, _, _, _, pos = permute(x_, indices, experts)
        return unpermute(rows * 1.5, weights, pos)

    def oracle_chain(x_, logits_):
        indices, weights = oracle.moe_route(logits_, top_k)
        rows, _, _, _, pos = oracle.moe_permute(x_, indices, experts)
        return oracle.moe_unpermute(rows * 1.5, weights, pos)

    leaves = [x.to(DEV).requires_grad_(True), logits.to(DEV).requires_grad_(True)]
    y = chain(diff.moe_route, diff.moe_permute, diff.moe_unpermute, *leaves)
    grads = torch.autograd.grad(y, leaves, grad.to(DEV))
    native = oracle_grads(oracle_chain, (x, logits), grad)
    truth = oracle_grads(oracle_chain, (x, logits), grad, wide=True)
    grade(grads[0], native[0], truth[0], dtype, f"grad_x {tokens}x{hidden}")
    # the logits are fp32 whatever the activations are; their gradient inherits the activations' rounding noise
    err = float((grads[1].cpu().double() - truth[1]).abs().max())
    budget = float((native[1].double() - truth[1]).abs().max())
    assert err <= max(4 * budget, FLOOR[dtype] * max(1.0, float(truth[1].abs().max()))), f"grad_logits: {err:.3e} vs budget {budget:.3e}"


def test_registry_serves_training_calls():
    x = randn(1300, 8, 256, dtype=torch.bfloat16).to(DEV).requires_grad_(True)
    out = kernels.swiglu(x, x, backend="b200")
    out.float().sum().backward()
    assert x.grad is not None and torch.isfinite(x.grad.float()).all()




@pytest.mark.parametrize("rows,cols,dtype", NORM_BWD_SHAPES)
@pytest.mark.parametrize("with_bias", [False, True])
def test_rms_norm_backward(rows, cols, dtype, with_bias):
    x = randn(1500 + cols, rows, cols, dtype=dtype)
    w = (1 + 0.1 * randn(1501, cols)).to(dtype)
    b = randn(1502, cols, dtype=dtype) if with_bias else None
    g = randn(1503 + cols, rows, cols, dtype=dtype)
    leaves = [t.to(DEV).requires_grad_(True) for t in (x, w, *([b] if with_bias else []))]
    y = diff.rms_norm(leaves[0], leaves[1], leaves[2] if with_bias else None, 1e-5)
    grads = torch.autograd.grad(y, leaves, g.to(DEV))
    fn = (lambda x_, w_, b_: oracle.rms_norm(x_, w_, b_, 1e-5)) if with_bias else (lambda x_, w_: oracle.rms_norm(x_, w_, None, 1e-5))
    inputs = (x, w, b) if with_bias else (x, w)
    native = oracle_grads(fn, inputs, g)
    truth = oracle_grads(fn, inputs, g, wide=True)
    for name, mine, nat, tru in zip(("grad_x", "grad_weight", "grad_bias"), grads, native, truth):
        grade(mine, nat, tru, dtype, f"{name} {rows}x{cols}")


@pytest.mark.parametrize("rows,cols,dtype", NORM_BWD_SHAPES[:10] + [(130, 2048, torch.float16), (1000, 128, torch.bfloat16), (40, 3072, torch.bfloat16), (20, 5120, torch.bfloat16)])
@pytest.mark.parametrize("offset,use_s", [(0.0, True), (1.0, True), (0.0, False)])
def test_add_rms_norm_backward(rows, cols, dtype, offset, use_s):
    x = randn(1600 + cols, rows, cols, dtype=dtype)
    r = randn(1601 + cols, rows, cols, dtype=dtype)
    w = (1 + 0.1 * randn(1602, cols)).to(dtype)
    gy = randn(1603 + cols, rows, cols, dtype=dtype)
    gs = randn(1604 + cols, rows, cols, dtype=dtype)

    def run(fn, tensors, wide=False):
        leaves = [t.double().requires_grad_(True) if wide else t.clone().requires_grad_(True) for t in tensors]
        y, s = fn(*leaves)
        outs, seeds = ([y, s], [gy, gs]) if use_s else ([y], [gy])
        seeds = [t.to(y.device).to(y.dtype) for t in seeds]
        return torch.autograd.grad(outs, leaves, seeds)

    fn = lambda x_, r_, w_: oracle.add_rms_norm(x_, r_, w_, 1e-5, offset)  # noqa: E731
    native, truth = run(fn, (x, r, w)), run(fn, (x, r, w), wide=True)
    mine = run(lambda x_, r_, w_: diff.add_rms_norm(x_, r_, w_, 1e-5, offset), (x.to(DEV), r.to(DEV), w.to(DEV)))
    for name, m, nat, tru in zip(("grad_x", "grad_residual", "grad_weight"), mine, native, truth):
        grade(m, nat, tru, dtype, f"{name} {rows}x{cols} offset={offset}")
    assert torch.equal(mine[0], mine[1])


def test_norm_backward_full_width_sample():
    w = workloads.add_rms_norm_bf16(scale=1 / 16)
    x, r, weight = (w.inputs[k] for k in ("x", "residual", "weight"))
    gy = randn(1700, *x.shape, dtype=torch.bfloat16)
    leaves = [t.to(DEV).requires_grad_(True) for t in (x, r, weight)]
    y, s = diff.add_rms_norm(*leaves, 1e-5, 0.0)
    mine = torch.autograd.grad(y, leaves, gy.to(DEV))
    cpu = [t.clone().requires_grad_(True) for t in (x, r, weight)]
    native = torch.autograd.grad(oracle.add_rms_norm(*cpu, 1e-5, 0.0)[0], cpu, gy)
    for name, m, n in zip(("grad_x", "grad_residual", "grad_weight"), mine, native):
        m = m.cpu()
        print(f"\n[add_rms_norm backward {name}] elements={n.numel()} not-bit-identical={int((m != n).sum())} max-abs={float((m.float() - n.float()).abs().max()):.3e}")
    assert float((mine[0].cpu().float() - native[0].float()).abs().max()) <= 2e-2


@pytest.mark.parametrize("name", [n for n in case_names() if n.startswith("grad_")])
def test_gradients_against_the_references_own(name):
    """Fixtures written by autograd through the real popcorn references (case dtype and fp64): every gradient of the
    CUDA path is within popcorn's own bound of the fp64 one, twice the reference's error or the dtype's floor."""
    t, meta = load_case(name)
    keys = [k for k in t if f"grad_{k}" in t]
    leaves = {k: t[k].to(DEV).requires_grad_(True) for k in keys}
    op = meta["op"]
    if op == "rms_norm":
        outs = (diff.rms_norm(leaves["x"], leaves["weight"], leaves["bias"], meta["eps"]),)
    elif op == "add_rms_norm":
        outs = diff.add_rms_norm(leaves["x"], leaves["residual"], leaves["weight"], meta["eps"], meta["offset"])
    elif op == "swiglu":
        outs = (diff.swiglu(leaves["a"], leaves["b"]),)
    else:
        outs = (diff.momoe(leaves["x"], leaves["gate_weight"], leaves["up_weight"], leaves["down_weight"], leaves["router_logits"], meta["top_k"]),)
    seeds = [t[f"cotangent{i}"].to(DEV) for i in range(len(outs))]
    grads = torch.autograd.grad(outs, list(leaves.values()), seeds)
    for key, mine in zip(keys, grads):
        dtype = torch.bfloat16 if op == "momoe" else t[key].dtype  # momoe: 16-bit intermediates bound the fp32 logits' gradient too
        grade(mine, t[f"grad_{key}"], t[f"truth_{key}"], dtype, f"{name} grad {key}")
