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

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
FLOOR = {torch.float32: 2e-5, torch.float16: 1e-3, torch.bfloat16: 2e-2}


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


def test_registry_serves_training_calls():
    x = randn(1300, 8, 256, dtype=torch.bfloat16).to(DEV).requires_grad_(True)
    out = kernels.swiglu(x, x, backend="b200")
    out.float().sum().backward()
    assert x.grad is not None and torch.isfinite(x.grad.float()).all()
