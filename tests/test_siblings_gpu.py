"""The memory-bound siblings behind the same ABI: geglu, rms_norm_gated, l2_norm, layer_norm.

Same bar as the five benchmark ops: golden vectors produced by the real popcorn references, seeded shapes
against the CPU oracle, max-abs <= 2e-2 for 16-bit inputs and <= 1e-5 for fp32 inputs.
"""

import pytest
import torch

from oracle import reference_ops as oracle
from popcorn_b200 import ops
from tests.golden.golden_io import case_names, load_case
from tests.test_parity_gpu import BF16, F16, F32, check, gpu, randn

pytestmark = pytest.mark.gpu

# Share of elements that must be bit-identical to the reference, per op (the max-abs bound always applies).
#  geglu: the reference forms 0.5*x*(1 + tanh(u)) and loses relative precision in 1 + tanh(u) for negative x;
#         the kernel evaluates the same function as x / (1 + exp(-2u)) without that cancellation, so about 1.5 %
#         of the (small) negative outputs land on the neighbouring 16-bit value.
#  l2norm: PyTorch's CPU rsqrt of a 16-bit tensor rounds sqrt(v) to T before the reciprocal in its vectorised
#         loop but not in its scalar tail, so the reference's scale differs by one unit of T between rows of
#         one tensor and between machines; the kernel always takes 1/sqrt in fp32 and rounds once.  A row whose
#         scale differs differs in most of its elements, by one unit of T.
EXACT = {"geglu": 0.97, "rmsgated": 0.99, "l2norm": 0.0, "layernorm": 0.99}


@pytest.mark.parametrize("name", [n for n in case_names() if n.startswith(("geglu", "rmsgated", "l2norm", "layernorm"))])
def test_golden_siblings(name):
    t, meta = load_case(name)
    if name.startswith("geglu"):
        g = gpu(t["gate_up"])
        cols = g.shape[1] // 2
        got = ops.geglu(g[:, :cols], g[:, cols:])
    elif name.startswith("rmsgated"):
        got = ops.rms_norm_gated(gpu(t["x"]), gpu(t["g"]), gpu(t["weight"]), gpu(t.get("bias")), meta["activation"], meta["eps"])
    elif name.startswith("l2norm"):
        got = ops.l2_norm(gpu(t["x"]), meta["eps"])
    else:
        got = ops.layer_norm(gpu(t["x"]), gpu(t["weight"]), gpu(t.get("bias")), meta["eps"])
    check(got, t["y"], exact_fraction=EXACT[name.split("_")[0]], what=name)


@pytest.mark.parametrize("rows,cols,dtype", [(1, 8, BF16), (7, 136, BF16), (64, 14336, BF16), (5, 33, BF16), (3, 1000, F16), (129, 257, F32), (300, 16, BF16)])
def test_geglu_shapes(rows, cols, dtype):
    gate_up = randn(2000 + cols, rows, 2 * cols, dtype=dtype, scale=2.0)
    g = gpu(gate_up)
    check(ops.geglu(g[:, :cols], g[:, cols:]), oracle.geglu(gate_up[:, :cols], gate_up[:, cols:]), exact_fraction=EXACT["geglu"], what=f"geglu {rows}x{cols}")


SHAPES = [(1, 8, BF16), (3, 256, BF16), (5, 264, BF16), (9, 512, F16), (7, 1024, BF16), (4, 2048, BF16), (3, 4096, BF16), (2, 8192, BF16), (2, 16384, BF16),
          (1, 20000, BF16), (1000, 128, F32), (33, 4096, F32), (6, 100, F32), (5, 33, BF16), (2, 12288, F32),
          (1030, 128, BF16), (515, 64, BF16), (301, 16, F32), (77, 72, F16)]


@pytest.mark.parametrize("rows,cols,dtype", SHAPES)
def test_rms_norm_gated_shapes(rows, cols, dtype):
    x, g = randn(2100 + cols, rows, cols, dtype=dtype), randn(2101 + cols, rows, cols, dtype=dtype, scale=2.0)
    w, b = (1 + 0.1 * randn(2102, cols)).to(dtype), randn(2103, cols, dtype=dtype)
    for bias, activation, eps in ((None, "swish", 1e-6), (b, "sigmoid", 1e-5)):
        check(ops.rms_norm_gated(gpu(x), gpu(g), gpu(w), gpu(bias), activation, eps), oracle.rms_norm_gated(x, g, w, bias, activation, eps),
              exact_fraction=0.99, what=f"rms_norm_gated {rows}x{cols} {activation}")


@pytest.mark.parametrize("rows,cols,dtype", SHAPES)
def test_l2_norm_shapes(rows, cols, dtype):
    x = randn(2200 + cols, rows, cols, dtype=dtype)
    for eps in (1e-6, 1e-5):
        check(ops.l2_norm(gpu(x), eps), oracle.l2_norm(x, eps), exact_fraction=EXACT["l2norm"], what=f"l2_norm {rows}x{cols}")


@pytest.mark.parametrize("rows,cols,dtype", SHAPES)
def test_layer_norm_shapes(rows, cols, dtype):
    x = (randn(2300 + cols, rows, cols) + 0.3).to(dtype)
    w, b = (1 + 0.1 * randn(2301, cols)).to(dtype), randn(2302, cols, dtype=dtype)
    for bias, eps in ((None, 1e-6), (b, 1e-5)):
        check(ops.layer_norm(gpu(x), gpu(w), gpu(bias), eps), oracle.layer_norm(x, w, bias, eps), exact_fraction=0.99, what=f"layer_norm {rows}x{cols}")


def test_sibling_strided_views_and_empty():
    buf = randn(2400, 6, 5, 512 + 64, dtype=BF16)
    w = (1 + 0.1 * randn(2401, 512)).to(BF16)
    x, g = buf[..., 32:544], buf[..., 64:576]
    dev = gpu(buf)
    check(ops.rms_norm_gated(dev[..., 32:544], dev[..., 64:576], gpu(w)), oracle.rms_norm_gated(x, g, w), exact_fraction=0.99)
    check(ops.layer_norm(dev[..., 32:544], gpu(w)), oracle.layer_norm(x, w), exact_fraction=0.99)
    check(ops.l2_norm(dev[..., 1:513]), oracle.l2_norm(buf[..., 1:513]), exact_fraction=0.0)  # 2-byte aligned: scalar kernel
    empty = torch.empty(0, 64, dtype=BF16, device="cuda:0")
    ones = torch.ones(64, dtype=BF16, device="cuda:0")
    assert ops.geglu(empty, empty).shape == ops.l2_norm(empty).shape == ops.layer_norm(empty, ones).shape == (0, 64)
