"""Grouped expert GEMM (tcgen05 tensor cores) against the CPU oracle and the registered momoe reference.

Operands are bf16 / fp16, products are exact, sums are fp32 in another order than the CPU's, and the result
is rounded once, so almost every element is bit-identical and the rest differ by one unit of the 16-bit
type.  The bound is therefore max-abs <= 2e-2 * max(1, |y|) for bf16 (one unit of bf16 at |y| in [4, 8) is
already 3.1e-2) and 2e-3 * max(1, |y|) for fp16; outputs are O(1) (unit-init weights, like the reference's
own test inputs).
"""

import pytest
import torch

from oracle import reference_ops as oracle
from popcorn_b200 import _lib, ops
from tests.golden.golden_io import case_names, load_case
from tests.test_parity_gpu import BF16, F16, gpu, randn

pytestmark = pytest.mark.gpu


def close(got, want, what, exact_fraction=0.98):
    got = got.cpu()
    assert got.shape == want.shape and got.dtype == want.dtype, (what, got.shape, want.shape)
    if want.numel() == 0:
        return
    bound = 2e-2 if want.dtype == BF16 else 2e-3
    excess = (got.double() - want.double()).abs() / want.double().abs().clamp(min=1.0)
    assert float(excess.max()) <= bound, f"{what}: |diff| / max(1, |y|) = {float(excess.max()):.3e} exceeds {bound:.0e}"
    same = float((got == want).double().mean())
    assert same >= exact_fraction, f"{what}: only {same:.5f} of elements are bit-identical"


def make(counts, k, n, dtype, seed, pad=0):
    offsets = torch.tensor([0, *torch.tensor(counts).cumsum(0).tolist()], dtype=torch.int32)
    total = int(offsets[-1]) + pad
    rows = randn(seed, total, k, dtype=dtype)
    gate = (randn(seed + 1, len(counts), k, n) / k ** 0.5).to(dtype)
    up = (randn(seed + 2, len(counts), k, n) / k ** 0.5).to(dtype)
    return rows, gate, up, offsets


CASES = [
    # per-expert row counts, k, n, dtype
    ([128], 64, 256, BF16), ([128, 70], 128, 256, BF16), ([1], 8, 8, BF16), ([5, 0, 3], 72, 40, BF16),
    ([300, 0, 17, 129], 512, 384, BF16), ([37, 250, 0, 128, 1], 1024, 512, F16), ([0, 0, 260], 200, 264, BF16),
    ([129] * 16, 256, 128, BF16), ([640, 513], 320, 1032, F16),
]


@pytest.mark.parametrize("counts,k,n,dtype", CASES)
def test_single_projection(counts, k, n, dtype):
    rows, weight, _, offsets = make(counts, k, n, dtype, 5000 + k, pad=3)
    got = ops.moe_grouped_gemm(gpu(rows), gpu(weight), gpu(offsets))
    close(got, oracle.moe_grouped_gemm(rows, weight, offsets), f"grouped gemm {counts} k={k} n={n}")
    assert _lib.wait_timeouts() == 0
    assert not got[int(offsets[-1]):].any(), "rows outside every segment must stay zero"


@pytest.mark.parametrize("counts,k,n,dtype", CASES)
def test_gate_up_swiglu_projection(counts, k, n, dtype):
    rows, gate, up, offsets = make(counts, k, n, dtype, 5100 + k)
    got = ops.moe_grouped_gemm(gpu(rows), gpu(gate), gpu(offsets), gpu(up))
    close(got, oracle.moe_grouped_gemm(rows, gate, offsets, up), f"gate/up {counts} k={k} n={n}")
    assert _lib.wait_timeouts() == 0


@pytest.mark.parametrize("pair", ["1", "0"])
@pytest.mark.parametrize("counts,k,n,dtype", CASES)
def test_gathered_operand_equals_the_permuted_rows(counts, k, n, dtype, pair, monkeypatch):
    """The A rows fetched through the permutation by four-row gathered copies: bit-identical to the projection of the
    materialised rows, alone and fused with SwiGLU, as CTA pairs and as single CTAs."""
    monkeypatch.setenv("B200_GEMM_PAIR", pair)
    rows, gate, up, offsets = make(counts, k, n, dtype, 5300 + k)
    total = int(offsets[-1])
    tokens = max(total // 2, 1) + 5
    gen = torch.Generator().manual_seed(5301 + k)
    x = randn(5302 + k, tokens, k, dtype=dtype)
    perm = torch.randint(0, tokens, (total,), generator=gen, dtype=torch.int32)  # tokens repeat, like top_k > 1
    gathered_rows = x[perm.long()]
    for second in (None, up):
        want = ops.moe_grouped_gemm(gpu(gathered_rows), gpu(gate), gpu(offsets), gpu(second))
        got = ops.moe_grouped_gemm_gathered(gpu(x), gpu(perm), gpu(gate), gpu(offsets), gpu(second))
        assert torch.equal(got, want), f"gathered {counts} k={k} n={n} dual={second is not None}"
    wide = gpu(torch.cat((x, x), dim=1))  # token rows given as a column slice
    got = ops.moe_grouped_gemm_gathered(wide[:, :k], gpu(perm), gpu(gate), gpu(offsets))
    assert torch.equal(got, ops.moe_grouped_gemm(gpu(gathered_rows), gpu(gate), gpu(offsets)))
    assert _lib.wait_timeouts() == 0


def test_strided_rows_and_many_tiles_per_cta():
    """More tiles than SMs (persistent CTAs reuse both accumulators and wrap the ring) and rows given as a column slice."""
    counts = [257] * 40
    rows, weight, _, offsets = make(counts, 192, 512, BF16, 5200)
    wide = gpu(torch.cat((rows, rows), dim=1))
    got = ops.moe_grouped_gemm(wide[:, :192], gpu(weight), gpu(offsets))
    close(got, oracle.moe_grouped_gemm(rows, weight, offsets), "many tiles")
    assert _lib.wait_timeouts() == 0


@pytest.mark.parametrize("name", [n for n in case_names() if n.startswith("moe16")])
def test_golden_momoe_through_the_grouped_projections(name):
    """route -> permute -> gate/up + SwiGLU -> down -> unpermute, all on the GPU, against the registered momoe reference."""
    t, meta = load_case(name)
    top_k = meta["top_k"]
    experts = t["gate_weight"].shape[0]
    x = gpu(t["x"].reshape(-1, t["x"].shape[-1]))
    idx, w = ops.moe_route(gpu(t["router_logits"].reshape(-1, experts)), top_k)
    assert torch.equal(idx.cpu(), t["topk_indices"].reshape(-1, top_k))
    rows, counts, offsets, perm, pos = ops.moe_permute(x, idx, experts)
    hidden_act = ops.moe_grouped_gemm(rows, gpu(t["gate_weight"]), offsets, gpu(t["up_weight"]))
    out_rows = ops.moe_grouped_gemm(hidden_act, gpu(t["down_weight"]), offsets)
    y = ops.moe_unpermute(out_rows, w, pos).cpu().reshape(t["y"].shape)
    assert y.dtype == t["y"].dtype
    assert float((y.float() - t["y"].float()).abs().max()) <= 2e-2, name
    # and against the same chain on the CPU oracle (same intermediate roundings): only summation order differs
    o_rows, _, o_offsets, _, o_pos = oracle.moe_permute(t["x"].reshape(-1, t["x"].shape[-1]), idx.cpu(), experts)
    o_hidden = oracle.moe_grouped_gemm(o_rows, t["gate_weight"], o_offsets, t["up_weight"])
    close(hidden_act, o_hidden, name + " hidden")
    assert _lib.wait_timeouts() == 0


@pytest.mark.parametrize("name", [n for n in case_names() if n.startswith("moe16")])
def test_golden_momoe_op(name):
    """The registered op itself, through the registry mirror, against the reference's output."""
    from popcorn_b200 import kernels

    t, meta = load_case(name)
    y = kernels.momoe(gpu(t["x"]), gpu(t["gate_weight"]), gpu(t["up_weight"]), gpu(t["down_weight"]), gpu(t["router_logits"]),
                      meta["top_k"], backend="b200")
    assert y.shape == t["y"].shape and y.dtype == t["y"].dtype
    assert float((y.cpu().float() - t["y"].float()).abs().max()) <= 2e-2, name
    with pytest.raises(TypeError):
        ops.momoe(gpu(t["x"].float()), gpu(t["gate_weight"].float()), gpu(t["up_weight"].float()), gpu(t["down_weight"].float()),
                  gpu(t["router_logits"]), meta["top_k"])


def test_large_segments_against_the_library_matmul():
    """Eight experts of 2048-2300 rows at the benchmark's hidden and intermediate sizes, against fp32 matmuls of the same
    16-bit operands on the GPU (the CPU oracle would take minutes here)."""
    counts = [2048, 2300, 2100, 2048, 2049, 2047, 2200, 2048]
    rows, gate, up, offsets = make(counts, 4096, 1536, BF16, 5400)
    d_rows, d_gate, d_up, d_off = gpu(rows), gpu(gate), gpu(up), gpu(offsets)
    got = ops.moe_grouped_gemm(d_rows, d_gate, d_off, d_up)
    down = gpu((randn(5403, len(counts), 1536, 4096) / 1536 ** 0.5).to(BF16))
    got_down = ops.moe_grouped_gemm(got, down, d_off)
    torch.backends.cuda.matmul.allow_tf32 = False
    bounds = offsets.tolist()
    for e in range(len(counts)):
        seg = d_rows[bounds[e]:bounds[e + 1]].float()
        want = (torch.nn.functional.silu(seg @ d_gate[e].float()) * (seg @ d_up[e].float())).to(BF16)
        close(got[bounds[e]:bounds[e + 1]], want.cpu(), f"expert {e} gate/up")
        want_down = (got[bounds[e]:bounds[e + 1]].float() @ down[e].float()).to(BF16)
        close(got_down[bounds[e]:bounds[e + 1]], want_down.cpu(), f"expert {e} down")
    assert _lib.wait_timeouts() == 0


def test_offsets_beyond_the_buffer_are_clamped():
    rows, weight, _, offsets = make([100, 60], 64, 64, BF16, 5500)
    wrong = offsets.clone()
    wrong[-1] += 500  # claims rows the buffers do not have
    got = ops.moe_grouped_gemm(gpu(rows), gpu(weight), gpu(wrong))
    close(got, oracle.moe_grouped_gemm(rows, weight, offsets), "clamped offsets")


def test_empty_and_rejected_inputs():
    rows, weight, _, offsets = make([4, 4], 16, 16, BF16, 5300)
    empty = ops.moe_grouped_gemm(gpu(rows[:0]), gpu(weight), gpu(torch.zeros(3, dtype=torch.int32)))
    assert empty.shape == (0, 16)
    none = ops.moe_grouped_gemm(gpu(rows), gpu(weight), gpu(torch.zeros(3, dtype=torch.int32)))
    assert not none.any()
    with pytest.raises(TypeError):
        ops.moe_grouped_gemm(gpu(rows.float()), gpu(weight.float()), gpu(offsets))
    with pytest.raises(TypeError):
        ops.moe_grouped_gemm(gpu(rows), gpu(weight), gpu(offsets.long()))
    with pytest.raises(ValueError):
        ops.moe_grouped_gemm(gpu(rows), gpu(weight[:, :8]), gpu(offsets))
    with pytest.raises(_lib.B200Error):  # rows of 12 elements are not 16-byte multiples
        ops.moe_grouped_gemm(gpu(rows[:, :12].contiguous()), gpu(weight[:, :12].contiguous()), gpu(offsets))
