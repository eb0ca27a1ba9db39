"""The five benchmark configurations at FULL size: CUDA path against the CPU oracle.

Inputs come from popcorn_b200.workloads (seeded, same draw protocol as popcorn's
harness).  Each test prints how many elements are not bit-identical and the
worst absolute difference, then applies the specified bound (max-abs <= 2e-2 for
bf16, <= 1e-5 for fp32, equality for indices / counts / gathered rows), and
checks size-independent properties of the result as well.
"""

import pytest
import torch

from oracle import reference_ops as oracle
from popcorn_b200 import ops, workloads

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def report(name, got, want, bound):
    got = got.cpu()
    diff = (got.float() - want.float()).abs()
    worst = float(diff.max())
    differing = int((got != want).sum())
    over = int((diff > bound).sum())
    print(f"\n[{name}] elements={want.numel()} not-bit-identical={differing} max-abs={worst:.4e} over-bound={over}")
    assert over == 0, f"{name}: {over} elements exceed max-abs {bound}; worst {worst:.4e}"
    return differing


def test_config1_rms_norm_fp32():
    w = workloads.rms_norm_fp32()
    x, weight = w.inputs["x"], w.inputs["weight"]
    got = ops.rms_norm(x.to(DEV), weight.to(DEV), None, w.args["eps"])
    report("C1 rms_norm fp32 4096x4096", got, oracle.rms_norm(x, weight, None, w.args["eps"]), 1e-5)
    # property: with unit weight every row has mean square 1 (up to eps and rounding)
    unit = ops.rms_norm(x.to(DEV), torch.ones_like(weight).to(DEV), None, w.args["eps"])
    assert torch.allclose(unit.square().mean(-1), torch.ones(x.shape[0], device=DEV), atol=1e-4)


def test_config2_add_rms_norm_bf16():
    w = workloads.add_rms_norm_bf16()
    x, r, weight = w.inputs["x"], w.inputs["residual"], w.inputs["weight"]
    y, s = ops.add_rms_norm(x.to(DEV), r.to(DEV), weight.to(DEV), w.args["eps"], w.args["offset"])
    want_y, want_s = oracle.add_rms_norm(x, r, weight, w.args["eps"], w.args["offset"])
    assert torch.equal(s.cpu(), want_s), "C2: the updated residual stream must be bit-identical"
    differing = report("C2 add_rms_norm bf16 16384x8192", y, want_y, 2e-2)
    assert differing <= want_y.numel() * 1e-4
    # property: the fused op equals rms_norm applied to its own residual output
    assert torch.equal(ops.rms_norm(s, weight.to(DEV), None, w.args["eps"]), y)


def test_config3_rotary_bf16():
    w = workloads.rotary_bf16()
    q, k, cos, sin = (w.inputs[n] for n in ("q", "k", "cos", "sin"))
    dq, dk, dcos, dsin = q.to(DEV), k.to(DEV), cos.to(DEV), sin.to(DEV)
    out_q = ops.rotary_embedding(dq, dcos, dsin)
    out_k = ops.rotary_embedding(dk, dcos, dsin)
    ops.rotary_embedding_qk_(dq, dk, dcos, dsin)  # in place, one launch
    assert torch.equal(dq, out_q) and torch.equal(dk, out_k)
    assert report("C3 rotary q bf16 8x4096x32x128", out_q, oracle.rotary_embedding(q, cos, sin), 2e-2) == 0
    assert report("C3 rotary k bf16 8x4096x8x128", out_k, oracle.rotary_embedding(k, cos, sin), 2e-2) == 0
    # property: rotating back with -sin restores the input up to two bf16 roundings
    back = ops.rotary_embedding(out_k, dcos, -dsin)
    assert float((back.float() - k.to(DEV).float()).abs().max()) <= 6e-2
    # property: position 0 has angle 0 and is left untouched
    assert torch.equal(out_q[:, 0], q.to(DEV)[:, 0])


def test_config4_swiglu_bf16():
    w = workloads.swiglu_bf16()
    gate_up, cols = w.inputs["gate_up"], w.args["cols"]
    dev = gate_up.to(DEV)
    got = ops.swiglu(dev[:, :cols], dev[:, cols:])
    differing = report("C4 swiglu bf16 32768x14336", got, oracle.swiglu(gate_up[:, :cols], gate_up[:, cols:]), 2e-2)
    assert differing <= got.numel() * 1e-4
    # property: a zero gate or a zero up-projection gives exactly zero
    assert not ops.swiglu(torch.zeros_like(dev[:64, :cols]), dev[:64, cols:]).any()
    assert not ops.swiglu(dev[:64, :cols], torch.zeros_like(dev[:64, cols:])).any()


def test_config5_moe_permute_unpermute():
    w = workloads.moe_bf16()
    x, logits = w.inputs["x"], w.inputs["router_logits"]
    experts, top_k = w.args["experts"], w.args["top_k"]
    tokens = x.shape[0]
    assert oracle.route_is_unambiguous(logits, top_k), "synthetic logits must have no tie inside the top-(k+1)"
    want_idx, want_w = oracle.moe_route(logits, top_k)
    want_counts, want_offsets, want_perm, want_pos = oracle.moe_index(want_idx, experts)

    dx = x.to(DEV)
    idx, wts = ops.moe_route(logits.to(DEV), top_k)
    assert torch.equal(idx.cpu(), want_idx), "C5: top-k expert indices differ"
    report("C5 route weights fp32", wts, want_w, 1e-5)
    rows, counts, offsets, perm, pos = ops.moe_permute(dx, idx, experts)
    assert torch.equal(counts.cpu(), want_counts), "C5: expert counts differ"
    assert torch.equal(offsets.cpu(), want_offsets), "C5: expert offsets differ"
    assert torch.equal(perm.cpu(), want_perm), "C5: permutation index differs"
    assert torch.equal(pos.cpu(), want_pos), "C5: inverse permutation differs"
    print(f"\n[C5 index] counts min={int(counts.min())} max={int(counts.max())} total={int(counts.sum())}")
    # gathered rows, compared on the device against an index_select of the same input
    assert torch.equal(rows, dx.index_select(0, perm.long())), "C5: gathered rows differ"
    assert torch.equal(rows.cpu()[: 1 << 16], x.index_select(0, want_perm[: 1 << 16].long()))
    assert torch.equal(ops.moe_gather(dx, perm), rows)

    # unpermute against the oracle, with per-row scaling so the eight terms of a token differ
    gen = torch.Generator().manual_seed(5)
    row_scale = (0.5 + torch.rand(tokens * top_k, 1, generator=gen)).to(torch.bfloat16)
    scaled = rows * row_scale.to(DEV)
    y = ops.moe_unpermute(scaled, wts, pos)
    want_y = oracle.moe_unpermute(scaled.cpu(), wts.cpu(), want_pos)
    assert report("C5 unpermute bf16 65536x4096", y, want_y, 2e-2) == 0, "same weights, same order: must be bit-identical"

    # property: permute then unpermute with weights that sum to one returns x up to rounding
    round_trip = ops.moe_unpermute(rows, wts, pos)
    err = (round_trip.float() - dx.float()).abs()
    assert float(err.max()) <= 2e-2 * max(1.0, float(dx.float().abs().max()) / 4)
    # property: every token appears exactly top_k times and offsets partition the rows
    assert int(counts.sum()) == tokens * top_k and torch.equal(offsets[1:] - offsets[:-1], counts)
    assert torch.equal(torch.bincount(perm.long(), minlength=tokens), torch.full((tokens,), top_k, device=DEV))
