"""The b200 backend driven by popcorn itself, on the GPU: registered with `plugin.register()`, selected by popcorn's own
dispatcher (src/popcorn/core/dispatcher.py:287-309), invoked by its `Implementation.invoke` (:160-170), graded by its
own comparison harness (src/popcorn/bench/compare.py:182-303) and ranked by its own tuner from the rows its own store
wrote (src/popcorn/bench/store.py:358-380, src/popcorn/core/policy.py:74-119).

Everything is compared with `KERNELS[op].reference` — popcorn's registered PyTorch definition — evaluated on the same
device tensors.  Tolerances: max-abs <= 2e-2 for 16-bit inputs, <= 1e-5 for fp32 inputs, integer outputs equal.
"""

import json
import os

import pytest
import torch

from popcorn_b200 import ops, plugin, workloads
from tests import popcorn_location

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not popcorn_location.available(), reason=popcorn_location.MISSING)]

DEV = "cuda:0"
BF16, F32 = torch.bfloat16, torch.float32
MAX_ABS = {torch.float32: 1e-5, torch.float16: 2e-2, torch.bfloat16: 2e-2}


@pytest.fixture(scope="module")
def popcorn(tmp_path_factory):
    """The real popcorn with an empty report cache of its own and the b200 backend registered on it."""
    before = os.environ.get("POPCORN_CACHE_DIR")
    module = popcorn_location.import_popcorn(tmp_path_factory.mktemp("popcorn_cache"))
    served = plugin.register()
    assert set(served) == {*plugin.EXISTING_OPS, *plugin.NEW_OPS}
    for op in module.KERNELS.values():  # rows read before the cache moved must not decide anything here
        op.tuner.forget()
    yield module
    if before is None:
        os.environ.pop("POPCORN_CACHE_DIR", None)
    else:
        os.environ["POPCORN_CACHE_DIR"] = before


def forced_three_ways(op, *args):
    """The three ways popcorn lets a caller force a backend; all must run the same implementation."""
    first = op(*args, backend="b200")
    second = op["b200"](*args)
    with op["b200"] as scoped:
        third = scoped(*args)
    return first, second, third


def outputs(value):
    return list(value) if isinstance(value, (tuple, list)) else [value]


def close(got, want, what, row_sums=False):
    """max-abs within the dtype's bound.  `row_sums`: the output scales every element by a per-row fp32 sum that this
    backend and torch's GPU kernels add up in different orders.  A last-bit difference in that factor moves a few of
    the reference's intermediate roundings (normalised value to 16 bits, then times the weight to 16 bits again) to the
    neighbouring 16-bit value; times a weight above one and rounded again that is up to two steps of the output, and
    from |y| >= 2 two bf16 steps (0.03125) are more than 2e-2.  Such elements may differ by at most two steps of the
    output dtype, and there must be at most a handful per million; everything else is within the bound."""
    assert got.shape == want.shape and got.dtype == want.dtype and got.device == want.device, what
    if not want.is_floating_point():
        assert torch.equal(got, want), f"{what}: integer output differs"
        return
    if not want.numel():
        return
    diff = (got.double() - want.double()).abs()
    over = diff > MAX_ABS[want.dtype]
    if row_sums and want.dtype != torch.float32 and bool(over.any()):
        larger = torch.maximum(want.double().abs(), got.double().abs())[over]
        step = torch.finfo(want.dtype).eps * 2.0 ** torch.floor(torch.log2(larger))
        assert bool((diff[over] <= 2 * step).all()), f"{what}: a difference larger than two {want.dtype} steps"
        assert int(over.sum()) <= max(4, want.numel() // 250_000), f"{what}: {int(over.sum())} one-step differences above {MAX_ABS[want.dtype]:.0e}"
        return
    worst = float(diff.max())
    assert worst <= MAX_ABS[want.dtype], f"{what}: max-abs {worst:.3e} exceeds {MAX_ABS[want.dtype]:.0e} ({int(over.sum())} elements)"


def served_by_b200(op, *args):
    """Run `op` forced three ways, check that the three results are one and the same, return the outputs as a list."""
    before = ops._lib.launch_count()
    runs = [outputs(value) for value in forced_three_ways(op, *args)]
    assert ops._lib.launch_count() >= before + 3, f"{op.name}: no kernel of the library was launched"
    for other in runs[1:]:
        for a, b in zip(runs[0], other):
            assert torch.equal(a, b), f"{op.name}: forcing forms disagree"
    return runs[0]


# ------------------------------------------------------------------ the five configurations, forced --

def test_config1_rms_norm_fp32(popcorn):
    w = workloads.rms_norm_fp32().to(DEV)
    op = popcorn.KERNELS["rms_norm"]
    (y,) = served_by_b200(op, w.inputs["x"], w.inputs["weight"], None, w.args["eps"])
    close(y, op.reference(w.inputs["x"], w.inputs["weight"], None, w.args["eps"]), "rms_norm fp32")


def test_config2_add_rms_norm_bf16(popcorn):
    w = workloads.add_rms_norm_bf16(scale=0.5).to(DEV)
    op = popcorn.KERNELS["add_rms_norm"]
    args = (w.inputs["x"], w.inputs["residual"], w.inputs["weight"], w.args["eps"], w.args["offset"])
    y, s = served_by_b200(op, *args)
    want_y, want_s = op.reference(*args)
    assert torch.equal(s, want_s), "add_rms_norm: the residual stream is not bit-identical"
    close(y, want_y, "add_rms_norm bf16", row_sums=True)


def test_config3_rotary_bf16(popcorn):
    w = workloads.rotary_bf16(scale=0.25).to(DEV)
    op = popcorn.KERNELS["rotary_embedding"]
    for name in ("q", "k"):
        args = (w.inputs[name], w.inputs["cos"], w.inputs["sin"], False)
        (y,) = served_by_b200(op, *args)
        want = op.reference(*args)
        close(y, want, f"rotary_embedding {name}")
        assert float((y == want).double().mean()) >= 0.9999, f"rotary_embedding {name}: not (almost) bit-identical"


def test_config4_swiglu_bf16(popcorn):
    w = workloads.swiglu_bf16(scale=0.25).to(DEV)
    cols = w.args["cols"]
    a, b = w.inputs["gate_up"][:, :cols], w.inputs["gate_up"][:, cols:]  # strided halves of one buffer
    op = popcorn.KERNELS["swiglu"]
    (y,) = served_by_b200(op, a, b)
    close(y, op.reference(a, b), "swiglu bf16")


def test_config5_moe_steps(popcorn):
    w = workloads.moe_bf16(scale=0.25).to(DEV)
    x, logits, experts, top_k = w.inputs["x"], w.inputs["router_logits"], w.args["experts"], w.args["top_k"]
    route, permute, unpermute = (popcorn.KERNELS[n] for n in ("moe_route", "moe_permute", "moe_unpermute"))
    indices, weights = served_by_b200(route, logits, top_k)
    want_indices, want_weights = route.reference(logits, top_k)
    assert torch.equal(indices, want_indices), "moe_route: expert indices differ"
    close(weights, want_weights, "moe_route weights")
    got = served_by_b200(permute, x, indices, experts)
    want = permute.reference(x, indices, experts)
    for name, g, t in zip(("rows", "counts", "offsets", "perm", "pos"), got, want):
        assert g.dtype == t.dtype and torch.equal(g, t), f"moe_permute: {name} differs"
    (y,) = served_by_b200(unpermute, got[0], weights, got[4])
    close(y, unpermute.reference(got[0], weights, got[4]), "moe_unpermute")


def test_training_calls_go_through_the_dispatcher(popcorn):
    """Inputs that require grad reach the differentiable sources; gradients against autograd through the reference."""
    gen = torch.Generator().manual_seed(71)
    x = torch.randn(256, 2048, generator=gen).to(BF16).to(DEV).requires_grad_()
    weight = (1 + 0.1 * torch.randn(2048, generator=gen)).to(BF16).to(DEV).requires_grad_()
    cotangent = torch.randn(256, 2048, generator=gen).to(BF16).to(DEV)
    op = popcorn.KERNELS["rms_norm"]
    assert not op["b200"].forward_only
    ours = torch.autograd.grad(op(x, weight, None, 1e-6, backend="b200"), (x, weight), cotangent)
    theirs = torch.autograd.grad(op.reference(x, weight, None, 1e-6), (x, weight), cotangent)
    xd, wd = x.detach().double().requires_grad_(), weight.detach().double().requires_grad_()
    truth = torch.autograd.grad(op.reference(xd, wd, None, 1e-6), (xd, wd), cotangent.double())
    for name, mine, ref, exact in zip(("x", "weight"), ours, theirs, truth):
        # popcorn's own rule: no further from fp64 than twice the reference's own distance, or the dtype's floor
        err, budget = float((mine.double() - exact).abs().max()), float((ref.double() - exact).abs().max())
        assert err <= max(2 * budget, 2e-2 * float(exact.abs().max())), f"grad {name}: {err} against a budget of {budget}"


# ------------------------------------------------------------------ calls the kernels do not take --

def test_declined_calls_fall_through_to_another_backend(popcorn):
    """The references promote mixed dtypes and take any stride; the kernels do not.  Those calls must be vetoed by the
    predicate (so that an unforced call is served by another backend and a forced one gets popcorn's DispatchError),
    never reach the op and raise from inside it."""
    DispatchError = popcorn.core.errors.DispatchError
    x = torch.randn(8, 256, device=DEV, dtype=BF16)
    w32 = torch.ones(256, device=DEV)
    cases = [
        ("rms_norm", (x, w32, None, 1e-6)),                                   # fp32 weight on bf16 activations
        ("add_rms_norm", (x, x, w32, 1e-6, 0.0)),
        ("swiglu", (x, x.float())),
        ("rotary_embedding", (torch.randn(2, 16, 64, 4, device=DEV, dtype=BF16).transpose(2, 3),     # head_dim strided
                              torch.ones(16, 32, device=DEV), torch.zeros(16, 32, device=DEV), False)),
        ("moe_route", (torch.randn(4, 2048, device=DEV), 2)),                 # more experts than the kernel's limit
        ("moe_route", (torch.randn(4, 64, device=DEV), 40)),                  # top_k beyond the kernel's limit
    ]
    for name, args in cases:
        op = popcorn.KERNELS[name]
        bound = op._bind(*args)
        assert plugin.declined(name, **bound) is not None, name
        assert op["b200"].rejects(op._values(bound), bound) is not None, name
        with pytest.raises(DispatchError, match="rejected"):
            op(*args, backend="b200")
        want = op.reference(*args)
        for got, ref in zip(outputs(op(*args)), outputs(want)):               # unforced: served, by someone else
            torch.testing.assert_close(got, ref)
    # and the direct call of the op does refuse each of them, which is what the veto mirrors
    for name, args in cases:
        with pytest.raises((TypeError, ValueError, RuntimeError)):
            getattr(ops, name)(*args)


# ------------------------------------------------------------------ popcorn's own grader and tuner --

def representable_cases():
    gen = torch.Generator().manual_seed(72)

    def t(*shape, dtype=BF16, mean=0.0, std=1.0):
        return (mean + std * torch.randn(shape, generator=gen)).to(dtype).to(DEV)

    gate_up = t(4096, 2 * 4096)
    logits = t(16384, 64, dtype=F32)
    half = torch.cos(torch.randn(1, 512, 64, generator=gen))
    return [
        ("rms_norm", (t(4096, 4096, dtype=F32), t(4096, dtype=F32, mean=1.0, std=0.02), None, 1e-6)),
        ("rms_norm", (t(4096, 4096), t(4096, mean=1.0, std=0.1), None, 1e-6)),
        ("add_rms_norm", (t(4096, 8192), t(4096, 8192), t(8192, mean=1.0, std=0.1), 1e-5, 0.0)),
        ("swiglu", (gate_up[:, :4096], gate_up[:, 4096:])),
        ("rope", (t(4, 16, 512, 128), t(4, 4, 512, 128), half.repeat(1, 1, 2).to(BF16).to(DEV), (1 - half * half).sqrt().repeat(1, 1, 2).to(BF16).to(DEV))),
        ("layer_norm", (t(4096, 4096), t(4096, mean=1.0, std=0.1), t(4096, std=0.1), 1e-6)),
        ("l2_norm", (t(8192, 2048), 1e-6)),
        ("geglu", (gate_up[:, :4096], gate_up[:, 4096:])),
        ("rms_norm_gated", (t(4096, 4096), t(4096, 4096), t(4096, mean=1.0, std=0.1), None, "swish", 1e-6)),
        ("moe_route", (logits, 8)),
        ("moe_permute", (t(16384, 2048), ops.moe_route(logits, 8)[0], 64)),
    ]


def test_popcorns_grader_passes_the_backend_and_its_tuner_then_selects_it(popcorn):
    graded = []
    for name, args in representable_cases():
        op = popcorn.KERNELS[name]
        with torch.no_grad():
            records = op.benchmark(*args, backend="b200")                     # compare_inputs + do_bench + store.write_user
        assert [r.impl for r in records] == ["b200"], name
        result = records[0].result
        assert result.status == "pass", f"{name}: popcorn graded the backend {result.status}: {result.reason}"
        assert result.benchmarked and result.bench.get("fwd_ms") and result.bench.get("ref_fwd_ms"), (name, result.bench_error)
        assert result.fwd, f"{name}: no output was graded"
        graded.append((name, args, result))
    # the rows are in popcorn's own per-user store, written by popcorn
    from popcorn.bench.store import user_reports

    directory = user_reports()
    assert str(directory).startswith(os.environ["POPCORN_CACHE_DIR"])
    for name in {name for name, _, _ in graded}:
        rows = [json.loads(line) for line in (directory / f"{name}.jsonl").read_text().splitlines() if line.strip()]
        assert any(row["impl"] == "b200" and row["status"] == "pass" and row["benchmarked"] for row in rows), name
    # an unforced call is now decided by the tuner from those rows: b200 wherever it measured faster than the reference
    for name, args, result in graded:
        op = popcorn.KERNELS[name]
        with torch.no_grad():
            bound = op._bind(*args)
            values = op._values(bound)
            call = popcorn.core.config.call_config(op, values, bound)
            chosen = op.tuner.select(call, op._eligible(values, bound), None, op._cache_signature(bound), op.tuner.policy.bind(None))
            faster = result.bench["fwd_ms"] * (1 + op.tuner.policy.indifference) < result.bench["ref_fwd_ms"]
            assert chosen.name == ("b200" if faster else chosen.name), f"{name}: tuner chose {chosen.name} with {result.bench}"
            assert faster, f"{name}: b200 {result.bench['fwd_ms']} ms is not faster than the reference's {result.bench['ref_fwd_ms']} ms"
            before = ops._lib.launch_count()
            got = op(*args)                                                   # no backend=, no scope
            assert ops._lib.launch_count() > before, f"{name}: the unforced call did not run the b200 kernels"
            for g, r in zip(outputs(got), outputs(op.reference(*args))):
                close(g, r, f"{name} (auto-selected)", row_sums="norm" in name)


def test_popcorns_grader_on_the_calls_it_cannot_store(popcorn):
    """Mixed float dtypes (bf16 activations, fp32 tables) and the integer-indexed MoE steps: graded by compare_inputs
    directly, the function `op.benchmark` hands every case to."""
    from popcorn.bench.compare import compare_inputs

    w = workloads.rotary_bf16(scale=0.125).to(DEV)
    m = workloads.moe_bf16(scale=1 / 16).to(DEV)
    indices, weights = ops.moe_route(m.inputs["router_logits"], m.args["top_k"])
    rows, _, _, _, pos = ops.moe_permute(m.inputs["x"], indices, m.args["experts"])
    cases = [
        ("rotary_embedding", dict(x=w.inputs["q"], cos=w.inputs["cos"], sin=w.inputs["sin"], interleaved=False)),
        ("rotary_embedding", dict(x=w.inputs["k"], cos=w.inputs["cos"], sin=w.inputs["sin"], interleaved=True)),
        ("moe_route", dict(router_logits=m.inputs["router_logits"], top_k=m.args["top_k"])),
        ("moe_permute", dict(x=m.inputs["x"], indices=indices, experts=m.args["experts"])),
        ("moe_unpermute", dict(rows=rows, weights=weights, pos=pos)),
    ]
    for name, inputs in cases:
        op = popcorn.KERNELS[name]
        with torch.no_grad():
            result = compare_inputs(lambda **kwargs: op["b200"].invoke(kwargs), op.reference, [inputs], backward=False, benchmark=False)
        assert result.status == "pass", f"{name}: {result.status}: {result.reason}"
