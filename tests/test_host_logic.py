"""Host-side behaviour that needs no GPU: the registry mirror, the popcorn plugin, input checks."""

import pytest
import torch

from tests import popcorn_location
from popcorn_b200 import kernels, ops, registry, workloads


def test_ops_refuse_cpu_tensors():
    x = torch.randn(4, 8)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        ops.rms_norm(x, torch.ones(8))
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        ops.swiglu(x, x)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        ops.moe_route(x, 2)


def test_missing_library_is_an_import_error(monkeypatch, tmp_path):
    from popcorn_b200 import _lib

    _lib.library.cache_clear()
    monkeypatch.setattr(_lib, "LIBRARY_PATH", tmp_path / "nope.so")
    with pytest.raises(ImportError, match="popcorn_b200.build"):
        _lib.library()
    _lib.library.cache_clear()


def test_rows_view_keeps_strided_halves_in_place():
    gate_up = torch.zeros(6, 32)
    a, lda = ops._rows(gate_up[:, :16])
    b, ldb = ops._rows(gate_up[:, 16:])
    assert lda == ldb == 32 and a.data_ptr() == gate_up.data_ptr() and b.data_ptr() == gate_up.data_ptr() + 16 * 4
    flat, ld = ops._rows(torch.zeros(2, 3, 8))
    assert flat.shape == (6, 8) and ld == 8
    copied, ld = ops._rows(torch.zeros(4, 8, 3).transpose(1, 2))  # last dim not contiguous -> packed copy
    assert copied.is_contiguous() and ld == 8


def test_mirror_registry_surface():
    assert set(registry.KERNELS) >= {"rms_norm", "add_rms_norm", "rotary_embedding", "rope", "swiglu", "geglu", "rms_norm_gated", "l2_norm",
                                     "layer_norm", "moe_route", "moe_permute", "moe_unpermute"}
    op = kernels.rms_norm
    assert op.available_backends() == ("b200",)
    assert op.params == ("x", "weight", "bias", "eps")
    with pytest.raises(registry.DispatchError, match="unknown backend"):
        op["fla"]
    with pytest.raises(ValueError, match="already registered"):
        op.register("b200", source="popcorn_b200.ops.rms_norm")
    with pytest.raises(ValueError, match="invalid backend name"):
        op.register("Not Valid")


def test_mirror_dispatch_forced_scoped_and_ordered():
    calls = []

    @registry.register_kernel(name="_test_scale")
    def scale(x, factor=2.0):
        """Multiply."""

    try:
        scale.register("first")(lambda x, factor: calls.append("first") or x * factor)
        scale.register("second", predicate=lambda **kw: kw["factor"] != 3.0)(lambda x, factor: calls.append("second") or x * factor)
        x = torch.ones(2)
        assert torch.equal(scale(x), x * 2) and calls == ["first"]
        assert torch.equal(scale(x, backend="second"), x * 2) and calls[-1] == "second"
        assert torch.equal(scale["second"](x, 4.0), x * 4) and calls[-1] == "second"
        with scale["second"] as scoped:
            scoped(x)
            assert calls[-1] == "second"
        scale(x)
        assert calls[-1] == "first"
        with pytest.raises(registry.DispatchError, match="rejected call"):
            scale(x, 3.0, backend="second")
        with pytest.raises(TypeError, match="parameters must be exactly"):
            scale.register("bad")(lambda x: x)
        assert "bad" not in scale.available_backends()
    finally:
        del registry.KERNELS["_test_scale"]


def test_forward_only_backend_declines_grad():
    @registry.register_kernel(name="_test_forward_only")
    def double(x):
        """Twice x."""

    try:
        double.register("b200", forward_only=True)(lambda x: x * 2)
        x = torch.ones(8, requires_grad=True)
        with pytest.raises(registry.DispatchError, match="no backward implementation"):
            double(x, backend="b200")
        with pytest.raises(registry.DispatchError, match="no registered backend"):
            double(x)
        assert torch.equal(double(x.detach()), torch.full((8,), 2.0))
    finally:
        del registry.KERNELS["_test_forward_only"]
    # every op of the backend has backward kernels and serves training calls
    for name in ("rms_norm", "add_rms_norm", "swiglu", "geglu", "rotary_embedding", "rope", "llama4_rope", "qk_norm_rope", "l2_norm", "layer_norm",
                 "rms_norm_gated", "moe_route", "moe_permute", "moe_unpermute", "moe_grouped_gemm", "momoe"):
        assert not registry.KERNELS[name]["b200"].forward_only


def test_workload_shapes_and_bytes():
    w = workloads.add_rms_norm_bf16(scale=1 / 1024)
    assert w.inputs["x"].shape == (16, 8192) and w.inputs["x"].dtype == torch.bfloat16
    assert w.algorithmic_bytes["add_rms_norm"] == 4 * 16 * 8192 * 2 + 8192 * 2
    full = {"rms_norm_fp32": 134_234_112, "add_rms_norm_bf16": 1_073_758_208, "swiglu_bf16": 2_818_572_288}
    # byte formulas at full size, without materialising the tensors
    assert 2 * 4096 * 4096 * 4 + 4096 * 4 == full["rms_norm_fp32"]
    assert 4 * 16384 * 8192 * 2 + 8192 * 2 == full["add_rms_norm_bf16"]
    assert 3 * 32768 * 14336 * 2 == full["swiglu_bf16"]
    m = workloads.moe_bf16(scale=1 / 256)
    assert m.algorithmic_bytes["permute"] == 256 * 4096 * 2 + 2048 * 4096 * 2 + 2048 * 4
    shard = m.shard(1, 2)
    assert shard.tokens == 128 and shard.inputs["x"].shape[0] == 128
    assert torch.equal(shard.inputs["x"], m.inputs["x"][128:])
    r = workloads.rotary_bf16(scale=0.25, seq=64)
    assert r.inputs["q"].shape == (2, 64, 32, 128) and r.inputs["cos"].shape == (64, 64)
    assert r.shard(0, 2).inputs["q"].shape[0] == 1 and r.shard(0, 2).inputs["cos"].shape == (64, 64)




@pytest.mark.skipif(not popcorn_location.available(), reason=popcorn_location.MISSING)
def test_plugin_registers_on_real_popcorn(tmp_path, monkeypatch):
    popcorn = popcorn_location.import_popcorn(tmp_path, monkeypatch)

    from popcorn_b200 import plugin

    served = plugin.register()
    assert served == [*plugin.EXISTING_OPS, *plugin.NEW_OPS]
    assert plugin.register() == served  # idempotent
    for name in served:
        op = popcorn.KERNELS[name]
        assert "b200" in op.available_backends()
        assert op["b200"].forward_only == (name not in plugin.DIFFERENTIABLE_OPS)
    # existing ops keep the reference last and their other backends intact
    assert popcorn.KERNELS["swiglu"].available_backends()[-1] == "torch"
    # popcorn resolves the bare source and checks it against the reference signature
    from popcorn_b200 import autograd as differentiable

    impl = popcorn.KERNELS["add_rms_norm"]["b200"]
    impl._prepare()
    assert impl.source_fn is differentiable.add_rms_norm
    for name in ("rope", "llama4_rope", "geglu", "qk_norm_rope"):
        impl = popcorn.KERNELS[name]["b200"]
        impl._prepare()  # the bare source must accept the reference's parameters positionally
        assert impl.source_fn is getattr(differentiable, name)
    impl = popcorn.KERNELS["momoe"]["b200"]
    impl._prepare()
    assert impl.source_fn is differentiable.momoe
    # momoe is served for 16-bit activations only (tensor-core operands)
    assert not plugin.accepts_16bit(x=torch.zeros(1, 2, 8), gate_weight=torch.zeros(2, 8, 8))
    # CPU calls are declined by the predicate rather than served by a fallback
    x = torch.randn(4, 8)
    with pytest.raises(popcorn.core.errors.DispatchError, match="rejected"):
        popcorn.KERNELS["swiglu"](x, x, backend="b200")
    # unforced CPU calls still reach popcorn's own torch reference
    assert torch.equal(popcorn.KERNELS["swiglu"](x, x), torch.nn.functional.silu(x) * x)
    # the new ops' torch definitions agree with the oracle
    from oracle import reference_ops as oracle

    logits = torch.randn(32, 8, generator=torch.Generator().manual_seed(3))
    idx, w = popcorn.KERNELS["moe_route"].reference(logits, 2)
    oidx, ow = oracle.moe_route(logits, 2)
    assert torch.equal(idx, oidx) and torch.equal(w, ow)
    got = popcorn.KERNELS["moe_permute"].reference(x.repeat(8, 1), idx, 8)
    want = oracle.moe_permute(x.repeat(8, 1), oidx, 8)
    assert all(torch.equal(g, w_) for g, w_ in zip(got, want))
    y = popcorn.KERNELS["moe_unpermute"].reference(want[0], ow, want[4])
    torch.testing.assert_close(y, oracle.moe_unpermute(want[0], ow, want[4]), rtol=1e-5, atol=1e-6)


def test_host_pipeline_chunks_cover_the_rows_once():
    from popcorn_b200.host import chunk_bounds

    ramped = chunk_bounds(16384, 1024)
    assert ramped[:3] == [(0, 128), (128, 384), (384, 896)] and ramped[-1] == (16256, 16384) and len(ramped) == 21
    for rows, chunk in [(1, 1024), (1000, 1024), (4095, 1024), (4096, 1024), (4097, 1024), (5000, 7), (100000, 1000), (9, 1)]:
        bounds = chunk_bounds(rows, chunk)
        assert bounds[0][0] == 0 and bounds[-1][1] == rows
        assert all(a[1] == b[0] for a, b in zip(bounds, bounds[1:])) and all(0 < hi - lo <= chunk for lo, hi in bounds)
    assert chunk_bounds(0, 64) == []


def test_dispatch_rules_mirror_the_ops_argument_checks():
    """`plugin.RULES[op]` names a reason for every call the op itself would refuse (shape, dtype and limit checks;
    placement is `plugin.accepts`, which needs a GPU), and none for the calls it takes."""
    from popcorn_b200 import plugin

    bf16, f32 = torch.bfloat16, torch.float32
    x, w = torch.zeros(4, 64, dtype=bf16), torch.ones(64, dtype=bf16)
    taken = {
        "rms_norm": dict(x=x, weight=w, bias=None, eps=1e-6),
        "layer_norm": dict(x=x, weight=w, bias=w, eps=1e-6),
        "add_rms_norm": dict(x=x, residual=x, weight=w, eps=1e-6, offset=0.0),
        "rms_norm_gated": dict(x=x, g=x, weight=w, bias=None, activation="sigmoid", eps=1e-6),
        "l2_norm": dict(x=x, eps=1e-6),
        "swiglu": dict(a=x, b=x), "geglu": dict(a=x, b=x),
        "rotary_embedding": dict(x=torch.zeros(2, 8, 4, 64, dtype=bf16), cos=torch.zeros(8, 16), sin=torch.zeros(8, 16), interleaved=False),
        "rope": dict(q=torch.zeros(2, 4, 8, 64, dtype=bf16), k=torch.zeros(2, 1, 8, 64, dtype=bf16), cos=torch.zeros(1, 8, 64, dtype=bf16), sin=torch.zeros(1, 8, 64, dtype=bf16)),
        "qk_norm_rope": dict(q=torch.zeros(2, 4, 8, 64, dtype=bf16), k=torch.zeros(2, 1, 8, 64, dtype=bf16), q_weight=w, k_weight=w,
                             cos=torch.zeros(2, 8, 64, dtype=bf16), sin=torch.zeros(2, 8, 64, dtype=bf16), eps=1e-6),
        "llama4_rope": dict(q=torch.zeros(2, 8, 4, 64, dtype=bf16), k=torch.zeros(2, 8, 1, 64, dtype=bf16), freqs=torch.zeros(8, 32, 2, dtype=bf16)),
        "moe_route": dict(router_logits=torch.zeros(4, 64), top_k=8),
        "moe_permute": dict(x=x, indices=torch.zeros(4, 2, dtype=torch.int32), experts=8),
        "moe_unpermute": dict(rows=torch.zeros(8, 64, dtype=bf16), weights=torch.zeros(4, 2), pos=torch.zeros(4, 2, dtype=torch.int32)),
        "momoe": dict(x=torch.zeros(1, 4, 64, dtype=bf16), gate_weight=torch.zeros(8, 64, 32, dtype=bf16), up_weight=torch.zeros(8, 64, 32, dtype=bf16),
                      down_weight=torch.zeros(8, 32, 64, dtype=bf16), router_logits=torch.zeros(1, 4, 8), top_k=2),
    }
    assert set(taken) == set(plugin.RULES) == {*plugin.EXISTING_OPS, *plugin.NEW_OPS}
    for name, arguments in taken.items():
        assert plugin.RULES[name](**arguments) is None, name
    refused = [
        ("rms_norm", dict(weight=w.float())), ("rms_norm", dict(bias=w.float())), ("rms_norm", dict(weight=torch.ones(32, dtype=bf16))),
        ("layer_norm", dict(weight=w.float())), ("add_rms_norm", dict(residual=x.float())), ("add_rms_norm", dict(residual=x[:2])),
        ("rms_norm_gated", dict(activation="relu")), ("rms_norm_gated", dict(g=x.float())),
        ("swiglu", dict(b=x.float())), ("geglu", dict(b=x[:, :32])),
        ("rotary_embedding", dict(x=torch.zeros(2, 8, 64, 4, dtype=bf16).transpose(2, 3))),      # head_dim strided
        ("rotary_embedding", dict(cos=torch.zeros(8, 48), sin=torch.zeros(8, 48))),               # 2 * half > head_dim
        ("rotary_embedding", dict(cos=torch.zeros(8, 16, dtype=torch.float16), sin=torch.zeros(8, 16, dtype=torch.float16))),
        ("rotary_embedding", dict(cos=torch.zeros(1, 8, 1, 16), sin=torch.zeros(1, 8, 1, 16))),   # broadcastable, not [seq, half]
        ("rope", dict(cos=torch.zeros(1, 8, 64), sin=torch.zeros(1, 8, 64))),                     # fp32 tables on bf16 q
        ("rope", dict(k=torch.zeros(2, 1, 9, 64, dtype=bf16))),
        ("qk_norm_rope", dict(q_weight=w.float())), ("llama4_rope", dict(freqs=torch.zeros(8, 32, 2))),
        ("moe_route", dict(router_logits=torch.zeros(4, 2048))), ("moe_route", dict(top_k=40)), ("moe_route", dict(top_k=0)),
        ("moe_permute", dict(indices=torch.zeros(4, 2, dtype=torch.int64))), ("moe_permute", dict(experts=4096)),
        ("moe_unpermute", dict(weights=torch.zeros(4, 2, dtype=bf16))), ("moe_unpermute", dict(pos=torch.zeros(4, 2, dtype=torch.int64))),
        ("momoe", dict(x=torch.zeros(1, 4, 64))), ("momoe", dict(down_weight=torch.zeros(8, 32, 64))),
        ("momoe", dict(router_logits=torch.zeros(1, 4, 9))),
    ]
    for name, change in refused:
        reason = plugin.RULES[name](**{**taken[name], **change})
        assert isinstance(reason, str) and reason, (name, sorted(change))
    # on a machine without a GPU every predicate declines (placement comes first) instead of raising
    for name, arguments in taken.items():
        assert plugin.PREDICATES[name](**arguments) is False
        assert "CUDA" in plugin.declined(name, **arguments)
