"""The CPU oracle against golden vectors produced by the real popcorn references.

The fixtures were written by tests/golden/make_golden.py, which imports popcorn
and calls KERNELS[op].reference on CPU.  Floating-point outputs must agree to
within one unit in the last place of the output dtype (they are bit-identical on
the machine that generated them; a host with another SIMD width may order the
row sums of the norms differently); integer outputs must be equal.
"""

import pytest
import torch

from oracle import reference_ops as oracle
from tests.golden.golden_io import case_names, load_case

ULP = {torch.float32: 2.0**-23, torch.float16: 2.0**-10, torch.bfloat16: 2.0**-7}


def assert_close_ulps(got, want, ulps=1.0):
    assert got.dtype == want.dtype and got.shape == want.shape
    g, w = got.double(), want.double()
    tol = ulps * ULP[want.dtype] * w.abs().clamp_min(2.0**-20)
    bad = (g - w).abs() > tol
    assert not bad.any(), f"{int(bad.sum())} of {bad.numel()} elements differ by more than {ulps} ulp"


def names(prefix):
    found = [n for n in case_names() if n.startswith(prefix)]
    assert found, f"no golden case named {prefix}*"
    return found


@pytest.mark.parametrize("name", names("rms_norm"))
def test_rms_norm(name):
    t, meta = load_case(name)
    assert_close_ulps(oracle.rms_norm(t["x"], t["weight"], t.get("bias"), meta["eps"]), t["y"])


@pytest.mark.parametrize("name", names("add_rms_norm"))
def test_add_rms_norm(name):
    t, meta = load_case(name)
    y, s = oracle.add_rms_norm(t["x"], t["residual"], t["weight"], meta["eps"], meta["offset"])
    assert torch.equal(s, t["s"])
    assert_close_ulps(y, t["y"])


@pytest.mark.parametrize("name", names("rope"))
def test_rotary_embedding(name):
    t, meta = load_case(name)
    assert torch.equal(oracle.rotary_embedding(t["x"], t["cos"], t["sin"], meta["interleaved"]), t["y"])


@pytest.mark.parametrize("name", names("pairedrope"))
def test_paired_rope(name):
    t, _ = load_case(name)
    yq, yk = oracle.rope(t["q"], t["k"], t["cos"], t["sin"])
    assert torch.equal(yq, t["yq"]) and torch.equal(yk, t["yk"])


@pytest.mark.parametrize("name", names("qknormrope"))
def test_qk_norm_rope(name):
    t, meta = load_case(name)
    yq, yk = oracle.qk_norm_rope(t["q"], t["k"], t["q_weight"], t["k_weight"], t["cos"], t["sin"], meta["eps"])
    assert torch.equal(yq, t["yq"]) and torch.equal(yk, t["yk"])


@pytest.mark.parametrize("name", names("llama4rope"))
def test_llama4_rope(name):
    t, _ = load_case(name)
    yq, yk = oracle.llama4_rope(t["q"], t["k"], t["freqs"])
    assert torch.equal(yq, t["yq"]) and torch.equal(yk, t["yk"])


@pytest.mark.parametrize("name", names("swiglu"))
def test_swiglu(name):
    t, _ = load_case(name)
    cols = t["gate_up"].shape[1] // 2
    assert_close_ulps(oracle.swiglu(t["gate_up"][:, :cols], t["gate_up"][:, cols:]), t["y"])


@pytest.mark.parametrize("name", names("geglu"))
def test_geglu(name):
    t, _ = load_case(name)
    cols = t["gate_up"].shape[1] // 2
    assert_close_ulps(oracle.geglu(t["gate_up"][:, :cols], t["gate_up"][:, cols:]), t["y"])


@pytest.mark.parametrize("name", names("rmsgated"))
def test_rms_norm_gated(name):
    t, meta = load_case(name)
    assert_close_ulps(oracle.rms_norm_gated(t["x"], t["g"], t["weight"], t.get("bias"), meta["activation"], meta["eps"]), t["y"])


@pytest.mark.parametrize("name", names("l2norm"))
def test_l2_norm(name):
    t, meta = load_case(name)
    assert_close_ulps(oracle.l2_norm(t["x"], meta["eps"]), t["y"])


@pytest.mark.parametrize("name", names("layernorm"))
def test_layer_norm(name):
    t, meta = load_case(name)
    assert_close_ulps(oracle.layer_norm(t["x"], t["weight"], t.get("bias"), meta["eps"]), t["y"])


@pytest.mark.parametrize("name", names("momoe"))
def test_route(name):
    t, meta = load_case(name)
    logits = t["router_logits"]
    assert oracle.route_is_unambiguous(logits, meta["top_k"])
    indices, weights = oracle.moe_route(logits, meta["top_k"])
    assert torch.equal(indices, t["topk_indices"])
    assert_close_ulps(weights, t["topk_weights"], ulps=2)


@pytest.mark.parametrize("name", names("momoe"))
def test_route_permute_unpermute_chain_reproduces_momoe(name):
    """route -> permute -> expert MLPs -> unpermute equals the registered momoe reference."""
    t, meta = load_case(name)
    y = oracle.momoe_from_steps(t["x"], t["gate_weight"], t["up_weight"], t["down_weight"], t["router_logits"], meta["top_k"])
    # fp32 matmuls summed in a different order than the reference's einsum
    torch.testing.assert_close(y, t["y"], rtol=1e-4, atol=1e-5)


def test_index_is_a_stable_sort_by_expert():
    gen = torch.Generator().manual_seed(7)
    tokens, top_k, experts = 97, 4, 11
    indices = torch.stack([torch.randperm(experts, generator=gen)[:top_k] for _ in range(tokens)]).to(torch.int32)
    counts, offsets, perm, pos = oracle.moe_index(indices, experts)
    assert int(counts.sum()) == tokens * top_k and int(offsets[-1]) == tokens * top_k
    assert torch.equal(offsets[1:] - offsets[:-1], counts)
    flat = indices.reshape(-1)
    for e in range(experts):
        lo, hi = int(offsets[e]), int(offsets[e + 1])
        expect = torch.nonzero((indices == e).any(dim=1)).reshape(-1).to(torch.int32)
        assert torch.equal(perm[lo:hi], expect)  # ascending token ids: the reference's col_idx
    assert torch.equal(perm[pos.reshape(-1).long()], torch.arange(tokens).repeat_interleave(top_k).to(torch.int32))
    assert torch.equal(flat[(pos.reshape(-1).argsort())], flat.sort(stable=True).values)


def sha256(t):
    import hashlib

    return hashlib.sha256(t.contiguous().numpy().tobytes()).hexdigest()


@pytest.mark.parametrize("name", names("moeindex_"))
def test_index_equals_the_references_own_kernel(name):
    """counts / cumsums / col_idx written by the reference's find_used_experts + scatter_cols_kernel
    (src/popcorn/impls/momoe_tl.py:1071-1161) on a GPU, fixtures made by tests/golden/make_moe_index_golden.py."""
    t, meta = load_case(name)
    if "topk_indices" in t:
        if "router_logits" in t:
            routed, _ = oracle.moe_route(t["router_logits"], meta["top_k"])
            assert torch.equal(routed, t["topk_indices"])
        indices = t["topk_indices"]
    else:  # the full-size configuration: inputs from the seed, long outputs kept as digests
        from popcorn_b200 import workloads

        w = workloads.moe_bf16()
        indices, _ = oracle.moe_route(w.inputs["router_logits"], meta["top_k"])
        assert sha256(indices) == meta["topk_indices_sha256"]
    counts, offsets, perm, pos = oracle.moe_index(indices, meta["experts"])
    assert torch.equal(counts, t["counts"]) and torch.equal(offsets, t["cumsums"])
    if "col_idx" in t:
        assert torch.equal(perm, t["col_idx"])
    else:
        edge = t["col_idx_head"].numel()
        assert torch.equal(perm[:edge], t["col_idx_head"]) and torch.equal(perm[-edge:], t["col_idx_tail"])
        assert sha256(perm) == meta["col_idx_sha256"]


def test_unpermute_matches_einsum():
    """The fixed summation order stays within fp32 rounding of the reference's einsum (momoe.py:53)."""
    gen = torch.Generator().manual_seed(8)
    tokens, top_k, experts, hidden = 50, 3, 6, 24
    x = torch.randn(tokens, hidden, generator=gen)
    logits = torch.randn(tokens, experts, generator=gen)
    indices, weights = oracle.moe_route(logits, top_k)
    rows, _, _, _, pos = oracle.moe_permute(x, indices, experts)
    rows = rows * 1.5
    y = oracle.moe_unpermute(rows, weights, pos)
    dense = torch.zeros(tokens, experts, hidden)
    gates = torch.zeros(tokens, experts)
    for t in range(tokens):
        for k in range(top_k):
            dense[t, indices[t, k]] = rows[pos[t, k]]
            gates[t, indices[t, k]] = weights[t, k]
    torch.testing.assert_close(y, torch.einsum("ted,te->td", dense, gates), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("name", names("moe16"))
def test_moe16_chain_with_expert_projections(name):
    """16-bit momoe cases: the chain with the grouped expert projections (whose intermediate and expert
    outputs are rounded to the 16-bit type, as the incumbent kernels do) stays within the 16-bit bound of
    the registered reference, which keeps fp32 throughout."""
    t, meta = load_case(name)
    top_k = meta["top_k"]
    experts = t["gate_weight"].shape[0]
    x = t["x"].reshape(-1, t["x"].shape[-1])
    indices, weights = oracle.moe_route(t["router_logits"].reshape(-1, experts), top_k)
    assert torch.equal(indices, t["topk_indices"].reshape(-1, top_k))
    rows, _, offsets, _, pos = oracle.moe_permute(x, indices, experts)
    hidden_act = oracle.moe_grouped_gemm(rows, t["gate_weight"], offsets, t["up_weight"])
    out_rows = oracle.moe_grouped_gemm(hidden_act, t["down_weight"], offsets)
    y = oracle.moe_unpermute(out_rows, weights, pos).reshape(t["y"].shape)
    assert y.dtype == t["y"].dtype
    assert float((y.float() - t["y"].float()).abs().max()) <= 2e-2
    exact = oracle.momoe_from_steps(t["x"], t["gate_weight"], t["up_weight"], t["down_weight"], t["router_logits"], top_k)
    assert float((exact.float() - t["y"].float()).abs().max()) <= 2e-2 and float((exact == t["y"]).float().mean()) > 0.99


def _oracle_call(op, t, meta):
    """The oracle's restatement of `op` on the tensors of a gradient fixture (leaves given by name)."""
    if op == "rms_norm":
        return lambda x, weight, bias: oracle.rms_norm(x, weight, bias, meta["eps"])
    if op == "add_rms_norm":
        return lambda x, residual, weight: oracle.add_rms_norm(x, residual, weight, meta["eps"], meta["offset"])
    if op == "swiglu":
        return oracle.swiglu
    return lambda x, gate_weight, up_weight, down_weight, router_logits: oracle.momoe_from_steps(
        x, gate_weight, up_weight, down_weight, router_logits, meta["top_k"])


@pytest.mark.parametrize("name", names("grad_"))
def test_autograd_through_the_oracle_gives_the_references_gradients(name):
    """The backward kernels are checked against autograd through the oracle; this pins that autograd to the gradients
    the real references produce (fixtures: autograd through KERNELS[op].reference in the case dtype and in fp64)."""
    t, meta = load_case(name)
    leaves = {k: v.clone().requires_grad_() for k, v in t.items() if f"grad_{k}" in t}
    outs = _oracle_call(meta["op"], t, meta)(*leaves.values())
    outs = outs if isinstance(outs, tuple) else (outs,)
    seeds = [t[f"cotangent{i}"] for i in range(len(outs))]
    grads = torch.autograd.grad(outs, list(leaves.values()), seeds)
    for key, got in zip(leaves, grads):
        want, truth = t[f"grad_{key}"], t[f"truth_{key}"]
        if meta["op"] == "momoe":
            # the oracle evaluates the routed pairs only and sums them in another order than the dense reference
            budget = float((want.double() - truth).abs().max())
            err = float((got.double() - truth).abs().max())
            floor = (2e-2 if got.dtype != torch.float32 else 2e-5) * max(1.0, float(truth.abs().max()))
            assert err <= max(2 * budget, floor), f"{name} grad {key}: {err:.3e} vs the reference's own {budget:.3e}"
        else:
            assert_close_ulps(got, want, 1.0)
