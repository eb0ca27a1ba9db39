"""Generate tests/golden/*.npz by running the REAL popcorn references.

Run it where the reference source tree is available:

    PYTHONPATH=<popcorn checkout>/src python tests/golden/make_golden.py

It imports `popcorn.kernels`, draws inputs the way popcorn's own harness does
(src/popcorn/bench/grid.py:682-715: a CPU generator seeded per case, `torch.randn`
in fp32 in signature order, an optional affine transform, then a cast to the
case dtype), calls `KERNELS[op].reference(...)` on CPU and stores inputs and
outputs bit-exactly.  The committed fixtures let the oracle be checked on
machines where popcorn itself is not installed.
"""

from __future__ import annotations

import os
import sys
import tempfile
import warnings
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
from tests.golden.golden_io import save_case  # noqa: E402

os.environ.setdefault("POPCORN_CACHE_DIR", tempfile.mkdtemp(prefix="popcorn-cache-"))
warnings.filterwarnings("ignore")
import popcorn.kernels  # noqa: E402,F401
from popcorn import KERNELS  # noqa: E402

BF16, F16, F32 = torch.bfloat16, torch.float16, torch.float32


def randn(gen: torch.Generator, *shape: int) -> torch.Tensor:
    return torch.randn(shape, generator=gen)


def rms_norm_cases() -> None:
    ref = KERNELS["rms_norm"].reference
    for name, seed, rows, cols, dtype, eps, with_bias in [
        ("rms_norm_f32_5x64", 0, 5, 64, F32, 1e-6, False),
        ("rms_norm_f32_3x50_bias", 1, 3, 50, F32, 1e-5, True),
        ("rms_norm_bf16_7x264_bias", 2, 7, 264, BF16, 1e-5, True),
        ("rms_norm_bf16_4x1024", 3, 4, 1024, BF16, 1e-6, False),
        ("rms_norm_f16_3x40", 4, 3, 40, F16, 1e-6, False),
    ]:
        gen = torch.Generator().manual_seed(seed)
        x = randn(gen, rows, cols).to(dtype)
        weight = (1 + 0.1 * randn(gen, cols)).to(dtype)
        bias = randn(gen, cols).to(dtype) if with_bias else None
        y = ref(x, weight, bias, eps)
        tensors = {"x": x, "weight": weight, "y": y}
        if bias is not None:
            tensors["bias"] = bias
        save_case(name, tensors, {"op": "rms_norm", "eps": eps})


def add_rms_norm_cases() -> None:
    ref = KERNELS["add_rms_norm"].reference
    for name, seed, rows, cols, dtype, eps, offset in [
        ("add_rms_norm_bf16_6x256", 10, 6, 256, BF16, 1e-5, 0.0),
        ("add_rms_norm_bf16_4x72_offset1", 11, 4, 72, BF16, 1e-6, 1.0),
        ("add_rms_norm_f32_3x50", 12, 3, 50, F32, 1e-6, 0.0),
        ("add_rms_norm_f16_5x128_offset1", 13, 5, 128, F16, 1e-5, 1.0),
        ("add_rms_norm_bf16_2x8192", 14, 2, 8192, BF16, 1e-5, 0.0),
    ]:
        gen = torch.Generator().manual_seed(seed)
        x = randn(gen, rows, cols).to(dtype)
        residual = randn(gen, rows, cols).to(dtype)
        weight = (1 + 0.1 * randn(gen, cols)).to(dtype)
        y, s = ref(x, residual, weight, eps, offset)
        save_case(name, {"x": x, "residual": residual, "weight": weight, "y": y, "s": s},
                  {"op": "add_rms_norm", "eps": eps, "offset": offset})


def rope_tables(seq: int, half: int, theta: float = 500000.0) -> tuple[torch.Tensor, torch.Tensor]:
    inv = theta ** (-torch.arange(0, 2 * half, 2, dtype=torch.float32) / (2 * half))
    ang = torch.outer(torch.arange(seq, dtype=torch.float32), inv)
    return ang.cos(), ang.sin()


def rotary_cases() -> None:
    ref = KERNELS["rotary_embedding"].reference
    for name, seed, shape, half, dtype, cs_dtype, interleaved in [
        ("rope_bf16_neox_2x16x4x64", 20, (2, 16, 4, 64), 32, BF16, F32, False),
        ("rope_bf16_neox_partial_1x8x2x64_h16", 21, (1, 8, 2, 64), 16, BF16, F32, False),
        ("rope_bf16_gptj_2x8x3x32", 22, (2, 8, 3, 32), 16, BF16, F32, True),
        ("rope_f32_neox_1x8x2x16", 23, (1, 8, 2, 16), 8, F32, F32, False),
        ("rope_f16_neox_cs16_2x4x2x32", 24, (2, 4, 2, 32), 16, F16, F16, False),
        ("rope_bf16_neox_odd_1x5x3x20_h5", 25, (1, 5, 3, 20), 5, BF16, F32, False),
        ("rope_bf16_neox_2x8x8x128", 26, (2, 8, 8, 128), 64, BF16, F32, False),
    ]:
        gen = torch.Generator().manual_seed(seed)
        x = randn(gen, *shape).to(dtype)
        cos, sin = rope_tables(shape[1], half)
        cos, sin = cos.to(cs_dtype), sin.to(cs_dtype)
        y = ref(x, cos, sin, interleaved)
        save_case(name, {"x": x, "cos": cos, "sin": sin, "y": y}, {"op": "rotary_embedding", "interleaved": interleaved})


def paired_rope_cases() -> None:
    ref = KERNELS["rope"].reference
    for name, seed, batch, hq, hk, seq, dim, dtype, cos_batch in [
        ("pairedrope_bf16_2x4x2x16x64", 50, 2, 4, 2, 16, 64, BF16, 1),
        ("pairedrope_bf16_2x8x2x8x128_cb2", 51, 2, 8, 2, 8, 128, BF16, 2),
        ("pairedrope_f32_1x2x1x8x16", 52, 1, 2, 1, 8, 16, F32, 1),
        ("pairedrope_f16_2x3x1x5x20", 53, 2, 3, 1, 5, 20, F16, 1),
    ]:
        gen = torch.Generator().manual_seed(seed)
        q = randn(gen, batch, hq, seq, dim).to(dtype)
        k = randn(gen, batch, hk, seq, dim).to(dtype)
        # the reference's test inputs: cos / sin of a random angle table whose first half is repeated (rope.py:13-14)
        cos = torch.cos(randn(gen, cos_batch, seq, dim)).chunk(2, -1)[0].repeat(1, 1, 2).to(dtype)
        sin = torch.sin(randn(gen, cos_batch, seq, dim)).chunk(2, -1)[0].repeat(1, 1, 2).to(dtype)
        yq, yk = ref(q, k, cos, sin)
        save_case(name, {"q": q, "k": k, "cos": cos, "sin": sin, "yq": yq, "yk": yk}, {"op": "rope"})


def notebook_qk_norm_rope():
    """The reference of the fused op the kernel-writing notebook defines (examples/03_write_a_kernel.ipynb,
    the code cell that registers `qk_norm_rope`), executed from the notebook as it stands."""
    import json

    import popcorn

    notebook = Path(popcorn.__file__).resolve().parents[2] / "examples" / "03_write_a_kernel.ipynb"
    cells = json.loads(notebook.read_text())["cells"]
    source = next("".join(c["source"]) for c in cells if c["cell_type"] == "code" and "def qk_norm_rope(" in "".join(c["source"]))
    from jaxtyping import Float
    from popcorn import Tag, register_kernel
    from popcorn.kernels._utils import rms

    scope = {"torch": torch, "Tensor": torch.Tensor, "Float": Float, "KERNELS": KERNELS, "Tag": Tag,
             "register_kernel": register_kernel, "rms": rms}
    exec(compile(source, str(notebook), "exec", dont_inherit=True), scope)
    return scope["qk_norm_rope"].reference


def qk_norm_rope_cases() -> None:
    ref = notebook_qk_norm_rope()
    for name, seed, batch, hq, hk, seq, dim, dtype, cos_batch, eps in [
        ("qknormrope_bf16_2x4x2x16x128", 60, 2, 4, 2, 16, 128, BF16, 1, 1e-6),
        ("qknormrope_bf16_2x8x2x8x64_cb2", 61, 2, 8, 2, 8, 64, BF16, 2, 1e-5),
        ("qknormrope_f32_1x2x1x8x16", 62, 1, 2, 1, 8, 16, F32, 1, 1e-6),
        ("qknormrope_f16_2x3x1x5x20", 63, 2, 3, 1, 5, 20, F16, 1, 1e-6),
    ]:
        gen = torch.Generator().manual_seed(seed)
        q = randn(gen, batch, hq, seq, dim).to(dtype)
        k = randn(gen, batch, hk, seq, dim).to(dtype)
        q_weight = randn(gen, dim).to(dtype)
        k_weight = randn(gen, dim).to(dtype)
        # the notebook's test tables: first half repeated, like a real rope cache (cell 3, `_table`)
        cos = torch.cos(randn(gen, cos_batch, seq, dim)).chunk(2, -1)[0].repeat(1, 1, 2).to(dtype)
        sin = torch.sin(randn(gen, cos_batch, seq, dim)).chunk(2, -1)[0].repeat(1, 1, 2).to(dtype)
        yq, yk = ref(q, k, q_weight, k_weight, cos, sin, eps)
        save_case(name, {"q": q, "k": k, "q_weight": q_weight, "k_weight": k_weight, "cos": cos, "sin": sin, "yq": yq, "yk": yk},
                  {"op": "qk_norm_rope", "eps": eps})


def llama4_rope_cases() -> None:
    ref = KERNELS["llama4_rope"].reference
    for name, seed, batch, seq, hq, hk, dim, dtype in [
        ("llama4rope_bf16_2x16x4x2x64", 70, 2, 16, 4, 2, 64, BF16),
        ("llama4rope_bf16_1x8x8x2x128", 71, 1, 8, 8, 2, 128, BF16),
        ("llama4rope_f32_2x8x2x1x16", 72, 2, 8, 2, 1, 16, F32),
        ("llama4rope_f16_2x5x3x1x20", 73, 2, 5, 3, 1, 20, F16),
    ]:
        gen = torch.Generator().manual_seed(seed)
        q = randn(gen, batch, seq, hq, dim).to(dtype)
        k = randn(gen, batch, seq, hk, dim).to(dtype)
        # the reference's test inputs: unit (cos, sin) pairs of a random angle (llama4_rope.py:9-11)
        angles = randn(gen, seq, dim // 2, 2)[..., 0]
        freqs = torch.stack((angles.cos(), angles.sin()), -1).to(dtype)
        yq, yk = ref(q, k, freqs)
        save_case(name, {"q": q, "k": k, "freqs": freqs, "yq": yq, "yk": yk}, {"op": "llama4_rope"})


def swiglu_cases() -> None:
    ref = KERNELS["swiglu"].reference
    for name, seed, rows, cols, dtype, scale in [
        ("swiglu_bf16_9x136", 30, 9, 136, BF16, 1.0),
        ("swiglu_bf16_4x1024_wide", 31, 4, 1024, BF16, 4.0),
        ("swiglu_f32_5x33", 32, 5, 33, F32, 1.0),
        ("swiglu_f16_6x72", 33, 6, 72, F16, 2.0),
    ]:
        gen = torch.Generator().manual_seed(seed)
        gate_up = (scale * randn(gen, rows, 2 * cols)).to(dtype)
        a, b = gate_up[:, :cols], gate_up[:, cols:]
        save_case(name, {"gate_up": gate_up, "y": ref(a, b)}, {"op": "swiglu"})


def sibling_cases() -> None:
    for name, seed, rows, cols, dtype, scale in [("geglu_bf16_9x136", 60, 9, 136, BF16, 1.5), ("geglu_f32_5x33", 61, 5, 33, F32, 1.0), ("geglu_f16_6x72", 62, 6, 72, F16, 2.0)]:
        gen = torch.Generator().manual_seed(seed)
        gate_up = (scale * randn(gen, rows, 2 * cols)).to(dtype)
        save_case(name, {"gate_up": gate_up, "y": KERNELS["geglu"].reference(gate_up[:, :cols], gate_up[:, cols:])}, {"op": "geglu"})
    for name, seed, rows, cols, dtype, with_bias, activation, eps in [
        ("rmsgated_bf16_6x256_swish", 70, 6, 256, BF16, False, "swish", 1e-6),
        ("rmsgated_bf16_5x264_sigmoid_bias", 71, 5, 264, BF16, True, "sigmoid", 1e-5),
        ("rmsgated_f32_3x50_swish_bias", 72, 3, 50, F32, True, "swish", 1e-6),
        ("rmsgated_f16_4x128_sigmoid", 73, 4, 128, F16, False, "sigmoid", 1e-5),
    ]:
        gen = torch.Generator().manual_seed(seed)
        x, g = randn(gen, rows, cols).to(dtype), randn(gen, rows, cols).to(dtype)
        weight = (1 + 0.1 * randn(gen, cols)).to(dtype)
        bias = randn(gen, cols).to(dtype) if with_bias else None
        tensors = {"x": x, "g": g, "weight": weight, "y": KERNELS["rms_norm_gated"].reference(x, g, weight, bias, activation, eps)}
        if bias is not None:
            tensors["bias"] = bias
        save_case(name, tensors, {"op": "rms_norm_gated", "activation": activation, "eps": eps})
    for name, seed, rows, cols, dtype, eps in [("l2norm_bf16_40x128", 80, 40, 128, BF16, 1e-6), ("l2norm_f32_7x50", 81, 7, 50, F32, 1e-5),
                                               ("l2norm_f16_5x264", 82, 5, 264, F16, 1e-6), ("l2norm_bf16_3x4096", 83, 3, 4096, BF16, 1e-5)]:
        gen = torch.Generator().manual_seed(seed)
        x = randn(gen, rows, cols).to(dtype)
        save_case(name, {"x": x, "y": KERNELS["l2_norm"].reference(x, eps)}, {"op": "l2_norm", "eps": eps})
    for name, seed, rows, cols, dtype, with_bias, eps in [("layernorm_bf16_6x256_bias", 90, 6, 256, BF16, True, 1e-6), ("layernorm_f32_5x50", 91, 5, 50, F32, False, 1e-5),
                                                          ("layernorm_f16_4x136_bias", 92, 4, 136, F16, True, 1e-5), ("layernorm_bf16_3x4096", 93, 3, 4096, BF16, False, 1e-6)]:
        gen = torch.Generator().manual_seed(seed)
        x = (randn(gen, rows, cols) + 0.5).to(dtype)
        weight = (1 + 0.1 * randn(gen, cols)).to(dtype)
        bias = randn(gen, cols).to(dtype) if with_bias else None
        tensors = {"x": x, "weight": weight, "y": KERNELS["layer_norm"].reference(x, weight, bias, eps)}
        if bias is not None:
            tensors["bias"] = bias
        save_case(name, tensors, {"op": "layer_norm", "eps": eps})


def momoe_cases() -> None:
    ref = KERNELS["momoe"].reference
    for name, seed, batch, seq, hidden, inter, experts, top_k, dtype in [
        ("momoe_f32_e8_k1", 40, 2, 12, 32, 16, 8, 1, F32),
        ("momoe_f32_e8_k2", 41, 2, 12, 32, 16, 8, 2, F32),
        ("momoe_f32_e8_k6", 42, 1, 20, 32, 16, 8, 6, F32),
        ("momoe_f32_e64_k8", 43, 1, 48, 16, 8, 64, 8, F32),
        # 16-bit cases for the tensor-core expert projections (separate prefix: their tests carry 16-bit tolerances)
        ("moe16_bf16_e8_k2", 44, 2, 40, 64, 32, 8, 2, BF16),
        ("moe16_bf16_e16_k4", 45, 1, 300, 128, 72, 16, 4, BF16),
        ("moe16_f16_e4_k2", 46, 1, 96, 64, 40, 4, 2, F16),
    ]:
        gen = torch.Generator().manual_seed(seed)
        # signature order: x, gate_weight, up_weight, down_weight, router_logits (momoe.py:34-41);
        # weights are scaled by 1/sqrt(fan_in) as the reference's test_inputs do (momoe.py:26-30)
        x = randn(gen, batch, seq, hidden).to(dtype)
        gate_w = (randn(gen, experts, hidden, inter) / hidden**0.5).to(dtype)
        up_w = (randn(gen, experts, hidden, inter) / hidden**0.5).to(dtype)
        down_w = (randn(gen, experts, inter, hidden) / inter**0.5).to(dtype)
        logits = randn(gen, batch, seq, experts)
        y = ref(x, gate_w, up_w, down_w, logits, top_k)
        # the routing lines on their own (momoe.py:47-49), for the route oracle
        probs = torch.softmax(logits.float(), -1)
        picked = probs.topk(top_k, -1)
        gates = picked.values / picked.values.sum(-1, keepdim=True)
        save_case(
            name,
            {"x": x, "gate_weight": gate_w, "up_weight": up_w, "down_weight": down_w, "router_logits": logits,
             "y": y, "topk_indices": picked.indices.to(torch.int32), "topk_weights": gates},
            {"op": "momoe", "top_k": top_k},
        )


def gradient_cases() -> None:
    """Gradients by autograd through the registered references: in the case dtype (what a training call gets) and in
    fp64 (what popcorn's harness grades against, src/popcorn/bench/compare.py:243-277)."""

    def record(name, op, tensors, constants, meta):
        ref = KERNELS[op].reference

        def grads(cast):
            leaves = {k: cast(v).detach().clone().requires_grad_() for k, v in tensors.items()}
            outs = ref(*leaves.values(), *constants)
            outs = outs if isinstance(outs, tuple) else (outs,)
            gen = torch.Generator().manual_seed(meta["seed"] + 1000)
            seeds = [randn(gen, *o.shape).to(o.dtype) for o in outs]
            found = torch.autograd.grad(outs, list(leaves.values()), seeds, allow_unused=True)
            return seeds, dict(zip(leaves, found))

        seeds, native = grads(lambda t: t)
        _, truth = grads(lambda t: t.double())
        stored = dict(tensors)
        stored.update({f"cotangent{i}": c for i, c in enumerate(seeds)})
        stored.update({f"grad_{k}": g for k, g in native.items() if g is not None})
        stored.update({f"truth_{k}": g for k, g in truth.items() if g is not None})
        save_case(name, stored, {"op": op, **meta})

    gen = torch.Generator().manual_seed(60)
    x, w, b = randn(gen, 24, 256).to(BF16), (1 + 0.1 * randn(gen, 256)).to(BF16), randn(gen, 256).to(BF16)
    record("grad_rms_norm_bf16_24x256_bias", "rms_norm", {"x": x, "weight": w, "bias": b}, (1e-5,), {"seed": 60, "eps": 1e-5})
    gen = torch.Generator().manual_seed(61)
    x, r, w = randn(gen, 24, 512).to(BF16), randn(gen, 24, 512).to(BF16), (1 + 0.1 * randn(gen, 512)).to(BF16)
    record("grad_add_rms_norm_bf16_24x512_offset1", "add_rms_norm", {"x": x, "residual": r, "weight": w}, (1e-6, 1.0),
           {"seed": 61, "eps": 1e-6, "offset": 1.0})
    gen = torch.Generator().manual_seed(62)
    a, bb = randn(gen, 24, 256).to(BF16), randn(gen, 24, 256).to(BF16)
    record("grad_swiglu_bf16_24x256", "swiglu", {"a": a, "b": bb}, (), {"seed": 62})
    gen = torch.Generator().manual_seed(63)
    batch, seq, hidden, inter, experts, top_k = 1, 48, 64, 32, 8, 2
    tensors = {
        "x": randn(gen, batch, seq, hidden).to(BF16),
        "gate_weight": (randn(gen, experts, hidden, inter) / hidden**0.5).to(BF16),
        "up_weight": (randn(gen, experts, hidden, inter) / hidden**0.5).to(BF16),
        "down_weight": (randn(gen, experts, inter, hidden) / inter**0.5).to(BF16),
        "router_logits": randn(gen, batch, seq, experts),
    }
    record("grad_momoe_bf16_e8_k2", "momoe", tensors, (top_k,), {"seed": 63, "top_k": top_k})


def main() -> None:
    torch.manual_seed(0)
    rms_norm_cases()
    add_rms_norm_cases()
    rotary_cases()
    paired_rope_cases()
    qk_norm_rope_cases()
    llama4_rope_cases()
    swiglu_cases()
    sibling_cases()
    momoe_cases()
    gradient_cases()
    import popcorn

    print("popcorn", getattr(popcorn, "__version__", "?"), "torch", torch.__version__)


if __name__ == "__main__":
    main()
