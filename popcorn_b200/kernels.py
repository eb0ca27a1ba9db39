"""Op declarations on the local registry mirror, each with the `b200` backend attached.

The existing popcorn ops keep popcorn's names, parameter order and defaults
(src/popcorn/kernels/rms_norm.py:16-21, add_rms_norm.py:8-14,
rotary_embedding.py:15-20, rope.py:24-29, llama4_rope.py:27-31, swiglu.py:10; qk_norm_rope is the
fused op of examples/03_write_a_kernel.ipynb); the MoE steps are new ops because
popcorn only has them fused inside `momoe` (src/popcorn/kernels/momoe.py:47-53).
The declaration bodies are never executed: an op here is its signature plus the
backends registered on it.
"""

from __future__ import annotations

from popcorn_b200.registry import register_kernel

BACKEND = "b200"


@register_kernel
def rms_norm(x, weight, bias=None, eps=1e-6):
    """Root-mean-square normalization over the last dimension."""


@register_kernel
def add_rms_norm(x, residual, weight, eps=1e-6, offset=0.0):
    """Residual add fused with RMS norm; returns (normalized sum, new residual stream)."""


@register_kernel
def rotary_embedding(x, cos, sin, interleaved=False):
    """Rotary position embedding, GPT-NeoX halves or GPT-J interleaved pairs."""


@register_kernel
def rope(q, k, cos, sin):
    """Paired Llama-style rotary embedding of queries and keys, layout (batch, heads, seq, head_dim)."""


@register_kernel
def qk_norm_rope(q, k, q_weight, k_weight, cos, sin, eps=1e-6):
    """Per-head RMS normalization of queries and keys followed by the paired rotary embedding."""


@register_kernel
def llama4_rope(q, k, freqs):
    """Paired Llama 4 rotary embedding, frequencies as (cos, sin) pairs; layout (batch, seq, heads, head_dim)."""


@register_kernel
def swiglu(a, b):
    """SwiGLU gating: silu(a) * b."""


@register_kernel
def geglu(a, b):
    """GEGLU gating with the tanh-approximate GELU: gelu(a) * b."""


@register_kernel
def rms_norm_gated(x, g, weight, bias=None, activation="swish", eps=1e-6):
    """RMS norm scaled by a swish or sigmoid gate."""


@register_kernel
def l2_norm(x, eps=1e-6):
    """L2 normalization along the last dimension."""


@register_kernel
def layer_norm(x, weight, bias=None, eps=1e-6):
    """Layer normalization: standardize the last dimension, then scale and shift."""


@register_kernel
def moe_route(router_logits, top_k=2):
    """Softmax over experts, top-k selection, renormalized gate weights."""


@register_kernel
def moe_permute(x, indices, experts):
    """Stable sort of (token, slot) pairs by expert and the row gather into that order."""


@register_kernel
def moe_unpermute(rows, weights, pos):
    """Gate-weighted sum of expert rows back into token order."""


@register_kernel
def moe_grouped_gemm(rows, weight, offsets, up_weight=None):
    """Per-expert projection of expert-major rows; with up_weight, silu(rows @ weight) * (rows @ up_weight)."""


@register_kernel
def momoe(x, gate_weight, up_weight, down_weight, router_logits, top_k=2):
    """Mixture of experts over SwiGLU MLPs, routed to the top-k experts by softmax probability."""


# ops with backward kernels are registered in their differentiable form
for _op in (rms_norm, add_rms_norm, rms_norm_gated, l2_norm, layer_norm, rotary_embedding, rope, llama4_rope, qk_norm_rope, swiglu, geglu,
            moe_route, moe_permute, moe_unpermute, moe_grouped_gemm, momoe):
    _op.register(BACKEND, source=f"popcorn_b200.autograd.{_op.name}")
del _op
