"""Differentiable forms of the ops that have a backward kernel.

`popcorn_b200.ops` is forward-only.  The functions here wrap an op and its
backward kernel in a `torch.autograd.Function`, so they can be registered with
popcorn WITHOUT `forward_only=True` and serve training calls too, the way
popcorn's own CUDA SwiGLU does (src/popcorn/impls/swiglu_cu.py:8-23) and its
Triton rotary kernel does with the conjugate rotation
(src/popcorn/impls/rotary_embedding_tl.py:95-110).
"""

from __future__ import annotations

import torch
from torch import Tensor

from popcorn_b200 import ops


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a: Tensor, b: Tensor) -> Tensor:
        ctx.save_for_backward(a, b)
        with torch.no_grad():
            return ops.swiglu(a, b)

    @staticmethod
    def backward(ctx, grad_out: Tensor):
        a, b = ctx.saved_tensors
        with torch.no_grad():
            grad_a, grad_b = ops.swiglu_backward(grad_out.contiguous(), a, b)
        return grad_a, grad_b


class _GeGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a: Tensor, b: Tensor) -> Tensor:
        ctx.save_for_backward(a, b)
        with torch.no_grad():
            return ops.geglu(a, b)

    @staticmethod
    def backward(ctx, grad_out: Tensor):
        a, b = ctx.saved_tensors
        with torch.no_grad():
            grad_a, grad_b = ops.geglu_backward(grad_out.contiguous(), a, b)
        return grad_a, grad_b


class _PairedRope(torch.autograd.Function):
    """rope(q, k, cos, sin): y1 = x1 c1 - x2 s1, y2 = x2 c2 + x1 s2 per half, so the transpose is the same kernel with
    the sine table's halves swapped and negated (for a table with repeated halves: the opposite angle)."""

    @staticmethod
    def forward(ctx, q: Tensor, k: Tensor, cos: Tensor, sin: Tensor):
        ctx.save_for_backward(cos, sin)
        with torch.no_grad():
            return ops.rope(q, k, cos, sin)

    @staticmethod
    def backward(ctx, grad_q: Tensor, grad_k: Tensor):
        cos, sin = ctx.saved_tensors
        first, second = sin.chunk(2, -1)
        with torch.no_grad():
            dq, dk = ops.rope(grad_q.contiguous(), grad_k.contiguous(), cos, -torch.cat((second, first), -1))
        return dq, dk, None, None


class _QkNormRope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q: Tensor, k: Tensor, q_weight: Tensor, k_weight: Tensor, cos: Tensor, sin: Tensor, eps: float):
        ctx.save_for_backward(q, k, q_weight, k_weight, cos, sin)
        ctx.eps = eps
        with torch.no_grad():
            return ops.qk_norm_rope(q, k, q_weight, k_weight, cos, sin, eps)

    @staticmethod
    def backward(ctx, grad_q: Tensor, grad_k: Tensor):
        q, k, q_weight, k_weight, cos, sin = ctx.saved_tensors
        with torch.no_grad():
            dq, dk, dqw, dkw = ops.qk_norm_rope_backward(grad_q, grad_k, q, k, q_weight, k_weight, cos, sin, ctx.eps)
        return dq, dk, dqw, dkw, None, None, None


class _RmsNormGated(torch.autograd.Function):
    """out = z * gate(g), z = rms_norm(x, weight, bias), gate = silu or sigmoid.  The backward is a composition of kernels
    that exist: the gate backward (swiglu_backward or sigmoid_gate_backward on (grad_out, g, z)) yields (grad_g, grad_z)
    with autograd's roundings, and rms_norm_backward turns grad_z into the gradients of x, weight and bias; z is
    recomputed by the forward norm kernel, not saved."""

    @staticmethod
    def forward(ctx, x: Tensor, g: Tensor, weight: Tensor, bias: Tensor | None, activation: str, eps: float) -> Tensor:
        ctx.save_for_backward(x, g, weight, bias)
        ctx.eps, ctx.activation = eps, activation
        with torch.no_grad():
            return ops.rms_norm_gated(x, g, weight, bias, activation, eps)

    @staticmethod
    def backward(ctx, grad_out: Tensor):
        x, g, weight, bias = ctx.saved_tensors
        gate_backward = ops.swiglu_backward if ctx.activation == "swish" else ops.sigmoid_gate_backward
        with torch.no_grad():
            z = ops.rms_norm(x, weight, bias, ctx.eps)
            grad_g, grad_z = gate_backward(grad_out.contiguous(), g, z)
            grad_x, grad_w, grad_b = ops.rms_norm_backward(grad_z, x, weight, bias is not None, ctx.eps)
        return grad_x, grad_g, grad_w, grad_b, None, None


class _L2Norm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, eps: float) -> Tensor:
        ctx.save_for_backward(x)
        ctx.eps = eps
        with torch.no_grad():
            return ops.l2_norm(x, eps)

    @staticmethod
    def backward(ctx, grad_y: Tensor):
        (x,) = ctx.saved_tensors
        with torch.no_grad():
            return ops.l2_norm_backward(grad_y.contiguous(), x, ctx.eps), None


class _LayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, weight: Tensor, bias: Tensor | None, eps: float) -> Tensor:
        ctx.save_for_backward(x, weight)
        ctx.with_bias, ctx.eps = bias is not None, eps
        with torch.no_grad():
            return ops.layer_norm(x, weight, bias, eps)

    @staticmethod
    def backward(ctx, grad_y: Tensor):
        x, weight = ctx.saved_tensors
        with torch.no_grad():
            grad_x, grad_w, grad_b = ops.layer_norm_backward(grad_y.contiguous(), x, weight, ctx.with_bias, ctx.eps)
        return grad_x, grad_w, grad_b, None


class _MoeRoute(torch.autograd.Function):
    """weights = softmax over the picked logits, so d logits[e_k] = w_k (d w_k - sum_j w_j d w_j) on the picked
    experts and zero elsewhere (the selection itself carries no gradient, as in the reference, momoe.py:47-49)."""

    @staticmethod
    def forward(ctx, router_logits: Tensor, top_k: int):
        with torch.no_grad():
            indices, weights = ops.moe_route(router_logits, top_k)
        ctx.save_for_backward(indices, weights)
        ctx.shape, ctx.dtype = router_logits.shape, router_logits.dtype
        ctx.mark_non_differentiable(indices)
        return indices, weights

    @staticmethod
    def backward(ctx, _grad_indices, grad_weights: Tensor):
        indices, weights = ctx.saved_tensors
        inner = (weights * grad_weights).sum(-1, keepdim=True)
        picked = weights * (grad_weights - inner)
        grad_logits = torch.zeros(ctx.shape, dtype=torch.float32, device=weights.device)
        grad_logits.scatter_(-1, indices.long(), picked)
        return grad_logits.to(ctx.dtype), None


class _MoePermute(torch.autograd.Function):
    """rows[pos[t, k]] = x[t]: every token row collects the gradients of its top_k copies, which is the combine
    kernel with unit weights."""

    @staticmethod
    def forward(ctx, x: Tensor, indices: Tensor, experts: int):
        with torch.no_grad():
            rows, counts, offsets, perm, pos = ops.moe_permute(x, indices, experts)
        ctx.save_for_backward(pos)
        ctx.mark_non_differentiable(counts, offsets, perm, pos)
        return rows, counts, offsets, perm, pos

    @staticmethod
    def backward(ctx, grad_rows: Tensor, *_unused):
        (pos,) = ctx.saved_tensors
        with torch.no_grad():
            grad_x = ops.moe_unpermute(grad_rows.contiguous(), torch.ones(pos.shape, dtype=torch.float32, device=pos.device), pos)
        return grad_x, None, None


class _MoeUnpermute(torch.autograd.Function):
    @staticmethod
    def forward(ctx, rows: Tensor, weights: Tensor, pos: Tensor) -> Tensor:
        ctx.save_for_backward(rows, weights, pos)
        with torch.no_grad():
            return ops.moe_unpermute(rows, weights, pos)

    @staticmethod
    def backward(ctx, grad_y: Tensor):
        rows, weights, pos = ctx.saved_tensors
        with torch.no_grad():
            grad_rows, grad_weights = ops.moe_unpermute_backward(grad_y.contiguous(), rows, weights, pos)
        return grad_rows, grad_weights, None


class _GroupedGemm(torch.autograd.Function):
    """out = rows @ weight[e]: the gradients are two more grouped GEMMs on the same tensor-core kernel, one that reads
    the weights along their rows and one that contracts over each expert's rows."""

    @staticmethod
    def forward(ctx, rows: Tensor, weight: Tensor, offsets: Tensor) -> Tensor:
        ctx.save_for_backward(rows, weight, offsets)
        with torch.no_grad():
            return ops.moe_grouped_gemm(rows, weight, offsets)

    @staticmethod
    def backward(ctx, grad_out: Tensor):
        rows, weight, offsets = ctx.saved_tensors
        grad_out = grad_out.contiguous()
        with torch.no_grad():
            grad_rows = ops.moe_grouped_gemm_dgrad(grad_out, weight, offsets) if ctx.needs_input_grad[0] else None
            grad_weight = ops.moe_grouped_gemm_wgrad(rows, grad_out, offsets) if ctx.needs_input_grad[1] else None
        return grad_rows, grad_weight, None


class _GroupedGateUp(torch.autograd.Function):
    """silu(rows @ gate[e]) * (rows @ up[e]) for training: one pass computes both projections and keeps them (16-bit,
    like the incumbent's saved activations, src/popcorn/impls/momoe_tl.py:180-190), the SwiGLU kernel forms the
    product; backward = SwiGLU backward, one GEMM summing both branches into grad_rows, two weight gradients."""

    @staticmethod
    def forward(ctx, rows: Tensor, gate_weight: Tensor, up_weight: Tensor, offsets: Tensor) -> Tensor:
        width = gate_weight.shape[2]
        with torch.no_grad():
            both = ops.moe_grouped_gemm_gate_up(rows, gate_weight, up_weight, offsets)
            out = ops.swiglu(both[:, :width], both[:, width:])
        ctx.save_for_backward(rows, gate_weight, up_weight, offsets, both)
        return out

    @staticmethod
    def backward(ctx, grad_out: Tensor):
        rows, gate_weight, up_weight, offsets, both = ctx.saved_tensors
        width = gate_weight.shape[2]
        with torch.no_grad():
            grad_gate, grad_up = ops.swiglu_backward(grad_out.contiguous(), both[:, :width], both[:, width:])
            grad_rows = ops.moe_grouped_gemm_dgrad(grad_gate, gate_weight, offsets, grad_up, up_weight) if ctx.needs_input_grad[0] else None
            grad_gate_weight = ops.moe_grouped_gemm_wgrad(rows, grad_gate, offsets) if ctx.needs_input_grad[1] else None
            grad_up_weight = ops.moe_grouped_gemm_wgrad(rows, grad_up, offsets) if ctx.needs_input_grad[2] else None
        return grad_rows, grad_gate_weight, grad_up_weight, None


class _Llama4Rope(torch.autograd.Function):
    """Multiplication by unit complex numbers: the transpose multiplies by their conjugates."""

    @staticmethod
    def forward(ctx, q: Tensor, k: Tensor, freqs: Tensor):
        ctx.save_for_backward(freqs)
        with torch.no_grad():
            return ops.llama4_rope(q, k, freqs)

    @staticmethod
    def backward(ctx, grad_q: Tensor, grad_k: Tensor):
        (freqs,) = ctx.saved_tensors
        conjugate = torch.stack((freqs[..., 0], -freqs[..., 1]), -1)
        with torch.no_grad():
            dq, dk = ops.llama4_rope(grad_q.contiguous(), grad_k.contiguous(), conjugate)
        return dq, dk, None


class _Rotary(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, cos: Tensor, sin: Tensor, interleaved: bool) -> Tensor:
        ctx.save_for_backward(cos, sin)
        ctx.interleaved = interleaved
        with torch.no_grad():
            return ops.rotary_embedding(x, cos, sin, interleaved)

    @staticmethod
    def backward(ctx, grad_out: Tensor):
        cos, sin = ctx.saved_tensors
        # the transpose of a rotation is the rotation by the opposite angle; pass-through channels pass through
        with torch.no_grad():
            grad_x = ops.rotary_embedding(grad_out.contiguous(), cos, -sin, ctx.interleaved)
        return grad_x, None, None, None


class _RmsNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, weight: Tensor, bias: Tensor | None, eps: float) -> Tensor:
        ctx.save_for_backward(x, weight)
        ctx.with_bias, ctx.eps = bias is not None, eps
        with torch.no_grad():
            return ops.rms_norm(x, weight, bias, eps)

    @staticmethod
    def backward(ctx, grad_y: Tensor):
        x, weight = ctx.saved_tensors
        with torch.no_grad():
            grad_x, grad_w, grad_b = ops.rms_norm_backward(grad_y.contiguous(), x, weight, ctx.with_bias, ctx.eps)
        return grad_x, grad_w, grad_b, None


class _AddRmsNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, residual: Tensor, weight: Tensor, eps: float, offset: float):
        with torch.no_grad():
            y, s = ops.add_rms_norm(x, residual, weight, eps, offset)
        ctx.save_for_backward(s, weight)
        ctx.eps, ctx.offset = eps, offset
        return y, s

    @staticmethod
    def backward(ctx, grad_y: Tensor | None, grad_s: Tensor | None):
        s, weight = ctx.saved_tensors
        if grad_y is None:  # only the residual stream was used downstream
            return grad_s, grad_s, torch.zeros_like(weight), None, None
        with torch.no_grad():
            grad_x, grad_w = ops.add_rms_norm_backward(grad_y.contiguous(), None if grad_s is None else grad_s.contiguous(),
                                                       s, weight, ctx.eps, ctx.offset)
        return grad_x, grad_x, grad_w, None, None


def rms_norm(x: Tensor, weight: Tensor, bias: Tensor | None = None, eps: float = 1e-6) -> Tensor:
    """RMS norm with gradients for x, weight and bias."""
    return _RmsNorm.apply(x, weight, bias, eps)


def add_rms_norm(x: Tensor, residual: Tensor, weight: Tensor, eps: float = 1e-6, offset: float = 0.0) -> tuple[Tensor, Tensor]:
    """Residual add + RMS norm with gradients for x, residual and weight."""
    return _AddRmsNorm.apply(x, residual, weight, eps, offset)


def swiglu(a: Tensor, b: Tensor) -> Tensor:
    """silu(a) * b with gradients for a and b."""
    return _SwiGLU.apply(a, b)


def rotary_embedding(x: Tensor, cos: Tensor, sin: Tensor, interleaved: bool = False) -> Tensor:
    """Rotary embedding with a gradient for x (cos and sin are constants, as in the reference)."""
    return _Rotary.apply(x, cos.detach(), sin.detach(), interleaved)


def geglu(a: Tensor, b: Tensor) -> Tensor:
    """gelu_tanh(a) * b with gradients for a and b."""
    return _GeGLU.apply(a, b)


def rope(q: Tensor, k: Tensor, cos: Tensor, sin: Tensor) -> tuple[Tensor, Tensor]:
    """Paired rotary embedding with gradients for q and k (cos and sin are constants, as in the reference)."""
    return _PairedRope.apply(q, k, cos.detach(), sin.detach())


def llama4_rope(q: Tensor, k: Tensor, freqs: Tensor) -> tuple[Tensor, Tensor]:
    """Llama 4 rotary embedding with gradients for q and k (freqs are constants, as in the reference)."""
    return _Llama4Rope.apply(q, k, freqs.detach())


def qk_norm_rope(q: Tensor, k: Tensor, q_weight: Tensor, k_weight: Tensor, cos: Tensor, sin: Tensor, eps: float = 1e-6) -> tuple[Tensor, Tensor]:
    """Fused per-head RMSNorm + paired rotary embedding with gradients for q, k and both weights."""
    return _QkNormRope.apply(q, k, q_weight, k_weight, cos.detach(), sin.detach(), eps)


def rms_norm_gated(x: Tensor, g: Tensor, weight: Tensor, bias: Tensor | None = None, activation: str = "swish", eps: float = 1e-6) -> Tensor:
    """Gated RMS norm (swish or sigmoid gate) with gradients for x, g, weight and bias."""
    if activation not in ("swish", "sigmoid"):
        raise ValueError(f"rms_norm_gated: activation must be 'swish' or 'sigmoid', got {activation!r}")
    return _RmsNormGated.apply(x, g, weight, bias, activation, eps)


def l2_norm(x: Tensor, eps: float = 1e-6) -> Tensor:
    """L2 normalization with a gradient for x."""
    return _L2Norm.apply(x, eps)


def layer_norm(x: Tensor, weight: Tensor, bias: Tensor | None = None, eps: float = 1e-6) -> Tensor:
    """Layer normalization with gradients for x, weight and bias."""
    return _LayerNorm.apply(x, weight, bias, eps)


def moe_route(router_logits: Tensor, top_k: int = 2) -> tuple[Tensor, Tensor]:
    """Routing with a gradient from the gate weights back to the logits of the picked experts."""
    return _MoeRoute.apply(router_logits, top_k)


def moe_permute(x: Tensor, indices: Tensor, experts: int) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
    """Permutation into expert-major rows with a gradient for x."""
    return _MoePermute.apply(x, indices, experts)


def moe_unpermute(rows: Tensor, weights: Tensor, pos: Tensor) -> Tensor:
    """Weighted combine with gradients for the expert rows and the gate weights."""
    return _MoeUnpermute.apply(rows, weights, pos)


def _needs_grad(*tensors: Tensor | None) -> bool:
    return torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in tensors)


def moe_grouped_gemm(rows: Tensor, weight: Tensor, offsets: Tensor, up_weight: Tensor | None = None) -> Tensor:
    """Per-expert projection with gradients for rows and weights.  Inference calls take the fused kernel; a training call
    with `up_weight` keeps the two 16-bit pre-activations, so its SwiGLU input is rounded once more than the fused form's."""
    if not _needs_grad(rows, weight, up_weight):
        return ops.moe_grouped_gemm(rows, weight, offsets, up_weight)
    if up_weight is None:
        return _GroupedGemm.apply(rows, weight, offsets)
    return _GroupedGateUp.apply(rows, weight, up_weight, offsets)


def momoe(x: Tensor, gate_weight: Tensor, up_weight: Tensor, down_weight: Tensor, router_logits: Tensor, top_k: int = 2) -> Tensor:
    """Mixture of SwiGLU expert MLPs with gradients for x, the three weights and the router logits: the chain of
    `ops.momoe` built from the differentiable steps (the routed experts only; gradients of unrouted pairs are zero in
    the reference too, where their gate weight is exactly zero, src/popcorn/kernels/momoe.py:47-53)."""
    if not _needs_grad(x, gate_weight, up_weight, down_weight, router_logits):
        return ops.momoe(x, gate_weight, up_weight, down_weight, router_logits, top_k)
    ops.check_momoe(x, gate_weight, up_weight, down_weight, router_logits)
    experts, hidden, _ = gate_weight.shape
    indices, weights = moe_route(router_logits.reshape(-1, experts).float(), int(top_k))
    rows, _, offsets, _, pos = moe_permute(x.reshape(-1, hidden), indices, experts)
    hidden_act = moe_grouped_gemm(rows, gate_weight, offsets, up_weight)
    out_rows = moe_grouped_gemm(hidden_act, down_weight, offsets)
    return moe_unpermute(out_rows, weights, pos).reshape(x.shape)
