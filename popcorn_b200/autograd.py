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
