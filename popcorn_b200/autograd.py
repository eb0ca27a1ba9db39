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


def swiglu(a: Tensor, b: Tensor) -> Tensor:
    """silu(a) * b with gradients for a and b."""
    return _SwiGLU.apply(a, b)


def rotary_embedding(x: Tensor, cos: Tensor, sin: Tensor, interleaved: bool = False) -> Tensor:
    """Rotary embedding with a gradient for x (cos and sin are constants, as in the reference)."""
    return _Rotary.apply(x, cos.detach(), sin.detach(), interleaved)
