"""The ops of the `b200` backend, with the signatures of popcorn's references.

Each function takes CUDA tensors, allocates its outputs with torch, and enqueues
one or more sm_100a kernels of libpopcorn_b200.so on the current stream of the
input's device.  Nothing here computes on the host and nothing falls back to
PyTorch arithmetic: a CPU tensor, an unsupported dtype or a missing library is
an error.  The ops are forward-only (no autograd), like popcorn backends
registered with ``forward_only=True``
(src/popcorn/core/dispatcher.py:130-131).

Signatures served (names and order are popcorn's):
  rms_norm(x, weight, bias=None, eps=1e-6)                 src/popcorn/kernels/rms_norm.py:16-21
  add_rms_norm(x, residual, weight, eps=1e-6, offset=0.0)  src/popcorn/kernels/add_rms_norm.py:8-14
  rotary_embedding(x, cos, sin, interleaved=False)         src/popcorn/kernels/rotary_embedding.py:15-20
  swiglu(a, b)                                             src/popcorn/kernels/swiglu.py:10
  rope(q, k, cos, sin)                                     src/popcorn/kernels/rope.py:24-29
  geglu(a, b)                                              src/popcorn/kernels/geglu.py:9
  rms_norm_gated(x, g, weight, bias=None, activation="swish", eps=1e-6)   src/popcorn/kernels/rms_norm_gated.py:13-20
  l2_norm(x, eps=1e-6)                                     src/popcorn/kernels/l2_norm.py:9
  layer_norm(x, weight, bias=None, eps=1e-6)               src/popcorn/kernels/layer_norm.py:9-14
and the MoE steps popcorn only has fused inside `momoe`
(src/popcorn/kernels/momoe.py:47-53, src/popcorn/impls/momoe_tl.py:1071-1161):
  moe_route, moe_index, moe_scatter_rows, moe_permute, moe_gather, moe_unpermute.
"""

from __future__ import annotations

import ctypes

import torch
from torch import Tensor

from popcorn_b200 import _lib

_DTYPES = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}


def _dtype_code(t: Tensor, what: str) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TypeError(f"{what}: dtype {t.dtype} is not supported (float32, float16, bfloat16)") from None


def _require_cuda(*tensors: Tensor | None) -> torch.device:
    device = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("popcorn_b200 ops run on CUDA tensors only; there is no CPU implementation")
        if device is None:
            device = t.device
        elif t.device != device:
            raise RuntimeError(f"tensors live on different devices: {device} and {t.device}")
    assert device is not None
    return device


def _forbid_grad(*tensors: Tensor | None) -> None:
    if torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in tensors):
        raise RuntimeError("popcorn_b200 ops are forward-only; call them under torch.no_grad() or detach the inputs")


def _rows(t: Tensor) -> tuple[Tensor, int]:
    """View `t` [..., D] as [rows, D] with a contiguous last dim; returns (view, leading dimension)."""
    width = t.shape[-1]
    if t.dim() == 2 and (t.stride(1) == 1 or width == 1):
        return t, (t.stride(0) if t.shape[0] > 1 else max(width, 1))
    if t.dim() >= 1 and (t.stride(-1) == 1 or width == 1):
        try:
            flat = t.view(-1, width)
        except RuntimeError:
            flat = None
        if flat is not None and (flat.stride(1) == 1 or width == 1):
            return flat, (flat.stride(0) if flat.shape[0] > 1 else max(width, 1))
    flat = t.reshape(-1, width).contiguous()
    return flat, max(width, 1)


class _DevicePointer(ctypes.c_void_p):
    """A device address that keeps its tensor alive for as long as the pointer object exists.

    Call sites write `_ptr(weight.contiguous())` inside the argument list of `_lib.call`.  When the tensor
    is not contiguous that expression makes a copy whose only reference is this object; without it the copy
    would go back to the caching allocator before the launch, and the next `.contiguous()` in the same
    argument list could be handed the same block (two operands would then alias).  The argument tuple holds
    every pointer until the call has enqueued its kernels, after which stream order protects the block."""

    tensor: Tensor | None = None


def _ptr(t: Tensor | None) -> ctypes.c_void_p:
    pointer = _DevicePointer(0 if t is None else t.data_ptr())
    pointer.tensor = t
    return pointer


def _stream(device: torch.device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def rms_norm(x: Tensor, weight: Tensor, bias: Tensor | None = None, eps: float = 1e-6) -> Tensor:
    """Root-mean-square normalisation over the last dimension (rms_norm.py:16-30)."""
    device = _require_cuda(x, weight, bias)
    _forbid_grad(x, weight, bias)
    code = _dtype_code(x, "rms_norm")
    width = x.shape[-1]
    if weight.shape != (width,) or (bias is not None and bias.shape != (width,)):
        raise ValueError(f"rms_norm: weight/bias must have shape ({width},)")
    if weight.dtype != x.dtype or (bias is not None and bias.dtype != x.dtype):
        raise TypeError("rms_norm: weight and bias must have the dtype of x")
    x2, ldx = _rows(x)
    y = torch.empty(x.shape, dtype=x.dtype, device=device)
    y2 = y.view(-1, width)
    with torch.cuda.device(device):
        _lib.call(
            "b200_rms_norm", _ptr(x2), _ptr(weight.contiguous()), _ptr(None if bias is None else bias.contiguous()), _ptr(y2),
            x2.shape[0], width, ldx, max(width, 1), code, float(eps), _stream(device),
        )
    return y


def add_rms_norm(
    x: Tensor, residual: Tensor, weight: Tensor, eps: float = 1e-6, offset: float = 0.0
) -> tuple[Tensor, Tensor]:
    """s = x + residual; returns (rms_norm(s) * (weight + offset), s) (add_rms_norm.py:8-23)."""
    device = _require_cuda(x, residual, weight)
    _forbid_grad(x, residual, weight)
    code = _dtype_code(x, "add_rms_norm")
    width = x.shape[-1]
    if residual.shape != x.shape:
        raise ValueError("add_rms_norm: x and residual must have the same shape")
    if weight.shape != (width,):
        raise ValueError(f"add_rms_norm: weight must have shape ({width},)")
    if residual.dtype != x.dtype or weight.dtype != x.dtype:
        raise TypeError("add_rms_norm: residual and weight must have the dtype of x")
    x2, ldx = _rows(x)
    r2, ldr = _rows(residual)
    y = torch.empty(x.shape, dtype=x.dtype, device=device)
    s = torch.empty(x.shape, dtype=x.dtype, device=device)
    ld = max(width, 1)
    with torch.cuda.device(device):
        _lib.call(
            "b200_add_rms_norm", _ptr(x2), _ptr(r2), _ptr(weight.contiguous()), _ptr(y), _ptr(s),
            x2.shape[0], width, ldx, ldr, ld, ld, code, float(eps), float(offset), _stream(device),
        )
    return y, s


def _norm_scratch(rows: int, cols: int, with_bias: bool, device: torch.device) -> Tensor:
    need = ctypes.c_size_t(0)
    with torch.cuda.device(device):
        _lib.call("b200_rms_norm_backward_scratch_bytes", rows, cols, int(with_bias), ctypes.byref(need))
    return torch.empty(max(need.value, 16), dtype=torch.uint8, device=device)


def rms_norm_backward(grad_y: Tensor, x: Tensor, weight: Tensor, with_bias: bool = False, eps: float = 1e-6) -> tuple[Tensor, Tensor, Tensor | None]:
    """(grad_x, grad_weight, grad_bias or None) of rms_norm(x, weight, bias, eps)."""
    device = _require_cuda(grad_y, x, weight)
    code = _dtype_code(x, "rms_norm_backward")
    width = x.shape[-1]
    if grad_y.shape != x.shape or weight.shape != (width,) or not (grad_y.dtype == weight.dtype == x.dtype):
        raise ValueError("rms_norm_backward: grad_y must match x, and weight must be [hidden] of the same dtype")
    g2, ldg = _rows(grad_y)
    x2, ldx = _rows(x)
    grad_x = torch.empty(x.shape, dtype=x.dtype, device=device)
    grad_w = torch.empty(width, dtype=x.dtype, device=device)
    grad_b = torch.empty(width, dtype=x.dtype, device=device) if with_bias else None
    scratch = _norm_scratch(x2.shape[0], width, with_bias, device)
    with torch.cuda.device(device):
        _lib.call("b200_rms_norm_backward", _ptr(g2), _ptr(x2), _ptr(weight.contiguous()), _ptr(grad_x), _ptr(grad_w), _ptr(grad_b),
                  x2.shape[0], width, ldg, ldx, max(width, 1), code, float(eps), _ptr(scratch), ctypes.c_size_t(scratch.numel()), _stream(device))
    return grad_x, grad_w, grad_b


def add_rms_norm_backward(grad_y: Tensor, grad_s: Tensor | None, s: Tensor, weight: Tensor, eps: float = 1e-6, offset: float = 0.0) -> tuple[Tensor, Tensor]:
    """(grad_x = grad_residual, grad_weight) of add_rms_norm; `s` is the residual stream the forward returned."""
    device = _require_cuda(grad_y, grad_s, s, weight)
    code = _dtype_code(s, "add_rms_norm_backward")
    width = s.shape[-1]
    if grad_y.shape != s.shape or (grad_s is not None and grad_s.shape != s.shape) or weight.shape != (width,):
        raise ValueError("add_rms_norm_backward: gradients must match s, and weight must be [hidden]")
    gy2, ldgy = _rows(grad_y)
    s2, lds = _rows(s)
    gs2, ldgs = _rows(grad_s) if grad_s is not None else (None, 0)
    grad_x = torch.empty(s.shape, dtype=s.dtype, device=device)
    grad_w = torch.empty(width, dtype=s.dtype, device=device)
    scratch = _norm_scratch(s2.shape[0], width, False, device)
    with torch.cuda.device(device):
        _lib.call("b200_add_rms_norm_backward", _ptr(gy2), _ptr(gs2), _ptr(s2), _ptr(weight.contiguous()), _ptr(grad_x), _ptr(grad_w),
                  s2.shape[0], width, ldgy, ldgs, lds, max(width, 1), code, float(eps), float(offset),
                  _ptr(scratch), ctypes.c_size_t(scratch.numel()), _stream(device))
    return grad_x, grad_w


def _rope_check(x: Tensor, cos: Tensor, sin: Tensor, name: str) -> tuple[int, int]:
    if x.dim() != 4:
        raise ValueError(f"{name}: x must be [batch, seq, heads, head_dim]")
    if cos.shape != sin.shape or cos.dim() != 2 or cos.shape[0] != x.shape[1]:
        raise ValueError(f"{name}: cos and sin must both be [seq, half]")
    half = cos.shape[1]
    if 2 * half > x.shape[-1]:
        raise ValueError(f"{name}: 2*half={2 * half} exceeds head_dim={x.shape[-1]}")
    if cos.dtype != sin.dtype or cos.dtype not in (torch.float32, x.dtype):
        raise TypeError(f"{name}: cos/sin must be float32 or the dtype of x")
    if x.shape[-1] > 1 and x.stride(-1) != 1:
        raise ValueError(f"{name}: the head_dim dimension of x must be contiguous")
    return half, _DTYPES[cos.dtype]


def rotary_embedding(x: Tensor, cos: Tensor, sin: Tensor, interleaved: bool = False) -> Tensor:
    """Rotary position embedding, out of place (rotary_embedding.py:15-40)."""
    device = _require_cuda(x, cos, sin)
    _forbid_grad(x)
    code = _dtype_code(x, "rotary_embedding")
    half, cs_code = _rope_check(x, cos, sin, "rotary_embedding")
    out = torch.empty(x.shape, dtype=x.dtype, device=device)
    b, s, h, d = x.shape
    with torch.cuda.device(device):
        _lib.call(
            "b200_rope", _ptr(x), _ptr(cos.contiguous()), _ptr(sin.contiguous()), _ptr(out), b, s, h, d, half,
            x.stride(0), x.stride(1), x.stride(2), out.stride(0), out.stride(1), out.stride(2),
            code, cs_code, int(bool(interleaved)), _stream(device),
        )
    return out


def rotary_embedding_(x: Tensor, cos: Tensor, sin: Tensor, interleaved: bool = False) -> Tensor:
    """In-place variant of rotary_embedding: rotates x where it lies and returns it."""
    device = _require_cuda(x, cos, sin)
    _forbid_grad(x)
    code = _dtype_code(x, "rotary_embedding_")
    half, cs_code = _rope_check(x, cos, sin, "rotary_embedding_")
    b, s, h, d = x.shape
    with torch.cuda.device(device):
        _lib.call(
            "b200_rope", _ptr(x), _ptr(cos.contiguous()), _ptr(sin.contiguous()), _ptr(x), b, s, h, d, half,
            x.stride(0), x.stride(1), x.stride(2), x.stride(0), x.stride(1), x.stride(2),
            code, cs_code, int(bool(interleaved)), _stream(device),
        )
    return x


def rotary_embedding_qk_(q: Tensor, k: Tensor, cos: Tensor, sin: Tensor, interleaved: bool = False) -> tuple[Tensor, Tensor]:
    """Rotate q and k in place with one launch (the cos/sin row is fetched once for both)."""
    device = _require_cuda(q, k, cos, sin)
    _forbid_grad(q, k)
    code = _dtype_code(q, "rotary_embedding_qk_")
    if k.dtype != q.dtype:
        raise TypeError("rotary_embedding_qk_: q and k must share a dtype")
    half, cs_code = _rope_check(q, cos, sin, "rotary_embedding_qk_")
    _rope_check(k, cos, sin, "rotary_embedding_qk_")
    if q.shape[:2] != k.shape[:2] or q.shape[-1] != k.shape[-1]:
        raise ValueError("rotary_embedding_qk_: q and k must agree in batch, seq and head_dim")
    b, s, hq, d = q.shape
    with torch.cuda.device(device):
        _lib.call(
            "b200_rope_qk", _ptr(q), _ptr(k), _ptr(cos.contiguous()), _ptr(sin.contiguous()), b, s, hq, k.shape[2], d, half,
            q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
            code, cs_code, int(bool(interleaved)), _stream(device),
        )
    return q, k


def rope(q: Tensor, k: Tensor, cos: Tensor, sin: Tensor) -> tuple[Tensor, Tensor]:
    """Paired Llama-style rotary embedding of q and k, layout (batch, heads, seq, head_dim) (rope.py:24-36)."""
    device = _require_cuda(q, k, cos, sin)
    _forbid_grad(q, k)
    code = _dtype_code(q, "rope")
    if q.dim() != 4 or k.dim() != 4 or q.shape[0] != k.shape[0] or q.shape[2:] != k.shape[2:]:
        raise ValueError("rope: q and k must be [batch, heads, seq, head_dim] and agree in batch, seq and head_dim")
    batch, q_heads, seq, head_dim = q.shape
    if cos.shape != sin.shape or cos.dim() != 3 or cos.shape[1:] != (seq, head_dim) or cos.shape[0] not in (1, batch):
        raise ValueError("rope: cos and sin must be [1 or batch, seq, head_dim]")
    if not (k.dtype == cos.dtype == sin.dtype == q.dtype):
        raise TypeError("rope: q, k, cos and sin must share a dtype")
    if head_dim % 2:
        raise ValueError("rope: head_dim must be even")
    q = q if head_dim <= 1 or q.stride(-1) == 1 else q.contiguous()
    k = k if head_dim <= 1 or k.stride(-1) == 1 else k.contiguous()
    q_out = torch.empty(q.shape, dtype=q.dtype, device=device)
    k_out = torch.empty(k.shape, dtype=k.dtype, device=device)
    with torch.cuda.device(device):
        _lib.call(
            "b200_rope_paired", _ptr(q), _ptr(k), _ptr(cos.contiguous()), _ptr(sin.contiguous()), _ptr(q_out), _ptr(k_out),
            batch, q_heads, k.shape[1], seq, head_dim, cos.shape[0],
            q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
            q_out.stride(0), q_out.stride(1), q_out.stride(2), k_out.stride(0), k_out.stride(1), k_out.stride(2),
            code, _stream(device),
        )
    return q_out, k_out


def qk_norm_rope(q: Tensor, k: Tensor, q_weight: Tensor, k_weight: Tensor, cos: Tensor, sin: Tensor, eps: float = 1e-6) -> tuple[Tensor, Tensor]:
    """Per-head RMSNorm of q and k, then the paired rotary embedding, in one launch.

    The fused op of the reference's kernel-writing notebook (examples/03_write_a_kernel.ipynb, cell 3),
    equal to rope(rms_norm(q, q_weight), rms_norm(k, k_weight), cos, sin); layout (batch, heads, seq, head_dim).
    """
    device = _require_cuda(q, k, q_weight, k_weight, cos, sin)
    _forbid_grad(q, k, q_weight, k_weight)
    code = _dtype_code(q, "qk_norm_rope")
    if q.dim() != 4 or k.dim() != 4 or q.shape[0] != k.shape[0] or q.shape[2:] != k.shape[2:]:
        raise ValueError("qk_norm_rope: q and k must be [batch, heads, seq, head_dim] and agree in batch, seq and head_dim")
    batch, q_heads, seq, head_dim = q.shape
    if cos.shape != sin.shape or cos.dim() != 3 or cos.shape[1:] != (seq, head_dim) or cos.shape[0] not in (1, batch):
        raise ValueError("qk_norm_rope: cos and sin must be [1 or batch, seq, head_dim]")
    if q_weight.shape != (head_dim,) or k_weight.shape != (head_dim,):
        raise ValueError("qk_norm_rope: q_weight and k_weight must be [head_dim]")
    if not (k.dtype == cos.dtype == sin.dtype == q_weight.dtype == k_weight.dtype == q.dtype):
        raise TypeError("qk_norm_rope: all tensors must share a dtype")
    if head_dim % 2:
        raise ValueError("qk_norm_rope: head_dim must be even")
    q = q if head_dim <= 1 or q.stride(-1) == 1 else q.contiguous()
    k = k if head_dim <= 1 or k.stride(-1) == 1 else k.contiguous()
    q_out = torch.empty(q.shape, dtype=q.dtype, device=device)
    k_out = torch.empty(k.shape, dtype=k.dtype, device=device)
    with torch.cuda.device(device):
        _lib.call(
            "b200_qk_norm_rope", _ptr(q), _ptr(k), _ptr(q_weight.contiguous()), _ptr(k_weight.contiguous()),
            _ptr(cos.contiguous()), _ptr(sin.contiguous()), _ptr(q_out), _ptr(k_out),
            batch, q_heads, k.shape[1], seq, head_dim, cos.shape[0],
            q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
            q_out.stride(0), q_out.stride(1), q_out.stride(2), k_out.stride(0), k_out.stride(1), k_out.stride(2),
            float(eps), code, _stream(device),
        )
    return q_out, k_out


def qk_norm_rope_backward(grad_q_out: Tensor, grad_k_out: Tensor, q: Tensor, k: Tensor, q_weight: Tensor, k_weight: Tensor,
                          cos: Tensor, sin: Tensor, eps: float = 1e-6) -> tuple[Tensor, Tensor, Tensor, Tensor]:
    """(grad_q, grad_k, grad_q_weight, grad_k_weight) of qk_norm_rope; the row statistics are recomputed from q and k."""
    device = _require_cuda(grad_q_out, grad_k_out, q, k, q_weight, k_weight, cos, sin)
    code = _dtype_code(q, "qk_norm_rope_backward")
    if grad_q_out.shape != q.shape or grad_k_out.shape != k.shape or q.dim() != 4 or k.dim() != 4:
        raise ValueError("qk_norm_rope_backward: the output gradients must have the shapes of q and k")
    batch, q_heads, seq, head_dim = q.shape
    if not (grad_q_out.dtype == grad_k_out.dtype == k.dtype == q_weight.dtype == k_weight.dtype == cos.dtype == sin.dtype == q.dtype):
        raise TypeError("qk_norm_rope_backward: all tensors must share a dtype")
    q = q if head_dim <= 1 or q.stride(-1) == 1 else q.contiguous()
    k = k if head_dim <= 1 or k.stride(-1) == 1 else k.contiguous()
    grad_q = torch.empty(q.shape, dtype=q.dtype, device=device)
    grad_k = torch.empty(k.shape, dtype=k.dtype, device=device)
    grad_qw = torch.empty(head_dim, dtype=q.dtype, device=device)
    grad_kw = torch.empty(head_dim, dtype=q.dtype, device=device)
    need = ctypes.c_size_t(0)
    with torch.cuda.device(device):
        _lib.call("b200_qk_norm_rope_backward_scratch_bytes", batch, seq, head_dim, code, ctypes.byref(need))
        scratch = torch.empty(max(need.value, 16), dtype=torch.uint8, device=device)
        _lib.call(
            "b200_qk_norm_rope_backward", _ptr(grad_q_out.contiguous()), _ptr(grad_k_out.contiguous()), _ptr(q), _ptr(k),
            _ptr(q_weight.contiguous()), _ptr(k_weight.contiguous()), _ptr(cos.contiguous()), _ptr(sin.contiguous()),
            _ptr(grad_q), _ptr(grad_k), _ptr(grad_qw), _ptr(grad_kw),
            batch, q_heads, k.shape[1], seq, head_dim, cos.shape[0],
            q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
            float(eps), code, _ptr(scratch), ctypes.c_size_t(scratch.numel()), _stream(device),
        )
    return grad_q, grad_k, grad_qw, grad_kw


def llama4_rope(q: Tensor, k: Tensor, freqs: Tensor) -> tuple[Tensor, Tensor]:
    """Llama 4 rotary embedding of q and k, layout (batch, seq, heads, head_dim), freqs [seq, head_dim/2, 2]
    as (cos, sin) pairs (llama4_rope.py:27-39)."""
    device = _require_cuda(q, k, freqs)
    _forbid_grad(q, k)
    code = _dtype_code(q, "llama4_rope")
    if q.dim() != 4 or k.dim() != 4 or q.shape[:2] != k.shape[:2] or q.shape[3] != k.shape[3]:
        raise ValueError("llama4_rope: q and k must be [batch, seq, heads, head_dim] and agree in batch, seq and head_dim")
    batch, seq, q_heads, head_dim = q.shape
    if head_dim % 2:
        raise ValueError("llama4_rope: head_dim must be even")
    if freqs.shape != (seq, head_dim // 2, 2):
        raise ValueError("llama4_rope: freqs must be [seq, head_dim/2, 2]")
    if not (k.dtype == freqs.dtype == q.dtype):
        raise TypeError("llama4_rope: q, k and freqs must share a dtype")
    q = q if head_dim <= 1 or q.stride(-1) == 1 else q.contiguous()
    k = k if head_dim <= 1 or k.stride(-1) == 1 else k.contiguous()
    q_out = torch.empty(q.shape, dtype=q.dtype, device=device)
    k_out = torch.empty(k.shape, dtype=k.dtype, device=device)
    with torch.cuda.device(device):
        _lib.call(
            "b200_llama4_rope", _ptr(q), _ptr(k), _ptr(freqs.contiguous()), _ptr(q_out), _ptr(k_out),
            batch, seq, q_heads, k.shape[2], head_dim,
            q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
            q_out.stride(0), q_out.stride(1), q_out.stride(2), k_out.stride(0), k_out.stride(1), k_out.stride(2),
            code, _stream(device),
        )
    return q_out, k_out


def swiglu(a: Tensor, b: Tensor) -> Tensor:
    """silu(a) * b (swiglu.py:10-18); a and b may be strided column halves of one buffer."""
    device = _require_cuda(a, b)
    _forbid_grad(a, b)
    code = _dtype_code(a, "swiglu")
    if a.shape != b.shape or a.dtype != b.dtype:
        raise ValueError("swiglu: a and b must have the same shape and dtype")
    width = a.shape[-1]
    a2, lda = _rows(a)
    b2, ldb = _rows(b)
    out = torch.empty(a.shape, dtype=a.dtype, device=device)
    with torch.cuda.device(device):
        _lib.call("b200_swiglu", _ptr(a2), _ptr(b2), _ptr(out), a2.shape[0], width, lda, ldb, max(width, 1), code, _stream(device))
    return out


def geglu(a: Tensor, b: Tensor) -> Tensor:
    """gelu_tanh(a) * b (geglu.py:8-17); a and b may be strided column halves of one buffer."""
    device = _require_cuda(a, b)
    _forbid_grad(a, b)
    code = _dtype_code(a, "geglu")
    if a.shape != b.shape or a.dtype != b.dtype:
        raise ValueError("geglu: a and b must have the same shape and dtype")
    width = a.shape[-1]
    a2, lda = _rows(a)
    b2, ldb = _rows(b)
    out = torch.empty(a.shape, dtype=a.dtype, device=device)
    with torch.cuda.device(device):
        _lib.call("b200_geglu", _ptr(a2), _ptr(b2), _ptr(out), a2.shape[0], width, lda, ldb, max(width, 1), code, _stream(device))
    return out


def rms_norm_gated(x: Tensor, g: Tensor, weight: Tensor, bias: Tensor | None = None, activation: str = "swish", eps: float = 1e-6) -> Tensor:
    """RMS norm scaled by a swish or sigmoid gate (rms_norm_gated.py:12-29)."""
    device = _require_cuda(x, g, weight, bias)
    _forbid_grad(x, g, weight, bias)
    code = _dtype_code(x, "rms_norm_gated")
    width = x.shape[-1]
    if activation not in ("swish", "sigmoid"):
        raise ValueError("rms_norm_gated: activation must be 'swish' or 'sigmoid'")
    if g.shape != x.shape or weight.shape != (width,) or (bias is not None and bias.shape != (width,)):
        raise ValueError("rms_norm_gated: g must match x; weight and bias must be [hidden]")
    if not (g.dtype == weight.dtype == x.dtype) or (bias is not None and bias.dtype != x.dtype):
        raise TypeError("rms_norm_gated: all tensors must share a dtype")
    x2, ldx = _rows(x)
    g2, ldg = _rows(g)
    y = torch.empty(x.shape, dtype=x.dtype, device=device)
    with torch.cuda.device(device):
        _lib.call("b200_rms_norm_gated", _ptr(x2), _ptr(g2), _ptr(weight.contiguous()), _ptr(None if bias is None else bias.contiguous()), _ptr(y),
                  x2.shape[0], width, ldx, ldg, max(width, 1), code, int(activation == "sigmoid"), float(eps), _stream(device))
    return y


def l2_norm(x: Tensor, eps: float = 1e-6) -> Tensor:
    """x / sqrt(sum(x^2) + eps) over the last dimension, evaluated in the dtype of x (l2_norm.py:8-14)."""
    device = _require_cuda(x)
    _forbid_grad(x)
    code = _dtype_code(x, "l2_norm")
    width = x.shape[-1]
    x2, ldx = _rows(x)
    y = torch.empty(x.shape, dtype=x.dtype, device=device)
    with torch.cuda.device(device):
        _lib.call("b200_l2_norm", _ptr(x2), _ptr(y), x2.shape[0], width, ldx, max(width, 1), code, float(eps), _stream(device))
    return y


def layer_norm(x: Tensor, weight: Tensor, bias: Tensor | None = None, eps: float = 1e-6) -> Tensor:
    """Layer normalisation over the last dimension (layer_norm.py:8-20)."""
    device = _require_cuda(x, weight, bias)
    _forbid_grad(x, weight, bias)
    code = _dtype_code(x, "layer_norm")
    width = x.shape[-1]
    if weight.shape != (width,) or (bias is not None and bias.shape != (width,)):
        raise ValueError(f"layer_norm: weight/bias must have shape ({width},)")
    if weight.dtype != x.dtype or (bias is not None and bias.dtype != x.dtype):
        raise TypeError("layer_norm: weight and bias must have the dtype of x")
    x2, ldx = _rows(x)
    y = torch.empty(x.shape, dtype=x.dtype, device=device)
    with torch.cuda.device(device):
        _lib.call("b200_layer_norm", _ptr(x2), _ptr(weight.contiguous()), _ptr(None if bias is None else bias.contiguous()), _ptr(y),
                  x2.shape[0], width, ldx, max(width, 1), code, float(eps), _stream(device))
    return y


def l2_norm_backward(grad_y: Tensor, x: Tensor, eps: float = 1e-6) -> Tensor:
    """grad_x of l2_norm(x, eps) (what autograd derives from l2_norm.py:14)."""
    device = _require_cuda(grad_y, x)
    code = _dtype_code(x, "l2_norm_backward")
    if grad_y.shape != x.shape or grad_y.dtype != x.dtype:
        raise ValueError("l2_norm_backward: grad_y must match x")
    width = x.shape[-1]
    g2, ldg = _rows(grad_y)
    x2, ldx = _rows(x)
    grad_x = torch.empty(x.shape, dtype=x.dtype, device=device)
    with torch.cuda.device(device):
        _lib.call("b200_l2_norm_backward", _ptr(g2), _ptr(x2), _ptr(grad_x), x2.shape[0], width, ldg, ldx, max(width, 1), code, float(eps), _stream(device))
    return grad_x


def layer_norm_backward(grad_y: Tensor, x: Tensor, weight: Tensor, with_bias: bool = False, eps: float = 1e-6) -> tuple[Tensor, Tensor, Tensor | None]:
    """(grad_x, grad_weight, grad_bias or None) of layer_norm(x, weight, bias, eps)."""
    device = _require_cuda(grad_y, x, weight)
    code = _dtype_code(x, "layer_norm_backward")
    width = x.shape[-1]
    if grad_y.shape != x.shape or weight.shape != (width,) or not (grad_y.dtype == weight.dtype == x.dtype):
        raise ValueError("layer_norm_backward: grad_y must match x, and weight must be [hidden] of the same dtype")
    g2, ldg = _rows(grad_y)
    x2, ldx = _rows(x)
    grad_x = torch.empty(x.shape, dtype=x.dtype, device=device)
    grad_w = torch.empty(width, dtype=x.dtype, device=device)
    grad_b = torch.empty(width, dtype=x.dtype, device=device) if with_bias else None
    need = ctypes.c_size_t(0)
    with torch.cuda.device(device):
        _lib.call("b200_layer_norm_backward_scratch_bytes", x2.shape[0], width, ctypes.byref(need))
        scratch = torch.empty(max(need.value, 16), dtype=torch.uint8, device=device)
        _lib.call("b200_layer_norm_backward", _ptr(g2), _ptr(x2), _ptr(weight.contiguous()), _ptr(grad_x), _ptr(grad_w), _ptr(grad_b),
                  x2.shape[0], width, ldg, ldx, max(width, 1), code, float(eps), _ptr(scratch), ctypes.c_size_t(scratch.numel()), _stream(device))
    return grad_x, grad_w, grad_b


def swiglu_backward(grad_out: Tensor, a: Tensor, b: Tensor) -> tuple[Tensor, Tensor]:
    """Gradients of swiglu(a, b) with respect to a and b (what autograd derives from swiglu.py:18)."""
    return _gate_backward("b200_swiglu_backward", grad_out, a, b)


def geglu_backward(grad_out: Tensor, a: Tensor, b: Tensor) -> tuple[Tensor, Tensor]:
    """Gradients of geglu(a, b) with respect to a and b (what autograd derives from geglu.py:17)."""
    return _gate_backward("b200_geglu_backward", grad_out, a, b)


def sigmoid_gate_backward(grad_out: Tensor, a: Tensor, b: Tensor) -> tuple[Tensor, Tensor]:
    """Gradients of sigmoid(a) * b with respect to a and b (the sigmoid gate of rms_norm_gated.py:29)."""
    return _gate_backward("b200_sigmoid_gate_backward", grad_out, a, b)


def _gate_backward(entry: str, grad_out: Tensor, a: Tensor, b: Tensor) -> tuple[Tensor, Tensor]:
    device = _require_cuda(grad_out, a, b)
    code = _dtype_code(a, entry)
    if not (grad_out.shape == a.shape == b.shape) or not (grad_out.dtype == a.dtype == b.dtype):
        raise ValueError(f"{entry}: grad_out, a and b must share shape and dtype")
    width = a.shape[-1]
    g2, ldg = _rows(grad_out)
    a2, lda = _rows(a)
    b2, ldb = _rows(b)
    grad_a = torch.empty(a.shape, dtype=a.dtype, device=device)
    grad_b = torch.empty(a.shape, dtype=a.dtype, device=device)
    ld = max(width, 1)
    with torch.cuda.device(device):
        _lib.call(entry, _ptr(g2), _ptr(a2), _ptr(b2), _ptr(grad_a), _ptr(grad_b), a2.shape[0], width,
                  ldg, lda, ldb, ld, ld, code, _stream(device))
    return grad_a, grad_b


def moe_route(router_logits: Tensor, top_k: int) -> tuple[Tensor, Tensor]:
    """softmax over experts -> top_k -> renormalise (momoe.py:47-49).

    Returns (indices int32 [..., top_k] in descending-probability order, weights float32 [..., top_k])."""
    device = _require_cuda(router_logits)
    _forbid_grad(router_logits)
    code = _dtype_code(router_logits, "moe_route")
    experts = router_logits.shape[-1]
    logits2, ld = _rows(router_logits)
    lead = router_logits.shape[:-1]
    indices = torch.empty((*lead, top_k), dtype=torch.int32, device=device)
    weights = torch.empty((*lead, top_k), dtype=torch.float32, device=device)
    with torch.cuda.device(device):
        _lib.call("b200_moe_route", _ptr(logits2), _ptr(indices), _ptr(weights), logits2.shape[0], experts, int(top_k), ld, code, _stream(device))
    return indices, weights


def moe_index(indices: Tensor, experts: int) -> tuple[Tensor, Tensor, Tensor, Tensor]:
    """Expert histogram, exclusive scan and stable permutation (momoe_tl.py:1071-1161).

    indices: int32 [tokens, top_k].  Returns (counts [experts], offsets [experts + 1],
    perm [tokens*top_k] = token id at each sorted position, pos [tokens, top_k] = sorted
    position of each pair), all int32."""
    device = _require_cuda(indices)
    if indices.dim() != 2 or indices.dtype != torch.int32:
        raise TypeError("moe_index: indices must be an int32 [tokens, top_k] tensor")
    indices = indices.contiguous()
    tokens, top_k = indices.shape
    counts = torch.empty(experts, dtype=torch.int32, device=device)
    offsets = torch.empty(experts + 1, dtype=torch.int32, device=device)
    perm = torch.empty(tokens * top_k, dtype=torch.int32, device=device)
    pos = torch.empty((tokens, top_k), dtype=torch.int32, device=device)
    need = ctypes.c_size_t(0)
    _lib.call("b200_moe_index_scratch_bytes", tokens, top_k, int(experts), ctypes.byref(need))
    scratch = torch.empty(max(need.value, 16), dtype=torch.uint8, device=device)
    with torch.cuda.device(device):
        _lib.call(
            "b200_moe_index", _ptr(indices), tokens, top_k, int(experts), _ptr(counts), _ptr(offsets), _ptr(perm), _ptr(pos),
            _ptr(scratch), ctypes.c_size_t(scratch.numel()), _stream(device),
        )
    return counts, offsets, perm, pos


def moe_route_index(router_logits: Tensor, top_k: int, want_perm: bool = True) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor | None, Tensor]:
    """moe_route followed by moe_index on its picks, as one call: (indices, weights, counts, offsets, perm, pos).
    want_perm=False leaves `perm` out (None): the permute / unpermute kernels only read `pos`.

    router_logits: [tokens, experts].  Same results as the two calls, one trip through the C ABI (momoe.py:47-49 and
    find_used_experts, momoe_tl.py:1071-1161, run back to back in every momoe forward)."""
    device = _require_cuda(router_logits)
    _forbid_grad(router_logits)
    code = _dtype_code(router_logits, "moe_route_index")
    if router_logits.dim() != 2:
        raise ValueError("moe_route_index: router_logits must be [tokens, experts]")
    tokens, experts = router_logits.shape
    top_k = int(top_k)
    logits2, ld = _rows(router_logits)
    indices = torch.empty((tokens, top_k), dtype=torch.int32, device=device)
    weights = torch.empty((tokens, top_k), dtype=torch.float32, device=device)
    counts = torch.empty(experts, dtype=torch.int32, device=device)
    offsets = torch.empty(experts + 1, dtype=torch.int32, device=device)
    perm = torch.empty(tokens * top_k, dtype=torch.int32, device=device) if want_perm else None
    pos = torch.empty((tokens, top_k), dtype=torch.int32, device=device)
    need = ctypes.c_size_t(0)
    _lib.call("b200_moe_index_scratch_bytes", tokens, top_k, int(experts), ctypes.byref(need))
    scratch = torch.empty(max(need.value, 16), dtype=torch.uint8, device=device)
    with torch.cuda.device(device):
        _lib.call(
            "b200_moe_route_index", _ptr(logits2), _ptr(indices), _ptr(weights), tokens, int(experts), top_k, ld, code,
            _ptr(counts), _ptr(offsets), _ptr(perm), _ptr(pos), _ptr(scratch), ctypes.c_size_t(scratch.numel()), _stream(device),
        )
    return indices, weights, counts, offsets, perm, pos


def moe_scatter_rows(x: Tensor, pos: Tensor) -> Tensor:
    """rows[pos[t, k]] = x[t] for every slot k: each token row is read once and written top_k times.

    `pos` is the inverse permutation from moe_index; a negative entry skips that slot."""
    device = _require_cuda(x, pos)
    _forbid_grad(x)
    code = _dtype_code(x, "moe_scatter_rows")
    if x.dim() != 2 or pos.dim() != 2 or pos.shape[0] != x.shape[0] or pos.dtype != torch.int32:
        raise ValueError("moe_scatter_rows: x must be [tokens, hidden] and pos int32 [tokens, top_k]")
    tokens, hidden = x.shape
    top_k = pos.shape[1]
    x2, ldx = _rows(x)
    rows = torch.empty((tokens * top_k, hidden), dtype=x.dtype, device=device)
    with torch.cuda.device(device):
        _lib.call("b200_moe_permute", _ptr(x2), _ptr(pos.contiguous()), _ptr(rows), tokens, top_k, hidden, ldx, max(hidden, 1), code, _stream(device))
    return rows


def moe_permute(x: Tensor, indices: Tensor, experts: int) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
    """Gather token rows into expert-contiguous order (momoe_tl.py:156-158, 408-476).

    x: [tokens, hidden]; indices: int32 [tokens, top_k].  Returns (rows [tokens*top_k, hidden],
    counts, offsets, perm, pos); rows[p] = x[perm[p]], pairs sorted stably by expert."""
    _require_cuda(x, indices)
    if x.dim() != 2 or indices.dim() != 2 or indices.shape[0] != x.shape[0]:
        raise ValueError("moe_permute: x must be [tokens, hidden] and indices [tokens, top_k]")
    counts, offsets, perm, pos = moe_index(indices, experts)
    return moe_scatter_rows(x, pos), counts, offsets, perm, pos


def moe_gather(x: Tensor, src_rows: Tensor) -> Tensor:
    """out[p] = x[src_rows[p]] for an int32 row index (negative entries leave the row unwritten)."""
    device = _require_cuda(x, src_rows)
    _forbid_grad(x)
    code = _dtype_code(x, "moe_gather")
    if x.dim() != 2 or src_rows.dim() != 1 or src_rows.dtype != torch.int32:
        raise TypeError("moe_gather: x must be [rows, hidden] and src_rows an int32 vector")
    x2, ldx = _rows(x)
    hidden = x.shape[1]
    out = torch.empty((src_rows.shape[0], hidden), dtype=x.dtype, device=device)
    with torch.cuda.device(device):
        _lib.call("b200_moe_gather", _ptr(x2), _ptr(src_rows.contiguous()), _ptr(out), src_rows.shape[0], hidden, ldx, max(hidden, 1), code, _stream(device))
    return out


def moe_unpermute(rows: Tensor, weights: Tensor, pos: Tensor) -> Tensor:
    """y[t] = sum_k weights[t, k] * rows[pos[t, k]] in fp32, ascending expert order (momoe.py:52-53)."""
    device = _require_cuda(rows, weights, pos)
    _forbid_grad(rows, weights)
    code = _dtype_code(rows, "moe_unpermute")
    if rows.dim() != 2 or weights.shape != pos.shape or pos.dim() != 2:
        raise ValueError("moe_unpermute: rows must be [n, hidden]; weights and pos [tokens, top_k]")
    if weights.dtype != torch.float32 or pos.dtype != torch.int32:
        raise TypeError("moe_unpermute: weights must be float32 and pos int32")
    tokens, top_k = pos.shape
    hidden = rows.shape[1]
    r2, ldr = _rows(rows)
    y = torch.empty((tokens, hidden), dtype=rows.dtype, device=device)
    with torch.cuda.device(device):
        _lib.call(
            "b200_moe_unpermute", _ptr(r2), _ptr(weights.contiguous()), _ptr(pos.contiguous()), _ptr(y),
            tokens, top_k, hidden, ldr, max(hidden, 1), code, _stream(device),
        )
    return y


def moe_unpermute_backward(grad_y: Tensor, rows: Tensor, weights: Tensor, pos: Tensor) -> tuple[Tensor, Tensor]:
    """(grad_rows, grad_weights) of moe_unpermute(rows, weights, pos) (what autograd derives from momoe.py:52-53)."""
    device = _require_cuda(grad_y, rows, weights, pos)
    code = _dtype_code(rows, "moe_unpermute_backward")
    if rows.dim() != 2 or weights.shape != pos.shape or pos.dim() != 2 or grad_y.shape != (pos.shape[0], rows.shape[1]):
        raise ValueError("moe_unpermute_backward: rows [n, hidden], weights / pos [tokens, top_k], grad_y [tokens, hidden]")
    if weights.dtype != torch.float32 or pos.dtype != torch.int32 or grad_y.dtype != rows.dtype:
        raise TypeError("moe_unpermute_backward: weights float32, pos int32, grad_y in the dtype of rows")
    tokens, top_k = pos.shape
    hidden = rows.shape[1]
    g2, ldg = _rows(grad_y)
    r2, ldr = _rows(rows)
    # every row is written when pos is a permutation of all rows (the normal case); otherwise the rest must read as zero
    make = torch.empty if pos.numel() == rows.shape[0] else torch.zeros
    grad_rows = make(rows.shape, dtype=rows.dtype, device=device)
    grad_weights = torch.empty(pos.shape, dtype=torch.float32, device=device)
    with torch.cuda.device(device):
        _lib.call("b200_moe_unpermute_backward", _ptr(g2), _ptr(r2), _ptr(weights.contiguous()), _ptr(pos.contiguous()), _ptr(grad_rows),
                  _ptr(grad_weights), tokens, top_k, hidden, ldg, ldr, max(hidden, 1), code, _stream(device))
    return grad_rows, grad_weights


def moe_grouped_gemm(rows: Tensor, weight: Tensor, offsets: Tensor, up_weight: Tensor | None = None, out: Tensor | None = None,
                     zero_fill: bool = True) -> Tensor:
    """Expert MLP projection over the expert-major rows of `moe_permute` (momoe.py:50-52, momoe_tl.py:90-330).

    out[p] = rows[p] @ weight[e(p)], or silu(rows[p] @ weight[e(p)]) * (rows[p] @ up_weight[e(p)]) when `up_weight`
    is given (`weight` is then the gate projection); e(p) is the expert whose segment [offsets[e], offsets[e+1])
    holds row p.  weight: [experts, in_features, out_features] as in the reference; fp32 accumulation on the tensor
    cores, one rounding to the dtype of rows.  Rows outside every segment are zero, or left as they are when the
    caller supplies `out` ([n, out_features], contiguous rows) or passes zero_fill=False (callers whose segments
    cover every row, or that never read the rows outside them, save a full write pass over the output)."""
    device = _require_cuda(rows, weight, offsets, *([up_weight] if up_weight is not None else []))
    _forbid_grad(rows, weight)
    code = _dtype_code(rows, "moe_grouped_gemm")
    if rows.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError("moe_grouped_gemm: bf16 or fp16 operands only (fp32 accumulation)")
    if rows.dim() != 2 or weight.dim() != 3 or weight.shape[1] != rows.shape[1]:
        raise ValueError("moe_grouped_gemm: rows must be [n, in_features] and weight [experts, in_features, out_features]")
    if weight.dtype != rows.dtype or (up_weight is not None and (up_weight.dtype != rows.dtype or up_weight.shape != weight.shape)):
        raise ValueError("moe_grouped_gemm: weights must have the dtype of rows (and up_weight the shape of weight)")
    experts, k, n = weight.shape
    if offsets.dtype != torch.int32 or offsets.shape != (experts + 1,):
        raise TypeError("moe_grouped_gemm: offsets must be int32 [experts + 1]")
    r2, ldr = _rows(rows)
    total = r2.shape[0]
    if out is None:
        make = torch.zeros if zero_fill and total else torch.empty
        out = make((total, n), dtype=rows.dtype, device=device)
    elif out.shape != (total, n) or out.dtype != rows.dtype or out.device != device or (total and n > 1 and out.stride(1) != 1):
        raise ValueError("moe_grouped_gemm: out must be [n, out_features] in the dtype and on the device of rows")
    ldo = out.stride(0) if total > 1 else max(n, 1)
    with torch.cuda.device(device):
        _lib.call(
            "b200_moe_grouped_gemm", _ptr(r2), _ptr(weight.contiguous()), _ptr(None if up_weight is None else up_weight.contiguous()),
            _ptr(offsets.contiguous()), _ptr(out), total, k, n, experts, ldr, ldo, code, _stream(device),
        )
    return out


def moe_grouped_gemm_gathered(x: Tensor, perm: Tensor, weight: Tensor, offsets: Tensor, up_weight: Tensor | None = None,
                              zero_fill: bool = True) -> Tensor:
    """moe_grouped_gemm over the rows x[perm] without materialising them: the kernel's operand loads fetch the token
    rows through `perm` (int32 [rows], the permutation of moe_index), like the gathered A operand of the reference's
    lin1 kernel (momoe_tl.py:156-158).  Returns [rows, out_features], expert-major, bit-identical to
    moe_grouped_gemm(x[perm], ...).  Measured on 524288 rows x 4096 -> 2 x 1536: 26.6 ms against 9.5 ms for the
    projection of materialised rows plus 0.74 ms for the permute pass that makes them (one four-row gathered copy
    per ~45 cycles per SM, where the 128 x 256 tile needs one per 16), so `momoe` keeps the permute pass; this form
    pays only where the row buffer itself is the problem (memory, or a handful of rows per expert)."""
    device = _require_cuda(x, perm, weight, offsets, *([up_weight] if up_weight is not None else []))
    _forbid_grad(x, weight)
    code = _dtype_code(x, "moe_grouped_gemm_gathered")
    if x.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError("moe_grouped_gemm_gathered: bf16 or fp16 operands only (fp32 accumulation)")
    if x.dim() != 2 or weight.dim() != 3 or weight.shape[1] != x.shape[1]:
        raise ValueError("moe_grouped_gemm_gathered: x must be [tokens, in_features] and weight [experts, in_features, out_features]")
    if weight.dtype != x.dtype or (up_weight is not None and (up_weight.dtype != x.dtype or up_weight.shape != weight.shape)):
        raise ValueError("moe_grouped_gemm_gathered: weights must have the dtype of x (and up_weight the shape of weight)")
    experts, k, n = weight.shape
    if offsets.dtype != torch.int32 or offsets.shape != (experts + 1,) or perm.dtype != torch.int32 or perm.dim() != 1:
        raise TypeError("moe_grouped_gemm_gathered: offsets must be int32 [experts + 1] and perm int32 [rows]")
    x2, ldx = _rows(x)
    total = perm.shape[0]
    out = (torch.zeros if zero_fill and total else torch.empty)((total, n), dtype=x.dtype, device=device)
    with torch.cuda.device(device):
        _lib.call(
            "b200_moe_grouped_gemm_gathered", _ptr(x2), _ptr(perm.contiguous()), _ptr(weight.contiguous()),
            _ptr(None if up_weight is None else up_weight.contiguous()), _ptr(offsets.contiguous()), _ptr(out),
            x2.shape[0], total, k, n, experts, ldx, max(n, 1), code, _stream(device),
        )
    return out


def _gemm_operands(name: str, rows: Tensor, weight: Tensor, offsets: Tensor, width: int, *more: Tensor | None):
    """Common checks of the grouped-GEMM calls: a 16-bit [n, width] token-major operand, [experts, k, n] weights, int32 offsets."""
    device = _require_cuda(rows, weight, offsets, *[t for t in more if t is not None])
    _forbid_grad(rows, weight, *more)
    code = _dtype_code(rows, name)
    if rows.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError(f"{name}: bf16 or fp16 operands only (fp32 accumulation)")
    if weight.dim() != 3 or rows.dim() != 2 or rows.shape[1] != width:
        raise ValueError(f"{name}: expected a [rows, {width}] operand against [experts, in_features, out_features] weights")
    for t in (weight, *more):
        if t is not None and t.dtype != rows.dtype:
            raise TypeError(f"{name}: all operands must share a dtype")
    if offsets.dtype != torch.int32 or offsets.shape != (weight.shape[0] + 1,):
        raise TypeError(f"{name}: offsets must be int32 [experts + 1]")
    return device, code


def moe_grouped_gemm_gate_up(rows: Tensor, gate_weight: Tensor, up_weight: Tensor, offsets: Tensor) -> Tensor:
    """[rows @ gate_weight[e] | rows @ up_weight[e]] as one [n, 2 * out_features] buffer: the pre-activations a
    training call keeps for the SwiGLU backward (momoe_tl.py:180-190 saves the same two tensors)."""
    experts, k, n = gate_weight.shape
    device, code = _gemm_operands("moe_grouped_gemm_gate_up", rows, gate_weight, offsets, k, up_weight)
    if up_weight.shape != gate_weight.shape:
        raise ValueError("moe_grouped_gemm_gate_up: gate and up weights must have one shape")
    r2, ldr = _rows(rows)
    total = r2.shape[0]
    out = torch.zeros((total, 2 * n), dtype=rows.dtype, device=device)
    with torch.cuda.device(device):
        _lib.call("b200_moe_grouped_gemm_gate_up", _ptr(r2), _ptr(gate_weight.contiguous()), _ptr(up_weight.contiguous()),
                  _ptr(offsets.contiguous()), _ptr(out), total, k, n, experts, ldr, max(2 * n, 1), code, _stream(device))
    return out


def moe_grouped_gemm_dgrad(grad_out: Tensor, weight: Tensor, offsets: Tensor, grad_out2: Tensor | None = None,
                           weight2: Tensor | None = None) -> Tensor:
    """grad_rows[p] = grad_out[p] @ weight[e(p)]^T (+ grad_out2[p] @ weight2[e(p)]^T): the gradient of
    `moe_grouped_gemm` with respect to its rows; rows outside every segment get zeros.  The two gradients may be
    column halves of one buffer (they must share a row stride)."""
    experts, k, n = weight.shape
    device, code = _gemm_operands("moe_grouped_gemm_dgrad", grad_out, weight, offsets, n, grad_out2, weight2)
    if (grad_out2 is None) != (weight2 is None):
        raise ValueError("moe_grouped_gemm_dgrad: grad_out2 and weight2 go together")
    g1, ld = _rows(grad_out)
    g2 = None
    if grad_out2 is not None:
        if grad_out2.shape != grad_out.shape or weight2.shape != weight.shape:
            raise ValueError("moe_grouped_gemm_dgrad: the second pair must have the shapes of the first")
        g2, ld2 = _rows(grad_out2)
        if ld2 != ld:
            g1, g2 = g1.contiguous(), g2.contiguous()
            ld = max(n, 1)
    total = g1.shape[0]
    out = torch.zeros((total, k), dtype=grad_out.dtype, device=device)
    with torch.cuda.device(device):
        _lib.call("b200_moe_grouped_gemm_dgrad", _ptr(g1), _ptr(weight.contiguous()), _ptr(g2), _ptr(None if weight2 is None else weight2.contiguous()),
                  _ptr(offsets.contiguous()), _ptr(out), total, k, n, experts, ld, max(k, 1), code, _stream(device))
    return out


def moe_grouped_gemm_wgrad(rows: Tensor, grad_out: Tensor, offsets: Tensor) -> Tensor:
    """grad_weight[e] = rows[segment e]^T @ grad_out[segment e], [experts, in_features, out_features]: the gradient of
    `moe_grouped_gemm` with respect to its weight (experts without rows get zeros)."""
    device = _require_cuda(rows, grad_out, offsets)
    _forbid_grad(rows, grad_out)
    code = _dtype_code(rows, "moe_grouped_gemm_wgrad")
    if rows.dtype not in (torch.bfloat16, torch.float16) or grad_out.dtype != rows.dtype:
        raise TypeError("moe_grouped_gemm_wgrad: bf16 or fp16 operands of one dtype only (fp32 accumulation)")
    if rows.dim() != 2 or grad_out.dim() != 2 or rows.shape[0] != grad_out.shape[0]:
        raise ValueError("moe_grouped_gemm_wgrad: rows [n, in_features] and grad_out [n, out_features] must have the same n")
    if offsets.dtype != torch.int32 or offsets.dim() != 1 or offsets.numel() < 1:
        raise TypeError("moe_grouped_gemm_wgrad: offsets must be int32 [experts + 1]")
    experts = offsets.numel() - 1
    r2, ldr = _rows(rows)
    g2, ldg = _rows(grad_out)
    total, k, n = r2.shape[0], r2.shape[1], g2.shape[1]
    out = torch.empty((experts, k, n), dtype=rows.dtype, device=device)
    with torch.cuda.device(device):
        _lib.call("b200_moe_grouped_gemm_wgrad", _ptr(r2), _ptr(g2), _ptr(offsets.contiguous()), _ptr(out), total, k, n, experts, ldr, ldg,
                  code, _stream(device))
    return out


def check_momoe(x: Tensor, gate_weight: Tensor, up_weight: Tensor, down_weight: Tensor, router_logits: Tensor) -> None:
    """Argument checks of `momoe`, shared with its differentiable form."""
    _require_cuda(x, gate_weight, up_weight, down_weight, router_logits)
    if x.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError("momoe: bf16 or fp16 activations and weights only (the expert projections run on 16-bit tensor-core operands)")
    if not (gate_weight.dtype == up_weight.dtype == down_weight.dtype == x.dtype):
        raise TypeError("momoe: x and the three weights must share a dtype")
    experts, hidden, inter = gate_weight.shape
    if x.shape[-1] != hidden or up_weight.shape != gate_weight.shape or down_weight.shape != (experts, inter, hidden):
        raise ValueError("momoe: expected x [..., hidden], gate/up [experts, hidden, intermediate], down [experts, intermediate, hidden]")
    if router_logits.shape != (*x.shape[:-1], experts):
        raise ValueError("momoe: router_logits must be [..., experts] over the tokens of x")


def momoe(x: Tensor, gate_weight: Tensor, up_weight: Tensor, down_weight: Tensor, router_logits: Tensor, top_k: int = 2) -> Tensor:
    """Mixture of SwiGLU expert MLPs, routed to the top-k experts by softmax probability (momoe.py:34-53).

    The reference evaluates every expert on every token in fp32; here only the routed (token, expert) pairs are
    computed: route -> permute into expert-major rows -> gate/up projection + SwiGLU and down projection on the tensor
    cores (16-bit operands, fp32 accumulation, 16-bit intermediate, like the incumbent kernels,
    momoe_tl.py:90-330) -> weighted unpermute in fp32.  x: [batch, seq, hidden] bf16 or fp16."""
    _forbid_grad(x, gate_weight, up_weight, down_weight, router_logits)
    check_momoe(x, gate_weight, up_weight, down_weight, router_logits)
    experts, hidden, _ = gate_weight.shape
    flat = x.reshape(-1, hidden)
    _, weights, _, offsets, _, pos = moe_route_index(router_logits.reshape(-1, experts).float(), int(top_k), want_perm=False)
    rows = moe_scatter_rows(flat, pos)
    # The rows are permuted by a pass of their own (0.74 ms for 65536 tokens x top-8 x 4096): fetching them through the
    # permutation inside the first projection (moe_grouped_gemm_gathered) is bit-identical but its four-row gathered
    # copies feed a 128 x 256 tile at a third of the rate the tensor pipe consumes it (26.6 ms against 9.5 + 0.74).
    # Rows outside the segments (pairs with an invalid expert) are never read again: neither output needs a zero fill.
    hidden_act = moe_grouped_gemm(rows, gate_weight, offsets, up_weight, zero_fill=False)
    out_rows = moe_grouped_gemm(hidden_act, down_weight, offsets, zero_fill=False)
    return moe_unpermute(out_rows, weights, pos).reshape(x.shape)


def _pointer_array(pointers: list[int]) -> ctypes.Array:
    return (ctypes.c_void_p * len(pointers))(*pointers)


def moe_ep_destinations(
    indices: Tensor, pos: Tensor, local_offsets: Tensor, dst_base: Tensor, experts_per_rank: int
) -> tuple[Tensor, Tensor]:
    """Owner rank and row in the owner's exchange buffer for every (token, slot) pair (all int32).

    dst_rank = indices // experts_per_rank; dst_row = dst_base[expert] + (pos - local_offsets[expert])."""
    device = _require_cuda(indices, pos, local_offsets, dst_base)
    tokens, top_k = indices.shape
    experts = dst_base.shape[0]
    for name, t in (("indices", indices), ("pos", pos), ("local_offsets", local_offsets), ("dst_base", dst_base)):
        if t.dtype != torch.int32:
            raise TypeError(f"moe_ep_destinations: {name} must be int32")
    dst_rank = torch.empty((tokens, top_k), dtype=torch.int32, device=device)
    dst_row = torch.empty((tokens, top_k), dtype=torch.int32, device=device)
    with torch.cuda.device(device):
        _lib.call(
            "b200_moe_ep_destinations", _ptr(indices.contiguous()), _ptr(pos.contiguous()), _ptr(local_offsets.contiguous()),
            _ptr(dst_base.contiguous()), tokens, top_k, experts, int(experts_per_rank), _ptr(dst_rank), _ptr(dst_row), _stream(device),
        )
    return dst_rank, dst_row


EP_WAIT_BUDGET_NS = 2_000_000_000  # how long a rank waits for its peers inside a kernel before it gives up


def moe_ep_meta_bytes() -> int:
    """Size of the per-rank flag-and-counts buffer of the expert-parallel exchange (to be zeroed and mapped by all ranks)."""
    need = ctypes.c_size_t(0)
    _lib.call("b200_moe_ep_meta_bytes", ctypes.byref(need))
    return int(need.value)


def moe_ep_exchange(counts: Tensor, meta_ptrs: list[int], rank: int, capacity_rows: int, epoch: int, status: Tensor,
                    budget_ns: int = EP_WAIT_BUDGET_NS) -> tuple[Tensor, Tensor, Tensor]:
    """Exchange the per-expert counts with every rank through peer memory and derive this rank's addressing on the device.

    counts: int32 [experts] of this rank (moe_index); meta_ptrs: every rank's meta buffer as mapped here; status: int32 [2]
    device tensor that collects the first failure (see the header).  Returns (dst_base int32 [experts], expert_offsets
    int32 [experts / world + 1], info int32 [4] = rows received, rows sent to other ranks, largest receive, world), all
    on the device: nothing is read back."""
    device = _require_cuda(counts, status)
    if counts.dtype != torch.int32 or counts.dim() != 1 or status.dtype != torch.int32 or status.numel() < 2:
        raise TypeError("moe_ep_exchange: counts must be int32 [experts] and status int32 [2]")
    world, experts = len(meta_ptrs), counts.shape[0]
    dst_base = torch.empty(experts, dtype=torch.int32, device=device)
    expert_offsets = torch.empty(experts // max(world, 1) + 1, dtype=torch.int32, device=device)
    info = torch.empty(4, dtype=torch.int32, device=device)
    with torch.cuda.device(device):
        _lib.call("b200_moe_ep_exchange", _ptr(counts.contiguous()), _pointer_array(meta_ptrs), world, int(rank), experts, int(capacity_rows),
                  ctypes.c_int32(int(epoch) & 0xffffffff), int(budget_ns), _ptr(dst_base), _ptr(expert_offsets), _ptr(info), _ptr(status), _stream(device))
    return dst_base, expert_offsets, info


def moe_ep_barrier(meta_ptrs: list[int], rank: int, channel: int, epoch: int, status: Tensor, budget_ns: int = EP_WAIT_BUDGET_NS) -> None:
    """Stream-ordered rendezvous of all ranks through flags in peer memory (bounded wait; failures go to `status`)."""
    device = _require_cuda(status)
    with torch.cuda.device(device):
        _lib.call("b200_moe_ep_barrier", _pointer_array(meta_ptrs), len(meta_ptrs), int(rank), int(channel), ctypes.c_int32(int(epoch) & 0xffffffff),
                  int(budget_ns), _ptr(status), _stream(device))


def moe_permute_multi(x: Tensor, dst_buf: Tensor, dst_row: Tensor, buffer_ptrs: list[int], ld_rows: int | None = None) -> None:
    """buffer[dst_buf[t, k]][dst_row[t, k]] = x[t]: the dispatch half of the expert-parallel exchange.

    buffer_ptrs: device addresses of every rank's exchange buffer as mapped into this process (row-major,
    `ld_rows` elements per row, default hidden).  The rows are stored straight into peer memory."""
    device = _require_cuda(x, dst_buf, dst_row)
    _forbid_grad(x)
    code = _dtype_code(x, "moe_permute_multi")
    if x.dim() != 2 or dst_buf.shape != dst_row.shape or dst_row.dim() != 2 or dst_row.shape[0] != x.shape[0]:
        raise ValueError("moe_permute_multi: x must be [tokens, hidden]; dst_buf and dst_row [tokens, top_k]")
    if dst_buf.dtype != torch.int32 or dst_row.dtype != torch.int32:
        raise TypeError("moe_permute_multi: dst_buf and dst_row must be int32")
    tokens, hidden = x.shape
    x2, ldx = _rows(x)
    with torch.cuda.device(device):
        _lib.call(
            "b200_moe_permute_multi", _ptr(x2), _ptr(dst_buf.contiguous()), _ptr(dst_row.contiguous()), _pointer_array(buffer_ptrs),
            len(buffer_ptrs), tokens, dst_row.shape[1], hidden, ldx, ld_rows or max(hidden, 1), code, _stream(device),
        )


def moe_unpermute_multi(
    buffer_ptrs: list[int], src_buf: Tensor, src_row: Tensor, weights: Tensor, hidden: int, dtype: torch.dtype, ld_rows: int | None = None
) -> Tensor:
    """y[t] = sum_k weights[t, k] * buffer[src_buf[t, k]][src_row[t, k]]: the combine half of the exchange.

    The rows are loaded straight out of peer memory; accumulation is fp32 in ascending expert order."""
    device = _require_cuda(src_buf, src_row, weights)
    if src_buf.shape != src_row.shape or weights.shape != src_row.shape or src_row.dim() != 2:
        raise ValueError("moe_unpermute_multi: src_buf, src_row and weights must all be [tokens, top_k]")
    if src_buf.dtype != torch.int32 or src_row.dtype != torch.int32 or weights.dtype != torch.float32:
        raise TypeError("moe_unpermute_multi: src_buf / src_row must be int32 and weights float32")
    try:
        code = _DTYPES[dtype]
    except KeyError:
        raise TypeError(f"moe_unpermute_multi: dtype {dtype} is not supported") from None
    tokens, top_k = src_row.shape
    y = torch.empty((tokens, hidden), dtype=dtype, device=device)
    with torch.cuda.device(device):
        _lib.call(
            "b200_moe_unpermute_multi", _pointer_array(buffer_ptrs), len(buffer_ptrs), _ptr(src_buf.contiguous()), _ptr(src_row.contiguous()),
            _ptr(weights.contiguous()), _ptr(y), tokens, top_k, hidden, ld_rows or max(hidden, 1), max(hidden, 1), code, _stream(device),
        )
    return y
