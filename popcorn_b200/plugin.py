"""Attach the `b200` backend to popcorn's own registry.

    import popcorn_b200.plugin
    popcorn_b200.plugin.register()            # needs `popcorn` importable
    popcorn.KERNELS["rms_norm"](x, w, backend="b200")

For the eleven ops popcorn already defines, this is one `op.register(name,
source=..., predicate=...)` line each, the same form popcorn's own backends
use (src/popcorn/kernels/rms_norm.py:33-59, add_rms_norm.py:26-28,
rotary_embedding.py:43-45, rope.py:39, swiglu.py:21-31).  The sources are the
differentiable functions of popcorn_b200.autograd (every op has backward kernels,
so none is registered `forward_only`); they are bare: each takes the reference's
parameters positionally in the reference's order, which is what popcorn checks
when the source is first resolved (src/popcorn/core/dispatcher.py:184-201).

popcorn has no standalone MoE routing / permute / unpermute ops: those steps are
fused inside `momoe` (src/popcorn/kernels/momoe.py:47-53,
src/popcorn/impls/momoe_tl.py:1071-1161).  `register()` therefore also defines
three new ops with `register_kernel`.  popcorn requires every op to carry a
PyTorch definition of its semantics; the three small torch functions below are
those definitions.  popcorn's harness may call them as the op's `torch` entry;
no code path of popcorn_b200 ever does.
"""

import functools
from typing import Any

import torch
from torch import Tensor

BACKEND = "b200"
EXISTING_OPS = ("rms_norm", "add_rms_norm", "rotary_embedding", "rope", "llama4_rope", "swiglu", "geglu", "rms_norm_gated", "l2_norm", "layer_norm", "momoe")
NEW_OPS = ("moe_route", "moe_permute", "moe_unpermute", "qk_norm_rope")
DIFFERENTIABLE_OPS = ("rms_norm", "add_rms_norm", "swiglu", "geglu", "rotary_embedding", "rope", "llama4_rope", "qk_norm_rope", "rms_norm_gated", "l2_norm", "layer_norm",
                      "moe_route", "moe_permute", "moe_unpermute", "momoe")

_SUPPORTED = (torch.float32, torch.float16, torch.bfloat16)
_SIXTEEN_BIT = (torch.float16, torch.bfloat16)
MAX_EXPERTS, MAX_TOP_K = 1024, 32  # limits of b200_moe_route / b200_moe_index (include/popcorn_b200.h)


@functools.cache
def _is_blackwell(index: int) -> bool:
    return torch.cuda.get_device_capability(index)[0] == 10


def accepts(**arguments: Any) -> bool:
    """The part of every predicate that looks at placement: CUDA tensors on one compute-capability-10 device, in a
    dtype the kernels implement."""
    tensors = [value for value in arguments.values() if isinstance(value, Tensor)]
    if not tensors or not all(t.is_cuda and (not t.is_floating_point() or t.dtype in _SUPPORTED) for t in tensors):
        return False
    return len({t.device for t in tensors}) == 1 and _is_blackwell(tensors[0].device.index)


# --- what each op of popcorn_b200.ops insists on, as a reason string (None = the op takes the call) ---------------------
# popcorn treats a predicate as a veto and moves on to the next backend (src/popcorn/core/dispatcher.py:126-137), while an
# exception from the selected backend reaches the caller.  The references accept more than the kernels do (they promote
# mixed dtypes, broadcast, take any strides), so each rule below restates the argument checks of the op it guards:
# a call the op would refuse is declined here and popcorn serves it from another backend.

def _one_dtype(first: Tensor, **others: Tensor | None) -> str | None:
    for name, t in others.items():
        if t is not None and t.dtype != first.dtype:
            return f"{name} is {t.dtype}, not {first.dtype}"
    return None


def _vector(width: int, **vectors: Tensor | None) -> str | None:
    for name, t in vectors.items():
        if t is not None and tuple(t.shape) != (width,):
            return f"{name} must be [{width}]"
    return None


def _norm_rule(x, weight, bias=None, **_):
    return _one_dtype(x, weight=weight, bias=bias) or _vector(x.shape[-1] if x.dim() else 0, weight=weight, bias=bias)


def _add_rms_norm_rule(x, residual, weight, **_):
    if residual.shape != x.shape:
        return "x and residual differ in shape"
    return _one_dtype(x, residual=residual, weight=weight) or _vector(x.shape[-1] if x.dim() else 0, weight=weight)


def _rms_norm_gated_rule(x, g, weight, bias=None, activation="swish", **_):
    if activation not in ("swish", "sigmoid"):
        return f"activation {activation!r}"
    if g.shape != x.shape:
        return "x and g differ in shape"
    return _one_dtype(x, g=g, weight=weight, bias=bias) or _vector(x.shape[-1] if x.dim() else 0, weight=weight, bias=bias)


def _gate_rule(a, b, **_):
    return None if a.shape == b.shape and a.dtype == b.dtype else "a and b differ in shape or dtype"


def _rotary_rule(x, cos, sin, **_):
    if x.dim() != 4:
        return "x is not [batch, seq, heads, head_dim]"
    if cos.shape != sin.shape or cos.dim() != 2 or cos.shape[0] != x.shape[1]:
        return "cos and sin are not both [seq, half]"
    if 2 * cos.shape[1] > x.shape[-1]:
        return "2 * half exceeds head_dim"
    if cos.dtype != sin.dtype or cos.dtype not in (torch.float32, x.dtype):
        return "cos / sin are neither float32 nor the dtype of x"
    if x.shape[-1] > 1 and x.stride(-1) != 1:
        return "head_dim of x is not contiguous"
    return None


def _paired_rule(q, k, cos, sin, **weights):
    if q.dim() != 4 or k.dim() != 4 or q.shape[0] != k.shape[0] or q.shape[2:] != k.shape[2:]:
        return "q and k are not [batch, heads, seq, head_dim] with one batch, seq and head_dim"
    batch, _, seq, head_dim = q.shape
    if cos.shape != sin.shape or cos.dim() != 3 or tuple(cos.shape[1:]) != (seq, head_dim) or cos.shape[0] not in (1, batch):
        return "cos and sin are not [1 or batch, seq, head_dim]"
    if head_dim % 2:
        return "head_dim is odd"
    tensors = {name: t for name, t in weights.items() if isinstance(t, Tensor)}
    return _one_dtype(q, k=k, cos=cos, sin=sin, **tensors) or _vector(head_dim, **tensors)


def _llama4_rule(q, k, freqs, **_):
    if q.dim() != 4 or k.dim() != 4 or q.shape[:2] != k.shape[:2] or q.shape[3] != k.shape[3]:
        return "q and k are not [batch, seq, heads, head_dim] with one batch, seq and head_dim"
    if q.shape[3] % 2 or tuple(freqs.shape) != (q.shape[1], q.shape[3] // 2, 2):
        return "freqs is not [seq, head_dim / 2, 2]"
    return _one_dtype(q, k=k, freqs=freqs)


def _route_rule(router_logits, top_k=2, **_):
    experts = router_logits.shape[-1] if router_logits.dim() else 0
    if not 1 <= int(top_k) <= min(experts, MAX_TOP_K) or experts > MAX_EXPERTS:
        return f"top_k {top_k} of {experts} experts is outside 1..{MAX_TOP_K} of 1..{MAX_EXPERTS}"
    return None


def _permute_rule(x, indices, experts, **_):
    if x.dim() != 2 or indices.dim() != 2 or indices.shape[0] != x.shape[0] or indices.dtype != torch.int32:
        return "x is not [tokens, hidden] with int32 indices [tokens, top_k]"
    if not 1 <= int(experts) <= MAX_EXPERTS or not 1 <= indices.shape[1] <= MAX_TOP_K:
        return f"{experts} experts / top_k {indices.shape[1]} are outside the kernels' limits"
    return None


def _unpermute_rule(rows, weights, pos, **_):
    if rows.dim() != 2 or weights.shape != pos.shape or pos.dim() != 2:
        return "rows is not [n, hidden] with weights and pos [tokens, top_k]"
    if weights.dtype != torch.float32 or pos.dtype != torch.int32:
        return "weights are not float32 or pos is not int32"
    return None


def _momoe_rule(x, gate_weight, up_weight, down_weight, router_logits, top_k=2, **_):
    if x.dtype not in _SIXTEEN_BIT:
        return "the expert projections take bf16 / fp16 operands only"
    if gate_weight.dim() != 3:
        return "gate_weight is not [experts, hidden, intermediate]"
    experts, hidden, inter = gate_weight.shape
    if x.shape[-1] != hidden or up_weight.shape != gate_weight.shape or tuple(down_weight.shape) != (experts, inter, hidden):
        return "weights are not [experts, hidden, intermediate] x 2 and [experts, intermediate, hidden]"
    if tuple(router_logits.shape) != (*x.shape[:-1], experts):
        return "router_logits is not [..., experts] over the tokens of x"
    return _one_dtype(x, gate_weight=gate_weight, up_weight=up_weight, down_weight=down_weight) or _route_rule(router_logits, top_k)


RULES = {
    "rms_norm": _norm_rule, "layer_norm": _norm_rule, "add_rms_norm": _add_rms_norm_rule, "rms_norm_gated": _rms_norm_gated_rule,
    "l2_norm": lambda **_: None, "swiglu": _gate_rule, "geglu": _gate_rule, "rotary_embedding": _rotary_rule, "rope": _paired_rule,
    "qk_norm_rope": _paired_rule, "llama4_rope": _llama4_rule, "moe_route": _route_rule, "moe_permute": _permute_rule,
    "moe_unpermute": _unpermute_rule, "momoe": _momoe_rule,
}


def declined(name: str, **arguments: Any) -> str | None:
    """Why the b200 implementation of op `name` must not be given this call, or None when it serves it."""
    if not accepts(**arguments):
        return "needs CUDA tensors in float32 / float16 / bfloat16 on one compute-capability-10 device"
    return RULES[name](**arguments)


def _predicate(name: str):
    def predicate(**arguments: Any) -> bool:
        return declined(name, **arguments) is None

    predicate.__name__ = predicate.__qualname__ = f"accepts_{name}"
    return predicate


PREDICATES = {name: _predicate(name) for name in RULES}
accepts_16bit = PREDICATES["momoe"]


def _define_moe_ops(popcorn: Any) -> None:
    from jaxtyping import Float, Int

    register_kernel, Tag = popcorn.register_kernel, popcorn.Tag

    @register_kernel(test_args={"top_k": [2, 8]}, tags={Tag.FEATURE_MIXER})
    def moe_route(
        router_logits: Float[Tensor, "tokens experts"],
        top_k: int = 2,
    ) -> tuple[Int[Tensor, "tokens top_k"], Float[Tensor, "tokens top_k"]]:
        r"""Softmax top-k routing with the picked probabilities renormalized to sum one.

        $$w_e = \frac{p_e}{\sum_{e' \in \mathrm{top}k(p)} p_{e'}}, \qquad p = \mathrm{softmax}(r)$$
        """
        probs = torch.softmax(router_logits.to(torch.promote_types(router_logits.dtype, torch.float32)), -1)
        picked = probs.topk(top_k, -1)
        return picked.indices.to(torch.int32), picked.values / picked.values.sum(-1, keepdim=True)

    @register_kernel(tags={Tag.FEATURE_MIXER})
    def moe_permute(
        x: Float[Tensor, "tokens hidden"],
        indices: Int[Tensor, "tokens top_k"],
        experts: int,
    ) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
        r"""Stable sort of (token, slot) pairs by expert, and the token rows gathered into that order.

        $$\mathrm{rows}_p = x_{\pi(p)}, \qquad \pi = \mathrm{argsort}_{\mathrm{stable}}(\mathrm{indices})$$
        """
        tokens, top_k = indices.shape
        flat = indices.reshape(-1).long()
        counts = torch.bincount(flat, minlength=experts)[:experts]
        offsets = torch.cat((counts.new_zeros(1), counts.cumsum(0)))
        order = torch.sort(flat, stable=True).indices
        perm = order // top_k
        pos = torch.empty_like(order)
        pos[order] = torch.arange(order.numel(), device=order.device)
        return x[perm], counts.int(), offsets.int(), perm.int(), pos.view(tokens, top_k).int()

    @register_kernel(tags={Tag.FEATURE_MIXER})
    def moe_unpermute(
        rows: Float[Tensor, "rows hidden"],
        weights: Float[Tensor, "tokens slots"],
        pos: Int[Tensor, "tokens slots"],
    ) -> Float[Tensor, "tokens hidden"]:
        r"""Gate-weighted sum of expert rows back into token order, accumulated in fp32.

        $$y_t = \sum_k w_{t,k}\, \mathrm{rows}_{\mathrm{pos}(t,k)}$$
        """
        picked = rows[pos.long()].to(torch.promote_types(rows.dtype, torch.float32))
        return torch.einsum("tkd,tk->td", picked, weights.to(picked.dtype)).to(rows.dtype)


def _define_qk_norm_rope(popcorn: Any) -> None:
    """The fused op popcorn's kernel-writing notebook builds (examples/03_write_a_kernel.ipynb) but does not ship."""
    from jaxtyping import Float

    from popcorn.kernels._utils import rms

    register_kernel, Tag = popcorn.register_kernel, popcorn.Tag
    paired_rope = popcorn.KERNELS["rope"].reference

    def repeated_halves(f):
        return lambda t: f(t).chunk(2, -1)[0].repeat(1, 1, 2)

    @register_kernel(
        test_args={"eps": [1e-6]},
        test_inputs={"cos": repeated_halves(torch.cos), "sin": repeated_halves(torch.sin)},
        tags={Tag.NORMALIZATION, Tag.POSITIONAL, Tag.FUSED},
    )
    def qk_norm_rope(
        q: Float[Tensor, "batch q_heads seq head_dim"],
        k: Float[Tensor, "batch kv_heads seq head_dim"],
        q_weight: Float[Tensor, "head_dim"],
        k_weight: Float[Tensor, "head_dim"],
        cos: Float[Tensor, "cos_batch seq head_dim"],
        sin: Float[Tensor, "cos_batch seq head_dim"],
        eps: float = 1e-6,
    ) -> tuple[Float[Tensor, "batch q_heads seq head_dim"], Float[Tensor, "batch kv_heads seq head_dim"]]:
        r"""RMS normalization of every query and key head, then the paired rotary embedding.

        $$y = \hat{x} \odot \cos_t + \mathrm{rot}_{1/2}(\hat{x}) \odot \sin_t, \qquad
          \hat{x} = \frac{x}{\sqrt{\overline{x^2} + \varepsilon}} \odot w$$
        """
        return paired_rope(rms(q, eps) * q_weight, rms(k, eps) * k_weight, cos, sin)


def register(backend: str = BACKEND) -> list[str]:
    """Register the b200 backend on popcorn's ops; returns the names of the ops it now serves."""
    import popcorn
    import popcorn.kernels  # noqa: F401  (fills popcorn.KERNELS)

    served = []
    if not all(name in popcorn.KERNELS for name in NEW_OPS[:3]):
        _define_moe_ops(popcorn)
    if "qk_norm_rope" not in popcorn.KERNELS:
        _define_qk_norm_rope(popcorn)
    for name in (*EXISTING_OPS, *NEW_OPS):
        op = popcorn.KERNELS[name]
        if backend not in op.available_backends():
            predicate = PREDICATES[name]
            if name in DIFFERENTIABLE_OPS:  # backward kernels exist: serve training calls too
                op.register(backend, source=f"popcorn_b200.autograd.{name}", predicate=predicate)
            else:
                op.register(backend, source=f"popcorn_b200.ops.{name}", predicate=predicate, forward_only=True)
        served.append(name)
    return served
