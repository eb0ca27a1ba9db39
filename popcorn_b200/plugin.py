"""Attach the `b200` backend to popcorn's own registry.

    import popcorn_b200.plugin
    popcorn_b200.plugin.register()            # needs `popcorn` importable
    popcorn.KERNELS["rms_norm"](x, w, backend="b200")

For the eleven ops popcorn already defines, this is one `op.register(name,
source=..., forward_only=True)` line each, the same form popcorn's own backends
use (src/popcorn/kernels/rms_norm.py:33-59, add_rms_norm.py:26-28,
rotary_embedding.py:43-45, rope.py:39, swiglu.py:21-31).  The sources are bare: each
popcorn_b200.ops function takes the reference's parameters positionally in the
reference's order, which is what popcorn checks when the source is first
resolved (src/popcorn/core/dispatcher.py:184-201).

popcorn has no standalone MoE routing / permute / unpermute ops: those steps are
fused inside `momoe` (src/popcorn/kernels/momoe.py:47-53,
src/popcorn/impls/momoe_tl.py:1071-1161).  `register()` therefore also defines
three new ops with `register_kernel`.  popcorn requires every op to carry a
PyTorch definition of its semantics; the three small torch functions below are
those definitions.  popcorn's harness may call them as the op's `torch` entry;
no code path of popcorn_b200 ever does.
"""

from typing import Any

import torch
from torch import Tensor

BACKEND = "b200"
EXISTING_OPS = ("rms_norm", "add_rms_norm", "rotary_embedding", "rope", "llama4_rope", "swiglu", "geglu", "rms_norm_gated", "l2_norm", "layer_norm", "momoe")
NEW_OPS = ("moe_route", "moe_permute", "moe_unpermute", "qk_norm_rope")
DIFFERENTIABLE_OPS = ("rms_norm", "add_rms_norm", "swiglu", "geglu", "rotary_embedding", "rope", "llama4_rope", "qk_norm_rope", "rms_norm_gated", "l2_norm", "layer_norm",
                      "moe_route", "moe_permute", "moe_unpermute", "momoe")

_SUPPORTED = (torch.float32, torch.float16, torch.bfloat16)


def accepts(**arguments: Any) -> bool:
    """Dispatch predicate: CUDA tensors in a dtype the kernels implement."""
    tensors = [value for value in arguments.values() if isinstance(value, Tensor)]
    return bool(tensors) and all(
        t.is_cuda and (not t.is_floating_point() or t.dtype in _SUPPORTED) for t in tensors
    )


def accepts_16bit(**arguments: Any) -> bool:
    """`accepts`, narrowed to bf16 / fp16 activations with weights of the same dtype: the expert projections of
    momoe run on 16-bit tensor-core operands (router logits may be any supported float dtype)."""
    x = arguments.get("x")
    if not accepts(**arguments) or not isinstance(x, Tensor) or x.dtype not in (torch.float16, torch.bfloat16):
        return False
    return all(t.dtype == x.dtype for name, t in arguments.items() if isinstance(t, Tensor) and name.endswith("_weight"))


PREDICATES = {"momoe": accepts_16bit}


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
            predicate = PREDICATES.get(name, accepts)
            if name in DIFFERENTIABLE_OPS:  # backward kernels exist: serve training calls too
                op.register(backend, source=f"popcorn_b200.autograd.{name}", predicate=predicate)
            else:
                op.register(backend, source=f"popcorn_b200.ops.{name}", predicate=predicate, forward_only=True)
        served.append(name)
    return served
