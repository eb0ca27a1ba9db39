"""CPU restatement of popcorn's PyTorch references for the b200 backend's ops.

TEST INFRASTRUCTURE ONLY.  This module is the checker the CUDA kernels are
compared against (tests/, the smoke entry point, and bench.py's CPU-baseline and
reference arms).  Nothing under popcorn_b200/ imports it and it is never the
thing that is shipped or measured as the product.

Parity status
  * rms_norm, add_rms_norm, rotary_embedding, swiglu, and the routing lines of
    momoe restate registered popcorn references; they are pinned by the golden
    vectors in tests/golden/, which were produced by running the real reference
    (popcorn 0.1.1 imported from its source tree; see tests/golden/make_golden.py).
  * moe_index / moe_permute / moe_unpermute have no standalone registered op in
    the reference (the steps exist only fused inside the Triton `momoe`
    implementation).  Their index semantics are pinned against the reference's
    own kernel: tests/golden/moeindex_*.npz hold the `counts`, `cumsums_N` and
    `col_idx` outputs of `find_used_experts` + `scatter_cols_kernel`
    (src/popcorn/impls/momoe_tl.py:1071-1161) run on a B200 on the routing of
    every momoe fixture and of the MoE benchmark configuration
    (tests/golden/make_moe_index_golden.py); `moe_index` reproduces them
    bit-for-bit (tests/test_oracle_golden.py).  `pos`, the inverse map, is not
    materialised by the reference and is checked as the inverse of `perm`.
    The weighted combine is pinned through the chain: route -> permute ->
    per-expert MLP -> unpermute built from these functions reproduces the
    registered `momoe` reference output on the golden cases.

Every function runs on CPU tensors with plain torch ops, in the same order of
operations (and therefore the same intermediate roundings) as the reference.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import Tensor


def _to_fp32_or_wider(t: Tensor) -> Tensor:
    """Reference: upcast(), src/popcorn/kernels/_utils.py:6-7."""
    return t.to(torch.promote_types(t.dtype, torch.float32))


def _unit_rms(t: Tensor, eps: float) -> Tensor:
    """Reference: rms(), src/popcorn/kernels/_utils.py:14-16 (result cast back to t.dtype)."""
    wide = _to_fp32_or_wider(t)
    mean_sq = wide.square().mean(dim=-1, keepdim=True)
    return (wide * torch.rsqrt(mean_sq + eps)).to(t.dtype)


def rms_norm(x: Tensor, weight: Tensor, bias: Tensor | None = None, eps: float = 1e-6) -> Tensor:
    """Reference: rms_norm, src/popcorn/kernels/rms_norm.py:16-30."""
    y = _unit_rms(x, eps) * weight
    if bias is not None:
        y = y + bias
    return y


def add_rms_norm(x: Tensor, residual: Tensor, weight: Tensor, eps: float = 1e-6, offset: float = 0.0) -> tuple[Tensor, Tensor]:
    """Reference: add_rms_norm, src/popcorn/kernels/add_rms_norm.py:8-23."""
    stream = x + residual
    return _unit_rms(stream, eps) * (weight + offset), stream


def rotary_embedding(x: Tensor, cos: Tensor, sin: Tensor, interleaved: bool = False) -> Tensor:
    """Reference: rotary_embedding, src/popcorn/kernels/rotary_embedding.py:15-40."""
    half = cos.shape[-1]
    c = _to_fp32_or_wider(cos)[None, :, None, :]
    s = _to_fp32_or_wider(sin)[None, :, None, :]
    if interleaved:
        first = _to_fp32_or_wider(x[..., 0 : 2 * half : 2])
        second = _to_fp32_or_wider(x[..., 1 : 2 * half : 2])
        turned = torch.stack((first * c - second * s, first * s + second * c), dim=-1).flatten(-2)
    else:
        first = _to_fp32_or_wider(x[..., :half])
        second = _to_fp32_or_wider(x[..., half : 2 * half])
        turned = torch.cat((first * c - second * s, first * s + second * c), dim=-1)
    turned = turned.to(x.dtype)
    if 2 * half == x.shape[-1]:
        return turned
    return torch.cat((turned, x[..., 2 * half :]), dim=-1)


def rope(q: Tensor, k: Tensor, cos: Tensor, sin: Tensor) -> tuple[Tensor, Tensor]:
    """Reference: rope, src/popcorn/kernels/rope.py:8-36 (layout batch, heads, seq, head_dim)."""
    def turned(x: Tensor) -> Tensor:
        first, second = x.chunk(2, -1)
        return torch.cat((-second, first), -1)

    c, s = cos[:, None], sin[:, None]
    return q * c + turned(q) * s, k * c + turned(k) * s


def qk_norm_rope(q: Tensor, k: Tensor, q_weight: Tensor, k_weight: Tensor, cos: Tensor, sin: Tensor, eps: float = 1e-6) -> tuple[Tensor, Tensor]:
    """Reference: qk_norm_rope, examples/03_write_a_kernel.ipynb cell 3 (per-head RMSNorm via
    src/popcorn/kernels/_utils.py:14-16, then the rotation of src/popcorn/kernels/rope.py:24-36)."""
    return rope(_unit_rms(q, eps) * q_weight, _unit_rms(k, eps) * k_weight, cos, sin)


def llama4_rope(q: Tensor, k: Tensor, freqs: Tensor) -> tuple[Tensor, Tensor]:
    """Reference: llama4_rope, src/popcorn/kernels/llama4_rope.py:14-39 (layout batch, seq, heads, head_dim;
    freqs [seq, head_dim/2, 2] = (cos, sin) per channel pair)."""
    f_re, f_im = freqs[None, :, None, :, 0], freqs[None, :, None, :, 1]

    def turned(x: Tensor) -> Tensor:
        pairs = x.unflatten(-1, (-1, 2))
        re, im = pairs[..., 0], pairs[..., 1]
        return torch.stack((re * f_re - im * f_im, re * f_im + im * f_re), -1).flatten(-2)

    return turned(q), turned(k)


def swiglu(a: Tensor, b: Tensor) -> Tensor:
    """Reference: swiglu, src/popcorn/kernels/swiglu.py:10-18."""
    return F.silu(a) * b


def geglu(a: Tensor, b: Tensor) -> Tensor:
    """Reference: geglu, src/popcorn/kernels/geglu.py:8-17."""
    return F.gelu(a, approximate="tanh") * b


def rms_norm_gated(x: Tensor, g: Tensor, weight: Tensor, bias: Tensor | None = None, activation: str = "swish", eps: float = 1e-6) -> Tensor:
    """Reference: rms_norm_gated, src/popcorn/kernels/rms_norm_gated.py:12-29."""
    out = _unit_rms(x, eps) * weight
    if bias is not None:
        out = out + bias
    return out * (F.silu(g) if activation == "swish" else torch.sigmoid(g))


def l2_norm(x: Tensor, eps: float = 1e-6) -> Tensor:
    """Reference: l2_norm, src/popcorn/kernels/l2_norm.py:8-14."""
    return x * torch.rsqrt(x.pow(2).sum(-1, keepdim=True) + eps)


def layer_norm(x: Tensor, weight: Tensor, bias: Tensor | None = None, eps: float = 1e-6) -> Tensor:
    """Reference: layer_norm, src/popcorn/kernels/layer_norm.py:8-20."""
    return F.layer_norm(x, weight.shape, weight, bias, eps)


def moe_route(router_logits: Tensor, top_k: int) -> tuple[Tensor, Tensor]:
    """Reference: routing lines of momoe, src/popcorn/kernels/momoe.py:47-49.

    Returns (indices int32 [..., top_k], weights float32-or-wider [..., top_k]); indices are
    in torch.topk order (descending probability)."""
    probs = torch.softmax(_to_fp32_or_wider(router_logits), dim=-1)
    picked = probs.topk(top_k, dim=-1)
    weights = picked.values / picked.values.sum(dim=-1, keepdim=True)
    return picked.indices.to(torch.int32), weights


def route_is_unambiguous(router_logits: Tensor, top_k: int) -> bool:
    """True when no row has equal probabilities among its top_k + 1 largest.

    torch.topk does not define an order among equal values, so index parity can
    only be demanded of inputs for which this holds."""
    probs = torch.softmax(_to_fp32_or_wider(router_logits), dim=-1)
    width = min(top_k + 1, probs.shape[-1])
    head = probs.topk(width, dim=-1).values
    return bool((head[..., :-1] != head[..., 1:]).all()) if width > 1 else True


def moe_index(indices: Tensor, experts: int) -> tuple[Tensor, Tensor, Tensor, Tensor]:
    """Restates find_used_experts / scatter_cols_kernel, src/popcorn/impls/momoe_tl.py:1071-1161.

    counts  = pairs per expert                     (:1135  counts = mask.sum(1))
    offsets = exclusive prefix, total at the end   (:1085-1101)
    perm    = token ids, ascending inside each expert, experts in order (:1104-1112 col_idx)
    pos     = inverse map [tokens, top_k] (not materialised by the reference)
    All int32."""
    tokens, top_k = indices.shape
    flat = indices.reshape(-1).to(torch.int64)
    counts = torch.bincount(flat, minlength=experts)[:experts]
    offsets = torch.zeros(experts + 1, dtype=torch.int64)
    offsets[1:] = torch.cumsum(counts, 0)
    order = torch.sort(flat, stable=True).indices  # flat pair id at each sorted position
    perm = torch.div(order, top_k, rounding_mode="floor")
    pos = torch.empty(tokens * top_k, dtype=torch.int64)
    pos[order] = torch.arange(tokens * top_k, dtype=torch.int64)
    return counts.to(torch.int32), offsets.to(torch.int32), perm.to(torch.int32), pos.view(tokens, top_k).to(torch.int32)


def moe_permute(x: Tensor, indices: Tensor, experts: int) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
    """Row gather of src/popcorn/impls/momoe_tl.py:156-158 / :408-476: rows[p] = x[perm[p]]."""
    counts, offsets, perm, pos = moe_index(indices, experts)
    rows = x.index_select(0, perm.to(torch.int64))
    return rows, counts, offsets, perm, pos


def moe_scatter_rows(x: Tensor, pos: Tensor) -> Tensor:
    """rows[pos[t, k]] = x[t]: the same gather written from the token side."""
    tokens, top_k = pos.shape
    rows = torch.empty((tokens * top_k, x.shape[1]), dtype=x.dtype)
    rows[pos.reshape(-1).to(torch.int64)] = x.repeat_interleave(top_k, dim=0)
    return rows


def moe_ep_destinations(indices: Tensor, pos: Tensor, local_offsets: Tensor, dst_base: Tensor, experts_per_rank: int) -> tuple[Tensor, Tensor]:
    """Expert-parallel addressing (no counterpart in the reference, which is single-GPU): the owner rank of
    each pair's expert and the pair's row in that rank's expert-major buffer."""
    e = indices.to(torch.int64)
    dst_rank = torch.div(e, experts_per_rank, rounding_mode="floor")
    dst_row = dst_base.to(torch.int64)[e] + (pos.to(torch.int64) - local_offsets.to(torch.int64)[e])
    return dst_rank.to(torch.int32), dst_row.to(torch.int32)


def moe_gather(x: Tensor, src_rows: Tensor) -> Tensor:
    return x.index_select(0, src_rows.to(torch.int64))


def moe_unpermute(rows: Tensor, weights: Tensor, pos: Tensor) -> Tensor:
    """Gate-weighted sum back to token order, src/popcorn/kernels/momoe.py:52-53.

    The reference contracts the expert axis with an fp32 einsum and casts once.
    The summation order of an einsum is not specified; this restatement fixes it
    to ascending expert index (= ascending pos), one rounded fp32 product and one
    rounded fp32 add per term, starting from +0."""
    tokens, top_k = pos.shape
    order = torch.argsort(pos.to(torch.int64), dim=1)
    pos_sorted = torch.gather(pos.to(torch.int64), 1, order)
    w_sorted = torch.gather(weights.to(torch.float32), 1, order)
    acc = torch.zeros((tokens, rows.shape[1]), dtype=torch.float32)
    for k in range(top_k):
        term = rows.index_select(0, pos_sorted[:, k]).to(torch.float32) * w_sorted[:, k : k + 1]
        acc = acc + term
    return acc.to(rows.dtype)


def momoe_from_steps(x: Tensor, gate_weight: Tensor, up_weight: Tensor, down_weight: Tensor, router_logits: Tensor, top_k: int) -> Tensor:
    """The registered `momoe` op (src/popcorn/kernels/momoe.py:34-53) rebuilt from the steps above.

    Used only to pin route / permute / unpermute end to end against the reference's output:
    tokens are routed, permuted into expert-contiguous rows, each expert's slice goes through
    its SwiGLU MLP in fp32, and the results are combined by moe_unpermute."""
    lead = x.shape[:-1]
    hidden = x.shape[-1]
    experts = gate_weight.shape[0]
    flat = _to_fp32_or_wider(x).reshape(-1, hidden)
    indices, weights = moe_route(router_logits.reshape(-1, experts), top_k)
    rows, counts, offsets, _, pos = moe_permute(flat, indices, experts)
    out_rows = torch.empty_like(rows)
    for e in range(experts):
        lo, hi = int(offsets[e]), int(offsets[e + 1])
        if hi == lo:
            continue
        chunk = rows[lo:hi]
        hidden_act = (chunk @ _to_fp32_or_wider(up_weight[e])) * F.silu(chunk @ _to_fp32_or_wider(gate_weight[e]))
        out_rows[lo:hi] = hidden_act @ _to_fp32_or_wider(down_weight[e])
    y = moe_unpermute(out_rows, weights.to(torch.float32), pos)
    return y.reshape(*lead, hidden).to(x.dtype)


def moe_grouped_gemm(rows: Tensor, weight: Tensor, offsets: Tensor, up_weight: Tensor | None = None) -> Tensor:
    """The expert MLP projections of momoe restricted to the rows each expert actually receives
    (reference: src/popcorn/kernels/momoe.py:50-52, fp32 einsums over every (token, expert) pair; the
    incumbent computes exactly these segments, src/popcorn/impls/momoe_tl.py:90-330).

    out[p] = rows[p] @ weight[e], or silu(rows[p] @ weight[e]) * (rows[p] @ up_weight[e]), in fp32, rounded once.
    Unpinned on its own (no standalone reference function); the chain route -> permute -> projections ->
    unpermute is pinned against the registered momoe reference."""
    out = torch.zeros(rows.shape[0], weight.shape[2], dtype=rows.dtype)
    bounds = offsets.tolist()
    for e in range(weight.shape[0]):
        lo, hi = bounds[e], bounds[e + 1]
        if hi <= lo:
            continue
        segment = rows[lo:hi].float()
        y = segment @ weight[e].float()
        if up_weight is not None:
            y = F.silu(y) * (segment @ up_weight[e].float())
        out[lo:hi] = y.to(rows.dtype)
    return out


def moe_grouped_gemm_gate_up(rows: Tensor, gate_weight: Tensor, up_weight: Tensor, offsets: Tensor) -> Tensor:
    """[rows @ gate_weight[e] | rows @ up_weight[e]], each rounded once: the two pre-activations of the expert MLP
    (the operands of F.silu(...) * ... in src/popcorn/kernels/momoe.py:51)."""
    return torch.cat((moe_grouped_gemm(rows, gate_weight, offsets), moe_grouped_gemm(rows, up_weight, offsets)), dim=1)


def moe_grouped_gemm_dgrad(grad_out: Tensor, weight: Tensor, offsets: Tensor, grad_out2: Tensor | None = None,
                           weight2: Tensor | None = None) -> Tensor:
    """What autograd derives for the rows of moe_grouped_gemm: grad_out @ weight[e]^T (+ grad_out2 @ weight2[e]^T),
    fp32, rounded once (the derivative of the einsums in src/popcorn/kernels/momoe.py:50-52)."""
    out = torch.zeros(grad_out.shape[0], weight.shape[1], dtype=grad_out.dtype)
    bounds = offsets.tolist()
    for e in range(weight.shape[0]):
        lo, hi = bounds[e], bounds[e + 1]
        if hi <= lo:
            continue
        y = grad_out[lo:hi].float() @ weight[e].float().t()
        if grad_out2 is not None:
            y = y + grad_out2[lo:hi].float() @ weight2[e].float().t()
        out[lo:hi] = y.to(grad_out.dtype)
    return out


def moe_grouped_gemm_wgrad(rows: Tensor, grad_out: Tensor, offsets: Tensor) -> Tensor:
    """What autograd derives for the weight of moe_grouped_gemm: per expert rows[segment]^T @ grad_out[segment] in
    fp32, rounded once; zeros for an expert without rows."""
    experts = offsets.numel() - 1
    out = torch.zeros(experts, rows.shape[1], grad_out.shape[1], dtype=rows.dtype)
    bounds = offsets.tolist()
    for e in range(experts):
        lo, hi = bounds[e], bounds[e + 1]
        if hi > lo:
            out[e] = (rows[lo:hi].float().t() @ grad_out[lo:hi].float()).to(rows.dtype)
    return out
