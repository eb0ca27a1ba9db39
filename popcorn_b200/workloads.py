"""Seeded synthetic inputs for the five benchmark configurations, and their byte counts.

Inputs are drawn the way popcorn's harness draws them
(src/popcorn/bench/grid.py:675-716): a CPU ``torch.Generator`` seeded per case,
``torch.randn`` in fp32 in a fixed order, an affine transform, then a cast to the
case dtype.  ``scale`` shrinks the token dimension only (rows, batch*seq or
tokens), so a scaled case keeps the row width, the dtype and the value
distribution of the full one.

Algorithmic bytes are the bytes an ideal kernel must move: every input element
read once, every output element written once, small tables (weights, cos/sin)
once.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch
from torch import Tensor


@dataclass
class Workload:
    name: str  # rms_norm | add_rms_norm | rotary_embedding | swiglu | moe
    dtype: torch.dtype
    tokens: int
    inputs: dict[str, Tensor]
    args: dict[str, Any] = field(default_factory=dict)
    # bytes per phase; single-kernel workloads have one phase named like the workload
    algorithmic_bytes: dict[str, int] = field(default_factory=dict)

    def to(self, device: torch.device | str) -> "Workload":
        moved = {k: v.to(device) for k, v in self.inputs.items()}
        return Workload(self.name, self.dtype, self.tokens, moved, dict(self.args), dict(self.algorithmic_bytes))

    def shard(self, rank: int, world: int) -> "Workload":
        """The contiguous token shard of `rank` (tables and weights are replicated)."""
        def cut(t: Tensor, dim: int = 0) -> Tensor:
            n = t.shape[dim]
            lo, hi = n * rank // world, n * (rank + 1) // world
            return t.narrow(dim, lo, hi - lo)

        per_token = {
            "rms_norm": ("x",), "add_rms_norm": ("x", "residual"), "rotary_embedding": ("q", "k"), "rope": ("q", "k"),
            "swiglu": ("gate_up",), "moe": ("x", "router_logits"),
        }[self.name]
        inputs = {k: (cut(v) if k in per_token else v) for k, v in self.inputs.items()}
        first = inputs[per_token[0]]
        tokens = first.shape[0] * (first.shape[1] if self.name == "rotary_embedding" else first.shape[2] if self.name == "rope" else 1)
        scale = tokens / max(self.tokens, 1)
        nbytes = {k: int(v * scale) for k, v in self.algorithmic_bytes.items()}
        return Workload(self.name, self.dtype, tokens, inputs, dict(self.args), nbytes)


def _scaled(n: int, scale: float, multiple: int = 1) -> int:
    return max(multiple, int(round(n * scale / multiple)) * multiple)


def rms_norm_fp32(scale: float = 1.0, rows: int = 4096, cols: int = 4096) -> Workload:
    """Config 1: x [4096, 4096] fp32 ~ N(0,1), weight ~ N(1, 0.02), eps 1e-6, seed 0."""
    rows = _scaled(rows, scale)
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(rows, cols, generator=gen)
    weight = 1 + 0.02 * torch.randn(cols, generator=gen)
    nbytes = 2 * rows * cols * 4 + cols * 4
    return Workload("rms_norm", torch.float32, rows, {"x": x, "weight": weight}, {"eps": 1e-6}, {"rms_norm": nbytes})


def add_rms_norm_bf16(scale: float = 1.0, rows: int = 16384, cols: int = 8192) -> Workload:
    """Config 2: x, residual [16384, 8192] bf16 ~ N(0,1), weight ~ N(1, 0.1), eps 1e-5, seed 1."""
    rows = _scaled(rows, scale)
    gen = torch.Generator().manual_seed(1)
    x = torch.randn(rows, cols, generator=gen).to(torch.bfloat16)
    residual = torch.randn(rows, cols, generator=gen).to(torch.bfloat16)
    weight = (1 + 0.1 * torch.randn(cols, generator=gen)).to(torch.bfloat16)
    nbytes = 4 * rows * cols * 2 + cols * 2
    return Workload("add_rms_norm", torch.bfloat16, rows, {"x": x, "residual": residual, "weight": weight},
                    {"eps": 1e-5, "offset": 0.0}, {"add_rms_norm": nbytes})


def rope_tables(seq: int, half: int, theta: float = 500000.0) -> tuple[Tensor, Tensor]:
    inv = theta ** (-torch.arange(0, 2 * half, 2, dtype=torch.float32) / (2 * half))
    ang = torch.outer(torch.arange(seq, dtype=torch.float32), inv)
    return ang.cos(), ang.sin()


def rotary_bf16(scale: float = 1.0, batch: int = 8, seq: int = 4096, q_heads: int = 32, k_heads: int = 8, head_dim: int = 128) -> Workload:
    """Config 3: q [8, 4096, 32, 128], k [8, 4096, 8, 128] bf16, positions 0..seq-1, theta 500000, seed 2."""
    batch = _scaled(batch, scale)
    gen = torch.Generator().manual_seed(2)
    q = torch.randn(batch, seq, q_heads, head_dim, generator=gen).to(torch.bfloat16)
    k = torch.randn(batch, seq, k_heads, head_dim, generator=gen).to(torch.bfloat16)
    cos, sin = rope_tables(seq, head_dim // 2)
    nbytes = 2 * (q.numel() + k.numel()) * 2 + (cos.numel() + sin.numel()) * 4
    return Workload("rotary_embedding", torch.bfloat16, batch * seq, {"q": q, "k": k, "cos": cos, "sin": sin},
                    {"interleaved": False}, {"rotary_embedding": nbytes})


def paired_rope_bf16(scale: float = 1.0, batch: int = 8, seq: int = 4096, q_heads: int = 32, k_heads: int = 8, head_dim: int = 128) -> Workload:
    """The shapes of config 3 in the layout of popcorn's paired `rope` op: q [8, 32, 4096, 128], k [8, 8, 4096, 128],
    bf16 tables [1, 4096, 128] with the first half repeated (positions 0..seq-1, theta 500000), seed 2."""
    batch = _scaled(batch, scale)
    gen = torch.Generator().manual_seed(2)
    q = torch.randn(batch, q_heads, seq, head_dim, generator=gen).to(torch.bfloat16)
    k = torch.randn(batch, k_heads, seq, head_dim, generator=gen).to(torch.bfloat16)
    cos, sin = rope_tables(seq, head_dim // 2)
    cos = cos.repeat(1, 2)[None].to(torch.bfloat16)
    sin = sin.repeat(1, 2)[None].to(torch.bfloat16)
    nbytes = 2 * (q.numel() + k.numel()) * 2 + (cos.numel() + sin.numel()) * 2
    return Workload("rope", torch.bfloat16, batch * seq, {"q": q, "k": k, "cos": cos, "sin": sin}, {}, {"rope": nbytes})


def swiglu_bf16(scale: float = 1.0, rows: int = 32768, cols: int = 14336) -> Workload:
    """Config 4: gate_up [32768, 2*14336] bf16 ~ N(0,1); gate = first half, up = second half, seed 3."""
    rows = _scaled(rows, scale)
    gen = torch.Generator().manual_seed(3)
    gate_up = torch.randn(rows, 2 * cols, generator=gen).to(torch.bfloat16)
    nbytes = 3 * rows * cols * 2
    return Workload("swiglu", torch.bfloat16, rows, {"gate_up": gate_up}, {"cols": cols}, {"swiglu": nbytes})


def moe_bf16(scale: float = 1.0, tokens: int = 65536, hidden: int = 4096, experts: int = 64, top_k: int = 8) -> Workload:
    """Config 5: x [65536, 4096] bf16 ~ N(0,1), router logits fp32 [65536, 64] ~ N(0,1), top-8, seed 4."""
    tokens = _scaled(tokens, scale)
    gen = torch.Generator().manual_seed(4)
    x = torch.randn(tokens, hidden, generator=gen).to(torch.bfloat16)
    logits = torch.randn(tokens, experts, generator=gen)
    pairs = tokens * top_k
    nbytes = {
        "route": tokens * experts * 4 + 2 * pairs * 4,
        "index": 3 * pairs * 4,
        # x read once (unique bytes), every gathered row written once, the inverse map read once
        "permute": tokens * hidden * 2 + pairs * hidden * 2 + pairs * 4,
        "unpermute": pairs * hidden * 2 + 2 * pairs * 4 + tokens * hidden * 2,
    }
    return Workload("moe", torch.bfloat16, tokens, {"x": x, "router_logits": logits}, {"experts": experts, "top_k": top_k}, nbytes)


CONFIGS = {
    "rms_norm_fp32": rms_norm_fp32,
    "add_rms_norm_bf16": add_rms_norm_bf16,
    "rotary_bf16": rotary_bf16,
    "paired_rope_bf16": paired_rope_bf16,
    "swiglu_bf16": swiglu_bf16,
    "moe_bf16": moe_bf16,
}
