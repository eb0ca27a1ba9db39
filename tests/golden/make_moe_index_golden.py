"""Generate tests/golden/moeindex_*.npz with the REFERENCE's own index kernel, on a CUDA machine.

    python tests/golden/make_moe_index_golden.py [OUTPUT_DIR]      # default: tests/golden

The only reference code that computes per-expert counts, their exclusive prefix and the per-expert token lists is
`find_used_experts` with its Triton `scatter_cols_kernel` (src/popcorn/impls/momoe_tl.py:1071-1161).  This script
imports that module from the unmodified popcorn install (sys.path, else baseline/_ref), builds `mask_NM` from router
logits exactly as the reference's `momoe` does (:1277-1281: softmax, top-k, scatter of ones, transpose), calls
`find_used_experts(mask_NM, top_k)` and stores its outputs bit-exactly:

    counts    [experts]        pairs per expert                         (:1135)
    cumsums   [experts + 1]    exclusive prefix, total in the last slot (:1094-1101)
    col_idx   [tokens * top_k] token ids, expert-major                  (:1104-1112)

`which_Msum` (the slot a pair gets from an atomic counter, :1113-1115) depends on the order in which programs
arrive and is left out.  Cases: the router logits of every momoe_* / moe16_* fixture, a 1/16-size and the full-size
MoE benchmark configuration (65536 tokens, 64 experts, top-8, seed 4).  For the full-size case col_idx (2 MiB) is
stored as a SHA-256 digest plus its first and last 4096 entries.
"""

from __future__ import annotations

import hashlib
import os
import sys
import tempfile
import warnings
from pathlib import Path

import torch

REPO = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(REPO))
from tests.golden import golden_io  # noqa: E402

os.environ.setdefault("POPCORN_CACHE_DIR", tempfile.mkdtemp(prefix="popcorn-cache-"))
warnings.filterwarnings("ignore")
try:
    import popcorn  # noqa: F401
except ImportError:
    sys.path.insert(0, str(REPO / "baseline" / "_ref"))
from popcorn.impls.momoe_tl import find_used_experts  # noqa: E402

EDGE = 4096


def reference_index(router_logits: torch.Tensor, top_k: int) -> dict[str, torch.Tensor]:
    """mask_NM as the reference's momoe builds it, then its find_used_experts."""
    logits = router_logits.reshape(-1, router_logits.shape[-1]).to("cuda")
    probs = torch.softmax(logits.float(), -1)
    picked = probs.topk(top_k, -1)
    mask_NM = torch.zeros_like(probs, dtype=torch.int32).scatter(-1, picked.indices, 1).T.contiguous()
    cumsums_N, col_idx, counts, _which = find_used_experts(mask_NM, top_k)
    torch.cuda.synchronize()
    return {"topk_indices": picked.indices.to(torch.int32).cpu(), "counts": counts.to(torch.int32).cpu(),
            "cumsums": cumsums_N.cpu(), "col_idx": col_idx.cpu()}


def digest(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().numpy().tobytes()).hexdigest()


def main() -> None:
    if not torch.cuda.is_available():
        raise SystemExit("find_used_experts launches a Triton kernel: run this on a CUDA machine")
    out = Path(sys.argv[1]) if len(sys.argv) > 1 else golden_io.GOLDEN_DIR
    out.mkdir(parents=True, exist_ok=True)
    written = []
    for name in [name for name in golden_io.case_names() if name.startswith(("momoe_", "moe16_"))]:
        tensors, meta = golden_io.load_case(name)
        found = reference_index(tensors["router_logits"], meta["top_k"])
        assert torch.equal(found["topk_indices"], tensors["topk_indices"].reshape(-1, meta["top_k"])), name
        stored = {"router_logits": tensors["router_logits"].reshape(-1, tensors["router_logits"].shape[-1]), **found}
        written.append(golden_io.save_case(f"moeindex_{name}", stored, {"op": "moe_index", "top_k": meta["top_k"],
                                                                        "experts": tensors["router_logits"].shape[-1]}, out))
    from popcorn_b200 import workloads

    for label, scale in (("config5_sixteenth", 1 / 16), ("config5_full", 1.0)):
        w = workloads.moe_bf16(scale=scale)
        found = reference_index(w.inputs["router_logits"], w.args["top_k"])
        meta = {"op": "moe_index", "top_k": w.args["top_k"], "experts": w.args["experts"], "tokens": w.tokens, "seed": 4, "scale": scale}
        if scale == 1.0:  # inputs are regenerated from the seed; the long output is kept as a digest
            meta["col_idx_sha256"] = digest(found["col_idx"])
            meta["topk_indices_sha256"] = digest(found["topk_indices"])
            stored = {"counts": found["counts"], "cumsums": found["cumsums"],
                      "col_idx_head": found["col_idx"][:EDGE].clone(), "col_idx_tail": found["col_idx"][-EDGE:].clone()}
        else:
            stored = found
        written.append(golden_io.save_case(f"moeindex_{label}", stored, meta, out))
    for path in written:
        print(path, path.stat().st_size)


if __name__ == "__main__":
    main()
