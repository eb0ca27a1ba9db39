"""Read/write the golden fixtures: one .npz per case, tensors stored bit-exactly.

numpy has no bfloat16, so 16-bit floats are stored as their int16 bit patterns
under the key "<name>|<torch dtype>"; scalars go into a JSON string under "meta".
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any

import numpy as np
import torch

GOLDEN_DIR = Path(__file__).resolve().parent
_BITS = {torch.bfloat16: torch.int16, torch.float16: torch.int16}


def save_case(name: str, tensors: dict[str, torch.Tensor], meta: dict[str, Any], directory: Path | None = None) -> Path:
    arrays: dict[str, np.ndarray] = {"meta": np.array(json.dumps(meta))}
    for key, value in tensors.items():
        value = value.detach().cpu().contiguous()
        dtype_name = str(value.dtype).removeprefix("torch.")
        raw = value.view(_BITS[value.dtype]) if value.dtype in _BITS else value
        arrays[f"{key}|{dtype_name}"] = raw.numpy()
    path = (directory or GOLDEN_DIR) / f"{name}.npz"
    np.savez_compressed(path, **arrays)
    return path


def load_case(name: str) -> tuple[dict[str, torch.Tensor], dict[str, Any]]:
    with np.load(GOLDEN_DIR / f"{name}.npz") as data:
        meta = json.loads(str(data["meta"]))
        tensors = {}
        for key in data.files:
            if key == "meta":
                continue
            label, dtype_name = key.split("|")
            dtype = getattr(torch, dtype_name)
            value = torch.from_numpy(np.array(data[key]))
            tensors[label] = value.view(dtype) if dtype in _BITS else value
    return tensors, meta


def case_names() -> list[str]:
    return sorted(path.stem for path in GOLDEN_DIR.glob("*.npz"))
