"""Readers for the fixtures under tests/golden/ (see tests/golden/make_golden.py)."""
from pathlib import Path

import numpy as np
import torch

GOLDEN = Path(__file__).resolve().parent / "golden"


def load_projections():
    """{case: {name: float32 tensor}}; bf16-valued entries are decoded from their stored bit patterns."""
    raw = np.load(GOLDEN / "projections.npz")
    out = {}
    for key in raw.files:
        case, name = key.split("/")
        arr = raw[key]
        if name.endswith("@bf16"):
            t = torch.from_numpy(arr.copy()).view(torch.bfloat16).to(torch.float32)
            name = name[:-5]
        else:
            t = torch.from_numpy(arr.copy())
        out.setdefault(case, {})[name] = t
    return out


def load_delta_rule():
    raw = np.load(GOLDEN / "delta_rule.npz")
    return {k: torch.from_numpy(raw[k].copy()) for k in raw.files}


def load_layers():
    """{"group/name": tensor}: attention, causal GQA attention, norm and rope cases (float32; int32 index arrays)."""
    raw = np.load(GOLDEN / "layers.npz")
    return {k: torch.from_numpy(raw[k].copy()) for k in raw.files}
