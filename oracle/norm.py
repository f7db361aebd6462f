"""Oracle for the row-wise stages around the projections (test infrastructure only; see the package docstring):
bias-free LayerNorm (`Norm`, src/archs/modernbert.rs:1006-1034), RMSNorm scaled by (1 + weight) (`RmsNorm`,
src/archs/qwen35_text.rs:178-203), rotate-half RoPE (candle `rope`; `Attention::rotary`,
src/archs/qwen35_text.rs:296-310) and the reference's fused RoPE + split kernel restated index by index
(`rope_qkv`, src/kernels/modernbert.cu:31-62).

Pinning: the reference's own test of this stage (`fused_rope_qkv_matches_candle`, src/archs/modernbert.rs:768-817)
holds no expected numbers; it checks that the fused kernel and the plain rope agree within 0.03 (bf16) on inputs
given by formula. `rope_qkv_test_inputs` restates those inputs and `tests/test_oracle.py` repeats that check
between `rope_qkv_indexed` and `rope`. The norms are restated from the formulas in the cited code; LayerNorm is
cross-checked against `torch.nn.functional.layer_norm`."""
from __future__ import annotations

import math

import numpy as np
import torch

from .projection import round_bf16


def layer_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, dtype: str = "f32", bias=None) -> torch.Tensor:
    """Without `bias` the encoder's `Norm`; with it the `layer_norm` of the decision heads (src/models/laya.rs:85-86,258)."""
    x = x.to(torch.float32)
    mean = x.mean(-1, keepdim=True)
    var = (x - mean).square().mean(-1, keepdim=True)
    y = (x - mean) / (var + eps).sqrt() * weight.to(torch.float32)
    if bias is not None:
        y = y + bias.to(torch.float32)
    return round_bf16(y) if dtype == "bf16" else y


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, dtype: str = "f32") -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * (1 + weight) in f32 (src/archs/qwen35_text.rs:185-202)."""
    x = x.to(torch.float32)
    scale = 1.0 / (x.square().mean(-1, keepdim=True) + eps).sqrt()
    y = x * scale * (weight.to(torch.float32) + 1.0)
    return round_bf16(y) if dtype == "bf16" else y


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rotary_dim: int = -1, bf16_ops: bool = False) -> torch.Tensor:
    """Rotate-half on `[L, H, D]` with tables `[L, rotary_dim / 2]`; columns past `rotary_dim` pass through.
    `bf16_ops`: the Qwen3.5 path evaluates `x * cos + rotate_half(x) * sin` with bf16 tensor ops
    (src/archs/qwen35_text.rs:296-310), so each product and the sum is rounded to bf16 (three roundings); without it
    the products and the sum are f32 (the ModernBERT kernel, src/kernels/modernbert.cu:48-57) and the caller rounds."""
    d = x.shape[-1] if rotary_dim < 0 else rotary_dim
    h = d // 2
    x1, x2 = x[..., :h], x[..., h:d]
    c, s = cos.unsqueeze(1), sin.unsqueeze(1)
    if bf16_ops:
        r = round_bf16
        return torch.cat([r(r(x1 * c) + r(-x2 * s)), r(r(x2 * c) + r(x1 * s)), x[..., d:]], dim=-1)
    return torch.cat([x1 * c - x2 * s, x1 * s + x2 * c, x[..., d:]], dim=-1)


def rope_qkv_indexed(qkv: np.ndarray, cos: np.ndarray, sin: np.ndarray, length: int, heads: int, dim: int, dtype: str = "f32"):
    """The reference kernel thread by thread (src/kernels/modernbert.cu:31-62): `qkv` flat `[B * L, 3, heads, dim]`,
    tables flat `[L, dim / 2]`; returns q, k, v flat `[B * L, heads, dim]` each (the kernel's token-major planes)."""
    r = (lambda v: float(round_bf16(torch.tensor(v, dtype=torch.float32)))) if dtype == "bf16" else (lambda v: v)
    half = dim // 2
    tokens = qkv.size // (3 * heads * dim)
    pairs = tokens * heads * half
    flat = qkv.reshape(-1).astype(np.float32)
    out = np.zeros(3 * pairs * 2, dtype=np.float32)
    plane = pairs * 2
    for index in range(pairs):
        column = index % half
        head = (index // half) % heads
        token = index // (heads * half)
        position = token % length
        ib = token * (3 * heads * dim) + head * dim + column
        ob = token * (heads * dim) + head * dim + column
        c, s = np.float32(cos.reshape(-1)[position * half + column]), np.float32(sin.reshape(-1)[position * half + column])
        for src, dst in ((ib, ob), (ib + heads * dim, plane + ob)):
            a, b = flat[src], flat[src + half]
            out[dst] = r(a * c - b * s)
            out[dst + half] = r(a * s + b * c)
        vb = ib + 2 * heads * dim
        out[2 * plane + ob] = flat[vb]
        out[2 * plane + ob + half] = flat[vb + half]
    shape = (tokens, heads, dim)
    return out[:plane].reshape(shape), out[plane:2 * plane].reshape(shape), out[2 * plane:].reshape(shape)


def rope_qkv_test_inputs():
    """Inputs of `fused_rope_qkv_matches_candle` (src/archs/modernbert.rs:768-790): tables cos / sin of 0.13 i,
    `[5, 4]`; qkv values ((37 i mod 127) - 63) / 21, `[2, 5, 3, 2, 8]`."""
    cos = np.array([math.cos(np.float32(i) * np.float32(0.13)) for i in range(20)], dtype=np.float32).reshape(5, 4)
    sin = np.array([math.sin(np.float32(i) * np.float32(0.13)) for i in range(20)], dtype=np.float32).reshape(5, 4)
    values = np.array([((i * 37 % 127) - 63.0) / 21.0 for i in range(480)], dtype=np.float32).reshape(2, 5, 3, 2, 8)
    return cos, sin, values
