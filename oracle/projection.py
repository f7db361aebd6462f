"""Oracle for the projection path (test infrastructure only; see the package docstring).

Two precisions, selected by `dtype`:
  * "f32"  - everything in float32: the reference's CPU path (`--features cpu`, `--dtype f32`).
  * "bf16" - the reference's bf16 run restated on the CPU: every tensor op result is rounded to bf16 where the
             reference materialises a bf16 tensor (after the matmul, after the bias add, after the activation,
             after the gate product, after the residual add), with the contraction itself accumulated in f32.
"""
from __future__ import annotations

from typing import Optional

import torch


def round_bf16(t: torch.Tensor) -> torch.Tensor:
    """Round-to-nearest-even to bf16, returned as float32."""
    return t.to(torch.bfloat16).to(torch.float32)


def _r(t: torch.Tensor, dtype: str) -> torch.Tensor:
    return round_bf16(t) if dtype == "bf16" else t


def gelu_erf(x: torch.Tensor) -> torch.Tensor:
    """Exact-erf GELU, `x * Phi(x)`: candle's `gelu_erf` (src/archs/modernbert.rs:531) and the CUDA kernel's
    `value * normcdff(value)` (src/kernels/modernbert.cu:11-12)."""
    return x * 0.5 * (1.0 + torch.erf(x * 0.7071067811865476))


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, *, act: Optional[str] = None,
           residual: Optional[torch.Tensor] = None, dtype: str = "bf16") -> torch.Tensor:
    """`x.apply(&Linear)` = `x Wᵀ (+ b)` (weight `[out, in]`: src/archs/modernbert.rs:1036-1046,
    src/archs/qwen35_text.rs:174-176), then the optional activation of the head Linears
    (src/models/laya.rs:133-155) and the caller's residual add (src/archs/modernbert.rs:882-886,
    src/archs/qwen35_text.rs:938-939). Returns float32 holding values of the requested precision."""
    x = x.to(torch.float32)
    w = w.to(torch.float32)
    y = _r(x @ w.t(), dtype)
    if bias is not None:
        y = _r(y + bias.to(torch.float32), dtype)
    if act == "relu":
        y = torch.relu(y)
    elif act == "gelu":
        y = _r(gelu_erf(y), dtype)
    elif act is not None:
        raise ValueError(act)
    if residual is not None:
        y = _r(y + residual.to(torch.float32), dtype)
    return y


def geglu(p: torch.Tensor, dtype: str = "bf16") -> torch.Tensor:
    """`geglu(projected)`: first half activated, second half multiplies, with the kernel's two roundings
    `T(float(T(gelu(x))) * gate)` (src/kernels/modernbert.cu:4-14; CPU form src/archs/modernbert.rs:531-532)."""
    inner = p.shape[-1] // 2
    act = _r(gelu_erf(p[..., :inner].to(torch.float32)), dtype)
    return _r(act * p[..., inner:].to(torch.float32), dtype)


def swiglu(gate: torch.Tensor, up: torch.Tensor, dtype: str = "bf16") -> torch.Tensor:
    """`gate.silu()? * up` in the model dtype (src/archs/qwen35_text.rs:239)."""
    g = gate.to(torch.float32)
    s = _r(g / (1.0 + torch.exp(-g)), dtype)
    return _r(s * up.to(torch.float32), dtype)


def mlp_modernbert(x, wi, wo, residual=None, dtype: str = "bf16"):
    """`Mlp::forward` (src/archs/modernbert.rs:521-533) and the layer's `x + mlp` (:884-886)."""
    h = geglu(linear(x, wi, dtype=dtype), dtype)
    return linear(h, wo, residual=residual, dtype=dtype)


def mlp_qwen35(x, wg, wu, wd, residual=None, dtype: str = "bf16"):
    """`Mlp::forward` (src/archs/qwen35_text.rs:232-240) and the layer's residual (:939)."""
    h = swiglu(linear(x, wg, dtype=dtype), linear(x, wu, dtype=dtype), dtype)
    return linear(h, wd, residual=residual, dtype=dtype)
