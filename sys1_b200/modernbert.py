"""Projection side of the ModernBERT layer (`src/archs/modernbert.rs`): Wqkv, Wo(+residual), Wi+GeGLU, MLP-out(+residual).

Same member names as the reference structs (`Attention { wqkv, wo }` :137-175, `Mlp { input, output }`
:494-534). Attention itself, norms and RoPE are outside this path and stay with the caller.
"""
from __future__ import annotations

from typing import Optional

import torch

from ._lib import EPI_GEGLU
from .linear import Linear, fused_linear


class Mlp:
    """`Mlp::forward` (src/archs/modernbert.rs:521-533): `output( geglu( input(x) ) )`, GeGLU fused into the
    first projection's epilogue with the rounding of `src/kernels/modernbert.cu:4-14`."""

    def __init__(self, input: Linear, output: Linear):
        self.input = input
        self.output = output

    def gated(self, x: torch.Tensor) -> torch.Tensor:
        """`geglu(x.apply(&self.input))` → `[T, I]`."""
        return fused_linear(x, self.input.weight, epilogue=EPI_GEGLU)

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """With `residual`, also performs the caller's `x + mlp(...)` (src/archs/modernbert.rs:884-886)."""
        return self.output.forward(self.gated(x), residual=residual)

    __call__ = forward


class AttentionProjections:
    """The two Linears of `Attention` (src/archs/modernbert.rs:156-167): `wqkv` and `wo`."""

    def __init__(self, wqkv: Linear, wo: Linear):
        self.wqkv = wqkv
        self.wo = wo

    def qkv(self, x: torch.Tensor) -> torch.Tensor:
        """`x.apply(&self.wqkv)` (src/archs/modernbert.rs:184-187) → `[T, 3·H·D]`."""
        return self.wqkv.forward(x)

    def out(self, attended: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """`attended.apply(&self.wo)` (:191) and, with `residual`, the layer's `x + ·` (:882-883)."""
        return self.wo.forward(attended, residual=residual)
