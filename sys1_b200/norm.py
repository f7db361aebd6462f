"""Row-wise stages either side of the projections, through the C ABI: bias-free LayerNorm / (1 + w) RMSNorm
(`s1_norm`) and the in-place rotate-half rotary embedding (`s1_rope`). CUDA bf16 tensors only; no CPU fallback."""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import device

LAYER_NORM, RMS_NORM, COPY = 0, 1, 2


def _rows(t: torch.Tensor, name: str) -> torch.Tensor:
    if not t.is_cuda or t.dtype != torch.bfloat16 or t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name} must be a bf16 CUDA matrix with contiguous rows (no CPU fallback)")
    return t


def norm(x: torch.Tensor, weight: torch.Tensor, eps: float, kind: int = LAYER_NORM, gather: Optional[torch.Tensor] = None,
         out: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """`Norm::forward` (src/archs/modernbert.rs:1024-1034; kind 0) or `RmsNorm::forward`
    (src/archs/qwen35_text.rs:191-203; kind 1) on `x [rows, width]`. With `gather` (int32 CUDA `[rows]`) the rows are
    `x[gather]`: embedding lookup and embedding norm in one pass. `out` may be `x`."""
    _rows(x, "x")
    rows = x.shape[0] if gather is None else gather.shape[0]
    width = x.shape[1]
    if gather is not None and (not gather.is_cuda or gather.dtype != torch.int32 or not gather.is_contiguous()):
        raise ValueError("gather must be a contiguous int32 CUDA vector")
    if kind != COPY and (weight is None or weight.dtype != torch.bfloat16 or not weight.is_cuda or weight.numel() != width
                         or not weight.is_contiguous()):
        raise ValueError("weight must be a contiguous bf16 CUDA vector of the row width")
    if bias is not None and (bias.dtype != torch.bfloat16 or not bias.is_cuda or bias.numel() != width or not bias.is_contiguous()):
        raise ValueError("bias must be a contiguous bf16 CUDA vector of the row width")
    if out is None:
        out = torch.empty((rows, width), dtype=torch.bfloat16, device=x.device)
    _rows(out, "out")
    if rows == 0:
        return out
    ctx = device.load(x.device.index)
    rc = ctx._lib.s1_norm(ctx.handle, C.c_void_p(x.data_ptr()), x.stride(0), C.c_void_p(gather.data_ptr() if gather is not None else 0),
                          x.shape[0] if gather is not None else 0, C.c_void_p(weight.data_ptr() if weight is not None else 0),
                          C.c_void_p(bias.data_ptr() if bias is not None else 0), C.c_float(eps), int(kind),
                          C.c_void_p(out.data_ptr()), out.stride(0), rows, width)
    ctx.check(rc)
    return out


def rope_(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor, heads: int, head_stride: int,
          rotary_dim: int) -> torch.Tensor:
    """Rotates, in place, `heads` consecutive heads of every row of `x [T, ld]` (head h at column `h * head_stride`,
    first `rotary_dim` columns of the head) by the table rows `cos/sin[positions[t]]` (f32 `[P, rotary_dim / 2]`).
    On a packed Wqkv output: `heads = 2 * H` (`RotaryEmbedding::apply_qkv`, src/kernels/modernbert.cu:31-62)."""
    _rows(x, "x")
    for name, t in (("cos", cos), ("sin", sin)):
        if not t.is_cuda or t.dtype != torch.float32 or t.dim() != 2 or not t.is_contiguous() or t.shape[1] != rotary_dim // 2:
            raise ValueError(f"{name} must be a contiguous f32 CUDA table [positions, rotary_dim / 2]")
    if not positions.is_cuda or positions.dtype != torch.int32 or not positions.is_contiguous() or positions.numel() != x.shape[0]:
        raise ValueError("positions must be a contiguous int32 CUDA vector with one entry per row")
    if x.shape[0] == 0:
        return x
    ctx = device.load(x.device.index)
    rc = ctx._lib.s1_rope(ctx.handle, C.c_void_p(x.data_ptr()), x.stride(0), C.c_void_p(cos.data_ptr()), C.c_void_p(sin.data_ptr()),
                          C.c_void_p(positions.data_ptr()), min(cos.shape[0], sin.shape[0]), x.shape[0], int(heads), int(head_stride),
                          int(rotary_dim))
    ctx.check(rc)
    return x


def head_norm_rope_(x: torch.Tensor, heads: int, head_stride: int, head_dim: int, weight: torch.Tensor, eps: float,
                    cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor, rotary_dim: int, bf16_ops: bool = True) -> torch.Tensor:
    """`q_norm` / `k_norm` followed by `Attention::rotary` (src/archs/qwen35_text.rs:296-339) in one pass, in place
    (`s1_head_norm_rope`): per-head RMSNorm x (1 + weight) over `head_dim` columns of `heads` heads per row of
    `x [T, ld]` (head h at column `h * head_stride`), then the partial rotation of the first `rotary_dim` columns.
    `bf16_ops`: round each product and the sum to bf16 as candle's bf16 tensor ops do (the reference's arithmetic)."""
    _rows(x, "x")
    for name, t in (("cos", cos), ("sin", sin)):
        if not t.is_cuda or t.dtype != torch.float32 or t.dim() != 2 or not t.is_contiguous() or t.shape[1] != rotary_dim // 2:
            raise ValueError(f"{name} must be a contiguous f32 CUDA table [positions, rotary_dim / 2]")
    if not positions.is_cuda or positions.dtype != torch.int32 or not positions.is_contiguous() or positions.numel() != x.shape[0]:
        raise ValueError("positions must be a contiguous int32 CUDA vector with one entry per row")
    if weight.dtype != torch.bfloat16 or not weight.is_cuda or weight.numel() != head_dim or not weight.is_contiguous():
        raise ValueError("weight must be a contiguous bf16 CUDA vector of length head_dim")
    if x.shape[0] == 0:
        return x
    ctx = device.load(x.device.index)
    rc = ctx._lib.s1_head_norm_rope(ctx.handle, C.c_void_p(x.data_ptr()), x.stride(0), int(head_stride), int(heads), int(head_dim),
                                    C.c_void_p(weight.data_ptr()), C.c_float(eps), C.c_void_p(cos.data_ptr()), C.c_void_p(sin.data_ptr()),
                                    C.c_void_p(positions.data_ptr()), min(cos.shape[0], sin.shape[0]), int(rotary_dim), x.shape[0],
                                    1 if bf16_ops else 0)
    ctx.check(rc)
    return x


def add_rows(x: torch.Tensor, table: torch.Tensor, index: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """`x + table[index]` row by row through `s1_add_rows` (`hidden.broadcast_add(type_ids.apply(&type_embedding))`,
    src/models/laya.rs:431, with one index per packed token). `out` may be `x`."""
    _rows(x, "x")
    _rows(table, "table")
    if not index.is_cuda or index.dtype != torch.int32 or not index.is_contiguous() or index.numel() != x.shape[0]:
        raise ValueError("index must be a contiguous int32 CUDA vector with one entry per row")
    if out is None:
        out = torch.empty_like(x)
    _rows(out, "out")
    if x.shape[0] == 0:
        return out
    ctx = device.load(x.device.index)
    ctx.check(ctx._lib.s1_add_rows(ctx.handle, C.c_void_p(x.data_ptr()), x.stride(0), C.c_void_p(table.data_ptr()), table.stride(0),
                                   C.c_void_p(index.data_ptr()), table.shape[0], C.c_void_p(out.data_ptr()), out.stride(0), x.shape[0],
                                   x.shape[1]))
    return out


def embedding(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """`ids.apply(&embedding)` (src/archs/qwen35_text.rs:978-980): the rows `table[ids]` (ids int32 CUDA), through
    `s1_norm` with kind 2 (rows copied through the index); an id outside the table is reported at the next sync."""
    return norm(table, None, 0.0, COPY, gather=ids)
