"""Projection layers behind the C ABI: the host-side mirror of candle's `Linear` as sys1 uses it.

`Linear(weight, bias)` / `linear_no_bias` follow `src/archs/modernbert.rs:1036-1046` and
`src/archs/qwen35_text.rs:174-176` (weight `[out, in]`, `forward(x) = x Wᵀ (+ b)`); the extra keyword
arguments fold in what the reference runs as separate kernels right after the projection.
Inputs are bf16 CUDA tensors; anything else raises (no fallback).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib, device
from ._lib import ACT_GELU, ACT_NONE, ACT_RELU, EPI_GEGLU, EPI_NONE, EPI_SWIGLU, LinearDesc

_ACTS = {None: ACT_NONE, "relu": ACT_RELU, "gelu": ACT_GELU}


def _check(t: torch.Tensor, name: str) -> None:
    if t.is_cuda and t.dtype is torch.bfloat16 and t.dim() == 2 and t.stride(1) == 1:
        return  # the common case, kept short: this runs several times per launch
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (this path has no CPU fallback)")
    if t.dtype != torch.bfloat16:
        raise ValueError(f"{name} must be bf16, got {t.dtype}")
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name} must be 2-D with contiguous rows, got shape {tuple(t.shape)} strides {t.stride()}")


def _ptr(t: Optional[torch.Tensor]) -> C.c_void_p:
    return C.c_void_p(0 if t is None else t.data_ptr())


def fused_linear(x: torch.Tensor, weight: torch.Tensor, *, weight_up: Optional[torch.Tensor] = None,
                 bias: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
                 epilogue: int = EPI_NONE, act: Optional[str] = None, out: Optional[torch.Tensor] = None,
                 ctx: Optional[device.Context] = None) -> torch.Tensor:
    """y = epilogue(x Wᵀ) (+ residual) through `s1_linear`. x `[T, K]`, weight `[N, K]` (row views allowed)."""
    _check(x, "x")
    _check(weight, "weight")
    T, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K:
        raise ValueError(f"weight is {tuple(weight.shape)}, x has K={K}")
    n_out = N // 2 if epilogue == EPI_GEGLU else N
    if weight_up is not None:
        _check(weight_up, "weight_up")
        if tuple(weight_up.shape) != (N, K):
            raise ValueError("weight_up must have the shape of weight")
    if residual is not None:
        _check(residual, "residual")
        if tuple(residual.shape) != (T, n_out):
            raise ValueError(f"residual must be {(T, n_out)}, got {tuple(residual.shape)}")
    if bias is not None and (bias.dtype != torch.bfloat16 or not bias.is_cuda or bias.numel() != N or not bias.is_contiguous()):
        raise ValueError("bias must be a contiguous bf16 CUDA vector of length N")
    if out is None:
        out = torch.empty((T, n_out), dtype=torch.bfloat16, device=x.device)
    else:
        _check(out, "out")
        if tuple(out.shape) != (T, n_out):
            raise ValueError(f"out must be {(T, n_out)}")
    if T == 0:
        return out
    if ctx is None:
        ctx = device.load(x.device.index)
    desc = LinearDesc(w=weight.data_ptr(), ldw=weight.stride(0),
                      w_up=0 if weight_up is None else weight_up.data_ptr(),
                      ldw_up=0 if weight_up is None else weight_up.stride(0),
                      bias=0 if bias is None else bias.data_ptr(),
                      N=N, K=K, epilogue=epilogue, act=_ACTS[act])
    rc = ctx._lib.s1_linear(ctx.handle, C.byref(desc), _ptr(x), x.stride(0), _ptr(residual),
                            0 if residual is None else residual.stride(0), _ptr(out), out.stride(0), T)
    ctx.check(rc)
    return out


def linear_rope(x: torch.Tensor, weight: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor,
                rotated_heads: int, out: Optional[torch.Tensor] = None, ctx: Optional[device.Context] = None) -> torch.Tensor:
    """`x W^T` with the rotate-half rotary embedding applied to the first `rotated_heads` 64-column heads of the
    output in the projection's epilogue (`s1_linear_rope`): Wqkv and `RotaryEmbedding::apply_qkv` of the reference
    (src/archs/modernbert.rs:184-205) as one launch. Tables f32 `[positions, 32]`, positions int32 `[T]`."""
    _check(x, "x")
    _check(weight, "weight")
    T, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K:
        raise ValueError(f"weight is {tuple(weight.shape)}, x has K={K}")
    for name, t in (("cos", cos), ("sin", sin)):
        if not t.is_cuda or t.dtype != torch.float32 or t.dim() != 2 or t.shape[1] != 32 or not t.is_contiguous():
            raise ValueError(f"{name} must be a contiguous f32 CUDA table [positions, 32]")
    if not positions.is_cuda or positions.dtype != torch.int32 or not positions.is_contiguous() or positions.numel() != T:
        raise ValueError("positions must be a contiguous int32 CUDA vector with one entry per row")
    if out is None:
        out = torch.empty((T, N), dtype=torch.bfloat16, device=x.device)
    else:
        _check(out, "out")
    if T == 0:
        return out
    if ctx is None:
        ctx = device.load(x.device.index)
    desc = LinearDesc(w=weight.data_ptr(), ldw=weight.stride(0), w_up=0, ldw_up=0, bias=0, N=N, K=K, epilogue=EPI_NONE, act=_ACTS[None])
    rc = ctx._lib.s1_linear_rope(ctx.handle, C.byref(desc), _ptr(x), x.stride(0), _ptr(out), out.stride(0), T, _ptr(cos), _ptr(sin),
                                 _ptr(positions), min(cos.shape[0], sin.shape[0]), int(rotated_heads))
    ctx.check(rc)
    return out


class Linear:
    """`candle_nn::Linear` as the reference builds it: `weight [out, in]`, optional `bias [out]`."""

    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
        _check(weight, "weight")
        self.weight = weight
        self.bias = bias

    def forward(self, x: torch.Tensor, *, residual: Optional[torch.Tensor] = None, act: Optional[str] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """`x.apply(&linear)`, optionally followed by the activation and the residual add of the caller."""
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        r2 = None if residual is None else residual.reshape(-1, residual.shape[-1])
        y = fused_linear(x2, self.weight, bias=self.bias, residual=r2, act=act, out=out)
        return y.reshape(*lead, y.shape[-1])

    __call__ = forward


def linear_no_bias(weight: torch.Tensor) -> Linear:
    """`linear_no_bias_dtype` (src/archs/modernbert.rs:1036-1046) for an already-loaded bf16 weight."""
    return Linear(weight, None)
