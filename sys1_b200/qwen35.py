"""Projection side and linear-attention recurrence of the Qwen3.5 layer (`src/archs/qwen35_text.rs`).

`Mlp` mirrors `Mlp { gate, up, down }` (:205-241); `chunked_delta_rule` mirrors the free function of the same
name (:789-807). Norms, RoPE, attention and the causal conv stay with the caller.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import device
from ._lib import EPI_SWIGLU
from .linear import Linear, fused_linear


class Mlp:
    """`down( silu(gate(x)) * up(x) )` (src/archs/qwen35_text.rs:232-240); gate/up are one contraction with the
    SwiGLU product in its epilogue; with `residual` the caller's `x + mlp(...)` (:939) is fused into `down`."""

    def __init__(self, gate: Linear, up: Linear, down: Linear):
        self.gate, self.up, self.down = gate, up, down

    def gated(self, x: torch.Tensor) -> torch.Tensor:
        return fused_linear(x, self.gate.weight, weight_up=self.up.weight, epilogue=EPI_SWIGLU)

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        return self.down.forward(self.gated(x), residual=residual)

    __call__ = forward


_workspaces = {}


def _workspace(dev: torch.device, nbytes: int) -> torch.Tensor:
    """Device scratch for the chunked kernels, grown on demand and kept per device (the library itself never
    allocates; a Rust caller would hand it a buffer from candle's pool the same way)."""
    ws = _workspaces.get(dev)
    if ws is None or ws.numel() < nbytes + 1024:
        ws = torch.empty(nbytes + 1024, dtype=torch.uint8, device=dev)
        _workspaces[dev] = ws
    return ws


def delta_rule_chunked_packed(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor,
                              cu_seqlens_host, ctx: Optional[device.Context] = None) -> torch.Tensor:
    """The recurrence in 64-token chunks on the tensor cores (`s1_delta_rule_chunked`): bf16 operand precision,
    f32 state; q, k, v `[T, H, 128]`. `cu_seqlens_host`: int32 offsets on the HOST (numpy array or CPU tensor)."""
    import numpy as np
    for name, t in (("q", q), ("k", k), ("v", v), ("g", g), ("beta", beta)):
        if not t.is_cuda or t.dtype != torch.float32 or not t.is_contiguous():
            raise ValueError(f"{name} must be a contiguous f32 CUDA tensor (no CPU fallback)")
    cu = np.ascontiguousarray(cu_seqlens_host.cpu().numpy() if isinstance(cu_seqlens_host, torch.Tensor) else cu_seqlens_host,
                              dtype=np.int32)
    T, H, Dk = q.shape
    Dv = v.shape[-1]
    out = torch.empty((T, H, Dv), dtype=torch.float32, device=q.device)
    if T == 0:
        return out
    if ctx is None:
        ctx = device.load(q.device.index)
    nseq = int(cu.shape[0] - 1)
    need = int(ctx._lib.s1_delta_rule_chunked_workspace(nseq, T, H))
    ws = _workspace(q.device, need)
    ptr = (ws.data_ptr() + 1023) // 1024 * 1024
    rc = ctx._lib.s1_delta_rule_chunked(ctx.handle, *(C.c_void_p(t.data_ptr()) for t in (q, k, v, g, beta)),
                                        cu.ctypes.data_as(C.POINTER(C.c_int32)), nseq, T, H, Dk, Dv,
                                        C.c_void_p(out.data_ptr()), C.c_void_p(ptr), need)
    ctx.check(rc)
    return out


def delta_rule_packed(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor,
                      cu_seqlens: torch.Tensor, ctx: Optional[device.Context] = None) -> torch.Tensor:
    """Gated delta rule on the packed layout, exact f32 token-by-token form: q, k `[T, H, 128]`, v `[T, H, Dv]`,
    g, beta `[T, H]` (f32, CUDA, contiguous), cu_seqlens int32 `[B+1]` on the same device. Returns `[T, H, Dv]`."""
    for name, t in (("q", q), ("k", k), ("v", v), ("g", g), ("beta", beta)):
        if not t.is_cuda or t.dtype != torch.float32 or not t.is_contiguous():
            raise ValueError(f"{name} must be a contiguous f32 CUDA tensor (no CPU fallback)")
    if cu_seqlens.dtype != torch.int32 or not cu_seqlens.is_cuda or not cu_seqlens.is_contiguous():
        raise ValueError("cu_seqlens must be a contiguous int32 CUDA tensor")
    T, H, Dk = q.shape
    Dv = v.shape[-1]
    if k.shape != q.shape or v.shape[:2] != (T, H) or g.shape != (T, H) or beta.shape != (T, H):
        raise ValueError("inconsistent shapes")
    out = torch.empty((T, H, Dv), dtype=torch.float32, device=q.device)
    if T == 0:
        return out
    if ctx is None:
        ctx = device.load(q.device.index)
    rc = ctx._lib.s1_delta_rule(ctx.handle, *(C.c_void_p(t.data_ptr()) for t in (q, k, v, g, beta, cu_seqlens)),
                                int(cu_seqlens.numel() - 1), T, H, Dk, Dv, C.c_void_p(out.data_ptr()))
    ctx.check(rc)
    return out


def chunked_delta_rule(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor,
                       beta: torch.Tensor) -> torch.Tensor:
    """Same signature and layouts as the reference (src/archs/qwen35_text.rs:789-795): q, k `[B, H, L, Dk]`,
    v `[B, H, L, Dv]`, g, beta `[B, H, L]`; returns `[B, L, H, Dv]`."""
    B, H, L, Dk = q.shape
    Dv = v.shape[-1]
    tok = lambda t: t.transpose(1, 2).reshape(B * L, H, -1).contiguous()
    cu = torch.arange(0, (B + 1) * L, L, dtype=torch.int32, device=q.device)
    out = delta_rule_packed(tok(q), tok(k), tok(v), g.transpose(1, 2).reshape(B * L, H).contiguous(),
                            beta.transpose(1, 2).reshape(B * L, H).contiguous(), cu)
    return out.reshape(B, L, H, Dv)


# ------------------------------------------------------------------------------------------------ linear attention
def _bf16(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda or t.dtype != torch.bfloat16 or t.stride(-1) != 1:
        raise ValueError(f"{name} must be a bf16 CUDA tensor with contiguous rows (no CPU fallback)")


def conv_silu(x: torch.Tensor, weight: torch.Tensor, positions: torch.Tensor, ctx: Optional[device.Context] = None) -> torch.Tensor:
    """`cuda_conv_silu(projected, conv)` (src/archs/qwen35_text.rs:652-735) on the packed layout: x `[T, C]` bf16,
    weight `[C, 1, taps]` bf16, positions int32 `[T]` (token index inside its sequence)."""
    _bf16(x, "x")
    _bf16(weight, "weight")
    T, Cc = x.shape
    w = weight.reshape(Cc, -1).contiguous()
    y = torch.empty((T, Cc), dtype=torch.bfloat16, device=x.device)
    if ctx is None:
        ctx = device.load(x.device.index)
    ctx.check(ctx._lib.s1_conv_silu(ctx.handle, C.c_void_p(x.data_ptr()), x.stride(0), C.c_void_p(w.data_ptr()),
                                    C.c_void_p(positions.data_ptr()), T, Cc, w.shape[1], C.c_void_p(y.data_ptr()), y.stride(0)))
    return y


class LinearAttention:
    """`LinearAttention` (src/archs/qwen35_text.rs:414-630) on a packed batch, same member names: `qkv`, `z`, `b`,
    `a`, `output` (Linear), `conv` `[C, 1, taps]`, `decay` (= -exp(A_log), f32), `dt_bias` (f32), `norm` `[128]`.
    Key and value head dim 128. `forward(x, batch)` takes `x [T, hidden]` bf16 and the `PackedBatch` that produced it."""

    def __init__(self, qkv: Linear, z: Linear, b: Linear, a: Linear, conv: torch.Tensor, decay: torch.Tensor,
                 dt_bias: torch.Tensor, norm: torch.Tensor, output: Linear, key_heads: int, value_heads: int, eps: float):
        self.qkv, self.z, self.b, self.a, self.output = qkv, z, b, a, output
        self.conv, self.decay, self.dt_bias, self.norm = conv, decay.float().contiguous(), dt_bias.float().contiguous(), norm
        self.key_heads, self.value_heads, self.eps = key_heads, value_heads, eps

    def forward(self, x: torch.Tensor, cu_seqlens_host, positions: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        import numpy as np
        ctx = device.load(x.device.index)
        T = x.shape[0]
        cu = np.ascontiguousarray(cu_seqlens_host, dtype=np.int32)
        mixed = conv_silu(self.qkv.forward(x), self.conv, positions, ctx)         # project_and_mix (:515-526)
        zz, bb, aa = self.z.forward(x), self.b.forward(x), self.a.forward(x)
        y = torch.empty((T, self.value_heads * 128), dtype=torch.bfloat16, device=x.device)
        need = int(ctx._lib.s1_gated_delta_rule_workspace(len(cu) - 1, T, self.value_heads))
        ws = _workspace(x.device, need)
        ptr = (ws.data_ptr() + 1023) // 1024 * 1024
        rc = ctx._lib.s1_gated_delta_rule(
            ctx.handle, C.c_void_p(mixed.data_ptr()), mixed.stride(0), C.c_void_p(bb.data_ptr()), C.c_void_p(aa.data_ptr()),
            bb.stride(0), C.c_void_p(self.dt_bias.data_ptr()), C.c_void_p(self.decay.data_ptr()), C.c_void_p(zz.data_ptr()),
            zz.stride(0), C.c_void_p(self.norm.data_ptr()), C.c_float(self.eps), cu.ctypes.data_as(C.POINTER(C.c_int32)),
            len(cu) - 1, T, self.key_heads, self.value_heads, C.c_void_p(y.data_ptr()), y.stride(0), C.c_void_p(ptr), need)
        ctx.check(rc)
        return self.output.forward(y, residual=residual)                           # out_proj (+ the layer's residual, :938)
