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


_attn_ws = {}


def attention_varlen(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens_host, window: int = -1,
                     scale: Optional[float] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """`scaled_dot_product_attention` + `merge_heads` (src/archs/modernbert.rs:249-351) on a packed batch through
    `s1_attention`: q, k, v bf16 `[T, H, 64]` views whose rows are contiguous (token stride free), bidirectional,
    keys limited to the query's own sequence and, with `window >= 0`, to `|i - j| <= window`. Returns `[T, H * 64]`."""
    import ctypes as C
    import numpy as np
    from . import device
    T, H, D = q.shape
    for name, t in (("q", q), ("k", k), ("v", v)):
        if not t.is_cuda or t.dtype != torch.bfloat16 or t.stride(2) != 1 or t.stride(1) != D:
            raise ValueError(f"{name} must be a bf16 CUDA tensor [T, H, 64] with contiguous heads (no CPU fallback)")
    cu = np.ascontiguousarray(cu_seqlens_host, dtype=np.int32)
    if out is None:
        out = torch.empty((T, H * D), dtype=torch.bfloat16, device=q.device)
    if T == 0:
        return out
    ctx = device.load(q.device.index)
    need = int(ctx._lib.s1_attention_workspace(len(cu) - 1, T))
    ws = _attn_ws.get(q.device)
    if ws is None or ws.numel() < need:
        ws = torch.empty(max(need, 1 << 16), dtype=torch.uint8, device=q.device)
        _attn_ws[q.device] = ws
    rc = ctx._lib.s1_attention(ctx.handle, C.c_void_p(q.data_ptr()), q.stride(0), C.c_void_p(k.data_ptr()), k.stride(0),
                               C.c_void_p(v.data_ptr()), v.stride(0), cu.ctypes.data_as(C.POINTER(C.c_int32)), len(cu) - 1, T, H, D,
                               int(window), C.c_float(D ** -0.5 if scale is None else scale), C.c_void_p(out.data_ptr()),
                               out.stride(0), C.c_void_p(ws.data_ptr()), ws.numel())
    ctx.check(rc)
    return out


class Encoder:
    """`Encoder::forward` (src/archs/modernbert.rs:958-989) on a token-packed batch. The four projections of every
    layer run through the C ABI (Wqkv; Wo with the residual stream updated in place; Wi with GeGLU; MLP-out with the
    residual stream updated in place). Everything else - embedding lookup, LayerNorm (no bias), RoPE, softmax
    attention - is outside this repository's path and is done here with PyTorch operators, as harness code:
    attention is `scaled_dot_product_attention` per sequence, with the +-`local_attention/2` band on local layers.

    `weights`: dict with the names of `oracle.modernbert.init_weights` (bf16 CUDA tensors); `cfg`: any object with
    the fields of `oracle.modernbert.EncoderConfig`."""

    def __init__(self, weights, cfg, attention: str = "s1"):
        """`attention`: "s1" = this library's flash-form kernel (`s1_attention`), "torch" = PyTorch's
        `scaled_dot_product_attention` per sequence with an explicit band mask (harness fallback for comparison)."""
        self.attention = attention
        self.cfg = cfg
        self.w = weights
        self.layers = []
        for i in range(cfg.num_hidden_layers):
            p = f"layers.{i}."
            self.layers.append((AttentionProjections(Linear(weights[p + "Wqkv"]), Linear(weights[p + "Wo"])),
                                Mlp(Linear(weights[p + "Wi"]), Linear(weights[p + "mlp_Wo"]))))
        self._tables = {}
        self._bands = {}

    def _rope_tables(self, theta: float, length: int, dev):
        key = (theta, dev)
        if key not in self._tables or self._tables[key][0].shape[0] < length:
            d = self.cfg.hidden_size // self.cfg.num_attention_heads
            inv = torch.tensor([1.0 / (theta ** (j / d)) for j in range(0, d, 2)], dtype=torch.float32, device=dev)
            fr = torch.arange(max(length, 512), dtype=torch.float32, device=dev).unsqueeze(1) * inv.unsqueeze(0)
            self._tables[key] = (fr.cos(), fr.sin())
        return self._tables[key]

    def _band(self, length: int, dev):
        key = (length, dev)
        if key not in self._bands:
            idx = torch.arange(length, device=dev)
            self._bands[key] = (idx.unsqueeze(0) - idx.unsqueeze(1)).abs() <= self.cfg.local_attention // 2
        return self._bands[key]

    def _layer(self, i: int, x: torch.Tensor, bounds, pos: torch.Tensor, max_len: int) -> torch.Tensor:
        """`Layer::forward` (src/archs/modernbert.rs:857-887) for layer `i`; updates the residual stream `x` in place."""
        cfg = self.cfg
        F = torch.nn.functional
        H, D = cfg.num_attention_heads, cfg.hidden_size // cfg.num_attention_heads
        T, dev = x.shape[0], x.device
        ln = lambda t, name: F.layer_norm(t, (cfg.hidden_size,), self.w[name], None, cfg.layer_norm_eps)
        proj, mlp = self.layers[i]
        p = f"layers.{i}."
        local = i % cfg.global_attn_every_n_layers != 0
        n = x if i == 0 else ln(x, p + "attn_norm")
        qkv = proj.qkv(n).view(T, 3, H, D)
        cos, sin = self._rope_tables(cfg.local_rope_theta if local else cfg.global_rope_theta, max_len, dev)
        c, s = cos[pos].unsqueeze(1), sin[pos].unsqueeze(1)

        def rot(t):
            t = t.float()
            t1, t2 = t[..., : D // 2], t[..., D // 2:]
            return torch.cat([t1 * c - t2 * s, t1 * s + t2 * c], dim=-1).to(torch.bfloat16)

        q, k, v = rot(qkv[:, 0]), rot(qkv[:, 1]), qkv[:, 2]
        attn = torch.empty((T, H * D), dtype=torch.bfloat16, device=dev)
        if self.attention == "s1" and D == 64:
            attention_varlen(q, k, v, bounds, window=cfg.local_attention // 2 if local else -1, out=attn)
        else:
            for a, b in zip(bounds[:-1], bounds[1:]):
                if a == b:
                    continue
                mask = self._band(b - a, dev) if local else None
                o = F.scaled_dot_product_attention(q[a:b].transpose(0, 1).unsqueeze(0), k[a:b].transpose(0, 1).unsqueeze(0),
                                                   v[a:b].transpose(0, 1).unsqueeze(0), attn_mask=mask)
                attn[a:b] = o[0].transpose(0, 1).reshape(b - a, H * D)
        proj.wo.forward(attn, residual=x, out=x)                                  # x += attn Wo^T
        mlp.output.forward(mlp.gated(ln(x, p + "mlp_norm")), residual=x, out=x)   # x += geglu(LN(x) Wi^T) Wout^T
        return x

    def layer_forward(self, i: int, x: torch.Tensor, cu_seqlens, positions: torch.Tensor) -> torch.Tensor:
        """One layer on a given residual stream (a copy is updated and returned): for layer-by-layer checks."""
        bounds = [int(v) for v in cu_seqlens]
        max_len = max((b - a for a, b in zip(bounds[:-1], bounds[1:])), default=0)
        return self._layer(i, x.clone(), bounds, positions.long(), max_len)

    def forward(self, ids: torch.Tensor, cu_seqlens, positions: torch.Tensor, collect: bool = False):
        """ids int64 `[T]` (CUDA), cu_seqlens host int offsets `[B+1]`, positions int `[T]` (CUDA). Returns the final
        hidden states `[T, hidden]` bf16 (and, with `collect`, the residual stream after every layer)."""
        cfg = self.cfg
        F = torch.nn.functional
        H, D = cfg.num_attention_heads, cfg.hidden_size // cfg.num_attention_heads
        T = ids.shape[0]
        dev = ids.device
        eps = cfg.layer_norm_eps
        ln = lambda t, name: F.layer_norm(t, (cfg.hidden_size,), self.w[name], None, eps)
        x = ln(self.w["tok_embeddings"][ids], "embeddings_norm").contiguous()
        bounds = [int(v) for v in cu_seqlens]
        max_len = max((b - a for a, b in zip(bounds[:-1], bounds[1:])), default=0)
        pos = positions.long()
        states = []
        for i in range(len(self.layers)):
            x = self._layer(i, x, bounds, pos, max_len)
            if collect:
                states.append(x.clone())
        y = ln(x, "final_norm")
        return (y, states) if collect else y
