"""Projection side of the ModernBERT layer (`src/archs/modernbert.rs`): Wqkv, Wo(+residual), Wi+GeGLU, MLP-out(+residual).

Same member names as the reference structs (`Attention { wqkv, wo }` :137-175, `Mlp { input, output }`
:494-534, `Norm` :1006-1034, `RotaryEmbedding` :58-129), each a thin caller of the C ABI, and `Encoder`, the
layer stack on a token-packed batch.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import norm as _norm
from ._lib import EPI_GEGLU
from .linear import Linear, fused_linear, linear_rope


class Norm:
    """The bias-free LayerNorm of the reference (`Norm`, src/archs/modernbert.rs:1006-1034) through `s1_norm`."""

    def __init__(self, weight: torch.Tensor, eps: float):
        self.weight = weight.contiguous()
        self.eps = float(eps)

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None, gather: Optional[torch.Tensor] = None) -> torch.Tensor:
        return _norm.norm(x, self.weight, self.eps, _norm.LAYER_NORM, gather=gather, out=out)

    __call__ = forward


class RotaryEmbedding:
    """`RotaryEmbedding { sin, cos }` of the reference (tables `[positions, head_dim / 2]`, f32). `apply_qkv` is the
    reference's fused `rope_qkv` call (src/kernels/modernbert.cu:31-62) on the packed layout: q and k heads of the
    Wqkv output are rotated where they lie, each token by the table row of its position inside its own sequence."""

    def __init__(self, theta: float, head_dim: int, max_positions: int, dev):
        inv = torch.tensor([1.0 / (theta ** (j / head_dim)) for j in range(0, head_dim, 2)], dtype=torch.float32, device=dev)
        fr = torch.arange(max_positions, dtype=torch.float32, device=dev).unsqueeze(1) * inv.unsqueeze(0)
        self.cos, self.sin = fr.cos().contiguous(), fr.sin().contiguous()
        self.head_dim = head_dim

    def project_qkv(self, x: torch.Tensor, wqkv: Linear, positions: torch.Tensor, heads: int) -> torch.Tensor:
        """`x.apply(&self.wqkv)` followed by `apply_qkv` (src/archs/modernbert.rs:184-205) as one launch: the rotation
        happens in the projection's epilogue (`s1_linear_rope`)."""
        return linear_rope(x, wqkv.weight, self.cos, self.sin, positions, 2 * heads)

    def apply_qkv(self, qkv: torch.Tensor, positions: torch.Tensor, heads: int) -> torch.Tensor:
        """qkv bf16 `[T, 3 * heads * head_dim]`, positions int32 `[T]`; rotates the 2 * heads q and k heads in place."""
        return _norm.rope_(qkv, self.cos, self.sin, positions, 2 * heads, self.head_dim, self.head_dim)


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
    ws = ctx.workspace(need)
    planned = ctx.plan_covers(len(cu) - 1, T)   # the batch's tables are already on the device: no per-call copy
    rc = ctx._lib.s1_attention(ctx.handle, C.c_void_p(q.data_ptr()), q.stride(0), C.c_void_p(k.data_ptr()), k.stride(0),
                               C.c_void_p(v.data_ptr()), v.stride(0), None if planned else cu.ctypes.data_as(C.POINTER(C.c_int32)), len(cu) - 1, T, H, D,
                               int(window), C.c_float(D ** -0.5 if scale is None else scale), C.c_void_p(out.data_ptr()),
                               out.stride(0), C.c_void_p(ws.data_ptr()), ws.numel())
    ctx.check(rc)
    return out


class Encoder:
    """`Encoder::forward` (src/archs/modernbert.rs:958-989) on a token-packed batch, every stage through the C ABI:
    embedding lookup + embedding norm (`s1_norm` with a row index), per layer attn_norm -> Wqkv with RoPE in its
    epilogue (`s1_linear_rope`) -> flash-form attention (`s1_attention`) -> Wo with the residual stream updated in
    place -> mlp_norm -> Wi with GeGLU -> MLP-out with the residual stream updated in place, and the final norm.

    `weights`: dict of bf16 CUDA tensors under the checkpoint's names: `tok_embeddings [vocab, hidden]`,
    `embeddings_norm [hidden]`, `final_norm [hidden]` and, for every layer i, `layers.i.Wqkv [3 hidden, hidden]`,
    `layers.i.Wo [hidden, hidden]`, `layers.i.Wi [2 I, hidden]`, `layers.i.mlp_Wo [hidden, I]`, `layers.i.mlp_norm
    [hidden]` and (i > 0; layer 0 has none, :846-851) `layers.i.attn_norm [hidden]`.
    `cfg`: any object with the fields `hidden_size`, `num_hidden_layers`, `num_attention_heads`, `layer_norm_eps`,
    `global_attn_every_n_layers` (layer i is global iff i % n == 0, :920), `local_attention` (window = half of it,
    :977), `global_rope_theta`, `local_rope_theta`. Head dim must be 64."""

    def __init__(self, weights, cfg):
        self.cfg = cfg
        self.w = weights
        self.head_dim = cfg.hidden_size // cfg.num_attention_heads
        if self.head_dim != 64:
            raise ValueError("s1_attention is built for head_dim 64")
        self.layers = []
        self.norms = {}
        for i in range(cfg.num_hidden_layers):
            p = f"layers.{i}."
            self.layers.append((AttentionProjections(Linear(weights[p + "Wqkv"]), Linear(weights[p + "Wo"])),
                                Mlp(Linear(weights[p + "Wi"]), Linear(weights[p + "mlp_Wo"]))))
        for name, t in weights.items():
            if name.endswith("norm"):
                self.norms[name] = Norm(t, cfg.layer_norm_eps)
        self._rotary = {}

    def _rope(self, theta: float, length: int, dev) -> RotaryEmbedding:
        key = (theta, dev)
        if key not in self._rotary or self._rotary[key].cos.shape[0] < length:
            self._rotary[key] = RotaryEmbedding(theta, self.head_dim, max(length, 8192), dev)
        return self._rotary[key]

    def _ln(self, x: torch.Tensor, name: str, gather: Optional[torch.Tensor] = None) -> torch.Tensor:
        return self.norms[name](x, gather=gather)

    def _layer(self, i: int, x: torch.Tensor, bounds, pos: torch.Tensor, max_len: int) -> torch.Tensor:
        """`Layer::forward` (src/archs/modernbert.rs:857-887) for layer `i`; updates the residual stream `x` in place."""
        cfg = self.cfg
        H, D = cfg.num_attention_heads, self.head_dim
        T, dev = x.shape[0], x.device
        proj, mlp = self.layers[i]
        p = f"layers.{i}."
        local = i % cfg.global_attn_every_n_layers != 0
        n = x if i == 0 else self._ln(x, p + "attn_norm")
        rotary = self._rope(cfg.local_rope_theta if local else cfg.global_rope_theta, max_len, dev)
        attn = torch.empty((T, H * D), dtype=torch.bfloat16, device=dev)
        qkv = rotary.project_qkv(n, proj.wqkv, pos, H)   # Wqkv with RoPE in its epilogue
        q, k, v = qkv.view(T, 3, H, D).unbind(1)
        attention_varlen(q, k, v, bounds, window=cfg.local_attention // 2 if local else -1, out=attn)
        proj.wo.forward(attn, residual=x, out=x)                                        # x += attn Wo^T
        mlp.output.forward(mlp.gated(self._ln(x, p + "mlp_norm")), residual=x, out=x)   # x += geglu(LN(x) Wi^T) Wout^T
        return x

    @staticmethod
    def _bounds(cu_seqlens):
        bounds = [int(v) for v in cu_seqlens]
        return bounds, max((b - a for a, b in zip(bounds[:-1], bounds[1:])), default=0)

    def layer_forward(self, i: int, x: torch.Tensor, cu_seqlens, positions: torch.Tensor) -> torch.Tensor:
        """One layer on a given residual stream (a copy is updated and returned): for layer-by-layer checks."""
        bounds, max_len = self._bounds(cu_seqlens)
        return self._layer(i, x.clone(), bounds, positions.to(torch.int32).contiguous(), max_len)

    def forward(self, ids: torch.Tensor, cu_seqlens, positions: torch.Tensor, collect: bool = False):
        """ids int `[T]` (CUDA), cu_seqlens host int offsets `[B+1]`, positions int `[T]` (CUDA). Returns the final
        hidden states `[T, hidden]` bf16 (and, with `collect`, the residual stream after every layer)."""
        x = self._ln(self.w["tok_embeddings"], "embeddings_norm", gather=ids.to(torch.int32).contiguous())
        bounds, max_len = self._bounds(cu_seqlens)
        pos = positions.to(torch.int32).contiguous()
        states = []
        from . import device
        ctx = device.load(x.device.index)
        previous = getattr(ctx, "_plan", None)
        ctx.use_plan(self._plan(ctx, bounds))        # one table copy per batch, not one per layer
        try:
            for i in range(len(self.layers)):
                x = self._layer(i, x, bounds, pos, max_len)
                if collect:
                    states.append(x.clone())
        finally:
            ctx.use_plan(previous)
        y = self._ln(x, "final_norm")
        return (y, states) if collect else y

    def _plan(self, ctx, bounds):
        """The batch plan of these sequence offsets; the last few are kept, so a batch that comes again costs no copy."""
        key = (id(ctx), tuple(bounds))
        cache = self.__dict__.setdefault("_plans", {})
        if key not in cache:
            if len(cache) >= 4:
                cache.pop(next(iter(cache)))
            cache[key] = ctx.batch_plan(bounds, bounds[-1])
        return cache[key]
