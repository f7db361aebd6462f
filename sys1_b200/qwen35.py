"""Projection side and linear-attention recurrence of the Qwen3.5 layer (`src/archs/qwen35_text.rs`).

`Mlp` mirrors `Mlp { gate, up, down }` (:205-241); `chunked_delta_rule` mirrors the free function of the same
name (:789-807); `RmsNorm`, `FullAttention`, `LinearAttention`, `Layer` and `Decoder` mirror the structs of the same
names on a token-packed batch. Everything runs through the C ABI.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import device
from . import norm as _norm
from ._lib import EPI_SWIGLU
from .linear import Linear, fused_linear


class RmsNorm:
    """`RmsNorm` (src/archs/qwen35_text.rs:178-203): x / sqrt(mean(x^2) + eps) * (1 + weight), through `s1_norm`."""

    def __init__(self, weight: torch.Tensor, eps: float):
        self.weight, self.eps = weight.contiguous(), float(eps)

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        return _norm.norm(x, self.weight, self.eps, _norm.RMS_NORM, out=out)

    __call__ = forward


class Mlp:
    """`down( silu(gate(x)) * up(x) )` (src/archs/qwen35_text.rs:232-240); gate/up are one contraction with the
    SwiGLU product in its epilogue; with `residual` the caller's `x + mlp(...)` (:939) is fused into `down`."""

    def __init__(self, gate: Linear, up: Linear, down: Linear):
        self.gate, self.up, self.down = gate, up, down

    def gated(self, x: torch.Tensor) -> torch.Tensor:
        return fused_linear(x, self.gate.weight, weight_up=self.up.weight, epilogue=EPI_SWIGLU)

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None, inplace: bool = False) -> torch.Tensor:
        """`inplace`: write `residual + mlp(x)` into `residual` itself (the residual stream updated in memory by the
        projection's store, no read of it by the SMs)."""
        return self.down.forward(self.gated(x), residual=residual, out=residual if inplace else None)

    __call__ = forward


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
    ptr = ctx.workspace(need).data_ptr()
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
                 dt_bias: torch.Tensor, norm: torch.Tensor, output: Linear, key_heads: int, value_heads: int, eps: float,
                 merge_inputs: bool = True, recurrence: str = "chunked", fuse_conv: bool = True):
        """`recurrence`: "chunked" (default) evaluates the gated delta rule in 64-token chunks on the tensor cores with
        bf16 operands and f32 state (`s1_gated_delta_rule`; within 2e-2 of the output scale of the f32 recurrence, which
        is the layer-level bound of this path); "exact" runs the token-sequential f32 kernel (`s1_delta_rule`, the
        reference's own arithmetic and its 1e-4 bound), about three times slower.
        `fuse_conv` (chunked recurrence, 4 taps): the causal conv + SiLU is applied by the recurrence's first kernel to the rows
        it stages (`s1_gated_delta_rule_conv`) instead of by a kernel of its own that writes the `[T, channels]` tensor out and
        the next one reads back; bit-identical to the two calls.
        `merge_inputs`: stack the four input projections, which share their input, into one weight `[N_qkv + N_z + 2 Hv,
        K]` at load time, so that they run as one contraction (two of them are only `Hv` = 16 or 48 columns wide, a
        launch each for next to no work); the outputs are column views of one buffer."""
        self.qkv, self.z, self.b, self.a, self.output = qkv, z, b, a, output
        self.conv, self.decay, self.dt_bias, self.norm = conv, decay.float().contiguous(), dt_bias.float().contiguous(), norm
        self.key_heads, self.value_heads, self.eps = key_heads, value_heads, eps
        if recurrence not in ("chunked", "exact"):
            raise ValueError("recurrence must be 'chunked' or 'exact'")
        self.recurrence = recurrence
        self.conv_taps = conv.reshape(conv.shape[0], -1).contiguous()   # [C, taps]
        self.fuse_conv = bool(fuse_conv) and recurrence == "chunked" and self.conv_taps.shape[1] == 4
        self.merged = None
        if merge_inputs and all(l.bias is None for l in (qkv, z, b, a)):
            # b and a are only `value_heads` rows each (6 on a tensor-parallel rank of the large model): padded with zero
            # rows to a multiple of 8, the width the projection kernel stores in
            def pad8(w):
                extra = (-w.shape[0]) % 8
                return w if extra == 0 else torch.cat([w, torch.zeros(extra, w.shape[1], dtype=w.dtype, device=w.device)], dim=0)
            parts = [qkv.weight, z.weight, pad8(b.weight), pad8(a.weight)]
            if all(w.shape[0] % 8 == 0 for w in parts):
                self.merged = Linear(torch.cat(parts, dim=0).contiguous())
                self._splits = [(w.shape[0], n) for w, n in zip(parts, (qkv.weight.shape[0], z.weight.shape[0], b.weight.shape[0], a.weight.shape[0]))]

    def _inputs(self, x: torch.Tensor):
        """mixed-pre-conv, z, b, a: the four input projections of `x` (`project_and_mix` up to the conv, :515-526, :567-568)."""
        if self.merged is None:
            return self.qkv.forward(x), self.z.forward(x), self.b.forward(x), self.a.forward(x)
        y = self.merged.forward(x)
        outs, at = [], 0
        for padded, n in self._splits:
            outs.append(y[:, at:at + n])
            at += padded
        return tuple(outs)

    def forward(self, x: torch.Tensor, cu_seqlens_host, positions: torch.Tensor, residual: Optional[torch.Tensor] = None,
                inplace: bool = False) -> torch.Tensor:
        y = self.mix(x, cu_seqlens_host, positions)
        return self.output.forward(y, residual=residual, out=residual if inplace else None)  # out_proj (+ the layer's residual, :938)

    def mix(self, x: torch.Tensor, cu_seqlens_host, positions: torch.Tensor) -> torch.Tensor:
        """Everything up to the input of `out_proj`: `[T, value_heads * 128]` bf16."""
        import numpy as np
        ctx = device.load(x.device.index)
        T = x.shape[0]
        cu = np.ascontiguousarray(cu_seqlens_host, dtype=np.int32)
        pre, zz, bb, aa = self._inputs(x)
        y = torch.empty((T, self.value_heads * 128), dtype=torch.bfloat16, device=x.device)
        P = lambda t: C.c_void_p(t.data_ptr())
        if self.recurrence == "exact":
            mixed = conv_silu(pre, self.conv, positions, ctx)                     # project_and_mix (:515-526)
            self._exact(ctx, mixed, zz, bb, aa, cu, y)
            return y
        need = int(ctx._lib.s1_gated_delta_rule_workspace(len(cu) - 1, T, self.value_heads))
        ptr = ctx.workspace(need).data_ptr()
        planned = ctx.plan_covers(len(cu) - 1, T)
        offsets = None if planned else cu.ctypes.data_as(C.POINTER(C.c_int32))
        tail = (P(bb), P(aa), bb.stride(0), P(self.dt_bias), P(self.decay), P(zz), zz.stride(0), P(self.norm), C.c_float(self.eps), offsets,
                len(cu) - 1, T, self.key_heads, self.value_heads, P(y), y.stride(0), C.c_void_p(ptr), need)
        if self.fuse_conv:
            pos = positions if positions.dtype == torch.int32 and positions.is_contiguous() else positions.to(torch.int32).contiguous()
            rc = ctx._lib.s1_gated_delta_rule_conv(ctx.handle, P(pre), pre.stride(0), P(self.conv_taps), P(pos), *tail)
        else:
            mixed = conv_silu(pre, self.conv, positions, ctx)                     # project_and_mix (:515-526)
            rc = ctx._lib.s1_gated_delta_rule(ctx.handle, P(mixed), mixed.stride(0), *tail)
        ctx.check(rc)
        return y

    def _exact(self, ctx, mixed, zz, bb, aa, cu, y) -> None:
        """The reference's own precision: `delta_inputs` -> token-sequential f32 recurrence -> `finish_delta`
        (`s1_delta_inputs`, `s1_delta_rule`, `s1_delta_finish`), f32 between the three."""
        T, Hv = mixed.shape[0], self.value_heads
        f32 = dict(dtype=torch.float32, device=mixed.device)
        q, k, v = (torch.empty((T, Hv, 128), **f32) for _ in range(3))
        g, beta = (torch.empty((T, Hv), **f32) for _ in range(2))
        P = lambda t: C.c_void_p(t.data_ptr())
        ctx.check(ctx._lib.s1_delta_inputs(ctx.handle, P(mixed), mixed.stride(0), P(bb), P(aa), bb.stride(0), P(self.dt_bias),
                                           P(self.decay), T, self.key_heads, Hv, P(q), P(k), P(v), P(g), P(beta)))
        cu_dev = torch.from_numpy(cu).to(mixed.device)
        o = delta_rule_packed(q, k, v, g, beta, cu_dev, ctx)
        ctx.check(ctx._lib.s1_delta_finish(ctx.handle, P(o), P(zz), zz.stride(0), P(self.norm), C.c_float(self.eps), T, Hv,
                                           P(y), y.stride(0)))


class RopeParams:
    """`RopeParams` (src/archs/qwen35_text.rs:101-165) for text-only inputs (the three position axes coincide):
    tables `[positions, rotary_dim / 2]`, phase = position / theta^(2 j / rotary_dim), values rounded to the model
    dtype (bf16) as the reference casts its tables, kept as f32 for `s1_rope`."""

    def __init__(self, theta: float, rotary_dim: int, max_positions: int, dev):
        div = torch.tensor([float(theta) ** (2.0 * j / rotary_dim) for j in range(rotary_dim // 2)], dtype=torch.float64).to(torch.float32).to(dev)
        phase = torch.arange(max_positions, dtype=torch.float32, device=dev).unsqueeze(1) / div.unsqueeze(0)
        self.cos = phase.cos().to(torch.bfloat16).float().contiguous()
        self.sin = phase.sin().to(torch.bfloat16).float().contiguous()
        self.rotary_dim = rotary_dim


def attention_causal_gqa(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens_host, gate: Optional[torch.Tensor] = None,
                         out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal grouped-query attention over a packed batch through `s1_attention_gqa` (head dim 256):
    q `[T, H, 256]` (rows may be strided: the query halves of the interleaved q_proj output), k, v `[T, KV, 256]`,
    optional `gate [T, H, 256]` (pre-sigmoid; the output is multiplied by sigmoid(gate)). Returns `[T, H * 256]`."""
    import numpy as np
    T, H, D = q.shape
    KV = k.shape[1]
    cu = np.ascontiguousarray(cu_seqlens_host, dtype=np.int32)
    if out is None:
        out = torch.empty((T, H * D), dtype=torch.bfloat16, device=q.device)
    if T == 0:
        return out
    for name, t in (("q", q), ("k", k), ("v", v)) + ((("gate", gate),) if gate is not None else ()):
        if not t.is_cuda or t.dtype != torch.bfloat16 or t.stride(2) != 1:
            raise ValueError(f"{name} must be a bf16 CUDA tensor [T, heads, 256] with contiguous head rows (no CPU fallback)")
    ctx = device.load(q.device.index)
    need = int(ctx._lib.s1_attention_gqa_workspace(len(cu) - 1, T))
    ws = ctx.workspace(need)
    planned = ctx.plan_covers(len(cu) - 1, T)
    rc = ctx._lib.s1_attention_gqa(
        ctx.handle, C.c_void_p(q.data_ptr()), q.stride(0), q.stride(1), C.c_void_p(k.data_ptr()), k.stride(0), k.stride(1),
        C.c_void_p(v.data_ptr()), v.stride(0), v.stride(1), C.c_void_p(gate.data_ptr() if gate is not None else 0),
        gate.stride(0) if gate is not None else 0, gate.stride(1) if gate is not None else 0,
        None if planned else cu.ctypes.data_as(C.POINTER(C.c_int32)), len(cu) - 1, T, H, KV, D, C.c_float(D ** -0.5), C.c_void_p(out.data_ptr()),
        out.stride(0), C.c_void_p(ws.data_ptr()), ws.numel())
    ctx.check(rc)
    return out


class FullAttention:
    """`FullAttention` (src/archs/qwen35_text.rs:242-411) on a packed batch, same member names: `q` (query and output
    gate interleaved per head), `k`, `v`, `output`, `q_norm`, `k_norm`. The three input projections share their input and
    run as one contraction over the stacked weight `[q | k | v]`; `q_norm` / `k_norm` and the partial rotation are one
    pass each over the query halves and the key heads (`s1_head_norm_rope`), rounding as candle's bf16 ops do."""

    def __init__(self, q: Linear, k: Linear, v: Linear, output: Linear, q_norm: RmsNorm, k_norm: RmsNorm, heads: int, kv_heads: int,
                 head_dim: int, rope: RopeParams):
        self.q, self.k, self.v, self.output, self.q_norm, self.k_norm = q, k, v, output, q_norm, k_norm
        self.heads, self.kv_heads, self.head_dim, self.rope = heads, kv_heads, head_dim, rope
        self.merged = None
        if all(l.bias is None for l in (q, k, v)):
            self.merged = Linear(torch.cat([q.weight, k.weight, v.weight], dim=0).contiguous())

    def forward(self, x: torch.Tensor, cu_seqlens_host, positions: torch.Tensor, residual: Optional[torch.Tensor] = None,
                inplace: bool = False) -> torch.Tensor:
        gated = self.mix(x, cu_seqlens_host, positions)
        return self.output.forward(gated, residual=residual, out=residual if inplace else None)

    def mix(self, x: torch.Tensor, cu_seqlens_host, positions: torch.Tensor) -> torch.Tensor:
        """Everything up to the input of `o_proj`: the gated attention output `[T, heads * head_dim]` bf16."""
        T, H, KV, D = x.shape[0], self.heads, self.kv_heads, self.head_dim
        if self.merged is not None:
            qkv = self.merged.forward(x)                        # [T, H * 2 * D + 2 * KV * D]
            qg, k, v = qkv[:, :2 * H * D], qkv[:, 2 * H * D:2 * H * D + KV * D], qkv[:, 2 * H * D + KV * D:]
        else:
            qg, k, v = self.q.forward(x), self.k.forward(x), self.v.forward(x)
        r = self.rope
        # per head [query | gate]: norm + rotation of the query halves, then of the key heads, each where it lies
        _norm.head_norm_rope_(qg, H, 2 * D, D, self.q_norm.weight, self.q_norm.eps, r.cos, r.sin, positions, r.rotary_dim)
        _norm.head_norm_rope_(k, KV, D, D, self.k_norm.weight, self.k_norm.eps, r.cos, r.sin, positions, r.rotary_dim)
        q4 = qg.unflatten(1, (H, 2, D))
        return attention_causal_gqa(q4[:, :, 0], k.unflatten(1, (KV, D)), v.unflatten(1, (KV, D)), cu_seqlens_host, gate=q4[:, :, 1])


class Layer:
    """`Layer` (src/archs/qwen35_text.rs:890-940): x + mixer(RMS(x)), then x + MLP(RMS(x)); both residual adds are
    fused into the output projections."""

    def __init__(self, input_norm: RmsNorm, mixer, post_norm: RmsNorm, mlp: Mlp):
        self.input_norm, self.mixer, self.post_norm, self.mlp = input_norm, mixer, post_norm, mlp

    def forward(self, x: torch.Tensor, cu_seqlens_host, positions: torch.Tensor, inplace: bool = False) -> torch.Tensor:
        """`inplace`: update the residual stream `x` in memory (both adds become part of the projections' stores)."""
        x = self.mixer.forward(self.input_norm(x), cu_seqlens_host, positions, residual=x, inplace=inplace)
        return self.mlp.forward(self.post_norm(x), residual=x, inplace=inplace)


class Decoder:
    """`Decoder::forward` (src/archs/qwen35_text.rs:942-1005) on a token-packed batch.

    `weights`: dict of CUDA tensors under the checkpoint's names (bf16 unless noted): `embed_tokens [vocab, hidden]`,
    `norm [hidden]` and per layer i `layers.i.input_layernorm`, `layers.i.post_attention_layernorm` `[hidden]`,
    `layers.i.mlp.{gate_proj, up_proj} [I, hidden]`, `layers.i.mlp.down_proj [hidden, I]`; full-attention layers:
    `layers.i.self_attn.q_proj [2 H D, hidden]` (query and gate interleaved per head), `.k_proj`, `.v_proj [KV D, hidden]`,
    `.o_proj [hidden, H D]`, `.q_norm`, `.k_norm [D]`; linear-attention layers: `layers.i.linear_attn.in_proj_qkv
    [2 Hk 128 + Hv 128, hidden]`, `.in_proj_z [Hv 128, hidden]`, `.in_proj_b`, `.in_proj_a [Hv, hidden]`, `.conv1d
    [C, 1, taps]`, `.A_log`, `.dt_bias [Hv]` (f32), `.norm [128]`, `.out_proj [hidden, Hv 128]`.
    `cfg`: any object with `num_hidden_layers`, `layer_type(i)` ("full_attention" / "linear_attention"),
    `num_attention_heads`, `num_key_value_heads`, `head_dim`, `rms_norm_eps`, `rope_theta`, `rotary_dim`,
    `linear_num_key_heads`, `linear_num_value_heads`.
    `recurrence`: "chunked" (default; tensor cores, bf16 operands) or "exact" (f32, token-sequential) for the
    linear-attention layers, see `LinearAttention`."""

    def __init__(self, weights, cfg, max_positions: int = 8192, recurrence: str = "chunked"):
        self.cfg, self.w = cfg, weights
        dev = weights["embed_tokens"].device
        lin = lambda name: Linear(weights[name])
        rope = RopeParams(cfg.rope_theta, cfg.rotary_dim, max_positions, dev)
        self.layers = []
        for i in range(cfg.num_hidden_layers):
            p = f"layers.{i}."
            if cfg.layer_type(i) == "full_attention":
                a = p + "self_attn."
                mixer = FullAttention(lin(a + "q_proj"), lin(a + "k_proj"), lin(a + "v_proj"), lin(a + "o_proj"),
                                      RmsNorm(weights[a + "q_norm"], cfg.rms_norm_eps), RmsNorm(weights[a + "k_norm"], cfg.rms_norm_eps),
                                      cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, rope)
            else:
                a = p + "linear_attn."
                mixer = LinearAttention(lin(a + "in_proj_qkv"), lin(a + "in_proj_z"), lin(a + "in_proj_b"), lin(a + "in_proj_a"),
                                        weights[a + "conv1d"], -torch.exp(weights[a + "A_log"].float()), weights[a + "dt_bias"].float(),
                                        weights[a + "norm"], lin(a + "out_proj"), cfg.linear_num_key_heads, cfg.linear_num_value_heads,
                                        cfg.rms_norm_eps, recurrence=recurrence)
            self.layers.append(Layer(RmsNorm(weights[p + "input_layernorm"], cfg.rms_norm_eps), mixer,
                                     RmsNorm(weights[p + "post_attention_layernorm"], cfg.rms_norm_eps),
                                     Mlp(lin(p + "mlp.gate_proj"), lin(p + "mlp.up_proj"), lin(p + "mlp.down_proj"))))
        self.norm = RmsNorm(weights["norm"], cfg.rms_norm_eps)

    def forward(self, ids: torch.Tensor, cu_seqlens_host, positions: torch.Tensor, collect: bool = False):
        x = _norm.embedding(self.w["embed_tokens"], ids.to(torch.int32).contiguous())
        pos = positions.to(torch.int32).contiguous()
        states = []
        ctx = device.load(x.device.index)
        bounds = [int(v) for v in cu_seqlens_host]
        previous = getattr(ctx, "_plan", None)
        ctx.use_plan(batch_plan_cached(self, ctx, bounds))   # one table copy per batch, not one per layer
        try:
            for layer in self.layers:
                x = layer.forward(x, cu_seqlens_host, pos, inplace=True)  # x is this call's own buffer (the embedding rows)
                if collect:
                    states.append(x.clone())
        finally:
            ctx.use_plan(previous)
        y = self.norm(x)
        return (y, states) if collect else y


def batch_plan_cached(owner, ctx, bounds):
    """The batch plan (`s1_batch_plan`) of these sequence offsets on this context; `owner` keeps the last few, so a
    batch that comes again costs no copy."""
    key = (id(ctx), tuple(bounds))
    cache = owner.__dict__.setdefault("_plans", {})
    if key not in cache:
        if len(cache) >= 8:
            cache.pop(next(iter(cache)))
        cache[key] = ctx.batch_plan(bounds, bounds[-1])
    return cache[key]
