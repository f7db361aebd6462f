"""Oracle for the ModernBERT encoder forward (test infrastructure only; see the package docstring).

Restates `Encoder::forward` / `Layer::forward` / `Attention::forward` of src/archs/modernbert.rs (:958-989,
:857-887, :176-192) for sequences without padding, one sequence at a time (which is what the reference's padded
batch computes for each row once padded keys are masked out):
  x = LN(tok_emb[ids]); per layer i: n = x (i == 0, no attn_norm weight: :846-851) or LN(x);
  qkv = n Wqkv^T -> [L, 3, H, D]; rotate-half RoPE on q, k with f32 tables, theta global / local (:58-110, :908-929);
  a = softmax(q k^T / sqrt(D) + mask) v, mask = -10000 where |i - j| > local_attention / 2 on local layers
  (i % global_attn_every_n_layers != 0, :920, :973-977, :1058-1076); x = x + a Wo^T; m = LN(x) Wi^T;
  x = x + geglu(m) Wout^T; finally LN(x) (:988).
LayerNorm has a weight and no bias (`LayerNorm::new_no_bias`, :1006-1034).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Sequence

import torch

from .norm import layer_norm, rope
from .projection import geglu, linear, round_bf16

MASK_VALUE = -10_000.0  # ATTENTION_MASK_VALUE, src/archs/modernbert.rs:23


@dataclass(frozen=True)
class EncoderConfig:
    vocab_size: int = 50368
    hidden_size: int = 768
    num_hidden_layers: int = 22
    num_attention_heads: int = 12
    intermediate_size: int = 1152
    layer_norm_eps: float = 1e-5
    global_attn_every_n_layers: int = 3
    local_attention: int = 128
    global_rope_theta: float = 160000.0
    local_rope_theta: float = 10000.0

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads


def init_weights(cfg: EncoderConfig, seed: int) -> Dict[str, torch.Tensor]:
    """Random-init weights N(0, 0.02) from `seed`, norm weights 1 (float32; cast by the caller)."""
    g = torch.Generator().manual_seed(seed)
    w = {"tok_embeddings": torch.randn(cfg.vocab_size, cfg.hidden_size, generator=g) * 0.02,
         "embeddings_norm": torch.ones(cfg.hidden_size), "final_norm": torch.ones(cfg.hidden_size)}
    for i in range(cfg.num_hidden_layers):
        p = f"layers.{i}."
        w[p + "Wqkv"] = torch.randn(3 * cfg.hidden_size, cfg.hidden_size, generator=g) * 0.02
        w[p + "Wo"] = torch.randn(cfg.hidden_size, cfg.hidden_size, generator=g) * 0.02
        w[p + "Wi"] = torch.randn(2 * cfg.intermediate_size, cfg.hidden_size, generator=g) * 0.02
        w[p + "mlp_Wo"] = torch.randn(cfg.hidden_size, cfg.intermediate_size, generator=g) * 0.02
        if i > 0:
            w[p + "attn_norm"] = torch.ones(cfg.hidden_size)
        w[p + "mlp_norm"] = torch.ones(cfg.hidden_size)
    return w


def rope_tables(cfg: EncoderConfig, theta: float, length: int):
    d = cfg.head_dim
    inv = torch.tensor([1.0 / (theta ** (j / d)) for j in range(0, d, 2)], dtype=torch.float32)
    freqs = torch.arange(length, dtype=torch.float32).unsqueeze(1) * inv.unsqueeze(0)
    return freqs.cos(), freqs.sin()


def encoder_layer(i: int, x: torch.Tensor, w: Dict[str, torch.Tensor], cfg: EncoderConfig, dtype: str = "f32") -> torch.Tensor:
    """`Layer::forward` (src/archs/modernbert.rs:857-887) for layer `i` of one unpadded sequence: residual stream
    `x [L, hidden]` in, residual stream out."""
    r = (lambda t: round_bf16(t)) if dtype == "bf16" else (lambda t: t)
    L = x.shape[0]
    H, D = cfg.num_attention_heads, cfg.head_dim
    p = f"layers.{i}."
    local = i % cfg.global_attn_every_n_layers != 0
    n = x if i == 0 else layer_norm(x, w[p + "attn_norm"], cfg.layer_norm_eps, dtype)
    qkv = linear(n, w[p + "Wqkv"], dtype=dtype).reshape(L, 3, H, D)
    cos, sin = rope_tables(cfg, cfg.local_rope_theta if local else cfg.global_rope_theta, L)
    q, k, v = r(rope(qkv[:, 0], cos, sin)), r(rope(qkv[:, 1], cos, sin)), qkv[:, 2]
    scores = r(torch.einsum("ihd,jhd->hij", r(q * D ** -0.5), k))
    if local:
        idx = torch.arange(L)
        scores = scores + torch.where((idx.unsqueeze(0) - idx.unsqueeze(1)).abs() > cfg.local_attention // 2,
                                      MASK_VALUE, 0.0)
    probs = r(torch.softmax(scores, dim=-1))
    attn = r(torch.einsum("hij,jhd->ihd", probs, v)).reshape(L, H * D)
    x = linear(attn, w[p + "Wo"], residual=x, dtype=dtype)
    m = geglu(linear(layer_norm(x, w[p + "mlp_norm"], cfg.layer_norm_eps, dtype), w[p + "Wi"], dtype=dtype), dtype)
    return linear(m, w[p + "mlp_Wo"], residual=x, dtype=dtype)


def encoder_forward(ids: torch.Tensor, w: Dict[str, torch.Tensor], cfg: EncoderConfig, dtype: str = "f32",
                    collect: bool = False):
    """One unpadded sequence `ids [L]` -> final hidden `[L, hidden]` (float32 values of the requested precision);
    with `collect`, also the list of hidden states after every layer."""
    x = layer_norm(w["tok_embeddings"][ids].to(torch.float32), w["embeddings_norm"], cfg.layer_norm_eps, dtype)
    states: List[torch.Tensor] = []
    for i in range(cfg.num_hidden_layers):
        x = encoder_layer(i, x, w, cfg, dtype)
        if collect:
            states.append(x)
    y = layer_norm(x, w["final_norm"], cfg.layer_norm_eps, dtype)
    return (y, states) if collect else y


def local_attention_mask(length: int, max_distance: int) -> torch.Tensor:
    """`local_attention_mask` (src/archs/modernbert.rs:1058-1076): `[L, L]`, -10000 where |i - j| > max_distance, else 0."""
    idx = torch.arange(length)
    return torch.where((idx.unsqueeze(0) - idx.unsqueeze(1)).abs() > max_distance, MASK_VALUE, 0.0)


def global_attention_mask(keep: torch.Tensor, target_length: int) -> torch.Tensor:
    """`global_attention_mask` (src/archs/modernbert.rs:1048-1056): `keep [B, S]` (1 = token, 0 = padding) ->
    `[B, 1, target_length, S]` with -10000 on the padded keys."""
    b, s = keep.shape
    return (1.0 - keep.to(torch.float32).reshape(b, 1, 1, s).expand(b, 1, target_length, s)) * MASK_VALUE


def attention_softmax(scores: torch.Tensor, dtype: str = "f32") -> torch.Tensor:
    """`attention_softmax` (src/archs/modernbert.rs:393-399): half-precision scores are widened to f32 for the
    softmax and the probabilities rounded back."""
    p = torch.softmax(scores.to(torch.float32), dim=-1)
    return round_bf16(p) if dtype == "bf16" else p


def eager_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, mask=None, dtype: str = "f32") -> torch.Tensor:
    """`eager_attention` (src/archs/modernbert.rs:337-351) in the reference's own layout: q, k, v `[B, H, L, D]`,
    additive `mask` broadcastable to `[B, H, L, S]`; returns `[B, H, L, D]`."""
    r = (lambda t: round_bf16(t)) if dtype == "bf16" else (lambda t: t)
    scores = r(r(q.float() * scale) @ k.float().transpose(-2, -1))
    if mask is not None:
        scores = r(scores + mask)
    return r(attention_softmax(scores, dtype) @ v.float())


def windowed_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, mask, window: int, dtype: str = "f32") -> torch.Tensor:
    """`cpu_windowed_attention` (src/archs/modernbert.rs:353-391): query blocks of ceil(window / 2) rows, each against
    the keys within `window` of the block, the matching part of the mask cut out; short inputs take the dense path."""
    length = q.shape[2]
    if length <= window + window // 4:
        return eager_attention(q, k, v, scale, mask, dtype)
    block = max((window + 1) // 2, 1)
    outs = []
    for qs in range(0, length, block):
        ql = min(block, length - qs)
        ks, ke = max(qs - window, 0), min(qs + ql + window, length)
        m = None
        if mask is not None:
            m = mask[qs:qs + ql, ks:ke].reshape(1, 1, ql, ke - ks) if mask.dim() == 2 else mask[:, :, qs:qs + ql, ks:ke]
        outs.append(eager_attention(q[:, :, qs:qs + ql], k[:, :, ks:ke], v[:, :, ks:ke], scale, m, dtype))
    return torch.cat(outs, dim=2)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int = -1, dtype: str = "f32") -> torch.Tensor:
    """`eager_attention` with the local mask (src/archs/modernbert.rs:337-351, :1058-1076) for one unpadded sequence:
    q, k, v `[L, H, D]` -> `[L, H * D]`; keys with |i - j| > window get -10000 added (window < 0: no mask)."""
    r = (lambda t: round_bf16(t)) if dtype == "bf16" else (lambda t: t)
    L, H, D = q.shape
    scores = r(torch.einsum("ihd,jhd->hij", r(q.float() * D ** -0.5), k.float()))
    if window >= 0:
        idx = torch.arange(L)
        scores = scores + torch.where((idx.unsqueeze(0) - idx.unsqueeze(1)).abs() > window, MASK_VALUE, 0.0)
    probs = r(torch.softmax(scores, dim=-1))
    return r(torch.einsum("hij,jhd->ihd", probs, v.float())).reshape(L, H * D)
