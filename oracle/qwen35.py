"""Oracle for the Qwen3.5 text decoder forward (test infrastructure only; see the package docstring).

Restates `Decoder::forward_embeds` / `Layer::forward` / `FullAttention::forward` / `LinearAttention::forward` of
src/archs/qwen35_text.rs (:982-1005, :932-940, :312-411, :491-629) for one unpadded sequence:
  x = embed[ids]; per layer: x = x + mixer(RMS(x)); x = x + MLP(RMS(x)); finally RMS(x),
  RMS(x) = x / sqrt(mean(x^2) + eps) * (1 + w) in f32 (:183-203).
Full attention (:312-411): qg = x Wq^T -> [L, H, 2, D] (query and output gate interleaved per head);
  q = rope(RMS_D(qg[:, :, 0])), gate = sigmoid(qg[:, :, 1]), k = rope(RMS_D(x Wk^T)), v = x Wv^T, KV heads repeated
  H / KV times (kv head h serves query heads h r .. h r + r - 1, :363-369); causal softmax in f32 of q k^T * D^-1/2;
  out = (attn * gate) Wo^T. RoPE rotates the first rotary_dim = D * partial_rotary_factor columns (rotate-half inside
  that span), phase_j = pos / theta^(2 j / rotary_dim), tables cast to the model dtype (:101-165, :296-310).
Linear attention: the composition of the delta-rule stages in oracle/delta_rule.py.

Pinned by `tests/test_oracle.py` against the `transformers` Qwen3.5 text model (an independent implementation of
the same architecture) on random-init weights in f32.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Tuple

import torch

from .delta_rule import causal_conv_silu, delta_inputs, finish_delta, sequential_delta_rule
from .norm import rms_norm, rope
from .projection import linear, round_bf16, swiglu


@dataclass(frozen=True)
class DecoderConfig:
    """Defaults: the Qwen3.5-small shape of the benchmark configuration."""
    vocab_size: int = 151936
    hidden_size: int = 1024
    intermediate_size: int = 3584
    num_hidden_layers: int = 24
    num_attention_heads: int = 8
    num_key_value_heads: int = 2
    head_dim: int = 256
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e7
    partial_rotary_factor: float = 0.25
    linear_num_key_heads: int = 16
    linear_num_value_heads: int = 16
    linear_key_head_dim: int = 128
    linear_value_head_dim: int = 128
    linear_conv_kernel_dim: int = 4
    full_attention_interval: int = 4  # layer i is full attention iff (i + 1) % interval == 0

    @property
    def rotary_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor)

    def layer_type(self, i: int) -> str:
        return "full_attention" if (i + 1) % self.full_attention_interval == 0 else "linear_attention"


def init_weights(cfg: DecoderConfig, seed: int) -> Dict[str, torch.Tensor]:
    """Random-init weights under the checkpoint's tensor names (f32; N(0, 0.02) matrices, small norm weights)."""
    g = torch.Generator().manual_seed(seed)
    mk = lambda *shape, s=0.02: torch.randn(*shape, generator=g) * s
    H, KV, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    Hk, Hv, Dk, Dv = cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
    w = {"embed_tokens": mk(cfg.vocab_size, cfg.hidden_size, s=1.0), "norm": mk(cfg.hidden_size, s=0.1)}
    for i in range(cfg.num_hidden_layers):
        p = f"layers.{i}."
        w[p + "input_layernorm"] = mk(cfg.hidden_size, s=0.1)
        w[p + "post_attention_layernorm"] = mk(cfg.hidden_size, s=0.1)
        w[p + "mlp.gate_proj"] = mk(cfg.intermediate_size, cfg.hidden_size)
        w[p + "mlp.up_proj"] = mk(cfg.intermediate_size, cfg.hidden_size)
        w[p + "mlp.down_proj"] = mk(cfg.hidden_size, cfg.intermediate_size)
        if cfg.layer_type(i) == "full_attention":
            w[p + "self_attn.q_proj"] = mk(H * D * 2, cfg.hidden_size)
            w[p + "self_attn.k_proj"] = mk(KV * D, cfg.hidden_size)
            w[p + "self_attn.v_proj"] = mk(KV * D, cfg.hidden_size)
            w[p + "self_attn.o_proj"] = mk(cfg.hidden_size, H * D)
            w[p + "self_attn.q_norm"] = mk(D, s=0.1)
            w[p + "self_attn.k_norm"] = mk(D, s=0.1)
        else:
            width = 2 * Hk * Dk + Hv * Dv
            w[p + "linear_attn.in_proj_qkv"] = mk(width, cfg.hidden_size)
            w[p + "linear_attn.in_proj_z"] = mk(Hv * Dv, cfg.hidden_size)
            w[p + "linear_attn.in_proj_b"] = mk(Hv, cfg.hidden_size, s=0.1)
            w[p + "linear_attn.in_proj_a"] = mk(Hv, cfg.hidden_size, s=0.1)
            w[p + "linear_attn.conv1d"] = mk(width, 1, cfg.linear_conv_kernel_dim, s=0.3)
            w[p + "linear_attn.A_log"] = mk(Hv, s=0.5)
            w[p + "linear_attn.dt_bias"] = mk(Hv, s=0.5)
            w[p + "linear_attn.norm"] = 1.0 + mk(Dv, s=0.1)
            w[p + "linear_attn.out_proj"] = mk(cfg.hidden_size, Hv * Dv)
    return w


def rope_tables(cfg: DecoderConfig, length: int, dtype: str = "f32") -> Tuple[torch.Tensor, torch.Tensor]:
    """cos, sin `[L, rotary_dim / 2]`: phase = position / theta^(2 j / rotary_dim) (src/archs/qwen35_text.rs:119-163);
    cast to the model dtype like the reference's tables."""
    rd = cfg.rotary_dim
    div = torch.tensor([float(cfg.rope_theta) ** (2.0 * j / rd) for j in range(rd // 2)], dtype=torch.float64).to(torch.float32)
    phase = torch.arange(length, dtype=torch.float32).unsqueeze(1) / div.unsqueeze(0)
    cos, sin = phase.cos(), phase.sin()
    return (round_bf16(cos), round_bf16(sin)) if dtype == "bf16" else (cos, sin)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, dtype: str = "f32") -> torch.Tensor:
    """Eager causal GQA attention (src/archs/qwen35_text.rs:361-398): q `[L, H, D]`, k, v `[L, KV, D]` -> `[L, H, D]`.
    Scores (q k^T) * scale in the model dtype, softmax in f32, probabilities cast back before they multiply v."""
    r = round_bf16 if dtype == "bf16" else (lambda t: t)
    L, H, D = q.shape
    rep = H // k.shape[1]
    kk = k.float().repeat_interleave(rep, dim=1)
    vv = v.float().repeat_interleave(rep, dim=1)
    scores = r(r(torch.einsum("ihd,jhd->hij", q.float(), kk)) * D ** -0.5)
    idx = torch.arange(L)
    scores = scores.masked_fill(idx.unsqueeze(0) > idx.unsqueeze(1), float("-inf"))
    probs = r(torch.softmax(scores, dim=-1))
    return r(torch.einsum("hij,jhd->ihd", probs, vv))


def full_attention(x: torch.Tensor, w: Dict[str, torch.Tensor], p: str, cfg: DecoderConfig, dtype: str = "f32") -> torch.Tensor:
    r = round_bf16 if dtype == "bf16" else (lambda t: t)
    L = x.shape[0]
    H, KV, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    cos, sin = rope_tables(cfg, L, dtype)
    qg = linear(x, w[p + "q_proj"], dtype=dtype).reshape(L, H, 2, D)
    q = r(rope(rms_norm(qg[:, :, 0], w[p + "q_norm"], cfg.rms_norm_eps, dtype), cos, sin, cfg.rotary_dim, bf16_ops=dtype == "bf16"))
    gate = r(torch.sigmoid(qg[:, :, 1])).reshape(L, H * D)
    k = r(rope(rms_norm(linear(x, w[p + "k_proj"], dtype=dtype).reshape(L, KV, D), w[p + "k_norm"], cfg.rms_norm_eps, dtype),
               cos, sin, cfg.rotary_dim, bf16_ops=dtype == "bf16"))
    v = linear(x, w[p + "v_proj"], dtype=dtype).reshape(L, KV, D)
    attn = causal_attention(q, k, v, dtype).reshape(L, H * D)
    return linear(r(attn * gate), w[p + "o_proj"], dtype=dtype)


def linear_attention(x: torch.Tensor, w: Dict[str, torch.Tensor], p: str, cfg: DecoderConfig, dtype: str = "f32") -> torch.Tensor:
    Hk, Hv, Dk, Dv = cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
    mixed = causal_conv_silu(linear(x, w[p + "in_proj_qkv"], dtype=dtype).unsqueeze(0), w[p + "conv1d"], dtype=dtype)
    q, k, v, g, beta = delta_inputs(mixed, linear(x, w[p + "in_proj_b"], dtype=dtype).unsqueeze(0),
                                    linear(x, w[p + "in_proj_a"], dtype=dtype).unsqueeze(0), w[p + "dt_bias"],
                                    -torch.exp(w[p + "A_log"].float()), Hk, Hv, Dk, Dv)
    o = sequential_delta_rule(q, k, v, g, beta)
    y = finish_delta(o, linear(x, w[p + "in_proj_z"], dtype=dtype).unsqueeze(0), w[p + "norm"], cfg.rms_norm_eps,
                     out_bf16=dtype == "bf16")[0]
    return linear(y, w[p + "out_proj"], dtype=dtype)


def decoder_layer(i: int, x: torch.Tensor, w: Dict[str, torch.Tensor], cfg: DecoderConfig, dtype: str = "f32") -> torch.Tensor:
    """`Layer::forward` (src/archs/qwen35_text.rs:932-940)."""
    r = round_bf16 if dtype == "bf16" else (lambda t: t)
    p = f"layers.{i}."
    n = rms_norm(x, w[p + "input_layernorm"], cfg.rms_norm_eps, dtype)
    if cfg.layer_type(i) == "full_attention":
        mixed = full_attention(n, w, p + "self_attn.", cfg, dtype)
    else:
        mixed = linear_attention(n, w, p + "linear_attn.", cfg, dtype)
    x = r(x + mixed)
    n = rms_norm(x, w[p + "post_attention_layernorm"], cfg.rms_norm_eps, dtype)
    h = swiglu(linear(n, w[p + "mlp.gate_proj"], dtype=dtype), linear(n, w[p + "mlp.up_proj"], dtype=dtype), dtype)
    return linear(h, w[p + "mlp.down_proj"], residual=x, dtype=dtype)


def decoder_forward(ids: torch.Tensor, w: Dict[str, torch.Tensor], cfg: DecoderConfig, dtype: str = "f32", collect: bool = False):
    """One unpadded sequence `ids [L]` -> final hidden `[L, hidden]`; with `collect`, also the stream after every layer."""
    r = round_bf16 if dtype == "bf16" else (lambda t: t)
    x = r(w["embed_tokens"][ids].to(torch.float32))
    states: List[torch.Tensor] = []
    for i in range(cfg.num_hidden_layers):
        x = decoder_layer(i, x, w, cfg, dtype)
        if collect:
            states.append(x)
    y = rms_norm(x, w["norm"], cfg.rms_norm_eps, dtype)
    return (y, states) if collect else y
