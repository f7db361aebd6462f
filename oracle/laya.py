"""Oracle for the decision head of the Laya model (test infrastructure only; see the package docstring): the
type-embedding add, `HeadLayer::forward` and the scorer (src/models/laya.rs:125-157, :431-441, :508-518) for one
unpadded sequence. Biased Linears, LayerNorm with bias (eps 1e-5), heads of 64, softmax in f32, ReLU feed-forward.
Restated from the cited code; no reference test holds numbers for it (its snapshot tests need checkpoints)."""
from __future__ import annotations

from typing import Dict

import torch

from .norm import layer_norm
from .projection import linear, round_bf16


def head_layer(x: torch.Tensor, w: Dict[str, torch.Tensor], p: str, dtype: str = "f32") -> torch.Tensor:
    """`HeadLayer::forward` (src/models/laya.rs:125-157) on `x [L, hidden]`; weights under the checkpoint's names
    (`self_attn.in_proj_weight`, `self_attn.in_proj_bias`, `self_attn.out_proj.{weight,bias}`, `norm1/2.{weight,bias}`,
    `linear1/2.{weight,bias}`) with prefix `p`."""
    r = round_bf16 if dtype == "bf16" else (lambda t: t)
    L, hidden = x.shape
    H = hidden // 64
    n = layer_norm(x, w[p + "norm1.weight"], 1e-5, dtype, bias=w[p + "norm1.bias"])
    qkv = linear(n, w[p + "self_attn.in_proj_weight"], bias=w[p + "self_attn.in_proj_bias"], dtype=dtype).reshape(L, 3, H, 64)
    q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]
    scores = r(torch.einsum("ihd,jhd->hij", r(q * 64 ** -0.5), k))
    probs = r(torch.softmax(scores, dim=-1))
    attn = r(torch.einsum("hij,jhd->ihd", probs, v)).reshape(L, hidden)
    x = linear(attn, w[p + "self_attn.out_proj.weight"], bias=w[p + "self_attn.out_proj.bias"], residual=x, dtype=dtype)
    n = layer_norm(x, w[p + "norm2.weight"], 1e-5, dtype, bias=w[p + "norm2.bias"])
    h = linear(n, w[p + "linear1.weight"], bias=w[p + "linear1.bias"], act="relu", dtype=dtype)
    return linear(h, w[p + "linear2.weight"], bias=w[p + "linear2.bias"], residual=x, dtype=dtype)


def init_head_weights(hidden: int, seed: int, layers: int = 2) -> Dict[str, torch.Tensor]:
    """Random weights of the decision head under the checkpoint's names (src/models/laya.rs:76-88, :224-270): `type_emb`
    `[3, hidden]`, `head.layers.i.*`, `scorer.0` (LayerNorm), `scorer.1` (hidden -> hidden), `scorer.3` (hidden -> 1)."""
    g = torch.Generator().manual_seed(seed)
    mk = lambda *shape, s=0.02: torch.randn(*shape, generator=g) * s
    w = {"type_emb.weight": mk(3, hidden, s=0.5)}
    for i in range(layers):
        p = f"head.layers.{i}."
        w[p + "self_attn.in_proj_weight"], w[p + "self_attn.in_proj_bias"] = mk(3 * hidden, hidden, s=0.04), mk(3 * hidden, s=0.1)
        w[p + "self_attn.out_proj.weight"], w[p + "self_attn.out_proj.bias"] = mk(hidden, hidden), mk(hidden, s=0.1)
        w[p + "linear1.weight"], w[p + "linear1.bias"] = mk(4 * hidden, hidden), mk(4 * hidden, s=0.1)
        w[p + "linear2.weight"], w[p + "linear2.bias"] = mk(hidden, 4 * hidden), mk(hidden, s=0.1)
        for n in ("norm1", "norm2"):
            w[p + n + ".weight"], w[p + n + ".bias"] = 1.0 + mk(hidden, s=0.1), mk(hidden, s=0.1)
    w["scorer.0.weight"], w["scorer.0.bias"] = 1.0 + mk(hidden, s=0.1), mk(hidden, s=0.1)
    w["scorer.1.weight"], w["scorer.1.bias"] = mk(hidden, hidden, s=0.05), mk(hidden, s=0.1)
    w["scorer.3.weight"], w["scorer.3.bias"] = mk(1, hidden, s=0.05), mk(1, s=0.1)
    return w


def decision_head(hidden: torch.Tensor, kind: int, markers, w: Dict[str, torch.Tensor], layers: int = 2, dtype: str = "f32") -> torch.Tensor:
    """Type embedding + head layers + scorer at the marker rows of one sequence -> one logit per marker."""
    r = round_bf16 if dtype == "bf16" else (lambda t: t)
    x = r(hidden + w["type_emb.weight"][kind])
    for i in range(layers):
        x = head_layer(x, w, f"head.layers.{i}.", dtype)
    sel = x[torch.as_tensor(list(markers), dtype=torch.long)]
    n = layer_norm(sel, w["scorer.0.weight"], 1e-5, dtype, bias=w["scorer.0.bias"])
    h = linear(n, w["scorer.1.weight"], bias=w["scorer.1.bias"], act="gelu", dtype=dtype)
    return linear(h, w["scorer.3.weight"], bias=w["scorer.3.bias"], dtype=dtype)[:, 0]
