"""Pieces of the decision model's batch path (`src/models/laya.rs`) on the token-packed layout.

`deduplicate` mirrors the free function of the same name (:689-707). `Scorer` mirrors `Laya::score_batched` +
`Laya::score` (:476-518): the hidden states of the marker tokens are selected, normalised (`scorer_norm`, a LayerNorm
with bias), passed through `scorer_in` + GELU(erf) and `scorer_out` (one logit per marker). On the packed layout a marker
of sequence s at position p is row `cu_seqlens[s] + p` (the reference indexes a padded `[batch, length]` block with
`row * length + position`, :489-494); selection and norm are one `s1_norm` call with a row index, the two Linears are
`s1_linear` with bias / activation. No CPU fallback.
"""
from __future__ import annotations

from typing import Hashable, List, Sequence, Tuple

import numpy as np
import torch

from . import norm as _norm
from .linear import Linear


def deduplicate(items: Sequence[Hashable]) -> Tuple[List[Hashable], List[int]]:
    """`deduplicate` (src/models/laya.rs:689-707): the distinct items in order of first appearance, and for every
    input item the index of its representative. An item's key is the item itself (the reference keys on question
    kind, token ids and marker positions: pass such a tuple)."""
    unique: List[Hashable] = []
    indices: List[int] = []
    seen = {}
    for item in items:
        index = seen.get(item)
        if index is None:
            index = len(unique)
            seen[item] = index
            unique.append(item)
        indices.append(index)
    return unique, indices


def marker_rows(cu_seqlens_host, markers: Sequence[Sequence[int]]) -> Tuple[np.ndarray, List[int]]:
    """Packed row of every marker (`cu_seqlens[s] + position`) and the marker count per sequence, the counterpart of
    `row * length + position` on the padded block (src/models/laya.rs:485-494). Positions outside their sequence raise."""
    cu = np.asarray(cu_seqlens_host, dtype=np.int64)
    if len(markers) != len(cu) - 1:
        raise ValueError("one marker list per sequence")
    rows: List[int] = []
    counts: List[int] = []
    for s, positions in enumerate(markers):
        length = int(cu[s + 1] - cu[s])
        for p in positions:
            if not 0 <= int(p) < length:
                raise ValueError(f"marker {p} outside sequence {s} of {length} tokens")
            rows.append(int(cu[s]) + int(p))
        counts.append(len(positions))
    return np.asarray(rows, dtype=np.int32), counts


class Scorer:
    """`scorer.0` (LayerNorm with bias), `scorer.1` (Linear + bias, GELU), `scorer.3` (Linear to one logit)
    (src/models/laya.rs:258-270, :508-518). `scorer_out` has one output feature; the library's projections want a
    multiple of 8, so its weight and bias are padded with zero rows once at load and column 0 is read back."""

    def __init__(self, norm_weight: torch.Tensor, norm_bias: torch.Tensor, scorer_in: Linear, scorer_out: Linear, eps: float = 1e-5):
        self.norm_weight, self.norm_bias, self.eps = norm_weight.contiguous(), norm_bias.contiguous(), float(eps)
        self.scorer_in = scorer_in
        w, b = scorer_out.weight, scorer_out.bias
        pad = (-w.shape[0]) % 8
        if pad:
            w = torch.cat([w, torch.zeros(pad, w.shape[1], dtype=w.dtype, device=w.device)])
            if b is not None:
                b = torch.cat([b, torch.zeros(pad, dtype=b.dtype, device=b.device)])
        self.scorer_out = Linear(w.contiguous(), None if b is None else b.contiguous())
        self.outputs = scorer_out.weight.shape[0]

    def score_packed(self, hidden: torch.Tensor, cu_seqlens_host, markers: Sequence[Sequence[int]]) -> List[List[float]]:
        """hidden bf16 `[T, hidden]` (CUDA, packed); returns the logits of every sequence's markers, like
        `score_batched` (one list per sequence, one value per marker)."""
        rows, counts = marker_rows(cu_seqlens_host, markers)
        if rows.size == 0:
            return [[] for _ in counts]
        index = torch.from_numpy(rows).to(hidden.device)
        selected = _norm.norm(hidden, self.norm_weight, self.eps, _norm.LAYER_NORM, gather=index, bias=self.norm_bias)
        h = self.scorer_in.forward(selected, act="gelu")
        logits = self.scorer_out.forward(h)[:, : self.outputs].float().cpu()
        if self.outputs != 1:
            raise ValueError("the scorer ends in one logit per marker")
        flat = logits[:, 0].tolist()
        out, at = [], 0
        for n in counts:
            out.append(flat[at:at + n])
            at += n
        return out


class HeadLayer:
    """`HeadLayer` (src/models/laya.rs:56-158), a pre-norm transformer layer with biased Linears and a ReLU feed-forward of
    4 x hidden, on the packed layout. Same member names: `qkv` (`self_attn.in_proj_weight / _bias`), `projection`
    (`self_attn.out_proj`), `norm1`, `norm2` (LayerNorm with bias, eps 1e-5), `linear1`, `linear2`; heads of 64.
        x = x + projection(attention(qkv(norm1(x))));   x = x + linear2(relu(linear1(norm2(x))))
    The reference masks padded keys with -inf (:411-424); a packed batch has none, so the attention is `s1_attention`
    over each sequence's own tokens. Bias, ReLU and both residual adds ride in the projections' epilogues."""

    def __init__(self, qkv: Linear, projection: Linear, norm1, norm2, linear1: Linear, linear2: Linear, eps: float = 1e-5):
        self.qkv, self.projection, self.linear1, self.linear2 = qkv, projection, linear1, linear2
        self.norm1, self.norm2, self.eps = norm1, norm2, float(eps)   # (weight, bias) pairs
        self.heads = qkv.weight.shape[1] // 64

    def forward(self, x: torch.Tensor, cu_seqlens_host) -> torch.Tensor:
        from .modernbert import attention_varlen
        T, hidden = x.shape
        n = _norm.norm(x, self.norm1[0], self.eps, _norm.LAYER_NORM, bias=self.norm1[1])
        qkv = self.qkv.forward(n).view(T, 3, self.heads, 64)
        attn = attention_varlen(qkv[:, 0], qkv[:, 1], qkv[:, 2], cu_seqlens_host, window=-1)
        x = self.projection.forward(attn, residual=x)
        n = _norm.norm(x, self.norm2[0], self.eps, _norm.LAYER_NORM, bias=self.norm2[1])
        return self.linear2.forward(self.linear1.forward(n, act="relu"), residual=x)


class DecisionHead:
    """What `Laya::forward` runs after the encoder (src/models/laya.rs:431-441) on a packed batch: the type embedding of
    each sequence's question kind added to all its tokens, the `HeadLayer`s, then the scorer at the marker rows."""

    def __init__(self, type_embedding: torch.Tensor, layers: Sequence[HeadLayer], scorer: Scorer):
        self.type_embedding, self.layers, self.scorer = type_embedding.contiguous(), list(layers), scorer

    def forward(self, hidden: torch.Tensor, cu_seqlens_host, kinds: Sequence[int], markers: Sequence[Sequence[int]]) -> List[List[float]]:
        """hidden bf16 `[T, hidden]` (the encoder's output, packed), `kinds[s]` the question kind of sequence s, `markers[s]`
        its marker positions. Returns one list of logits per sequence."""
        cu = np.asarray(cu_seqlens_host, dtype=np.int64)
        if len(kinds) != len(cu) - 1:
            raise ValueError("one question kind per sequence")
        per_token = np.repeat(np.asarray(kinds, dtype=np.int32), np.diff(cu))
        x = _norm.add_rows(hidden, self.type_embedding, torch.from_numpy(per_token).to(hidden.device))
        for layer in self.layers:
            x = layer.forward(x, cu_seqlens_host)
        return self.scorer.score_packed(x, cu_seqlens_host, markers)
