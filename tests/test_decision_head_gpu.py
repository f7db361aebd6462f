"""The decision head of the Laya model on the packed layout (`sys1_b200.laya.DecisionHead`): type-embedding add
(`s1_add_rows`), two `HeadLayer`s (biased Linears, LayerNorm with bias, bidirectional attention, ReLU feed-forward:
src/models/laya.rs:56-158) and the scorer at the marker rows, against the CPU oracle's restatement, sequence by sequence."""
import numpy as np
import pytest
import torch

import oracle
from conftest import max_rel
from sys1_b200 import batching, laya, norm
from sys1_b200.linear import Linear

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _head(w, layers=2):
    d = {k: v.to(torch.bfloat16).to(DEV) for k, v in w.items()}
    hl = []
    for i in range(layers):
        p = f"head.layers.{i}."
        hl.append(laya.HeadLayer(Linear(d[p + "self_attn.in_proj_weight"], d[p + "self_attn.in_proj_bias"]),
                                 Linear(d[p + "self_attn.out_proj.weight"], d[p + "self_attn.out_proj.bias"]),
                                 (d[p + "norm1.weight"], d[p + "norm1.bias"]), (d[p + "norm2.weight"], d[p + "norm2.bias"]),
                                 Linear(d[p + "linear1.weight"], d[p + "linear1.bias"]), Linear(d[p + "linear2.weight"], d[p + "linear2.bias"])))
    scorer = laya.Scorer(d["scorer.0.weight"], d["scorer.0.bias"], Linear(d["scorer.1.weight"], d["scorer.1.bias"]),
                         Linear(d["scorer.3.weight"], d["scorer.3.bias"]))
    return laya.DecisionHead(d["type_emb.weight"], hl, scorer), hl


@pytest.mark.parametrize("hidden,lens", [(256, [150, 40, 1, 300]), (768, [64, 200])])
def test_decision_head_matches_the_oracle(ctx, hidden, lens):
    w = {k: v.to(torch.bfloat16).float() for k, v in oracle.laya.init_head_weights(hidden, 11).items()}
    head, layers = _head(w)
    b, _ = batching.pack_next(lens, batching.BatcherConfig(token_budget=1 << 20))
    g = torch.Generator().manual_seed(12)
    x = torch.randn(b.total_tokens, hidden, generator=g).to(torch.bfloat16)
    kinds = [int(k) for k in torch.randint(0, 3, (len(lens),), generator=g)]
    markers = [sorted(set(int(p) for p in torch.randint(0, n, (min(n, 3),), generator=g))) for n in lens]
    # one head layer on its own, on identical input
    got_layer = layers[0].forward(x.to(DEV), b.cu_seqlens)
    want_layer = torch.cat([oracle.laya.head_layer(x[a:z].float(), w, "head.layers.0.", "f32") for a, z in zip(b.cu_seqlens[:-1], b.cu_seqlens[1:])])
    assert max_rel(got_layer, want_layer) <= 2e-2
    got = head.forward(x.to(DEV), b.cu_seqlens, kinds, markers)
    ctx.sync()
    for s, (a, z) in enumerate(zip(b.cu_seqlens[:-1], b.cu_seqlens[1:])):
        want = oracle.laya.decision_head(x[a:z].float(), kinds[s], markers[s], w, dtype="f32")
        assert len(got[s]) == len(markers[s])
        assert float((torch.tensor(got[s]) - want).abs().max()) <= 2e-2 * max(1.0, float(want.abs().max()))
        if len(markers[s]) > 1 and float((want.sort().values.diff()).abs().min()) > 0.05:
            assert torch.equal(torch.tensor(got[s]).argsort(), want.argsort())  # the decision: same ordering of the options


def test_add_rows_is_the_type_embedding_add(ctx):
    g = torch.Generator().manual_seed(2)
    x = torch.randn(100, 264, generator=g).to(torch.bfloat16)
    table = torch.randn(3, 264, generator=g).to(torch.bfloat16)
    idx = torch.randint(0, 3, (100,), generator=g).to(torch.int32)
    y = norm.add_rows(x.to(DEV)[:, :256], table.to(DEV)[:, :256], idx.to(DEV))     # strided views
    want = oracle.round_bf16(x[:, :256].float() + table[idx.long(), :256].float())
    assert torch.equal(y.float().cpu(), want)
    bad = idx.clone()
    bad[7] = 3
    norm.add_rows(x.to(DEV)[:, :256], table.to(DEV)[:, :256], bad.to(DEV))
    with pytest.raises(Exception, match="outside the table"):
        ctx.sync()
    ctx.sync()
