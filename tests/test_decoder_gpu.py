"""Qwen3.5 decoder on a packed batch through the C ABI against the CPU oracle: the causal grouped-query attention
kernel alone (`s1_attention_gqa`, head dim 256, fused output gate), and a small hybrid stack (linear-attention and
full-attention layers) layer by layer on identical inputs (max-relative 2e-2) and as a whole trajectory."""
import numpy as np
import pytest
import torch

import oracle
from conftest import max_rel
from sys1_b200 import batching, qwen35

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("lens,H,KV,gated", [([128], 1, 1, False), ([5], 2, 1, True), ([300, 1, 129, 64], 4, 2, True),
                                             ([1000], 8, 2, True), ([65, 640], 2, 2, False)])
def test_causal_gqa_attention_matches_the_oracle(ctx, lens, H, KV, gated):
    cu = np.cumsum([0] + lens).astype(np.int32)
    T = int(cu[-1])
    g = torch.Generator().manual_seed(17 * len(lens) + H)
    qg = torch.randn(T, H, 2, 256, generator=g).to(torch.bfloat16)   # query and gate interleaved per head, as q_proj emits
    qg[:, :, 0] *= 1.5
    k = torch.randn(T, KV, 256, generator=g).to(torch.bfloat16)
    v = torch.randn(T, KV, 256, generator=g).to(torch.bfloat16)
    d = qg.to(DEV)
    got = qwen35.attention_causal_gqa(d[:, :, 0], k.to(DEV), v.to(DEV), cu, gate=d[:, :, 1] if gated else None).float().cpu()
    ctx.sync()
    want = torch.empty(T, H * 256)
    for a, z in zip(cu[:-1], cu[1:]):
        if z > a:
            o = oracle.causal_attention(qg[a:z, :, 0], k[a:z], v[a:z], dtype="f32").reshape(z - a, H * 256)
            if gated:
                o = o * torch.sigmoid(qg[a:z, :, 1].float()).reshape(z - a, H * 256)
            want[a:z] = o
    assert torch.isfinite(got).all()
    assert max_rel(got, want) <= 2e-2


def test_causal_gqa_sequences_do_not_see_each_other(ctx):
    lens = [200, 333, 90]
    cu = np.cumsum([0] + lens).astype(np.int32)
    g = torch.Generator().manual_seed(9)
    q, k, v = (torch.randn(int(cu[-1]), h, 256, generator=g).to(torch.bfloat16).to(DEV) for h in (4, 2, 2))
    packed = qwen35.attention_causal_gqa(q, k, v, cu)
    a, z = int(cu[1]), int(cu[2])
    alone = qwen35.attention_causal_gqa(q[a:z], k[a:z], v[a:z], np.array([0, z - a], dtype=np.int32))
    assert torch.equal(packed[a:z], alone)


def _small_cfg():
    return oracle.DecoderConfig(vocab_size=500, hidden_size=256, intermediate_size=384, num_hidden_layers=4, num_attention_heads=2,
                                num_key_value_heads=1, head_dim=256, linear_num_key_heads=4, linear_num_value_heads=8)


def test_small_hybrid_stack(ctx):
    cfg = _small_cfg()
    w = oracle.qwen35.init_weights(cfg, 41)
    keep_f32 = ("A_log", "dt_bias")
    w = {k: (t if k.endswith(keep_f32) else t.to(torch.bfloat16).float()) for k, t in w.items()}
    lens = [200, 77, 1, 140]
    b, _ = batching.pack_next(lens, batching.BatcherConfig(token_budget=1 << 20))
    g = torch.Generator().manual_seed(42)
    ids = torch.randint(0, cfg.vocab_size, (b.total_tokens,), generator=g)
    dw = {k: (t.to(DEV) if k.endswith(keep_f32) else t.to(torch.bfloat16).to(DEV)) for k, t in w.items()}
    dec = qwen35.Decoder(dw, cfg)
    pos = torch.from_numpy(b.positions).to(DEV)
    y, states = dec.forward(ids.to(DEV), b.cu_seqlens, pos, collect=True)
    ctx.sync()
    out = {}
    for dtype in ("f32", "bf16"):
        want_y = torch.empty(b.total_tokens, cfg.hidden_size)
        want_states = [torch.empty(b.total_tokens, cfg.hidden_size) for _ in range(cfg.num_hidden_layers)]
        for a, z in zip(b.cu_seqlens[:-1], b.cu_seqlens[1:]):
            yy, ss = oracle.decoder_forward(ids[a:z], w, cfg, dtype=dtype, collect=True)
            want_y[a:z] = yy
            for dst, src in zip(want_states, ss):
                dst[a:z] = src
        out[dtype] = (want_y, want_states)
    # layer by layer on identical inputs: the bf16 restatement's stream before layer i feeds both sides
    x_in = w["embed_tokens"][ids]
    for i in range(cfg.num_hidden_layers):
        got = dec.layers[i].forward(x_in.to(torch.bfloat16).to(DEV), b.cu_seqlens, pos.to(torch.int32))
        want = torch.empty_like(x_in)
        for a, z in zip(b.cu_seqlens[:-1], b.cu_seqlens[1:]):
            want[a:z] = oracle.decoder_layer(i, x_in[a:z], w, cfg, dtype="f32")
        assert max_rel(got, want) <= 2e-2, f"layer {i} ({cfg.layer_type(i)}) on the oracle's input"
        x_in = out["bf16"][1][i]
    for i, got in enumerate(states):
        w32, w16 = out["f32"][1][i], out["bf16"][1][i]
        bound = max(2e-2, 1.5 * max_rel(w16, w32))
        assert max_rel(got, w16) <= bound and max_rel(got, w32) <= bound, f"trajectory, layer {i}"
    assert max_rel(y, out["f32"][0]) <= max(2e-2, 1.5 * max_rel(out["bf16"][0], out["f32"][0]))
    # last-token hidden state against a random probe matrix (the stand-in for decision logits): same ordering
    probe = torch.randn(4, cfg.hidden_size, generator=g) * 0.05
    for z in b.cu_seqlens[1:]:
        got = y[z - 1].float().cpu() @ probe.t()
        want = out["f32"][0][z - 1] @ probe.t()
        assert torch.equal(got.argsort(), want.argsort())


def test_causal_gqa_full_size_batch_properties(ctx):
    """The decoder benchmark's batch (T = 16384, 8 query / 2 KV heads, lengths 64-2048): packed versus alone bit-identical
    for a short and the longest sequence, and the first token of every sequence attends to itself only (output = v * gate)."""
    T, H, KV = 16384, 8, 2
    lens = batching.synthetic_lengths(1004, 64, 2048, T)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    g = torch.Generator(device=DEV).manual_seed(6)
    q = torch.randn(T, H, 256, device=DEV, generator=g).to(torch.bfloat16)
    k = torch.randn(T, KV, 256, device=DEV, generator=g).to(torch.bfloat16)
    v = torch.randn(T, KV, 256, device=DEV, generator=g).to(torch.bfloat16)
    packed = qwen35.attention_causal_gqa(q, k, v, cu)
    for s in (int(np.argmin(lens)), int(np.argmax(lens))):
        a, z = int(cu[s]), int(cu[s + 1])
        alone = qwen35.attention_causal_gqa(q[a:z], k[a:z], v[a:z], np.array([0, z - a], dtype=np.int32))
        assert torch.equal(packed[a:z], alone)
    ctx.sync()
    first = torch.from_numpy(cu[:-1].astype(np.int64)).to(DEV)
    want = v[first].repeat_interleave(H // KV, dim=1).reshape(len(first), H * 256)
    assert torch.equal(packed[first], want)
