"""Parity with the CPU oracle at the shapes the benchmark configurations name, not at toy sizes:

  * ModernBERT-base on its configured input - ids uniform over the 50368-token vocabulary, 8 sequences of 512, seed
    1001 - all 22 layers, every layer within max-relative 2e-2 of the f32 oracle on the oracle's own input, and the
    decision of a mean-pool linear head (argmax and ordering) identical;
  * ModernBERT-large shape (hidden 1024, 16 heads, GeGLU 2 x 2624: MLP-out K = 2624 = 41 x 64, Wi N = 5248): global and
    local layers on a packed batch with sequences longer than the 129-token band, and the two odd-sized projections alone;
  * Qwen3.5-small real shape (hidden 1024, 16 + 16 delta-rule heads of 128, 8 query / 2 KV heads of 256, SwiGLU 3584,
    rotary 64): one (linear, linear, linear, full) group on about 2048 packed tokens;
  * the per-rank shard of the 27B-shaped model under 8-way tensor parallelism, on one GPU: 6 value / 2 key delta-rule
    heads (repeat 3), 3 query / 1 KV heads, gate / up 5120 -> 2 x 2176, down 2176 -> 5120 read through the row stride of the
    unsharded matrix (17408). A shard computes a layer of a narrower model, which is what the oracle is given.
Tolerance everywhere: max-relative 2e-2 (the bf16 acceptance bound) against the f32 oracle fed the same input."""
import numpy as np
import pytest
import torch

import oracle
from conftest import max_rel
from sys1_b200 import batching, linear, modernbert, qwen35
from sys1_b200._lib import EPI_GEGLU
from test_encoder_gpu import _check_layers, _run

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_modernbert_base_on_its_configured_input(ctx):
    cfg = oracle.EncoderConfig()  # 22 layers, 768, 12 x 64, GeGLU 2 x 1152, window 128, global every 3rd, vocab 50368
    ids = torch.randint(0, 50368, (8, 512), generator=torch.Generator().manual_seed(1001)).reshape(-1)
    y, states, out, b, isolated = _run(cfg, [512] * 8, 1001, ids=ids)
    _check_layers(states, out, isolated)
    print("base 8x512 isolated per-layer max-rel:", " ".join(f"{e:.2e}" for e in isolated))
    want_y = out["f32"][0]
    head = torch.randn(4, cfg.hidden_size, generator=torch.Generator().manual_seed(5)) * 0.02
    for a, z in zip(b.cu_seqlens[:-1], b.cu_seqlens[1:]):
        got = y[a:z].float().cpu().mean(0) @ head.t()
        want = want_y[a:z].mean(0) @ head.t()
        assert int(got.argmax()) == int(want.argmax())
        assert torch.equal(got.argsort(), want.argsort())


def test_modernbert_large_shape_layers(ctx):
    cfg = oracle.EncoderConfig(vocab_size=2000, hidden_size=1024, num_hidden_layers=4, num_attention_heads=16, intermediate_size=2624)
    y, states, out, _, isolated = _run(cfg, [300, 17, 131, 1, 260], 1003)  # layers 0, 3 global; 1, 2 local; three sequences beyond the band
    _check_layers(states, out, isolated)
    print("large-shape isolated per-layer max-rel:", " ".join(f"{e:.2e}" for e in isolated))
    assert max_rel(y, out["f32"][0]) <= 2e-2


@pytest.mark.parametrize("T", [300, 4200])
def test_large_shape_odd_projections_alone(ctx, T):
    """MLP-out K = 2624 (41 K-steps of 64, the last stage of the ring half used) with the residual, in place and not;
    Wi N = 5248 with GeGLU (41 column pairs of 64: the last 256-wide tile is half empty)."""
    g = torch.Generator().manual_seed(2624 + T)
    x = torch.randn(T, 1024, generator=g).to(torch.bfloat16)
    h = torch.randn(T, 2624, generator=g).to(torch.bfloat16)
    res = torch.randn(T, 1024, generator=g).to(torch.bfloat16)
    wi = (torch.randn(5248, 1024, generator=g) * 0.02).to(torch.bfloat16)
    wout = (torch.randn(1024, 2624, generator=g) * 0.02).to(torch.bfloat16)
    got = linear.fused_linear(h.to(DEV), wout.to(DEV), residual=res.to(DEV))
    stream = res.to(DEV).clone()
    linear.fused_linear(h.to(DEV), wout.to(DEV), residual=stream, out=stream)
    gated = linear.fused_linear(x.to(DEV), wi.to(DEV), epilogue=EPI_GEGLU)
    ctx.sync()
    want = oracle.linear(h, wout, residual=res, dtype="f32")
    assert max_rel(got, want) <= 2e-2 and max_rel(stream, want) <= 2e-2
    want16 = oracle.linear(h, wout, residual=res, dtype="bf16")
    assert ((got.float().cpu() - want16).abs() > 0).float().mean() < 0.05  # at most a bf16 step on a few elements
    assert gated.shape == (T, 2624)
    assert max_rel(gated, oracle.geglu(oracle.linear(x, wi, dtype="f32"), dtype="f32")) <= 2e-2


def _decoder_layers_on_oracle_inputs(cfg, w, lens, seed, down_ld=None):
    """Every layer of the stack, each on the bf16 oracle's residual stream before it, against the f32 oracle's layer."""
    keep_f32 = ("A_log", "dt_bias")
    w = {k: (t if k.endswith(keep_f32) else t.to(torch.bfloat16).float()) for k, t in w.items()}
    b, _ = batching.pack_next(lens, batching.BatcherConfig(token_budget=1 << 20))
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, cfg.vocab_size, (b.total_tokens,), generator=g)
    dw = {k: (t.to(DEV) if k.endswith(keep_f32) else t.to(torch.bfloat16).to(DEV)) for k, t in w.items()}
    if down_ld is not None:
        # the row-parallel shard as a tensor-parallel rank sees it: a K range of the unsharded matrix, row stride down_ld
        for name in [n for n in dw if n.endswith("mlp.down_proj")]:
            full = torch.zeros(dw[name].shape[0], down_ld, dtype=torch.bfloat16, device=DEV)
            lo = 3 * dw[name].shape[1]
            full[:, lo:lo + dw[name].shape[1]] = dw[name]
            dw[name] = full[:, lo:lo + dw[name].shape[1]]
            assert dw[name].stride(0) == down_ld
    dec = qwen35.Decoder(dw, cfg)
    pos = torch.from_numpy(b.positions).to(DEV)
    x_in = w["embed_tokens"][ids]
    errs = []
    for i in range(cfg.num_hidden_layers):
        got = dec.layers[i].forward(x_in.to(torch.bfloat16).to(DEV), b.cu_seqlens, pos)
        want32, want16 = torch.empty_like(x_in), torch.empty_like(x_in)
        for a, z in zip(b.cu_seqlens[:-1], b.cu_seqlens[1:]):
            want32[a:z] = oracle.decoder_layer(i, x_in[a:z], w, cfg, dtype="f32")
            want16[a:z] = oracle.decoder_layer(i, x_in[a:z], w, cfg, dtype="bf16")
        errs.append(max_rel(got, want32))
        x_in = want16
    return errs


def test_qwen35_small_real_shape_layer_group(ctx):
    cfg = oracle.DecoderConfig(vocab_size=2000, num_hidden_layers=4)  # hidden 1024, Hk = Hv = 16, 8 q / 2 kv x 256, I 3584, rotary 64
    assert (cfg.hidden_size, cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.num_attention_heads, cfg.num_key_value_heads,
            cfg.intermediate_size, cfg.rotary_dim) == (1024, 16, 16, 8, 2, 3584, 64)
    errs = _decoder_layers_on_oracle_inputs(cfg, oracle.qwen35.init_weights(cfg, 1004), [700, 64, 1100, 190], 1004)
    print("qwen3.5-small real-shape per-layer max-rel:", " ".join(f"{e:.2e}" for e in errs))
    for i, e in enumerate(errs):
        assert e <= 2e-2, f"layer {i} ({cfg.layer_type(i)}): {e:.3e}"


def test_27b_tensor_parallel_rank_shard_shapes(ctx):
    cfg = oracle.DecoderConfig(vocab_size=1000, hidden_size=5120, intermediate_size=2176, num_hidden_layers=4, num_attention_heads=3,
                               num_key_value_heads=1, head_dim=256, linear_num_key_heads=2, linear_num_value_heads=6)
    errs = _decoder_layers_on_oracle_inputs(cfg, oracle.qwen35.init_weights(cfg, 1005), [600, 300, 124], 1005, down_ld=17408)
    print("27B TP-8 shard per-layer max-rel:", " ".join(f"{e:.2e}" for e in errs))
    for i, e in enumerate(errs):
        assert e <= 2e-2, f"layer {i} ({cfg.layer_type(i)}): {e:.3e}"
