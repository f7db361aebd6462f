"""Pins the CPU oracle: the reference's self-contained known-answer tests, replayed, plus the committed
golden fixtures (which freeze the oracle's own outputs)."""
import math

import numpy as np
import pytest
import torch

import oracle
from golden_io import load_delta_rule, load_projections


def _closed_form(count, width, factor):
    # `((index * 13 % 29) as f32 - 14.) * factor` (src/archs/qwen35_text.rs:1398-1402, 1327-1331)
    return torch.tensor([((i * 13 % 29) - 14.0) * factor for i in range(count * width)], dtype=torch.float32)


def test_delta_rule_matches_scalar_recurrence_across_chunk_boundary():
    """src/archs/qwen35_text.rs:1391-1439: L70, Dk4, Dv3, g=-0.1, beta=0.45, tolerance 1e-4; the expected values
    come from the same scalar loop the reference test runs."""
    L, Dk, Dv = 70, 4, 3
    q = _closed_form(L, Dk, 0.01).reshape(1, 1, L, Dk)
    k = _closed_form(L, Dk, 0.012).reshape(1, 1, L, Dk)
    v = _closed_form(L, Dv, 0.02).reshape(1, 1, L, Dv)
    g = torch.full((1, 1, L), -0.1)
    beta = torch.full((1, 1, L), 0.45)
    # in-test scalar loop, written out as in the reference test
    state = [[0.0] * Dv for _ in range(Dk)]
    expected = torch.zeros(L, Dv)
    qf, kf, vf = q.flatten().tolist(), k.flatten().tolist(), v.flatten().tolist()
    for step in range(L):
        decay = math.exp(-0.1)
        for row in range(Dk):
            for col in range(Dv):
                state[row][col] *= decay
        for col in range(Dv):
            remembered = sum(kf[step * Dk + row] * state[row][col] for row in range(Dk))
            delta = (vf[step * Dv + col] - remembered) * 0.45
            for row in range(Dk):
                state[row][col] += kf[step * Dk + row] * delta
            expected[step, col] = sum(qf[step * Dk + row] * state[row][col] for row in range(Dk))
    for fn in (oracle.chunked_delta_rule, oracle.sequential_delta_rule,
               lambda *a: oracle.sequential_delta_rule(*a, use_c=False)):
        out = fn(q, k, v, g, beta)[0, :, 0, :]
        assert (out - expected).abs().max() < 1e-4


def test_delta_rule_kernel_shape_chunked_equals_sequential():
    """Inputs of src/archs/qwen35_text.rs:1320-1389 (B2, H2, L290, Dk128, Dv16, g=-0.002, beta=0.5): the
    reference compares its CUDA kernel with the chunked form at 1e-4; here the two oracle forms must agree."""
    B, H, L, Dk, Dv = 2, 2, 290, 128, 16
    q = _closed_form(B * H * L, Dk, 0.001).reshape(B, H, L, Dk)
    k = _closed_form(B * H * L, Dk, 0.006).reshape(B, H, L, Dk)
    v = _closed_form(B * H * L, Dv, 0.008).reshape(B, H, L, Dv)
    g = torch.full((B, H, L), -0.002)
    beta = torch.full((B, H, L), 0.5)
    a = oracle.chunked_delta_rule(q, k, v, g, beta)
    b = oracle.sequential_delta_rule(q, k, v, g, beta)
    assert a.shape == (B, L, H, Dv)
    assert (a - b).abs().max() < 1e-4


def test_delta_rule_stays_finite_with_large_negative_gates():
    """src/archs/qwen35_text.rs:1441-1462: ones, g=-8, L=64."""
    q = torch.ones(1, 1, 64, 4)
    v = torch.ones(1, 1, 64, 3)
    g = torch.full((1, 1, 64), -8.0)
    beta = torch.full((1, 1, 64), 0.5)
    for fn in (oracle.chunked_delta_rule, oracle.sequential_delta_rule):
        assert torch.isfinite(fn(q, q, v, g, beta)).all()


def test_geglu_sixteen_values():
    """src/archs/modernbert.rs:743-766: 2x8 input, first half activated with exact-erf GELU, second half
    multiplies; tolerance 1e-5 for f32, 0.04 for bf16. Expected values from the closed form in float64."""
    values = [-4.0, -1.5, -0.25, 0.0, 0.5, 1.25, 3.0, 5.0, 2.0, -0.75, 0.125, -3.5, 1.0, 0.5, -2.0, 4.5]
    x = torch.tensor(values).reshape(2, 8)
    expected = torch.tensor([[0.5 * a * (1 + math.erf(a / math.sqrt(2))) * b
                              for a, b in zip(row[:4], row[4:])] for row in x.tolist()])
    assert (oracle.geglu(x, dtype="f32") - expected).abs().max() <= 1e-5
    assert (oracle.geglu(x, dtype="bf16") - expected).abs().max() <= 0.04


def test_linear_definition_small_integers():
    """`Linear::forward(x) = x W^T + b` on integers small enough to be exact in every precision."""
    x = torch.tensor([[1., 2., 3.], [0., -1., 4.]])
    w = torch.tensor([[1., 0., -1.], [2., 2., 2.]])
    b = torch.tensor([10., -10.])
    want = torch.tensor([[8., 2.], [6., -4.]])
    for dt in ("f32", "bf16"):
        assert torch.equal(oracle.linear(x, w, b, dtype=dt), want)
        assert torch.equal(oracle.linear(x, w, b, act="relu", residual=torch.ones(2, 2), dtype=dt),
                           torch.relu(want) + 1)


def test_swiglu_and_mlp_shapes():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(5, 8, generator=g)
    wg, wu, wd = torch.randn(6, 8, generator=g), torch.randn(6, 8, generator=g), torch.randn(8, 6, generator=g)
    y = oracle.mlp_qwen35(x, wg, wu, wd, residual=x, dtype="f32")
    ref = x + (torch.nn.functional.silu(x @ wg.t()) * (x @ wu.t())) @ wd.t()
    assert torch.allclose(y, ref, atol=1e-5)
    wi = torch.randn(12, 8, generator=g)
    y = oracle.mlp_modernbert(x, wi, wd, residual=x, dtype="f32")
    p = x @ wi.t()
    ref = x + (torch.nn.functional.gelu(p[:, :6]) * p[:, 6:]) @ wd.t()
    assert torch.allclose(y, ref, atol=1e-5)


def test_delta_inputs_and_finish_follow_the_reference_conventions():
    """q/k heads repeat as [Hk, repeat] (key head h_k serves value heads h_k*r .. h_k*r+r-1,
    src/archs/qwen35_text.rs:552-559); the output norm multiplies by `weight`, not 1+weight (:622)."""
    g = torch.Generator().manual_seed(1)
    B, L, Hk, Hv, Dk, Dv = 1, 3, 2, 4, 8, 4
    mixed = torch.randn(B, L, 2 * Hk * Dk + Hv * Dv, generator=g)
    b, a = torch.randn(B, L, Hv, generator=g), torch.randn(B, L, Hv, generator=g)
    dt_bias, neg_a = torch.randn(Hv, generator=g), -torch.rand(Hv, generator=g)
    q, k, v, gate, beta = oracle.delta_inputs(mixed, b, a, dt_bias, neg_a, Hk, Hv, Dk, Dv)
    assert q.shape == (B, Hv, L, Dk) and v.shape == (B, Hv, L, Dv) and gate.shape == (B, Hv, L)
    assert torch.equal(q[:, 0], q[:, 1]) and torch.equal(k[:, 2], k[:, 3]) and not torch.equal(q[:, 1], q[:, 2])
    assert torch.allclose(k.square().sum(-1), torch.ones(B, Hv, L), atol=1e-4)
    assert (gate <= 0).all() and ((beta > 0) & (beta < 1)).all()
    o = torch.randn(B, L, Hv, Dv, generator=g)
    z = torch.randn(B, L, Hv * Dv, generator=g)
    w = torch.zeros(Dv)
    assert torch.equal(oracle.finish_delta(o, z, w, 1e-6), torch.zeros(B, L, Hv * Dv))


def test_golden_projections_frozen():
    for case, d in load_projections().items():
        assert torch.equal(oracle.linear(d["x"], d["w"]), d["plain"]), case
        assert torch.allclose(oracle.linear(d["x"], d["w"], dtype="f32"), d["plain_f32"], rtol=1e-5, atol=1e-6), case
        assert torch.equal(oracle.linear(d["x"], d["w"], residual=d["res"]), d["res_out"]), case
        # activations go through libm-dependent erf / exp: allow one bf16 step on a handful of elements
        for name, got in (("geglu", oracle.geglu(oracle.linear(d["x"], d["w"]))),
                          ("swiglu", oracle.swiglu(oracle.linear(d["x"], d["w"]), oracle.linear(d["x"], d["w2"]))),
                          ("bias_gelu_res", oracle.linear(d["x"], d["w"], d["bias"], act="gelu", residual=d["res"]))):
            diff = (got - d[name]).abs()
            assert diff.max() <= 2 ** -7 * d[name].abs().max(), (case, name)
            assert (diff > 0).float().mean() < 1e-3, (case, name)


def test_golden_delta_rule_frozen():
    d = load_delta_rule()
    cu = d["cu_seqlens"].tolist()
    for s in range(len(cu) - 1):
        sl = slice(cu[s], cu[s + 1])
        tr = lambda t: t[sl].transpose(0, 1).unsqueeze(0).contiguous()
        o = oracle.sequential_delta_rule(tr(d["q"]), tr(d["k"]), tr(d["v"]), d["g"][sl].t().unsqueeze(0).contiguous(),
                                         d["beta"][sl].t().unsqueeze(0).contiguous())
        assert torch.allclose(o[0], d["out"][sl], atol=1e-6)
        c = oracle.chunked_delta_rule(tr(d["q"]), tr(d["k"]), tr(d["v"]), d["g"][sl].t().unsqueeze(0).contiguous(),
                                      d["beta"][sl].t().unsqueeze(0).contiguous())
        assert (c[0] - d["out"][sl]).abs().max() < 1e-4


def test_conv_silu_inputs_of_the_reference_kernel_test():
    """Inputs of `conv_cuda_matches_candle_across_batches_and_padding` (src/archs/qwen35_text.rs:1264-1318):
    B2, L7, C31, K4, closed-form values; the vectorised oracle against a tap-by-tap scalar loop, 1e-3 as there."""
    B, L, Cc, K = 2, 7, 31, 4
    x = torch.tensor([((i * 17 % 41) - 20.0) * 0.04 for i in range(B * L * Cc)]).reshape(B, L, Cc)
    w = torch.tensor([((i * 11 % 23) - 11.0) * 0.02 for i in range(Cc * K)]).reshape(Cc, 1, K)
    for dt in ("f32", "bf16"):
        got = oracle.causal_conv_silu(x.to(torch.bfloat16) if dt == "bf16" else x, w.to(torch.bfloat16) if dt == "bf16" else w, dtype=dt)
        xx = x.to(torch.bfloat16).float() if dt == "bf16" else x
        ww = w.to(torch.bfloat16).float().reshape(Cc, K) if dt == "bf16" else w.reshape(Cc, K)
        want = torch.zeros(B, L, Cc)
        for b in range(B):
            for t in range(L):
                for c in range(Cc):
                    acc = 0.0
                    for tap in range(K):
                        src = t + tap - K + 1
                        if src >= 0:
                            acc += float(xx[b, src, c]) * float(ww[c, tap])
                    want[b, t, c] = acc / (1.0 + math.exp(-acc))
        assert (got - want).abs().max() < (1e-3 if dt == "f32" else 0.04)
    # the first token of every batch row sees only its own tap (zero left padding per row)
    got = oracle.causal_conv_silu(x, w, dtype="f32")
    first = x[:, 0] * w.reshape(Cc, K)[:, K - 1]
    assert torch.allclose(got[:, 0], first / (1 + torch.exp(-first)), atol=1e-6)


def test_encoder_oracle_matches_an_independent_implementation():
    """The ModernBERT encoder restatement against `transformers`' ModernBertModel (an independent implementation of
    the same architecture, eager attention, f32) on random weights: agreement to 1e-4. The reference's own encoder
    snapshot (src/archs/modernbert.rs:1445-1504) needs a Hugging Face checkpoint that is not available offline."""
    transformers = pytest.importorskip("transformers")
    cfg = oracle.EncoderConfig(vocab_size=500, hidden_size=128, num_hidden_layers=4, num_attention_heads=2,
                               intermediate_size=192)
    w = oracle.init_weights(cfg, 3)
    g = torch.Generator().manual_seed(4)
    for k in w:
        if "norm" in k:
            w[k] = w[k] + 0.1 * torch.randn(w[k].shape, generator=g)
    hc = transformers.ModernBertConfig(
        vocab_size=500, hidden_size=128, num_hidden_layers=4, num_attention_heads=2, intermediate_size=192,
        max_position_embeddings=512, norm_eps=1e-5, norm_bias=False, global_attn_every_n_layers=3, local_attention=128,
        global_rope_theta=160000.0, local_rope_theta=10000.0, attention_bias=False, mlp_bias=False,
        attn_implementation="eager", embedding_dropout=0.0, mlp_dropout=0.0, attention_dropout=0.0, pad_token_id=0)
    model = transformers.ModernBertModel(hc).eval().float()
    sd = {"embeddings.tok_embeddings.weight": w["tok_embeddings"], "embeddings.norm.weight": w["embeddings_norm"],
          "final_norm.weight": w["final_norm"]}
    for i in range(4):
        p = f"layers.{i}."
        sd.update({p + "attn.Wqkv.weight": w[p + "Wqkv"], p + "attn.Wo.weight": w[p + "Wo"], p + "mlp.Wi.weight": w[p + "Wi"],
                   p + "mlp.Wo.weight": w[p + "mlp_Wo"], p + "mlp_norm.weight": w[p + "mlp_norm"]})
        if i > 0:
            sd[p + "attn_norm.weight"] = w[p + "attn_norm"]
    result = model.load_state_dict(sd, strict=False)
    assert not result.missing_keys and not result.unexpected_keys
    ids = torch.randint(1, 500, (180,), generator=g)  # longer than the 129-token band
    with torch.no_grad():
        ref = model(input_ids=ids.unsqueeze(0), attention_mask=torch.ones(1, 180, dtype=torch.long)).last_hidden_state[0]
    assert (oracle.encoder_forward(ids, w, cfg) - ref).abs().max() < 1e-4


def test_rope_index_arithmetic_matches_plain_rope_on_the_reference_test_inputs():
    """The check of `fused_rope_qkv_matches_candle` (src/archs/modernbert.rs:768-817): fused split kernel, restated
    index by index, against the plain rotate-half rope on the test's formula inputs; bf16 tolerance 0.03, and here
    also exact agreement in f32; v passes through unchanged."""
    cos, sin, values = oracle.rope_qkv_test_inputs()
    B, L, _, H, D = values.shape
    for dtype, tol in (("f32", 1e-6), ("bf16", 0.03)):
        src = oracle.round_bf16(torch.from_numpy(values)).numpy() if dtype == "bf16" else values
        q, k, v = oracle.rope_qkv_indexed(src, cos, sin, L, H, D, dtype=dtype)
        for b in range(B):
            x = torch.from_numpy(src[b])  # [L, 3, H, D]
            want_q = oracle.rope(x[:, 0], torch.from_numpy(cos), torch.from_numpy(sin))
            want_k = oracle.rope(x[:, 1], torch.from_numpy(cos), torch.from_numpy(sin))
            assert np.abs(q[b * L:(b + 1) * L] - want_q.numpy()).max() <= tol
            assert np.abs(k[b * L:(b + 1) * L] - want_k.numpy()).max() <= tol
            assert np.array_equal(v[b * L:(b + 1) * L], src[b][:, 2])


def test_norms_match_their_definitions():
    g = torch.Generator().manual_seed(9)
    x = torch.randn(7, 96, generator=g) * 3 + 0.5
    w = torch.randn(96, generator=g)
    want = torch.nn.functional.layer_norm(x, (96,), w, None, 1e-5)
    assert (oracle.layer_norm(x, w, 1e-5) - want).abs().max() < 1e-5
    rms = oracle.rms_norm(x, w, 1e-6)
    assert torch.allclose(rms, x / (x.pow(2).mean(-1, keepdim=True) + 1e-6).sqrt() * (1 + w), atol=1e-5)
    # partial rotation leaves the tail of every head alone
    cos, sin = torch.rand(7, 8), torch.rand(7, 8)
    y = oracle.rope(x.view(7, 3, 32), cos, sin, rotary_dim=16)
    assert torch.equal(y[..., 16:], x.view(7, 3, 32)[..., 16:])


def test_qwen35_decoder_oracle_matches_transformers():
    """The decoder restatement (full attention with interleaved gate, per-head q / k norms, partial rope, causal
    GQA; linear attention; (1 + w) RMSNorm; SwiGLU) against `transformers`' Qwen3.5 text model, an independent
    implementation of the same architecture, on random-init weights in f32."""
    cfg_mod = pytest.importorskip("transformers.models.qwen3_5.configuration_qwen3_5")
    mod = pytest.importorskip("transformers.models.qwen3_5.modeling_qwen3_5")
    cfg = oracle.DecoderConfig(vocab_size=100, hidden_size=64, intermediate_size=96, num_hidden_layers=4, num_attention_heads=2,
                               num_key_value_heads=1, head_dim=32, linear_num_key_heads=2, linear_num_value_heads=4,
                               linear_key_head_dim=16, linear_value_head_dim=16)
    w = oracle.qwen35.init_weights(cfg, 77)
    hf_cfg = cfg_mod.Qwen3_5TextConfig(
        vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size,
        num_hidden_layers=cfg.num_hidden_layers, num_attention_heads=cfg.num_attention_heads,
        num_key_value_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim, rms_norm_eps=cfg.rms_norm_eps,
        linear_num_key_heads=cfg.linear_num_key_heads, linear_num_value_heads=cfg.linear_num_value_heads,
        linear_key_head_dim=cfg.linear_key_head_dim, linear_value_head_dim=cfg.linear_value_head_dim,
        layer_types=[cfg.layer_type(i) for i in range(cfg.num_hidden_layers)],
        rope_parameters={"rope_type": "default", "rope_theta": cfg.rope_theta, "partial_rotary_factor": cfg.partial_rotary_factor,
                         "mrope_section": [2, 1, 1]})
    model = mod.Qwen3_5TextModel(hf_cfg).eval()
    sd = model.state_dict()
    for name, t in w.items():
        key = name if name in sd else name + ".weight"
        assert key in sd and sd[key].shape == t.shape, (name, key)
        sd[key].copy_(t)
    ids = torch.randint(0, cfg.vocab_size, (37,), generator=torch.Generator().manual_seed(78))
    with torch.no_grad():
        want = model(input_ids=ids.unsqueeze(0)).last_hidden_state[0]
    got = oracle.decoder_forward(ids, w, cfg, dtype="f32")
    assert (got - want).abs().max() <= 1e-4 * float(want.abs().max())


def test_layers_fixture_is_what_the_oracle_computes():
    """tests/golden/layers.npz freezes oracle outputs for attention, causal GQA attention, norms and RoPE."""
    from golden_io import load_layers
    L = load_layers()
    qkv, cu = L["attn/qkv"], L["attn/cu_seqlens"].tolist()
    for name, window in (("global", -1), ("band", 64)):
        got = torch.cat([oracle.attention(qkv[a:z, 0], qkv[a:z, 1], qkv[a:z, 2], window) for a, z in zip(cu[:-1], cu[1:])])
        assert torch.allclose(got, L[f"attn/{name}"], atol=1e-6)
    x, w, b = L["norm/x"], L["norm/w"], L["norm/b"]
    assert torch.equal(oracle.layer_norm(x, w, 1e-5, dtype="bf16", bias=b), L["norm/layer_bias"])
    assert torch.equal(oracle.rms_norm(x, w - 1, 1e-6, dtype="bf16"), L["norm/rms"])
