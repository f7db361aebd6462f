"""Known-answer tests the reference itself holds for the attention masks, the softmax, the windowed attention, the
RMSNorm and the rotary tables, replayed against the oracle's restatements (CPU only). Inputs and expected values are
the ones written in the reference's tests (cited per case); none needs a checkpoint."""
import math

import torch

import oracle
from oracle.modernbert import MASK_VALUE, rope_tables


def test_local_attention_mask_only_exposes_nearby_tokens():
    """src/archs/modernbert.rs:1408-1422: length 4, distance 1."""
    M = MASK_VALUE
    want = torch.tensor([[0.0, 0.0, M, M], [0.0, 0.0, 0.0, M], [M, 0.0, 0.0, 0.0], [M, M, 0.0, 0.0]])
    assert torch.equal(oracle.local_attention_mask(4, 1), want)
    assert MASK_VALUE == -10000.0  # ATTENTION_MASK_VALUE, :23


def test_global_attention_mask_hides_padding_tokens():
    """src/archs/modernbert.rs:1424-1443: keep = [[1, 1, 0]], target length 2."""
    got = oracle.global_attention_mask(torch.tensor([[1, 1, 0]]), 2).flatten()
    assert torch.equal(got, torch.tensor([0.0, 0.0, MASK_VALUE, 0.0, 0.0, MASK_VALUE]))


def test_windowed_attention_matches_dense_attention():
    """src/archs/modernbert.rs:1506-1533: q, k, v = arange(48) / 37, 29, 19 as [1, 2, 6, 4], scale 0.5, window 2, with the
    local mask alone and with the padding mask added; block-banded == dense within 1e-5."""
    values = torch.arange(48, dtype=torch.float32).reshape(1, 2, 6, 4)
    q, k, v = values / 37.0, values / 29.0, values / 19.0
    local = oracle.local_attention_mask(6, 2)
    glob = oracle.global_attention_mask(torch.tensor([[1.0, 1.0, 1.0, 1.0, 0.0, 0.0]]), 6)
    for mask in (local, glob + local):
        dense = oracle.eager_attention(q, k, v, 0.5, mask)
        windowed = oracle.windowed_attention(q, k, v, 0.5, mask, 2)
        assert windowed.shape == dense.shape
        assert float((dense - windowed).abs().max()) < 1e-5
    # the packed-layout form the GPU tests compare with (one sequence, heads on the middle axis, no padded keys) agrees
    # with the reference's eager form on the local mask
    packed = oracle.attention(q[0].transpose(0, 1), k[0].transpose(0, 1), v[0].transpose(0, 1), window=2)
    dense = oracle.eager_attention(q, k, v, 4 ** -0.5, local)[0].transpose(0, 1).reshape(6, 8)
    assert float((packed - dense).abs().max()) < 1e-6


def test_bf16_softmax_handles_padding_masks_without_nans():
    """src/archs/modernbert.rs:1535-1553: softmax of [0, -inf] in bf16 is exactly [1, 0]."""
    scores = oracle.round_bf16(torch.tensor([[0.0, float("-inf")]]))
    out = oracle.attention_softmax(scores, "bf16").flatten()
    assert torch.isfinite(out).all()
    assert out.tolist() == [1.0, 0.0]


def test_bf16_attention_masks_remain_finite():
    """src/archs/modernbert.rs:1555-1580: the masks survive the cast to bf16 (finite, still below -1000)."""
    glob = oracle.round_bf16(oracle.global_attention_mask(torch.tensor([[1.0, 0.0]]), 2)).flatten()
    local = oracle.round_bf16(oracle.local_attention_mask(4, 1)).flatten()
    both = torch.cat([glob, local])
    assert torch.isfinite(both).all()
    assert (glob < -1000).any() and (local < -1000).any()


def test_rms_norm_matches_the_open_coded_reference():
    """src/archs/qwen35_text.rs:1214-1262: width 4096, weight = 2 i / width - 1, values ((71 i mod 503) - 251) / 37 as
    [1, 3, width]; expected = the open-coded formula of :1031-1039; 1e-5 in f32, 1e-2 in bf16."""
    width = 4096
    weight = torch.arange(width, dtype=torch.float32) * (2.0 / width) - 1.0
    values = torch.tensor([((i * 71 % 503) - 251.0) / 37.0 for i in range(3 * width)], dtype=torch.float32).reshape(1, 3, width)
    for dtype, tol in (("f32", 1e-5), ("bf16", 1e-2)):
        x = oracle.round_bf16(values) if dtype == "bf16" else values
        wt = oracle.round_bf16(weight) if dtype == "bf16" else weight
        variance = x.square().mean(-1, keepdim=True)
        expected = x * (1.0 / (variance + 1e-6).sqrt()) * (wt + 1.0)
        if dtype == "bf16":
            expected = oracle.round_bf16(expected)
        actual = oracle.rms_norm(x, wt, 1e-6, dtype)
        assert float((expected - actual).abs().max()) <= tol


def test_rotary_tables_resolve_every_position():
    """src/archs/modernbert.rs:1359-1406: ModernBERT-large shape (head dim 64), theta 160000, 8192 positions, f32
    tables; the sin rows of neighbouring positions differ by more than 1e-7 at 1, 255, 257, 2047, 2049, 4095, 4097, 8190."""
    cfg = oracle.EncoderConfig(hidden_size=1024, num_hidden_layers=28, num_attention_heads=16, intermediate_size=2624)
    cos, sin = rope_tables(cfg, 160000.0, 8192)
    assert cos.dtype == torch.float32 and sin.dtype == torch.float32 and sin.shape == (8192, 32)
    for position in (1, 255, 257, 2047, 2049, 4095, 4097, 8190):
        assert float((sin[position] - sin[position + 1]).abs().max()) > 1e-7, f"positions {position} and {position + 1} share a row"
    # inv_freq as the reference forms it (:69-72): f32(1 / theta^(j / dim))
    inv0 = 1.0 / math.pow(160000.0, 2 / 64)
    assert abs(float(sin[1, 1]) - math.sin(inv0)) < 1e-6
