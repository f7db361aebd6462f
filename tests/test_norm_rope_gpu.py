"""`s1_norm` and `s1_rope` through the C ABI against the CPU oracle on identical seeded inputs. Both kernels compute
in f32 and round once to bf16, as the oracle's bf16 mode does, so the outputs must agree to within one bf16 step of
the f32 result (a different summation order may move a value across a rounding boundary): the bound below is
2^-7 relative to the element, and nearly all elements must be bit-identical."""
import numpy as np
import pytest
import torch

import oracle
from sys1_b200 import _lib, device, norm
from sys1_b200.modernbert import RotaryEmbedding

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _close_one_step(got: torch.Tensor, want: torch.Tensor, min_exact: float = 0.98):
    got, want = got.float().cpu(), want.float()
    err = (got - want).abs()
    assert bool((err <= want.abs() * 2.0 ** -7 + 1e-30).all()), float((err / want.abs().clamp_min(1e-30)).max())
    assert float((got == want).float().mean()) >= min_exact


@pytest.mark.parametrize("kind", [norm.LAYER_NORM, norm.RMS_NORM])
@pytest.mark.parametrize("rows,width", [(1, 8), (37, 64), (100, 128), (33, 256), (19, 768), (65, 1024), (9, 1536), (5, 2048),
                                        (7, 2560), (70, 4096), (3, 5120), (41, 6144), (5, 8192), (1000, 1024)])
def test_norm_matches_oracle(ctx, kind, rows, width):
    g = torch.Generator().manual_seed(rows * 7 + width + kind)
    x = (torch.randn(rows, width, generator=g) * 2 + 0.3).to(torch.bfloat16)
    w = (torch.randn(width, generator=g) * 0.5 + (1.0 if kind == 0 else 0.0)).to(torch.bfloat16)
    eps = 1e-5 if kind == 0 else 1e-6
    want = (oracle.layer_norm if kind == 0 else oracle.rms_norm)(x.float(), w.float(), eps, dtype="bf16")
    got = norm.norm(x.to(DEV), w.to(DEV), eps, kind)
    _close_one_step(got, want)


def test_norm_strided_rows_in_place_and_per_head(ctx):
    g = torch.Generator().manual_seed(3)
    T, H, D = 50, 4, 128
    buf = torch.randn(T, H * D + 64, generator=g).to(torch.bfloat16)  # rows with padding
    w = (torch.randn(D, generator=g) * 0.1).to(torch.bfloat16)
    d = buf.to(DEV)
    # per-head q-norm (src/archs/qwen35_text.rs:286-287): rows = tokens x heads on a view of the first H * D columns
    heads = d[:, : H * D]
    for h in range(H):
        col = heads[:, h * D:(h + 1) * D]
        norm.norm(col, w.to(DEV), 1e-6, norm.RMS_NORM, out=col)  # in place, row stride = H * D + 64
    want = oracle.rms_norm(buf[:, : H * D].float().view(T, H, D), w.float(), 1e-6, dtype="bf16").view(T, H * D)
    _close_one_step(d[:, : H * D], want)
    assert torch.equal(d[:, H * D:].cpu(), buf[:, H * D:])  # padding untouched


def test_norm_with_row_index_is_embedding_lookup_plus_norm(ctx):
    g = torch.Generator().manual_seed(4)
    table = torch.randn(300, 256, generator=g).to(torch.bfloat16)
    w = torch.randn(256, generator=g).to(torch.bfloat16)
    ids = torch.randint(0, 300, (77,), generator=g, dtype=torch.int32)
    got = norm.norm(table.to(DEV), w.to(DEV), 1e-5, norm.LAYER_NORM, gather=ids.to(DEV))
    want = oracle.layer_norm(table[ids.long()].float(), w.float(), 1e-5, dtype="bf16")
    _close_one_step(got, want)
    # an index outside the table is reported at the next sync and the context stays usable
    bad = ids.clone()
    bad[5] = 300
    norm.norm(table.to(DEV), w.to(DEV), 1e-5, norm.LAYER_NORM, gather=bad.to(DEV))
    with pytest.raises(RuntimeError, match="outside the table"):
        ctx.sync()
    ctx.sync()
    got = norm.norm(table.to(DEV), w.to(DEV), 1e-5, norm.LAYER_NORM, gather=ids.to(DEV))
    _close_one_step(got, want)


def test_norm_rejects_bad_arguments(ctx):
    x = torch.zeros(4, 64, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ValueError):
        norm.norm(x.cpu(), w, 1e-5)
    with pytest.raises(RuntimeError):
        norm.norm(x[:, :60], w[:60].contiguous(), 1e-5)  # width not a multiple of 8
    with pytest.raises(RuntimeError):
        norm.norm(x, w, 1e-5, kind=3)
    assert norm.norm(x[:0], w, 1e-5).shape == (0, 64)


@pytest.mark.parametrize("T,H,D,rot", [(5, 2, 16, 16), (130, 12, 64, 64), (257, 16, 64, 64), (40, 4, 256, 64), (33, 3, 128, 32)])
def test_rope_on_packed_qkv_matches_oracle(ctx, T, H, D, rot):
    g = torch.Generator().manual_seed(T + D)
    qkv = torch.randn(T, 3 * H * D, generator=g).to(torch.bfloat16)
    P = 64
    pos = torch.randint(0, P, (T,), generator=g, dtype=torch.int32)
    fr = torch.arange(P, dtype=torch.float32).unsqueeze(1) * torch.rand(rot // 2, generator=g).unsqueeze(0)
    cos, sin = fr.cos().contiguous(), fr.sin().contiguous()
    d = qkv.to(DEV)
    norm.rope_(d, cos.to(DEV), sin.to(DEV), pos.to(DEV), 2 * H, D, rot)
    x = qkv.float().view(T, 3, H, D)
    c, s = cos[pos.long()], sin[pos.long()]
    want_q = oracle.round_bf16(oracle.rope(x[:, 0], c, s, rotary_dim=rot))
    want_k = oracle.round_bf16(oracle.rope(x[:, 1], c, s, rotary_dim=rot))
    got = d.cpu().float().view(T, 3, H, D)
    assert torch.equal(got[:, 0], want_q) and torch.equal(got[:, 1], want_k)  # same f32 arithmetic: bit-exact
    assert torch.equal(got[:, 2], x[:, 2])  # v untouched


def test_rope_reference_test_inputs_widened_to_a_16_column_head(ctx):
    """The value and table formulas of the reference's own test (src/archs/modernbert.rs:768-790) at the smallest
    head this kernel takes (16 columns instead of 8: one 16-byte access per half)."""
    B, L, H, D = 2, 5, 2, 16
    n = B * L * 3 * H * D
    values = torch.tensor([((i * 37 % 127) - 63.0) / 21.0 for i in range(n)]).view(B * L, 3 * H * D).to(torch.bfloat16)
    cos = torch.tensor([np.cos(np.float32(i) * np.float32(0.13)) for i in range(L * D // 2)], dtype=torch.float32).view(L, D // 2)
    sin = torch.tensor([np.sin(np.float32(i) * np.float32(0.13)) for i in range(L * D // 2)], dtype=torch.float32).view(L, D // 2)
    pos = torch.arange(B * L, dtype=torch.int32) % L
    d = values.to(DEV)
    norm.rope_(d, cos.to(DEV), sin.to(DEV), pos.to(DEV), 2 * H, D, D)
    q, k, v = oracle.rope_qkv_indexed(values.float().numpy(), cos.numpy(), sin.numpy(), L, H, D, dtype="bf16")
    got = d.cpu().float().view(B * L, 3, H, D).numpy()
    assert np.abs(got[:, 0] - q).max() <= 0.03 and np.abs(got[:, 1] - k).max() <= 0.03  # the reference's tolerance
    assert np.array_equal(got[:, 0], q) and np.array_equal(got[:, 1], k) and np.array_equal(got[:, 2], v)


def test_rope_position_outside_the_table_is_reported(ctx):
    x = torch.ones(8, 3 * 64, dtype=torch.bfloat16, device=DEV)
    rot = RotaryEmbedding(10000.0, 64, 16, DEV)
    pos = torch.arange(8, dtype=torch.int32, device=DEV)
    pos[3] = 16
    rot.apply_qkv(x, pos, 1)
    with pytest.raises(RuntimeError, match="outside the table"):
        ctx.sync()
    ctx.sync()
    assert torch.equal(x[3].cpu(), torch.ones(3 * 64, dtype=torch.bfloat16))  # that token left as it was


@pytest.mark.parametrize("T,H,hidden", [(4100, 16, 1024), (4096, 12, 768), (300, 4, 256), (5000, 3, 512)])
def test_projection_with_rope_in_its_epilogue_equals_the_two_calls(ctx, T, H, hidden):
    """`s1_linear_rope` against `s1_linear` followed by `s1_rope`: bit-identical, both where the fused tile runs (a wave
    or more of 256 x 256 tiles, rotated width a multiple of 128 columns) and where the library falls back to two passes
    (few tokens; 3 heads = 384 rotated columns)."""
    from sys1_b200.linear import fused_linear, linear_rope
    g = torch.Generator().manual_seed(T + H)
    x = torch.randn(T, hidden, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(3 * H * 64, hidden, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    P = 700
    pos = torch.randint(0, P, (T,), generator=g, dtype=torch.int32).to(DEV)
    rot = RotaryEmbedding(10000.0, 64, P, DEV)
    got = linear_rope(x, w, rot.cos, rot.sin, pos, 2 * H)
    want = fused_linear(x, w)
    norm.rope_(want, rot.cos, rot.sin, pos, 2 * H, 64, 64)
    ctx.sync()
    assert torch.equal(got, want)
    # and against the oracle on a sample of rows
    rows = torch.randint(0, T, (40,), generator=g)
    y = oracle.linear(x[rows].float().cpu(), w.float().cpu(), dtype="bf16").view(40, 3, H, 64)
    c, s = rot.cos[pos[rows].long()].cpu(), rot.sin[pos[rows].long()].cpu()
    ref_q = oracle.round_bf16(oracle.rope(y[:, 0], c, s))
    assert (got[rows].float().cpu().view(40, 3, H, 64)[:, 0] - ref_q).abs().max() <= 2e-2 * float(ref_q.abs().max())


def test_layer_norm_with_bias_and_the_scorer_on_marker_rows(ctx):
    """`s1_norm` with a bias (the heads' `layer_norm`) and the scorer chain of src/models/laya.rs:476-518 on the packed
    layout: marker rows selected and normalised in one call, Linear + bias + GELU(erf), Linear to one logit."""
    from sys1_b200 import laya
    from sys1_b200.linear import Linear
    g = torch.Generator().manual_seed(21)
    hidden, lens = 256, [40, 3, 77]
    cu = np.cumsum([0] + lens).astype(np.int32)
    T = int(cu[-1])
    h = torch.randn(T, hidden, generator=g).to(torch.bfloat16)
    nw, nb = (1 + 0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16), (0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16)
    w1, b1 = (torch.randn(hidden, hidden, generator=g) * 0.05).to(torch.bfloat16), (0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16)
    w2, b2 = (torch.randn(1, hidden, generator=g) * 0.05).to(torch.bfloat16), (0.1 * torch.randn(1, generator=g)).to(torch.bfloat16)
    got_n = norm.norm(h.to(DEV), nw.to(DEV), 1e-5, bias=nb.to(DEV))
    _close_one_step(got_n, oracle.layer_norm(h.float(), nw.float(), 1e-5, dtype="bf16", bias=nb.float()))
    markers = [[0, 39, 7], [], [76, 76, 1, 30]]
    scorer = laya.Scorer(nw.to(DEV), nb.to(DEV), Linear(w1.to(DEV), b1.to(DEV)), Linear(w2.to(DEV), b2.to(DEV)))
    got = scorer.score_packed(h.to(DEV), cu, markers)
    ctx.sync()
    assert [len(v) for v in got] == [3, 0, 4]
    rows, _ = laya.marker_rows(cu, markers)
    sel = oracle.layer_norm(h[torch.from_numpy(rows).long()].float(), nw.float(), 1e-5, dtype="f32", bias=nb.float())
    want = oracle.linear(oracle.linear(sel, w1, b1, act="gelu", dtype="f32"), w2, b2, dtype="f32")[:, 0]
    flat = torch.tensor([v for seq in got for v in seq])
    assert (flat - want).abs().max() <= 2e-2 * max(1.0, float(want.abs().max()))
    assert got[2][0] == got[2][1]  # the same marker twice gives the same logit


def test_copy_kind_is_the_embedding_lookup(ctx):
    g = torch.Generator().manual_seed(8)
    table = torch.randn(500, 1024, generator=g).to(torch.bfloat16).to(DEV)
    ids = torch.randint(0, 500, (300,), generator=g, dtype=torch.int32).to(DEV)
    got = norm.embedding(table, ids)
    ctx.sync()
    assert torch.equal(got, table[ids.long()])
