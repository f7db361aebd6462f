"""The reference's own known-answer inputs for the stages around the projections, run through the kernels:
attention masks (src/archs/modernbert.rs:1408-1443), windowed versus dense attention (:1506-1533), RMSNorm
(src/archs/qwen35_text.rs:1214-1262), rotary tables (src/archs/modernbert.rs:1359-1406); the fused per-head norm + rope
against the two separate calls and against candle's bf16 rounding; and the failure paths that need no fault: argument
rejection and a bounded wait that runs out by itself."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from conftest import max_rel
from sys1_b200 import _lib, modernbert, norm, qwen35

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _embed(t, width=64):
    """[L, H, d] -> [L, H, 64] with zero columns: dot products and outputs of the first d columns are unchanged."""
    out = torch.zeros(t.shape[0], t.shape[1], width)
    out[..., : t.shape[-1]] = t
    return out.to(torch.bfloat16)


def test_windowed_attention_reference_inputs(ctx):
    """q, k, v = arange(48) / 37, 29, 19 as [1, 2, 6, 4], scale 0.5, window 2 (:1506-1533), rounded to bf16 and widened to
    the kernel's head dim with zeros. The padded variant (4 real tokens + 2 masked) is the packed layout's 4-token sequence."""
    values = torch.arange(48, dtype=torch.float32).reshape(1, 2, 6, 4)
    q, k, v = (oracle.round_bf16(values / d) for d in (37.0, 29.0, 19.0))
    local = oracle.local_attention_mask(6, 2)
    glob = oracle.global_attention_mask(torch.tensor([[1.0, 1.0, 1.0, 1.0, 0.0, 0.0]]), 6)
    tok = lambda t: _embed(t[0].transpose(0, 1)).to(DEV)  # [L, H, 64]
    got = modernbert.attention_varlen(tok(q), tok(k), tok(v), np.array([0, 6], dtype=np.int32), window=2, scale=0.5)
    want = oracle.eager_attention(q, k, v, 0.5, local)[0].transpose(0, 1)          # [6, 2, 4]
    assert max_rel(got.view(6, 2, 64)[..., :4], want) <= 2e-2
    assert float(got.view(6, 2, 64)[..., 4:].float().abs().max()) == 0.0
    got4 = modernbert.attention_varlen(tok(q)[:4], tok(k)[:4], tok(v)[:4], np.array([0, 4], dtype=np.int32), window=2, scale=0.5)
    want4 = oracle.eager_attention(q, k, v, 0.5, glob + local)[0].transpose(0, 1)[:4]
    assert max_rel(got4.view(4, 2, 64)[..., :4], want4) <= 2e-2
    ctx.sync()


def test_local_mask_only_exposes_nearby_tokens(ctx):
    """The property `local_attention_mask` states (:1408-1422): with window w a query's output does not depend on keys
    and values farther than w. (Not bit for bit: the kernel rescales its accumulator when ANY row of a warp has seen its
    maximum grow, so a neighbour row's band can move the reference point a row's probabilities are rounded against.)"""
    g = torch.Generator().manual_seed(3)
    L, H, w = 300, 2, 64
    q, k, v = (torch.randn(L, H, 64, generator=g).to(torch.bfloat16).to(DEV) for _ in range(3))
    cu = np.array([0, L], dtype=np.int32)
    base = modernbert.attention_varlen(q, k, v, cu, window=w).clone()
    i = 150
    k2, v2 = k.clone(), v.clone()
    far = torch.tensor([j for j in range(L) if abs(j - i) > w], device=DEV)
    k2[far] = 9.0
    v2[far] = -7.0
    moved = modernbert.attention_varlen(q, k2, v2, cu, window=w)
    scale = float(base[i].float().abs().max())
    assert float((base[i].float() - moved[i].float()).abs().max()) <= 2 ** -7 * scale
    assert float((base[i + w + 5].float() - moved[i + w + 5].float()).abs().max()) > 0.5   # that row does see replaced keys
    ctx.sync()


def test_rms_norm_reference_inputs(ctx):
    """Width 4096, three rows, weight 2 i / width - 1 (:1214-1262); bf16 bound of the reference: 1e-2 absolute."""
    width = 4096
    weight = oracle.round_bf16(torch.arange(width, dtype=torch.float32) * (2.0 / width) - 1.0)
    values = oracle.round_bf16(torch.tensor([((i * 71 % 503) - 251.0) / 37.0 for i in range(3 * width)]).reshape(3, width))
    got = norm.norm(values.to(torch.bfloat16).to(DEV), weight.to(torch.bfloat16).to(DEV), 1e-6, norm.RMS_NORM).float().cpu()
    variance = values.square().mean(-1, keepdim=True)
    expected = oracle.round_bf16(values * (1.0 / (variance + 1e-6).sqrt()) * (weight + 1.0))
    assert float((got - expected).abs().max()) <= 1e-2
    ctx.sync()


def test_rotary_tables_resolve_every_position_on_the_device(ctx):
    """`RotaryEmbedding` tables as the encoder builds them (f32, 8192 positions, theta 160000): neighbouring positions
    rotate the same head differently at 1, 255, 257, 2047, 2049, 4095, 4097, 8190 (:1359-1406)."""
    rot = modernbert.RotaryEmbedding(160000.0, 64, 8192, DEV)
    assert rot.sin.dtype == torch.float32 and rot.sin.shape == (8192, 32)
    pos = torch.tensor([p + d for p in (1, 255, 257, 2047, 2049, 4095, 4097, 8190) for d in (0, 1)], dtype=torch.int32, device=DEV)
    assert float((rot.sin[pos[0::2].long()] - rot.sin[pos[1::2].long()]).abs().amax(dim=1).min()) > 1e-7
    x = torch.ones(len(pos), 3 * 64, dtype=torch.bfloat16, device=DEV)
    rot.apply_qkv(x, pos, 1)
    assert not any(torch.equal(x[2 * i, :128], x[2 * i + 1, :128]) for i in range(len(pos) // 2))
    assert torch.equal(x[:, 128:], torch.ones_like(x[:, 128:]))  # v is untouched
    ctx.sync()


@pytest.mark.parametrize("T,H,D,rot,stride_mult", [(70, 8, 256, 64, 2), (33, 2, 256, 64, 1), (129, 3, 128, 32, 1), (10, 4, 64, 64, 2)])
def test_head_norm_rope_fused_pass(ctx, T, H, D, rot, stride_mult):
    g = torch.Generator().manual_seed(T + H)
    stride = stride_mult * D
    x = (torch.randn(T, H * stride + 8, generator=g) * 2).to(torch.bfloat16)   # row wider than the heads: ld != H * stride
    w = (torch.randn(D, generator=g) * 0.2).to(torch.bfloat16)
    pos = torch.randint(0, 500, (T,), generator=g).to(torch.int32)
    rp = qwen35.RopeParams(1e7, rot, 512, DEV)
    # bf16_ops = 0 is bit-identical to s1_norm on the head rows followed by s1_rope
    a = x.to(DEV).clone()
    norm.head_norm_rope_(a, H, stride, D, w.to(DEV), 1e-6, rp.cos, rp.sin, pos.to(DEV), rot, bf16_ops=False)
    b = x.to(DEV).clone()
    for h in range(H):
        rows = b[:, h * stride:h * stride + D]
        norm.norm(rows, w.to(DEV), 1e-6, norm.RMS_NORM, out=rows)
    norm.rope_(b, rp.cos, rp.sin, pos.to(DEV), H, stride, rot)
    assert torch.equal(a, b)
    # bf16_ops = 1 is candle's bf16 arithmetic (three roundings), which the oracle restates
    c = x.to(DEV).clone()
    norm.head_norm_rope_(c, H, stride, D, w.to(DEV), 1e-6, rp.cos, rp.sin, pos.to(DEV), rot, bf16_ops=True)
    ctx.sync()
    heads = torch.stack([x[:, h * stride:h * stride + D] for h in range(H)], dim=1).float()
    cos, sin = rp.cos.cpu()[pos.long()], rp.sin.cpu()[pos.long()]
    want = oracle.rope(oracle.rms_norm(heads, w.float(), 1e-6, "bf16"), cos, sin, rot, bf16_ops=True)
    got = torch.stack([c[:, h * stride:h * stride + D] for h in range(H)], dim=1).float().cpu()
    want = oracle.round_bf16(want)
    # (f32 sums in another order can move a value by one bf16 step here and there)
    assert float((got != want).float().mean()) < 0.01 and max_rel(got, want) <= 2 ** -7
    # columns outside the heads (the gate halves, the row tail) are untouched
    if stride_mult == 2:
        assert torch.equal(c[:, D:stride].cpu(), x[:, D:stride])
    assert torch.equal(c[:, H * stride:].cpu(), x[:, H * stride:])


def test_arguments_that_must_be_rejected(ctx):
    x = torch.zeros(16, 64, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(64, 4, dtype=torch.bfloat16, device=DEV)
    pos = torch.zeros(16, dtype=torch.int32, device=DEV)
    P = lambda t: C.c_void_p(t.data_ptr())
    # the convolution cannot run in place: a token reads the rows before it
    rc = ctx._lib.s1_conv_silu(ctx.handle, P(x), 64, P(w), P(pos), 16, 64, 4, P(x), 64)
    assert rc == _lib.S1_EINVAL and b"overlaps" in ctx._lib.s1_last_error(ctx.handle)
    rc = ctx._lib.s1_conv_silu(ctx.handle, P(x), 64, P(w), P(pos), 15, 64, 4, C.c_void_p(x.data_ptr() + 128), 64)
    assert rc == _lib.S1_EINVAL
    q = torch.zeros(8, 1, 64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(_lib.S1Error, match="scale"):
        modernbert.attention_varlen(q, q, q, np.array([0, 8], dtype=np.int32), scale=0.0)
    with pytest.raises(_lib.S1Error, match="scale"):
        modernbert.attention_varlen(q, q, q, np.array([0, 8], dtype=np.int32), scale=-0.125)
    with pytest.raises(_lib.S1Error):
        ctx.set_option("debug", 1)  # timing ablations are not part of the production build
    ctx.sync()


def test_a_bounded_wait_that_runs_out_is_reported_and_the_context_survives(ctx):
    """`s1_selftest_bounded_wait`: a wait nothing can satisfy (no copy or MMA in flight) gives up after
    "wait_limit_cycles", the kernel returns by itself, `s1_sync` says S1_EKERNEL, and the next call on the same context
    works. Nothing traps or faults."""
    ctx.sync()
    ctx.set_option("wait_limit_cycles", 4_000_000)  # a couple of milliseconds
    try:
        ctx.check(ctx._lib.s1_selftest_bounded_wait(ctx.handle))
        with pytest.raises(_lib.S1Error) as info:
            ctx.sync()
        assert info.value.code == _lib.S1_EKERNEL and "bounded wait" in str(info.value)
    finally:
        ctx.set_option("wait_limit_cycles", 2_000_000_000)
    ctx.sync()  # the status was cleared: the context is clean again
    from sys1_b200 import linear
    g = torch.Generator().manual_seed(0)
    a = torch.randn(200, 64, generator=g).to(torch.bfloat16)
    wt = (torch.randn(128, 64, generator=g) * 0.1).to(torch.bfloat16)
    y = linear.fused_linear(a.to(DEV), wt.to(DEV))
    ctx.sync()
    assert max_rel(y, oracle.linear(a, wt, dtype="f32")) <= 2e-2
