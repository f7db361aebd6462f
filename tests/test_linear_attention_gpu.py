"""The stages around the gated delta rule (conv + SiLU, delta_inputs, finish_delta) and the whole
Qwen3.5 linear-attention layer on a packed batch, against the CPU oracle."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from conftest import max_rel
from sys1_b200 import batching, linear, qwen35

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_conv_silu_packed_matches_the_oracle(ctx):
    """Closed-form inputs in the style of the reference's kernel test (src/archs/qwen35_text.rs:1264-1318), two
    sequences packed back to back: each restarts its left padding. Tolerance 1e-3 as in the reference."""
    lens, Cc, K = [7, 5], 32, 4
    T = sum(lens)
    x = torch.tensor([((i * 17 % 41) - 20.0) * 0.04 for i in range(T * Cc)]).reshape(T, Cc).to(torch.bfloat16)
    w = torch.tensor([((i * 11 % 23) - 11.0) * 0.02 for i in range(Cc * K)]).reshape(Cc, 1, K).to(torch.bfloat16)
    b, _ = batching.pack_next(lens, batching.BatcherConfig(token_budget=64))
    got = qwen35.conv_silu(x.to(DEV), w.to(DEV), torch.from_numpy(b.positions).to(DEV)).float().cpu()
    want = torch.cat([oracle.causal_conv_silu(x[a:z].unsqueeze(0), w)[0] for a, z in zip(b.cu_seqlens[:-1], b.cu_seqlens[1:])])
    assert (got - want).abs().max() < 1e-3
    assert not torch.allclose(got[7], oracle.causal_conv_silu(x.unsqueeze(0), w)[0][7], atol=1e-3)  # boundary matters


@pytest.mark.parametrize("lens,Cc,K", [([40, 3, 70], 64, 4), ([16, 16, 1, 31], 8, 4), ([33, 20], 32, 3)])
def test_conv_silu_longer_sequences_and_other_tap_counts(ctx, lens, Cc, K):
    """Sequences that span several of the kernel's 16-token walks, boundaries on and off the walk boundaries, and a
    tap count served by the per-token kernel; bit-exact against the oracle's per-tap bf16 rounding up to the final SiLU."""
    T = sum(lens)
    g = torch.Generator().manual_seed(T + Cc)
    x = torch.randn(T, Cc, generator=g).to(torch.bfloat16)
    w = (torch.randn(Cc, 1, K, generator=g) * 0.4).to(torch.bfloat16)
    b, _ = batching.pack_next(lens, batching.BatcherConfig(token_budget=1024))
    got = qwen35.conv_silu(x.to(DEV), w.to(DEV), torch.from_numpy(b.positions).to(DEV)).float().cpu()
    want = torch.cat([oracle.causal_conv_silu(x[a:z].unsqueeze(0), w)[0] for a, z in zip(b.cu_seqlens[:-1], b.cu_seqlens[1:])])
    assert (got - want).abs().max() <= 2.0 ** -7 * want.abs().max()
    assert float((got == want).float().mean()) > 0.99


def _layer(seed, hidden=256, Hk=4, Hv=8):
    g = torch.Generator().manual_seed(seed)
    width = 2 * Hk * 128 + Hv * 128
    mk = lambda n, k, s=0.05: (torch.randn(n, k, generator=g) * s).to(torch.bfloat16)
    return dict(qkv=mk(width, hidden), z=mk(Hv * 128, hidden), b=mk(Hv, hidden, 0.3), a=mk(Hv, hidden, 0.3),
                conv=(torch.randn(width, 1, 4, generator=g) * 0.4).to(torch.bfloat16), A_log=torch.randn(Hv, generator=g) * 0.5,
                dt_bias=torch.randn(Hv, generator=g) * 0.5, norm=(1 + 0.1 * torch.randn(128, generator=g)).to(torch.bfloat16),
                out=mk(hidden, Hv * 128), Hk=Hk, Hv=Hv, hidden=hidden)


def test_delta_inputs_and_finish_match_the_oracle(ctx):
    P = _layer(3)
    Hk, Hv = P["Hk"], P["Hv"]
    g = torch.Generator().manual_seed(4)
    T = 50
    mixed = torch.randn(T, 2 * Hk * 128 + Hv * 128, generator=g).to(torch.bfloat16)
    bb, aa = (torch.randn(T, Hv, generator=g).to(torch.bfloat16) for _ in range(2))
    neg = -torch.exp(P["A_log"])
    want = oracle.delta_inputs(mixed.unsqueeze(0), bb.unsqueeze(0), aa.unsqueeze(0), P["dt_bias"], neg, Hk, Hv, 128, 128)
    outs = [torch.empty(T, Hv, 128, device=DEV) for _ in range(3)] + [torch.empty(T, Hv, device=DEV) for _ in range(2)]
    md, bd, ad = mixed.to(DEV), bb.to(DEV), aa.to(DEV)
    dtb, ng = P["dt_bias"].to(DEV), neg.to(DEV)
    ctx.check(ctx._lib.s1_delta_inputs(ctx.handle, md.data_ptr(), md.stride(0), bd.data_ptr(), ad.data_ptr(), bd.stride(0),
                                       dtb.data_ptr(), ng.data_ptr(), T, Hk, Hv, *(C.c_void_p(o.data_ptr()) for o in outs)))
    ctx.sync()
    for got, ref in zip(outs, want):  # oracle layout [1, H, L, ...] -> [L, H, ...]
        ref = ref[0].transpose(0, 1)
        assert torch.allclose(got.cpu(), ref, atol=2e-6, rtol=1e-5)
    o = torch.randn(T, Hv, 128, generator=g)
    z = torch.randn(T, Hv * 128, generator=g).to(torch.bfloat16)
    y = torch.empty(T, Hv * 128, dtype=torch.bfloat16, device=DEV)
    od, zd, nd = o.to(DEV), z.to(DEV), P["norm"].to(DEV)
    ctx.check(ctx._lib.s1_delta_finish(ctx.handle, od.data_ptr(), zd.data_ptr(), zd.stride(0), nd.data_ptr(), C.c_float(1e-6),
                                       T, Hv, y.data_ptr(), y.stride(0)))
    ctx.sync()
    want = oracle.finish_delta(o.unsqueeze(0), z.unsqueeze(0), P["norm"], 1e-6)[0]
    assert max_rel(y, want) <= 2 ** -7


def test_linear_attention_layer_on_a_packed_batch(ctx):
    """in_proj -> conv + SiLU -> delta_inputs -> recurrence -> finish -> out_proj + residual against the oracle's
    composition of the same reference steps (src/archs/qwen35_text.rs:491-629), per sequence."""
    P = _layer(11)
    Hk, Hv, hidden = P["Hk"], P["Hv"], P["hidden"]
    lens = [70, 9, 130]
    b, _ = batching.pack_next(lens, batching.BatcherConfig(token_budget=512))
    g = torch.Generator().manual_seed(12)
    x = torch.randn(b.total_tokens, hidden, generator=g).to(torch.bfloat16)
    lin = lambda w: linear.linear_no_bias(w.to(DEV))
    layer = qwen35.LinearAttention(lin(P["qkv"]), lin(P["z"]), lin(P["b"]), lin(P["a"]), P["conv"].to(DEV),
                                   (-torch.exp(P["A_log"])).to(DEV), P["dt_bias"].to(DEV), P["norm"].to(DEV), lin(P["out"]),
                                   Hk, Hv, 1e-6)
    got = layer.forward(x.to(DEV), b.cu_seqlens, torch.from_numpy(b.positions).to(DEV), residual=x.to(DEV))
    ctx.sync()
    want = torch.empty(b.total_tokens, hidden)
    for a, z in zip(b.cu_seqlens[:-1], b.cu_seqlens[1:]):
        xs = x[a:z]
        mixed = oracle.causal_conv_silu(oracle.linear(xs, P["qkv"]).unsqueeze(0), P["conv"])
        q, k, v, gg, beta = oracle.delta_inputs(mixed, oracle.linear(xs, P["b"]).unsqueeze(0), oracle.linear(xs, P["a"]).unsqueeze(0),
                                                P["dt_bias"], -torch.exp(P["A_log"]), Hk, Hv, 128, 128)
        o = oracle.sequential_delta_rule(q, k, v, gg, beta)
        y = oracle.finish_delta(o, oracle.linear(xs, P["z"]).unsqueeze(0), P["norm"], 1e-6)[0]
        want[a:z] = oracle.linear(y, P["out"], residual=xs)
    assert torch.isfinite(got).all()
    assert max_rel(got, want) <= 2e-2


@pytest.mark.parametrize("lens,Hk,Hv", [([70, 9, 130], 4, 8), ([1, 2, 3, 64, 65, 127, 128, 129, 5], 2, 2), ([700, 61], 2, 6),
                                        ([2048, 1500, 64, 1, 483], 16, 16)])
def test_conv_inside_the_recurrence_is_bit_identical_to_the_two_calls(ctx, lens, Hk, Hv):
    """`s1_gated_delta_rule_conv` applies the causal conv + SiLU to the rows its first kernel stages, with three rows of
    history per 64-token chunk; `s1_conv_silu` followed by `s1_gated_delta_rule` is the same arithmetic in two passes.
    Sequences shorter than the history, ending on and next to chunk boundaries, and key heads shared by several value heads."""
    P = _layer(21 + Hv, hidden=128, Hk=Hk, Hv=Hv)
    b, _ = batching.pack_next(lens, batching.BatcherConfig(token_budget=2048))
    g = torch.Generator().manual_seed(22)
    x = torch.randn(b.total_tokens, P["hidden"], generator=g).to(torch.bfloat16).to(DEV)
    lin = lambda w: linear.linear_no_bias(w.to(DEV))
    pos = torch.from_numpy(b.positions).to(DEV)
    outs = []
    for fuse in (True, False):
        layer = qwen35.LinearAttention(lin(P["qkv"]), lin(P["z"]), lin(P["b"]), lin(P["a"]), P["conv"].to(DEV),
                                       (-torch.exp(P["A_log"])).to(DEV), P["dt_bias"].to(DEV), P["norm"].to(DEV), lin(P["out"]),
                                       Hk, Hv, 1e-6, fuse_conv=fuse)
        assert layer.fuse_conv == fuse
        outs.append(layer.mix(x, b.cu_seqlens, pos).clone())
    ctx.sync()
    assert torch.isfinite(outs[0]).all()
    assert torch.equal(outs[0], outs[1])
