"""Parity of the fused projection (`s1_linear`, through the C ABI) with the CPU oracle.

Tolerances
  * against the f32 oracle: max-relative <= 2e-2 (the bound stated for bf16 runs);
  * against the bf16-mirroring oracle: the two differ only where a different f32 summation order flips a bf16
    rounding, so at most one bf16 step (2^-7 relative to the element) on a small fraction of the elements (under 5 %).
"""
import ctypes as C

import pytest
import torch

import oracle
from conftest import max_rel
from golden_io import load_projections
from sys1_b200 import _lib, linear, modernbert, qwen35
from sys1_b200._lib import EPI_GEGLU, EPI_NONE, EPI_SWIGLU

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev_bf16(t):
    return t.to(DEV).to(torch.bfloat16)


def assert_matches_bf16_oracle(y, want, what=""):
    y = y.float().cpu()
    diff = (y - want).abs()
    scale = want.abs().max().clamp_min(1e-6)
    assert diff.max() <= 2 ** -6 * scale, f"{what}: max diff {diff.max():.3e} vs scale {scale:.3e}"
    # elements deep in the GELU tail (|want| below 1e-3 of the scale) are left out of the count: there the f32
    # oracle's 1 + erf cancels to zero while x * Phi(x) evaluated on the tail side does not; both are ~0
    frac = ((diff > 0) & (want.abs() >= 1e-3 * scale)).float().mean().item()
    assert frac < 0.05, f"{what}: {frac:.4f} of the elements differ from the bf16 oracle"


@pytest.mark.parametrize("bn", [0, 128, 256, 384, 512])
def test_golden_fixtures(ctx, bn):
    ctx.set_option("gemm_bn", bn)
    try:
        for case, d in load_projections().items():
            x, w, w2, bias, res = (dev_bf16(d[k]) for k in ("x", "w", "w2", "bias", "res"))
            assert_matches_bf16_oracle(linear.fused_linear(x, w), d["plain"], f"{case} plain")
            assert max_rel(linear.fused_linear(x, w), d["plain_f32"]) <= 2e-2
            assert_matches_bf16_oracle(linear.fused_linear(x, w, residual=res), d["res_out"], f"{case} residual")
            assert_matches_bf16_oracle(linear.fused_linear(x, w, bias=bias, act="gelu", residual=res),
                                       d["bias_gelu_res"], f"{case} bias+gelu+res")
            assert_matches_bf16_oracle(linear.fused_linear(x, w, bias=bias, act="relu"), d["bias_relu"], f"{case} relu")
            assert_matches_bf16_oracle(linear.fused_linear(x, w, epilogue=EPI_GEGLU), d["geglu"], f"{case} geglu")
            assert max_rel(linear.fused_linear(x, w, epilogue=EPI_GEGLU), d["geglu_f32"]) <= 2e-2
            assert_matches_bf16_oracle(linear.fused_linear(x, w, weight_up=w2, epilogue=EPI_SWIGLU), d["swiglu"],
                                       f"{case} swiglu")
        ctx.sync()
    finally:
        ctx.set_option("gemm_bn", 0)


def _base_weights(seed=1002):
    g = torch.Generator().manual_seed(seed)
    mk = lambda n, k: (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16)
    return dict(wqkv=mk(2304, 768), wo=mk(768, 768), wi=mk(2304, 768), wout=mk(768, 1152))


def test_modernbert_base_projections_packed_2048(ctx):
    """The four ModernBERT-base projections with their fused epilogues on a packed batch of 2048 tokens."""
    from sys1_b200 import batching
    lens = batching.synthetic_lengths(1002, 16, 512, 2048)
    T = int(lens.sum())
    g = torch.Generator().manual_seed(7)
    x = torch.randn(T, 768, generator=g).to(torch.bfloat16)
    attn = torch.randn(T, 768, generator=g).to(torch.bfloat16)
    W = _base_weights()
    xd, ad = x.to(DEV), attn.to(DEV)
    Wd = {k: v.to(DEV) for k, v in W.items()}
    proj = modernbert.AttentionProjections(linear.linear_no_bias(Wd["wqkv"]), linear.linear_no_bias(Wd["wo"]))
    mlp = modernbert.Mlp(linear.linear_no_bias(Wd["wi"]), linear.linear_no_bias(Wd["wout"]))

    qkv = proj.qkv(xd)
    assert_matches_bf16_oracle(qkv, oracle.linear(x, W["wqkv"]), "Wqkv")
    assert max_rel(qkv, oracle.linear(x, W["wqkv"], dtype="f32")) <= 2e-2
    h1 = proj.out(ad, residual=xd)
    assert_matches_bf16_oracle(h1, oracle.linear(attn, W["wo"], residual=x), "Wo + residual")
    gated = mlp.gated(xd)
    assert_matches_bf16_oracle(gated, oracle.geglu(oracle.linear(x, W["wi"])), "Wi + GeGLU")
    y = mlp(xd, residual=xd)
    want32 = oracle.mlp_modernbert(x, W["wi"], W["wout"], residual=x, dtype="f32")
    assert max_rel(y, want32) <= 2e-2
    # hidden states within tolerance and the per-token argmax (decision ordering stand-in) identical
    want16 = oracle.mlp_modernbert(x, W["wi"], W["wout"], residual=x, dtype="bf16")
    assert max_rel(y, want16) <= 2 ** -6
    ctx.sync()


def test_qwen35_mlp_swiglu(ctx):
    g = torch.Generator().manual_seed(1004)
    T, H, I = 700, 1024, 3584
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    wg, wu = ((torch.randn(I, H, generator=g) * 0.02).to(torch.bfloat16) for _ in range(2))
    wd = (torch.randn(H, I, generator=g) * 0.02).to(torch.bfloat16)
    mlp = qwen35.Mlp(*(linear.linear_no_bias(w.to(DEV)) for w in (wg, wu, wd)))
    y = mlp(x.to(DEV), residual=x.to(DEV))
    assert max_rel(y, oracle.mlp_qwen35(x, wg, wu, wd, residual=x, dtype="f32")) <= 2e-2
    assert max_rel(y, oracle.mlp_qwen35(x, wg, wu, wd, residual=x, dtype="bf16")) <= 2 ** -6


@pytest.mark.parametrize("T", [1, 7, 127, 128, 129, 255, 257, 1000])
def test_ragged_token_counts(ctx, T):
    g = torch.Generator().manual_seed(T)
    x = torch.randn(T, 136, generator=g).to(torch.bfloat16)
    w = (torch.randn(272, 136, generator=g) * 0.05).to(torch.bfloat16)
    y = linear.fused_linear(x.to(DEV), w.to(DEV))
    assert_matches_bf16_oracle(y, oracle.linear(x, w), f"T={T}")
    y = linear.fused_linear(x.to(DEV), w.to(DEV), epilogue=EPI_GEGLU)
    assert_matches_bf16_oracle(y, oracle.geglu(oracle.linear(x, w)), f"T={T} geglu")


@pytest.mark.parametrize("N,K", [(8, 8), (16, 1024), (48, 5120), (776, 72), (2624 * 2, 1024)])
def test_ragged_feature_sizes(ctx, N, K):
    g = torch.Generator().manual_seed(N * 7 + K)
    T = 300
    x = torch.randn(T, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)
    assert_matches_bf16_oracle(linear.fused_linear(x.to(DEV), w.to(DEV)), oracle.linear(x, w), f"N={N} K={K}")
    if N % 16 == 0:
        assert_matches_bf16_oracle(linear.fused_linear(x.to(DEV), w.to(DEV), epilogue=EPI_GEGLU),
                                   oracle.geglu(oracle.linear(x, w)), f"geglu N={N} K={K}")


def test_output_padding_is_left_untouched(ctx):
    """Stores are clipped at T rows and N columns: a canary around a strided output view must survive."""
    T, N, K = 130, 264, 64
    g = torch.Generator().manual_seed(3)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    big = torch.full((T + 64, N + 72), 7.0, dtype=torch.bfloat16, device=DEV)
    view = big[:T, :N]
    linear.fused_linear(x, w, out=view)
    ctx.sync()
    assert torch.equal(view, linear.fused_linear(x, w))
    assert (big[T:] == 7).all() and (big[:, N:] == 7).all()


def test_tensor_parallel_shards_without_copies(ctx):
    """Column-parallel = a row range of W, row-parallel = a K range of W (strided view) and of x; both go through
    `ldw` / `ldx` with no repacking. The partial sums of the row-parallel shards add up to the full product."""
    g = torch.Generator().manual_seed(1005)
    T, N, K, tp = 384, 512, 1024, 4
    x = torch.randn(T, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.03).to(torch.bfloat16).to(DEV)
    full = linear.fused_linear(x, w)
    cols = torch.cat([linear.fused_linear(x, w[r * N // tp:(r + 1) * N // tp]) for r in range(tp)], dim=1)
    assert torch.equal(cols, full)
    parts = [linear.fused_linear(x[:, r * K // tp:(r + 1) * K // tp], w[:, r * K // tp:(r + 1) * K // tp]) for r in range(tp)]
    summed = torch.stack([p.float() for p in parts]).sum(0)
    assert max_rel(summed, oracle.linear(x.cpu(), w.cpu(), dtype="f32")) <= 2e-2
    # paired shards: a rank takes the same column range of the activated and of the gate half
    I = N // 2
    lo, hi = I // tp, 2 * I // tp
    shard = torch.cat([w[lo:hi], w[I + lo:I + hi]])
    assert torch.equal(linear.fused_linear(x, shard, epilogue=EPI_GEGLU), linear.fused_linear(x, w, epilogue=EPI_GEGLU)[:, lo:hi])


def test_full_budget_row_independence_and_samples(ctx):
    """At the full 32768-token budget: a token's output does not depend on its batch (bit-exact against the same
    rows run alone), and sampled rows match the oracle."""
    g = torch.Generator().manual_seed(32768)
    T = 32768
    W = _base_weights()
    x = torch.randn(T, 768, generator=g).to(torch.bfloat16)
    rows = torch.randint(0, T, (256,), generator=g)
    rows[:4] = torch.tensor([0, 127, 128, T - 1])
    xd = x.to(DEV)
    for name, w, epi in (("wqkv", W["wqkv"], EPI_NONE), ("wi", W["wi"], EPI_GEGLU)):
        full = linear.fused_linear(xd, w.to(DEV), epilogue=epi)
        alone = linear.fused_linear(xd[rows.to(DEV)].contiguous(), w.to(DEV), epilogue=epi)
        assert torch.equal(full[rows.to(DEV)], alone), name
        want = oracle.linear(x[rows], w)
        want = oracle.geglu(want) if epi == EPI_GEGLU else want
        assert_matches_bf16_oracle(alone, want, f"{name} sampled rows")
    res = torch.randn(T, 768, generator=g).to(torch.bfloat16)
    full = linear.fused_linear(xd, W["wo"].to(DEV), residual=res.to(DEV))
    assert_matches_bf16_oracle(full[rows.to(DEV)], oracle.linear(x[rows], W["wo"], residual=res[rows]), "wo sampled rows")
    ctx.sync()


def test_raw_c_abi_call_and_error_codes(ctx):
    """Straight through ctypes, as a foreign caller would: descriptor struct, device pointers, status codes."""
    lib = _lib.load_library()
    T, N, K = 64, 32, 64
    x = torch.ones(T, K, dtype=torch.bfloat16, device=DEV)
    w = torch.full((N, K), 0.5, dtype=torch.bfloat16, device=DEV)
    y = torch.zeros(T, N, dtype=torch.bfloat16, device=DEV)
    d = _lib.LinearDesc(w=w.data_ptr(), ldw=K, w_up=0, ldw_up=0, bias=0, N=N, K=K, epilogue=0, act=0)
    before = lib.s1_launch_count(ctx.handle)
    rc = lib.s1_linear(ctx.handle, C.byref(d), x.data_ptr(), K, None, 0, y.data_ptr(), N, T)
    assert rc == _lib.S1_OK and lib.s1_sync(ctx.handle) == _lib.S1_OK
    assert lib.s1_launch_count(ctx.handle) == before + 1
    assert (y == 32).all()
    bad = _lib.LinearDesc(w=w.data_ptr(), ldw=K, w_up=0, ldw_up=0, bias=0, N=N, K=60, epilogue=0, act=0)
    assert lib.s1_linear(ctx.handle, C.byref(bad), x.data_ptr(), K, None, 0, y.data_ptr(), N, T) == _lib.S1_EINVAL
    assert b"multiples of 8" in lib.s1_last_error(ctx.handle)
    assert lib.s1_linear(ctx.handle, C.byref(d), x.data_ptr() + 2, K, None, 0, y.data_ptr(), N, T) == _lib.S1_EINVAL
    d.epilogue = 2  # SWIGLU without w_up
    assert lib.s1_linear(ctx.handle, C.byref(d), x.data_ptr(), K, None, 0, y.data_ptr(), N, T) == _lib.S1_EINVAL
    d.epilogue = 0
    assert lib.s1_linear(ctx.handle, C.byref(d), x.data_ptr(), K, None, 0, y.data_ptr(), N, 0) == _lib.S1_EINVAL
    assert lib.s1_set_option(ctx.handle, b"nonsense", 1) == _lib.S1_EINVAL


def test_residual_stream_updated_in_place(ctx):
    """`y` aliasing `residual`: the tile is added to the buffer in memory; same values as the out-of-place form."""
    g = torch.Generator().manual_seed(11)
    T, N, K = 1000, 768, 1152
    x = torch.randn(T, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16).to(DEV)
    res = torch.randn(T, N, generator=g).to(torch.bfloat16).to(DEV)
    want = linear.fused_linear(x, w, residual=res)
    stream = res.clone()
    got = linear.fused_linear(x, w, residual=stream, out=stream)
    ctx.sync()
    assert got.data_ptr() == stream.data_ptr()
    assert_matches_bf16_oracle(got, oracle.linear(x.cpu(), w.cpu(), residual=res.cpu()), "in-place residual")
    assert (got.float() - want.float()).abs().max() <= 2 ** -7 * want.float().abs().max()


@pytest.mark.parametrize("bn", [0, 128, 256, 512])
def test_tiles_drawn_at_run_time_give_the_same_result(ctx, bn):
    """`dynamic_tiles`: the CTAs draw their tiles from a counter instead of working through fixed shares. Which CTA computes
    a tile does not change the tile, so every epilogue must give bit-identical results, launch after launch (the counter
    is put back by the kernel itself), for tile counts below, at and far above the number of CTAs."""
    g = torch.Generator().manual_seed(77)
    for T, K, N in [(300, 256, 512), (9000, 768, 2304), (40000, 320, 1536)]:
        x = dev_bf16(torch.randn(T, K, generator=g))
        w = dev_bf16(torch.randn(N, K, generator=g) * 0.05)
        r = dev_bf16(torch.randn(T, N, generator=g))
        ctx.set_option("gemm_bn", bn)
        try:
            want = [linear.fused_linear(x, w), linear.fused_linear(x, w, residual=r),
                    linear.fused_linear(x, w, epilogue=EPI_GEGLU), linear.fused_linear(x, w[: N // 2], weight_up=w[N // 2:], epilogue=EPI_SWIGLU)]
            ctx.set_option("dynamic_tiles", 1)
            for _ in range(3):
                got = [linear.fused_linear(x, w), linear.fused_linear(x, w, residual=r),
                       linear.fused_linear(x, w, epilogue=EPI_GEGLU), linear.fused_linear(x, w[: N // 2], weight_up=w[N // 2:], epilogue=EPI_SWIGLU)]
                for a, b in zip(got, want):
                    assert torch.equal(a, b)
        finally:
            ctx.set_option("dynamic_tiles", 0)
            ctx.set_option("gemm_bn", 0)
    ctx.sync()
