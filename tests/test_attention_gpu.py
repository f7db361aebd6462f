"""`s1_attention` (flash-form bidirectional attention with an optional band, packed batch, head dim 64) against the
CPU oracle's restatement of the reference's eager attention. bf16 inputs; tolerance 2e-2 of the output scale."""
import numpy as np
import pytest
import torch

import oracle
from conftest import max_rel
from sys1_b200 import modernbert

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(lens, H, window, seed):
    cu = np.cumsum([0] + lens).astype(np.int32)
    T = int(cu[-1])
    g = torch.Generator().manual_seed(seed)
    qkv = torch.randn(T, 3, H, 64, generator=g).to(torch.bfloat16)
    qkv[:, 0] *= 2.0  # sharper softmax than N(0, 1) scores
    d = qkv.to(DEV)
    got = modernbert.attention_varlen(d[:, 0], d[:, 1], d[:, 2], cu, window=window).float().cpu()
    want = torch.empty(T, H * 64)
    for a, z in zip(cu[:-1], cu[1:]):
        if z > a:
            want[a:z] = oracle.attention(qkv[a:z, 0], qkv[a:z, 1], qkv[a:z, 2], window)
    return got, want


@pytest.mark.parametrize("lens,H,window", [
    ([128], 1, -1), ([5], 2, -1), ([129, 1, 300], 3, -1), ([700, 64], 2, 64), ([130, 0, 257, 1], 4, 64), ([1000], 12, 64),
    ([1500], 2, -1),
])
def test_attention_matches_the_oracle(ctx, lens, H, window):
    got, want = _case(lens, H, window, 11 * len(lens) + H)
    ctx.sync()
    assert torch.isfinite(got).all()
    assert max_rel(got, want) <= 2e-2


def test_sequences_do_not_see_each_other(ctx):
    """The rows of a sequence are bit-identical whether it is packed with others or run alone."""
    lens = [200, 333, 90]
    cu = np.cumsum([0] + lens).astype(np.int32)
    g = torch.Generator().manual_seed(9)
    qkv = torch.randn(int(cu[-1]), 3, 4, 64, generator=g).to(torch.bfloat16).to(DEV)
    for window in (-1, 64):
        packed = modernbert.attention_varlen(qkv[:, 0], qkv[:, 1], qkv[:, 2], cu, window=window)
        a, z = int(cu[1]), int(cu[2])
        alone = modernbert.attention_varlen(qkv[a:z, 0], qkv[a:z, 1], qkv[a:z, 2], np.array([0, z - a], dtype=np.int32), window=window)
        assert torch.equal(packed[a:z], alone)


@pytest.mark.parametrize("window", [-1, 64])
def test_row_maximum_that_keeps_growing(ctx, window):
    """Keys whose scores grow along the sequence by far more than 2^8 in total: the running output has to be
    rescaled again and again (the kernel rescales lazily, only past a growth threshold), and early keys end up with
    weights that underflow - the result must still match the oracle."""
    L, H = 1200, 2
    g = torch.Generator().manual_seed(31)
    q = torch.randn(L, H, 64, generator=g)
    k = torch.randn(L, H, 64, generator=g) * 0.3
    v = torch.randn(L, H, 64, generator=g)
    ramp = torch.linspace(0.0, 300.0, L).view(L, 1, 1)      # k gains a growing component along q's mean direction
    k = k + ramp * q.mean(0, keepdim=True) / q.mean(0, keepdim=True).norm(dim=-1, keepdim=True)
    q = q + 6.0 * q.mean(0, keepdim=True) / q.mean(0, keepdim=True).norm(dim=-1, keepdim=True)
    q, k, v = (t.to(torch.bfloat16) for t in (q, k, v))
    cu = np.array([0, L], dtype=np.int32)
    got = modernbert.attention_varlen(q.to(DEV), k.to(DEV), v.to(DEV), cu, window=window).float().cpu()
    ctx.sync()
    want = oracle.attention(q, k, v, window)
    scores = torch.einsum("ihd,jhd->hij", q.float(), k.float()) * 0.125 * 1.4426950408889634
    # precondition of the case: even inside one 129-key band the maximum grows by more than two rescale thresholds
    assert float((scores[:, 600, 600:665].max(-1).values - scores[:, 600, 536:600].max(-1).values).min()) > 16.0
    assert torch.isfinite(got).all()
    assert max_rel(got, want) <= 2e-2


def test_edge_cases_empty_batch_window_wider_than_sequences_and_strided_views(ctx):
    # nothing to do
    q = torch.zeros(0, 2, 64, dtype=torch.bfloat16, device=DEV)
    assert modernbert.attention_varlen(q, q, q, np.array([0], dtype=np.int32)).shape == (0, 128)
    # a window wider than every sequence is global attention
    lens = [50, 7, 120]
    cu = np.cumsum([0] + lens).astype(np.int32)
    g = torch.Generator().manual_seed(77)
    qkv = torch.randn(int(cu[-1]), 3 * 2 * 64 + 16, generator=g).to(torch.bfloat16).to(DEV)  # padded rows: ld = 400
    v4 = qkv[:, : 3 * 128].view(-1, 3, 2, 64)
    wide = modernbert.attention_varlen(v4[:, 0], v4[:, 1], v4[:, 2], cu, window=500)
    glob = modernbert.attention_varlen(v4[:, 0], v4[:, 1], v4[:, 2], cu, window=-1)
    ctx.sync()
    assert torch.equal(wide, glob)
    # window 0: every token attends to itself only, so the output is v
    self_only = modernbert.attention_varlen(v4[:, 0], v4[:, 1], v4[:, 2], cu, window=0)
    ctx.sync()
    assert torch.equal(self_only.view(-1, 2, 64), v4[:, 2])
    # bad arguments are refused before anything is launched
    with pytest.raises(RuntimeError):
        modernbert.attention_varlen(v4[:, 0], v4[:, 1], v4[:, 2], np.array([0, 10], dtype=np.int32))  # does not end at T


def test_full_size_batch_properties(ctx):
    """The encoder benchmark's batch (T = 32768, 16 heads, log-uniform lengths up to 8192): a sequence's rows are
    bit-identical whether it runs inside the packed batch or alone, global and banded, and sampled rows match the
    oracle (which could not finish the whole batch in reasonable time)."""
    from sys1_b200 import batching
    T, H = 32768, 16
    lens = batching.synthetic_lengths(1003, 8, 8192, T, log_uniform=True)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    g = torch.Generator(device=DEV).manual_seed(5)
    qkv = torch.randn(T, 3, H, 64, device=DEV, generator=g).to(torch.bfloat16)
    order = np.argsort(lens)
    picks = [int(order[len(order) // 2]), int(order[-1])]  # a median-length sequence and the longest one
    for window in (-1, 64):
        packed = modernbert.attention_varlen(qkv[:, 0], qkv[:, 1], qkv[:, 2], cu, window=window)
        for s in picks:
            a, z = int(cu[s]), int(cu[s + 1])
            alone = modernbert.attention_varlen(qkv[a:z, 0], qkv[a:z, 1], qkv[a:z, 2], np.array([0, z - a], dtype=np.int32), window=window)
            assert torch.equal(packed[a:z], alone)
        s = picks[0]
        a, z = int(cu[s]), int(cu[s + 1])
        if z - a <= 1500:
            sub = qkv[a:z].cpu()
            want = oracle.attention(sub[:, 0], sub[:, 1], sub[:, 2], window)
            assert max_rel(packed[a:z].float().cpu(), want) <= 2e-2
    ctx.sync()


def test_batch_plan_replaces_the_per_call_tables(ctx):
    """`s1_batch_plan`: the query-block tables built once per batch; the calls then pass no offsets and copy nothing, and
    their results are bit-identical to the per-call form, for the global and the banded variant."""
    lens = [300, 1, 129, 64, 700]
    cu = np.cumsum([0] + lens).astype(np.int32)
    T = int(cu[-1])
    g = torch.Generator().manual_seed(23)
    q, k, v = (torch.randn(T, 4, 64, generator=g).to(torch.bfloat16).to(DEV) for _ in range(3))
    want = {w: modernbert.attention_varlen(q, k, v, cu, window=w).clone() for w in (-1, 64)}
    plan = ctx.batch_plan(cu, T)
    ctx.use_plan(plan)
    try:
        assert ctx.plan_covers(len(lens), T)
        for w in (-1, 64):
            assert torch.equal(modernbert.attention_varlen(q, k, v, cu, window=w), want[w])
        # a batch of another shape is not covered by the plan: its call falls back to its own table
        other = modernbert.attention_varlen(q[:300], k[:300], v[:300], np.array([0, 300], dtype=np.int32))
        assert torch.equal(other, want[-1][:300])
        # raw calls: no offsets and no plan for that shape -> rejected; no offsets with the plan -> accepted without a workspace
        import ctypes as C
        out = torch.empty(T, 256, dtype=torch.bfloat16, device=DEV)
        P = lambda t: C.c_void_p(t.data_ptr())
        rc = ctx._lib.s1_attention(ctx.handle, P(q), 256, P(k), 256, P(v), 256, None, len(lens) + 1, T, 4, 64, -1, C.c_float(0.125), P(out), 256, None, 0)
        assert rc == -1 and b"no batch plan" in ctx._lib.s1_last_error(ctx.handle)
        rc = ctx._lib.s1_attention(ctx.handle, P(q), 256, P(k), 256, P(v), 256, None, len(lens), T, 4, 64, -1, C.c_float(0.125), P(out), 256, None, 0)
        assert rc == 0
        assert torch.equal(out, want[-1])
    finally:
        ctx.use_plan(None)
    ctx.sync()


def test_batch_plans_live_until_released(ctx):
    """A plan stays known to its context however many others are built after it (a stack caches the plans of its recent
    batches) and is forgotten when released, which the Python tensor does by itself when it is dropped."""
    import ctypes as C
    cu = np.array([0, 200, 456], dtype=np.int32)
    first = ctx.batch_plan(cu, 456)
    later = [ctx.batch_plan(np.array([0, 128 + i], dtype=np.int32), 128 + i) for i in range(40)]
    ctx.use_plan(first)
    assert ctx.plan_covers(2, 456)
    ctx.use_plan(None)
    pointer = first.data_ptr()
    keep = first._s1_owner   # the memory stays allocated: only the plan object goes
    del first
    rc = ctx._lib.s1_use_batch_plan(ctx.handle, C.c_void_p(pointer))
    assert rc == -1 and b"no plan was built" in ctx._lib.s1_last_error(ctx.handle)
    # releasing the plan in use leaves none in use; releasing an unknown buffer is not an error
    ctx.use_plan(later[0])
    assert ctx._lib.s1_batch_plan_release(ctx.handle, C.c_void_p(later[0].data_ptr())) == 0
    assert ctx._lib.s1_batch_plan_release(ctx.handle, C.c_void_p(later[0].data_ptr())) == 0
    q = torch.randn(128, 4, 64).to(torch.bfloat16).to(DEV)
    out = torch.empty(128, 256, dtype=torch.bfloat16, device=DEV)
    P = lambda t: C.c_void_p(t.data_ptr())
    rc = ctx._lib.s1_attention(ctx.handle, P(q), 256, P(q), 256, P(q), 256, None, 1, 128, 4, 64, -1, C.c_float(0.125), P(out), 256, None, 0)
    assert rc == -1 and b"no batch plan" in ctx._lib.s1_last_error(ctx.handle)
    ctx._plan = None
    del keep, later
    ctx.sync()
