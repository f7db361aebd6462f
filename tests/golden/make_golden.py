"""Regenerates the golden fixtures in this directory from the CPU oracle (run from the repo root):

    python tests/golden/make_golden.py

The oracle is first checked against the reference's own self-contained known-answer tests (see
tests/test_oracle.py); these files then freeze its outputs on small seeded inputs so that the GPU parity tests
have a fixed target that does not depend on the CPU library version on the GPU box.
Inputs are stored too (bf16 inputs as their float32 values), so a test never has to regenerate them.
"""
from pathlib import Path
import sys

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
import oracle  # noqa: E402

OUT = Path(__file__).resolve().parent


def bf(t):
    return t.to(torch.bfloat16).to(torch.float32)


def projections():
    g = torch.Generator().manual_seed(1002)
    cases = {}
    for name, (T, N, K) in {"tiny": (40, 48, 64), "ragged": (150, 144, 200), "tile_edges": (130, 272, 64)}.items():
        x = bf(torch.randn(T, K, generator=g))
        w = bf(torch.randn(N, K, generator=g) * 0.02)
        w2 = bf(torch.randn(N, K, generator=g) * 0.02)
        bias = bf(torch.randn(N, generator=g) * 0.1)
        res = bf(torch.randn(T, N, generator=g))
        cases[name] = dict(
            x=x, w=w, w2=w2, bias=bias, res=res,
            plain=oracle.linear(x, w),
            plain_f32=oracle.linear(x, w, dtype="f32"),
            res_out=oracle.linear(x, w, residual=res),
            bias_gelu_res=oracle.linear(x, w, bias, act="gelu", residual=res),
            bias_relu=oracle.linear(x, w, bias, act="relu"),
            geglu=oracle.geglu(oracle.linear(x, w)),
            geglu_f32=oracle.geglu(oracle.linear(x, w, dtype="f32"), dtype="f32"),
            swiglu=oracle.swiglu(oracle.linear(x, w), oracle.linear(x, w2)),
        )
    # bf16-valued arrays are stored as their 16-bit patterns (suffix "@bf16"); f32 results as float32
    flat = {}
    for c, d in cases.items():
        for k, v in d.items():
            if k.endswith("_f32"):
                flat[f"{c}/{k}"] = v.numpy()
            else:
                assert torch.equal(bf(v), v)
                flat[f"{c}/{k}@bf16"] = v.to(torch.bfloat16).view(torch.int16).numpy()
    np.savez_compressed(OUT / "projections.npz", **flat)


def delta_rule():
    g = torch.Generator().manual_seed(1004)
    lens = [70, 1, 33, 50]
    T, H, Dk, Dv = sum(lens), 2, 128, 32
    q = torch.randn(T, H, Dk, generator=g)
    k = torch.randn(T, H, Dk, generator=g)
    q = q / (q.square().sum(-1, keepdim=True) + 1e-6).sqrt() * Dk ** -0.5
    k = k / (k.square().sum(-1, keepdim=True) + 1e-6).sqrt()
    v = torch.randn(T, H, Dv, generator=g)
    gate = -torch.nn.functional.softplus(torch.randn(T, H, generator=g)) * 0.5
    beta = torch.sigmoid(torch.randn(T, H, generator=g))
    out = torch.empty(T, H, Dv)
    start = 0
    for n in lens:
        sl = slice(start, start + n)
        tr = lambda t: t[sl].transpose(0, 1).unsqueeze(0).contiguous()  # [1, H, n, D]
        o = oracle.sequential_delta_rule(tr(q), tr(k), tr(v), gate[sl].t().unsqueeze(0).contiguous(),
                                         beta[sl].t().unsqueeze(0).contiguous())  # [1, n, H, Dv]
        out[sl] = o[0]
        start += n
    np.savez_compressed(OUT / "delta_rule.npz", q=q.numpy(), k=k.numpy(), v=v.numpy(), g=gate.numpy(), beta=beta.numpy(),
                        cu_seqlens=np.cumsum([0] + lens).astype(np.int32), out=out.numpy())


def layers():
    """Attention (global and banded), norms, RoPE, causal GQA attention and one whole layer of each architecture:
    small seeded inputs and the oracle's f32 outputs (all stored as float32; bf16-valued inputs are exact in it)."""
    g = torch.Generator().manual_seed(1003)
    out = {}
    # ModernBERT attention, head dim 64, two sequences packed
    lens = [150, 37]
    T, H = sum(lens), 2
    qkv = bf(torch.randn(T, 3, H, 64, generator=g))
    qkv[:, 0] *= 2.0
    out["attn/cu_seqlens"] = np.cumsum([0] + lens).astype(np.int32)
    out["attn/qkv"] = qkv.numpy()
    for name, window in (("global", -1), ("band", 64)):
        o = torch.cat([oracle.attention(qkv[a:z, 0], qkv[a:z, 1], qkv[a:z, 2], window) for a, z in ((0, 150), (150, 187))])
        out[f"attn/{name}"] = o.numpy()
    # causal grouped-query attention with gate, head dim 256
    Hq, KV, glens = 2, 1, [70, 20]
    Tg = sum(glens)
    qg = bf(torch.randn(Tg, Hq, 2, 256, generator=g))
    kk, vv = bf(torch.randn(Tg, KV, 256, generator=g)), bf(torch.randn(Tg, KV, 256, generator=g))
    o = torch.cat([oracle.causal_attention(qg[a:z, :, 0], kk[a:z], vv[a:z]).reshape(z - a, Hq * 256) *
                   torch.sigmoid(qg[a:z, :, 1]).reshape(z - a, Hq * 256) for a, z in ((0, 70), (70, 90))])
    out.update({"gqa/cu_seqlens": np.cumsum([0] + glens).astype(np.int32), "gqa/qg": qg.numpy(), "gqa/k": kk.numpy(),
                "gqa/v": vv.numpy(), "gqa/out": o.numpy()})
    # norms and rope
    x = bf(torch.randn(33, 256, generator=g) * 2 + 0.3)
    w, b = bf(1 + 0.2 * torch.randn(256, generator=g)), bf(0.1 * torch.randn(256, generator=g))
    out.update({"norm/x": x.numpy(), "norm/w": w.numpy(), "norm/b": b.numpy(),
                "norm/layer": oracle.layer_norm(x, w, 1e-5, dtype="bf16").numpy(),
                "norm/layer_bias": oracle.layer_norm(x, w, 1e-5, dtype="bf16", bias=b).numpy(),
                "norm/rms": oracle.rms_norm(x, w - 1, 1e-6, dtype="bf16").numpy()})
    pos = torch.randint(0, 200, (33,), generator=g)
    fr = torch.arange(200, dtype=torch.float32).unsqueeze(1) * torch.rand(32, generator=g).unsqueeze(0)
    r = oracle.round_bf16(oracle.rope(x.view(33, 4, 64), fr.cos()[pos], fr.sin()[pos]))
    out.update({"rope/pos": pos.numpy().astype(np.int32), "rope/cos": fr.cos().numpy(), "rope/sin": fr.sin().numpy(),
                "rope/out": r.reshape(33, 256).numpy()})
    np.savez_compressed(OUT / "layers.npz", **out)


if __name__ == "__main__":
    projections()
    delta_rule()
    layers()
    print("wrote", sorted(p.name for p in OUT.glob("*.npz")))
