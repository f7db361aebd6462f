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


if __name__ == "__main__":
    projections()
    delta_rule()
    print("wrote", sorted(p.name for p in OUT.glob("*.npz")))
