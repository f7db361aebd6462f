"""Oracle for the gated delta rule (test infrastructure only; see the package docstring).

`sequential_delta_rule` is the ground truth: the token-by-token recurrence of the reference's CUDA kernel
(src/kernels/qwen35.cu:53-97) and of its in-test scalar loop (src/archs/qwen35_text.rs:1419-1438).
`chunked_delta_rule` restates the reference's CPU fallback (src/archs/qwen35_text.rs:809-880): chunks of 32,
decay matrix masked before the exponential, triangular inverse by Neumann doubling.
Both take and return float32 in the reference's layout: q, k `[B, H, L, Dk]`, v `[B, H, L, Dv]`, g, beta
`[B, H, L]`; result `[B, L, H, Dv]` (the reference transposes before returning, :880).
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path
from typing import Tuple

import numpy as np
import torch

_HERE = Path(__file__).resolve().parent
_CLIB = None


def _c_lib():
    """The C restatement of the sequential recurrence (oracle/c/delta_rule_seq.c), if it has been built."""
    global _CLIB
    if _CLIB is None:
        so = _HERE / "c" / "liboracle_delta.so"
        if not so.exists():
            return None
        lib = C.CDLL(str(so))
        lib.oracle_delta_rule_seq.restype = None
        lib.oracle_delta_rule_seq.argtypes = [C.c_void_p] * 5 + [C.c_void_p] + [C.c_int] * 5
        _CLIB = lib
    return _CLIB


def sequential_delta_rule(q, k, v, g, beta, use_c: bool = True) -> torch.Tensor:
    """S <- S e^{g_t}; delta = (v_t - S^T k_t) beta_t; S <- S + k_t delta^T; o_t = S^T q_t, S0 = 0, all f32."""
    q, k, v, g, beta = (t.detach().to(torch.float32).contiguous().cpu() for t in (q, k, v, g, beta))
    B, H, L, Dk = q.shape
    Dv = v.shape[-1]
    out = torch.empty((B, L, H, Dv), dtype=torch.float32)
    lib = _c_lib() if use_c else None
    if lib is not None:
        lib.oracle_delta_rule_seq(q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(),
                                  out.data_ptr(), B, H, L, Dk, Dv)
        return out
    qn, kn, vn, gn, bn = (t.numpy() for t in (q, k, v, g, beta))
    on = out.numpy()
    for b in range(B):
        for h in range(H):
            S = np.zeros((Dk, Dv), dtype=np.float32)
            for t in range(L):
                S *= np.exp(gn[b, h, t]).astype(np.float32)
                r = kn[b, h, t] @ S
                d = (vn[b, h, t] - r) * bn[b, h, t]
                S += np.outer(kn[b, h, t], d).astype(np.float32)
                on[b, t, h] = qn[b, h, t] @ S
    return out


def chunked_delta_rule(q, k, v, g, beta, chunk: int = 32) -> torch.Tensor:
    """`chunked_delta_rule_fallback` (src/archs/qwen35_text.rs:809-880), op for op."""
    q, k, v, g, beta = (t.detach().to(torch.float32).cpu() for t in (q, k, v, g, beta))
    B, H, L, Dk = q.shape
    Dv = v.shape[-1]
    state = torch.zeros((B, H, Dk, Dv), dtype=torch.float32)
    outs = []
    for start in range(0, L, chunk):
        n = min(chunk, L - start)
        qi, ki, vi = q[:, :, start:start + n], k[:, :, start:start + n], v[:, :, start:start + n]
        bi = beta[:, :, start:start + n].unsqueeze(3)
        gi = g[:, :, start:start + n].cumsum(2)
        lower = torch.tril(torch.ones(n, n))
        eye = torch.eye(n)
        strict = lower - eye
        decay = ((gi.unsqueeze(3) - gi.unsqueeze(2)) * lower).exp() * lower
        kb, vb = ki * bi, vi * bi
        gexp = gi.exp()
        l = -((kb @ ki.transpose(-1, -2)) * decay * strict)
        inverse = l + eye
        power = l
        covered = 2
        while covered < n:
            power = power @ power
            inverse = inverse + power @ inverse
            covered *= 2
        value = inverse @ vb
        kcd = inverse @ (kb * gexp.unsqueeze(3))
        vnew = value - kcd @ state
        attn = (qi @ ki.transpose(-1, -2)) * decay
        inter = (qi * gexp.unsqueeze(3)) @ state
        outs.append(inter + attn @ vnew)
        last = gi[:, :, n - 1:n]
        upd = (ki * (last - gi).exp().unsqueeze(3)).transpose(-1, -2) @ vnew
        state = state * last.exp().unsqueeze(3) + upd
    return torch.cat(outs, 2).transpose(1, 2).contiguous()


def causal_conv_silu(x, weight, dtype: str = "bf16") -> torch.Tensor:
    """`causal_conv_silu` (src/archs/qwen35_text.rs:632-650; CUDA kernel src/kernels/qwen35.cu:3-29): depthwise
    causal conv over `x [B, L, C]` with `weight [C, 1, taps]` (zero left padding per batch row), then SiLU. In
    "bf16" the running sum and each product are rounded to bf16 tap by tap, as both reference paths do."""
    x = x.to(torch.float32)
    B, L, Cc = x.shape
    w = weight.to(torch.float32).reshape(Cc, -1)
    taps = w.shape[1]
    rnd = (lambda t: t.to(torch.bfloat16).to(torch.float32)) if dtype == "bf16" else (lambda t: t)
    padded = torch.nn.functional.pad(x, (0, 0, taps - 1, 0))
    mixed = torch.zeros_like(x)
    for tap in range(taps):
        mixed = rnd(mixed + rnd(padded[:, tap:tap + L] * w[:, tap].reshape(1, 1, Cc)))
    return rnd(mixed / (1.0 + torch.exp(-mixed)))


def delta_inputs(mixed, b_proj, a_proj, dt_bias, neg_exp_a, key_heads: int, value_heads: int, key_dim: int,
                 value_dim: int) -> Tuple[torch.Tensor, ...]:
    """`LinearAttention::delta_inputs` (src/archs/qwen35_text.rs:528-579) for `mixed [B, L, 2Kw+Vw]` (already
    through conv+SiLU), `b_proj`, `a_proj` `[B, L, Hv]`. Returns q, k, v, g, beta in `[B, H, L, ·]` f32."""
    B, L, _ = mixed.shape
    kw, vw = key_heads * key_dim, value_heads * value_dim
    q = mixed[..., :kw].reshape(B, L, key_heads, key_dim)
    k = mixed[..., kw:2 * kw].reshape(B, L, key_heads, key_dim)
    v = mixed[..., 2 * kw:2 * kw + vw].reshape(B, L, value_heads, value_dim)
    rep = value_heads // key_heads
    q = q.unsqueeze(3).expand(B, L, key_heads, rep, key_dim).reshape(B, L, value_heads, key_dim)
    k = k.unsqueeze(3).expand(B, L, key_heads, rep, key_dim).reshape(B, L, value_heads, key_dim)

    def l2(t):
        return t / (t.square().sum(-1, keepdim=True) + 1e-6).sqrt()

    q = l2(q.to(torch.float32)) * (key_dim ** -0.5)
    k = l2(k.to(torch.float32))
    v = v.to(torch.float32)
    beta = torch.sigmoid(b_proj.to(torch.float32))
    gi = a_proj.to(torch.float32) + dt_bias.to(torch.float32)
    softplus = torch.relu(gi) + torch.log(torch.exp(-gi.abs()) + 1.0)
    g = softplus * neg_exp_a.to(torch.float32)
    return (q.transpose(1, 2).contiguous(), k.transpose(1, 2).contiguous(), v.transpose(1, 2).contiguous(),
            g.transpose(1, 2).contiguous(), beta.transpose(1, 2).contiguous())


def finish_delta(o, z, norm_weight, eps: float, out_bf16: bool = True) -> torch.Tensor:
    """The part of `finish_delta` before out_proj (src/archs/qwen35_text.rs:605-626): per-head RMS norm with
    `weight` (not 1+weight), times SiLU(z), cast to the model dtype. o `[B, L, H, Dv]` f32, z `[B, L, H*Dv]`."""
    B, L, H, Dv = o.shape
    gate = z.reshape(B, L, H, Dv).to(torch.float32)
    var = o.square().mean(-1, keepdim=True)
    y = o / (var + eps).sqrt() * norm_weight.to(torch.float32)
    y = y * (gate / (1.0 + torch.exp(-gate)))
    y = y.reshape(B, L, H * Dv)
    return y.to(torch.bfloat16).to(torch.float32) if out_bf16 else y
