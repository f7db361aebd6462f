#!/usr/bin/env python
"""Benchmark of the projection hot path: the four ModernBERT-base projections with their fused epilogues over a
token-packed ragged batch (sequence lengths uniform in [16, 512] packed to a 32768-token budget).

One step = one pass of the path over one batch, chained as in a layer (x is the residual stream, updated in place):
    qkv = x Wqkv^T                      (768 -> 2304)
    x  += attn Wo^T                     (768 -> 768, residual fused)
    m   = geglu(x Wi^T)                 (768 -> 2 x 1152, GeGLU fused)
    x  += m Wout^T                      (1152 -> 768, residual fused)
Work counted per step: 2 * T * sum(K * N) flops (epilogue flops not counted).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--tokens T] [--impl reference]

Under torchrun (N > 1) every rank runs the same workload on its own GPU (independent replicas, no collective on
the data path); the reported value is the whole-job rate: N * work / max-over-ranks time.
`--impl reference` times the CPU oracle (the restatement of the reference's CPU path) on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# ModernBERT-base projections: (name, K, N rows of the weight, output width, epilogue)
HIDDEN, QKV, INTER = 768, 2304, 1152
PROJECTIONS = [
    ("wqkv", HIDDEN, QKV, QKV, "none"),
    ("wo+residual", HIDDEN, HIDDEN, HIDDEN, "residual"),
    ("wi+geglu", HIDDEN, 2 * INTER, INTER, "geglu"),
    ("mlp_out+residual", INTER, HIDDEN, HIDDEN, "residual"),
]
FLOPS_PER_TOKEN = sum(2 * k * n for _, k, n, _, _ in PROJECTIONS)  # 10,027,008
SEED = 1002
# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) per launch at T = 32768, from the ncu capture
# summarised in profiles/gemm_projections_T32768.md (scaled by T / 32768 for other sizes).
NCU_TRAFFIC_BYTES = {"wi+geglu": 88_296_704, "wqkv": 151_915_520, "wo+residual": 107_385_088,
                     "mlp_out+residual": 142_664_448}
FALLBACK_PEAK_TFLOPS = 1590.0


def algorithmic_bytes(name: str, T: int) -> int:
    for n, k, nw, nout, epi in PROJECTIONS:
        if n == name:
            b = 2 * (T * k + k * nw + T * nout)
            return b + (2 * T * nout if epi == "residual" else 0)
    raise KeyError(name)


def make_weights(device, dtype):
    g = torch.Generator().manual_seed(SEED)
    mk = lambda n, k: (torch.randn(n, k, generator=g) * 0.02).to(dtype).to(device)
    return {"wqkv": mk(QKV, HIDDEN), "wo": mk(HIDDEN, HIDDEN), "wi": mk(2 * INTER, HIDDEN), "wout": mk(HIDDEN, INTER)}


def measured_peak():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            d = json.loads(path.read_text())
            return float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
        except Exception:
            pass
    return FALLBACK_PEAK_TFLOPS, 1400.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-i", str(self.index), "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self, t0: float, t1: float):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.12)
        self.proc.terminate()
        rows = [r for t, r in self.rows if t0 - 0.05 <= t <= t1 + 0.1 and len(r) >= 6] or [r for _, r in self.rows if len(r) >= 6]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        mhz = sorted(int(r[0]) for r in rows if r[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": int(rows[0][1]) if rows[0][1].isdigit() else None,
                "reasons": reasons, "samples": len(rows)}


def run_cpu_arm(tokens: int, steps: int, warmup: int, budget_s: float = 20.0):
    """The oracle's CPU path (f32, all host threads) on a bounded sample of the same workload: `tokens` rows."""
    import oracle
    # torchrun pins OMP_NUM_THREADS=1; the CPU arm is meant to use every core the process may run on
    torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    torch.manual_seed(SEED)
    W = {k: v.float() for k, v in make_weights("cpu", torch.float32).items()}
    g = torch.Generator().manual_seed(SEED + 1)
    x = torch.randn(tokens, HIDDEN, generator=g)
    attn = torch.randn(tokens, HIDDEN, generator=g)

    def step():
        qkv = oracle.linear(x, W["wqkv"], dtype="f32")
        h = oracle.linear(attn, W["wo"], residual=x, dtype="f32")
        m = oracle.geglu(oracle.linear(h, W["wi"], dtype="f32"), dtype="f32")
        return qkv, oracle.linear(m, W["wout"], residual=h, dtype="f32")

    for _ in range(max(1, warmup)):
        step()
    times = []
    t_start = time.perf_counter()
    for _ in range(steps):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - t_start > budget_s:
            break
    dt = sum(times) / len(times)
    return FLOPS_PER_TOKEN * tokens / dt / 1e12, dt, len(times), torch.get_num_threads()


def run_encoder(args, rank, world, local_rank):
    """Secondary workload: ModernBERT-large-shaped encoder forward (28 layers, hidden 1024, 16 heads, GeGLU 2 x 2624,
    window 128, global every 3rd layer) over packed batches of `--tokens` tokens with log-uniform lengths in
    [8, 8192], one replica per GPU. Every stage goes through the C ABI: embedding lookup + norm, per layer norm, Wqkv,
    RoPE in place, attention, Wo + residual, norm, Wi + GeGLU, MLP-out + residual. The line also times one global
    and one banded attention launch on the same batch (`attention`: microseconds and algorithmic TFLOP/s, counting
    4 x head_dim flops per query-key pair inside the band)."""
    from types import SimpleNamespace
    from sys1_b200 import batching, device, modernbert
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=dev)
    cfg = SimpleNamespace(vocab_size=50368, hidden_size=1024, num_hidden_layers=28, num_attention_heads=16, intermediate_size=2624,
                          layer_norm_eps=1e-5, global_attn_every_n_layers=3, local_attention=128, global_rope_theta=160000.0,
                          local_rope_theta=10000.0)
    g = torch.Generator(device=dev).manual_seed(1003)
    mk = lambda *shape: (torch.randn(*shape, device=dev, generator=g) * 0.02).to(torch.bfloat16)
    w = {"tok_embeddings": mk(cfg.vocab_size, cfg.hidden_size), "embeddings_norm": torch.ones(cfg.hidden_size, device=dev, dtype=torch.bfloat16),
         "final_norm": torch.ones(cfg.hidden_size, device=dev, dtype=torch.bfloat16)}
    for i in range(cfg.num_hidden_layers):
        p = f"layers.{i}."
        w[p + "Wqkv"], w[p + "Wo"] = mk(3 * cfg.hidden_size, cfg.hidden_size), mk(cfg.hidden_size, cfg.hidden_size)
        w[p + "Wi"], w[p + "mlp_Wo"] = mk(2 * cfg.intermediate_size, cfg.hidden_size), mk(cfg.hidden_size, cfg.intermediate_size)
        w[p + "attn_norm"] = torch.ones(cfg.hidden_size, device=dev, dtype=torch.bfloat16)
        w[p + "mlp_norm"] = torch.ones(cfg.hidden_size, device=dev, dtype=torch.bfloat16)
    enc = modernbert.Encoder(w, cfg)
    ctx = device.load(local_rank)
    T = args.tokens
    lens = batching.synthetic_lengths(1003 + rank, 8, 8192, T, log_uniform=True)
    batch, _ = batching.pack_next(lens, batching.BatcherConfig(token_budget=T))
    ids = torch.randint(0, cfg.vocab_size, (T,), device=dev, generator=g)
    pos = torch.from_numpy(batch.positions).to(dev)
    warmup, steps = max(args.warmup, 3), min(args.steps, 20)
    for _ in range(warmup):
        enc.forward(ids, batch.cu_seqlens, pos)
    ctx.sync()
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()
    l0 = ctx.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        enc.forward(ids, batch.cu_seqlens, pos)
    e1.record()
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    launches = ctx.launch_count() - l0
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms = float(t[0])
    # end to end through the public call: token ids and positions from pinned host memory every step, final hidden states
    # back to pinned host memory every step (copies on side streams, overlapped with the previous / next step)
    from sys1_b200 import pipeline
    host_ids = ids.to(torch.int32).cpu().pin_memory()
    host_pos = pos.to(torch.int32).cpu().pin_memory()
    host_out = torch.empty(T, cfg.hidden_size, dtype=torch.bfloat16).pin_memory()
    pipe = pipeline.HostPipeline(dev, [(T,), (T,)], torch.int32, depth=2)
    fwd = lambda bufs: enc.forward(bufs[0], batch.cu_seqlens, bufs[1])
    for _ in range(2):
        pipe.submit([host_ids, host_pos], host_out, fwd)
    pipe.drain()
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()
    import time as _time
    t0 = _time.perf_counter()
    for _ in range(steps):
        pipe.submit([host_ids, host_pos], host_out, fwd)
    pipe.drain()
    ms_e2e = (_time.perf_counter() - t0) * 1e3 / steps
    if world > 1:
        t = torch.tensor([ms_e2e], device=dev, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms_e2e = float(t[0])
    H, D = cfg.num_attention_heads, cfg.hidden_size // cfg.num_attention_heads
    qkv = mk(3, T, H * D)
    attn_stats = {}
    for name, window in (("global", -1), ("local", cfg.local_attention // 2)):
        out = torch.empty(T, H * D, device=dev, dtype=torch.bfloat16)
        for _ in range(3):
            modernbert.attention_varlen(qkv[0].view(T, H, D), qkv[1].view(T, H, D), qkv[2].view(T, H, D), batch.cu_seqlens,
                                        window=window, out=out)
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for _ in range(10):
            modernbert.attention_varlen(qkv[0].view(T, H, D), qkv[1].view(T, H, D), qkv[2].view(T, H, D), batch.cu_seqlens,
                                        window=window, out=out)
        a1.record()
        torch.cuda.synchronize()
        us = a0.elapsed_time(a1) * 100.0
        pairs = 0
        for n in lens:
            n = int(n)
            pairs += n * n if window < 0 or n <= window else n * (2 * window + 1) - window * (window + 1)
        attn_stats[name] = {"us": us, "tflops": 4.0 * D * H * pairs / (us * 1e-6) / 1e12}
    if rank == 0:
        flops_tok = 28 * 2 * (1024 * 3072 + 1024 * 1024 + 1024 * 5248 + 2624 * 1024)
        print(json.dumps({"metric": "encoder tokens/s", "value": world * T / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
                          "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
                          "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                          "config": {"workload": f"ModernBERT-large-shaped encoder forward, packed T={T}, lengths log-uniform [8,8192], "
                                                 "every stage through the C ABI (projections, attention, norms, RoPE, embedding lookup)",
                                     "sequences": int(len(lens)), "parallelism": f"replicas x{world}"},
                          "projection_tflops": world * T * flops_tok / (ms * 1e-3) / 1e12, "attention": attn_stats,
                          "e2e": {"value": world * T / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                                  "h2d_bytes_per_step": 8 * T, "d2h_bytes_per_step": 2 * T * cfg.hidden_size},
                          "gpu_launches": launches}))
    if world > 1:
        torch.distributed.destroy_process_group()


def run_decoder(args, rank, world, local_rank):
    """Secondary workload: Qwen3.5-small-shaped hybrid decoder forward (24 layers = (linear, linear, linear, full) x 6,
    hidden 1024, 16 x 128 delta-rule heads, conv 4, full attention 8 query / 2 KV heads x 256, SwiGLU 3584) over a
    packed batch of `--tokens` tokens (default here 16384) with lengths uniform in [64, 2048], one replica per GPU.
    Every stage goes through the C ABI."""
    from types import SimpleNamespace
    from sys1_b200 import batching, device, qwen35
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=dev)
    cfg = SimpleNamespace(vocab_size=151936, hidden_size=1024, intermediate_size=3584, num_hidden_layers=24, num_attention_heads=8,
                          num_key_value_heads=2, head_dim=256, rms_norm_eps=1e-6, rope_theta=1e7, rotary_dim=64,
                          linear_num_key_heads=16, linear_num_value_heads=16, linear_key_head_dim=128, linear_value_head_dim=128,
                          linear_conv_kernel_dim=4, layer_type=lambda i: "full_attention" if (i + 1) % 4 == 0 else "linear_attention")
    g = torch.Generator(device=dev).manual_seed(1004)
    mk = lambda *shape, s=0.02: (torch.randn(*shape, device=dev, generator=g) * s).to(torch.bfloat16)
    H, KV, D, Hk, Hv = 8, 2, 256, 16, 16
    w = {"embed_tokens": mk(cfg.vocab_size, cfg.hidden_size, s=1.0), "norm": mk(cfg.hidden_size, s=0.1)}
    for i in range(cfg.num_hidden_layers):
        p = f"layers.{i}."
        w[p + "input_layernorm"], w[p + "post_attention_layernorm"] = mk(1024, s=0.1), mk(1024, s=0.1)
        w[p + "mlp.gate_proj"], w[p + "mlp.up_proj"], w[p + "mlp.down_proj"] = mk(3584, 1024), mk(3584, 1024), mk(1024, 3584)
        if cfg.layer_type(i) == "full_attention":
            a = p + "self_attn."
            w[a + "q_proj"], w[a + "k_proj"], w[a + "v_proj"], w[a + "o_proj"] = mk(H * D * 2, 1024), mk(KV * D, 1024), mk(KV * D, 1024), mk(1024, H * D)
            w[a + "q_norm"], w[a + "k_norm"] = mk(D, s=0.1), mk(D, s=0.1)
        else:
            a = p + "linear_attn."
            width = 2 * Hk * 128 + Hv * 128
            w[a + "in_proj_qkv"], w[a + "in_proj_z"] = mk(width, 1024), mk(Hv * 128, 1024)
            w[a + "in_proj_b"], w[a + "in_proj_a"] = mk(Hv, 1024, s=0.1), mk(Hv, 1024, s=0.1)
            w[a + "conv1d"] = mk(width, 1, 4, s=0.3)
            w[a + "A_log"] = torch.randn(Hv, device=dev, generator=g) * 0.5
            w[a + "dt_bias"] = torch.randn(Hv, device=dev, generator=g) * 0.5
            w[a + "norm"] = (1.0 + torch.randn(128, device=dev, generator=g) * 0.1).to(torch.bfloat16)
            w[a + "out_proj"] = mk(1024, Hv * 128)
    dec = qwen35.Decoder(w, cfg)
    ctx = device.load(local_rank)
    T = args.tokens if args.tokens != 32768 else 16384
    lens = batching.synthetic_lengths(1004 + rank, 64, 2048, T)
    batch, _ = batching.pack_next(lens, batching.BatcherConfig(token_budget=T))
    ids = torch.randint(0, cfg.vocab_size, (T,), device=dev, generator=g)
    pos = torch.from_numpy(batch.positions).to(dev)
    warmup, steps = max(args.warmup, 3), min(args.steps, 20)
    for _ in range(warmup):
        dec.forward(ids, batch.cu_seqlens, pos)
    ctx.sync()
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()
    l0 = ctx.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        dec.forward(ids, batch.cu_seqlens, pos)
    e1.record()
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms = float(t[0])
    ctx.sync()
    if rank == 0:
        flops_tok = 18 * 43_057_152 + 6 * 36_700_160  # projection flops per token: linear-attention / full-attention layers
        print(json.dumps({"metric": "decoder tokens/s", "value": world * T / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
                          "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
                          "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                          "config": {"workload": f"Qwen3.5-small-shaped hybrid decoder forward, packed T={T}, lengths U[64,2048], "
                                                 "every stage through the C ABI",
                                     "sequences": int(len(lens)), "parallelism": f"replicas x{world}"},
                          "projection_tflops": world * T * flops_tok / (ms * 1e-3) / 1e12,
                          "gpu_launches": ctx.launch_count() - l0}))
    if world > 1:
        torch.distributed.destroy_process_group()


def run_tp(args, rank, world, local_rank):
    """Secondary workload: the SwiGLU MLP of the 27B-shaped hybrid model (hidden 5120, intermediate 17408) on
    `--tokens` packed tokens, tensor-parallel over the ranks: gate / up column-parallel with the gating fused,
    down row-parallel with the residual fused on rank 0, the whole MLP in `--slabs` row slabs whose partial sums are
    exchanged by `s1_allreduce_bf16` under the projections of the next slab. Reports whole-job TFLOP/s, the
    same step without the exchange, and the bus bandwidth of the bare all-reduce of the full [T, 5120] output."""
    from sys1_b200 import device, tensor_parallel
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    H, I, T = 5120, 17408, args.tokens
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=dev)
        tp = tensor_parallel.TensorParallel.from_process_group(local_rank, comm_ctas=args.comm_ctas)
    else:
        tp = tensor_parallel.TensorParallel(device.load(local_rank), 0, 1)
    ctx = tp.ctx
    g = torch.Generator(device=dev).manual_seed(1005)
    mk = lambda *shape: (torch.randn(*shape, device=dev, generator=g) * 0.02).to(torch.bfloat16)
    # every rank builds only its own shard (same seed on all ranks: the full matrices would be identical)
    gate, up, down = mk(I // world, H), mk(I // world, H), mk(H, I // world)
    x = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
    out = torch.empty(T, H, device=dev, dtype=torch.bfloat16)
    mlp = tensor_parallel.Mlp(gate, up, down, tp, slabs=args.slabs, sharded=True, comm_sms=args.comm_sms)

    def step(exchange=True):
        mlp.forward(x, residual=x, out=out, exchange=exchange)

    def timed(fn, n):
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / n
        if world > 1:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            ms = float(t[0])
        return ms

    warmup, steps = max(args.warmup, 3), min(args.steps, 20)
    for _ in range(warmup):
        step()
    l0 = ctx.launch_count()
    ms = timed(step, steps)
    launches = ctx.launch_count() - l0
    ms_math = timed(lambda: step(False), steps)
    ms_ar = timed(lambda: ctx.all_reduce_(out), steps) if world > 1 else 0.0
    ctx.sync()
    if rank == 0:
        flops = 6.0 * T * H * I
        bytes_ar = T * H * 2
        print(json.dumps({"metric": "tensor-parallel MLP TFLOP/s", "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world,
                          "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
                          "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                          "config": {"workload": f"27B-shaped SwiGLU MLP (5120 -> 2 x 17408 -> 5120), T={T}, tensor parallel x{world}, "
                                                 f"gate/up, down and all-reduce in {args.slabs} row slabs, {args.comm_sms} SMs left to the all-reduce ({args.comm_ctas or 'default'} blocks)", "parallelism": f"tp{world}",
                                     "l2": "activations (x, h, out) exceed the 126 MB L2"},
                          "ms_without_exchange": ms_math, "ms_allreduce_alone": ms_ar,
                          "allreduce_busbw_gbs": (2.0 * (world - 1) / world * bytes_ar / (ms_ar * 1e-3) / 1e9) if world > 1 else None,
                          "exchange_hidden_frac": (1.0 - (ms - ms_math) / ms_ar) if world > 1 and ms_ar > 0 else None,
                          "gpu_launches": launches}))
    if world > 1:
        torch.distributed.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--cpu-sample-tokens", type=int, default=8192)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="projections", choices=["projections", "encoder", "decoder", "tp"],
                    help="projections (default, the headline microbench); encoder: ModernBERT-large forward, tokens/s; "
                         "tp: SwiGLU MLP of the 27B-shaped hybrid model, tensor-parallel over the ranks")
    ap.add_argument("--slabs", type=int, default=4, help="tp workload: row slabs the all-reduce is pipelined in")
    ap.add_argument("--comm-ctas", type=int, default=0, help="tp workload: blocks the all-reduce may use (0 = NCCL's default)")
    ap.add_argument("--comm-sms", type=int, default=16, help="tp workload: SMs the projections leave to the all-reduce of the previous slab")
    ap.add_argument("--graph", action="store_true",
                    help="replay each step from a CUDA graph (for small token budgets, where launching from Python is the bottleneck)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    T = args.tokens
    warmup = max(args.warmup, 3)
    config = {"workload": f"ModernBERT-base projection microbench, packed ragged batch, T={T} tokens "
                          "(lengths U[16,512]), Wqkv / Wo+residual / Wi+GeGLU / MLP-out+residual",
              "tokens": T, "hidden": HIDDEN, "intermediate": INTER, "parallelism": f"replicas x{world}",
              "l2": "4 rotating input sets (400 MB) + 226 MB of outputs per step exceed the 126 MB L2",
              "launch": "cuda graph replay" if args.graph else "eager",
              "timing": "K steps back to back between two events; per-kernel durations from 40 back-to-back launches of each "
                        "projection on the same rotating buffers between two events of their own",
              "residual": "in place (x += ...); alternate visits of a buffer use -Wo / -Wout to keep the stream bounded"}

    if args.impl == "reference":
        # rank 0 alone runs the CPU arm; the other ranks leave without work
        if rank != 0:
            return
        val, dt, n, cores = run_cpu_arm(args.cpu_sample_tokens, max(1, args.steps), warmup, budget_s=60.0)
        line = {"impl": "reference", "metric": "projection GEMM TFLOP/s", "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
                "steps": n, "warmup": warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
                "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                 "sample": f"{args.cpu_sample_tokens} of the {T} packed token rows per step, same four projections, "
                                           "torch CPU f32 oracle (restatement of the reference's candle CPU path; the Rust "
                                           "reference itself cannot be built here: no cargo/rustc)"},
                "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    if args.workload == "encoder" and args.impl != "reference":
        return run_encoder(args, rank, world, local_rank)
    if args.workload == "decoder" and args.impl != "reference":
        return run_decoder(args, rank, world, local_rank)
    if args.workload == "tp" and args.impl != "reference":
        return run_tp(args, rank, world, local_rank)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: there is no CPU fallback for the product path (use --impl reference for the CPU arm)")
    from sys1_b200 import batching, device, linear, modernbert
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    ctx = device.load(local_rank)

    # the batch: packed layout from the batcher (the projections ignore sequence boundaries, attention would not)
    lens = batching.synthetic_lengths(SEED + rank, 16, 512, T)
    batch, taken = batching.pack_next(lens, batching.BatcherConfig(token_budget=T))
    assert batch.total_tokens == T and taken == len(lens)
    W = make_weights(dev, torch.bfloat16)
    proj = modernbert.AttentionProjections(linear.linear_no_bias(W["wqkv"]), linear.linear_no_bias(W["wo"]))
    mlp = modernbert.Mlp(linear.linear_no_bias(W["wi"]), linear.linear_no_bias(W["wout"]))
    pos_proj, pos_mlp = proj, mlp

    NSETS = 4
    g = torch.Generator().manual_seed(SEED + 100 + rank)
    host_x = [torch.randn(T, HIDDEN, generator=g).to(torch.bfloat16).pin_memory() for _ in range(NSETS)]
    host_a = [torch.randn(T, HIDDEN, generator=g).to(torch.bfloat16).pin_memory() for _ in range(NSETS)]
    xs = [t.to(dev) for t in host_x]
    atts = [t.to(dev) for t in host_a]
    bf = dict(dtype=torch.bfloat16, device=dev)
    qkv, m = (torch.empty(T, n, **bf) for n in (QKV, INTER))
    host_y = [torch.empty(T, HIDDEN, dtype=torch.bfloat16).pin_memory() for _ in range(2)]

    ev = lambda: torch.cuda.Event(enable_timing=True)
    names = [p[0] for p in PROJECTIONS]

    # the device-resident arm keeps updating the same few residual-stream buffers in place; every other visit of a
    # buffer uses -Wo / -Wout (same work, opposite sign) so that the stream stays at its N(0, 1) scale instead of
    # growing step after step
    neg_proj = modernbert.AttentionProjections(proj.wqkv, linear.linear_no_bias(-W["wo"]))
    neg_mlp = modernbert.Mlp(mlp.input, linear.linear_no_bias(-W["wout"]))

    def step(x, a, negate=False):
        proj, mlp = (neg_proj, neg_mlp) if negate else (pos_proj, pos_mlp)
        proj.wqkv.forward(x, out=qkv)
        proj.wo.forward(a, residual=x, out=x)
        linear.fused_linear(x, mlp.input.weight, epilogue=linear.EPI_GEGLU, out=m)
        mlp.output.forward(m, residual=x, out=x)
        return x

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    # ---- device-resident arm ---------------------------------------------------------------------------------
    for i in range(2 * NSETS * ((warmup + 2 * NSETS - 1) // (2 * NSETS))):  # whole +/- cycles
        step(xs[i % NSETS], atts[i % NSETS], negate=bool((i // NSETS) & 1))
    ctx.sync()
    graphs = None
    if args.graph:
        # one graph per (buffer set, sign): the launches of a step with their tensor maps baked in
        cap = torch.cuda.Stream(dev)
        with torch.cuda.stream(cap):
            cap_ctx = device.load(local_rank)  # context of the capture stream, created before any capture
            step(xs[0], atts[0])
            cap_ctx.sync()
        graphs = {}
        for s_ in range(NSETS):
            for neg in (False, True):
                g_ = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g_, stream=cap):
                    step(xs[s_], atts[s_], negate=neg)
                graphs[(s_, neg)] = g_
        torch.cuda.synchronize()
    # per-kernel durations: each projection launched back to back on the rotating buffer sets between two events of its
    # own (an event between every two launches of a step would itself cost several microseconds per launch and keep
    # a projection's set-up from overlapping its predecessor's tail, which is what the timed loop below benefits from);
    # taken before the timed loop, each kernel on its own, so the burst peak is the matching denominator
    def one(name, i):
        x, a, neg = xs[i % NSETS], atts[i % NSETS], bool((i // NSETS) & 1)
        pj, ml = (neg_proj, neg_mlp) if neg else (pos_proj, pos_mlp)
        if name == "wqkv":
            pj.wqkv.forward(x, out=qkv)
        elif name == "wo+residual":
            pj.wo.forward(a, residual=x, out=x)
        elif name == "wi+geglu":
            linear.fused_linear(x, ml.input.weight, epilogue=linear.EPI_GEGLU, out=m)
        else:
            ml.output.forward(m, residual=x, out=x)

    per, reps = {}, 2 * NSETS * 5
    for n in names:
        for i in range(2 * NSETS):
            one(n, i)
        k0, k1 = ev(), ev()
        k0.record()
        for i in range(reps):
            one(n, i)
        k1.record()
        torch.cuda.synchronize()
        per[n] = k0.elapsed_time(k1) / reps

    launches0 = ctx.launch_count()
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.15)
    barrier()
    t0w = time.time()
    e0, e1 = ev(), ev()
    e0.record()
    for i in range(args.steps):
        if graphs is not None:
            graphs[(i % NSETS, bool((i // NSETS) & 1))].replay()
        else:
            step(xs[i % NSETS], atts[i % NSETS], negate=bool((i // NSETS) & 1))
    e1.record()
    barrier()
    t1w = time.time()
    ctx.sync()
    launches = ctx.launch_count() - launches0
    ms_total = e0.elapsed_time(e1)
    if graphs is not None:
        launches = 4 * args.steps  # replayed from the graphs (4 kernel nodes each), not counted by the context
    # ---- end-to-end arm: host buffers in, host buffer out, copies inside the timed region ----------------------
    # (copy-in of batch i+1 and copy-out of batch i-1 overlap the compute of batch i: sys1_b200.pipeline)
    from sys1_b200.pipeline import HostPipeline
    pipe = HostPipeline(dev, [(T, HIDDEN), (T, HIDDEN)], torch.bfloat16, depth=2)

    def e2e_step(i):
        pipe.submit([host_x[i % NSETS], host_a[i % NSETS]], host_y[i % 2], lambda bufs: step(bufs[0], bufs[1]))

    e2e_steps = max(3, min(args.steps, 40))
    for i in range(3):
        e2e_step(i)
    pipe.drain()
    barrier()
    f0, f1 = ev(), ev()
    f0.record()
    for i in range(e2e_steps):
        e2e_step(i)
    pipe.drain()
    f1.record()
    barrier()
    clocks = sampler.stop(t0w, t1w)
    ctx.sync()
    ms_e2e = f0.elapsed_time(f1)

    ms_step, ms_step_e2e = ms_total / args.steps, ms_e2e / e2e_steps
    if world > 1:
        t = torch.tensor([ms_step, ms_step_e2e], device=dev, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms_step, ms_step_e2e = float(t[0]), float(t[1])
    flops_step = FLOPS_PER_TOKEN * T
    value = world * flops_step / (ms_step * 1e-3) / 1e12
    e2e_value = world * flops_step / (ms_step_e2e * 1e-3) / 1e12

    if rank == 0:
        burst, sustained, peak_kind = measured_peak()
        dom = max(per, key=per.get)
        dom_proj = next(p for p in PROJECTIONS if p[0] == dom)
        dom_flops = 2 * T * dom_proj[1] * dom_proj[2]
        achieved = dom_flops / (per[dom] * 1e-3) / 1e12
        # a kernel timed alone between events in a run of a few tens of milliseconds: the burst figure applies
        line = {"metric": "projection GEMM TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
                "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "bf16", "data": "synthetic", "config": config,
                "roofline": {"bound": "tensor", "kernel": f"s1_gemm_kernel ({dom})", "achieved": achieved, "peak": burst,
                             "unit": "TFLOP/s", "frac": achieved / burst, "peak_source": f"{peak_kind} bf16 burst",
                             "frac_of_sustained": achieved / sustained, "flops_per_launch": dom_flops,
                             "us_per_launch": per[dom] * 1e3, "algorithmic_bytes": algorithmic_bytes(dom, T),
                             "traffic": (NCU_TRAFFIC_BYTES[dom] * T // 32768) if dom in NCU_TRAFFIC_BYTES else None},
                "per_projection": {n: {"us": per[n] * 1e3,
                                       "tflops": 2 * T * p[1] * p[2] / (per[n] * 1e-3) / 1e12,
                                       "gbs": algorithmic_bytes(n, T) / (per[n] * 1e-3) / 1e9}
                                   for n, p in zip(names, PROJECTIONS)},
                "e2e": {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": ms_step_e2e,
                        "h2d_bytes_per_step": 2 * T * HIDDEN * 2, "d2h_bytes_per_step": T * HIDDEN * 2},
                "gpu_launches": launches, "clocks": clocks}
        if not args.no_cpu_baseline:
            val, dt, n, cores = run_cpu_arm(args.cpu_sample_tokens, 1000, 1, budget_s=12.0)
            line["cpu_baseline"] = {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                    "sample": f"{args.cpu_sample_tokens} of the {T} token rows, same four projections, "
                                              f"torch CPU f32 oracle, {n} timed passes"}
        print(json.dumps(line))
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
