#!/usr/bin/env python
"""Benchmark of the projection hot path: the four ModernBERT-base projections with their fused epilogues over a
token-packed ragged batch (sequence lengths uniform in [16, 512] packed to a 32768-token budget).

One step = one pass of the path over one batch, chained as in a layer (x is the residual stream, updated in place):
    qkv = x Wqkv^T                      (768 -> 2304)
    x  += attn Wo^T                     (768 -> 768, residual fused)
    m   = geglu(x Wi^T)                 (768 -> 2 x 1152, GeGLU fused)
    x  += m Wout^T                      (1152 -> 768, residual fused)
Work counted per step: 2 * T * sum(K * N) flops (epilogue flops not counted).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--tokens T] [--impl reference] [--workload ...]

`metric` / `value` of the printed line are that microbenchmark. The same line carries, as blocks of their own:
  sustained  the same chain run back to back for at least two seconds, with the SM clock sampled under load
  budgets    the chain at the 2048- and 8192-token budgets (CUDA-graph replay and eager), TFLOP/s and algorithmic GB/s
  gpu_lib    the four contractions as plain library GEMMs (torch.matmul -> cuBLAS) without any epilogue
  encoder    ModernBERT-large-shaped encoder forward over a packed 32768-token batch, tokens/s, with its own e2e
  decoder    Qwen3.5-small-shaped hybrid decoder forward over a packed 16384-token batch, tokens/s
  tp         a (linear, linear, linear, full) layer group of the 27B-shaped hybrid model over a packed 65536-token batch,
             tensor-parallel over the ranks (one rank: unsharded), with the exchange timed alone and a parity field; the
             sums over ranks run as the library's own in-switch reduction kernel on symmetric memory, with the same step
             through ncclAllReduce timed beside it (`--exchange multimem | nccl | both`; `--timeline PATH` also writes one
             step's kernel timeline per rank)
Under torchrun (N > 1) the projection / encoder / decoder workloads run as independent replicas, one per GPU, with no
collective on the data path (whole-job rate = N x work / max-over-ranks time); the tp block is the one workload whose
ranks exchange data. `--impl reference` times the CPU oracle (the restatement of the reference's CPU path) on the host
cores for the workload named by `--workload`. `--workload encoder | decoder | tp` prints that block as a line of its own.
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
from types import SimpleNamespace

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
FALLBACK_PEAK_TFLOPS = 1590.0
FALLBACK_HBM_GBS = 6650.0


def algorithmic_bytes(name: str, T: int) -> int:
    for n, k, nw, nout, epi in PROJECTIONS:
        if n == name:
            b = 2 * (T * k + k * nw + T * nout)
            return b + (2 * T * nout if epi == "residual" else 0)
    raise KeyError(name)


def ncu_traffic(name: str, T: int):
    """DRAM bytes (read + write) per launch of a projection kernel, from the committed summary of an ncu capture:
    lines `name tokens bytes` in profiles/gemm_dram_traffic.txt, scaled by the token count. None if there is no entry."""
    path = ROOT / "profiles" / "gemm_dram_traffic.txt"
    if not path.exists():
        return None
    for line in path.read_text().splitlines():
        parts = line.split()
        if len(parts) >= 3 and parts[0] == name and parts[1].isdigit() and parts[2].isdigit():
            return int(parts[2]) * T // int(parts[1])
    return None


def make_weights(device, dtype):
    g = torch.Generator().manual_seed(SEED)
    mk = lambda n, k: (torch.randn(n, k, generator=g) * 0.02).to(dtype).to(device)
    return {"wqkv": mk(QKV, HIDDEN), "wo": mk(HIDDEN, HIDDEN), "wi": mk(2 * INTER, HIDDEN), "wout": mk(HIDDEN, INTER)}


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            d = json.loads(path.read_text())
            return {"burst": float(d["bf16_tflops"]), "sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                    "hbm": float(d.get("hbm_gbs", FALLBACK_HBM_GBS)), "kind": "measured"}
        except Exception:
            pass
    return {"burst": FALLBACK_PEAK_TFLOPS, "sustained": 1400.0, "hbm": FALLBACK_HBM_GBS, "kind": "fallback"}


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

    def summary(self, t0: float, t1: float):
        rows = [r for t, r in self.rows if t0 <= t <= t1 and len(r) >= 6]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples in the window"], "samples": 0}
        mhz = sorted(int(r[0]) for r in rows if r[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": int(rows[0][1]) if rows[0][1].isdigit() else None,
                "reasons": reasons, "samples": len(rows)}

    def stop(self):
        if self.proc is not None:
            time.sleep(0.12)
            self.proc.terminate()


def host_threads() -> int:
    # torchrun pins OMP_NUM_THREADS=1; the CPU arm is meant to use every core the process may run on
    n = max(1, len(os.sched_getaffinity(0)))
    torch.set_num_threads(n)
    return n


# ================================================================================================ CPU arms (oracle)
def cpu_projections(tokens: int, steps: int, warmup: int, budget_s: float):
    """The oracle's CPU path (f32, all host threads) on a bounded sample of the projection workload: `tokens` rows."""
    import oracle
    cores = host_threads()
    W = {k: v.float() for k, v in make_weights("cpu", torch.float32).items()}
    g = torch.Generator().manual_seed(SEED + 1)
    x = torch.randn(tokens, HIDDEN, generator=g)
    attn = torch.randn(tokens, HIDDEN, generator=g)

    def step():
        qkv = oracle.linear(x, W["wqkv"], dtype="f32")
        h = oracle.linear(attn, W["wo"], residual=x, dtype="f32")
        m = oracle.geglu(oracle.linear(h, W["wi"], dtype="f32"), dtype="f32")
        return qkv, oracle.linear(m, W["wout"], residual=h, dtype="f32")

    dt, n = _time_cpu(step, steps, warmup, budget_s)
    return FLOPS_PER_TOKEN * tokens / dt / 1e12, dt, n, cores


def _time_cpu(step, steps, warmup, budget_s):
    for _ in range(max(1, warmup)):
        step()
    times, t_start = [], time.perf_counter()
    for _ in range(max(1, steps)):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - t_start > budget_s:
            break
    return sum(times) / len(times), len(times)


def cpu_encoder_base(budget_s: float = 30.0):
    """The ModernBERT-base configuration whole, on the host: 22 layers, ids uniform over 50368, 8 sequences of 512, seed
    1001, f32 oracle, nothing extrapolated."""
    import oracle
    cores = host_threads()
    cfg = oracle.EncoderConfig()
    w = oracle.init_weights(cfg, 1001)
    ids = torch.randint(0, 50368, (8, 512), generator=torch.Generator().manual_seed(1001))

    def step():
        for row in ids:
            oracle.encoder_forward(row, w, cfg, dtype="f32")

    dt, n = _time_cpu(step, 5, 1, budget_s)
    return {"value": 4096 / dt, "unit": "tokens/s", "cores": cores, "kind": "port", "seconds_per_forward": dt,
            "sample": f"the whole configuration (22 layers, 8 x 512 tokens), f32 torch CPU oracle, {n} timed passes"}


def cpu_encoder(budget_s: float = 20.0):
    """ModernBERT-large-shaped oracle on the host: two layers (one global, one local) over log-uniform sequences that total
    4096 tokens, f32; tokens/s for the 28-layer model extrapolated by 14 (the layers alternate between those two kinds)."""
    import oracle
    from sys1_b200 import batching
    cores = host_threads()
    cfg = oracle.EncoderConfig(vocab_size=1024, hidden_size=1024, num_hidden_layers=2, num_attention_heads=16, intermediate_size=2624)
    w = oracle.init_weights(cfg, 1003)
    lens = batching.synthetic_lengths(1003, 8, 4096, 4096, log_uniform=True)
    g = torch.Generator().manual_seed(1003)
    seqs = [torch.randint(0, cfg.vocab_size, (int(n),), generator=g) for n in lens]

    def step():
        for ids in seqs:
            oracle.encoder_forward(ids, w, cfg, dtype="f32")

    dt, n = _time_cpu(step, 2, 1, budget_s)
    return {"value": 4096 / (dt * 14), "unit": "tokens/s", "cores": cores, "kind": "port", "seconds_per_sample": dt,
            "sample": f"2 of 28 layers (1 global + 1 local) on {len(seqs)} sequences totalling 4096 tokens, f32 torch CPU oracle, "
                      f"{n} timed passes; the 28-layer figure is that time x 14 (extrapolated)"}


def _decoder_group_weights(cfg, seed, dev, dtype):
    """Random weights of a decoder stack under the checkpoint's names, created on `dev`."""
    g = torch.Generator(device=dev).manual_seed(seed)
    mk = lambda *shape, s=0.02: (torch.randn(*shape, device=dev, generator=g) * s).to(dtype)
    H, KV, D, Hk, Hv = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.linear_num_key_heads, cfg.linear_num_value_heads
    hid, inter = cfg.hidden_size, cfg.intermediate_size
    w = {"norm": mk(hid, s=0.1)}
    if getattr(cfg, "vocab_size", 0):
        w["embed_tokens"] = mk(cfg.vocab_size, hid, s=1.0)
    for i in range(cfg.num_hidden_layers):
        p = f"layers.{i}."
        w[p + "input_layernorm"], w[p + "post_attention_layernorm"] = mk(hid, s=0.1), mk(hid, s=0.1)
        w[p + "mlp.gate_proj"], w[p + "mlp.up_proj"], w[p + "mlp.down_proj"] = mk(inter, hid), mk(inter, hid), mk(hid, inter)
        if cfg.layer_type(i) == "full_attention":
            a = p + "self_attn."
            w[a + "q_proj"], w[a + "k_proj"], w[a + "v_proj"], w[a + "o_proj"] = mk(H * D * 2, hid), mk(KV * D, hid), mk(KV * D, hid), mk(hid, H * D)
            w[a + "q_norm"], w[a + "k_norm"] = mk(D, s=0.1), mk(D, s=0.1)
        else:
            a = p + "linear_attn."
            width = 2 * Hk * 128 + Hv * 128
            w[a + "in_proj_qkv"], w[a + "in_proj_z"] = mk(width, hid), mk(Hv * 128, hid)
            w[a + "in_proj_b"], w[a + "in_proj_a"] = mk(Hv, hid, s=0.1), mk(Hv, hid, s=0.1)
            w[a + "conv1d"] = mk(width, 1, 4, s=0.3)
            w[a + "A_log"] = torch.randn(Hv, device=dev, generator=g) * 0.5
            w[a + "dt_bias"] = torch.randn(Hv, device=dev, generator=g) * 0.5
            w[a + "norm"] = (1.0 + torch.randn(128, device=dev, generator=g) * 0.1).to(dtype)
            w[a + "out_proj"] = mk(hid, Hv * 128)
    return w


def _decoder_cfg(shape: str, layers: int, vocab: int):
    lt = lambda i: "full_attention" if (i + 1) % 4 == 0 else "linear_attention"
    if shape == "small":   # Qwen3.5-small-shaped
        return SimpleNamespace(vocab_size=vocab, hidden_size=1024, intermediate_size=3584, num_hidden_layers=layers, num_attention_heads=8,
                               num_key_value_heads=2, head_dim=256, rms_norm_eps=1e-6, rope_theta=1e7, rotary_dim=64,
                               linear_num_key_heads=16, linear_num_value_heads=16, linear_key_head_dim=128, linear_value_head_dim=128,
                               linear_conv_kernel_dim=4, layer_type=lt)
    return SimpleNamespace(vocab_size=vocab, hidden_size=5120, intermediate_size=17408, num_hidden_layers=layers, num_attention_heads=24,
                           num_key_value_heads=4, head_dim=256, rms_norm_eps=1e-6, rope_theta=1e7, rotary_dim=64,
                           linear_num_key_heads=16, linear_num_value_heads=48, linear_key_head_dim=128, linear_value_head_dim=128,
                           linear_conv_kernel_dim=4, layer_type=lt)


def cpu_decoder(shape: str, tokens: int, budget_s: float = 20.0):
    """One (linear, linear, linear, full) layer group of the decoder shape on the host, f32 oracle, `tokens` packed tokens;
    tokens/s of the whole stack extrapolated by its number of groups (6 for the small shape, 16 for the 27B shape)."""
    import oracle
    from sys1_b200 import batching
    cores = host_threads()
    base = _decoder_cfg(shape, 4, 256)
    cfg = oracle.DecoderConfig(vocab_size=256, hidden_size=base.hidden_size, intermediate_size=base.intermediate_size, num_hidden_layers=4,
                               num_attention_heads=base.num_attention_heads, num_key_value_heads=base.num_key_value_heads,
                               linear_num_key_heads=base.linear_num_key_heads, linear_num_value_heads=base.linear_num_value_heads)
    w = {k: v.float() for k, v in _decoder_group_weights(base, 1004, torch.device("cpu"), torch.float32).items()}
    lo, hi = (64, 2048) if shape == "small" else (256, 8192)
    lens = batching.synthetic_lengths(1004, lo, min(hi, tokens), tokens)
    g = torch.Generator().manual_seed(1004)
    seqs = [torch.randint(0, 256, (int(n),), generator=g) for n in lens]

    def step():
        for ids in seqs:
            oracle.decoder_forward(ids, w, cfg, dtype="f32")

    dt, n = _time_cpu(step, 2, 1, budget_s)
    groups = 6 if shape == "small" else 16
    return {"value": tokens / (dt * groups), "unit": "tokens/s", "cores": cores, "kind": "port", "seconds_per_sample": dt,
            "sample": f"one (linear, linear, linear, full) group on {len(seqs)} sequences totalling {tokens} tokens, f32 torch CPU oracle, "
                      f"{n} timed passes; the whole stack is that time x {groups} (extrapolated)"}


# ================================================================================================ device helpers
def _barrier(world):
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()


def _max_over_ranks(values, dev, world):
    if world <= 1:
        return [float(v) for v in values]
    t = torch.tensor(list(values), device=dev, dtype=torch.float64)
    torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return [float(v) for v in t]


def _timed(fn, n, world, dev):
    """n calls of fn between two CUDA events on the current stream, a barrier + synchronize on both sides; the maximum
    over ranks of the per-call milliseconds."""
    _barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    _barrier(world)
    return _max_over_ranks([e0.elapsed_time(e1) / n], dev, world)[0]


# ================================================================================================ encoder
def encoder_block(args, rank, world, dev, steps, warmup, shape="large"):
    """`shape` "base": the ModernBERT-base configuration on its configured input (22 layers, hidden 768, 12 heads, GeGLU
    2 x 1152; ids uniform over 50368, 8 sequences of 512, seed 1001). Otherwise:
    ModernBERT-large-shaped encoder forward (28 layers, hidden 1024, 16 heads, GeGLU 2 x 2624, window 128, global every
    3rd layer) over a packed batch of 32768 tokens with log-uniform lengths in [8, 8192], one replica per GPU. Every stage
    goes through the C ABI. Also times one global and one banded attention launch on the same batch."""
    from sys1_b200 import batching, device, modernbert, pipeline
    cfg = SimpleNamespace(vocab_size=50368, hidden_size=1024, num_hidden_layers=28, num_attention_heads=16, intermediate_size=2624,
                          layer_norm_eps=1e-5, global_attn_every_n_layers=3, local_attention=128, global_rope_theta=160000.0,
                          local_rope_theta=10000.0)
    if shape == "base":
        cfg.hidden_size, cfg.num_hidden_layers, cfg.num_attention_heads, cfg.intermediate_size = 768, 22, 12, 1152
    g = torch.Generator(device=dev).manual_seed(1003)
    mk = lambda *shape: (torch.randn(*shape, device=dev, generator=g) * 0.02).to(torch.bfloat16)
    ones = lambda: torch.ones(cfg.hidden_size, device=dev, dtype=torch.bfloat16)
    w = {"tok_embeddings": mk(cfg.vocab_size, cfg.hidden_size), "embeddings_norm": ones(), "final_norm": ones()}
    for i in range(cfg.num_hidden_layers):
        p = f"layers.{i}."
        w[p + "Wqkv"], w[p + "Wo"] = mk(3 * cfg.hidden_size, cfg.hidden_size), mk(cfg.hidden_size, cfg.hidden_size)
        w[p + "Wi"], w[p + "mlp_Wo"] = mk(2 * cfg.intermediate_size, cfg.hidden_size), mk(cfg.hidden_size, cfg.intermediate_size)
        w[p + "attn_norm"], w[p + "mlp_norm"] = ones(), ones()
    enc = modernbert.Encoder(w, cfg)
    ctx = device.load(dev.index)
    T = args.encoder_tokens
    if shape == "base":
        import numpy as np
        T, lens = 4096, np.full(8, 512, dtype=np.int32)
        ids = torch.randint(0, 50368, (8, 512), generator=torch.Generator().manual_seed(1001)).reshape(-1).to(torch.int32).to(dev)
    else:
        lens = batching.synthetic_lengths(1003 + rank, 8, 8192, T, log_uniform=True)
        ids = torch.randint(0, cfg.vocab_size, (T,), device=dev, generator=g).to(torch.int32)
    batch, _ = batching.pack_next(lens, batching.BatcherConfig(token_budget=T))
    pos = torch.from_numpy(batch.positions).to(dev)
    fwd = lambda: enc.forward(ids, batch.cu_seqlens, pos)
    for _ in range(warmup):
        fwd()
    ctx.sync()
    l0 = ctx.launch_count()
    ms = _timed(fwd, steps, world, dev)
    launches = ctx.launch_count() - l0
    # the same forward replayed from one CUDA graph (the batch's tables come from the batch plan, so nothing in a pass copies
    # from host memory and the whole pass can be captured): what a serving loop does for a batch shape it sees again, and
    # the number that matters where a pass is a few hundred launches of a few microseconds each
    ms_graph = None
    if shape == "base" or args.graph:
        try:
            cap = torch.cuda.Stream(dev)
            with torch.cuda.stream(cap):
                cap_ctx = device.load(dev.index)   # the capture stream's context, created (and warmed) before the capture
                for _ in range(2):
                    fwd()
                cap_ctx.sync()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=cap):
                    y_graph = fwd()
            torch.cuda.synchronize()
            y_eager = fwd()
            graph.replay()
            torch.cuda.synchronize()
            if not torch.equal(y_graph, y_eager):
                raise RuntimeError("graph replay and eager pass disagree")
            ms_graph = _timed(graph.replay, steps, world, dev)
        except Exception as exc:  # noqa: BLE001 - the eager numbers stand on their own
            ms_graph = f"unavailable: {exc!r}"[:200]
    # end to end through the public call: token ids and positions from pinned host memory every step, final hidden states
    # back to pinned host memory every step (copies on side streams, overlapped with the previous / next step)
    host_ids, host_pos = ids.cpu().pin_memory(), pos.to(torch.int32).cpu().pin_memory()
    host_out = torch.empty(T, cfg.hidden_size, dtype=torch.bfloat16).pin_memory()
    pipe = pipeline.HostPipeline(dev, [(T,), (T,)], torch.int32, depth=2)
    run = lambda bufs: enc.forward(bufs[0], batch.cu_seqlens, bufs[1])
    for _ in range(2):
        pipe.submit([host_ids, host_pos], host_out, run)
    pipe.drain()
    _barrier(world)
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(steps):
        pipe.submit([host_ids, host_pos], host_out, run)
    pipe.drain()
    f1.record()
    _barrier(world)
    ms_e2e = _max_over_ranks([f0.elapsed_time(f1) / steps], dev, world)[0]
    H, D = cfg.num_attention_heads, cfg.hidden_size // cfg.num_attention_heads
    qkv = mk(3, T, H * D)
    attn_stats = {}
    for name, window in (("global", -1), ("local", cfg.local_attention // 2)):
        out = torch.empty(T, H * D, device=dev, dtype=torch.bfloat16)
        call = lambda: modernbert.attention_varlen(qkv[0].view(T, H, D), qkv[1].view(T, H, D), qkv[2].view(T, H, D), batch.cu_seqlens,
                                                   window=window, out=out)
        for _ in range(3):
            call()
        us = _timed(call, 10, 1, dev) * 1e3
        pairs = 0
        for n in lens:
            n = int(n)
            pairs += n * n if window < 0 or n <= window else n * (2 * window + 1) - window * (window + 1)
        attn_stats[name] = {"us": us, "tflops": 4.0 * D * H * pairs / (us * 1e-6) / 1e12}
    ctx.sync()
    hs, it = cfg.hidden_size, cfg.intermediate_size
    flops_tok = cfg.num_hidden_layers * 2 * (hs * 3 * hs + hs * hs + hs * 2 * it + it * hs)
    what = ("ModernBERT-base encoder forward, 22 layers, 8 sequences of 512 ids uniform over 50368 (seed 1001)" if shape == "base" else
            f"ModernBERT-large-shaped encoder forward, 28 layers, packed T={T} per GPU, lengths log-uniform [8,8192]")
    return {"metric": "encoder tokens/s", "value": world * T / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms, "steps": steps,
            "config": {"workload": what + ", every stage through the C ABI (projections, attention, norms, RoPE, embedding lookup)",
                       "sequences": int(len(lens)), "parallelism": f"replicas x{world}"},
            "projection_tflops": world * T * flops_tok / (ms * 1e-3) / 1e12, "attention": attn_stats,
            **({"graph_replay": ({"ms_per_step": ms_graph, "value": world * T / (ms_graph * 1e-3), "unit": "tokens/s"}
                                 if isinstance(ms_graph, float) else {"note": ms_graph})} if ms_graph is not None else {}),
            "e2e": {"value": world * T / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": 8 * T, "d2h_bytes_per_step": 2 * T * cfg.hidden_size},
            "gpu_launches": launches}


# ================================================================================================ decoder
def decoder_block(args, rank, world, dev, steps, warmup):
    """Qwen3.5-small-shaped hybrid decoder forward (24 layers = (linear, linear, linear, full) x 6, hidden 1024, 16 x 128
    delta-rule heads, conv 4, full attention 8 query / 2 KV heads x 256, SwiGLU 3584) over a packed batch of 16384 tokens
    with lengths uniform in [64, 2048], one replica per GPU. Every stage goes through the C ABI."""
    from sys1_b200 import batching, device, qwen35
    cfg = _decoder_cfg("small", 24, 151936)
    w = _decoder_group_weights(cfg, 1004, dev, torch.bfloat16)
    dec = qwen35.Decoder(w, cfg, recurrence=args.recurrence)
    ctx = device.load(dev.index)
    T = args.decoder_tokens
    lens = batching.synthetic_lengths(1004 + rank, 64, 2048, T)
    batch, _ = batching.pack_next(lens, batching.BatcherConfig(token_budget=T))
    g = torch.Generator(device=dev).manual_seed(1004)
    ids = torch.randint(0, cfg.vocab_size, (T,), device=dev, generator=g).to(torch.int32)
    pos = torch.from_numpy(batch.positions).to(dev)
    fwd = lambda: dec.forward(ids, batch.cu_seqlens, pos)
    for _ in range(warmup):
        fwd()
    ctx.sync()
    l0 = ctx.launch_count()
    ms = _timed(fwd, steps, world, dev)
    launches = ctx.launch_count() - l0
    ctx.sync()
    flops_tok = 18 * 43_057_152 + 6 * 36_700_160  # projection flops per token: linear-attention / full-attention layers
    return {"metric": "decoder tokens/s", "value": world * T / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms, "steps": steps,
            "config": {"workload": f"Qwen3.5-small-shaped hybrid decoder forward, 24 layers, packed T={T} per GPU, lengths U[64,2048], "
                                   "every stage through the C ABI" + ("" if args.recurrence == "chunked" else ", exact f32 token-sequential delta rule"),
                       "sequences": int(len(lens)), "parallelism": f"replicas x{world}"},
            "projection_tflops": world * T * flops_tok / (ms * 1e-3) / 1e12, "gpu_launches": launches}


# ================================================================================================ tensor parallel
def _kernel_timeline(step, ctx, rank, path):
    """Every kernel of one step with its start and duration (torch's profiler, i.e. CUPTI activity records; the step is
    run twice under the profiler and the second run is kept), written as CSV `name,start_us,duration_us` to
    `<path>.rank<r>.csv`: shows which kernels ran beside which (a sum over ranks beside the other micro-batch's projections)."""
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        step()
        ctx.sync()
        torch.cuda.synchronize()
        step()
        ctx.sync()
        torch.cuda.synchronize()
    ev = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA), key=lambda e: e.time_range.start)
    # the second run starts at the first device-to-device copy (the step's `x.copy_`) after the first run's last kernel
    copies = [i for i, e in enumerate(ev) if e.name.startswith("Memcpy DtoD")]
    ev = ev[copies[1]:] if len(copies) > 1 else ev
    t0 = ev[0].time_range.start if ev else 0
    with open(f"{path}.rank{rank}.csv", "w") as f:
        f.write("name,start_us,duration_us\n")
        for e in ev:
            f.write("%s,%.1f,%.1f\n" % (e.name[:80].replace(",", ";"), e.time_range.start - t0, e.time_range.end - e.time_range.start))


def tp_block(args, rank, world, dev, steps, warmup):
    """One (linear, linear, linear, full) layer group of the 27B-shaped hybrid model (hidden 5120, SwiGLU 17408, 16 key / 48
    value delta-rule heads of 128, 24 query / 4 KV heads of 256) over a packed batch of `--tp-tokens` tokens with lengths
    uniform in [256, 8192], tensor-parallel over the ranks: heads, conv channels and gate / up columns split by rank, o_proj /
    out_proj / down_proj row-parallel with the partial sums exchanged slab by slab (`s1_allreduce_bf16`) under the
    projections of the next slab. Strong scaling: the batch is the same at every N. Parity: the same group on 2048 tokens
    against the unsharded layers on this GPU, and every rank must hold bit-identical results."""
    from sys1_b200 import batching, device, qwen35, tensor_parallel
    cfg = _decoder_cfg("27b", 4, 0)
    if world > 1:
        tp = tensor_parallel.TensorParallel.from_process_group(dev.index, comm_ctas=args.comm_ctas)
    else:
        tp = tensor_parallel.TensorParallel(device.load(dev.index), 0, 1)
    ctx = tp.ctx
    w = _decoder_group_weights(cfg, 1005, dev, torch.bfloat16)   # the same full tensors on every rank (same seed)
    own = world > 1 and args.exchange in ("multimem", "both")
    # SMs the projections leave free while sums are in flight: NCCL's kernels need room of their own; the library's exchange
    # kernel is a few fat blocks and the projections draw their tiles at run time around it, so nothing is set aside
    comm_sms = args.comm_sms if args.comm_sms >= 0 else (0 if own else 16)
    dec = tensor_parallel.Decoder(w, cfg, tp, slabs=args.slabs, comm_sms=comm_sms, comm_ctas=args.comm_ctas)
    H = cfg.hidden_size
    if own:   # the residual stream lives in symmetric memory: its sums run as the library's in-switch reduction kernel
        tp.symmetric_arena((args.tp_tokens + 2048) * H * 2 + 4096)
    fresh = (lambda rows: tp.symmetric_empty((rows, H))) if own else (lambda rows: torch.empty(rows, H, dtype=torch.bfloat16, device=dev))

    def batch_of(T, seed):
        lens = batching.synthetic_lengths(seed, 256, min(8192, T), T)
        b, _ = batching.pack_next(lens, batching.BatcherConfig(token_budget=T))
        g = torch.Generator(device=dev).manual_seed(seed)
        return b, torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16), torch.from_numpy(b.positions).to(dev)

    # ---- parity on a small batch, layer by layer on identical inputs (the acceptance rule: max-relative 2e-2 per layer):
    #      every layer of the sharded group gets the residual stream the unsharded stack has before that layer; all ranks
    #      must hold bit-identical results. The whole group end to end is reported as well (two bf16 trajectories drift).
    pb, px, ppos = batch_of(2048, 2005)
    mbp = args.micro_batches if world > 1 else 1
    single = qwen35.Decoder({**w, "embed_tokens": px}, cfg)      # the embedded tokens stand in for the table: ids = arange
    y_one, states = single.forward(torch.arange(2048, device=dev, dtype=torch.int32), pb.cu_seqlens, ppos, collect=True)
    xp = fresh(2048)
    y_tp = dec.forward_embeds(xp.copy_(px), pb.cu_seqlens, ppos, micro_batches=mbp).clone()
    ctx.sync()
    rel = lambda a, b_: float((a.float() - b_.float()).abs().max() / b_.float().abs().max())
    per_layer, digest = [], y_tp.view(torch.int16).to(torch.int64).sum().reshape(1)
    x_in = px
    for i, layer in enumerate(dec.layers):
        got = layer.forward(xp.copy_(x_in), pb.cu_seqlens, ppos)
        per_layer.append(rel(got, states[i]))
        digest = digest + got.view(torch.int16).to(torch.int64).sum()
        x_in = states[i]
    ctx.sync()
    max_rel = rel(y_tp, y_one)
    rel_rms = float((y_tp.float() - y_one.float()).square().mean().sqrt() / y_one.float().square().mean().sqrt())
    same = True
    if world > 1:
        all_d = [torch.zeros_like(digest) for _ in range(world)]
        torch.distributed.all_gather(all_d, digest)
        same = all(int(d) == int(all_d[0]) for d in all_d)
    del single, y_one, y_tp, states

    # ---- timing at the configured budget
    T = args.tp_tokens
    b, x0, pos = batch_of(T, 1005)
    x = fresh(T)
    mbs = args.micro_batches if world > 1 else 1
    n_ar = 2 * cfg.num_hidden_layers

    def measure(decoder, micro_batches, pdl, n_steps, x=x):
        ctx.set_option("pdl", pdl)

        def step(exchange=True):
            x.copy_(x0)   # the stream is updated in place; the copy is part of neither variant's difference
            decoder.forward_embeds(x, b.cu_seqlens, pos, exchange=exchange, micro_batches=micro_batches)

        for _ in range(warmup):
            step()
        ctx.sync()
        l0 = ctx.launch_count()
        ms_ = _timed(step, n_steps, world, dev)
        launches_ = ctx.launch_count() - l0
        ms_math_ = _timed(lambda: step(False), n_steps, world, dev)
        ctx.sync()
        ctx.set_option("pdl", 1)
        return ms_, ms_math_, launches_

    pdl = 1 if args.tp_pdl < 0 else args.tp_pdl
    ms, ms_math, launches = measure(dec, mbs, pdl, steps)
    def bare_allreduces(buf):
        def bare():
            for _ in range(n_ar):
                ctx.all_reduce_(buf)
        bare()
        return _timed(bare, max(2, steps // 2), world, dev)

    busbw = lambda t_ms: 2.0 * (world - 1) / world * n_ar * T * H * 2 / (t_ms * 1e-3) / 1e9
    ms_ar = bare_allreduces(x) if world > 1 else 0.0
    ctx.sync()
    other = None
    if world > 1 and args.exchange == "both":   # the same step with the sums through NCCL, for comparison
        xn = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
        sms_n = args.comm_sms if args.comm_sms >= 0 else 16
        dec_n = tensor_parallel.Decoder(w, cfg, tp, slabs=args.slabs, comm_sms=sms_n)
        ms_n, ms_math_n, _ = measure(dec_n, mbs, pdl, steps, x=xn)
        ms_ar_n = bare_allreduces(xn)
        ctx.sync()
        del dec_n
        other = {"exchange": "nccl", "comm_sms": sms_n, "ms": ms_n, "ms_without_exchange": ms_math_n, "ms_allreduce_alone": ms_ar_n,
                 "allreduce_busbw_gbs": busbw(ms_ar_n), "exchange_hidden_frac": 1.0 - (ms_n - ms_math_n) / ms_ar_n}
        del xn
    if args.timeline:
        _kernel_timeline(lambda: (x.copy_(x0), dec.forward_embeds(x, b.cu_seqlens, pos, micro_batches=mbs)), ctx, rank, args.timeline)
    sweep = None
    if args.tp_sweep and world > 1:
        sweep = []
        for sweep_sms in ((0, 8, 16) if own else (8, 16, 32)):
            for blocks in ((4, 8, 16) if own else (args.comm_ctas,)):
                d2 = tensor_parallel.Decoder(w, cfg, tp, slabs=args.slabs, comm_sms=sweep_sms, comm_ctas=blocks)
                if own:
                    ctx.set_option("comm_ctas", blocks)
                for m in (1, 2, 4):
                    for p_ in ((1,) if own else (0, 1)):
                        a_, b_, _ = measure(d2, m, p_, 3)
                        sweep.append({"comm_sms": sweep_sms, "comm_ctas": blocks, "micro_batches": m, "pdl": p_, "ms": a_,
                                      "ms_without_exchange": b_, "hidden_frac": 1.0 - (a_ - b_) / ms_ar if ms_ar > 0 else None})
                del d2
        if own:
            ctx.set_option("comm_ctas", args.comm_ctas)
    flops = T * (3 * 766_443_520 + 744_488_960)   # projection flops of the group (three linear-attention + one full layer)
    return {"metric": "tensor-parallel layer-group TFLOP/s", "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms,
            "steps": steps, "scaling": "strong",
            "config": {"workload": f"27B-shaped (linear, linear, linear, full) layer group, packed T={T}, lengths U[256,8192], "
                                   f"tensor parallel x{world}; " +
                                   (f"{mbs} micro-batches of whole sequences alternate between computing and exchanging their partial sums"
                                    if mbs > 1 else f"row-parallel outputs exchanged in {args.slabs} row slabs") +
                                   f", {comm_sms} SMs left to the exchange ({args.comm_ctas or 'default'} blocks); sums over ranks by " +
                                   ("the library's own kernel (multimem.ld_reduce / multimem.st through the NVSwitch on symmetric memory)"
                                    if own else "ncclAllReduce" if world > 1 else "nothing (one rank)"),
                       "sequences": int(b.num_sequences), "parallelism": f"tp{world}"},
            "ms_without_exchange": ms_math, "ms_allreduce_alone": ms_ar, "allreduces_per_step": n_ar if world > 1 else 0,
            "allreduce_busbw_gbs": busbw(ms_ar) if world > 1 and ms_ar > 0 else None,
            "exchange": "multimem" if own else ("nccl" if world > 1 else None), **({"compared_with": other} if other else {}),
            "exchange_hidden_frac": (1.0 - (ms - ms_math) / ms_ar) if world > 1 and ms_ar > 0 else None,
            "parity": {"tokens": 2048, "per_layer_max_rel_vs_unsharded": per_layer, "bound": 2e-2, "ranks_bit_identical": bool(same),
                       "ok": bool(same and max(per_layer) <= 2e-2),
                       "whole_group_max_rel": max_rel, "whole_group_rel_rms": rel_rms,
                       "note": "per layer: the sharded layer and the unsharded layer on the same input; whole group: two bf16 "
                               "trajectories of four layers (per-rank partial sums are rounded to bf16 before they are added)"},
            "gpu_launches": launches, **({"sweep": sweep} if sweep is not None else {})}


# ================================================================================================ main workload
def projections_line(args, rank, world, local_rank):
    from sys1_b200 import batching, device, linear, modernbert
    from sys1_b200.pipeline import HostPipeline
    dev = torch.device("cuda", local_rank)
    ctx = device.load(local_rank)
    T = args.tokens
    warmup = max(args.warmup, 3)
    peaks = measured_peaks()
    W = make_weights(dev, torch.bfloat16)
    neg = {"wo": -W["wo"], "wout": -W["wout"]}
    ev = lambda: torch.cuda.Event(enable_timing=True)
    names = [p[0] for p in PROJECTIONS]
    NSETS = 4

    class Chain:
        """Buffers and the step of one token budget. The device-resident arm keeps updating the same few residual-stream
        buffers in place; every other visit of a buffer uses -Wo / -Wout (same work, opposite sign) so that the stream
        stays at its N(0, 1) scale instead of growing step after step."""

        def __init__(self, tokens, pinned):
            lens = batching.synthetic_lengths(SEED + rank, 16, 512, tokens)
            batch, taken = batching.pack_next(lens, batching.BatcherConfig(token_budget=tokens))
            assert batch.total_tokens == tokens and taken == len(lens)  # the projections ignore the boundaries, the layout is the batcher's
            g = torch.Generator().manual_seed(SEED + 100 + rank)
            mkh = lambda: torch.randn(tokens, HIDDEN, generator=g).to(torch.bfloat16)
            self.host_x = [mkh().pin_memory() if pinned else mkh() for _ in range(NSETS)]
            self.host_a = [mkh().pin_memory() if pinned else mkh() for _ in range(NSETS)]
            self.xs, self.atts = [t.to(dev) for t in self.host_x], [t.to(dev) for t in self.host_a]
            self.qkv = torch.empty(tokens, QKV, dtype=torch.bfloat16, device=dev)
            self.m = torch.empty(tokens, INTER, dtype=torch.bfloat16, device=dev)
            self.T = tokens

        def one(self, name, i, x=None, a=None):
            x = self.xs[i % NSETS] if x is None else x
            a = self.atts[i % NSETS] if a is None else a
            negate = bool((i // NSETS) & 1)
            if name == "wqkv":
                linear.fused_linear(x, W["wqkv"], out=self.qkv)
            elif name == "wo+residual":
                linear.fused_linear(a, neg["wo"] if negate else W["wo"], residual=x, out=x)
            elif name == "wi+geglu":
                linear.fused_linear(x, W["wi"], epilogue=linear.EPI_GEGLU, out=self.m)
            else:
                linear.fused_linear(self.m, neg["wout"] if negate else W["wout"], residual=x, out=x)

        def step(self, i, x=None, a=None):
            for n in names:
                self.one(n, i, x, a)
            return self.xs[i % NSETS] if x is None else x

    main = Chain(T, pinned=True)
    cycle = 2 * NSETS
    for i in range(cycle * ((warmup + cycle - 1) // cycle)):  # whole +/- cycles
        main.step(i)
    ctx.sync()

    def capture(chain):
        """One CUDA graph per (buffer set, sign): the launches of a step with their tensor maps baked in."""
        cap = torch.cuda.Stream(dev)
        with torch.cuda.stream(cap):
            cap_ctx = device.load(local_rank)  # context of the capture stream, created before any capture
            chain.step(0)
            cap_ctx.sync()
        graphs = []
        for i in range(cycle):
            g_ = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_, stream=cap):
                chain.step(i)
            graphs.append(g_)
        torch.cuda.synchronize()
        return graphs

    graphs = capture(main) if args.graph else None

    # per-kernel durations: each projection launched back to back on the rotating buffer sets between two events of its
    # own (an event between every two launches of a step would itself cost several microseconds per launch and keep
    # a projection's set-up from overlapping its predecessor's tail, which is what the timed loop below benefits from);
    # taken before the timed loop, each kernel on its own, so the burst peak is the matching denominator
    per, reps = {}, cycle * 5
    for n in names:
        for i in range(cycle):
            main.one(n, i)
        k0, k1 = ev(), ev()
        k0.record()
        for i in range(reps):
            main.one(n, i)
        k1.record()
        torch.cuda.synchronize()
        per[n] = k0.elapsed_time(k1) / reps

    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.15)
    launches0 = ctx.launch_count()
    _barrier(world)
    t0w = time.time()
    e0, e1 = ev(), ev()
    e0.record()
    for i in range(args.steps):
        if graphs is not None:
            graphs[i % cycle].replay()
        else:
            main.step(i)
    e1.record()
    _barrier(world)
    ctx.sync()
    launches = ctx.launch_count() - launches0
    ms_total = e0.elapsed_time(e1)
    if graphs is not None:
        launches = 4 * args.steps  # replayed from the graphs (4 kernel nodes each), not counted by the context
    ms_step = _max_over_ranks([ms_total / args.steps], dev, world)[0]
    flops_step = FLOPS_PER_TOKEN * T
    value = world * flops_step / (ms_step * 1e-3) / 1e12

    blocks = {}

    def attempt(name, fn):
        try:
            blocks[name] = fn()
        except Exception as exc:  # a secondary block must not cost the line
            blocks[name] = {"error": f"{type(exc).__name__}: {exc}"[:400]}
            torch.cuda.synchronize()

    # ---- sustained: the same chain back to back for at least two seconds, clocks sampled under load ----------------
    def sustained():
        n_batch, done, t_begin = 200, 0, time.time()
        s0, s1 = ev(), ev()
        _barrier(world)
        s0.record()
        while True:
            for i in range(n_batch):
                main.step(done + i)
            done += n_batch
            torch.cuda.synchronize()
            if time.time() - t_begin >= args.sustain_seconds:
                break
        s1.record()
        torch.cuda.synchronize()
        t_end = time.time()
        ms = _max_over_ranks([s0.elapsed_time(s1) / done], dev, world)[0]
        clk = sampler.summary(t_begin + 0.3, t_end)
        tf = world * flops_step / (ms * 1e-3) / 1e12
        return {"seconds": t_end - t_begin, "steps": done, "ms_per_step": ms, "value": tf, "unit": "TFLOP/s",
                "frac_of_sustained": tf / world / peaks["sustained"], "frac_of_burst": tf / world / peaks["burst"],
                "peak_source": f"{peaks['kind']} bf16: sustained {peaks['sustained']}, burst {peaks['burst']} TFLOP/s per GPU", "clocks": clk}

    if not args.profile:
        attempt("sustained", sustained)
    t1w = time.time()
    clocks = sampler.summary(t0w - 0.05, t1w + 0.05)
    clocks["window"] = "timed region and the sustained loop that follows it"
    sampler.stop()

    if args.profile:
        return {"metric": "projection GEMM TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
                "ms_per_step": ms_step, "per_projection_us": {n: per[n] * 1e3 for n in names}, "profile_run": True} if rank == 0 else None
    # ---- end-to-end arm: host buffers in, host buffer out, copies inside the timed region ----------------------------
    # (copy-in of batch i+1 and copy-out of batch i-1 overlap the compute of batch i: sys1_b200.pipeline)
    host_y = [torch.empty(T, HIDDEN, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    pipe = HostPipeline(dev, [(T, HIDDEN), (T, HIDDEN)], torch.bfloat16, depth=2)

    def e2e_step(i):
        pipe.submit([main.host_x[i % NSETS], main.host_a[i % NSETS]], host_y[i % 2], lambda bufs: main.step(0, bufs[0], bufs[1]))

    e2e_steps = max(3, min(args.steps, 40))
    for i in range(3):
        e2e_step(i)
    pipe.drain()
    _barrier(world)
    f0, f1 = ev(), ev()
    f0.record()
    for i in range(e2e_steps):
        e2e_step(i)
    pipe.drain()
    f1.record()
    _barrier(world)
    ctx.sync()
    ms_step_e2e = _max_over_ranks([f0.elapsed_time(f1) / e2e_steps], dev, world)[0]
    e2e_value = world * flops_step / (ms_step_e2e * 1e-3) / 1e12

    # ---- the smaller token budgets: CUDA-graph replay and eager ---------------------------------------------------------
    def budgets():
        out = {}
        for tb in (2048, 8192):
            ch = Chain(tb, pinned=False)
            for i in range(cycle):
                ch.step(i)
            ctx.sync()
            n = 40 * cycle
            ms_eager = _timed(lambda c=[0]: (ch.step(c[0]), c.__setitem__(0, c[0] + 1)), n, world, dev)
            gs = capture(ch)
            for g_ in gs:
                g_.replay()
            ms_graph = _timed(lambda c=[0]: (gs[c[0] % cycle].replay(), c.__setitem__(0, c[0] + 1)), n, world, dev)
            fl = FLOPS_PER_TOKEN * tb
            by = sum(algorithmic_bytes(nm, tb) for nm in names)
            out[str(tb)] = {"tokens": tb, "us_per_step_graph": ms_graph * 1e3, "us_per_step_eager": ms_eager * 1e3,
                            "tflops": world * fl / (ms_graph * 1e-3) / 1e12, "tflops_eager": world * fl / (ms_eager * 1e-3) / 1e12,
                            "frac_of_burst": fl / (ms_graph * 1e-3) / 1e12 / peaks["burst"],
                            "algorithmic_gbs": by / (ms_graph * 1e-3) / 1e9, "frac_of_hbm": by / (ms_graph * 1e-3) / 1e9 / peaks["hbm"],
                            "eager_over_graph": ms_eager / ms_graph}
            del gs, ch
        out["hbm_peak_gbs"] = peaks["hbm"]
        return out

    attempt("budgets", budgets)

    # ---- the library on the same contractions, without any epilogue -------------------------------------------------------
    def gpu_lib():
        out = {}
        x768, x1152 = main.xs[0], main.m
        for n, k, nw, nout, epi in PROJECTIONS:
            wt = {"wqkv": W["wqkv"], "wo+residual": W["wo"], "wi+geglu": W["wi"], "mlp_out+residual": W["wout"]}[n]
            xin = x1152 if k == INTER else x768
            y = torch.empty(T, nw, dtype=torch.bfloat16, device=dev)
            f = lambda: torch.matmul(xin, wt.t(), out=y)
            for _ in range(5):
                f()
            ms = _timed(f, 40, 1, dev)
            out[n] = {"us": ms * 1e3, "tflops": 2 * T * k * nw / (ms * 1e-3) / 1e12, "ours_us": per[n] * 1e3}
        out["note"] = "torch.matmul (cuBLAS) bf16, no bias / gating / residual; ours_us includes the fused epilogue"
        return out

    attempt("gpu_lib", gpu_lib)
    sec_steps, sec_warm = max(3, min(args.steps, 10)), 3
    del pipe, host_y
    if not args.no_secondary:
        attempt("encoder", lambda: encoder_block(args, rank, world, dev, sec_steps, sec_warm))
        torch.cuda.empty_cache()
        attempt("decoder", lambda: decoder_block(args, rank, world, dev, sec_steps, sec_warm))
        torch.cuda.empty_cache()
        attempt("tp", lambda: tp_block(args, rank, world, dev, max(3, min(args.steps, 5)), 2))
        torch.cuda.empty_cache()

    if rank != 0:
        return None
    dom = max(per, key=per.get)
    dom_proj = next(p for p in PROJECTIONS if p[0] == dom)
    dom_flops = 2 * T * dom_proj[1] * dom_proj[2]
    achieved = dom_flops / (per[dom] * 1e-3) / 1e12
    config = {"workload": f"ModernBERT-base projection microbench, packed ragged batch, T={T} tokens "
                          "(lengths U[16,512]), Wqkv / Wo+residual / Wi+GeGLU / MLP-out+residual",
              "tokens": T, "hidden": HIDDEN, "intermediate": INTER, "parallelism": f"replicas x{world}",
              "l2": "4 rotating input sets (400 MB) + 226 MB of outputs per step exceed the 126 MB L2",
              "launch": "cuda graph replay" if args.graph else "eager",
              "timing": "K steps back to back between two events; per-kernel durations from 40 back-to-back launches of each "
                        "projection on the same rotating buffers between two events of their own",
              "residual": "in place (x += ...); alternate visits of a buffer use -Wo / -Wout to keep the stream bounded"}
    # a kernel timed alone between events in a run of a few tens of milliseconds: the burst figure applies
    line = {"metric": "projection GEMM TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "config": config,
            "roofline": {"bound": "tensor", "kernel": f"s1_gemm_kernel ({dom})", "achieved": achieved, "peak": peaks["burst"],
                         "unit": "TFLOP/s", "frac": achieved / peaks["burst"], "peak_source": f"{peaks['kind']} bf16 burst",
                         "frac_of_sustained": achieved / peaks["sustained"], "flops_per_launch": dom_flops,
                         "us_per_launch": per[dom] * 1e3, "algorithmic_bytes": algorithmic_bytes(dom, T),
                         "traffic": ncu_traffic(dom, T)},
            "per_projection": {n: {"us": per[n] * 1e3, "tflops": 2 * T * p[1] * p[2] / (per[n] * 1e-3) / 1e12,
                                   "gbs": algorithmic_bytes(n, T) / (per[n] * 1e-3) / 1e9}
                               for n, p in zip(names, PROJECTIONS)},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": ms_step_e2e,
                    "h2d_bytes_per_step": 2 * T * HIDDEN * 2, "d2h_bytes_per_step": T * HIDDEN * 2},
            "gpu_launches": launches, "clocks": clocks}
    line.update(blocks)
    return line


def reference_line(args, warmup):
    """The CPU arm: the oracle on the host cores, for the workload named by --workload (bounded samples)."""
    T = args.tokens
    if args.workload == "projections":
        val, dt, n, cores = cpu_projections(args.cpu_sample_tokens, max(1, args.steps), warmup, budget_s=60.0)
        cb = {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port",
              "sample": f"{args.cpu_sample_tokens} of the {T} packed token rows per step, same four projections, torch CPU f32 oracle "
                        "(restatement of the reference's candle CPU path; the Rust reference itself cannot be built here: no cargo/rustc)"}
        metric, unit, ms = "projection GEMM TFLOP/s", "TFLOP/s", dt * 1e3
        workload = (f"ModernBERT-base projection microbench, packed ragged batch, T={T} tokens (lengths U[16,512]), "
                    "Wqkv / Wo+residual / Wi+GeGLU / MLP-out+residual")
    else:
        cb = cpu_encoder_base(60.0) if args.workload == "base" else cpu_encoder(60.0) if args.workload == "encoder" else cpu_decoder("small" if args.workload == "decoder" else "27b",
                                                                                2048 if args.workload == "decoder" else 512, 60.0)
        val, n = cb["value"], 1
        # one "step" of these arms is one timed pass over the sample the block describes
        ms = cb["seconds_per_forward"] * 1e3 if "seconds_per_forward" in cb else cb.get("seconds_per_sample", 0.0) * 1e3 or None
        metric, unit = {"base": "encoder tokens/s", "encoder": "encoder tokens/s", "decoder": "decoder tokens/s",
                        "tp": "27B layer-group tokens/s"}[args.workload], "tokens/s"
        workload = {"base": "ModernBERT-base encoder forward, 8 x 512 ids", "encoder": "ModernBERT-large-shaped encoder forward",
                    "decoder": "Qwen3.5-small-shaped hybrid decoder forward",
                    "tp": "27B-shaped hybrid decoder forward"}[args.workload] + " (CPU oracle; sample and extrapolation as the sample says)"
    return {"impl": "reference", "metric": metric, "value": val, "unit": unit, "n_gpus": args.gpus, "steps": n, "warmup": warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload, "tokens": T, "parallelism": "host cores"}, "cpu_baseline": cb,
            "e2e": {"value": val, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--cpu-sample-tokens", type=int, default=8192)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--profile", action="store_true",
                    help="a short run for a profiler: the timed loop only (no sustained loop, budgets, library GEMMs, end-to-end arm, "
                         "secondary workloads or CPU baseline)")
    ap.add_argument("--no-secondary", action="store_true", help="projections workload: leave out the encoder / decoder / tp blocks")
    ap.add_argument("--workload", default="projections", choices=["projections", "base", "encoder", "decoder", "tp"],
                    help="projections (default): the headline line with every block; encoder / decoder / tp: that block alone, as a line")
    ap.add_argument("--encoder-tokens", type=int, default=32768)
    ap.add_argument("--decoder-tokens", type=int, default=16384)
    ap.add_argument("--tp-tokens", type=int, default=65536)
    ap.add_argument("--recurrence", default="chunked", choices=["chunked", "exact"],
                    help="decoder: the gated delta rule in 64-token chunks on the tensor cores (default) or the exact f32 token-sequential kernel")
    ap.add_argument("--sustain-seconds", type=float, default=2.2)
    ap.add_argument("--slabs", type=int, default=4, help="tp: row slabs the exchange is pipelined in")
    ap.add_argument("--comm-ctas", type=int, default=0, help="tp: blocks the all-reduce may use (0 = NCCL's default)")
    ap.add_argument("--comm-sms", type=int, default=-1,
                    help="tp: SMs the projections leave to the exchange while it runs beside them (-1: 0 for the library's own exchange kernel, 16 for NCCL)")
    ap.add_argument("--tp-pdl", type=int, default=-1, help="tp: 0 / 1 turns programmatic dependent launch of the projections off / on (-1: default)")
    ap.add_argument("--micro-batches", type=int, default=2, help="tp: groups of whole sequences that alternate between computing and exchanging (1: row slabs inside each projection instead)")
    ap.add_argument("--exchange", default="both", choices=["multimem", "nccl", "both"],
                    help="tp: sums over ranks by the library's own in-switch reduction kernel on symmetric memory (multimem), by "
                         "ncclAllReduce (nccl), or the first with the second timed beside it (both, default)")
    ap.add_argument("--timeline", default="", help="tp: also write one step's kernel timeline (CSV per rank) to this path prefix")
    ap.add_argument("--tp-sweep", action="store_true", help="tp: also time the group for a grid of comm-sms x micro-batches x pdl settings")
    ap.add_argument("--graph", action="store_true",
                    help="replay each step from a CUDA graph (for small token budgets, where launching from Python is the bottleneck)")
    args = ap.parse_args()
    # stdout carries the one JSON line and nothing else: whatever libraries print (NCCL's version banner, for one) goes
    # to stderr from here on
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)

    def emit(line):
        os.write(json_fd, (json.dumps(line) + "\n").encode())

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    warmup = max(args.warmup, 3)

    if args.impl == "reference":
        if rank != 0:  # rank 0 alone runs the CPU arm; the other ranks leave without work
            return
        emit(reference_line(args, warmup))
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: there is no CPU fallback for the product path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=dev)
    try:
        if args.workload == "projections":
            line = projections_line(args, rank, world, local_rank)
            if line is not None and world == 1 and not args.no_cpu_baseline and not args.profile:
                val, dt, n, cores = cpu_projections(args.cpu_sample_tokens, 1000, 1, budget_s=12.0)
                line["cpu_baseline"] = {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                        "sample": f"{args.cpu_sample_tokens} of the {args.tokens} token rows, same four projections, "
                                                  f"torch CPU f32 oracle, {n} timed passes"}
                # the CPU oracle beside the secondary workloads too (bounded samples, extrapolated as each sample says)
                for name, fn in (("encoder", lambda: cpu_encoder(6.0)), ("decoder", lambda: cpu_decoder("small", 2048, 6.0)),
                                 ("tp", lambda: cpu_decoder("27b", 512, 6.0))):
                    if isinstance(line.get(name), dict) and "error" not in line[name]:
                        try:
                            line[name]["cpu_baseline"] = fn()
                        except Exception as exc:
                            line[name]["cpu_baseline"] = {"error": f"{type(exc).__name__}: {exc}"[:200]}
        else:
            steps = max(3, min(args.steps, 20))
            fn = {"base": lambda *a: encoder_block(*a, shape="base"), "encoder": encoder_block, "decoder": decoder_block, "tp": tp_block}[args.workload]
            block = fn(args, rank, world, dev, steps, warmup)
            line = None
            if rank == 0:
                line = {"n_gpus": world, "warmup": warmup, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
                        "data": "synthetic"}
                line.update(block)
        if rank == 0 and line is not None:
            emit(line)
    finally:
        if world > 1:
            torch.distributed.barrier()
            torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
