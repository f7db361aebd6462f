"""World-size-2 checks of the multi-rank host logic on CPU (gloo): replica sharding of sequences and the
tensor-parallel shard arithmetic (oracle partial products + all-reduce == unsharded oracle)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from sys1_b200 import batching, device


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # replicas: every sequence is served exactly once and the token load is balanced
        lens = batching.synthetic_lengths(1003, 8, 8192, 32768, log_uniform=True)
        mine = device.shard_sequences(lens, world, rank)
        counts = torch.zeros(len(lens), dtype=torch.int64)
        counts[mine] = 1
        tokens = torch.tensor([int(lens[mine].sum())])
        dist.all_reduce(counts)
        gathered = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(gathered, tokens)
        assert bool((counts == 1).all())
        loads = [int(t) for t in gathered]
        assert sum(loads) == int(lens.sum()) and max(loads) - min(loads) <= int(lens.max())
        # each replica packs its own batches
        batches = list(batching.pack_all(lens[mine], batching.BatcherConfig(token_budget=8192)))
        assert sum(b.total_tokens for b in batches) == loads[rank]

        # tensor parallel: column-parallel gate/up (SwiGLU) -> row-parallel down -> all-reduce, residual added once
        g = torch.Generator().manual_seed(1005)
        T, H, I = 64, 128, 256
        x = torch.randn(T, H, generator=g)
        wg, wu, wd = (torch.randn(I, H, generator=g) * 0.05, torch.randn(I, H, generator=g) * 0.05,
                      torch.randn(H, I, generator=g) * 0.05)
        h_local = oracle.swiglu(oracle.linear(x, device.column_parallel_shard(wg, rank, world), dtype="f32"),
                                oracle.linear(x, device.column_parallel_shard(wu, rank, world), dtype="f32"), dtype="f32")
        partial = oracle.linear(h_local, device.row_parallel_shard(wd, rank, world), dtype="f32")
        y = device.all_reduce_sum_(partial.clone()) + x
        want = oracle.mlp_qwen35(x, wg, wu, wd, residual=x, dtype="f32")
        assert torch.allclose(y, want, atol=1e-4)
        # GeGLU pairs shard together
        wi = torch.randn(2 * I, H, generator=g) * 0.05
        shard = device.column_parallel_shard(wi, rank, world, pairs=2)
        got = oracle.geglu(oracle.linear(x, shard, dtype="f32"), dtype="f32")
        full = oracle.geglu(oracle.linear(x, wi, dtype="f32"), dtype="f32")
        assert torch.allclose(got, full[:, rank * I // world:(rank + 1) * I // world], atol=1e-6)
        # a whole (linear-attention, full-attention) pair of layers: this rank's shard through the oracle, summed over ranks
        _check_layer_shards(world, [rank], reduce=device.all_reduce_sum_)
        q.put((rank, "ok"))
    except Exception as exc:  # pragma: no cover
        q.put((rank, repr(exc)))
    finally:
        dist.destroy_process_group()


def _tp_cfg():
    # the 27B head pattern (24 query / 4 KV heads, 16 key / 48 value delta-rule heads) at a small width
    return oracle.DecoderConfig(vocab_size=50, hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=24,
                                num_key_value_heads=4, head_dim=32, partial_rotary_factor=0.5, linear_num_key_heads=16,
                                linear_num_value_heads=48)


def _check_layer_shards(world, ranks, reduce=None):
    """Mixer and MLP of a linear-attention layer (index 0) and a full-attention layer (index 3): the oracle run on each
    rank's shard (a layer of a narrower model), partial outputs summed over the ranks, against the oracle on the full layer."""
    import dataclasses
    from sys1_b200 import tensor_parallel as tpar
    cfg = _tp_cfg()
    w = oracle.qwen35.init_weights(cfg, 7)
    Hr, KVr, Hkr, Hvr = tpar.local_heads(cfg, world)
    cfg_r = dataclasses.replace(cfg, num_attention_heads=Hr, num_key_value_heads=KVr, linear_num_key_heads=Hkr, linear_num_value_heads=Hvr)
    x = torch.randn(37, cfg.hidden_size, generator=torch.Generator().manual_seed(3))
    for i in (0, 3):
        kind = cfg.layer_type(i)
        p = f"layers.{i}."
        n = oracle.rms_norm(x, w[p + "input_layernorm"], cfg.rms_norm_eps)
        if kind == "full_attention":
            full = oracle.qwen35.full_attention(n, w, p + "self_attn.", cfg)
        else:
            full = oracle.qwen35.linear_attention(n, w, p + "linear_attn.", cfg)
        full_mlp = oracle.mlp_qwen35(n, w[p + "mlp.gate_proj"], w[p + "mlp.up_proj"], w[p + "mlp.down_proj"], dtype="f32")
        part, part_mlp = torch.zeros_like(full), torch.zeros_like(full_mlp)
        for r in ranks:
            sh = tpar.shard_layer_weights(w, p, cfg, kind, r, world)
            if kind == "full_attention":
                part += oracle.qwen35.full_attention(n, sh, "self_attn.", cfg_r)
            else:
                part += oracle.qwen35.linear_attention(n, sh, "linear_attn.", cfg_r)
            part_mlp += oracle.mlp_qwen35(n, sh["mlp.gate_proj"], sh["mlp.up_proj"], sh["mlp.down_proj"], dtype="f32")
            assert sh["mlp.down_proj"].stride(0) == cfg.intermediate_size  # a view of the full matrix, read through its row stride
        if reduce is not None:
            part, part_mlp = reduce(part), reduce(part_mlp)
        assert torch.allclose(part, full, atol=2e-5), f"{kind} over {world} ranks: {float((part - full).abs().max()):.2e}"
        assert torch.allclose(part_mlp, full_mlp, atol=2e-5)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_layer_shards_sum_to_the_unsharded_layer(world):
    """All ranks emulated in one process: query heads with the KV head they read (replicated when there are fewer KV
    heads than ranks), delta-rule value heads with their key heads, conv channels, A_log / dt_bias slices, gate / up
    columns, and the K ranges of the three row-parallel projections."""
    _check_layer_shards(world, list(range(world)))


def test_local_heads_of_the_27b_shape():
    from types import SimpleNamespace
    from sys1_b200 import tensor_parallel as tpar
    cfg = SimpleNamespace(num_attention_heads=24, num_key_value_heads=4, linear_num_key_heads=16, linear_num_value_heads=48)
    assert tpar.local_heads(cfg, 8) == (3, 1, 2, 6)
    assert tpar.local_heads(cfg, 4) == (6, 1, 4, 12)
    assert tpar.local_heads(cfg, 2) == (12, 2, 8, 24)
    with pytest.raises(ValueError):
        tpar.local_heads(cfg, 16)


@pytest.mark.timeout(120)
def test_two_ranks_gloo():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=100) for _ in range(world)]
    for p in procs:
        p.join(timeout=30)
    assert sorted(results) == [(0, "ok"), (1, "ok")], results


def test_shard_sequences_single_rank_is_identity():
    assert device.shard_sequences([5, 1, 9], 1, 0) == [0, 1, 2]
    a = device.shard_sequences([5, 1, 9, 9], 2, 0)
    b = device.shard_sequences([5, 1, 9, 9], 2, 1)
    assert sorted(a + b) == [0, 1, 2, 3]


def test_shard_helpers_reject_uneven_splits():
    w = torch.zeros(10, 24)
    with pytest.raises(ValueError):
        device.column_parallel_shard(w, 0, 4)
    with pytest.raises(ValueError):
        device.row_parallel_shard(w, 0, 2)


def test_split_sequences_into_micro_batches():
    from sys1_b200.tensor_parallel import split_sequences
    assert split_sequences([0, 10, 20, 30, 40], 2) == [(0, 2), (2, 4)]
    assert split_sequences([0, 100, 101, 102], 2) == [(0, 1), (1, 3)]
    assert split_sequences([0, 5], 3) == [(0, 1)]                     # fewer sequences than groups
    lens = batching.synthetic_lengths(1005, 256, 8192, 65536)
    cu = [0] + [int(v) for v in lens.cumsum()]
    for parts in (2, 4):
        groups = split_sequences(cu, parts)
        assert groups[0][0] == 0 and groups[-1][1] == len(lens) and all(a[1] == b[0] for a, b in zip(groups, groups[1:]))
        sizes = [cu[b] - cu[a] for a, b in groups]
        assert sum(sizes) == 65536 and max(sizes) - min(sizes) <= 2 * 8192  # cuts fall on sequence boundaries


def test_symmetric_arena_hands_out_aligned_slices_in_order():
    """`symmetric_empty` is a bump allocator over the registered arena: 256-byte aligned slices in call order (so that every
    rank, carving the same shapes, gets the same offsets), an error when the arena is full, everything free again after
    `symmetric_reset`. Checked on a plain CPU byte buffer standing in for the arena."""
    from sys1_b200 import tensor_parallel
    tp = tensor_parallel.TensorParallel.__new__(tensor_parallel.TensorParallel)
    tp.rank, tp.size = 0, 2
    with pytest.raises(RuntimeError):
        tp.symmetric_empty((4, 4))   # no arena yet
    tp._arena, tp._arena_at = torch.zeros(4096, dtype=torch.uint8), 0
    a = tp.symmetric_empty((3, 5))                      # 30 bytes -> next slice starts 256 further
    b = tp.symmetric_empty((100,), dtype=torch.float32)  # 400 bytes -> 512
    c = tp.symmetric_empty((8, 16))
    base = tp._arena.data_ptr()
    assert (a.data_ptr() - base, b.data_ptr() - base, c.data_ptr() - base) == (0, 256, 768)
    assert a.dtype == torch.bfloat16 and tuple(a.shape) == (3, 5) and b.dtype == torch.float32 and a.is_contiguous()
    a.fill_(1.0)
    b.fill_(2.0)
    assert float(a.float().sum()) == 15.0 and float(b.sum()) == 200.0   # the slices do not overlap
    with pytest.raises(RuntimeError):
        tp.symmetric_empty((4096,))
    tp.symmetric_reset()
    assert tp.symmetric_empty((2, 2)).data_ptr() == base
