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
        q.put((rank, "ok"))
    except Exception as exc:  # pragma: no cover
        q.put((rank, repr(exc)))
    finally:
        dist.destroy_process_group()


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
