"""Host-side argument checks that need no GPU: every operator of the package refuses CPU tensors (there is no CPU
path to fall back to), and the sharding helpers of the tensor-parallel layers produce views of the right shape."""
import numpy as np
import pytest
import torch

from sys1_b200 import device, linear, modernbert, norm, qwen35


def test_operators_refuse_cpu_tensors():
    x = torch.zeros(4, 64, dtype=torch.bfloat16)
    w = torch.zeros(64, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        norm.norm(x, w, 1e-5)
    with pytest.raises(ValueError):
        norm.rope_(x, torch.zeros(8, 32), torch.zeros(8, 32), torch.zeros(4, dtype=torch.int32), 1, 64, 64)
    with pytest.raises(ValueError):
        linear.fused_linear(x, torch.zeros(8, 64, dtype=torch.bfloat16))
    with pytest.raises(ValueError):
        linear.linear_rope(x, torch.zeros(192, 64, dtype=torch.bfloat16), torch.zeros(8, 32), torch.zeros(8, 32),
                           torch.zeros(4, dtype=torch.int32), 2)
    q = torch.zeros(4, 2, 64, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        modernbert.attention_varlen(q, q, q, np.array([0, 4], dtype=np.int32))
    q256 = torch.zeros(4, 2, 256, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        qwen35.attention_causal_gqa(q256, q256, q256, np.array([0, 4], dtype=np.int32))


def test_shard_views():
    w = torch.arange(16 * 32, dtype=torch.float32).reshape(16, 32)
    for rank in range(4):
        col = device.column_parallel_shard(w, rank, 4)
        row = device.row_parallel_shard(w, rank, 4)
        assert col.shape == (4, 32) and torch.equal(col, w[4 * rank:4 * rank + 4])
        assert row.shape == (16, 8) and torch.equal(row, w[:, 8 * rank:8 * rank + 8])
        assert col.data_ptr() == w[4 * rank].data_ptr() and row.stride(0) == 32  # views: no copies
    paired = device.column_parallel_shard(w, 1, 2, pairs=2)  # GeGLU halves: the same range of each half
    assert torch.equal(paired, torch.cat([w[4:8], w[12:16]]))
    with pytest.raises(ValueError):
        device.column_parallel_shard(w, 0, 3)
    with pytest.raises(ValueError):
        device.row_parallel_shard(w, 0, 3)


def test_deduplicate_keeps_first_occurrences_in_order():
    """`deduplicate` of src/models/laya.rs:689-707: representatives in order of first appearance, one index per input."""
    from sys1_b200 import laya
    a, b, c = ("kind0", (1, 2, 3), (0, 2)), ("kind0", (1, 2, 3), (0, 1)), ("kind1", (1, 2, 3), (0, 2))
    unique, indices = laya.deduplicate([a, b, a, c, b, a])
    assert unique == [a, b, c]
    assert indices == [0, 1, 0, 2, 1, 0]
    assert laya.deduplicate([]) == ([], [])


def test_marker_rows_on_the_packed_layout():
    from sys1_b200 import laya
    rows, counts = laya.marker_rows([0, 5, 5, 12], [[0, 4], [], [6, 1, 1]])
    assert rows.tolist() == [0, 4, 11, 6, 6] and counts == [2, 0, 3]
    with pytest.raises(ValueError):
        laya.marker_rows([0, 5], [[5]])          # position past the end of its sequence
    with pytest.raises(ValueError):
        laya.marker_rows([0, 5, 9], [[0]])       # one marker list per sequence
