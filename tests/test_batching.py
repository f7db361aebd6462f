"""Host logic of the packed-batch producer (native `s1_pack_batch` behind `sys1_b200.batching`)."""
import numpy as np
import pytest

from sys1_b200 import batching
from sys1_b200.batching import BatcherConfig


def test_packs_in_arrival_order_until_the_budget():
    b, taken = batching.pack_next([100, 200, 300, 400], BatcherConfig(token_budget=650))
    assert taken == 3 and b.total_tokens == 600 and b.padded_tokens == 640
    assert b.cu_seqlens.tolist() == [0, 100, 300, 600]
    assert b.positions[:3].tolist() == [0, 1, 2] and b.positions[100] == 0 and b.positions[599] == 299
    assert b.lengths.tolist() == [100, 200, 300]


def test_first_request_that_does_not_fit_waits_for_the_next_batch():
    # the reference keeps the overflowing job as `pending` for the next round (src/batching.rs:90-94)
    batches = list(batching.pack_all([5000, 10, 20, 3000, 100], BatcherConfig(token_budget=2048)))
    assert [b.total_tokens for b in batches] == [5000, 30, 3000, 100]
    assert sum(b.num_sequences for b in batches) == 5


def test_exact_fill_and_empty_sequences():
    b, taken = batching.pack_next([128, 0, 128], BatcherConfig(token_budget=256, pad_multiple=128))
    assert taken == 3 and b.total_tokens == 256 and b.padded_tokens == 256
    assert b.cu_seqlens.tolist() == [0, 128, 128, 256]


def test_max_batch_size_caps_the_count():
    b, taken = batching.pack_next([1] * 50, BatcherConfig(token_budget=1000, max_batch_size=32))
    assert taken == 32 and b.total_tokens == 32


def test_negative_length_is_an_error():
    with pytest.raises(Exception):
        batching.pack_next([10, -1], BatcherConfig(token_budget=64))


@pytest.mark.parametrize("budget", [2048, 8192, 32768])
def test_synthetic_lengths_hit_the_budget_exactly(budget):
    lens = batching.synthetic_lengths(1002, 16, 512, budget)
    assert int(lens.sum()) == budget and lens.min() >= 1 and lens.max() <= 512
    again = batching.synthetic_lengths(1002, 16, 512, budget)
    assert np.array_equal(lens, again)
    b, taken = batching.pack_next(lens, BatcherConfig(token_budget=budget))
    assert taken == len(lens) and b.total_tokens == budget and b.padded_tokens == budget


def test_log_uniform_lengths():
    lens = batching.synthetic_lengths(1003, 8, 8192, 32768, log_uniform=True)
    assert int(lens.sum()) == 32768 and lens.max() <= 8192
