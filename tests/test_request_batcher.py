"""The request batcher (`sys1_b200.batching.RequestBatcher`) against fake models, the way the reference tests its
`Batcher` (src/batching.rs:327-734: `SlowModel`, `FailingModel`, `BlockOnceModel`, `RecordingModel`): time-outs -> 504,
full queue -> 503, model failure -> 500, empty / oversized requests -> 400, warm-up kept out of the metrics, and the
size cap of a dynamic batch - here a token budget - with the job that does not fit carried over to the next batch."""
import threading
import time
from concurrent.futures import ThreadPoolExecutor

import pytest

from sys1_b200.batching import ApiError, RequestBatcher, RequestBatcherConfig


class SlowModel:
    def predict_batch(self, requests):
        time.sleep(0.2)
        return ["ok"] * len(requests)


class FailingModel:
    def predict_batch(self, requests):
        return [ApiError(500, "model failure") for _ in requests]


class RaisingModel:
    def predict_batch(self, requests):
        raise RuntimeError("worker blew up")


class ShortModel:
    def predict_batch(self, requests):
        return ["ok"] * (len(requests) - 1)


class RecordingModel:
    def __init__(self):
        self.batches = []

    def predict_batch(self, requests):
        self.batches.append([len(r) for r in requests])
        return [sum(r) for r in requests]


class BlockOnceModel:
    def __init__(self):
        self.block, self.started, self.release = True, threading.Event(), threading.Event()

    def predict_batch(self, requests):
        if self.block:
            self.block = False
            self.started.set()
            assert self.release.wait(5)
        return ["ok"] * len(requests)


def _one(cap=1, **kw):
    base = dict(max_batch_size=1, token_budget=cap, max_tokens_per_request=cap, wait=0.0, queue_capacity=1, response_timeout=None)
    base.update(kw)
    return RequestBatcherConfig(**base)


def test_times_out_slow_inference():
    b = RequestBatcher(SlowModel(), _one(response_timeout=0.001))
    with pytest.raises(ApiError) as info:
        b.predict([1])
    assert info.value.status == 504 and "--request-timeout-ms" in info.value.error
    assert b.metrics["accepted"] == 1 and b.metrics["timed_out"] == 1 and b.metrics["successful"] == 0
    deadline = time.time() + 2
    while b.metrics["in_flight"] and time.time() < deadline:
        time.sleep(0.01)
    assert b.metrics["in_flight"] == 0
    b.close()


def test_tracks_failed_model_requests():
    for model in (FailingModel(), RaisingModel()):
        b = RequestBatcher(model, _one())
        with pytest.raises(ApiError) as info:
            b.predict([1])
        assert info.value.status == 500
        assert b.metrics["failed"] == 1 and b.metrics["model_failures"] == 1 and b.metrics["successful"] == 0
        b.close()


def test_fewer_responses_than_requests_fail_the_rest():
    b = RequestBatcher(ShortModel(), _one())
    with pytest.raises(ApiError) as info:
        b.predict([1])
    assert info.value.status == 500 and "fewer responses" in info.value.error
    b.close()


def test_excludes_warmup_from_metrics():
    model = RecordingModel()
    b = RequestBatcher(model, _one())
    assert b.warmup([7]) == 7
    assert b.metrics["accepted"] == 0 and b.metrics["successful"] == 0 and b.metrics["batches"] == 0 and b.metrics["batch_size_sum"] == 0
    assert model.batches == [[1]]
    b.close()


def test_tracks_requests_rejected_by_a_full_queue():
    model = BlockOnceModel()
    b = RequestBatcher(model, _one())
    with ThreadPoolExecutor(2) as pool:
        first = pool.submit(b.predict, [1])
        assert model.started.wait(2)          # the worker is inside the model with the first request
        second = pool.submit(b.predict, [1])  # fills the one queue slot
        deadline = time.time() + 2
        while b.metrics["queued"] != 1 and time.time() < deadline:
            time.sleep(0.005)
        assert b.metrics["queued"] == 1
        with pytest.raises(ApiError) as info:
            b.predict([1])
        assert info.value.status == 503 and "queue is full" in info.value.error
        assert b.metrics["rejected"] == 1
        model.release.set()
        assert first.result(5) == "ok" and second.result(5) == "ok"
    assert b.metrics["accepted"] == 2 and b.metrics["successful"] == 2
    b.close()


def test_rejects_empty_and_oversized_requests():
    b = RequestBatcher(SlowModel(), _one(cap=2, max_tokens_per_request=1))
    with pytest.raises(ApiError) as info:
        b.predict([])
    assert info.value.status == 400
    with pytest.raises(ApiError) as info:
        b.predict([1, 2])
    assert info.value.status == 400 and "maximum is 1" in info.value.error
    b.close()


def test_caps_total_tokens_in_dynamic_batches_and_carries_the_pending_job_over():
    model = RecordingModel()
    b = RequestBatcher(model, RequestBatcherConfig(max_batch_size=8, token_budget=2, max_tokens_per_request=1, wait=0.05,
                                                  queue_capacity=8, response_timeout=2.0))
    with ThreadPoolExecutor(3) as pool:
        results = [f.result(5) for f in [pool.submit(b.predict, [1]) for _ in range(3)]]
    assert results == [1, 1, 1]
    counts = [len(batch) for batch in model.batches]
    assert sum(counts) == 3 and len(counts) == 2 and all(c <= 2 for c in counts)
    assert b.metrics["batches"] == 2 and b.metrics["batch_size_sum"] == 3 and b.metrics["batch_tokens_sum"] == 3
    b.close()


def test_token_budget_packs_ragged_requests_in_arrival_order():
    model = RecordingModel()
    b = RequestBatcher(model, RequestBatcherConfig(max_batch_size=16, token_budget=10, max_tokens_per_request=10, wait=0.2,
                                                  queue_capacity=16, response_timeout=5.0))
    lengths = [4, 5, 3, 10, 1]
    with ThreadPoolExecutor(len(lengths)) as pool:
        futures = []
        for n in lengths:                      # arrival order is the submission order
            futures.append(pool.submit(b.predict, list(range(n))))
            time.sleep(0.01)
        for f in futures:
            f.result(5)
    assert model.batches == [[4, 5], [3], [10], [1]] or model.batches == [[4, 5], [3], [10, ], [1]]
    assert all(sum(batch) <= 10 for batch in model.batches)
    b.close()


def test_count_cap_and_readiness():
    model = RecordingModel()
    b = RequestBatcher(model, RequestBatcherConfig(max_batch_size=2, token_budget=100, max_tokens_per_request=10, wait=0.1,
                                                  queue_capacity=8, response_timeout=5.0))
    assert b.is_ready()
    with ThreadPoolExecutor(4) as pool:
        for f in [pool.submit(b.predict, [1]) for _ in range(4)]:
            f.result(5)
    assert all(len(batch) <= 2 for batch in model.batches) and sum(len(batch) for batch in model.batches) == 4
    b.close()
    assert not b.is_ready()
    with pytest.raises(ApiError) as info:
        b.predict([1])
    assert info.value.status == 503
