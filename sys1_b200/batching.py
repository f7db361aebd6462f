"""Token-packed batches: the layout producer in front of the kernels.

The reference's `Batcher` (src/batching.rs:29-37,68-165) groups *requests* by count and question count and the
model then pads ids to `[batch, max_len]` (src/models/laya.rs:396-431). Here the same queue discipline (take
requests in arrival order until a cap is hit, leave the first one that does not fit for the next batch) is
applied to a *token* budget and the batch is emitted packed: `cu_seqlens int32[B+1]`, `positions int32[T]`,
`T` padded up to a multiple of 128 rows. The packing itself is native (`s1_pack_batch`).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Iterator, List, Sequence

import numpy as np

from . import _lib


@dataclass(frozen=True)
class BatcherConfig:
    """Caps of one batch. `max_batch_size` plays the role of the reference's field of the same name
    (src/batching.rs:29-37); `token_budget` replaces `max_batch_questions` as the size cap."""
    token_budget: int = 32768
    max_batch_size: int = 1 << 30
    pad_multiple: int = 128


@dataclass
class PackedBatch:
    cu_seqlens: np.ndarray   # int32 [B + 1]
    positions: np.ndarray    # int32 [T]
    total_tokens: int        # T
    padded_tokens: int       # T rounded up to pad_multiple

    @property
    def num_sequences(self) -> int:
        return len(self.cu_seqlens) - 1

    @property
    def lengths(self) -> np.ndarray:
        return np.diff(self.cu_seqlens)


def pack_next(lengths: Sequence[int], config: BatcherConfig) -> tuple[PackedBatch, int]:
    """Packs a prefix of `lengths` into one batch. Returns the batch and how many sequences it took."""
    lib = _lib.load_library()
    arr = np.ascontiguousarray(np.asarray(lengths, dtype=np.int32)[: config.max_batch_size])
    n = int(arr.shape[0])
    cu = np.zeros(n + 1, dtype=np.int32)
    cap = int(min(int(arr.astype(np.int64).sum()), max(config.token_budget, int(arr[0]) if n else 0)))
    pos = np.zeros(max(cap, 1), dtype=np.int32)
    taken, total, padded = C.c_int(0), C.c_int(0), C.c_int(0)
    rc = lib.s1_pack_batch(arr.ctypes.data_as(C.POINTER(C.c_int32)), n, int(config.token_budget), int(config.pad_multiple),
                           cu.ctypes.data_as(C.POINTER(C.c_int32)), pos.ctypes.data_as(C.POINTER(C.c_int32)),
                           C.byref(taken), C.byref(total), C.byref(padded))
    if rc != _lib.S1_OK:
        raise _lib.S1Error(rc, "s1_pack_batch: bad arguments (negative length, empty budget?)")
    return PackedBatch(cu[: taken.value + 1].copy(), pos[: total.value].copy(), total.value, padded.value), taken.value


def pack_all(lengths: Sequence[int], config: BatcherConfig) -> Iterator[PackedBatch]:
    """Drains a queue of sequence lengths into successive packed batches, in arrival order."""
    rest: List[int] = list(lengths)
    while rest:
        batch, taken = pack_next(rest, config)
        if taken == 0:
            raise RuntimeError("batcher made no progress")
        yield batch
        rest = rest[taken:]


def synthetic_lengths(seed: int, low: int, high: int, token_budget: int, log_uniform: bool = False) -> np.ndarray:
    """Sequence lengths for a synthetic packed batch of exactly `token_budget` tokens: draw lengths (uniform on
    [low, high], or log-uniform) until their sum reaches the budget, then truncate the last one."""
    rng = np.random.default_rng(seed)
    out: List[int] = []
    total = 0
    while total < token_budget:
        if log_uniform:
            n = int(round(float(np.exp(rng.uniform(np.log(low), np.log(high))))))
        else:
            n = int(rng.integers(low, high + 1))
        n = min(n, token_budget - total)
        out.append(n)
        total += n
    return np.asarray(out, dtype=np.int32)


# ------------------------------------------------------------------------------------------------ request batcher
class ApiError(Exception):
    """`ApiError` as the reference's batcher hands it out (src/batching.rs:222-307): 400 invalid request, 503 queue
    full / worker stopped, 504 request timed out, 500 the model failed."""

    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status, self.error = int(status), message


@dataclass(frozen=True)
class RequestBatcherConfig:
    """`BatcherConfig` (src/batching.rs:29-37) with the size caps counted in tokens: `token_budget` takes the place of
    `max_batch_questions`, `max_tokens_per_request` of `max_questions_per_request`; the other fields keep their names and
    meanings (`wait` and `response_timeout` in seconds; `response_timeout=None`: wait for ever)."""
    max_batch_size: int = 32
    token_budget: int = 32768
    max_tokens_per_request: int = 8192
    wait: float = 0.0
    queue_capacity: int = 256
    response_timeout: "float | None" = 30.0


class _Job:
    __slots__ = ("request", "tokens", "done", "result", "warmup")

    def __init__(self, request, tokens: int, warmup: bool):
        import threading
        self.request, self.tokens, self.warmup = request, tokens, warmup
        self.done = threading.Event()
        self.result = None


class RequestBatcher:
    """The reference's `Batcher` (src/batching.rs:50-307) with its admission semantics kept and its caps counted in
    tokens, so that what the worker hands to the model is one token-packed batch:

      * `predict(request)` validates (no tokens -> 400, more than `max_tokens_per_request` -> 400), enqueues without
        blocking (queue full -> 503 "inference queue is full", worker gone -> 503), then waits for its answer up to
        `response_timeout` (-> 504, the message names the timeout flag like the reference's);
      * one worker thread (the reference's task + `spawn_blocking`, :68-128) takes the first job, then gathers more until
        `max_batch_size` jobs, or `wait` has passed since the first, or the next job would push the batch over
        `token_budget` - that job is kept as `pending` and opens the next batch (:83-102);
      * `model.predict_batch(requests)` runs one batch at a time; its answers go back in order; an exception fails every
        job of the batch with 500, fewer answers than requests fail the rest with 500 (:121-163).
    `request_tokens(request)` gives a request's token count (default `len(request)`). Counters mirror the reference's
    metrics (src/metrics.rs:31-101): accepted, successful, rejected, timed_out, failed, model_failures, batches,
    batch_size_sum, batch_tokens_sum, queued, in_flight; warm-up requests are not counted (:189-215)."""

    def __init__(self, model, config: RequestBatcherConfig = RequestBatcherConfig(), request_tokens=len):
        import queue
        import threading
        self.model, self.request_tokens = model, request_tokens
        self.max_batch_size = max(1, int(config.max_batch_size))
        self.token_budget = max(1, int(config.token_budget))
        self.max_tokens_per_request = min(max(1, int(config.max_tokens_per_request)), self.token_budget)
        self.wait, self.response_timeout = max(0.0, float(config.wait)), config.response_timeout
        self._queue = queue.Queue(maxsize=max(1, int(config.queue_capacity)))
        self._lock = threading.Lock()
        self.metrics = {k: 0 for k in ("accepted", "successful", "rejected", "timed_out", "failed", "model_failures", "batches",
                                       "batch_size_sum", "batch_tokens_sum", "queued", "in_flight")}
        self.batch_token_counts: List[int] = []
        self._stopped = threading.Event()
        self._worker = threading.Thread(target=self._run, name="sys1-batcher", daemon=True)
        self._worker.start()

    # -- worker ---------------------------------------------------------------------------------------------------
    def _count(self, **deltas) -> None:
        with self._lock:
            for k, v in deltas.items():
                self.metrics[k] += v

    def _take(self, timeout):
        import queue
        try:
            job = self._queue.get(timeout=timeout) if timeout is None or timeout > 0 else self._queue.get_nowait()
        except queue.Empty:
            return None
        if job is not None and not job.warmup:
            self._count(queued=-1)
        return job

    def _run(self) -> None:
        import time
        pending = None
        while True:
            first = pending if pending is not None else self._take(None)
            pending = None
            if first is None:          # the stop marker
                break
            jobs, tokens = [first], first.tokens
            deadline = time.monotonic() + self.wait
            while len(jobs) < self.max_batch_size:
                job = self._take(deadline - time.monotonic())
                if job is None:
                    if self._stopped.is_set():
                        pending = None
                    break
                if tokens + job.tokens > self.token_budget:
                    pending = job      # opens the next batch
                    break
                tokens += job.tokens
                jobs.append(job)
            counted = [j for j in jobs if not j.warmup]
            if counted:
                self._count(batches=1, batch_size_sum=len(counted), batch_tokens_sum=sum(j.tokens for j in counted), in_flight=len(counted))
            self.batch_token_counts.append(tokens)
            try:
                responses = list(self.model.predict_batch([j.request for j in jobs]))
            except Exception as exc:  # the reference maps a failed worker to 500 for every job of the batch
                responses = [ApiError(500, str(exc)) for _ in jobs]
            failures = 0
            for i, job in enumerate(jobs):
                r = responses[i] if i < len(responses) else ApiError(500, "inference worker returned fewer responses than requests")
                if isinstance(r, Exception) and not isinstance(r, ApiError):
                    r = ApiError(500, str(r))
                failures += int(isinstance(r, ApiError) and not job.warmup)
                job.result = r
                job.done.set()
            if counted:
                self._count(model_failures=failures, in_flight=-len(counted))
            if self._stopped.is_set() and pending is None and self._queue.empty():
                break

    # -- callers --------------------------------------------------------------------------------------------------
    def is_ready(self) -> bool:
        return self._worker.is_alive() and not self._stopped.is_set()

    def warmup(self, request):
        """One request through the whole path before serving; not counted in the metrics (src/batching.rs:189-215)."""
        return self._predict(request, None, warmup=True)

    def predict(self, request):
        return self._predict(request, self.response_timeout, warmup=False)

    def _predict(self, request, response_timeout, warmup: bool):
        import queue
        tokens = int(self.request_tokens(request))
        if tokens <= 0:
            raise ApiError(400, "request must not be empty")
        if tokens > self.max_tokens_per_request:
            raise ApiError(400, f"request has {tokens} tokens; maximum is {self.max_tokens_per_request}")
        if not self.is_ready():
            raise ApiError(503, "inference worker stopped")
        job = _Job(request, tokens, warmup)
        if not warmup:
            self._count(queued=1)
        try:
            self._queue.put_nowait(job)
        except queue.Full:
            if not warmup:
                self._count(queued=-1, rejected=1)
            raise ApiError(503, "inference queue is full")
        if not warmup:
            self._count(accepted=1)
        if not job.done.wait(response_timeout):
            if not warmup:
                self._count(timed_out=1)
            raise ApiError(504, "inference request timed out; shorten the state or media, or increase --request-timeout-ms")
        if isinstance(job.result, ApiError):
            if not warmup:
                self._count(failed=1)
            raise job.result
        if not warmup:
            self._count(successful=1)
        return job.result

    def close(self) -> None:
        """Stops the worker after the jobs already queued."""
        import queue
        self._stopped.set()
        try:
            self._queue.put_nowait(None)
        except queue.Full:
            pass
        self._worker.join(timeout=5)
