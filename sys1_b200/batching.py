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
