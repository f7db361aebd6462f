"""GPU discovery and per-GPU contexts.

Mirrors `src/device.rs:43-56` of the reference (`load()` → device 0) but for a node of B200s:
`device_count()` enumerates the GPUs, `load(ordinal)` opens one context per GPU. A context wraps an `s1_ctx`
of the C ABI, bound to a CUDA stream (by default the stream PyTorch considers current at creation time, so the
library's work is ordered with the tensors' producers and consumers).
"""
from __future__ import annotations

import ctypes as C
import weakref
from typing import Dict, Optional, Tuple

import torch

from . import _lib
from ._lib import S1Error


def validate_available() -> None:
    """Same contract as `device::validate_available` (src/device.rs:3-15): raise if no usable GPU."""
    if device_count() <= 0:
        raise RuntimeError("CUDA backend selected, but no CUDA device is available")


def device_count() -> int:
    lib = _lib.load_library()
    n = C.c_int(0)
    lib.s1_device_count(C.byref(n))
    return int(n.value)


class Context:
    """Owner of one `s1_ctx`. Not thread-safe: one host thread at a time, like one `predict_batch` at a time."""

    def __init__(self, ordinal: int = 0, stream: Optional[torch.cuda.Stream] = None):
        self._lib = _lib.load_library()
        self.ordinal = int(ordinal)
        if stream is None:
            stream = torch.cuda.current_stream(self.ordinal)
        self.stream = stream
        handle = C.c_void_p()
        rc = self._lib.s1_ctx_create(self.ordinal, C.c_void_p(stream.cuda_stream), C.byref(handle))
        if rc != _lib.S1_OK:
            raise S1Error(rc, f"s1_ctx_create(device={ordinal}) failed; an sm_100 GPU is required, there is no fallback")
        self._h = handle

    # -- plumbing ---------------------------------------------------------------------------------
    @property
    def handle(self) -> C.c_void_p:
        if self._h is None:
            raise RuntimeError("context already destroyed")
        return self._h

    def check(self, rc: int) -> None:
        if rc != _lib.S1_OK:
            raise S1Error(rc, self._lib.s1_last_error(self.handle).decode("utf-8", "replace"))

    def sync(self) -> None:
        self.check(self._lib.s1_sync(self.handle))

    def workspace(self, nbytes: int) -> torch.Tensor:
        """Device scratch of this context (uint8, 1024-byte aligned start, at least `nbytes`), grown on demand. It
        belongs to the context - that is, to one stream - so kernels that use it are ordered one after the other; two
        contexts on one GPU never share it. The library itself allocates nothing: a Rust caller would hand it a
        buffer from candle's pool the same way."""
        ws = getattr(self, "_ws", None)
        if ws is None or ws.numel() < nbytes + 1024:
            ws = torch.empty(max(nbytes + 1024, 1 << 16), dtype=torch.uint8, device=torch.device("cuda", self.ordinal))
            self._ws = ws
        off = (-ws.data_ptr()) % 1024
        return ws[off:]

    # -- batch plans ------------------------------------------------------------------------------
    def batch_plan(self, cu_seqlens_host, total_tokens: int) -> torch.Tensor:
        """Builds the per-batch tables of the attention / delta-rule kernels once (`s1_batch_plan`) and returns the
        device buffer that holds them; `use_plan(plan)` then lets every layer's calls skip their own table copy."""
        import numpy as np
        cu = np.ascontiguousarray(cu_seqlens_host, dtype=np.int32)
        need = int(self._lib.s1_batch_plan_bytes(len(cu) - 1, int(total_tokens)))
        buf = torch.empty(need + 256, dtype=torch.uint8, device=torch.device("cuda", self.ordinal))
        plan = buf[(-buf.data_ptr()) % 256:]
        self.check(self._lib.s1_batch_plan(self.handle, cu.ctypes.data_as(C.POINTER(C.c_int32)), len(cu) - 1, int(total_tokens),
                                           C.c_void_p(plan.data_ptr()), need))
        plan._s1_shape = (len(cu) - 1, int(total_tokens))   # (num_seqs, total_tokens) the plan describes
        plan._s1_owner = buf
        # the context forgets the plan when the tensor goes (its memory may then hold anything)
        weakref.finalize(plan, Context._release_plan, weakref.ref(self), plan.data_ptr())
        return plan

    @staticmethod
    def _release_plan(ctx_ref, pointer: int) -> None:
        ctx = ctx_ref()
        if ctx is not None and getattr(ctx, "_h", None) is not None:
            ctx._lib.s1_batch_plan_release(ctx._h, C.c_void_p(pointer))

    def use_plan(self, plan: Optional[torch.Tensor]) -> None:
        self.check(self._lib.s1_use_batch_plan(self.handle, C.c_void_p(0 if plan is None else plan.data_ptr())))
        self._plan = plan

    def plan_covers(self, num_seqs: int, total_tokens: int) -> bool:
        """Whether the plan in use describes a batch of this shape (the caller vouches that it is the same batch)."""
        plan = getattr(self, "_plan", None)
        return plan is not None and plan._s1_shape == (int(num_seqs), int(total_tokens))

    def launch_count(self) -> int:
        return int(self._lib.s1_launch_count(self.handle))

    def set_option(self, name: str, value: int) -> None:
        self.check(self._lib.s1_set_option(self.handle, name.encode(), int(value)))

    # -- tensor-parallel exchange -----------------------------------------------------------------
    def comm_init(self, rank: int, size: int, unique_id: bytes) -> None:
        """Collective: every rank calls it with the id rank 0 got from `comm_unique_id()`."""
        if len(unique_id) != _lib.COMM_ID_BYTES:
            raise ValueError("the communicator id has 128 bytes")
        buf = C.create_string_buffer(unique_id, _lib.COMM_ID_BYTES)
        self.check(self._lib.s1_comm_init(self.handle, C.cast(buf, C.c_void_p), int(rank), int(size)))
        self.comm_rank, self.comm_size = int(rank), int(size)

    def exchange_register(self, rank: int, size: int, local_base: int, multicast_base: int, nbytes: int, flag_ptrs) -> None:
        """`s1_exchange_register`: sums of buffers inside `[local_base, local_base + nbytes)` (symmetric memory with a
        multicast mapping) run as this library's own NVSwitch kernel. `flag_ptrs[r]` = rank r's zeroed flag array as
        mapped on this GPU."""
        if len(flag_ptrs) != size:
            raise ValueError("one flag array per rank")
        arr = (C.c_void_p * size)(*[int(p) for p in flag_ptrs])
        self.check(self._lib.s1_exchange_register(self.handle, int(rank), int(size), C.c_void_p(int(local_base)),
                                                  C.c_void_p(int(multicast_base)), int(nbytes), arr, _lib.EXCHANGE_FLAG_BYTES))

    def all_reduce_(self, t: torch.Tensor, wait: bool = True) -> torch.Tensor:
        """In-place bf16 sum over the ranks (`s1_allreduce_bf16`), after the work queued on this context's stream.
        With `wait=False` the context's stream is not held back: call `all_reduce_wait()` before using `t`."""
        if not t.is_cuda or t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise ValueError("all_reduce_ takes a contiguous bf16 CUDA tensor")
        self.check(self._lib.s1_allreduce_bf16(self.handle, C.c_void_p(t.data_ptr()), t.numel()))
        if wait:
            self.all_reduce_wait()
        return t

    def all_reduce_wait(self) -> None:
        self.check(self._lib.s1_allreduce_wait(self.handle))

    def all_reduce_async_(self, t: torch.Tensor) -> int:
        """Issues the in-place sum over the ranks and returns its ticket; the context's stream is not held back.
        `all_reduce_wait_ticket(ticket)` orders the stream after this sum alone (later ones may still be in flight)."""
        self.all_reduce_(t, wait=False)
        return int(self._lib.s1_allreduce_ticket(self.handle))

    def all_reduce_wait_ticket(self, ticket: int) -> None:
        self.check(self._lib.s1_allreduce_wait_ticket(self.handle, int(ticket)))

    def close(self) -> None:
        if getattr(self, "_h", None) is not None:
            self._lib.s1_ctx_destroy(self._h)
            self._h = None

    def __del__(self):  # pragma: no cover - best effort
        try:
            self.close()
        except Exception:
            pass


_contexts: Dict[Tuple[int, int], Context] = {}


def sm_count(ctx: "Context") -> int:
    """Streaming multiprocessors of the context's GPU."""
    return torch.cuda.get_device_properties(ctx.ordinal).multi_processor_count


def comm_unique_id() -> bytes:
    """The id rank 0 creates and hands to every rank's `Context.comm_init` (over any channel)."""
    lib = _lib.load_library()
    buf = C.create_string_buffer(_lib.COMM_ID_BYTES)
    err = C.create_string_buffer(256)
    rc = lib.s1_comm_unique_id(C.cast(buf, C.c_void_p), err, 256)
    if rc != _lib.S1_OK:
        raise S1Error(rc, err.value.decode("utf-8", "replace"))
    return buf.raw


def load(ordinal: Optional[int] = None) -> Context:
    """Context for GPU `ordinal` (default: PyTorch's current device) on PyTorch's current stream."""
    if ordinal is None:
        ordinal = torch.cuda.current_device()
    stream = torch.cuda.current_stream(ordinal)
    key = (ordinal, stream.cuda_stream)
    ctx = _contexts.get(key)
    if ctx is None:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("no context exists for the capturing stream yet: call device.load() on that stream once "
                               "before the capture starts (creating a context allocates)")
        ctx = Context(ordinal, stream)
        _contexts[key] = ctx
    return ctx


# ------------------------------------------------------------------------------------------------ multi-GPU
def shard_sequences(lengths, world_size: int, rank: int):
    """Indices of the sequences replica `rank` serves: whole sequences, assigned longest-first to the replica with
    the fewest tokens so far (sequences never interact, so replicas need no collective). Deterministic on every
    rank; ties go to the lower rank."""
    import numpy as np
    lengths = np.asarray(lengths, dtype=np.int64)
    order = np.argsort(-lengths, kind="stable")
    loads = [0] * world_size
    mine = []
    for idx in order:
        r = min(range(world_size), key=lambda i: (loads[i], i))
        loads[r] += int(lengths[idx])
        if r == rank:
            mine.append(int(idx))
    return sorted(mine)


def column_parallel_shard(weight: torch.Tensor, rank: int, world_size: int, pairs: int = 1) -> torch.Tensor:
    """Row range of `weight [N, K]` owned by `rank` (its share of the output features). With `pairs = 2` the matrix
    is two stacked halves (GeGLU's activated / gate rows) and the rank takes the same range of each half.
    Single-half shards are views (passed to the library through `ldw`, no copy)."""
    n = weight.shape[0] // pairs
    if n % world_size:
        raise ValueError(f"{n} output features do not split over {world_size} ranks")
    lo, hi = rank * n // world_size, (rank + 1) * n // world_size
    if pairs == 1:
        return weight[lo:hi]
    return torch.cat([weight[h * n + lo:h * n + hi] for h in range(pairs)])


def row_parallel_shard(weight: torch.Tensor, rank: int, world_size: int) -> torch.Tensor:
    """K range of `weight [N, K]` owned by `rank` (a strided view; its partial product needs a sum over ranks)."""
    k = weight.shape[1]
    if k % (8 * world_size):
        raise ValueError(f"K={k} does not split over {world_size} ranks in multiples of 8")
    return weight[:, rank * k // world_size:(rank + 1) * k // world_size]


def all_reduce_sum_(t: torch.Tensor) -> torch.Tensor:
    """Sum over the ranks of the default process group (NCCL on GPUs, gloo on CPU): the exchange step that follows
    a row-parallel projection."""
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return t
