"""GPU discovery and per-GPU contexts.

Mirrors `src/device.rs:43-56` of the reference (`load()` → device 0) but for a node of B200s:
`device_count()` enumerates the GPUs, `load(ordinal)` opens one context per GPU. A context wraps an `s1_ctx`
of the C ABI, bound to a CUDA stream (by default the stream PyTorch considers current at creation time, so the
library's work is ordered with the tensors' producers and consumers).
"""
from __future__ import annotations

import ctypes as C
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

    def launch_count(self) -> int:
        return int(self._lib.s1_launch_count(self.handle))

    def set_option(self, name: str, value: int) -> None:
        self.check(self._lib.s1_set_option(self.handle, name.encode(), int(value)))

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


def load(ordinal: Optional[int] = None) -> Context:
    """Context for GPU `ordinal` (default: PyTorch's current device) on PyTorch's current stream."""
    if ordinal is None:
        ordinal = torch.cuda.current_device()
    stream = torch.cuda.current_stream(ordinal)
    key = (int(ordinal), int(stream.cuda_stream))
    ctx = _contexts.get(key)
    if ctx is None:
        ctx = Context(ordinal, stream)
        _contexts[key] = ctx
    return ctx
