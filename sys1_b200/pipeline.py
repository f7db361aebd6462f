"""Host-side pipelining of a device step: while batch i is computed, batch i+1 is copied in and the result of
batch i-1 is copied out, each on its own stream. This is plumbing around the C-ABI calls (the copies are
`cudaMemcpyAsync` from / to pinned host memory issued through PyTorch), not a kernel.

The reference keeps one batch in flight (src/batching.rs:68-128: the worker awaits `predict_batch` before it
gathers the next batch); with PCIe copies of tens of megabytes per batch that serialisation, not the kernels,
would set the end-to-end rate on a B200.
"""
from __future__ import annotations

from typing import Callable, List, Sequence

import torch


class HostPipeline:
    """`depth` sets of device input buffers; `step(inputs) -> result tensor` runs on the caller's current stream.
    `result` may be one of the input buffers (an in-place step)."""

    def __init__(self, device: torch.device, input_shapes: Sequence[Sequence[int]], dtype: torch.dtype, depth: int = 2):
        self.device = device
        self.depth = depth
        self.inputs: List[List[torch.Tensor]] = [[torch.empty(tuple(s), dtype=dtype, device=device) for s in input_shapes]
                                                 for _ in range(depth)]
        self.s_in = torch.cuda.Stream(device)
        self.s_out = torch.cuda.Stream(device)
        self.in_ready = [torch.cuda.Event() for _ in range(depth)]
        self.slot_free = [torch.cuda.Event() for _ in range(depth)]   # result copied out: the slot may be refilled
        self.done = [torch.cuda.Event() for _ in range(depth)]
        self._count = 0

    def submit(self, host_inputs: Sequence[torch.Tensor], host_out: torch.Tensor,
               step: Callable[[List[torch.Tensor]], torch.Tensor]) -> None:
        """Enqueue one batch: pinned `host_inputs` -> device, `step`, result -> pinned `host_out`. Returns at once;
        `drain()` (or a later `torch.cuda.synchronize()`) joins."""
        slot = self._count % self.depth
        comp = torch.cuda.current_stream(self.device)
        if self._count >= self.depth:
            self.s_in.wait_event(self.slot_free[slot])
        with torch.cuda.stream(self.s_in):
            for dst, src in zip(self.inputs[slot], host_inputs):
                dst.copy_(src, non_blocking=True)
            self.in_ready[slot].record(self.s_in)
        comp.wait_event(self.in_ready[slot])
        result = step(self.inputs[slot])
        self.done[slot].record(comp)
        self.s_out.wait_event(self.done[slot])
        result.record_stream(self.s_out)  # the caching allocator must not hand the result's memory out before the copy ran
        with torch.cuda.stream(self.s_out):
            host_out.copy_(result, non_blocking=True)
            self.slot_free[slot].record(self.s_out)
        self._count += 1

    def drain(self) -> None:
        self.s_in.synchronize()
        torch.cuda.current_stream(self.device).synchronize()
        self.s_out.synchronize()
