"""Tensor-parallel projections of the large hybrid model: column-parallel input projections, row-parallel output
projections and the one exchange step they need, a bf16 sum over the ranks.

The reference runs on one GPU (`device::load`, src/device.rs:43-56) and has no counterpart of this module; the
layers sharded here are its `Mlp` (src/archs/qwen35_text.rs:211-240), the attention projections (:266-285) and the
linear-attention projections (:437-489). One process per GPU; rank r owns
  * column-parallel weights: the rows `[r N / R, (r + 1) N / R)` of `W [N, K]` (a view: no copy), producing its
    share of the output features (heads, or gate/up columns);
  * row-parallel weights: the columns `[r K / R, (r + 1) K / R)` of `W [N, K]` (a strided view handed to the library
    through `ldw`: no copy), producing a partial `[T, N]` that is summed over ranks.
The residual stream is added by rank 0's projection epilogue only, so the sum over ranks yields `x + sum_r partial_r`
without a separate add. The sum is issued slab by slab of token rows (`s1_allreduce_bf16` on the context's
communication stream), so that the exchange of one slab overlaps the projection of the next.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import device
from ._lib import EPI_SWIGLU
from .linear import fused_linear


class TensorParallel:
    """Rank / size and the context that owns the communicator."""

    def __init__(self, ctx: device.Context, rank: int, size: int):
        self.ctx, self.rank, self.size = ctx, int(rank), int(size)

    @classmethod
    def from_process_group(cls, ordinal: int) -> "TensorParallel":
        """Builds the communicator over the ranks of `torch.distributed`'s default group (used only to carry the id)."""
        import torch.distributed as dist
        rank, size = dist.get_rank(), dist.get_world_size()
        box = [device.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        ctx = device.load(ordinal)
        if getattr(ctx, "comm_size", 0) != size:
            ctx.comm_init(rank, size, box[0])
        return cls(ctx, rank, size)

    def column_shard(self, weight: torch.Tensor) -> torch.Tensor:
        return device.column_parallel_shard(weight, self.rank, self.size)

    def row_shard(self, weight: torch.Tensor) -> torch.Tensor:
        return device.row_parallel_shard(weight, self.rank, self.size)


class RowParallelLinear:
    """`y = x W^T (+ residual)` with K split over the ranks: every rank multiplies its K range, the partials are
    summed in place over NVLink. `slabs` = number of row slabs the exchange is pipelined in."""

    def __init__(self, weight_shard: torch.Tensor, tp: TensorParallel, slabs: int = 4):
        self.weight, self.tp, self.slabs = weight_shard, tp, max(1, int(slabs))

    def forward(self, x_shard: torch.Tensor, residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        T, N = x_shard.shape[0], self.weight.shape[0]
        if out is None:
            out = torch.empty((T, N), dtype=torch.bfloat16, device=x_shard.device)
        if not out.is_contiguous():
            raise ValueError("the summed output must be contiguous")
        res = residual if self.tp.rank == 0 else None
        step = -(-T // self.slabs)
        step = max(128, -(-step // 128) * 128)  # whole 128-row tiles per slab
        for a in range(0, T, step):
            b = min(T, a + step)
            fused_linear(x_shard[a:b], self.weight, residual=None if res is None else res[a:b], out=out[a:b], ctx=self.tp.ctx)
            if self.tp.size > 1:
                self.tp.ctx.all_reduce_(out[a:b], wait=False)
        if self.tp.size > 1:
            self.tp.ctx.all_reduce_wait()
        return out

    __call__ = forward


class Mlp:
    """The SwiGLU MLP (`Mlp::forward`, src/archs/qwen35_text.rs:232-240) under tensor parallelism: gate / up split by
    output columns (each rank keeps matching gate and up columns), down split along K, one all-reduce."""

    def __init__(self, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, tp: TensorParallel, slabs: int = 4):
        self.tp = tp
        self.gate, self.up = tp.column_shard(gate), tp.column_shard(up)
        self.down = RowParallelLinear(tp.row_shard(down), tp, slabs)

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        h = fused_linear(x, self.gate, weight_up=self.up, epilogue=EPI_SWIGLU, ctx=self.tp.ctx)
        return self.down(h, residual=residual, out=out)

    __call__ = forward
