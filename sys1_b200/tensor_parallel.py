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
    def from_process_group(cls, ordinal: int, comm_ctas: int = 0) -> "TensorParallel":
        """Builds the communicator over the ranks of `torch.distributed`'s default group (used only to carry the id).
        `comm_ctas` bounds the blocks the collective runs on (0 = NCCL's default)."""
        import torch.distributed as dist
        rank, size = dist.get_rank(), dist.get_world_size()
        box = [device.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        ctx = device.load(ordinal)
        if getattr(ctx, "comm_size", 0) != size:
            ctx.set_option("comm_ctas", comm_ctas)
            ctx.comm_init(rank, size, box[0])
        return cls(ctx, rank, size)

    def column_shard(self, weight: torch.Tensor) -> torch.Tensor:
        return device.column_parallel_shard(weight, self.rank, self.size)

    def row_shard(self, weight: torch.Tensor) -> torch.Tensor:
        return device.row_parallel_shard(weight, self.rank, self.size)


class RowParallelLinear:
    """`y = x W^T (+ residual)` with K split over the ranks: every rank multiplies its K range, the partials are
    summed in place over NVLink. `slabs` = number of row slabs the exchange is pipelined in."""

    def __init__(self, weight_shard: torch.Tensor, tp: TensorParallel, slabs: int = 4, comm_sms: int = 16):
        """`comm_sms`: SMs left free by the projections of all but the first slab, so that the all-reduce of the
        previous slab can run beside them (a persistent grid over every SM would hold it back until it ends)."""
        self.weight, self.tp, self.slabs, self.comm_sms = weight_shard, tp, max(1, int(slabs)), int(comm_sms)

    def forward(self, x_shard: torch.Tensor, residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        T, N = x_shard.shape[0], self.weight.shape[0]
        if out is None:
            out = torch.empty((T, N), dtype=torch.bfloat16, device=x_shard.device)
        if not out.is_contiguous():
            raise ValueError("the summed output must be contiguous")
        res = residual if self.tp.rank == 0 else None
        step = -(-T // self.slabs)
        step = max(128, -(-step // 128) * 128)  # whole 128-row tiles per slab
        ctx = self.tp.ctx
        share = self.tp.size > 1 and self.comm_sms > 0 and T > step
        try:
            for a in range(0, T, step):
                b = min(T, a + step)
                if share and a > 0:
                    ctx.set_option("gemm_sms", max(2, device.sm_count(ctx) - self.comm_sms))
                fused_linear(x_shard[a:b], self.weight, residual=None if res is None else res[a:b], out=out[a:b], ctx=ctx)
                if self.tp.size > 1:
                    ctx.all_reduce_(out[a:b], wait=False)
        finally:
            if share:
                ctx.set_option("gemm_sms", 0)
        if self.tp.size > 1:
            ctx.all_reduce_wait()
        return out

    __call__ = forward


class Mlp:
    """The SwiGLU MLP (`Mlp::forward`, src/archs/qwen35_text.rs:232-240) under tensor parallelism: gate / up split by
    output columns (each rank keeps matching gate and up columns), down split along K, one sum over ranks. The whole
    MLP runs slab by slab of token rows - gate/up, down, all-reduce of that slab's partial output - so that the exchange
    of a slab travels under both projections of the next one; only the last slab's exchange is exposed."""

    def __init__(self, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, tp: TensorParallel, slabs: int = 4, sharded: bool = False,
                 comm_sms: int = 16):
        """`gate`, `up` `[I, H]`, `down` `[H, I]`: the full matrices (this rank's views are taken here), or with
        `sharded=True` this rank's shards (`[I / R, H]`, `[I / R, H]`, `[H, I / R]`). `comm_sms`: SMs the projections of
        all slabs but the first leave free, so that the all-reduce of the previous slab runs beside them (a persistent
        grid over every SM would hold the collective's blocks back until it ends)."""
        self.tp, self.slabs, self.comm_sms = tp, max(1, int(slabs)), int(comm_sms)
        self.gate, self.up = (gate, up) if sharded else (tp.column_shard(gate), tp.column_shard(up))
        self.down = down if sharded else tp.row_shard(down)

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                exchange: bool = True) -> torch.Tensor:
        T, N = x.shape[0], self.down.shape[0]
        ctx = self.tp.ctx
        if out is None:
            out = torch.empty((T, N), dtype=torch.bfloat16, device=x.device)
        if not out.is_contiguous():
            raise ValueError("the summed output must be contiguous")
        res = residual if self.tp.rank == 0 else None
        step = max(128, -(-(-(-T // self.slabs)) // 128) * 128)  # whole 128-row tiles per slab
        h = torch.empty((min(step, T), self.gate.shape[0]), dtype=torch.bfloat16, device=x.device)
        share = exchange and self.tp.size > 1 and self.comm_sms > 0 and T > step
        try:
            for a in range(0, T, step):
                b = min(T, a + step)
                if share and a > 0:
                    ctx.set_option("gemm_sms", max(2, device.sm_count(ctx) - self.comm_sms))
                fused_linear(x[a:b], self.gate, weight_up=self.up, epilogue=EPI_SWIGLU, out=h[: b - a], ctx=ctx)
                fused_linear(h[: b - a], self.down, residual=None if res is None else res[a:b], out=out[a:b], ctx=ctx)
                if exchange and self.tp.size > 1:
                    ctx.all_reduce_(out[a:b], wait=False)
        finally:
            if share:
                ctx.set_option("gemm_sms", 0)
        if exchange and self.tp.size > 1:
            ctx.all_reduce_wait()
        return out

    __call__ = forward
