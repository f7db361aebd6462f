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
from ._lib import EPI_SWIGLU, EXCHANGE_FLAG_BYTES
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

    def symmetric_arena(self, nbytes: int, group=None) -> None:
        """Collective. Allocates `nbytes` of symmetric memory (the same buffer on every rank plus its NVLink multicast
        mapping, from `torch.distributed._symmetric_memory`) and registers it with the context: sums of tensors carved
        out of it by `symmetric_empty` run as the library's own in-switch reduction kernel instead of the NCCL call.
        Torch only allocates and maps the memory; no torch collective touches it."""
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        group = dist.group.WORLD if group is None else group
        dev = torch.device("cuda", self.ctx.ordinal)
        nbytes = -(-int(nbytes) // 256) * 256
        arena = symm.empty(nbytes, dtype=torch.uint8, device=dev)
        arena_handle = symm.rendezvous(arena, group)
        flags = symm.empty(EXCHANGE_FLAG_BYTES // 4, dtype=torch.int32, device=dev)
        flags.zero_()
        flags_handle = symm.rendezvous(flags, group)
        if not arena_handle.multicast_ptr:
            raise RuntimeError("symmetric memory without a multicast mapping: the in-switch reduction needs NVSwitch")
        torch.cuda.synchronize(dev)
        dist.barrier(group)  # every rank's flags are zero before anyone can raise one
        self.ctx.exchange_register(self.rank, self.size, arena.data_ptr(), arena_handle.multicast_ptr, nbytes,
                                   [flags_handle.buffer_ptrs[r] for r in range(self.size)])
        self._arena, self._arena_at, self._arena_keep = arena, 0, (arena_handle, flags, flags_handle)

    def symmetric_empty(self, shape, dtype=torch.bfloat16) -> torch.Tensor:
        """A tensor inside the registered arena (256-byte aligned; a bump allocator: `symmetric_reset` frees all).
        Every rank must carve the same sequence of shapes, so that a tensor sits at the same offset everywhere."""
        arena = getattr(self, "_arena", None)
        if arena is None:
            raise RuntimeError("call symmetric_arena first")
        count = 1
        for d in shape:
            count *= int(d)
        nbytes = count * torch.empty((), dtype=dtype).element_size()
        if self._arena_at + nbytes > arena.numel():
            raise RuntimeError(f"symmetric arena of {arena.numel()} bytes is full ({self._arena_at} used, {nbytes} asked)")
        t = arena[self._arena_at:self._arena_at + nbytes].view(dtype).view(*shape)
        self._arena_at += -(-nbytes // 256) * 256
        return t

    def symmetric_reset(self) -> None:
        self._arena_at = 0

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

    def forward(self, x_shard: torch.Tensor, residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                exchange: bool = True) -> torch.Tensor:
        """`out` may be `residual` (the replicated residual stream updated in place on every rank: rank 0 adds into it,
        the other ranks overwrite it with their partial product, the sum over ranks restores `x + ...` everywhere).
        `exchange=False` skips the sum (timing the local math alone)."""
        T, N = x_shard.shape[0], self.weight.shape[0]
        if out is None:
            out = torch.empty((T, N), dtype=torch.bfloat16, device=x_shard.device)
        if not out.is_contiguous():
            raise ValueError("the summed output must be contiguous")
        res = residual if self.tp.rank == 0 else None
        step = -(-T // self.slabs)
        step = max(128, -(-step // 128) * 128)  # whole 128-row tiles per slab
        ctx = self.tp.ctx
        beside = exchange and self.tp.size > 1 and T > step   # a slab's sum runs beside the next slab's projections
        share = beside and self.comm_sms > 0
        if beside:
            ctx.set_option("dynamic_tiles", 1)   # a projection CTA held up by the collective's blocks must not hold up the launch
        try:
            for a in range(0, T, step):
                b = min(T, a + step)
                if share and a > 0:
                    ctx.set_option("gemm_sms", max(2, device.sm_count(ctx) - self.comm_sms))
                fused_linear(x_shard[a:b], self.weight, residual=None if res is None else res[a:b], out=out[a:b], ctx=ctx)
                if exchange and self.tp.size > 1:
                    ctx.all_reduce_(out[a:b], wait=False)
        finally:
            if beside:
                ctx.set_option("dynamic_tiles", 0)
            if share:
                ctx.set_option("gemm_sms", 0)
        if exchange and self.tp.size > 1:
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
        beside = exchange and self.tp.size > 1 and T > step   # a slab's sum runs beside the next slab's projections
        share = beside and self.comm_sms > 0
        if beside:
            ctx.set_option("dynamic_tiles", 1)   # a projection CTA held up by the collective's blocks must not hold up the launch
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
            if beside:
                ctx.set_option("dynamic_tiles", 0)
            if share:
                ctx.set_option("gemm_sms", 0)
        if exchange and self.tp.size > 1:
            ctx.all_reduce_wait()
        return out

    __call__ = forward


# ------------------------------------------------------------------------------------------------ whole layers
def local_heads(cfg, size: int):
    """Head counts one rank of `size` owns: (query heads, KV heads, delta-rule key heads, delta-rule value heads).
    Query heads and delta-rule value heads are split evenly; the delta-rule key heads follow their value heads (the
    repeat factor `Hv / Hk` is the same on every rank, src/archs/qwen35_text.rs:552-559); with fewer KV heads than ranks
    a rank holds the one KV head its query heads read (`repeat_kv`, :363-369) - KV heads are then replicated."""
    H, KV, Hk, Hv = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.linear_num_key_heads, cfg.linear_num_value_heads
    if H % size or Hk % size or Hv % size:
        raise ValueError(f"{H} query / {Hk} key / {Hv} value heads do not split over {size} ranks")
    Hr, group = H // size, H // KV
    if KV % size == 0:
        KVr = KV // size
    elif group % Hr == 0:
        KVr = 1
    else:
        raise ValueError(f"{KV} KV heads cannot serve {size} ranks of {Hr} query heads")
    return Hr, KVr, Hk // size, Hv // size


def shard_layer_weights(w, prefix: str, cfg, layer_type: str, rank: int, size: int):
    """The tensors of one decoder layer as rank `rank` of `size` holds them, under the layer's own names (`prefix`
    stripped): column-parallel projections are row ranges of the full matrices (heads, or matching gate / up columns),
    row-parallel ones (`o_proj`, `out_proj`, `down_proj`) K ranges taken as strided views - the library reads them through
    `ldw`, nothing is copied - and the per-head vectors (`A_log`, `dt_bias`, conv channels) follow their heads. Norm weights
    are replicated. Works on any device (the shard arithmetic is checked on CPU against the oracle)."""
    Hr, KVr, Hkr, Hvr = local_heads(cfg, size)
    H, KV, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    Hk, Hv = cfg.linear_num_key_heads, cfg.linear_num_value_heads
    g = lambda name: w[prefix + name]
    out = {"input_layernorm": g("input_layernorm"), "post_attention_layernorm": g("post_attention_layernorm")}
    inter = g("mlp.gate_proj").shape[0]
    if inter % size:
        raise ValueError(f"intermediate size {inter} does not split over {size} ranks")
    lo, hi = rank * inter // size, (rank + 1) * inter // size
    out["mlp.gate_proj"], out["mlp.up_proj"] = g("mlp.gate_proj")[lo:hi], g("mlp.up_proj")[lo:hi]
    out["mlp.down_proj"] = g("mlp.down_proj")[:, lo:hi]
    if layer_type == "full_attention":
        a = "self_attn."
        kv0 = (rank * Hr) // (H // KV) if KV % size else rank * KVr   # first KV head this rank's query heads read
        out[a + "q_proj"] = g(a + "q_proj")[rank * Hr * 2 * D:(rank + 1) * Hr * 2 * D]
        out[a + "k_proj"] = g(a + "k_proj")[kv0 * D:(kv0 + KVr) * D]
        out[a + "v_proj"] = g(a + "v_proj")[kv0 * D:(kv0 + KVr) * D]
        out[a + "o_proj"] = g(a + "o_proj")[:, rank * Hr * D:(rank + 1) * Hr * D]
        out[a + "q_norm"], out[a + "k_norm"] = g(a + "q_norm"), g(a + "k_norm")
    else:
        a = "linear_attn."
        kq = slice(rank * Hkr * 128, (rank + 1) * Hkr * 128)
        kk = slice(Hk * 128 + rank * Hkr * 128, Hk * 128 + (rank + 1) * Hkr * 128)
        vv = slice(2 * Hk * 128 + rank * Hvr * 128, 2 * Hk * 128 + (rank + 1) * Hvr * 128)
        hv = slice(rank * Hvr, (rank + 1) * Hvr)
        cat = lambda t: torch.cat([t[kq], t[kk], t[vv]], dim=0)
        out[a + "in_proj_qkv"] = cat(g(a + "in_proj_qkv"))
        out[a + "conv1d"] = cat(g(a + "conv1d"))
        out[a + "in_proj_z"] = g(a + "in_proj_z")[rank * Hvr * 128:(rank + 1) * Hvr * 128]
        out[a + "in_proj_b"], out[a + "in_proj_a"] = g(a + "in_proj_b")[hv], g(a + "in_proj_a")[hv]
        out[a + "A_log"], out[a + "dt_bias"] = g(a + "A_log")[hv], g(a + "dt_bias")[hv]
        out[a + "norm"] = g(a + "norm")
        out[a + "out_proj"] = g(a + "out_proj")[:, rank * Hvr * 128:(rank + 1) * Hvr * 128]
    return out


class Layer:
    """One decoder layer (`Layer::forward`, src/archs/qwen35_text.rs:932-940) under tensor parallelism: every rank runs
    the mixer and the MLP on its own heads / columns (`sys1_b200.qwen35.FullAttention` / `LinearAttention` built from this
    rank's shard, `Mlp` above), and the two row-parallel projections (`o_proj` / `out_proj`, `down_proj`) are followed by
    the sum over ranks. The residual stream is replicated; rank 0 adds it in its projection epilogue, so that the sum
    over ranks is `x + sum_r partial_r`. `forward` updates `x` in place on every rank."""

    def __init__(self, shard, cfg, layer_type: str, tp: TensorParallel, rope, slabs: int = 4, comm_sms: int = 16, recurrence: str = "chunked"):
        from . import qwen35
        from .linear import Linear
        Hr, KVr, Hkr, Hvr = local_heads(cfg, tp.size)
        lin = lambda name: Linear(shard[name])
        eps = cfg.rms_norm_eps
        self.tp = tp
        self.input_norm = qwen35.RmsNorm(shard["input_layernorm"], eps)
        self.post_norm = qwen35.RmsNorm(shard["post_attention_layernorm"], eps)
        if layer_type == "full_attention":
            a = "self_attn."
            self.mixer = qwen35.FullAttention(lin(a + "q_proj"), lin(a + "k_proj"), lin(a + "v_proj"), lin(a + "o_proj"),
                                              qwen35.RmsNorm(shard[a + "q_norm"], eps), qwen35.RmsNorm(shard[a + "k_norm"], eps),
                                              Hr, KVr, cfg.head_dim, rope)
        else:
            a = "linear_attn."
            self.mixer = qwen35.LinearAttention(lin(a + "in_proj_qkv"), lin(a + "in_proj_z"), lin(a + "in_proj_b"), lin(a + "in_proj_a"),
                                                shard[a + "conv1d"].contiguous(), -torch.exp(shard[a + "A_log"].float()),
                                                shard[a + "dt_bias"].float(), shard[a + "norm"], lin(a + "out_proj"), Hkr, Hvr, eps,
                                                recurrence=recurrence)
        self.mixer_out = RowParallelLinear(self.mixer.output.weight, tp, slabs=slabs, comm_sms=comm_sms)
        self.mlp = Mlp(shard["mlp.gate_proj"], shard["mlp.up_proj"], shard["mlp.down_proj"], tp, slabs=slabs, sharded=True, comm_sms=comm_sms)

    def forward(self, x: torch.Tensor, cu_seqlens_host, positions: torch.Tensor, exchange: bool = True) -> torch.Tensor:
        y = self.mixer.mix(self.input_norm(x), cu_seqlens_host, positions)
        self.mixer_out.forward(y, residual=x, out=x, exchange=exchange)       # x <- x + sum_r y_r W_r^T
        n = self.post_norm(x)
        self.mlp.forward(n, residual=x, out=x, exchange=exchange)             # x <- x + sum_r mlp_r(n)
        return x

    # The two halves of the layer for the micro-batch schedule of `Decoder.forward_embeds`: each leaves this rank's partial
    # (rank 0: partial + residual) in `x`, starts the sum over ranks without waiting for it, and returns its ticket.
    def mixer_part(self, x: torch.Tensor, cu_seqlens_host, positions: torch.Tensor, exchange: bool = True):
        y = self.mixer.mix(self.input_norm(x), cu_seqlens_host, positions)
        fused_linear(y, self.mixer.output.weight, residual=x if self.tp.rank == 0 else None, out=x, ctx=self.tp.ctx)
        return self.tp.ctx.all_reduce_async_(x) if exchange and self.tp.size > 1 else None

    def mlp_part(self, x: torch.Tensor, exchange: bool = True):
        h = fused_linear(self.post_norm(x), self.mlp.gate, weight_up=self.mlp.up, epilogue=EPI_SWIGLU, ctx=self.tp.ctx)
        fused_linear(h, self.mlp.down, residual=x if self.tp.rank == 0 else None, out=x, ctx=self.tp.ctx)
        return self.tp.ctx.all_reduce_async_(x) if exchange and self.tp.size > 1 else None


class Decoder:
    """A stack of tensor-parallel layers over a packed batch (`Decoder::forward_embeds`, src/archs/qwen35_text.rs:986-1005,
    from the embedded tokens to the final norm). `weights`: the FULL tensors under the checkpoint's names (see
    `sys1_b200.qwen35.Decoder`); every rank cuts its own shards out of them."""

    def __init__(self, weights, cfg, tp: TensorParallel, max_positions: int = 8192, slabs: int = 4, comm_sms: int = 16,
                 recurrence: str = "chunked", comm_ctas: int = 0):
        """`comm_ctas`: blocks of the library's own exchange kernel while it runs beside the projections (0 = its default)."""
        from . import qwen35
        dev = weights["norm"].device
        rope = qwen35.RopeParams(cfg.rope_theta, cfg.rotary_dim, max_positions, dev)
        self.cfg, self.tp, self.comm_sms, self.comm_ctas = cfg, tp, int(comm_sms), int(comm_ctas)
        self.layers = []
        for i in range(cfg.num_hidden_layers):
            kind = cfg.layer_type(i)
            shard = shard_layer_weights(weights, f"layers.{i}.", cfg, kind, tp.rank, tp.size)
            self.layers.append(Layer(shard, cfg, kind, tp, rope, slabs=slabs, comm_sms=comm_sms, recurrence=recurrence))
        self.norm = qwen35.RmsNorm(weights["norm"], cfg.rms_norm_eps)

    def forward_embeds(self, x: torch.Tensor, cu_seqlens_host, positions: torch.Tensor, exchange: bool = True,
                       micro_batches: int = 1) -> torch.Tensor:
        """`x [T, hidden]` bf16: the embedded tokens, identical on every rank; it is updated in place layer by layer.

        `micro_batches` > 1: the batch is cut into that many groups of whole sequences (sequences never interact), which
        move through every layer one after the other; a group's sum over ranks is started without waiting and only the
        group itself waits for it (by ticket) before its next stage, so one group computes while the other's partial sums
        travel: mixer(0), [sum(0) | mixer(1)], [sum(1) | mlp(0)], [sum(0) | mlp(1)], [sum(1) | next mixer(0)], ...
        The projections run on `SMs - comm_sms` SMs meanwhile so that the collective always finds room."""
        from .qwen35 import batch_plan_cached
        pos = positions.to(torch.int32).contiguous()
        ctx = self.tp.ctx
        previous = getattr(ctx, "_plan", None)
        if micro_batches <= 1:
            ctx.use_plan(batch_plan_cached(self, ctx, [int(c) for c in cu_seqlens_host]))
            try:
                for layer in self.layers:
                    x = layer.forward(x, cu_seqlens_host, pos, exchange=exchange)
            finally:
                ctx.use_plan(previous)
            return self.norm(x)
        if not x.is_contiguous():
            raise ValueError("the residual stream must be contiguous")
        groups = []
        for s0, s1 in split_sequences(cu_seqlens_host, micro_batches):
            a, b = int(cu_seqlens_host[s0]), int(cu_seqlens_host[s1])
            if b > a:
                cu_g = [int(c) - a for c in cu_seqlens_host[s0:s1 + 1]]
                groups.append((x[a:b], cu_g, pos[a:b], batch_plan_cached(self, ctx, cu_g)))
        tickets = [None] * len(groups)
        beside = exchange and self.tp.size > 1   # one group's sums run beside the other group's kernels
        carve = beside and self.comm_sms > 0
        if beside:
            ctx.set_option("dynamic_tiles", 1)   # a projection CTA held up by the collective's blocks must not hold up the launch
        if carve:
            ctx.set_option("gemm_sms", max(2, device.sm_count(ctx) - self.comm_sms))
        try:
            for layer in self.layers:
                for stage in (0, 1):
                    for i, (xg, cu, pg, plan) in enumerate(groups):
                        if tickets[i] is not None:
                            ctx.all_reduce_wait_ticket(tickets[i])
                        ctx.use_plan(plan)
                        # the step's very last sum has nothing left to run beside: it may take every block it can use
                        last = beside and layer is self.layers[-1] and stage == 1 and i == len(groups) - 1
                        if last:
                            ctx.set_option("comm_ctas", 32)
                        try:
                            tickets[i] = layer.mixer_part(xg, cu, pg, exchange) if stage == 0 else layer.mlp_part(xg, exchange)
                        finally:
                            if last:
                                ctx.set_option("comm_ctas", self.comm_ctas)
            for t in tickets:
                if t is not None:
                    ctx.all_reduce_wait_ticket(t)
        finally:
            ctx.use_plan(previous)
            if beside:
                ctx.set_option("dynamic_tiles", 0)
            if carve:
                ctx.set_option("gemm_sms", 0)
        return self.norm(x)


def split_sequences(cu_seqlens_host, parts: int):
    """Cuts the sequences of a packed batch into at most `parts` consecutive groups of about the same number of tokens:
    [(first sequence, one past the last), ...]. Groups are runs of whole sequences, so each is a packed batch of its own."""
    cu = [int(c) for c in cu_seqlens_host]
    n, total = len(cu) - 1, cu[-1]
    bounds = [0]
    for k in range(1, parts):
        target = total * k / parts
        # the sequence boundary closest to the k-th share of the tokens, never before the previous cut
        best = min(range(bounds[-1], n + 1), key=lambda s: abs(cu[s] - target))
        bounds.append(max(best, bounds[-1]))
    bounds.append(n)
    return [(a, b) for a, b in zip(bounds[:-1], bounds[1:]) if b > a]
