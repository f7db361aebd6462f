// s1_batch_plan: the per-batch tables of the attention and delta-rule kernels, built once.
//
// Every layer of a stack walks the same packed batch: the 128-query blocks of its sequences (in the order each
// attention kernel wants to start them) and the 64-token chunks of the delta rule. Without a plan each kernel call
// rebuilds its table on the host and copies it to the device - one small host-to-device copy per layer, which also
// keeps the call from being captured in a CUDA graph. With a plan the tables are built and copied once per batch
// (the reference builds its `cu_seqlens` once per batch as well, src/archs/modernbert.rs:431-443), and the kernel calls
// pass `cu_seqlens_host = NULL`.
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>

#include "context.h"

namespace {

constexpr size_t kMaxLivePlans = 4096;  // records of a few dozen bytes; a caller that never releases is told so
inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct Layout {
    size_t attn_global_off, attn_local_off, gqa_off, slots_off, seqs_off, total;
};
Layout layout(int num_seqs, int total_tokens) {
    const size_t max_blocks = static_cast<size_t>(total_tokens / 128 + num_seqs + 1);
    const size_t max_slots = static_cast<size_t>(total_tokens / 64 + num_seqs + 1);
    Layout L;
    size_t o = 0;
    L.attn_global_off = o, o = align_up(o + sizeof(S1QBlock) * max_blocks, 256);
    L.attn_local_off = o, o = align_up(o + sizeof(S1QBlock) * max_blocks, 256);
    L.gqa_off = o, o = align_up(o + sizeof(S1QBlock) * max_blocks, 256);
    L.slots_off = o, o = align_up(o + sizeof(S1ChunkSlot) * max_slots, 256);
    L.seqs_off = o, o = align_up(o + sizeof(S1SeqChunks) * static_cast<size_t>(num_seqs > 0 ? num_seqs : 1), 256);
    L.total = o;
    return L;
}
}  // namespace

extern "C" size_t s1_batch_plan_bytes(int num_seqs, int total_tokens) {
    if (num_seqs < 0 || total_tokens < 0) return 0;
    return layout(num_seqs, total_tokens).total;
}

extern "C" int s1_batch_plan(s1_ctx* ctx, const int32_t* cu_seqlens_host, int num_seqs, int total_tokens, void* plan,
                             size_t plan_bytes) {
    if (!ctx) return S1_EINVAL;
    if (!cu_seqlens_host || !plan) return s1_fail(ctx, S1_EINVAL, "s1_batch_plan: null pointer");
    if (num_seqs < 0 || total_tokens < 0) return s1_fail(ctx, S1_EINVAL, "s1_batch_plan: bad sizes");
    const Layout L = layout(num_seqs, total_tokens);
    if (plan_bytes < L.total) return s1_fail(ctx, S1_EINVAL, "s1_batch_plan: buffer of %zu bytes, %zu needed", plan_bytes, L.total);
    if (reinterpret_cast<uintptr_t>(plan) & 255u) return s1_fail(ctx, S1_EINVAL, "s1_batch_plan: the buffer must be 256-byte aligned");
    if (cu_seqlens_host[0] != 0 || cu_seqlens_host[num_seqs] != total_tokens)
        return s1_fail(ctx, S1_EINVAL, "s1_batch_plan: cu_seqlens must run from 0 to total_tokens");
    for (int s = 0; s < num_seqs; ++s)
        if (cu_seqlens_host[s + 1] < cu_seqlens_host[s]) return s1_fail(ctx, S1_EINVAL, "s1_batch_plan: cu_seqlens must not decrease");
    S1_CUDA_OK(ctx, cudaSetDevice(ctx->device));

    ctx->host_scratch.assign(L.total, 0);
    unsigned char* h = ctx->host_scratch.data();
    S1QBlock* ag = reinterpret_cast<S1QBlock*>(h + L.attn_global_off);
    S1QBlock* al = reinterpret_cast<S1QBlock*>(h + L.attn_local_off);
    S1QBlock* gq = reinterpret_cast<S1QBlock*>(h + L.gqa_off);
    S1ChunkSlot* slots = reinterpret_cast<S1ChunkSlot*>(h + L.slots_off);
    S1SeqChunks* seqs = reinterpret_cast<S1SeqChunks*>(h + L.seqs_off);
    int nb = 0, ns = 0;
    for (int s = 0; s < num_seqs; ++s) {
        const int a = cu_seqlens_host[s], b = cu_seqlens_host[s + 1], len = b - a;
        for (int q = 0; q * 128 < len; ++q) al[nb++] = S1QBlock{a, len, q, 0};
        seqs[s].first_slot = ns;
        seqs[s].num_chunks = (len + 63) / 64;
        for (int t = a; t < b; t += 64) slots[ns++] = S1ChunkSlot{t, (b - t < 64) ? b - t : 64};
    }
    std::copy(al, al + nb, ag);
    std::copy(al, al + nb, gq);
    // starting orders: bidirectional attention without a window - longest sequences first (a block's work grows with its
    // sequence); causal attention - latest blocks first (work grows with the position); delta-rule scan - longest first
    std::stable_sort(ag, ag + nb, [](const S1QBlock& x, const S1QBlock& y) { return x.seq_len > y.seq_len; });
    std::stable_sort(gq, gq + nb, [](const S1QBlock& x, const S1QBlock& y) { return x.qb > y.qb; });
    std::stable_sort(seqs, seqs + num_seqs, [](const S1SeqChunks& x, const S1SeqChunks& y) { return x.num_chunks > y.num_chunks; });
    // (a copy from pageable memory is staged before the call returns, so the host buffer can be reused at once)
    S1_CUDA_OK(ctx, cudaMemcpyAsync(plan, h, L.total, cudaMemcpyHostToDevice, ctx->stream));

    S1BatchPlan rec;
    rec.dev = static_cast<const unsigned char*>(plan);
    rec.num_seqs = num_seqs, rec.total_tokens = total_tokens, rec.num_blocks = nb, rec.num_slots = ns;
    rec.attn_global_off = L.attn_global_off, rec.attn_local_off = L.attn_local_off, rec.gqa_off = L.gqa_off;
    rec.slots_off = L.slots_off, rec.seqs_off = L.seqs_off;
    const S1BatchPlan* used = (ctx->plan_in_use >= 0) ? &ctx->plans[ctx->plan_in_use] : nullptr;
    const unsigned char* used_dev = used ? used->dev : nullptr;
    bool replaced = false;
    for (auto& p : ctx->plans)
        if (p.dev == rec.dev) p = rec, replaced = true;
    if (!replaced) {
        if (ctx->plans.size() >= kMaxLivePlans)
            return s1_fail(ctx, S1_EINVAL, "s1_batch_plan: %zu plans are alive on this context; release the ones no longer needed (s1_batch_plan_release)",
                           ctx->plans.size());
        ctx->plans.push_back(rec);
    }
    ctx->plan_in_use = -1;
    for (size_t i = 0; i < ctx->plans.size(); ++i)
        if (used_dev && ctx->plans[i].dev == used_dev) ctx->plan_in_use = static_cast<int>(i);
    return S1_OK;
}

extern "C" int s1_batch_plan_release(s1_ctx* ctx, const void* plan) {
    if (!ctx) return S1_EINVAL;
    const unsigned char* used_dev = (ctx->plan_in_use >= 0) ? ctx->plans[ctx->plan_in_use].dev : nullptr;
    for (size_t i = 0; i < ctx->plans.size(); ++i)
        if (ctx->plans[i].dev == plan) {
            ctx->plans.erase(ctx->plans.begin() + i);
            ctx->plan_in_use = -1;
            if (used_dev && used_dev != plan)
                for (size_t k = 0; k < ctx->plans.size(); ++k)
                    if (ctx->plans[k].dev == used_dev) ctx->plan_in_use = static_cast<int>(k);
            return S1_OK;
        }
    return S1_OK;  // not (or no longer) known: nothing to forget
}

extern "C" int s1_use_batch_plan(s1_ctx* ctx, const void* plan) {
    if (!ctx) return S1_EINVAL;
    if (!plan) {
        ctx->plan_in_use = -1;
        return S1_OK;
    }
    for (size_t i = 0; i < ctx->plans.size(); ++i)
        if (ctx->plans[i].dev == plan) {
            ctx->plan_in_use = static_cast<int>(i);
            return S1_OK;
        }
    return s1_fail(ctx, S1_EINVAL, "s1_use_batch_plan: no plan was built in this buffer on this context (s1_batch_plan)");
}
