// Bidirectional softmax attention over a token-packed batch, optional +-window band, head dim 64, on tcgen05.
//
// What the reference computes in `scaled_dot_product_attention` / `eager_attention`
// (src/archs/modernbert.rs:313-351) with its masks (`local_attention_mask`, :1058-1076: keys further than
// local_attention / 2 from the query are masked; padded keys never exist in the packed layout):
//     a_i = sum_j softmax_j( q_i . k_j / sqrt(D) ) v_j     over the keys j of the same sequence (|i - j| <= window)
// in flash form: the score matrix never leaves the chip. On a B200 the reference has no fused attention at all
// (its flash-attn path is refused for compute capability >= 10, build.rs:53-55) and materialises [L, L] scores.
//
// One CTA per (128-query block of one sequence, head); 5 warps:
//   warp 4      : TMA loads (Q once, K / V tiles of 128 keys through a 2-stage ring) and the MMAs:
//                 S = Q K^T (M = 128 queries, N = 128 keys, K = 64) and PV (M = 128, N = 64, K = 128 keys,
//                 V consumed as stored, token rows x dims = MN-major B operand), accumulators in TMEM
//   warps 0..3  : thread = query row = TMEM lane: online softmax in f32 (running max / sum per thread, no
//                 shuffles), P rounded to bf16 into a swizzled A-operand tile, O kept in 64 f32 registers
// Two CTAs fit per SM (112 KB shared memory, 256 TMEM columns each): one computes softmax while the other's MMAs run.
// Every mbarrier wait is bounded.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <cmath>

#include "context.h"
#include "ptx.cuh"

using namespace s1;

namespace {

constexpr int kHD = 64;                       // head dim
constexpr int kQB = 128;                      // queries per CTA = keys per tile
constexpr int kTile = kQB * kHD * 2;          // 16 KB: [128 tokens x 64 dims] bf16, 128-byte rows, 128B swizzle
// no alignment slack: two CTAs per SM leave 113.5 KB each; the dynamic window starts 1024-byte aligned (checked at run time)
constexpr int kAttnSmem = kTile /*Q*/ + 2 * 2 * kTile /*K, V x 2 stages*/ + 2 * kTile /*P: 2 tiles of 64 keys*/ + 128;

struct QBlock {
    int seq_start;  // first token of the sequence
    int seq_len;
    int qb;         // query block inside the sequence
    int pad;
};

struct AttnParams {
    const QBlock* blocks;
    __nv_bfloat16* out;
    long long ldo;
    int window;       // < 0: none
    float scale_log2; // scale * log2(e)
    int* status;
};

__device__ __forceinline__ uint32_t sw128(uint32_t row, uint32_t col) {
    return row * 128u + ((((col >> 3) ^ (row & 7u)) << 4) | ((col & 7u) << 1));
}
__device__ __forceinline__ uint64_t mn_desc(uint32_t smem_addr) {  // MN-major operand, one 64-element atom wide
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}
__device__ __forceinline__ uint32_t pack_bf16x2_attn(float a, float b) {
    const __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&t);
}
__device__ __forceinline__ float ex2(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

__global__ void __launch_bounds__(160, 2)
s1_attention_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t base = smem_u32(smem_raw);
    if (base & 1023u) {  // the swizzled tiles need 1024-byte alignment; never seen otherwise, reported instead of assumed
        if (threadIdx.x == 0 && atomicCAS(p.status, 0, 5) == 0) p.status[1] = blockIdx.x, p.status[2] = 39, p.status[3] = base & 1023u;
        return;
    }
    uint8_t* al = smem_raw;
    const uint32_t sq = base, skv = base + kTile, sp = base + 5 * kTile;  // stage s: K at skv + s*2*kTile, V right after
    uint64_t* bars = reinterpret_cast<uint64_t*>(al + 7 * kTile);
    // bars: 0 Q full; 1,2 KV full; 3,4 KV empty; 5 S ready; 6 P ready; 7 PV ready
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t b0 = smem_u32(bars);
    const uint32_t bar_q = b0, full0 = b0 + 8, empty0 = b0 + 24, bar_s = b0 + 40, bar_p = b0 + 48, bar_o = b0 + 56;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const QBlock qb = p.blocks[blockIdx.x];
    const int head = blockIdx.y;
    const int q_lo = qb.qb * kQB;                                  // first query (index inside the sequence)
    const int q_hi = min(q_lo + kQB, qb.seq_len) - 1;              // last valid query
    const int k_first = p.window < 0 ? 0 : max(0, q_lo - p.window);
    const int k_last = p.window < 0 ? qb.seq_len - 1 : min(qb.seq_len - 1, q_hi + p.window);
    const int kb_lo = k_first / kQB, kb_hi = k_last / kQB;         // key tiles kb_lo .. kb_hi
    const int nkb = kb_hi - kb_lo + 1;

    if (threadIdx.x == 0) {
        mbar_init(bar_q, 1);
        mbar_init(full0, 1);
        mbar_init(full0 + 8, 1);
        mbar_init(empty0, 1);
        mbar_init(empty0 + 8, 1);
        mbar_init(bar_s, 1);
        mbar_init(bar_p, 4);
        mbar_init(bar_o, 1);
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
    }
    if (warp == 4) {
        tmem_alloc(smem_u32(tmem_slot), 256);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    int fail = 0;

    if (warp == 4) {
        if (lane == 0) {
            const int x = head * kHD;
            mbar_arrive_expect_tx(bar_q, kTile);
            tma_load_2d(sq, &tmQ, x, qb.seq_start + q_lo, bar_q);
            auto load = [&](int i) {
                const int st = i & 1;
                const uint32_t fb = full0 + 8u * st, dst = skv + st * 2 * kTile;
                const int y = qb.seq_start + (kb_lo + i) * kQB;
                mbar_arrive_expect_tx(fb, 2 * kTile);
                tma_load_2d(dst, &tmK, x, y, fb);
                tma_load_2d(dst + kTile, &tmV, x, y, fb);
            };
            load(0);
            if (!mbar_wait(bar_q, 0, abort_flag)) fail = 1;
            for (int i = 0; i < nkb && !fail; ++i) {
                const int st = i & 1;
                const uint32_t kt = skv + st * 2 * kTile, vt = kt + kTile;
                if (i + 1 < nkb) {
                    if (i >= 1 && !mbar_wait(empty0 + 8u * ((i + 1) & 1), ((i - 1) >> 1) & 1, abort_flag)) { fail = 2; break; }
                    load(i + 1);
                }
                if (!mbar_wait(full0 + 8u * st, (i >> 1) & 1, abort_flag)) { fail = 3; break; }
                // S (TMEM columns 0..127) may be overwritten once the softmax warps have read block i-1: they say so
                // through bar_p of that block, which this thread has already waited on below
                tc_fence_after();
                {
                    constexpr uint32_t idesc = make_idesc(1, 128, 128);
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)
                        umma_bf16(tmem, make_sw128_kmajor_desc(sq) + 2u * kk, make_sw128_kmajor_desc(kt) + 2u * kk, idesc, kk ? 1u : 0u);
                    umma_commit(bar_s);
                }
                if (!mbar_wait(bar_p, i & 1, abort_flag)) { fail = 4; break; }
                tc_fence_after();
                {
                    constexpr uint32_t idesc = make_idesc(1, 128, 64) | (1u << 16);  // B (= V) is MN-major
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk)  // 16 keys per instruction
                        umma_bf16(tmem + 128, make_sw128_kmajor_desc(sp + (kk >> 2) * kTile) + 2u * (kk & 3), mn_desc(vt) + 128u * kk,
                                  idesc, kk ? 1u : 0u);
                    umma_commit(bar_o);
                    umma_commit(empty0 + 8u * st);
                }
            }
        }
        __syncwarp();
    } else {
        const int row = threadIdx.x;                       // query row of the block = TMEM lane
        const int qi = q_lo + row;                         // index inside the sequence
        const bool q_ok = qi < qb.seq_len;
        const uint32_t lane_addr = tmem + (static_cast<uint32_t>(warp * 32) << 16);
        float O[kHD];
#pragma unroll
        for (int d = 0; d < kHD; ++d) O[d] = 0.f;
        float m = -INFINITY, l = 0.f;
        const int lo = p.window < 0 ? 0 : qi - p.window, hi = p.window < 0 ? qb.seq_len - 1 : min(qb.seq_len - 1, qi + p.window);

        for (int i = 0; i < nkb; ++i) {
            const int j0 = (kb_lo + i) * kQB;              // first key of the tile (index inside the sequence)
            bool ok = mbar_wait(bar_s, i & 1, abort_flag);
            if (!__all_sync(0xffffffffu, ok)) { fail = 5; break; }
            tc_fence_after();
            // pass 1: row maximum over the keys this query may see
            float mx = -INFINITY;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t s[32];
                tmem_ld_32x32b_x32(lane_addr + c * 32, s);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    const int j = j0 + c * 32 + e;
                    if (j >= lo && j <= hi) mx = fmaxf(mx, __uint_as_float(s[e]));
                }
            }
            const float m_new = fmaxf(m, mx);
            const float alpha = (m_new == -INFINITY) ? 1.f : ex2((m - m_new) * p.scale_log2);  // m = -inf: ex2(-inf) = 0
            const float mref = (m_new == -INFINITY) ? 0.f : m_new;
            // pass 2: p = exp(scale (s - m)), row sum, bf16 P into the A-operand tiles
            float sum = 0.f;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t s[32];
                tmem_ld_32x32b_x32(lane_addr + c * 32, s);
                tmem_ld_wait();
                uint32_t pk[16];
#pragma unroll
                for (int e = 0; e < 32; e += 2) {
                    const int j = j0 + c * 32 + e;
                    const float p0 = (j >= lo && j <= hi) ? ex2((__uint_as_float(s[e]) - mref) * p.scale_log2) : 0.f;
                    const float p1 = (j + 1 >= lo && j + 1 <= hi) ? ex2((__uint_as_float(s[e + 1]) - mref) * p.scale_log2) : 0.f;
                    const __nv_bfloat162 t = __floats2bfloat162_rn(p0, p1);
                    sum += __low2float(t) + __high2float(t);  // the sum of what is actually multiplied with V
                    pk[e >> 1] = *reinterpret_cast<const uint32_t*>(&t);
                }
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int col = (c & 1) * 32 + 8 * e;  // column inside the 64-key tile c / 2
                    const uint32_t addr = sp + (c >> 1) * kTile + sw128(row, col);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pk[4 * e]), "r"(pk[4 * e + 1]),
                                 "r"(pk[4 * e + 2]), "r"(pk[4 * e + 3]) : "memory");
                }
            }
            l = l * alpha + sum;
            m = m_new;
            fence_proxy_async_smem();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_p);

            ok = mbar_wait(bar_o, i & 1, abort_flag);
            if (!__all_sync(0xffffffffu, ok)) { fail = 6; break; }
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t pv[32];
                tmem_ld_32x32b_x32(lane_addr + 128 + c * 32, pv);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 32; ++e) O[c * 32 + e] = fmaf(O[c * 32 + e], alpha, __uint_as_float(pv[e]));
            }
            tc_fence_before();
        }
        if (!fail && q_ok) {
            const float inv = 1.f / l;
            __nv_bfloat16* orow = p.out + static_cast<long long>(qb.seq_start + qi) * p.ldo + head * kHD;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                uint4 v;
                v.x = pack_bf16x2_attn(O[8 * e] * inv, O[8 * e + 1] * inv);
                v.y = pack_bf16x2_attn(O[8 * e + 2] * inv, O[8 * e + 3] * inv);
                v.z = pack_bf16x2_attn(O[8 * e + 4] * inv, O[8 * e + 5] * inv);
                v.w = pack_bf16x2_attn(O[8 * e + 6] * inv, O[8 * e + 7] * inv);
                *reinterpret_cast<uint4*>(orow + 8 * e) = v;
            }
        }
        __syncwarp();
    }
    if (fail && atomicCAS(p.status, 0, 4) == 0) {
        p.status[1] = blockIdx.x;
        p.status[2] = 30 + fail;
        p.status[3] = blockIdx.y;
    }
    if (*abort_flag) __nanosleep(200000);
    tc_fence_before();
    __syncthreads();
    if (warp == 4) {
        tc_fence_after();
        tmem_dealloc(tmem, 256);
    }
}

}  // namespace

extern "C" size_t s1_attention_workspace(int num_seqs, int total_tokens) {
    if (num_seqs < 0 || total_tokens < 0) return 0;
    return sizeof(QBlock) * static_cast<size_t>(total_tokens / kQB + num_seqs + 1);
}

extern "C" int s1_attention(s1_ctx* ctx, const void* q, long long ldq, const void* k, long long ldk, const void* v, long long ldv,
                            const int32_t* cu_seqlens_host, int num_seqs, int total_tokens, int heads, int head_dim, int window,
                            float scale, void* out, long long ldo, void* workspace, size_t workspace_bytes) {
    if (!ctx) return S1_EINVAL;
    if (!q || !k || !v || !cu_seqlens_host || !out || !workspace) return s1_fail(ctx, S1_EINVAL, "s1_attention: null pointer");
    if (head_dim != kHD) return s1_fail(ctx, S1_EINVAL, "s1_attention: head_dim must be 64 (got %d)", head_dim);
    if (heads < 1 || num_seqs < 0 || total_tokens < 0) return s1_fail(ctx, S1_EINVAL, "s1_attention: bad sizes");
    const long long width = 1LL * heads * kHD;
    if (ldq < width || ldk < width || ldv < width || ldo < width || (ldq % 8) || (ldk % 8) || (ldv % 8) || (ldo % 8))
        return s1_fail(ctx, S1_EINVAL, "s1_attention: rows need %lld columns and 16-byte alignment", width);
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(out) |
         reinterpret_cast<uintptr_t>(workspace)) & 15u)
        return s1_fail(ctx, S1_EINVAL, "s1_attention: pointers must be 16-byte aligned");
    if (workspace_bytes < s1_attention_workspace(num_seqs, total_tokens))
        return s1_fail(ctx, S1_EINVAL, "s1_attention: workspace of %zu bytes, %zu needed", workspace_bytes,
                       s1_attention_workspace(num_seqs, total_tokens));
    if (num_seqs == 0 || total_tokens == 0) return S1_OK;
    if (cu_seqlens_host[0] != 0 || cu_seqlens_host[num_seqs] != total_tokens)
        return s1_fail(ctx, S1_EINVAL, "s1_attention: cu_seqlens must run from 0 to total_tokens");
    S1_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    const size_t max_blocks = static_cast<size_t>(total_tokens / kQB + num_seqs + 1);
    ctx->host_scratch.resize(sizeof(QBlock) * max_blocks);
    QBlock* blocks = reinterpret_cast<QBlock*>(ctx->host_scratch.data());
    int nb = 0;
    for (int s = 0; s < num_seqs; ++s) {
        const int a = cu_seqlens_host[s], len = cu_seqlens_host[s + 1] - a;
        if (len < 0) return s1_fail(ctx, S1_EINVAL, "s1_attention: cu_seqlens must not decrease");
        for (int b = 0; b * kQB < len; ++b) blocks[nb++] = QBlock{a, len, b, 0};
    }
    if (nb == 0) return S1_OK;
    // without a window the work of a block grows with its sequence: longest sequences first
    if (window < 0) std::stable_sort(blocks, blocks + nb, [](const QBlock& x, const QBlock& y) { return x.seq_len > y.seq_len; });
    S1_CUDA_OK(ctx, cudaMemcpyAsync(workspace, blocks, sizeof(QBlock) * nb, cudaMemcpyHostToDevice, ctx->stream));

    CUtensorMap tq, tk, tv;
    int rc = s1_get_tmap(ctx, q, total_tokens, width, ldq, kQB, kHD, 2, 128, &tq);
    if (rc) return rc;
    rc = s1_get_tmap(ctx, k, total_tokens, width, ldk, kQB, kHD, 2, 128, &tk);
    if (rc) return rc;
    rc = s1_get_tmap(ctx, v, total_tokens, width, ldv, kQB, kHD, 2, 128, &tv);
    if (rc) return rc;
    AttnParams ap;
    ap.blocks = static_cast<const QBlock*>(workspace);
    ap.out = static_cast<__nv_bfloat16*>(out);
    ap.ldo = ldo;
    ap.window = window;
    ap.scale_log2 = scale * 1.4426950408889634f;
    ap.status = ctx->status_dev;
    static thread_local int configured_device = -1;
    if (configured_device != ctx->device) {
        S1_CUDA_OK(ctx, cudaFuncSetAttribute(s1_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmem));
        configured_device = ctx->device;
    }
    s1_attention_kernel<<<dim3(nb, heads), 160, kAttnSmem, ctx->stream>>>(tq, tk, tv, ap);
    S1_CUDA_OK(ctx, cudaGetLastError());
    ctx->launches += 1;
    return S1_OK;
}
