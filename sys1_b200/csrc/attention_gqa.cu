// Causal grouped-query softmax attention over a token-packed batch, head dim 256, on tcgen05: the attention core of
// the Qwen3.5 full-attention layer (`FullAttention::forward`, src/archs/qwen35_text.rs:312-411):
//     a_i = sum_{j <= i} softmax_j( q_i . k_j / sqrt(D) ) v_j     over the keys j of the same sequence,
// KV head h / (H / KV) serving query head h (`repeat_kv`, :363-369), and, fused into the write-out, the layer's
// output gate: out = bf16(a) * bf16(sigmoid(gate)) (:325-329, :408). The reference's eager path materialises
// [128, L] score chunks with a -inf mask per chunk (:371-393); here scores never leave the chip.
//
// One CTA per (128-query block of one sequence, query head), 9 warps, one CTA per SM (208 KB shared memory):
//   warp 8      : TMA loads (Q once: 4 column chunks of 64 dims; K and V tiles of 64 keys x 256 dims, each through
//                 its own 2-stage ring) and the MMAs: S = Q K^T (M = 128, N = 64 keys, K = 256: 16 instructions)
//                 and O += P V (M = 128, N = 4 x 64 dims, K = 64 keys: 16 instructions, V consumed as stored =
//                 MN-major B operand); S (64 columns) and O (256 columns) live in TMEM
//   warps 0..7  : two threads per query row (warps w and w + 4 read the same 32 TMEM lanes; one takes keys 0..31 of
//                 a step, the other 32..63, and at the end dims 0..127 / 128..255 of the output): scores into
//                 registers in one go (which frees S for the next tile), causal mask on the diagonal tiles only, the
//                 pair agrees on the row maximum through two spare TMEM columns, ex2 with the scale folded in, f32
//                 row sum, P rounded to bf16 into a swizzled A-operand tile; O is rescaled in TMEM only when a row
//                 maximum has grown by more than 2^8 since the last rescale.
// Key tiles past the diagonal of the query block are never loaded. Every mbarrier wait is bounded.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <cmath>

#include "context.h"
#include "ptx.cuh"

using namespace s1;

namespace {

constexpr int kD = 256;                 // head dim
constexpr int kQB = 128;                // queries per CTA
constexpr int kKB = 64;                 // keys per tile
constexpr int kQChunk = kQB * 64 * 2;   // 16 KB: [128 queries x 64 dims] bf16, 128-byte rows, 128B swizzle
constexpr int kKChunk = kKB * 64 * 2;   // 8 KB:  [64 keys x 64 dims]
constexpr int kQBytes = 4 * kQChunk, kKVBytes = 4 * kKChunk, kPBytes = kQB * kKB * 2;
constexpr int kGqaSmem = kQBytes + 2 * kKVBytes + 2 * kKVBytes + kPBytes + 128;

struct QBlock {
    int seq_start;
    int seq_len;
    int qb;
    int pad;
};

struct GqaParams {
    const QBlock* blocks;
    __nv_bfloat16* out;
    long long ldo;
    const __nv_bfloat16* gate;  // may be null
    long long ldg, gate_head_stride;
    long long q_head_stride, k_head_stride, v_head_stride;
    int heads_per_kv;
    float scale_log2;
    int* status;
};

__device__ __forceinline__ uint64_t mn_desc64(uint32_t smem_addr) {  // MN-major operand, one 64-element atom wide
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
    const __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&t);
}
__device__ __forceinline__ float ex2f(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

constexpr float kRescaleLog2 = 8.f;

// Barrier of the two warps that share a quarter of the query rows (ids 1..4; 0 is __syncthreads).
// The pair's barrier carrying one bit: true if any of its 64 threads says so.
__device__ __forceinline__ bool pair_any_gqa(int q4, bool mine) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 q, %1, 0;\n\t"
        "barrier.cta.red.or.pred p, %2, 64, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(r)
        : "r"(static_cast<uint32_t>(mine)), "r"(q4 + 1)
        : "memory");
    return r != 0;
}
__device__ __forceinline__ void pair_barrier_gqa(int q4) {
    if (q4 == 0) named_barrier<1, 64>();
    else if (q4 == 1) named_barrier<2, 64>();
    else if (q4 == 2) named_barrier<3, 64>();
    else named_barrier<4, 64>();
}

__global__ void __launch_bounds__(288, 1)
s1_attention_gqa_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                        const __grid_constant__ CUtensorMap tmV, const GqaParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t base = smem_u32(smem_raw);
    if (base & 1023u) {
        if (threadIdx.x == 0 && atomicCAS(p.status, 0, 5) == 0) p.status[1] = blockIdx.x, p.status[2] = 59, p.status[3] = base & 1023u;
        return;
    }
    const uint32_t sq = base, sk = base + kQBytes, sv = sk + 2 * kKVBytes, sp = sv + 2 * kKVBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + kQBytes + 4 * kKVBytes + kPBytes);
    // bars: 0 Q full; 1,2 K full; 3,4 V full; 5 S ready; 6 S read (8 warps); 7 P ready (8 warps); 8 PV done
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t b0 = smem_u32(bars);
    const uint32_t bar_q = b0, full_k = b0 + 8, full_v = b0 + 24, bar_s = b0 + 40, bar_sfree = b0 + 48, bar_p = b0 + 56, bar_o = b0 + 64;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const QBlock qb = p.blocks[blockIdx.x];
    const int head = blockIdx.y, kv_head = head / p.heads_per_kv;
    const int q_lo = qb.qb * kQB;
    const int q_hi = min(q_lo + kQB, qb.seq_len) - 1;
    const int nkb = q_hi / kKB + 1;  // keys 0 .. q_hi

    if (threadIdx.x == 0) {
        mbar_init(bar_q, 1);
        mbar_init(full_k, 1);
        mbar_init(full_k + 8, 1);
        mbar_init(full_v, 1);
        mbar_init(full_v + 8, 1);
        mbar_init(bar_s, 1);
        mbar_init(bar_sfree, 8);
        mbar_init(bar_p, 8);
        mbar_init(bar_o, 1);
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
    }
    if (warp == 8) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;  // columns 0..63: S, 64..319: O, 320..325: the row pairs' exchange
    int fail = 0;

    if (warp == 8) {
        if (lane == 0) {
            const int xq = static_cast<int>(head * p.q_head_stride);
            const int xk = static_cast<int>(kv_head * p.k_head_stride), xv = static_cast<int>(kv_head * p.v_head_stride);
            auto load_k = [&](int i) {
                const uint32_t fb = full_k + 8u * (i & 1);
                mbar_arrive_expect_tx(fb, kKVBytes);
#pragma unroll
                for (int c = 0; c < 4; ++c) tma_load_2d(sk + (i & 1) * kKVBytes + c * kKChunk, &tmK, xk + c * 64, qb.seq_start + i * kKB, fb);
            };
            auto load_v = [&](int i) {
                const uint32_t fb = full_v + 8u * (i & 1);
                mbar_arrive_expect_tx(fb, kKVBytes);
#pragma unroll
                for (int c = 0; c < 4; ++c) tma_load_2d(sv + (i & 1) * kKVBytes + c * kKChunk, &tmV, xv + c * 64, qb.seq_start + i * kKB, fb);
            };
            auto mma_s = [&](int i) {
                constexpr uint32_t idesc = make_idesc(1, 128, 64);
                const uint32_t kt = sk + (i & 1) * kKVBytes;
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)
                        umma_bf16(tmem, make_sw128_kmajor_desc(sq + c * kQChunk) + 2u * kk, make_sw128_kmajor_desc(kt + c * kKChunk) + 2u * kk,
                                  idesc, (c || kk) ? 1u : 0u);
                umma_commit(bar_s);
            };
            mbar_arrive_expect_tx(bar_q, kQBytes);
#pragma unroll
            for (int c = 0; c < 4; ++c) tma_load_2d(sq + c * kQChunk, &tmQ, xq + c * 64, qb.seq_start + q_lo, bar_q);
            load_k(0);
            load_v(0);
            if (nkb > 1) {
                load_k(1);
                load_v(1);
            }
            if (!mbar_wait(bar_q, 0, abort_flag)) fail = 1;
            if (!fail && !mbar_wait(full_k, 0, abort_flag)) fail = 2;
            if (!fail) {
                tc_fence_after();
                mma_s(0);
            }
            for (int i = 0; i < nkb && !fail; ++i) {
                if (i + 1 < nkb) {
                    if (!mbar_wait(full_k + 8u * ((i + 1) & 1), ((i + 1) >> 1) & 1, abort_flag)) { fail = 3; break; }
                    if (!mbar_wait(bar_sfree, i & 1, abort_flag)) { fail = 4; break; }
                    tc_fence_after();
                    mma_s(i + 1);
                    if (i + 2 < nkb) load_k(i + 2);
                }
                if (!mbar_wait(bar_p, i & 1, abort_flag)) { fail = 5; break; }
                if (i >= 1 && i + 1 < nkb) {
                    if (!mbar_wait(bar_o, (i - 1) & 1, abort_flag)) { fail = 6; break; }
                    load_v(i + 1);
                }
                if (!mbar_wait(full_v + 8u * (i & 1), (i >> 1) & 1, abort_flag)) { fail = 7; break; }
                tc_fence_after();
                {
                    constexpr uint32_t idesc = make_idesc(1, 128, 64) | (1u << 16);  // B (= V) is MN-major
                    const uint32_t vt = sv + (i & 1) * kKVBytes;
#pragma unroll
                    for (int nc = 0; nc < 4; ++nc)  // 64 output dims per accumulator block
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk)  // 16 keys per instruction
                            umma_bf16(tmem + 64 + nc * 64, make_sw128_kmajor_desc(sp) + 2u * kk, mn_desc64(vt + nc * kKChunk) + 128u * kk, idesc,
                                      (kk || i) ? 1u : 0u);
                    umma_commit(bar_o);
                }
            }
        }
        __syncwarp();
    } else {
        const int q4 = warp & 3, ch = warp >> 2;           // TMEM lane quarter; which 32 keys of a step / 128 output dims
        const int row = q4 * 32 + lane;
        const bool q_ok = q_lo + row < qb.seq_len;
        const int qi = min(q_lo + row, qb.seq_len - 1);
        const uint32_t lane_addr = tmem + (static_cast<uint32_t>(q4 * 32) << 16);
        const float c = p.scale_log2;
        const uint32_t prow = sp + static_cast<uint32_t>(row) * 128u, r7 = static_cast<uint32_t>(row) & 7u;
        float m_used = -INFINITY, l = 0.f;

        for (int i = 0; i < nkb; ++i) {
            const int j0 = i * kKB + ch * 32;              // first key of this thread's half of the step
            bool ok = mbar_wait(bar_s, i & 1, abort_flag);
            if (!__all_sync(0xffffffffu, ok)) { fail = 8; break; }
            tc_fence_after();
            uint32_t s[32];
            tmem_ld_32x32b_x32(lane_addr + ch * 32, s);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_sfree);
            if (i * kKB + kKB - 1 > q_lo) {  // a tile that touches the diagonal of this query block
                const int rel = qi - j0;     // keys 0 .. rel of this half are visible
#pragma unroll
                for (int e = 0; e < 32; ++e)
                    if (e > rel) s[e] = 0xff800000u;  // -inf
            }
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int e = 0; e < 32; e += 4) {
                mx0 = max3(mx0, __uint_as_float(s[e]), __uint_as_float(s[e + 1]));
                mx1 = max3(mx1, __uint_as_float(s[e + 2]), __uint_as_float(s[e + 3]));
            }
            const float mx_own = fmaxf(mx0, mx1);
            // One bit through the pair's barrier: does any row of this quarter need a new reference maximum (its own half's
            // maximum more than 2^8 above the one in use, or none in use yet)? Only then is the other half's maximum fetched
            // (two spare TMEM columns, double-buffered by step parity). NaN (both -inf) compares false; -inf -> finite gives
            // +inf, which rescales by ex2(-inf) = 0.
            const bool rescale = pair_any_gqa(q4, i == 0 || (mx_own - m_used) * c > kRescaleLog2);
            float alpha = 1.f;
            if (rescale) {
                const uint32_t xcol = lane_addr + 320 + 2 * (i & 1);
                tmem_st_32x32b_x1(xcol + ch, __float_as_uint(mx_own));
                tmem_st_wait();
                tc_fence_before();
                pair_barrier_gqa(q4);
                tc_fence_after();
                const float mx_other = __uint_as_float(tmem_ld_32x32b_x1(xcol + (ch ^ 1)));
                tmem_ld_wait();
                const float m_new = fmaxf(m_used, fmaxf(mx_own, mx_other));
                if (i == 0) {
                    m_used = m_new;
                } else if (m_new != -INFINITY) {
                    alpha = ex2f((m_used - m_new) * c);
                    m_used = m_new;
                }
            }
            const float neg_mc = (m_used == -INFINITY) ? 0.f : -m_used * c;
            uint32_t pk[16];
            float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
                const float p0 = ex2f(fmaf(__uint_as_float(s[e]), c, neg_mc));
                const float p1 = ex2f(fmaf(__uint_as_float(s[e + 1]), c, neg_mc));
                sum0 += p0;
                sum1 += p1;
                pk[e >> 1] = pack2(p0, p1);
            }
            l = fmaf(l, alpha, sum0 + sum1);
            if (i >= 1) {
                ok = mbar_wait(bar_o, (i - 1) & 1, abort_flag);
                if (!__all_sync(0xffffffffu, ok)) { fail = 9; break; }
                tc_fence_after();
                if (rescale) {  // this thread's 128 of the row's 256 output dims
#pragma unroll 1
                    for (int k4 = 0; k4 < 4; ++k4) {
                        uint32_t o[32];
                        tmem_ld_32x32b_x32(lane_addr + 64 + ch * 128 + k4 * 32, o);
                        tmem_ld_wait();
#pragma unroll
                        for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
                        tmem_st_32x32b_x32(lane_addr + 64 + ch * 128 + k4 * 32, o);
                    }
                    tmem_st_wait();
                }
            }
#pragma unroll
            for (int t = 0; t < 4; ++t) {  // 8 keys (16 bytes) per store: chunks ch * 4 .. ch * 4 + 3 of the row
                const uint32_t addr = prow + ((static_cast<uint32_t>(ch * 4 + t) ^ r7) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pk[4 * t]), "r"(pk[4 * t + 1]),
                             "r"(pk[4 * t + 2]), "r"(pk[4 * t + 3]) : "memory");
            }
            fence_proxy_async_smem();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_p);
        }
        if (!fail) {
            const bool ok = mbar_wait(bar_o, (nkb - 1) & 1, abort_flag);
            if (!__all_sync(0xffffffffu, ok)) fail = 10;
        }
        if (!fail) {
            tc_fence_after();
            tmem_st_32x32b_x1(lane_addr + 324 + ch, __float_as_uint(l));  // the row sum is the two halves' sums, in a fixed order
            tmem_st_wait();
            tc_fence_before();
            pair_barrier_gqa(q4);
            tc_fence_after();
            const float l0 = ch == 0 ? l : __uint_as_float(tmem_ld_32x32b_x1(lane_addr + 324));
            const float l1 = ch == 1 ? l : __uint_as_float(tmem_ld_32x32b_x1(lane_addr + 325));
            tmem_ld_wait();
            const float inv = 1.f / (l0 + l1);
            const long long tok = static_cast<long long>(qb.seq_start + qi);
            __nv_bfloat16* orow = p.out + tok * p.ldo + head * kD + ch * 128;
            const __nv_bfloat16* grow = p.gate ? p.gate + tok * p.ldg + head * p.gate_head_stride + ch * 128 : nullptr;
#pragma unroll 1
            for (int k4 = 0; k4 < 4; ++k4) {
                uint32_t o[32];
                tmem_ld_32x32b_x32(lane_addr + 64 + ch * 128 + k4 * 32, o);
                tmem_ld_wait();
                if (q_ok) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        float f[8];
#pragma unroll
                        for (int u = 0; u < 8; ++u) f[u] = __uint_as_float(o[8 * e + u]) * inv;
                        if (grow) {  // bf16(a) * bf16(sigmoid(gate)), rounded again: the reference's tensor ops, one by one
                            const uint4 graw = *reinterpret_cast<const uint4*>(grow + k4 * 32 + 8 * e);
                            const __nv_bfloat16* gv = reinterpret_cast<const __nv_bfloat16*>(&graw);
#pragma unroll
                            for (int u = 0; u < 8; ++u) {
                                const float g = __bfloat162float(gv[u]);
                                f[u] = bf16_round(f[u]) * bf16_round(1.f / (1.f + __expf(-g)));
                            }
                        }
                        uint4 v;
                        v.x = pack2(f[0], f[1]);
                        v.y = pack2(f[2], f[3]);
                        v.z = pack2(f[4], f[5]);
                        v.w = pack2(f[6], f[7]);
                        *reinterpret_cast<uint4*>(orow + k4 * 32 + 8 * e) = v;
                    }
                }
            }
            tc_fence_before();
        }
        __syncwarp();
    }
    if (fail && atomicCAS(p.status, 0, 4) == 0) {
        p.status[1] = blockIdx.x;
        p.status[2] = 50 + fail;
        p.status[3] = blockIdx.y;
    }
    if (*abort_flag) __nanosleep(200000);
    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

}  // namespace

extern "C" size_t s1_attention_gqa_workspace(int num_seqs, int total_tokens) {
    if (num_seqs < 0 || total_tokens < 0) return 0;
    return sizeof(QBlock) * static_cast<size_t>(total_tokens / kQB + num_seqs + 1);
}

extern "C" int s1_attention_gqa(s1_ctx* ctx, const void* q, long long ldq, long long q_head_stride, const void* k, long long ldk,
                                long long k_head_stride, const void* v, long long ldv, long long v_head_stride, const void* gate,
                                long long ldg, long long gate_head_stride, const int32_t* cu_seqlens_host, int num_seqs,
                                int total_tokens, int heads, int kv_heads, int head_dim, float scale, void* out, long long ldo,
                                void* workspace, size_t workspace_bytes) {
    if (!ctx) return S1_EINVAL;
    if (!q || !k || !v || !out) return s1_fail(ctx, S1_EINVAL, "s1_attention_gqa: null pointer");
    static_assert(sizeof(QBlock) == sizeof(S1QBlock), "the plan's query-block table has this kernel's layout");
    const S1BatchPlan* plan = cu_seqlens_host ? nullptr : ctx->active_plan(num_seqs, total_tokens);
    if (!cu_seqlens_host && !plan)
        return s1_fail(ctx, S1_EINVAL, "s1_attention_gqa: cu_seqlens_host is NULL and no batch plan for this batch is in use");
    if (!plan && !workspace) return s1_fail(ctx, S1_EINVAL, "s1_attention_gqa: null workspace");
    if (head_dim != kD) return s1_fail(ctx, S1_EINVAL, "s1_attention_gqa: head_dim must be 256 (got %d)", head_dim);
    if (heads < 1 || kv_heads < 1 || (heads % kv_heads) || num_seqs < 0 || total_tokens < 0)
        return s1_fail(ctx, S1_EINVAL, "s1_attention_gqa: heads must be a multiple of kv_heads");
    const long long qw = (heads - 1) * q_head_stride + kD, kw = (kv_heads - 1) * k_head_stride + kD, vw = (kv_heads - 1) * v_head_stride + kD;
    if (q_head_stride < kD || k_head_stride < kD || v_head_stride < kD || ldq < qw || ldk < kw || ldv < vw || ldo < 1LL * heads * kD ||
        ((ldq | ldk | ldv | ldo | q_head_stride | k_head_stride | v_head_stride) % 8))
        return s1_fail(ctx, S1_EINVAL, "s1_attention_gqa: heads must lie inside their rows, strides multiples of 8 elements");
    if (gate && (gate_head_stride < kD || ldg < (heads - 1) * gate_head_stride + kD || ((ldg | gate_head_stride) % 8)))
        return s1_fail(ctx, S1_EINVAL, "s1_attention_gqa: gate heads must lie inside their rows, strides multiples of 8 elements");
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(out) |
         reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(workspace)) & 15u)
        return s1_fail(ctx, S1_EINVAL, "s1_attention_gqa: pointers must be 16-byte aligned");
    if (!(scale > 0.f) || !(scale < 1e30f)) return s1_fail(ctx, S1_EINVAL, "s1_attention_gqa: scale must be positive and finite");
    if (!plan && workspace_bytes < s1_attention_gqa_workspace(num_seqs, total_tokens))
        return s1_fail(ctx, S1_EINVAL, "s1_attention_gqa: workspace of %zu bytes, %zu needed", workspace_bytes,
                       s1_attention_gqa_workspace(num_seqs, total_tokens));
    if (num_seqs == 0 || total_tokens == 0) return S1_OK;
    S1_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    int nb = 0;
    const QBlock* blocks_dev = nullptr;
    if (plan) {
        nb = plan->num_blocks;
        blocks_dev = reinterpret_cast<const QBlock*>(plan->dev + plan->gqa_off);
    } else {
        if (cu_seqlens_host[0] != 0 || cu_seqlens_host[num_seqs] != total_tokens)
            return s1_fail(ctx, S1_EINVAL, "s1_attention_gqa: cu_seqlens must run from 0 to total_tokens");
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(ctx->stream, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone)
            return s1_fail(ctx, S1_EINVAL, "s1_attention_gqa: with cu_seqlens_host the call copies a table from host memory and "
                                           "cannot be captured; build a batch plan first (s1_batch_plan)");
        const size_t max_blocks = static_cast<size_t>(total_tokens / kQB + num_seqs + 1);
        ctx->host_scratch.resize(sizeof(QBlock) * max_blocks);
        QBlock* blocks = reinterpret_cast<QBlock*>(ctx->host_scratch.data());
        for (int s = 0; s < num_seqs; ++s) {
            const int a = cu_seqlens_host[s], len = cu_seqlens_host[s + 1] - a;
            if (len < 0) return s1_fail(ctx, S1_EINVAL, "s1_attention_gqa: cu_seqlens must not decrease");
            for (int b = 0; b * kQB < len; ++b) blocks[nb++] = QBlock{a, len, b, 0};
        }
        if (nb == 0) return S1_OK;
        // a causal block's work grows with its position in the sequence: latest blocks first
        std::stable_sort(blocks, blocks + nb, [](const QBlock& x, const QBlock& y) { return x.qb > y.qb; });
        S1_CUDA_OK(ctx, cudaMemcpyAsync(workspace, blocks, sizeof(QBlock) * nb, cudaMemcpyHostToDevice, ctx->stream));
        blocks_dev = static_cast<const QBlock*>(workspace);
    }
    if (nb == 0) return S1_OK;

    CUtensorMap tq, tk, tv;
    int rc = s1_get_tmap(ctx, q, total_tokens, qw, ldq, kQB, 64, 2, 128, &tq);
    if (rc) return rc;
    rc = s1_get_tmap(ctx, k, total_tokens, kw, ldk, kKB, 64, 2, 128, &tk);
    if (rc) return rc;
    rc = s1_get_tmap(ctx, v, total_tokens, vw, ldv, kKB, 64, 2, 128, &tv);
    if (rc) return rc;
    GqaParams gp;
    gp.blocks = blocks_dev;
    gp.out = static_cast<__nv_bfloat16*>(out);
    gp.ldo = ldo;
    gp.gate = static_cast<const __nv_bfloat16*>(gate);
    gp.ldg = ldg;
    gp.gate_head_stride = gate_head_stride;
    gp.q_head_stride = q_head_stride;
    gp.k_head_stride = k_head_stride;
    gp.v_head_stride = v_head_stride;
    gp.heads_per_kv = heads / kv_heads;
    gp.scale_log2 = scale * 1.4426950408889634f;
    gp.status = ctx->status_dev;
    static thread_local int configured_device = -1;
    if (configured_device != ctx->device) {
        S1_CUDA_OK(ctx, cudaFuncSetAttribute(s1_attention_gqa_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGqaSmem));
        configured_device = ctx->device;
    }
    s1_attention_gqa_kernel<<<dim3(nb, heads), 288, kGqaSmem, ctx->stream>>>(tq, tk, tv, gp);
    S1_CUDA_OK(ctx, cudaGetLastError());
    ctx->launches += 1;
    return S1_OK;
}
