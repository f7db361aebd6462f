// Bidirectional softmax attention over a token-packed batch, optional +-window band, head dim 64, on tcgen05.
//
// What the reference computes in `scaled_dot_product_attention` / `eager_attention`
// (src/archs/modernbert.rs:313-351) with its masks (`local_attention_mask`, :1058-1076: keys further than
// local_attention / 2 from the query are masked; padded keys never exist in the packed layout):
//     a_i = sum_j softmax_j( q_i . k_j / sqrt(D) ) v_j     over the keys j of the same sequence (|i - j| <= window)
// in flash form: the score matrix never leaves the chip. On a B200 the reference has no fused attention at all
// (its flash-attn path is refused for compute capability >= 10, build.rs:53-55) and materialises [L, L] scores.
//
// One CTA per (128-query block of one sequence, head); 9 warps:
//   warp 8      : TMA loads (Q once; K and V tiles of 128 keys, each through its own 2-stage ring) and the MMAs:
//                 S = Q K^T (M = 128 queries, N = 128 keys, K = 64) and O += P V (M = 128, N = 64, K = 128 keys,
//                 V consumed as stored, token rows x dims = MN-major B operand); S and O live in TMEM
//   warps 0..7  : two threads per query row (warps w and w + 4 read the same 32 TMEM lanes; one takes keys 0..63 of
//                 the tile, the other keys 64..127). Each pulls its 64 scores into registers in one go (which frees
//                 S: the next tile's S = Q K^T runs under this tile's softmax), the pair agrees on the row maximum
//                 through two spare TMEM columns, then each exponentiates (f32, ex2 with the scale folded into one
//                 fma), adds up its part of the row sum and rounds P to bf16 into a swizzled A-operand tile. O stays
//                 in TMEM and is accumulated by the MMA itself; it is rescaled there only when a row maximum has
//                 grown by more than 2^8 since the last rescale (the final division by the row sum makes the
//                 reference maximum immaterial), so the common tile costs no pass over O at all.
// Key tiles of banded layers start at the first key of the band (no alignment to 128), so a query block meets two
// tiles, not three. Two CTAs fit per SM (112 KB shared memory, 256 TMEM columns each): four softmax warps per
// scheduler keep the special-function unit fed. Every mbarrier wait is bounded.
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
// Barrier of the two warps that share a quarter of the query rows (ids 1..4; 0 is __syncthreads).
__device__ __forceinline__ void pair_barrier(int q4) {
    if (q4 == 0) named_barrier<1, 64>();
    else if (q4 == 1) named_barrier<2, 64>();
    else if (q4 == 2) named_barrier<3, 64>();
    else named_barrier<4, 64>();
}
// The same barrier, carrying one bit: true if any of the 64 threads says so.
__device__ __forceinline__ bool pair_any(int q4, bool mine) {
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
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

constexpr float kRescaleLog2 = 8.f;  // O is rescaled when a row maximum has grown by more than this many powers of two

__global__ void __launch_bounds__(288, 2)
s1_attention_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t base = smem_u32(smem_raw);
    if (base & 1023u) {  // the swizzled tiles need 1024-byte alignment; never seen otherwise, reported instead of assumed
        if (threadIdx.x == 0 && atomicCAS(p.status, 0, 5) == 0) p.status[1] = blockIdx.x, p.status[2] = 39, p.status[3] = base & 1023u;
        return;
    }
    uint8_t* al = smem_raw;
    const uint32_t sq = base, sk = base + kTile, sv = base + 3 * kTile, sp = base + 5 * kTile;
    uint64_t* bars = reinterpret_cast<uint64_t*>(al + 7 * kTile);
    // bars: 0 Q full; 1,2 K full; 3,4 V full; 5 S ready; 6 S read (8 warps); 7 P ready (8 warps); 8 PV done
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t b0 = smem_u32(bars);
    const uint32_t bar_q = b0, full_k = b0 + 8, full_v = b0 + 24, bar_s = b0 + 40, bar_sfree = b0 + 48, bar_p = b0 + 56, bar_o = b0 + 64;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const QBlock qb = p.blocks[blockIdx.x];
    const int head = blockIdx.y;
    const int q_lo = qb.qb * kQB;                                  // first query (index inside the sequence)
    const int q_hi = min(q_lo + kQB, qb.seq_len) - 1;              // last valid query
    const int k_first = p.window < 0 ? 0 : max(0, q_lo - p.window);
    const int k_last = p.window < 0 ? qb.seq_len - 1 : min(qb.seq_len - 1, q_hi + p.window);
    const int nkb = (k_last - k_first) / kQB + 1;                  // key tile i holds keys k_first + 128 i ...

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
        tmem_alloc(smem_u32(tmem_slot), 256);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;  // columns 0..127: S, 128..191: O, 192..197: the row pairs' exchange
    int fail = 0;

    if (warp == 8) {
        if (lane == 0) {
            const int x = head * kHD;
            const int y0 = qb.seq_start + k_first;
            auto load_k = [&](int i) {
                const uint32_t fb = full_k + 8u * (i & 1);
                mbar_arrive_expect_tx(fb, kTile);
                tma_load_2d(sk + (i & 1) * kTile, &tmK, x, y0 + i * kQB, fb);
            };
            auto load_v = [&](int i) {
                const uint32_t fb = full_v + 8u * (i & 1);
                mbar_arrive_expect_tx(fb, kTile);
                tma_load_2d(sv + (i & 1) * kTile, &tmV, x, y0 + i * kQB, fb);
            };
            auto mma_s = [&](int i) {
                constexpr uint32_t idesc = make_idesc(1, 128, 128);
                const uint32_t kt = sk + (i & 1) * kTile;
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                    umma_bf16(tmem, make_sw128_kmajor_desc(sq) + 2u * kk, make_sw128_kmajor_desc(kt) + 2u * kk, idesc, kk ? 1u : 0u);
                umma_commit(bar_s);
            };
            mbar_arrive_expect_tx(bar_q, kTile);
            tma_load_2d(sq, &tmQ, x, qb.seq_start + q_lo, bar_q);
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
                    // S of tile i+1 as soon as the softmax warps hold tile i in registers: it runs under their softmax
                    if (!mbar_wait(full_k + 8u * ((i + 1) & 1), ((i + 1) >> 1) & 1, abort_flag)) { fail = 3; break; }
                    if (!mbar_wait(bar_sfree, i & 1, abort_flag)) { fail = 4; break; }
                    tc_fence_after();
                    mma_s(i + 1);
                    if (i + 2 < nkb) load_k(i + 2);  // its stage held K of tile i, whose S the softmax warps have read
                }
                if (!mbar_wait(bar_p, i & 1, abort_flag)) { fail = 5; break; }
                if (i >= 1 && i + 1 < nkb) {         // the other V stage held tile i-1: free once that PV has completed
                    if (!mbar_wait(bar_o, (i - 1) & 1, abort_flag)) { fail = 6; break; }
                    load_v(i + 1);
                }
                if (!mbar_wait(full_v + 8u * (i & 1), (i >> 1) & 1, abort_flag)) { fail = 7; break; }
                tc_fence_after();
                {
                    constexpr uint32_t idesc = make_idesc(1, 128, 64) | (1u << 16);  // B (= V) is MN-major
                    const uint32_t vt = sv + (i & 1) * kTile;
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk)  // 16 keys per instruction
                        umma_bf16(tmem + 128, make_sw128_kmajor_desc(sp + (kk >> 2) * kTile) + 2u * (kk & 3), mn_desc(vt) + 128u * kk,
                                  idesc, (kk || i) ? 1u : 0u);
                    umma_commit(bar_o);
                }
            }
        }
        __syncwarp();
    } else {
        const int q4 = warp & 3, ch = warp >> 2;           // TMEM lane quarter; which 64 keys of a tile / 32 output dims
        const int row = q4 * 32 + lane;                    // query row of the block = TMEM lane
        const bool q_ok = q_lo + row < qb.seq_len;
        const int qi = min(q_lo + row, qb.seq_len - 1);    // rows past the sequence compute like its last row; never stored
        const uint32_t lane_addr = tmem + (static_cast<uint32_t>(q4 * 32) << 16);
        const int lo = p.window < 0 ? 0 : max(0, qi - p.window), hi = p.window < 0 ? qb.seq_len - 1 : min(qb.seq_len - 1, qi + p.window);
        const uint32_t span = static_cast<uint32_t>(hi - lo);
        const float c = p.scale_log2;
        const uint32_t prow = sp + ch * kTile + static_cast<uint32_t>(row) * 128u, r7 = static_cast<uint32_t>(row) & 7u;
        float m_used = -INFINITY, l = 0.f;

        for (int i = 0; i < nkb; ++i) {
            const int j0 = k_first + i * kQB + ch * 64;    // first key of this thread's half tile (index inside the sequence)
            bool ok = mbar_wait(bar_s, i & 1, abort_flag);
            if (!__all_sync(0xffffffffu, ok)) { fail = 8; break; }
            tc_fence_after();
            uint32_t s[64];
            tmem_ld_32x32b_x32(lane_addr + ch * 64, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
            tmem_ld_32x32b_x32(lane_addr + ch * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_sfree);
            if (!(p.window < 0 && k_first + (i + 1) * kQB <= qb.seq_len)) {  // a tile that reaches past the band or the sequence
                const int rel = j0 - lo;
#pragma unroll
                for (int e = 0; e < 64; ++e)
                    if (static_cast<uint32_t>(rel + e) > span) s[e] = 0xff800000u;  // -inf
            }
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
            for (int e = 0; e < 64; e += 8) {
                mx0 = fmax3(mx0, __uint_as_float(s[e]), __uint_as_float(s[e + 1]));
                mx1 = fmax3(mx1, __uint_as_float(s[e + 2]), __uint_as_float(s[e + 3]));
                mx2 = fmax3(mx2, __uint_as_float(s[e + 4]), __uint_as_float(s[e + 5]));
                mx3 = fmax3(mx3, __uint_as_float(s[e + 6]), __uint_as_float(s[e + 7]));
            }
            const float mx_own = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
            // Does any row of this quarter need a new reference maximum - its own half's maximum more than 2^8 above the
            // one in use, or none in use yet? One bit through the pair's barrier settles it for both warps; only then is the
            // other half's maximum fetched (through two spare TMEM columns, double-buffered by tile parity). Most tiles past
            // a row's first few skip the exchange.
            // NaN (both -inf) compares false; -inf -> finite gives +inf, which rescales by ex2(-inf) = 0
            const bool rescale = pair_any(q4, i == 0 || (mx_own - m_used) * c > kRescaleLog2);
            float alpha = 1.f;
            if (rescale) {
                const uint32_t xcol = lane_addr + 192 + 2 * (i & 1);
                tmem_st_32x32b_x1(xcol + ch, __float_as_uint(mx_own));
                tmem_st_wait();
                tc_fence_before();
                pair_barrier(q4);
                tc_fence_after();
                const float mx_other = __uint_as_float(tmem_ld_32x32b_x1(xcol + (ch ^ 1)));
                tmem_ld_wait();
                const float m_new = fmaxf(m_used, fmaxf(mx_own, mx_other));
                if (i == 0) {
                    m_used = m_new;
                } else if (m_new != -INFINITY) {
                    alpha = ex2((m_used - m_new) * c);
                    m_used = m_new;
                }
            }
            const float neg_mc = (m_used == -INFINITY) ? 0.f : -m_used * c;
            uint32_t pk[32];
            float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
            for (int e = 0; e < 64; e += 2) {
                const float p0 = ex2(fmaf(__uint_as_float(s[e]), c, neg_mc));
                const float p1 = ex2(fmaf(__uint_as_float(s[e + 1]), c, neg_mc));
                sum0 += p0;
                sum1 += p1;
                pk[e >> 1] = pack_bf16x2_attn(p0, p1);
            }
            l = fmaf(l, alpha, sum0 + sum1);
            if (i >= 1) {  // P and O are the previous PV's operands until it has completed
                ok = mbar_wait(bar_o, (i - 1) & 1, abort_flag);
                if (!__all_sync(0xffffffffu, ok)) { fail = 9; break; }
                tc_fence_after();
                if (rescale) {  // this thread's 32 of the row's 64 output dims (i >= 1 here)
                    uint32_t o[32];
                    tmem_ld_32x32b_x32(lane_addr + 128 + ch * 32, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
                    tmem_st_32x32b_x32(lane_addr + 128 + ch * 32, o);
                    tmem_st_wait();
                }
            }
#pragma unroll
            for (int t = 0; t < 8; ++t) {  // 8 keys (16 bytes) per store into this half's P tile
                const uint32_t addr = prow + ((static_cast<uint32_t>(t) ^ r7) << 4);
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
            // the row sum is the two halves' sums, added in a fixed order
            tmem_st_32x32b_x1(lane_addr + 196 + ch, __float_as_uint(l));
            tmem_st_wait();
            tc_fence_before();
            pair_barrier(q4);
            tc_fence_after();
            const float l0 = ch == 0 ? l : __uint_as_float(tmem_ld_32x32b_x1(lane_addr + 196));
            const float l1 = ch == 1 ? l : __uint_as_float(tmem_ld_32x32b_x1(lane_addr + 197));
            tmem_ld_wait();
            const float inv = 1.f / (l0 + l1);
            __nv_bfloat16* orow = p.out + static_cast<long long>(qb.seq_start + qi) * p.ldo + head * kHD + ch * 32;
            uint32_t o[32];
            tmem_ld_32x32b_x32(lane_addr + 128 + ch * 32, o);
            tmem_ld_wait();
            if (q_ok) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    uint4 v;
                    v.x = pack_bf16x2_attn(__uint_as_float(o[8 * e]) * inv, __uint_as_float(o[8 * e + 1]) * inv);
                    v.y = pack_bf16x2_attn(__uint_as_float(o[8 * e + 2]) * inv, __uint_as_float(o[8 * e + 3]) * inv);
                    v.z = pack_bf16x2_attn(__uint_as_float(o[8 * e + 4]) * inv, __uint_as_float(o[8 * e + 5]) * inv);
                    v.w = pack_bf16x2_attn(__uint_as_float(o[8 * e + 6]) * inv, __uint_as_float(o[8 * e + 7]) * inv);
                    *reinterpret_cast<uint4*>(orow + 8 * e) = v;
                }
            }
            tc_fence_before();
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
    if (warp == 8) {
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
    if (!q || !k || !v || !out) return s1_fail(ctx, S1_EINVAL, "s1_attention: null pointer");
    const S1BatchPlan* plan = cu_seqlens_host ? nullptr : ctx->active_plan(num_seqs, total_tokens);
    if (!cu_seqlens_host && !plan)
        return s1_fail(ctx, S1_EINVAL, "s1_attention: cu_seqlens_host is NULL and no batch plan for this batch is in use");
    if (!plan && !workspace) return s1_fail(ctx, S1_EINVAL, "s1_attention: null workspace");
    if (head_dim != kHD) return s1_fail(ctx, S1_EINVAL, "s1_attention: head_dim must be 64 (got %d)", head_dim);
    if (heads < 1 || num_seqs < 0 || total_tokens < 0) return s1_fail(ctx, S1_EINVAL, "s1_attention: bad sizes");
    const long long width = 1LL * heads * kHD;
    if (ldq < width || ldk < width || ldv < width || ldo < width || (ldq % 8) || (ldk % 8) || (ldv % 8) || (ldo % 8))
        return s1_fail(ctx, S1_EINVAL, "s1_attention: rows need %lld columns and 16-byte alignment", width);
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(out) |
         reinterpret_cast<uintptr_t>(workspace)) & 15u)
        return s1_fail(ctx, S1_EINVAL, "s1_attention: pointers must be 16-byte aligned");
    static_assert(sizeof(QBlock) == sizeof(S1QBlock), "the plan's query-block table has this kernel's layout");
    if (!(scale > 0.f) || !(scale < 1e30f)) return s1_fail(ctx, S1_EINVAL, "s1_attention: scale must be positive and finite");
    if (!plan && workspace_bytes < s1_attention_workspace(num_seqs, total_tokens))
        return s1_fail(ctx, S1_EINVAL, "s1_attention: workspace of %zu bytes, %zu needed", workspace_bytes,
                       s1_attention_workspace(num_seqs, total_tokens));
    if (num_seqs == 0 || total_tokens == 0) return S1_OK;
    S1_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    int nb = 0;
    const QBlock* blocks_dev = nullptr;
    if (plan) {
        // the query-block table was built and copied once for the whole batch (s1_batch_plan)
        nb = plan->num_blocks;
        blocks_dev = reinterpret_cast<const QBlock*>(plan->dev + (window < 0 ? plan->attn_global_off : plan->attn_local_off));
    } else {
        if (cu_seqlens_host[0] != 0 || cu_seqlens_host[num_seqs] != total_tokens)
            return s1_fail(ctx, S1_EINVAL, "s1_attention: cu_seqlens must run from 0 to total_tokens");
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(ctx->stream, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone)
            return s1_fail(ctx, S1_EINVAL, "s1_attention: with cu_seqlens_host the call copies a table from host memory and "
                                           "cannot be captured; build a batch plan first (s1_batch_plan)");
        const size_t max_blocks = static_cast<size_t>(total_tokens / kQB + num_seqs + 1);
        ctx->host_scratch.resize(sizeof(QBlock) * max_blocks);
        QBlock* blocks = reinterpret_cast<QBlock*>(ctx->host_scratch.data());
        for (int s = 0; s < num_seqs; ++s) {
            const int a = cu_seqlens_host[s], len = cu_seqlens_host[s + 1] - a;
            if (len < 0) return s1_fail(ctx, S1_EINVAL, "s1_attention: cu_seqlens must not decrease");
            for (int b = 0; b * kQB < len; ++b) blocks[nb++] = QBlock{a, len, b, 0};
        }
        if (nb == 0) return S1_OK;
        // without a window the work of a block grows with its sequence: longest sequences first
        if (window < 0) std::stable_sort(blocks, blocks + nb, [](const QBlock& x, const QBlock& y) { return x.seq_len > y.seq_len; });
        S1_CUDA_OK(ctx, cudaMemcpyAsync(workspace, blocks, sizeof(QBlock) * nb, cudaMemcpyHostToDevice, ctx->stream));
        blocks_dev = static_cast<const QBlock*>(workspace);
    }
    if (nb == 0) return S1_OK;

    CUtensorMap tq, tk, tv;
    int rc = s1_get_tmap(ctx, q, total_tokens, width, ldq, kQB, kHD, 2, 128, &tq);
    if (rc) return rc;
    rc = s1_get_tmap(ctx, k, total_tokens, width, ldk, kQB, kHD, 2, 128, &tk);
    if (rc) return rc;
    rc = s1_get_tmap(ctx, v, total_tokens, width, ldv, kQB, kHD, 2, 128, &tv);
    if (rc) return rc;
    AttnParams ap;
    ap.blocks = blocks_dev;
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
    s1_attention_kernel<<<dim3(nb, heads), 288, kAttnSmem, ctx->stream>>>(tq, tk, tv, ap);
    S1_CUDA_OK(ctx, cudaGetLastError());
    ctx->launches += 1;
    return S1_OK;
}
