// The elementwise stages around the gated delta rule of the Qwen3.5 linear-attention layer, on the packed
// layout, and the entry point that chains them with the chunked recurrence:
//   s1_conv_silu      causal depthwise conv + SiLU   (src/kernels/qwen35.cu:3-29; src/archs/qwen35_text.rs:632-650)
//   s1_delta_inputs   split / head-repeat / L2-norm / gates  (`delta_inputs`, src/archs/qwen35_text.rs:528-579;
//                     the Metal build fuses the same steps in src/kernels/qwen35.metal:146-203)
//   s1_delta_finish   per-head RMS norm x weight x SiLU(z), cast to bf16 (`finish_delta`, :597-626, up to out_proj)
//   (s1_gated_delta_rule, in delta_chunked.cu, does the first of these inside its own first kernel and calls the last)
// All three are HBM-bound streaming kernels: 16-byte accesses, one warp per (token, head) row where a
// reduction over the head dimension is needed.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "context.h"

namespace {

__device__ __forceinline__ float bf16r(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// ------------------------------------------------------------------------------------------------ conv + SiLU
// y[t, c] = silu( sum_tap x[t + tap - taps + 1, c] * w[c, tap] ), taps that reach before the token's own sequence
// are skipped (zero left padding per sequence); the running sum and every product are rounded to bf16 tap by
// tap, as the reference kernel does.
__global__ void __launch_bounds__(256) s1_conv_silu_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                                                           const __nv_bfloat16* __restrict__ w, const int32_t* __restrict__ positions,
                                                           int T, int C, int taps, __nv_bfloat16* __restrict__ y, long long ldy) {
    const int groups = C / 8;  // 8 channels (16 bytes) per thread
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= static_cast<long long>(T) * groups) return;
    const int t = static_cast<int>(idx / groups), c0 = static_cast<int>(idx % groups) * 8;
    const int pos = positions[t];
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    for (int tap = 0; tap < taps; ++tap) {
        const int back = taps - 1 - tap;  // how many tokens before t this tap reads
        if (back > pos) continue;
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(x + static_cast<long long>(t - back) * ldx + c0));
        const __nv_bfloat16* xv = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float prod = bf16r(__bfloat162float(xv[e]) * __bfloat162float(w[static_cast<long long>(c0 + e) * taps + tap]));
            acc[e] = bf16r(acc[e] + prod);
        }
    }
    __nv_bfloat16 out[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) out[e] = __float2bfloat16_rn(acc[e] / (1.f + expf(-acc[e])));
    *reinterpret_cast<uint4*>(y + static_cast<long long>(t) * ldy + c0) = *reinterpret_cast<const uint4*>(out);
}

// The same arithmetic for the usual 4 taps, memory-bound: each thread takes 8 channels (16 bytes) of TT consecutive tokens.
//  * every row it needs (TT rows and the three before them) is requested up front, so TT + 3 independent 16-byte loads
//    are in flight per thread; each input row is read once (plus 3 / TT for the history) and the weights once per thread;
//  * the per-tap arithmetic is native bf16x2: `__hmul2_rn` is the exact product rounded once to bf16 and `__hadd2_rn` the
//    sum rounded once, which is what the reference's `T(__fadd_rn(float(value), float(T(product))))` yields (the f32
//    product of two bf16 values is exact; an f32 sum of two bf16 values is either exact or, when the exponents are
//    more than 16 bits apart, rounds to the larger operand either way);
//  * a tap that would read a token before the start of the sequence contributes a zero row (the reference skips it).
// SiLU in f32 with the fast exponential and reciprocal (relative error ~2^-22, far below the bf16 rounding that follows).
// TT = 8: 11 rows (44 registers) in flight per thread, three blocks per SM.
// x / (1 + e^-x) with the special-function unit's exponential and reciprocal (two instructions instead of two library calls)
__device__ __forceinline__ float silu_fast(float v) {
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(v * -1.4426950408889634f));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.f + e));
    return v * r;
}

template <int TT>
__global__ void __launch_bounds__(256, 3) s1_conv_silu_walk_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                                                                   const __nv_bfloat16* __restrict__ w, const int32_t* __restrict__ positions,
                                                                   int T, int C, __nv_bfloat16* __restrict__ y, long long ldy) {
    constexpr int TAPS = 4;
    const int groups = C / 8;
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long chunks = (T + TT - 1) / TT;
    if (idx >= chunks * groups) return;
    const int c0 = static_cast<int>(idx % groups) * 8;
    const int t0 = static_cast<int>(idx / groups) * TT;
    // rows t0 - 3 .. t0 + TT - 1, all requested before any is used
    uint4 rows[TT + TAPS - 1];
#pragma unroll
    for (int i = 0; i < TT + TAPS - 1; ++i) {
        const int t = t0 - (TAPS - 1) + i;
        rows[i] = make_uint4(0u, 0u, 0u, 0u);
        if (t >= 0 && t < T) rows[i] = __ldg(reinterpret_cast<const uint4*>(x + static_cast<long long>(t) * ldx + c0));
    }
    int pos[TT];
#pragma unroll
    for (int i = 0; i < TT; ++i) pos[i] = (t0 + i < T) ? __ldg(positions + t0 + i) : 0;
    // weights [8 channels][4 taps] (64 contiguous bytes) -> per tap four bf16x2 pairs of neighbouring channels
    uint32_t wraw[16];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint4 r = __ldg(reinterpret_cast<const uint4*>(w + static_cast<long long>(c0) * TAPS) + i);
        wraw[4 * i] = r.x, wraw[4 * i + 1] = r.y, wraw[4 * i + 2] = r.z, wraw[4 * i + 3] = r.w;
    }
    // channel ch holds taps (0,1) in wraw[2 ch] and (2,3) in wraw[2 ch + 1]; pair p = channels 2p, 2p + 1
    __nv_bfloat162 wt[TAPS][4];
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        const uint32_t a01 = wraw[4 * p], a23 = wraw[4 * p + 1], b01 = wraw[4 * p + 2], b23 = wraw[4 * p + 3];
        const uint32_t t0w = __byte_perm(a01, b01, 0x5410), t1w = __byte_perm(a01, b01, 0x7632);
        const uint32_t t2w = __byte_perm(a23, b23, 0x5410), t3w = __byte_perm(a23, b23, 0x7632);
        wt[0][p] = *reinterpret_cast<const __nv_bfloat162*>(&t0w);
        wt[1][p] = *reinterpret_cast<const __nv_bfloat162*>(&t1w);
        wt[2][p] = *reinterpret_cast<const __nv_bfloat162*>(&t2w);
        wt[3][p] = *reinterpret_cast<const __nv_bfloat162*>(&t3w);
    }
    const __nv_bfloat162 zero2 = __floats2bfloat162_rn(0.f, 0.f);
    // no sequence starts inside or just before this run of tokens (the usual case; the same for a whole warp when a row
    // has at least 32 channel groups): every tap of every token is live and no row has to be masked
    bool clean = true;
#pragma unroll
    for (int tt = 0; tt < TT; ++tt) clean = clean && (pos[tt] >= TAPS - 1 || t0 + tt >= T);
#pragma unroll
    for (int tt = 0; tt < TT; ++tt) {
        if (t0 + tt >= T) break;
        __nv_bfloat162 acc[4] = {zero2, zero2, zero2, zero2};
#pragma unroll
        for (int tap = 0; tap < TAPS; ++tap) {
            const uint4 r = rows[tt + tap];     // row t - (TAPS - 1 - tap)
            uint32_t rr[4] = {r.x, r.y, r.z, r.w};
            if (!clean && TAPS - 1 - tap > pos[tt]) rr[0] = rr[1] = rr[2] = rr[3] = 0u;  // a row of the previous sequence
#pragma unroll
            for (int p = 0; p < 4; ++p)  // the _rn forms are never contracted into one fma
                acc[p] = __hadd2_rn(acc[p], __hmul2_rn(*reinterpret_cast<const __nv_bfloat162*>(&rr[p]), wt[tap][p]));
        }
        uint32_t out[4];
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const float2 a = __bfloat1622float2(acc[p]);
            const __nv_bfloat162 o = __floats2bfloat162_rn(silu_fast(a.x), silu_fast(a.y));
            out[p] = *reinterpret_cast<const uint32_t*>(&o);
        }
        *reinterpret_cast<uint4*>(y + static_cast<long long>(t0 + tt) * ldy + c0) = make_uint4(out[0], out[1], out[2], out[3]);
    }
}

// ------------------------------------------------------------------------------------------------ delta inputs
// One warp per (token, value head): key head = value head / (Hv / Hk) (src/archs/qwen35_text.rs:552-559).
__global__ void __launch_bounds__(256) s1_delta_inputs_kernel(const __nv_bfloat16* __restrict__ mixed, long long ldm,
                                                              const __nv_bfloat16* __restrict__ bproj, const __nv_bfloat16* __restrict__ aproj,
                                                              long long ldba, const float* __restrict__ dt_bias,
                                                              const float* __restrict__ neg_exp_a, int T, int Hk, int Hv,
                                                              float* __restrict__ q, float* __restrict__ k, float* __restrict__ v,
                                                              float* __restrict__ g, float* __restrict__ beta) {
    const long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= static_cast<long long>(T) * Hv) return;
    const int t = static_cast<int>(wid / Hv), hv = static_cast<int>(wid % Hv);
    const int hk = hv / (Hv / Hk);
    const __nv_bfloat16* row = mixed + static_cast<long long>(t) * ldm;
    const int kw = Hk * 128;
    auto load4 = [&](const __nv_bfloat16* p, float (&f)[4]) {
        const uint2 raw = __ldg(reinterpret_cast<const uint2*>(p + 4 * lane));
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
        f[0] = __low2float(a), f[1] = __high2float(a), f[2] = __low2float(b), f[3] = __high2float(b);
    };
    float qf[4], kf[4], vf[4];
    load4(row + hk * 128, qf);
    load4(row + kw + hk * 128, kf);
    load4(row + 2 * kw + hv * 128, vf);
    float sq = qf[0] * qf[0] + qf[1] * qf[1] + qf[2] * qf[2] + qf[3] * qf[3];
    float sk = kf[0] * kf[0] + kf[1] * kf[1] + kf[2] * kf[2] + kf[3] * kf[3];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        sq += __shfl_xor_sync(0xffffffffu, sq, o);
        sk += __shfl_xor_sync(0xffffffffu, sk, o);
    }
    const float iq = 0.08838834764831845f / sqrtf(sq + 1e-6f);  // 128^-1/2 / sqrt(sum q^2 + 1e-6)
    const float ik = 1.f / sqrtf(sk + 1e-6f);
    const long long o = (static_cast<long long>(t) * Hv + hv) * 128 + 4 * lane;
    *reinterpret_cast<float4*>(q + o) = make_float4(qf[0] * iq, qf[1] * iq, qf[2] * iq, qf[3] * iq);
    *reinterpret_cast<float4*>(k + o) = make_float4(kf[0] * ik, kf[1] * ik, kf[2] * ik, kf[3] * ik);
    *reinterpret_cast<float4*>(v + o) = make_float4(vf[0], vf[1], vf[2], vf[3]);
    if (lane == 0) {
        const float bb = __bfloat162float(bproj[static_cast<long long>(t) * ldba + hv]);
        const float aa = __bfloat162float(aproj[static_cast<long long>(t) * ldba + hv]) + dt_bias[hv];
        beta[static_cast<long long>(t) * Hv + hv] = 1.f / (1.f + expf(-bb));
        const float softplus = fmaxf(aa, 0.f) + logf(expf(-fabsf(aa)) + 1.f);
        g[static_cast<long long>(t) * Hv + hv] = softplus * neg_exp_a[hv];
    }
}

// ------------------------------------------------------------------------------------------------ finish
__global__ void __launch_bounds__(256) s1_delta_finish_kernel(const float* __restrict__ o, const __nv_bfloat16* __restrict__ z,
                                                              long long ldz, const __nv_bfloat16* __restrict__ norm_w, float eps, int T,
                                                              int Hv, __nv_bfloat16* __restrict__ y, long long ldy) {
    const long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= static_cast<long long>(T) * Hv) return;
    const int t = static_cast<int>(wid / Hv), hv = static_cast<int>(wid % Hv);
    const float4 ov = __ldg(reinterpret_cast<const float4*>(o + (static_cast<long long>(t) * Hv + hv) * 128) + lane);
    float ss = ov.x * ov.x + ov.y * ov.y + ov.z * ov.z + ov.w * ov.w;
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, s);
    const float inv = rsqrtf(ss * (1.f / 128.f) + eps);
    const uint2 zr = __ldg(reinterpret_cast<const uint2*>(z + static_cast<long long>(t) * ldz + hv * 128 + 4 * lane));
    const uint2 wr = __ldg(reinterpret_cast<const uint2*>(norm_w + 4 * lane));
    const __nv_bfloat16* zv = reinterpret_cast<const __nv_bfloat16*>(&zr);
    const __nv_bfloat16* wv = reinterpret_cast<const __nv_bfloat16*>(&wr);
    const float of[4] = {ov.x, ov.y, ov.z, ov.w};
    __nv_bfloat16 out[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float gate = __bfloat162float(zv[e]);
        // fast exponential and reciprocal: relative error ~2^-22, far below the bf16 rounding of the result
        out[e] = __float2bfloat16_rn(of[e] * inv * __bfloat162float(wv[e]) * silu_fast(gate));
    }
    *reinterpret_cast<uint2*>(y + static_cast<long long>(t) * ldy + hv * 128 + 4 * lane) = *reinterpret_cast<const uint2*>(out);
}

inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

extern "C" int s1_conv_silu(s1_ctx* ctx, const void* x, long long ldx, const void* weight, const int32_t* positions,
                            int total_tokens, int channels, int taps, void* y, long long ldy) {
    if (!ctx) return S1_EINVAL;
    if (!x || !weight || !positions || !y) return s1_fail(ctx, S1_EINVAL, "s1_conv_silu: null pointer");
    if (total_tokens < 0 || channels < 8 || (channels % 8) || taps < 1 || taps > 16)
        return s1_fail(ctx, S1_EINVAL, "s1_conv_silu: channels must be a multiple of 8, 1 <= taps <= 16");
    if ((ldx % 8) || (ldy % 8) || ldx < channels || ldy < channels || !al16(x) || !al16(y))
        return s1_fail(ctx, S1_EINVAL, "s1_conv_silu: rows must be 16-byte aligned");
    {
        // every token reads the `taps - 1` rows before it, which another thread of the same launch would be overwriting:
        // the output must not overlap the input
        const char* xb = static_cast<const char*>(x);
        const char* yb = static_cast<const char*>(y);
        const long long xs = 2LL * (static_cast<long long>(total_tokens > 0 ? total_tokens - 1 : 0) * ldx + channels);
        const long long ys = 2LL * (static_cast<long long>(total_tokens > 0 ? total_tokens - 1 : 0) * ldy + channels);
        if (xb < yb + ys && yb < xb + xs)
            return s1_fail(ctx, S1_EINVAL, "s1_conv_silu: y overlaps x (the convolution cannot run in place)");
    }
    if (total_tokens == 0) return S1_OK;
    S1_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    if (taps == 4 && al16(weight)) {
        constexpr int TT = 8;
        const long long n = static_cast<long long>((total_tokens + TT - 1) / TT) * (channels / 8);
        s1_conv_silu_walk_kernel<TT><<<static_cast<unsigned>((n + 255) / 256), 256, 0, ctx->stream>>>(
            static_cast<const __nv_bfloat16*>(x), ldx, static_cast<const __nv_bfloat16*>(weight), positions, total_tokens, channels,
            static_cast<__nv_bfloat16*>(y), ldy);
    } else {
        const long long n = static_cast<long long>(total_tokens) * (channels / 8);
        s1_conv_silu_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, ctx->stream>>>(
            static_cast<const __nv_bfloat16*>(x), ldx, static_cast<const __nv_bfloat16*>(weight), positions, total_tokens, channels, taps,
            static_cast<__nv_bfloat16*>(y), ldy);
    }
    S1_CUDA_OK(ctx, cudaGetLastError());
    ctx->launches += 1;
    return S1_OK;
}

extern "C" int s1_delta_inputs(s1_ctx* ctx, const void* mixed, long long ldm, const void* b_proj, const void* a_proj,
                               long long ldba, const float* dt_bias, const float* neg_exp_a, int total_tokens, int key_heads,
                               int value_heads, float* q, float* k, float* v, float* g, float* beta) {
    if (!ctx) return S1_EINVAL;
    if (!mixed || !b_proj || !a_proj || !dt_bias || !neg_exp_a || !q || !k || !v || !g || !beta)
        return s1_fail(ctx, S1_EINVAL, "s1_delta_inputs: null pointer");
    if (key_heads < 1 || value_heads < key_heads || value_heads % key_heads)
        return s1_fail(ctx, S1_EINVAL, "s1_delta_inputs: value_heads must be a multiple of key_heads");
    const long long width = 2LL * key_heads * 128 + 1LL * value_heads * 128;
    if (ldm < width || (ldm % 4) || ldba < value_heads || !al16(mixed) || !al16(q) || !al16(k) || !al16(v))
        return s1_fail(ctx, S1_EINVAL, "s1_delta_inputs: mixed must have %lld columns per row, 8-byte aligned rows", width);
    if (total_tokens <= 0) return total_tokens == 0 ? S1_OK : s1_fail(ctx, S1_EINVAL, "s1_delta_inputs: negative token count");
    S1_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    const long long warps = static_cast<long long>(total_tokens) * value_heads;
    s1_delta_inputs_kernel<<<static_cast<unsigned>((warps + 7) / 8), 256, 0, ctx->stream>>>(
        static_cast<const __nv_bfloat16*>(mixed), ldm, static_cast<const __nv_bfloat16*>(b_proj), static_cast<const __nv_bfloat16*>(a_proj),
        ldba, dt_bias, neg_exp_a, total_tokens, key_heads, value_heads, q, k, v, g, beta);
    S1_CUDA_OK(ctx, cudaGetLastError());
    ctx->launches += 1;
    return S1_OK;
}

extern "C" int s1_delta_finish(s1_ctx* ctx, const float* o, const void* z, long long ldz, const void* norm_weight, float eps,
                               int total_tokens, int value_heads, void* y, long long ldy) {
    if (!ctx) return S1_EINVAL;
    if (!o || !z || !norm_weight || !y) return s1_fail(ctx, S1_EINVAL, "s1_delta_finish: null pointer");
    const long long width = 1LL * value_heads * 128;
    if (value_heads < 1 || ldz < width || ldy < width || (ldz % 4) || (ldy % 4) || !al16(o) || !al16(z) || !al16(y))
        return s1_fail(ctx, S1_EINVAL, "s1_delta_finish: z and y need %lld columns per row, 8-byte aligned rows", width);
    if (total_tokens <= 0) return total_tokens == 0 ? S1_OK : s1_fail(ctx, S1_EINVAL, "s1_delta_finish: negative token count");
    S1_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    const long long warps = static_cast<long long>(total_tokens) * value_heads;
    s1_delta_finish_kernel<<<static_cast<unsigned>((warps + 7) / 8), 256, 0, ctx->stream>>>(
        o, static_cast<const __nv_bfloat16*>(z), ldz, static_cast<const __nv_bfloat16*>(norm_weight), eps, total_tokens, value_heads,
        static_cast<__nv_bfloat16*>(y), ldy);
    S1_CUDA_OK(ctx, cudaGetLastError());
    ctx->launches += 1;
    return S1_OK;
}
