// The row-wise stages either side of the projections, on the packed layout:
//   s1_norm   LayerNorm without bias (ModernBERT `Norm`, src/archs/modernbert.rs:1006-1034: candle
//             `LayerNorm::new_no_bias`) and RMSNorm scaled by (1 + weight) (Qwen3.5 `RmsNorm`,
//             src/archs/qwen35_text.rs:178-203), optionally reading its rows through an index (the embedding
//             lookup that precedes the first norm, src/archs/modernbert.rs:1084-1092);
//   s1_rope   rotate-half rotary embedding applied in place to consecutive heads of every token row
//             (`rope_qkv`, src/kernels/modernbert.cu:31-62; partial rotation as in `Attention::rotary`,
//             src/archs/qwen35_text.rs:296-310). In place on the packed Wqkv output the q and k heads are rotated
//             where they lie and v is untouched, which is the layout s1_attention reads: the reference kernel's
//             copy into three separate [B, H, L, D] tensors is not needed.
// Both are HBM-bound streaming kernels: one 16-byte access per lane and step, statistics in f32, one rounding to
// bf16 at the end. Algorithmic bytes per row: 2 x width x 2 (norm), 2 x rotated columns x 2 (rope).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "context.h"

namespace {

struct NormParams {
    const __nv_bfloat16* x;
    long long ldx;
    const int32_t* gather;  // optional row index into x
    int gather_rows;
    const __nv_bfloat16* w;
    const __nv_bfloat16* b;  // optional bias (LayerNorm with bias: the heads' `layer_norm`, src/models/laya.rs:85-86,258)
    float eps;
    int kind;  // 0 LayerNorm (mean removed), 1 RMSNorm with (1 + w), 2 no normalisation: rows copied (through the index)
    __nv_bfloat16* y;
    long long ldy;
    long long rows;
    int width;
    int* status;
};

__device__ __forceinline__ void unpack8(const uint4& raw, float* f) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float2 t = __bfloat1622float2(h[e]);
        f[2 * e] = t.x;
        f[2 * e + 1] = t.y;
    }
}

__device__ __forceinline__ uint4 pack8(const float* f) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);
    return raw;
}

__device__ __forceinline__ float bf16r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

template <int LPR>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
    for (int off = LPR / 2; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

__device__ __forceinline__ const __nv_bfloat16* norm_row(const NormParams& p, long long row, bool& live) {
    long long r = row;
    if (live && p.gather) {
        const int id = p.gather[row];
        if (id < 0 || id >= p.gather_rows) {
            if (atomicCAS(p.status, 0, 101) == 0) {
                p.status[1] = static_cast<int>(blockIdx.x);
                p.status[2] = static_cast<int>(row);
                p.status[3] = id;
            }
            live = false;
        } else {
            r = id;
        }
    }
    return p.x + r * p.ldx;
}

// LPR lanes share a row and keep it in registers: MAXCH 16-byte chunks per lane (width <= 8 * LPR * MAXCH).
template <int MAXCH, int LPR>
__global__ void __launch_bounds__(256) s1_norm_kernel(const NormParams p) {
    constexpr int RPW = 32 / LPR;
    const int lane = threadIdx.x & 31, sub = lane % LPR;
    const long long warp = (static_cast<long long>(blockIdx.x) * 256 + threadIdx.x) >> 5;
    const long long row = warp * RPW + lane / LPR;
    bool live = row < p.rows;
    const __nv_bfloat16* src = norm_row(p, row, live);
    const int nchunks = p.width / 8;
    uint4 v[MAXCH];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < MAXCH; ++i) {
        const int c = sub + i * LPR;
        v[i] = make_uint4(0, 0, 0, 0);
        if (live && c < nchunks) {
            v[i] = *reinterpret_cast<const uint4*>(src + c * 8);
            float f[8];
            unpack8(v[i], f);
#pragma unroll
            for (int e = 0; e < 8; ++e) sum += f[e];
        }
    }
    const float inv_w = 1.f / static_cast<float>(p.width);
    const float mean = p.kind == 0 ? group_sum<LPR>(sum) * inv_w : 0.f;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < MAXCH; ++i) {
        if (sub + i * LPR < nchunks) {
            float f[8];
            unpack8(v[i], f);
#pragma unroll
            for (int e = 0; e < 8; ++e) sq += (f[e] - mean) * (f[e] - mean);
        }
    }
    const float rstd = 1.f / sqrtf(group_sum<LPR>(sq) * inv_w + p.eps);
    if (!live) return;
    const float one = p.kind == 1 ? 1.f : 0.f;
    __nv_bfloat16* dst = p.y + row * p.ldy;
#pragma unroll
    for (int i = 0; i < MAXCH; ++i) {
        const int c = sub + i * LPR;
        if (c < nchunks) {
            if (p.kind == 2) {
                *reinterpret_cast<uint4*>(dst + c * 8) = v[i];
                continue;
            }
            float f[8], g[8], bb[8];
            unpack8(v[i], f);
            unpack8(__ldg(reinterpret_cast<const uint4*>(p.w + c * 8)), g);
            unpack8(p.b ? __ldg(reinterpret_cast<const uint4*>(p.b + c * 8)) : make_uint4(0, 0, 0, 0), bb);
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = (f[e] - mean) * rstd * (g[e] + one) + bb[e];
            *reinterpret_cast<uint4*>(dst + c * 8) = pack8(f);
        }
    }
}

// Any width (beyond 6144): one warp per row, the row re-read from L1 for each pass.
__global__ void __launch_bounds__(256) s1_norm_wide_kernel(const NormParams p) {
    const int lane = threadIdx.x & 31;
    const long long row = (static_cast<long long>(blockIdx.x) * 256 + threadIdx.x) >> 5;
    bool live = row < p.rows;
    const __nv_bfloat16* src = norm_row(p, row, live);
    const int nchunks = live ? p.width / 8 : 0;
    float sum = 0.f;
    if (p.kind == 0) {
        for (int c = lane; c < nchunks; c += 32) {
            float f[8];
            unpack8(*reinterpret_cast<const uint4*>(src + c * 8), f);
#pragma unroll
            for (int e = 0; e < 8; ++e) sum += f[e];
        }
    }
    const float inv_w = 1.f / static_cast<float>(p.width);
    const float mean = p.kind == 0 ? group_sum<32>(sum) * inv_w : 0.f;
    float sq = 0.f;
    for (int c = lane; c < nchunks; c += 32) {
        float f[8];
        unpack8(*reinterpret_cast<const uint4*>(src + c * 8), f);
#pragma unroll
        for (int e = 0; e < 8; ++e) sq += (f[e] - mean) * (f[e] - mean);
    }
    const float rstd = 1.f / sqrtf(group_sum<32>(sq) * inv_w + p.eps);
    const float one = p.kind == 1 ? 1.f : 0.f;
    __nv_bfloat16* dst = p.y + row * p.ldy;
    for (int c = lane; c < nchunks; c += 32) {
        if (p.kind == 2) {
            *reinterpret_cast<uint4*>(dst + c * 8) = *reinterpret_cast<const uint4*>(src + c * 8);
            continue;
        }
        float f[8], g[8], bb[8];
        unpack8(*reinterpret_cast<const uint4*>(src + c * 8), f);
        unpack8(__ldg(reinterpret_cast<const uint4*>(p.w + c * 8)), g);
        unpack8(p.b ? __ldg(reinterpret_cast<const uint4*>(p.b + c * 8)) : make_uint4(0, 0, 0, 0), bb);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = (f[e] - mean) * rstd * (g[e] + one) + bb[e];
        *reinterpret_cast<uint4*>(dst + c * 8) = pack8(f);
    }
}

template <int MAXCH, int LPR>
void launch_norm(const NormParams& p, cudaStream_t stream) {
    const long long rows_per_block = 8 * (32 / LPR);
    const unsigned blocks = static_cast<unsigned>((p.rows + rows_per_block - 1) / rows_per_block);
    s1_norm_kernel<MAXCH, LPR><<<blocks, 256, 0, stream>>>(p);
}

// ------------------------------------------------------------------------------------------------------ rope
// One thread per 8 column pairs: columns [u*8, u*8+8) of the first half of the rotated span and their partners
// `rot/2` further on. out_lo = lo*cos - hi*sin, out_hi = lo*sin + hi*cos in f32, rounded once.
__global__ void __launch_bounds__(256) s1_rope_kernel(__nv_bfloat16* __restrict__ x, long long ldx, const float* __restrict__ cos_t,
                                                      const float* __restrict__ sin_t, const int32_t* __restrict__ positions,
                                                      int max_pos, int T, int heads, long long head_stride, int rot,
                                                      int* __restrict__ status) {
    const int upr = rot / 16;  // units per head
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= static_cast<long long>(T) * heads * upr) return;
    const int u = static_cast<int>(idx % upr);
    const int head = static_cast<int>((idx / upr) % heads);
    const long long t = idx / (static_cast<long long>(upr) * heads);
    const int pos = positions[t];
    if (pos < 0 || pos >= max_pos) {
        if (atomicCAS(status, 0, 102) == 0) {
            status[1] = static_cast<int>(blockIdx.x);
            status[2] = static_cast<int>(t);
            status[3] = pos;
        }
        return;
    }
    const int half = rot / 2;
    __nv_bfloat16* lo_p = x + t * ldx + head * head_stride + u * 8;
    __nv_bfloat16* hi_p = lo_p + half;
    float lo[8], hi[8], c[8], s[8];
    unpack8(*reinterpret_cast<const uint4*>(lo_p), lo);
    unpack8(*reinterpret_cast<const uint4*>(hi_p), hi);
    const float4* cp = reinterpret_cast<const float4*>(cos_t + static_cast<long long>(pos) * half + u * 8);
    const float4* sp = reinterpret_cast<const float4*>(sin_t + static_cast<long long>(pos) * half + u * 8);
    *reinterpret_cast<float4*>(c) = __ldg(cp);
    *reinterpret_cast<float4*>(c + 4) = __ldg(cp + 1);
    *reinterpret_cast<float4*>(s) = __ldg(sp);
    *reinterpret_cast<float4*>(s + 4) = __ldg(sp + 1);
    float a[8], b[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        a[e] = __fsub_rn(__fmul_rn(lo[e], c[e]), __fmul_rn(hi[e], s[e]));  // no fused multiply-add: each product rounded,
        b[e] = __fadd_rn(__fmul_rn(lo[e], s[e]), __fmul_rn(hi[e], c[e]));  // as the reference's tensor ops do
    }
    *reinterpret_cast<uint4*>(lo_p) = pack8(a);
    *reinterpret_cast<uint4*>(hi_p) = pack8(b);
}


// ------------------------------------------------------------------------------------------- per-head norm + rope
// RMSNorm scaled by (1 + weight) over the head_dim columns of every (token, head), rounded to bf16 as the reference
// materialises it, then the partial rotate-half rotation of the first `rot` columns, all in one pass over the data
// (`q_norm` / `k_norm` followed by `Attention::rotary`, src/archs/qwen35_text.rs:296-339). LPR lanes share a head.
// bf16_ops = 1 rounds the way candle's bf16 tensor ops do (:302): each product and the sum are bf16 values;
// bf16_ops = 0 forms the rotation in f32 and rounds once (the arithmetic of s1_rope).
template <int LPR>
__global__ void __launch_bounds__(256) s1_head_norm_rope_kernel(__nv_bfloat16* __restrict__ x, long long ldx, long long head_stride,
                                                               int heads, const __nv_bfloat16* __restrict__ w, float eps,
                                                               const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                                               const int32_t* __restrict__ positions, int max_pos, int rot,
                                                               long long rows, int bf16_ops, int* __restrict__ status) {
    constexpr int RPW = 32 / LPR;
    const int lane = threadIdx.x & 31, sub = lane % LPR;
    const long long warp = (static_cast<long long>(blockIdx.x) * 256 + threadIdx.x) >> 5;
    const long long row = warp * RPW + lane / LPR;
    const bool live = row < rows;
    const long long t = live ? row / heads : 0;
    const int h = live ? static_cast<int>(row % heads) : 0;
    __nv_bfloat16* ptr = x + t * ldx + h * head_stride + sub * 8;
    // Everything the row needs is requested before anything is computed: the token's position first (the table rows hang on
    // it), the row itself, then the cosine / sine entries of the lanes that rotate - the norm's reduction runs while they
    // are on their way, instead of three dependent round trips to memory one after the other.
    const int halfc = rot / 16;
    const bool rotates = live && sub < 2 * halfc;
    int pos = rotates ? __ldg(positions + t) : 0;
    const uint4 raw = live ? *reinterpret_cast<const uint4*>(ptr) : make_uint4(0, 0, 0, 0);
    const bool pos_ok = pos >= 0 && pos < max_pos;
    float c[8], sn[8];
    if (rotates && pos_ok) {
        const long long tb = static_cast<long long>(pos) * (rot / 2) + (sub % halfc) * 8;
        *reinterpret_cast<float4*>(c) = __ldg(reinterpret_cast<const float4*>(cos_t + tb));
        *reinterpret_cast<float4*>(c + 4) = __ldg(reinterpret_cast<const float4*>(cos_t + tb) + 1);
        *reinterpret_cast<float4*>(sn) = __ldg(reinterpret_cast<const float4*>(sin_t + tb));
        *reinterpret_cast<float4*>(sn + 4) = __ldg(reinterpret_cast<const float4*>(sin_t + tb) + 1);
    } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) c[e] = 1.f, sn[e] = 0.f;
    }
    float f[8];
    unpack8(raw, f);
    float sq = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) sq += f[e] * f[e];
    const float rstd = 1.f / sqrtf(group_sum<LPR>(sq) * (1.f / static_cast<float>(8 * LPR)) + eps);
    float g[8];
    unpack8(__ldg(reinterpret_cast<const uint4*>(w + sub * 8)), g);
    uint4 normed;
    {
        float y[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) y[e] = f[e] * rstd * (g[e] + 1.f);
        normed = pack8(y);
        unpack8(normed, f);  // the bf16 values the rotation starts from
    }
    // the partner half of the rotated span sits rot / 16 lanes away (every lane takes part in the exchange)
    uint4 other_raw;
    other_raw.x = __shfl_xor_sync(0xffffffffu, normed.x, halfc);
    other_raw.y = __shfl_xor_sync(0xffffffffu, normed.y, halfc);
    other_raw.z = __shfl_xor_sync(0xffffffffu, normed.z, halfc);
    other_raw.w = __shfl_xor_sync(0xffffffffu, normed.w, halfc);
    if (!live) return;
    if (rotates) {
        if (!pos_ok) {
            if (atomicCAS(status, 0, 102) == 0) {
                status[1] = static_cast<int>(blockIdx.x);
                status[2] = static_cast<int>(t);
                status[3] = pos;
            }
        } else {
            float o[8];
            unpack8(other_raw, o);
            const bool is_lo = sub < halfc;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float own_c = __fmul_rn(f[e], c[e]);
                const float oth_s = __fmul_rn(is_lo ? -o[e] : o[e], sn[e]);  // rotate_half = [-second, first]
                if (bf16_ops) f[e] = __fadd_rn(bf16r(own_c), bf16r(oth_s));
                else f[e] = is_lo ? __fsub_rn(own_c, __fmul_rn(o[e], sn[e])) : __fadd_rn(__fmul_rn(o[e], sn[e]), own_c);
            }
            normed = pack8(f);
        }
    }
    *reinterpret_cast<uint4*>(ptr) = normed;
}

// ------------------------------------------------------------------------------------------- indexed row add
// y[r, :] = bf16(x[r, :] + table[index[r], :]): one thread per 8 columns.
__global__ void __launch_bounds__(256) s1_add_rows_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                                                         const __nv_bfloat16* __restrict__ table, long long ldt,
                                                         const int32_t* __restrict__ index, int table_rows,
                                                         __nv_bfloat16* __restrict__ y, long long ldy, long long rows, int width,
                                                         int* __restrict__ status) {
    const int groups = width / 8;
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= rows * groups) return;
    const long long r = idx / groups;
    const int c = static_cast<int>(idx % groups) * 8;
    const int id = index[r];
    if (id < 0 || id >= table_rows) {
        if (atomicCAS(status, 0, 101) == 0) {
            status[1] = static_cast<int>(blockIdx.x);
            status[2] = static_cast<int>(r);
            status[3] = id;
        }
        return;
    }
    float a[8], b[8];
    unpack8(*reinterpret_cast<const uint4*>(x + r * ldx + c), a);
    unpack8(__ldg(reinterpret_cast<const uint4*>(table + static_cast<long long>(id) * ldt + c)), b);
#pragma unroll
    for (int e = 0; e < 8; ++e) a[e] += b[e];
    *reinterpret_cast<uint4*>(y + r * ldy + c) = pack8(a);
}

inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

extern "C" int s1_norm(s1_ctx* ctx, const void* x, long long ldx, const int32_t* gather, int gather_rows, const void* weight,
                       const void* bias, float eps, int kind, void* y, long long ldy, long long rows, int width) {
    if (!ctx) return S1_EINVAL;
    if (!x || !y || (!weight && kind != 2)) return s1_fail(ctx, S1_EINVAL, "s1_norm: null pointer");
    if (kind < 0 || kind > 2) return s1_fail(ctx, S1_EINVAL, "s1_norm: kind must be 0 (LayerNorm), 1 (RMSNorm) or 2 (copy)");
    if (rows < 0 || width < 8 || (width % 8)) return s1_fail(ctx, S1_EINVAL, "s1_norm: width must be a multiple of 8");
    if ((ldx % 8) || (ldy % 8) || ldx < width || ldy < width || !al16(x) || !al16(y) || !al16(weight) || !al16(bias))
        return s1_fail(ctx, S1_EINVAL, "s1_norm: rows and weight must be 16-byte aligned, ld >= width");
    if (gather && gather_rows <= 0) return s1_fail(ctx, S1_EINVAL, "s1_norm: gather needs the row count of x");
    if (rows == 0) return S1_OK;
    S1_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    NormParams p{static_cast<const __nv_bfloat16*>(x), ldx, gather, gather_rows, static_cast<const __nv_bfloat16*>(weight),
                 static_cast<const __nv_bfloat16*>(bias), eps, kind, static_cast<__nv_bfloat16*>(y), ldy, rows, width, ctx->status_dev};
    const int chunks = width / 8;
    if (chunks <= 8) launch_norm<1, 8>(p, ctx->stream);
    else if (chunks <= 16) launch_norm<1, 16>(p, ctx->stream);
    else if (chunks <= 32) launch_norm<1, 32>(p, ctx->stream);
    else if (chunks <= 64) launch_norm<2, 32>(p, ctx->stream);
    else if (chunks <= 128) launch_norm<4, 32>(p, ctx->stream);
    else if (chunks <= 256) launch_norm<8, 32>(p, ctx->stream);
    else if (chunks <= 512) launch_norm<16, 32>(p, ctx->stream);
    else if (chunks <= 768) launch_norm<24, 32>(p, ctx->stream);   // hidden 5120: the row still fits the warp's registers
    else s1_norm_wide_kernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, ctx->stream>>>(p);
    S1_CUDA_OK(ctx, cudaGetLastError());
    ctx->launches += 1;
    return S1_OK;
}

extern "C" int s1_rope(s1_ctx* ctx, void* x, long long ldx, const float* cos_table, const float* sin_table,
                       const int32_t* positions, int max_positions, int total_tokens, int heads, long long head_stride,
                       int rotary_dim) {
    if (!ctx) return S1_EINVAL;
    if (!x || !cos_table || !sin_table || !positions) return s1_fail(ctx, S1_EINVAL, "s1_rope: null pointer");
    if (total_tokens < 0 || heads < 1 || max_positions < 1 || rotary_dim < 16 || (rotary_dim % 16))
        return s1_fail(ctx, S1_EINVAL, "s1_rope: rotary_dim must be a multiple of 16");
    if (head_stride < rotary_dim || (head_stride % 8) || (ldx % 8) || ldx < (heads - 1) * head_stride + rotary_dim || !al16(x) ||
        !al16(cos_table) || !al16(sin_table))
        return s1_fail(ctx, S1_EINVAL, "s1_rope: heads must be 16-byte aligned and lie inside a row");
    if (total_tokens == 0) return S1_OK;
    S1_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    const long long n = static_cast<long long>(total_tokens) * heads * (rotary_dim / 16);
    s1_rope_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, ctx->stream>>>(
        static_cast<__nv_bfloat16*>(x), ldx, cos_table, sin_table, positions, max_positions, total_tokens, heads, head_stride,
        rotary_dim, ctx->status_dev);
    S1_CUDA_OK(ctx, cudaGetLastError());
    ctx->launches += 1;
    return S1_OK;
}

extern "C" int s1_head_norm_rope(s1_ctx* ctx, void* x, long long ldx, long long head_stride, int heads, int head_dim,
                                 const void* norm_weight, float eps, const float* cos_table, const float* sin_table,
                                 const int32_t* positions, int max_positions, int rotary_dim, int total_tokens, int bf16_ops) {
    if (!ctx) return S1_EINVAL;
    if (!x || !norm_weight || !cos_table || !sin_table || !positions) return s1_fail(ctx, S1_EINVAL, "s1_head_norm_rope: null pointer");
    if (head_dim != 64 && head_dim != 128 && head_dim != 256)
        return s1_fail(ctx, S1_EINVAL, "s1_head_norm_rope: head_dim must be 64, 128 or 256 (got %d)", head_dim);
    if (rotary_dim != 16 && rotary_dim != 32 && rotary_dim != 64 && rotary_dim != 128 && rotary_dim != 256)
        return s1_fail(ctx, S1_EINVAL, "s1_head_norm_rope: rotary_dim must be 16, 32, 64, 128 or 256 (got %d)", rotary_dim);
    if (rotary_dim > head_dim) return s1_fail(ctx, S1_EINVAL, "s1_head_norm_rope: rotary_dim exceeds head_dim");
    if (total_tokens < 0 || heads < 1 || max_positions < 1) return s1_fail(ctx, S1_EINVAL, "s1_head_norm_rope: bad sizes");
    if (head_stride < head_dim || (head_stride % 8) || (ldx % 8) || ldx < (heads - 1) * head_stride + head_dim || !al16(x) ||
        !al16(norm_weight) || !al16(cos_table) || !al16(sin_table))
        return s1_fail(ctx, S1_EINVAL, "s1_head_norm_rope: heads must be 16-byte aligned and lie inside a row");
    if (total_tokens == 0) return S1_OK;
    S1_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    const long long rows = static_cast<long long>(total_tokens) * heads;
    auto* xp = static_cast<__nv_bfloat16*>(x);
    auto* wp = static_cast<const __nv_bfloat16*>(norm_weight);
    const int lpr = head_dim / 8;
    const unsigned blocks = static_cast<unsigned>((rows + 8 * (32 / lpr) - 1) / (8 * (32 / lpr)));
#define S1_HNR(LPR_)                                                                                                       \
    s1_head_norm_rope_kernel<LPR_><<<blocks, 256, 0, ctx->stream>>>(xp, ldx, head_stride, heads, wp, eps, cos_table, sin_table, \
                                                                    positions, max_positions, rotary_dim, rows, bf16_ops, ctx->status_dev)
    if (lpr == 8) S1_HNR(8);
    else if (lpr == 16) S1_HNR(16);
    else S1_HNR(32);
#undef S1_HNR
    S1_CUDA_OK(ctx, cudaGetLastError());
    ctx->launches += 1;
    return S1_OK;
}

extern "C" int s1_add_rows(s1_ctx* ctx, const void* x, long long ldx, const void* table, long long ldt, const int32_t* index,
                           int table_rows, void* y, long long ldy, long long rows, int width) {
    if (!ctx) return S1_EINVAL;
    if (!x || !table || !index || !y) return s1_fail(ctx, S1_EINVAL, "s1_add_rows: null pointer");
    if (rows < 0 || table_rows < 1 || width < 8 || (width % 8)) return s1_fail(ctx, S1_EINVAL, "s1_add_rows: width must be a multiple of 8");
    if ((ldx % 8) || (ldy % 8) || (ldt % 8) || ldx < width || ldy < width || ldt < width || !al16(x) || !al16(y) || !al16(table))
        return s1_fail(ctx, S1_EINVAL, "s1_add_rows: rows must be 16-byte aligned, ld >= width");
    if (rows == 0) return S1_OK;
    S1_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    const long long n = rows * (width / 8);
    s1_add_rows_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, ctx->stream>>>(
        static_cast<const __nv_bfloat16*>(x), ldx, static_cast<const __nv_bfloat16*>(table), ldt, index, table_rows,
        static_cast<__nv_bfloat16*>(y), ldy, rows, width, ctx->status_dev);
    S1_CUDA_OK(ctx, cudaGetLastError());
    ctx->launches += 1;
    return S1_OK;
}
