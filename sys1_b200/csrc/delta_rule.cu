// Gated delta rule over token-packed ragged batches, f32, key dim 128.
//
// Replaces `chunked_delta_rule(q, k, v, g, beta)` (src/archs/qwen35_text.rs:789-807), i.e. the reference's CUDA
// kernel `qwen35_delta_f32` (src/kernels/qwen35.cu:53-97) and its pack step (src/archs/qwen35_text.rs:755-786):
//     S *= exp(g_t);  r = S^T k_t;  delta = (v_t - r) * beta_t;  S += k_t delta^T;  o_t = S^T q_t,   S0 = 0
// per (sequence, value head), S in R^{128 x Dv}.
//
// Work split: value columns are independent, so one CTA owns 32 columns of one (sequence, head) and walks the
// sequence token by token; its 4 warps own 32 key rows each (a thread keeps S[32 rows][its column] in
// registers), so the state never leaves the register file. The two dot products over the key dimension are
// finished across the 4 warps through shared memory (one __syncthreads per token). q / k / v / g / beta of the
// next 16 tokens are prefetched with cp.async while the current 16 are consumed; every CTA reads each input
// element once (the reference kernel re-reads the whole input stream from every value-column block and has no
// prefetch).
#include <cuda_runtime.h>
#include <stdint.h>

#include "context.h"

namespace {

constexpr int kDk = 128;   // key head dim (the reference's CUDA path requires 128 as well, qwen35_text.rs:747)
constexpr int kCols = 32;  // value columns per CTA
constexpr int kTok = 16;   // tokens per prefetch tile
constexpr int kThreads = 128;

struct DeltaParams {
    const float* q;  // [T, H, 128] (token stride ts_qk, head stride 128)
    const float* k;
    const float* v;  // [T, H, Dv]
    const float* g;  // [T, H]
    const float* beta;
    float* out;      // [T, H, Dv]
    const int32_t* cu_seqlens;  // [num_seqs + 1]
    int num_seqs, H, Dv;
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
    const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

struct __align__(16) Tile {
    float k[kTok][kDk];
    float q[kTok][kDk];
    float v[kTok][kCols];
    float g[kTok];
    float beta[kTok];
};

__global__ void __launch_bounds__(kThreads) s1_delta_seq_kernel(const DeltaParams p) {
    __shared__ Tile tiles[2];
    __shared__ float red[2][4][kCols];
    __shared__ float opart[kTok][4][kCols];

    const int col_blocks = (p.Dv + kCols - 1) / kCols;
    int b = blockIdx.x;
    const int cb = b % col_blocks;
    b /= col_blocks;
    const int head = b % p.H;
    const int seq = b / p.H;
    const int t_begin = p.cu_seqlens[seq];
    const int len = p.cu_seqlens[seq + 1] - t_begin;
    if (len <= 0) return;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const long long qk_ts = static_cast<long long>(p.H) * kDk;  // token stride of q / k
    const long long v_ts = static_cast<long long>(p.H) * p.Dv;
    const float* qbase = p.q + static_cast<long long>(t_begin) * qk_ts + head * kDk;
    const float* kbase = p.k + static_cast<long long>(t_begin) * qk_ts + head * kDk;
    const float* vbase = p.v + static_cast<long long>(t_begin) * v_ts + head * p.Dv + cb * kCols;
    const float* gbase = p.g + static_cast<long long>(t_begin) * p.H + head;
    const float* bbase = p.beta + static_cast<long long>(t_begin) * p.H + head;
    float* obase = p.out + static_cast<long long>(t_begin) * v_ts + head * p.Dv + cb * kCols;

    auto prefetch = [&](int tile_idx, int buf) {
        const int t0 = tile_idx * kTok;
        const int n = min(kTok, len - t0);
        Tile& tl = tiles[buf];
        // k and q: n rows of 128 floats = 32 x 16 B each
        for (int i = tid; i < n * 32; i += kThreads) {
            const int r = i >> 5, c = (i & 31) * 4;
            cp_async16(&tl.k[r][c], kbase + (t0 + r) * qk_ts + c);
            cp_async16(&tl.q[r][c], qbase + (t0 + r) * qk_ts + c);
        }
        for (int i = tid; i < n * 8; i += kThreads) {
            const int r = i >> 3, c = (i & 7) * 4;
            if (cb * kCols + c < p.Dv) cp_async16(&tl.v[r][c], vbase + (t0 + r) * v_ts + c);
            else *reinterpret_cast<float4*>(&tl.v[r][c]) = make_float4(0.f, 0.f, 0.f, 0.f);  // columns past Dv
        }
        if (tid < n) {
            cp_async4(&tl.g[tid], gbase + static_cast<long long>(t0 + tid) * p.H);
            cp_async4(&tl.beta[tid], bbase + static_cast<long long>(t0 + tid) * p.H);
        }
        cp_async_commit();
    };

    float S[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) S[i] = 0.f;

    const int num_tiles = (len + kTok - 1) / kTok;
    prefetch(0, 0);
    for (int ti = 0; ti < num_tiles; ++ti) {
        const int buf = ti & 1;
        if (ti + 1 < num_tiles) {
            prefetch(ti + 1, buf ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const Tile& tl = tiles[buf];
        const int n = min(kTok, len - ti * kTok);
        for (int t = 0; t < n; ++t) {
            const float decay = expf(tl.g[t]);
            const float4* k4 = reinterpret_cast<const float4*>(&tl.k[t][warp * 32]);
            float kk[32];
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float4 x = k4[i];
                kk[4 * i] = x.x;
                kk[4 * i + 1] = x.y;
                kk[4 * i + 2] = x.z;
                kk[4 * i + 3] = x.w;
                a0 = fmaf(x.x, S[4 * i], a0);
                a1 = fmaf(x.y, S[4 * i + 1], a1);
                a2 = fmaf(x.z, S[4 * i + 2], a2);
                a3 = fmaf(x.w, S[4 * i + 3], a3);
            }
            red[t & 1][warp][lane] = (a0 + a1) + (a2 + a3);
            __syncthreads();
            const float r = ((red[t & 1][0][lane] + red[t & 1][1][lane]) + (red[t & 1][2][lane] + red[t & 1][3][lane])) * decay;
            const float delta = (tl.v[t][lane] - r) * tl.beta[t];
            const float4* q4 = reinterpret_cast<const float4*>(&tl.q[t][warp * 32]);
            float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float4 x = q4[i];
                S[4 * i] = fmaf(kk[4 * i], delta, S[4 * i] * decay);
                S[4 * i + 1] = fmaf(kk[4 * i + 1], delta, S[4 * i + 1] * decay);
                S[4 * i + 2] = fmaf(kk[4 * i + 2], delta, S[4 * i + 2] * decay);
                S[4 * i + 3] = fmaf(kk[4 * i + 3], delta, S[4 * i + 3] * decay);
                o0 = fmaf(x.x, S[4 * i], o0);
                o1 = fmaf(x.y, S[4 * i + 1], o1);
                o2 = fmaf(x.z, S[4 * i + 2], o2);
                o3 = fmaf(x.w, S[4 * i + 3], o3);
            }
            opart[t][warp][lane] = (o0 + o1) + (o2 + o3);
        }
        __syncthreads();
        // finish the output dot products of this tile: n x 32 values, 128 threads
        for (int i = tid; i < n * kCols; i += kThreads) {
            const int t = i >> 5, c = i & 31;
            if (cb * kCols + c < p.Dv)
                obase[(ti * kTok + t) * v_ts + c] = (opart[t][0][c] + opart[t][1][c]) + (opart[t][2][c] + opart[t][3][c]);
        }
        // the next iteration's prefetch overwrites tiles[buf]; everyone is past reading it after the sync above
    }
}

}  // namespace

extern "C" int s1_delta_rule(s1_ctx* ctx, const float* q, const float* k, const float* v, const float* g,
                             const float* beta, const int32_t* cu_seqlens, int num_seqs, int total_tokens, int heads,
                             int key_dim, int value_dim, float* out) {
    if (!ctx) return S1_EINVAL;
    if (!q || !k || !v || !g || !beta || !cu_seqlens || !out) return s1_fail(ctx, S1_EINVAL, "s1_delta_rule: null pointer");
    if (key_dim != kDk) return s1_fail(ctx, S1_EINVAL, "s1_delta_rule: key_dim must be 128 (got %d)", key_dim);
    if (value_dim < 4 || value_dim % 4)
        return s1_fail(ctx, S1_EINVAL, "s1_delta_rule: value_dim must be a multiple of 4 (got %d)", value_dim);
    if (num_seqs < 0 || heads < 1 || total_tokens < 0)
        return s1_fail(ctx, S1_EINVAL, "s1_delta_rule: num_seqs=%d heads=%d total_tokens=%d", num_seqs, heads, total_tokens);
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15u)
        return s1_fail(ctx, S1_EINVAL, "s1_delta_rule: q, k, v must be 16-byte aligned");
    if (num_seqs == 0 || total_tokens == 0) return S1_OK;
    S1_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    DeltaParams p{q, k, v, g, beta, out, cu_seqlens, num_seqs, heads, value_dim};
    const long long blocks = static_cast<long long>(num_seqs) * heads * ((value_dim + kCols - 1) / kCols);
    if (blocks > 0x7fffffffLL) return s1_fail(ctx, S1_EINVAL, "s1_delta_rule: too many (sequence, head) pairs");
    s1_delta_seq_kernel<<<static_cast<unsigned>(blocks), kThreads, 0, ctx->stream>>>(p);
    S1_CUDA_OK(ctx, cudaGetLastError());
    ctx->launches += 1;
    return S1_OK;
}
