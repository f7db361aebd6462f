// Persistent, warp-specialised bf16 projection GEMM for sm_100a:
//   Y[T, N] = X[T, K] * W[N, K]^T   (f32 accumulate in TMEM, bf16 out)
// with the reference's follow-up elementwise ops folded into the epilogue
// (bias add, GeGLU / SwiGLU gating, residual add, bf16 casts in the reference's rounding order).
//
// Replaces, per call: candle `Linear::forward` (src/archs/modernbert.rs:184-191,522-532;
// src/archs/qwen35_text.rs:232-240,314-339,410,516,567-568,605-628) plus the GeGLU kernel
// (src/kernels/modernbert.cu:4-14) and the residual adds (src/archs/modernbert.rs:882-886,
// src/archs/qwen35_text.rs:938-939).
//
// Two shapes of the same kernel (template parameter CTAS):
//   CTAS = 1  one CTA per SM computes a 128 x BN tile (tcgen05.mma cta_group::1, M = 128).
//   CTAS = 2  a cluster of two CTAs (two SMs) computes a 256 x 256 (or 256 x 192) tile with cta_group::2 MMAs (M = 256):
//             each CTA stages its own 128 rows of X and its own 128-row half of the W tile, so the
//             L2 -> shared-memory traffic per SM drops by a third; the leader CTA issues the MMAs and each CTA
//             ends up with the accumulator of its own 128 rows in its own TMEM. No TMA multicast is used:
//             every CTA issues its own loads; only tcgen05.commit is multicast to the two CTAs' barriers.
//
// Roles inside a CTA (320 threads, 576 for the gated epilogues, static round-robin tile schedule, tile index n-fastest so the CTAs that
// run together share X rows and the whole (small) W through L2):
//   warp 0      : TMA producer  - 128-byte-swizzled boxes {64 x 128 rows} of X and {64 x BN/2 rows} of W into a
//                 ring of STAGES buffers guarded by full/empty mbarriers
//   warp 1      : TMEM allocation + single-thread tcgen05.mma issue (K = 16 per instruction), two TMEM
//                 accumulators so the epilogue of tile i overlaps the MMAs of tile i+1
//   warps 2..   : epilogue (8 or 16 warps) - tcgen05.ld of the warp's TMEM lane quarter, rounding/gating in registers,
//                 swizzled staging tile in shared memory, TMA store (full-line writes, clipped at the edges)
// Every wait is bounded (see mbar_wait); a wait that runs out raises a status word the host reads.
#pragma once
#include <cuda_bf16.h>

#include "ptx.cuh"

namespace s1 {

enum : int { EPI_NONE = 0, EPI_GEGLU = 1, EPI_SWIGLU = 2 };
enum : int { ACT_NONE = 0, ACT_RELU = 1, ACT_GELU = 2 };

struct GemmParams {
    int M;              // packed token rows
    int n_out;          // output columns written (N for plain, I for gated)
    int K;
    int tiles_m, tiles_n;
    int n_tile_stride;  // W rows advanced per n-tile for the first B box
    int half1_base;     // W row offset of the second B box (relative to tile_n * n_tile_stride)
    int act;            // ACT_* applied after bias (plain epilogue only)
    long long wait_limit;  // SM clock cycles any single wait may take before the kernel gives up ("wait_limit_cycles")
#ifdef S1_MEASURE
    int debug;          // timing ablations (results wrong by design): bit0 = skip output stores, bit1 = skip the epilogue
#endif
    long long ldr;      // elements between residual rows
    const __nv_bfloat16* residual;  // [M, n_out] or null
    const __nv_bfloat16* bias;      // [n_out] or null
    int* status;                    // device int[4]: {code, block, role, tile}; 0 = ok
    unsigned int* tile_counter;     // device uint[2], zero between launches: {next tile to hand out, units that are done}
    int dynamic_tiles;              // host side: launch the DYN kernel (tiles drawn at run time) where one is built
    // MODE 8 (rotary embedding in the epilogue): output columns [0, rope_cols) are heads of 64 columns whose halves are
    // rotated by the f32 table row of the token's position; columns past rope_cols are written as they are
    const float* rope_cos;          // [rope_max, 32]
    const float* rope_sin;
    const int* rope_pos;            // [M]
    int rope_max, rope_cols;
};

constexpr int kBM = 128;  // rows per CTA
constexpr int kBK = 64;   // 64 bf16 = 128 bytes = one swizzle row
constexpr int kEpiWarp0 = 2;
// Tile feed: how many tile numbers may be published and not yet read by the slowest role. The operand ring lets the
// producer run at most 6 tiles ahead of the MMA issuer (6 stages, one k-block per tile at worst), the two accumulators let
// the issuer run 2 ahead of the epilogue, and numbers are published 2 iterations ahead: 10 in all.
constexpr int kFeedSlots = 16;

// Epilogue warps: 8 for the plain epilogues; 16 for the gated ones, whose erf / exp evaluation is latency-bound and
// needs the extra warps to keep the issue slots busy.
template <int BN, int EPI>
struct EpiWarps {
    static constexpr int value = (EPI != EPI_NONE && BN == 256) ? 16 : 8;
};
template <int BN, int EPI>
constexpr int gemm_threads() { return 64 + 32 * EpiWarps<BN, EPI>::value; }

// Width of one TMA store of the epilogue: 64 columns (128-byte rows, two staging tiles of 4 KB per warp) for the
// plain 256-wide pair tile, whose output volume is the largest; 32 columns (64-byte rows) elsewhere.
template <int BN, int EPI, int CTAS>
struct StoreCfg {
    static constexpr bool kWide = (EPI == EPI_NONE && BN == 256 && CTAS == 2);
    static constexpr int kCols = kWide ? 64 : 32;
    static constexpr int kTileBytes = 32 * kCols * 2;
    static constexpr int kStagingBytes = kWide ? 64 * 1024 : 32 * 1024;  // all epilogue warps together
};

template <int BN, int CTAS>
struct GemmCfg {
    static_assert(CTAS == 1 || (CTAS == 2 && (BN == 256 || BN == 192)), "the CTA-pair kernel is 256 x 256 or 256 x 192");
    static constexpr int kABytes = kBM * kBK * 2;
    static constexpr int kBHalfBytes = (BN / 2) * kBK * 2;
    // one CTA stages both halves of the W tile; in a pair each CTA stages one
    static constexpr int kStageBytes = kABytes + (CTAS == 1 ? 2 : 1) * kBHalfBytes;
    static constexpr int kTmemCols = (2 * BN <= 256) ? 256 : 512;  // two accumulators, rounded up to a power of two
    // 224 KB of operand ring + epilogue staging: 6 (or 4) stages beside 32 KB of staging, 5 beside 64 KB
    static constexpr int stages(int staging_bytes) { return (224 * 1024 - staging_bytes) / kStageBytes; }
    static constexpr int smem_bytes(int staging_bytes) {
        return stages(staging_bytes) * kStageBytes + staging_bytes + 1024 /*align slack*/ + 512 /*barriers, tile feed*/;
    }
};

// Special-function unit forms (relative error about 2^-22, far below the bf16 rounding that follows).
__device__ __forceinline__ float rcp_approx(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float ex2_approx(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

// Exact-erf GELU x * Phi(x) (src/kernels/modernbert.cu:11-12 writes it as value * normcdff(value)),
// with Phi through erfc(|z|) = t exp(-z^2 + P(t)), t = 1 / (1 + |z| / 2), the Chebyshev fit of
// Numerical Recipes (erfcc): FRACTIONAL error below 1.2e-7 everywhere, so the tail (negative inputs) keeps full
// relative accuracy; evaluated on the tail side, nothing cancels. Two special-function ops and eleven FMAs.
__device__ __forceinline__ float gelu_erf_ref(float v) {
    const float z = fabsf(v) * 0.70710678118654752f;
    const float t = rcp_approx(fmaf(0.5f, z, 1.f));
    float u = fmaf(t, 0.17087277f, -0.82215223f);
    u = fmaf(t, u, 1.48851587f);
    u = fmaf(t, u, -1.13520398f);
    u = fmaf(t, u, 0.27886807f);
    u = fmaf(t, u, -0.18628806f);
    u = fmaf(t, u, 0.09678418f);
    u = fmaf(t, u, 0.37409196f);
    u = fmaf(t, u, 1.00002368f);
    u = fmaf(t, u, -1.26551223f);
    u = fmaf(-z, z, u);
    const float half_erfc = 0.5f * t * ex2_approx(1.4426950408889634f * u);  // Phi(-|v|)
    return v * (v >= 0.f ? 1.f - half_erfc : half_erfc);
}
// Packed pairs of f32 on the FMA pipe (one instruction for two lanes of work).
__device__ __forceinline__ void ffma2(float& d0, float& d1, float a0, float a1, float b0, float b1, float c0, float c1) {
    asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
        "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1), "f"(c0), "f"(c1));
}
__device__ __forceinline__ void fmul2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
    asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
        "mul.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
// gelu_erf_ref for two values at once: the same erfc fit, its polynomial and products as packed instructions, the
// factor log2(e) folded into the coefficients so that the exponent is one fma away from ex2.
__device__ __forceinline__ void gelu_erf_pair(float v0, float v1, float& g0, float& g1) {
    constexpr float L2E = 1.4426950408889634f;
    const float z0 = fabsf(v0) * 0.70710678118654752f, z1 = fabsf(v1) * 0.70710678118654752f;
    const float s0 = fabsf(v0) * (-0.70710678118654752f * L2E), s1 = fabsf(v1) * (-0.70710678118654752f * L2E);
    float d0, d1;
    ffma2(d0, d1, z0, z1, 0.5f, 0.5f, 1.f, 1.f);
    const float t0 = rcp_approx(d0), t1 = rcp_approx(d1);
    float u0, u1;
    ffma2(u0, u1, t0, t1, 0.17087277f * L2E, 0.17087277f * L2E, -0.82215223f * L2E, -0.82215223f * L2E);
    ffma2(u0, u1, t0, t1, u0, u1, 1.48851587f * L2E, 1.48851587f * L2E);
    ffma2(u0, u1, t0, t1, u0, u1, -1.13520398f * L2E, -1.13520398f * L2E);
    ffma2(u0, u1, t0, t1, u0, u1, 0.27886807f * L2E, 0.27886807f * L2E);
    ffma2(u0, u1, t0, t1, u0, u1, -0.18628806f * L2E, -0.18628806f * L2E);
    ffma2(u0, u1, t0, t1, u0, u1, 0.09678418f * L2E, 0.09678418f * L2E);
    ffma2(u0, u1, t0, t1, u0, u1, 0.37409196f * L2E, 0.37409196f * L2E);
    ffma2(u0, u1, t0, t1, u0, u1, 1.00002368f * L2E, 1.00002368f * L2E);
    ffma2(u0, u1, t0, t1, u0, u1, -1.26551223f * L2E, -1.26551223f * L2E);
    ffma2(u0, u1, s0, s1, z0, z1, u0, u1);  // log2(e) * (poly - z^2)
    const float e0 = ex2_approx(u0), e1 = ex2_approx(u1);
    float h0, h1, w0, w1;
    fmul2(h0, h1, t0, t1, e0, e1);                      // 2 Phi(-|v|)
    fmul2(w0, w1, h0, h1, 0.5f * v0, 0.5f * v1);        // v Phi(-|v|)
    g0 = v0 >= 0.f ? v0 - w0 : w0;
    g1 = v1 >= 0.f ? v1 - w1 : w1;
}
__device__ __forceinline__ float silu_ref(float v) { return v * rcp_approx(1.f + ex2_approx(-1.4426950408889634f * v)); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&t);
}
__device__ __forceinline__ void unpack_bf16x2(uint32_t v, float& lo, float& hi) {
    __nv_bfloat162 t = *reinterpret_cast<__nv_bfloat162*>(&v);
    lo = __low2float(t);
    hi = __high2float(t);
}

// Residual values of one epilogue warp's part of a tile (32 rows x CH*32 columns, one row per lane), fetched
// before the warp waits for the accumulator so that the memory latency hides behind the MMAs.
template <int CH>
__device__ __forceinline__ void fetch_residual(const GemmParams& p, int row0, int col0, int lane, uint4 (&res)[CH * 4]) {
    const int row = row0 + lane;
    const __nv_bfloat16* rrow = p.residual + static_cast<long long>(row) * p.ldr;
#pragma unroll
    for (int j = 0; j < CH * 4; ++j) {
        res[j] = make_uint4(0u, 0u, 0u, 0u);
        if (row < p.M && col0 + j * 8 < p.n_out) res[j] = __ldg(reinterpret_cast<const uint4*>(rrow + col0 + j * 8));
    }
}

// One epilogue warp, one tile: reads its 32 rows x (CH*32) accumulator columns out of TMEM, applies the epilogue
// and stores. `tempty_bar` is the (cluster-space) address of the barrier that hands the accumulator back.
// MODE (plain epilogue only): bit0 = residual add, bit1 = bias and/or activation present (general path);
// 4 = the output buffer already holds the residual: the tile is added to it by a TMA reduction.
template <int BN, int EPI, int MODE, int EW, int SW, int NBUF>
__device__ __forceinline__ void epilogue_tile(const GemmParams& p, const CUtensorMap* tmY, uint32_t taddr, int row0,
                                              int col0, uint32_t stage_buf, uint32_t& nstore, uint32_t tempty_bar,
                                              int lane, const uint4* res) {
    constexpr bool PAIRED = (EPI != EPI_NONE);
    constexpr int OUT_W = PAIRED ? BN / 2 : BN;
    constexpr int CH = OUT_W / (EW * 8);  // 32-column work units per warp per tile
    constexpr int UNIT = SW / 32;             // 32-column chunks per TMA store
    constexpr uint32_t TILE_BYTES = 32u * SW * 2u;
    static_assert(CH % UNIT == 0, "store width must divide the warp's columns");
    static_assert(CH >= 1, "tile too narrow for this many epilogue warps");
    uint32_t va[2][32];
    uint32_t vg[PAIRED ? 2 : 1][PAIRED ? 32 : 1];
    // staging + TMA store of one 32-column chunk of the warp's rows
    auto emit = [&](int cix, const uint32_t (&o)[16]) {
        const int ucol = col0 + (cix / UNIT) * SW;  // first column of the store this chunk belongs to
#ifdef S1_MEASURE
        if (p.debug & 1) return;
#endif
        if (row0 < p.M && ucol < p.n_out) {
            const uint32_t buf = stage_buf + (nstore % NBUF) * TILE_BYTES;
            if (cix % UNIT == 0) {
                // the staging tile about to be overwritten must have been read out by its TMA store
                if (lane == 0) tma_store_wait_read<NBUF - 1>();
                __syncwarp();
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t addr;
                if constexpr (SW == 64) {
                    // 128-byte rows, 128B swizzle: 16-byte chunk c of row r sits at chunk c ^ (r & 7)
                    addr = buf + lane * 128 + ((((cix % UNIT) * 4 + j) ^ (lane & 7)) << 4);
                } else {
                    // 64-byte rows, 64B swizzle: 16-byte chunk j of row r sits at chunk j ^ ((r >> 1) & 3)
                    addr = buf + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4);
                }
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(o[4 * j]), "r"(o[4 * j + 1]),
                             "r"(o[4 * j + 2]), "r"(o[4 * j + 3])
                             : "memory");
            }
            if (cix % UNIT == UNIT - 1) {
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    if constexpr (MODE == 4) tma_reduce_add_2d(tmY, buf, ucol, row0);  // y already holds the residual
                    else tma_store_2d(tmY, buf, ucol, row0);
                    tma_store_commit();
                }
                ++nstore;
            }
        }
    };
    // MODE 8: cos / sin of this lane's token (its row), fetched once per tile and used by every head of the tile
    float cs[MODE == 8 ? 32 : 1], sn[MODE == 8 ? 32 : 1], lo[MODE == 8 ? 32 : 1];
    bool rotate = false;
    if constexpr (MODE == 8) {
        static_assert(MODE != 8 || (UNIT == 2 && CH % 2 == 0), "a head's two chunks must form one store");
        rotate = col0 < p.rope_cols;  // the same for the whole warp
        if (rotate) {
            const int row = row0 + lane;
            int pos = row < p.M ? p.rope_pos[row] : 0;
            if (pos < 0 || pos >= p.rope_max) {
                if (atomicCAS(p.status, 0, 102) == 0) {
                    p.status[1] = static_cast<int>(blockIdx.x);
                    p.status[2] = row;
                    p.status[3] = pos;
                }
                pos = -1;
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                float4 c4 = make_float4(1.f, 1.f, 1.f, 1.f), s4 = make_float4(0.f, 0.f, 0.f, 0.f);  // a bad position leaves the token unrotated
                if (pos >= 0) {
                    c4 = __ldg(reinterpret_cast<const float4*>(p.rope_cos + static_cast<long long>(pos) * 32) + e);
                    s4 = __ldg(reinterpret_cast<const float4*>(p.rope_sin + static_cast<long long>(pos) * 32) + e);
                }
                cs[4 * e] = c4.x, cs[4 * e + 1] = c4.y, cs[4 * e + 2] = c4.z, cs[4 * e + 3] = c4.w;
                sn[4 * e] = s4.x, sn[4 * e + 1] = s4.y, sn[4 * e + 2] = s4.z, sn[4 * e + 3] = s4.w;
            }
        }
    }
    tmem_ld_32x32b_x32(taddr, va[0]);
    if constexpr (PAIRED) tmem_ld_32x32b_x32(taddr + BN / 2, vg[0]);
#pragma unroll
    for (int ci = 0; ci < CH; ++ci) {
        const int col = col0 + ci * 32;
        const uint4* rv = &res[(MODE & 1) ? ci * 4 : 0];
        tmem_ld_wait();
        if (ci + 1 < CH) {
            tmem_ld_32x32b_x32(taddr + (ci + 1) * 32, va[(ci + 1) & 1]);
            if constexpr (PAIRED) tmem_ld_32x32b_x32(taddr + BN / 2 + (ci + 1) * 32, vg[(ci + 1) & 1]);
        } else {
            // every TMEM read of this accumulator has landed in registers: hand it back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(tempty_bar);
        }
        uint32_t out[16];
        if constexpr (MODE == 8) {
            // handled below, a head (two chunks) at a time
        } else if constexpr (!PAIRED) {
            const uint32_t* v = va[ci & 1];
            if constexpr ((MODE & 2) == 0) {
                // y = bf16(acc) [+ residual, added in bf16 with one rounding like the reference's bf16 add]
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    __nv_bfloat162 t = __floats2bfloat162_rn(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
                    if constexpr (MODE & 1) {
                        const uint32_t rw = reinterpret_cast<const uint32_t*>(rv)[j];
                        t = __hadd2(t, *reinterpret_cast<const __nv_bfloat162*>(&rw));
                    }
                    out[j] = *reinterpret_cast<uint32_t*>(&t);
                }
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    float a = bf16_round(__uint_as_float(v[2 * j]));
                    float b = bf16_round(__uint_as_float(v[2 * j + 1]));
                    if (p.bias) {
                        const int cc = col + 2 * j;
                        if (cc < p.n_out) {
                            a = bf16_round(a + __bfloat162float(p.bias[cc]));
                            b = bf16_round(b + __bfloat162float(p.bias[cc + 1]));
                        }
                    }
                    if (p.act == ACT_RELU) {
                        a = fmaxf(a, 0.f);
                        b = fmaxf(b, 0.f);
                    } else if (p.act == ACT_GELU) {
                        a = bf16_round(gelu_erf_ref(a));
                        b = bf16_round(gelu_erf_ref(b));
                    }
                    if constexpr (MODE & 1) {
                        float r0, r1;
                        unpack_bf16x2(reinterpret_cast<const uint32_t*>(rv)[j], r0, r1);
                        a += r0;
                        b += r1;
                    }
                    out[j] = pack_bf16x2(a, b);
                }
            }
        } else {
            const uint32_t* v = va[ci & 1];
            const uint32_t* w = vg[ci & 1];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                // round both projections to bf16 (the reference materialises them), activate in f32, round,
                // multiply in bf16 (one rounding)
                __nv_bfloat162 a2 = __floats2bfloat162_rn(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
                __nv_bfloat162 g2 = __floats2bfloat162_rn(__uint_as_float(w[2 * j]), __uint_as_float(w[2 * j + 1]));
                const float a0 = __low2float(a2), a1 = __high2float(a2);
                __nv_bfloat162 act2;
#ifdef S1_MEASURE
                if (p.debug & 8) act2 = a2;
                else
#endif
                if constexpr (EPI == EPI_GEGLU) {
                    float g0, g1;
                    gelu_erf_pair(a0, a1, g0, g1);
                    act2 = __floats2bfloat162_rn(g0, g1);
                }
                else act2 = __floats2bfloat162_rn(silu_ref(a0), silu_ref(a1));
                __nv_bfloat162 o2 = __hmul2(act2, g2);
                out[j] = *reinterpret_cast<uint32_t*>(&o2);
            }
        }
        if constexpr (MODE == 8) {
            // the two chunks of a head leave together: at the odd chunk, the even one (kept in `lo`) is rotated with it
            if ((ci & 1) == 0) {
#pragma unroll
                for (int e = 0; e < 32; ++e) lo[e] = bf16_round(__uint_as_float(va[0][e]));
            } else {
                uint32_t out_lo[16];
                const uint32_t* v = va[1];
                if (rotate) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float h0 = bf16_round(__uint_as_float(v[2 * j])), h1 = bf16_round(__uint_as_float(v[2 * j + 1]));
                        const float l0 = lo[2 * j], l1 = lo[2 * j + 1];
                        // products rounded one by one (no fused multiply-add), as the unfused kernel and the reference do
                        out_lo[j] = pack_bf16x2(__fsub_rn(__fmul_rn(l0, cs[2 * j]), __fmul_rn(h0, sn[2 * j])),
                                                __fsub_rn(__fmul_rn(l1, cs[2 * j + 1]), __fmul_rn(h1, sn[2 * j + 1])));
                        out[j] = pack_bf16x2(__fadd_rn(__fmul_rn(l0, sn[2 * j]), __fmul_rn(h0, cs[2 * j])),
                                             __fadd_rn(__fmul_rn(l1, sn[2 * j + 1]), __fmul_rn(h1, cs[2 * j + 1])));
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        out_lo[j] = pack_bf16x2(lo[2 * j], lo[2 * j + 1]);
                        out[j] = pack_bf16x2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
                    }
                }
                emit(ci - 1, out_lo);
                emit(ci, out);
            }
        } else {
            emit(ci, out);
        }
    }
}

// DYN: the tiles past a unit's first are drawn at run time (see "tile feed" below); compiled as a kernel of its own so that
// the default kernels carry none of that code (their launches of a few tiles are sensitive to every instruction fetched).
template <int BN, int EPI, int MODE, int CTAS, bool DYN = false>
__global__ void __launch_bounds__(gemm_threads<BN, EPI>(), 1)
s1_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB0,
               const __grid_constant__ CUtensorMap tmB1, const __grid_constant__ CUtensorMap tmY,
               const GemmParams p) {
    using Cfg = GemmCfg<BN, CTAS>;
    using Store = StoreCfg<BN, EPI, CTAS>;
    constexpr int STAGES = Cfg::stages(Store::kStagingBytes);
    constexpr bool PAIRED = (EPI != EPI_NONE);
    constexpr int OUT_W = PAIRED ? BN / 2 : BN;  // output columns per tile
    constexpr int EW = EpiWarps<BN, EPI>::value;
    constexpr int CH = OUT_W / (EW * 8);  // 32-column work units per epilogue warp per tile

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_al + STAGES * Cfg::kStageBytes + Store::kStagingBytes);
    // bars[0..S) full, [S..2S) empty, [2S..2S+2) tmem_full, [2S+2..2S+4) tmem_empty
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    // tile feed: kFeedSlots barriers at +192 and kFeedSlots tile numbers behind them (see "tile feed" below)
    const uint32_t feed_bar0 = smem_u32(bars) + 192u;
    const uint32_t feed_tile0 = feed_bar0 + 8u * kFeedSlots;
    static_assert((2 * STAGES + 4) * 8 + 8 <= 192 && 192 + 12 * kFeedSlots <= 512, "barrier block layout");

    const uint32_t full0 = smem_u32(bars);
    const uint32_t empty0 = full0 + 8u * STAGES;
    const uint32_t tfull0 = full0 + 8u * (2 * STAGES);
    const uint32_t tempty0 = full0 + 8u * (2 * STAGES + 2);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t cta_rank = (CTAS == 2) ? cluster_ctarank() : 0u;  // 0 = leader (issues the MMAs)
    const int unit = (CTAS == 2) ? (blockIdx.x >> 1) : blockIdx.x;   // scheduling unit: CTA or CTA pair
    const int num_units = (CTAS == 2) ? (gridDim.x >> 1) : gridDim.x;
    const int num_tiles = p.tiles_m * p.tiles_n;
    const int num_kb = (p.K + kBK - 1) / kBK;
    // barriers of the leader CTA as seen from this CTA (cluster address space)
    const uint32_t lead_full0 = (CTAS == 2) ? map_to_cta(full0, 0) : full0;
    const uint32_t lead_tempty0 = (CTAS == 2) ? map_to_cta(tempty0, 0) : tempty0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8u * s, 1);
            mbar_init(empty0 + 8u * s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull0 + 8u * a, 1);
            mbar_init(tempty0 + 8u * a, EW * CTAS);
        }
        if constexpr (DYN)
            for (int f = 0; f < kFeedSlots; ++f) mbar_init(feed_bar0 + 8u * f, 1);
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB0);
        tma_prefetch_desc(&tmB1);
        tma_prefetch_desc(&tmY);
    }
    if (warp == 1) {
        if constexpr (CTAS == 2) {
            tmem_alloc_2cta(smem_u32(tmem_slot), Cfg::kTmemCols);
            tmem_relinquish_2cta();
        } else {
            tmem_alloc(smem_u32(tmem_slot), Cfg::kTmemCols);
            tmem_relinquish();
        }
    }
    tc_fence_before();
    __syncthreads();
    if constexpr (CTAS == 2) cluster_sync_all();  // the peer's barriers exist before anything remote touches them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // set-up done (barriers, TMEM, descriptor prefetch): it may have overlapped the tail of the previous kernel in the
    // stream; from here on this kernel touches memory that kernel may still be writing
    griddep_launch_dependents();
    griddep_wait();

    int fail_role = 0, fail_tile = -1;

    // ---- tile feed. Lane 0 of the leader's producer warp decides which tile each iteration works on and publishes it to
    // every role of the CTA (pair) through a small ring in shared memory: slot `(it - 1) % kFeedSlots` holds the tile of
    // iteration `it` >= 1 (-1: no more), its barrier's phase says it is there; iteration 0 is always tile `unit`.
    // In the default kernels (DYN = false) the sequence is the unit's fixed share (`unit + it * num_units`), which every role works out by itself:
    // nothing is published. In the DYN kernels (option `dynamic_tiles`; built for the 256 x 256 pair tiles) the tiles past the first are drawn from a counter in global memory (a draw n
    // stands for tile `num_units + n`): a CTA that reaches its SM late - blocks of a collective running beside the
    // projection were in the way - then finds little left to do, where a fixed share would make the whole launch wait
    // for it. Draws are issued a tile ahead of their use; the burst of draws at the start of a launch and the hand-over to
    // the peer CTA still cost 1 to 5 microseconds per launch, which is why it is an option.
    const int first_tile = (unit < num_tiles) ? unit : -1;
    bool drained = false;  // (drawer only) the counter has run past the last tile
    unsigned fixed_draws = 0;
    auto feed_draw_raw = [&]() -> unsigned {
        // fixed shares (tile `unit + k * num_units` for the k-th draw): the same feed, no traffic on the counter
        if constexpr (!DYN) return (fixed_draws++) * static_cast<unsigned>(num_units) + static_cast<unsigned>(unit);
        return atomicAdd(p.tile_counter, 1u);
    };
    // The drawer that learns there is nothing left says so once; the last of all units to say so puts both counters back
    // to zero for the next launch on this stream (which draws only after this grid has completed: stream order, or
    // griddepcontrol.wait). No unit draws again after it has said so.
    auto feed_drained = [&]() {
        if (drained) return;
        drained = true;
        if constexpr (!DYN) return;
        if (atomicAdd(p.tile_counter + 1, 1u) == static_cast<unsigned>(num_units) - 1u) {
            p.tile_counter[0] = 0u;
            p.tile_counter[1] = 0u;
        }
    };
    auto feed_resolve = [&](unsigned raw) -> int {
        const unsigned t = raw + static_cast<unsigned>(num_units);
        if (t < static_cast<unsigned>(num_tiles)) return static_cast<int>(t);
        feed_drained();
        return -1;
    };
    auto feed_publish = [&](uint32_t it, int tile) {
        if constexpr (!DYN) return;  // every role works the fixed sequence out by itself
        const uint32_t slot = (it - 1u) % kFeedSlots;
        st_shared_u32(feed_tile0 + 4u * slot, static_cast<uint32_t>(tile));
        mbar_arrive(feed_bar0 + 8u * slot);
        if constexpr (CTAS == 2) {
            st_cluster_u32(map_to_cta(feed_tile0 + 4u * slot, 1), static_cast<uint32_t>(tile));
            mbar_arrive_cluster(map_to_cta(feed_bar0 + 8u * slot, 1));
        }
    };
    // false: the wait ran out (or the CTA is unwinding); otherwise `tile` is the tile of iteration `it`, -1 at the end
    auto feed_take = [&](uint32_t it, int& tile) -> bool {
        if (it == 0) {
            tile = first_tile;
            return true;
        }
        if constexpr (!DYN) {
            const long long t = static_cast<long long>(it) * num_units + unit;
            tile = (first_tile >= 0 && t < num_tiles) ? static_cast<int>(t) : -1;
            return true;
        }
        const uint32_t slot = (it - 1u) % kFeedSlots;
        // the leader's roles read what a thread of their own CTA wrote; the peer's need the cluster-wide acquire
        const bool there = (CTAS == 2 && cta_rank != 0)
                               ? mbar_wait_cluster(feed_bar0 + 8u * slot, ((it - 1u) / kFeedSlots) & 1u, abort_flag, p.wait_limit)
                               : mbar_wait(feed_bar0 + 8u * slot, ((it - 1u) / kFeedSlots) & 1u, abort_flag, p.wait_limit);
        if (!there) return false;
        tile = static_cast<int>(ld_shared_u32(feed_tile0 + 4u * slot));
        return true;
    };

    // One look, no waiting: a role asks for the next iteration's tile before it starts on the current one (it is normally
    // there already, published two iterations ahead) and falls back to feed_take afterwards, so that the look-up costs
    // nothing between two tiles. (Waiting here would deadlock the first tile: its successor is published only once the
    // producer has issued all of its loads, which needs the MMA issuer to consume them.)
    auto feed_try = [&](uint32_t it, int& tile) -> bool {
        if constexpr (!DYN) return feed_take(it, tile);
        const uint32_t slot = (it - 1u) % kFeedSlots;
        const bool there = (CTAS == 2 && cta_rank != 0) ? mbar_try_wait_cluster(feed_bar0 + 8u * slot, ((it - 1u) / kFeedSlots) & 1u)
                                                        : mbar_try_wait(feed_bar0 + 8u * slot, ((it - 1u) / kFeedSlots) & 1u);
        if (!there) return false;
        tile = static_cast<int>(ld_shared_u32(feed_tile0 + 4u * slot));
        return true;
    };

    if (warp == 0) {
        // ------------------------------------------------------------- TMA producer (both CTAs of a pair)
        if (lane == 0) {
            uint32_t cnt = 0, it = 0;
            const bool draws = (cta_rank == 0);   // the peer's producer reads what the leader's publishes
            int tile = first_tile;
            int next = -2;                        // -2: the first two draws are still in flight
            unsigned raw1 = 0, raw2 = 0;
            if (draws) {
                if (tile >= 0 && num_tiles > num_units) raw1 = feed_draw_raw(), raw2 = feed_draw_raw();
                else if (tile >= 0) next = -3;    // one tile per unit at most: nothing to draw
                else feed_drained();
            }
            while (tile >= 0 && !fail_role) {
                // the draw for the iteration after next is in flight while this tile's loads are issued
                unsigned raw_new = 0;
                const bool drew = draws && next >= 0;
                if (drew) raw_new = feed_draw_raw();
                int ahead = -1;
                const bool looked = !draws && feed_try(it + 1, ahead);
                const int tm = tile / p.tiles_n, tn = tile % p.tiles_n;
                const int m0 = (tm * CTAS + static_cast<int>(cta_rank)) * kBM;
                const int r0 = tn * p.n_tile_stride;
                const int r1 = r0 + p.half1_base;
                for (int kb = 0; kb < num_kb; ++kb, ++cnt) {
                    const uint32_t s = cnt % STAGES, ph = (cnt / STAGES) & 1u;
                    if (!mbar_wait(empty0 + 8u * s, ph ^ 1u, abort_flag, p.wait_limit)) {
                        fail_role = 1;
                        fail_tile = tile;
                        break;
                    }
                    const uint32_t sa = smem_base + s * Cfg::kStageBytes;
                    if constexpr (CTAS == 1) {
                        const uint32_t fb = full0 + 8u * s;
                        mbar_arrive_expect_tx(fb, Cfg::kStageBytes);
                        tma_load_2d(sa, &tmA, kb * kBK, m0, fb);
                        tma_load_2d(sa + Cfg::kABytes, &tmB0, kb * kBK, r0, fb);
                        tma_load_2d(sa + Cfg::kABytes + Cfg::kBHalfBytes, &tmB1, kb * kBK, r1, fb);
                    } else {
                        // both CTAs' bytes are counted on the leader's barrier; only the leader arrives on it
                        const uint32_t fb = lead_full0 + 8u * s;
                        if (cta_rank == 0) mbar_arrive_expect_tx(full0 + 8u * s, 2 * Cfg::kStageBytes);
                        tma_load_2d_pair(sa, &tmA, kb * kBK, m0, fb);
                        if (cta_rank == 0) tma_load_2d_pair(sa + Cfg::kABytes, &tmB0, kb * kBK, r0, fb);
                        else tma_load_2d_pair(sa + Cfg::kABytes, &tmB1, kb * kBK, r1, fb);
                    }
                }
                if (fail_role) break;
                ++it;
                if (draws) {
                    if (next == -3) {            // single-tile launch
                        feed_drained();
                        feed_publish(1, -1);
                        tile = -1;
                    } else if (next == -2) {     // end of the first tile: both early draws are back by now
                        const int n1 = feed_resolve(raw1);
                        feed_publish(1, n1);
                        const int n2 = (n1 >= 0) ? feed_resolve(raw2) : -1;
                        if (n1 >= 0) feed_publish(2, n2);
                        tile = n1;
                        next = n2;
                    } else {
                        const int n2 = drew ? feed_resolve(raw_new) : -1;
                        if (next >= 0) feed_publish(it + 1, n2);
                        tile = next;
                        next = n2;
                    }
                } else if (looked) {
                    tile = ahead;
                } else if (!feed_take(it, tile)) {
                    fail_role = 5;
                    fail_tile = static_cast<int>(it);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------- MMA issuer (leader CTA only)
        if (lane == 0 && cta_rank == 0) {
            constexpr uint32_t idesc = make_idesc(1, kBM * CTAS, BN);
            uint32_t cnt = 0;
            int tile = first_tile;
            for (uint32_t it = 0; tile >= 0 && !fail_role; ++it) {
                int ahead = -1;
                const bool looked = feed_try(it + 1, ahead);
                const uint32_t acc = it & 1u, aph = (it >> 1) & 1u;
                if (!mbar_wait(tempty0 + 8u * acc, aph ^ 1u, abort_flag, p.wait_limit)) {
                    fail_role = 2;
                    fail_tile = tile;
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < num_kb; ++kb, ++cnt) {
                    const uint32_t s = cnt % STAGES, ph = (cnt / STAGES) & 1u;
                    if (!mbar_wait(full0 + 8u * s, ph, abort_flag, p.wait_limit)) {
                        fail_role = 3;
                        fail_tile = tile;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sa = smem_base + s * Cfg::kStageBytes;
                    const uint64_t da = make_sw128_kmajor_desc(sa);
                    const uint64_t db = make_sw128_kmajor_desc(sa + Cfg::kABytes);
#pragma unroll
                    for (int k = 0; k < kBK / 16; ++k) {
                        // +32 bytes along K per instruction = +2 in the (addr >> 4) field
                        if constexpr (CTAS == 2) umma_bf16_2cta(d_tmem, da + 2u * k, db + 2u * k, idesc, (kb | k) ? 1u : 0u);
                        else umma_bf16(d_tmem, da + 2u * k, db + 2u * k, idesc, (kb | k) ? 1u : 0u);
                    }
                    // shared-memory stage reusable (in both CTAs of a pair) once these MMAs retire
                    if constexpr (CTAS == 2) umma_commit_2cta(empty0 + 8u * s);
                    else umma_commit(empty0 + 8u * s);
                }
                if (fail_role) break;
                // accumulator complete (each CTA of a pair is told on its own barrier)
                if constexpr (CTAS == 2) umma_commit_2cta(tfull0 + 8u * acc);
                else umma_commit(tfull0 + 8u * acc);
                if (looked) {
                    tile = ahead;
                } else if (!feed_take(it + 1, tile)) {
                    fail_role = 6;
                    fail_tile = static_cast<int>(it + 1);
                }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------- epilogue warps
        // Warp (q, hh): TMEM lane quarter q = warp % 4 (rows q*32 .. q*32+31 of this CTA's 128, one row per lane),
        // column half hh.
        const int q = warp & 3;
        const int hh = (warp - kEpiWarp0) >> 2;
        constexpr int NBUF = Store::kStagingBytes / (EW * Store::kTileBytes);  // staging tiles per warp
        const uint32_t stage_buf = smem_base + STAGES * Cfg::kStageBytes + (warp - kEpiWarp0) * (Store::kStagingBytes / EW);
        uint32_t nstore = 0;
        int tile = first_tile;
        for (uint32_t it = 0; tile >= 0; ++it) {
            // one lane looks whether the next iteration's tile is already known; the warp shares the answer
            int ahead = -1, looked = 0;
            if (lane == 0) looked = feed_try(it + 1, ahead) ? 1 : 0;
            looked = __shfl_sync(0xffffffffu, looked, 0);
            ahead = __shfl_sync(0xffffffffu, ahead, 0);
            const int tm = tile / p.tiles_n, tn = tile % p.tiles_n;
            const uint32_t acc = it & 1u, aph = (it >> 1) & 1u;
            const int row0 = (tm * CTAS + static_cast<int>(cta_rank)) * kBM + q * 32;
            const int col0 = tn * OUT_W + hh * (CH * 32);
            uint4 res[(MODE & 1) ? CH * 4 : 1];
            if constexpr (!PAIRED && (MODE & 1)) fetch_residual<CH>(p, row0, col0, lane, res);
            // the whole warp must agree before any .sync.aligned tcgen05 instruction
            const bool ready = mbar_wait(tfull0 + 8u * acc, aph, abort_flag, p.wait_limit);
            if (!__all_sync(0xffffffffu, ready)) {
                fail_role = 4;
                fail_tile = tile;
                break;
            }
            tc_fence_after();
            const uint32_t tempty_bar = lead_tempty0 + 8u * acc;
            bool skip = false;
#ifdef S1_MEASURE
            if (p.debug & 2) {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(tempty_bar);
                skip = true;
            }
#endif
            if (!skip) {
                const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16) + hh * (CH * 32);
                epilogue_tile<BN, EPI, MODE, EW, Store::kCols, NBUF>(p, &tmY, taddr, row0, col0, stage_buf, nstore, tempty_bar, lane, res);
            }
            if (!looked) {
                const bool fed = feed_take(it + 1, ahead);
                if (!__all_sync(0xffffffffu, fed)) {
                    fail_role = 7;
                    fail_tile = static_cast<int>(it + 1);
                    break;
                }
            }
            tile = ahead;
        }
        if (lane == 0) tma_store_wait<0>();  // smem reads and global writes of this warp's stores are complete
        __syncwarp();
    }

    if (fail_role) {
        // first failing thread of the grid records where it gave up; the host turns it into an error
        if (atomicCAS(p.status, 0, 1) == 0) {
            p.status[1] = blockIdx.x;
            p.status[2] = fail_role;
            p.status[3] = fail_tile;
        }
    }
    if (*abort_flag) {
        // give copies that are still in flight time to land before shared memory is released
        __nanosleep(200000);
    }
    tc_fence_before();
    __syncthreads();
    // a pair leaves together: the leader's MMAs read the peer's shared memory, the peer arrives on the leader's barriers
    if constexpr (CTAS == 2) cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        if constexpr (CTAS == 2) tmem_dealloc_2cta(tmem_base, Cfg::kTmemCols);
        else tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

}  // namespace s1
