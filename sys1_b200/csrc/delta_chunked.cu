// Chunked gated delta rule on the 5th-generation tensor cores (tcgen05 / TMEM / TMA), chunk = 64 tokens,
// key dim = value dim = 128, bf16 operands with f32 accumulation, f32 state.
//
// Same function as `chunked_delta_rule` (src/archs/qwen35_text.rs:789-880), in the chunk form of its CPU
// fallback (:809-880) with 64-token chunks instead of 32 and the triangular inverse by forward substitution
// instead of Neumann doubling:
//     G = cumsum(g) inside the chunk,  A_ij = beta_i (k_i . k_j) e^{G_i - G_j}  (j < i),  Tm = (I + A)^-1
//     W = Tm (beta e^G K),  U = Tm (beta V),  P_ij = (q_i . k_j) e^{G_i - G_j}  (j <= i)
//     V' = U - W S,   O = (Q e^G) S + P V',   S <- e^{G_last} S + (K e^{G_last - G})^T V'
//
// Two kernels:
//  * s1_delta_prep_kernel  - everything that does not involve the state S, for all chunks in parallel
//    (one CTA per pair of chunks of one head: the two chunks are stacked into M = 128 MMAs; K K^T, Q K^T and
//    Tm [beta e^G K | beta V] run on tcgen05, the 64 x 64 triangular solves in f32 on the CUDA cores). It writes
//    W, Q e^G, U^T, K e^{G_last - G} and P as bf16 into a workspace, already in the operand layouts the second
//    kernel feeds to the tensor cores.
//  * s1_delta_scan_kernel  - one CTA per (sequence, head) walks the chunks in order. The state lives in f32
//    registers (thread = value row, 128 key columns); per chunk it issues three MMAs in transposed form so that
//    M = Dv = 128:  (W S)^T = S^T W^T,  O^T = S^T (Q e^G)^T + V'^T P^T,  dS^T = V'^T K~ ; operands arrive by TMA
//    (two-stage ring), V'^T and the bf16 copy of S^T are rewritten in shared memory by the warps between MMAs.
// Every mbarrier wait is bounded; a wait that runs out raises the context's status word.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>

#include "context.h"
#include "ptx.cuh"

using namespace s1;

namespace {

constexpr int kC = 64;     // chunk length (tokens)
constexpr int kD = 128;    // key dim = value dim
constexpr int kTileBytes = 128 * 64 * 2;  // one operand tile: 128 rows x 64 bf16, 128-byte swizzle

struct SlotInfo {  // one chunk slot of the workspace
    int tok_start;  // first token (row of the packed batch)
    int len;        // valid tokens in the chunk (1..64)
};
struct SeqInfo {
    int first_slot;
    int num_chunks;
};

// Byte offset of element (row, col) inside a [rows x 64] bf16 tile with 128-byte rows and the 128B swizzle.
__device__ __forceinline__ uint32_t sw128(uint32_t row, uint32_t col) {
    return row * 128u + ((((col >> 3) ^ (row & 7u)) << 4) | ((col & 7u) << 1));
}

// Shared-memory descriptor of an MN-major bf16 operand stored as tiles of [K rows x 64 MN elements] (128-byte rows,
// 128B swizzle): 8 K-rows form a 1024-byte swizzle atom (SBO = 1024, the K direction), the next 64 MN elements
// are `tile_stride` bytes further (LBO). An MMA consumes 16 K-rows: advance the address by 2048 bytes (+128 here).
__device__ __forceinline__ uint64_t make_sw128_mnmajor_desc(uint32_t smem_addr, uint32_t tile_stride) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>((tile_stride >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}
constexpr uint32_t kBMnMajor = 1u << 16;  // instruction-descriptor bit: B operand is MN-major

// 16-byte asynchronous copy global -> shared; `bytes` = 16, or 0 to write zeros without reading.
__device__ __forceinline__ void cp_async16_zfill(uint32_t dst, const void* src, uint32_t bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit_group() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void st_shared_v2(uint32_t addr, uint32_t a, uint32_t b) {
    asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ void st_shared_b16(uint32_t addr, __nv_bfloat16 v) {
    asm volatile("st.shared.b16 [%0], %1;" ::"r"(addr), "h"(*reinterpret_cast<unsigned short*>(&v)) : "memory");
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint4 v) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
    __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&t);
}
// x / (1 + e^-x) on the special-function unit: the same two instructions as s1_conv_silu's, so both give the same bits.
__device__ __forceinline__ float silu_sfu(float v) {
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(v * -1.4426950408889634f));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.f + e));
    return v * r;
}

#ifdef S1_MEASURE
// Timing aid of measurement builds only: SM clock stamps of one CTA's phases (read back with s1_measure_read_stamps).
__device__ long long s1_phase_stamps[64];
#define S1_STAMP(k)                                                                                   \
    do {                                                                                              \
        if (blockIdx.x == gridDim.x / 2 && blockIdx.y == gridDim.y - 1 && threadIdx.x == 0) s1_phase_stamps[k] = clock64(); \
    } while (0)
#else
#define S1_STAMP(k) do { } while (0)
#endif

struct PrepParams {
    const float* q;
    const float* k;
    const float* v;
    const float* g;
    const float* beta;
    const SlotInfo* slots;
    int num_slots, H;
    __nv_bfloat16* wq;   // [H * slots * 128, 128]: rows 0..63 of a slot block = W, rows 64..127 = Q e^G
    __nv_bfloat16* ut;   // [H * slots * 128 (dv), 64 (token)]
    __nv_bfloat16* kn;   // [H * slots * 64 (token), 128 (dk)]: K e^{G_last - G}
    __nv_bfloat16* p;    // [H * slots * 64 (i), 64 (j)]
    float* decay;        // [H * slots]  e^{G_last}
    int* status;
    // fused-input form (s1_gated_delta_rule): q, k, v, g, beta are derived in the kernel from the layer's bf16 tensors
    const __nv_bfloat16* mixed;  // [T, 2 * Hk * 128 + H * 128] = [q | k | v] after conv + SiLU
    long long ldm;
    const __nv_bfloat16* bproj;  // [T, H]
    const __nv_bfloat16* aproj;  // [T, H]
    long long ldba;
    const float* dt_bias;        // [H]
    const float* neg_exp_a;      // [H]
    int Hk;                      // key heads (H value heads; key head = value head / (H / Hk))
    // conv form (s1_gated_delta_rule_conv): `mixed` is the projection BEFORE the causal conv + SiLU; the kernel applies them
    // to the rows it stages (src/kernels/qwen35.cu:3-29; 4 taps, same arithmetic as s1_conv_silu)
    const __nv_bfloat16* conv_w;   // [2 * Hk * 128 + H * 128, 4]
    const int32_t* positions;      // [T] index of every token inside its sequence
};

// The f32 matrix A of each chunk is kept transposed in shared memory, AT[j][i] = A[i][j] (64 floats per row): the thread
// that forms row i of A writes a column of AT (lanes = consecutive addresses), and the substitution reads four or sixteen
// consecutive i of one j with 16-byte loads that every lane of a warp shares.
constexpr int kAStride = 64;
constexpr int kTRows = 48;    // rows of the solved columns kept in shared memory for the later 16-row blocks (rows 48.. are never re-read)
constexpr int kPrepSmem = 2 * kTileBytes /*Kop*/ + 2 * kTileBytes /*Qop*/ + 2 * 2 * kTileBytes /*XT*/ +
                          2 * kTileBytes /*Top*/ + 128 * kAStride * 4 /*A^T*/ + 128 * 4 * 4 /*G, beta, e^G, e^(Glast-G)*/ +
                          kTRows * 128 * 4 /*solved rows*/ + 1024 + 64;

constexpr int kPrepThreads = 512;  // four threads per stacked token row: each owns a quarter of the features / columns
constexpr int kPrepRowsPerWarp = 128 / (kPrepThreads / 32);  // rows a warp stages and converts in the row-wise phases (8)

// FUSED = false: q, k (already normalised), v, g, beta given as f32 (the drop-in form of `chunked_delta_rule`).
// FUSED = true : the steps of `delta_inputs` (src/archs/qwen35_text.rs:528-579) happen here: bf16 rows of the mixed
//                projection are staged, L2-normalised per row by the warp that converts them, gates from a / b.
//                CONV (with FUSED): the staged rows are the projection before the depthwise causal conv; every row's conv +
//                SiLU is formed on the way from the staging area to the operands (three rows of history per chunk are
//                staged with it), so the conv kernel's pass over the [T, channels] tensor and back disappears.
template <bool FUSED, bool CONV = false>
__global__ void __launch_bounds__(kPrepThreads, 1) s1_delta_prep_kernel(const PrepParams p) {
    static_assert(FUSED || !CONV, "the conv form reads the layer's bf16 projection");
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* al = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t kop = base;                       // 2 tiles [128 rows x 64 dk]
    const uint32_t qop = kop + 2 * kTileBytes;       // 2 tiles
    const uint32_t xt = qop + 2 * kTileBytes;        // 4 tiles [128 tokens x 64 features]: beta e^G K (2), beta V (2)
    const uint32_t top = xt + 4 * kTileBytes;        // 2 tiles [128 rows (i) x 64 (j)]
    float* amat = reinterpret_cast<float*>(al + 10 * kTileBytes);  // [128][kAStride]
    float* gsh = amat + 128 * kAStride;              // cumulative gate per stacked row
    float* bsh = gsh + 128;
    float* egs = bsh + 128;   // e^G per stacked row
    float* egl = egs + 128;   // e^{G_last - G}
    float* tbuf = egl + 128;  // [kTRows][128]: entry j of the solved column of stacked row r at tbuf[j * 128 + r]
    uint64_t* bar = reinterpret_cast<uint64_t*>(tbuf + kTRows * 128);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    S1_STAMP(0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q4 = warp & 3;             // TMEM lane quarter of this warp
    const int fq = warp >> 2;            // which quarter of the features / of the chunk's columns this thread handles
    const int r = q4 * 32 + lane;        // stacked token row = TMEM lane
    const int half = r >> 6, i = r & 63;  // which of the two chunks, row inside it
    const int head = blockIdx.y;
    const int slot = 2 * blockIdx.x + half;
    const bool slot_ok = slot < p.num_slots;
    const SlotInfo si = slot_ok ? p.slots[slot] : SlotInfo{0, 0};
    const bool valid = i < si.len;
    const long long tok = si.tok_start + i;
    const long long hs = static_cast<long long>(head) * p.num_slots + slot;  // (head, slot) block index

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(bar), 1);
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(tmem_slot), 256);
        tmem_relinquish();
    }

    // ---- raw f32 rows of Q and K: all 128 KB requested at once with cp.async (rows past a chunk's end are
    //      zero-filled), into staging areas that alias buffers which are not in use yet:
    //      Q over the B-operand tiles (xt), K over the Tm operand and the A matrix (top, amat)
    const SlotInfo s0 = p.slots[min(2 * static_cast<int>(blockIdx.x), p.num_slots - 1)];
    const SlotInfo s1 = (2 * blockIdx.x + 1 < p.num_slots) ? p.slots[2 * blockIdx.x + 1] : SlotInfo{0, 0};
    const uint32_t stage_q = xt, stage_k = top, stage_v = kop;
    // conv form: history rows of q, k in the (not yet used) solved-rows buffer, those of v over the Q tiles once they are
    // consumed; the rows after conv + SiLU of q in the upper half of xt, of k where A^T goes later
    const uint32_t halo_qk = smem_u32(tbuf), halo_v = qop;
    const uint32_t post_q = xt + 2 * kTileBytes, post_k = smem_u32(amat);
    int pos0[2] = {0, 0};
    constexpr int kRowBytes = FUSED ? 256 : 512;  // staged row: 128 bf16 or 128 f32
    const int kw = FUSED ? p.Hk * 128 : 0;
    const int hk = FUSED ? head / (p.H / p.Hk) : 0;
    if constexpr (FUSED) {
#pragma unroll 4
        for (int u = 0; u < kPrepRowsPerWarp / 2; ++u) {  // one 16-byte piece per lane: two 256-byte rows per warp instruction
            const int row = warp * kPrepRowsPerWarp + 2 * u + (lane >> 4), ri = row & 63;
            const SlotInfo sr = (row >> 6) ? s1 : s0;
            const bool rv = ri < sr.len;
            const long long src = rv ? static_cast<long long>(sr.tok_start + ri) * p.ldm + hk * 128 + 8 * (lane & 15) : 0;
            cp_async16_zfill(stage_q + row * 256 + (lane & 15) * 16, p.mixed + src, rv ? 16u : 0u);
            cp_async16_zfill(stage_k + row * 256 + (lane & 15) * 16, p.mixed + src + (rv ? kw : 0), rv ? 16u : 0u);
        }
        if constexpr (CONV) {
            // the three rows before each chunk's first token (zero where the sequence starts later): q rows of chunk 0, 1,
            // then k rows of chunk 0, 1; two rows per warp instruction, six instructions
            pos0[0] = s0.len > 0 ? __ldg(p.positions + s0.tok_start) : 0;
            pos0[1] = s1.len > 0 ? __ldg(p.positions + s1.tok_start) : 0;
            if (warp < 6) {
                const int r12 = 2 * warp + (lane >> 4);
                const int which = r12 / 6, hh = (r12 % 6) / 3, back = 3 - r12 % 3;
                const SlotInfo sr = hh ? s1 : s0;
                const bool rv = sr.len > 0 && pos0[hh] >= back;
                const long long src = rv ? static_cast<long long>(sr.tok_start - back) * p.ldm + hk * 128 + which * kw + 8 * (lane & 15) : 0;
                cp_async16_zfill(halo_qk + r12 * 256 + (lane & 15) * 16, p.mixed + src, rv ? 16u : 0u);
            }
        }
    } else {
#pragma unroll 4
        for (int u = 0; u < kPrepRowsPerWarp; ++u) {
            const int row = warp * kPrepRowsPerWarp + u, ri = row & 63;
            const SlotInfo sr = (row >> 6) ? s1 : s0;
            const bool rv = ri < sr.len;
            const long long base_f = rv ? (static_cast<long long>(sr.tok_start + ri) * p.H + head) * kD + 4 * lane : 0;
            cp_async16_zfill(stage_q + row * 512 + lane * 16, p.q + base_f, rv ? 16u : 0u);
            cp_async16_zfill(stage_k + row * 512 + lane * 16, p.k + base_f, rv ? 16u : 0u);
        }
    }
    cp_async_commit_group();
    S1_STAMP(2);   // loads requested

    // ---- gates: inclusive cumulative sum inside each chunk (two warps per chunk)
    float gi = 0.f, bi = 0.f;
    if (valid) {
        if constexpr (FUSED) {  // beta = sigmoid(b), g = softplus(a + dt_bias) * (-exp(A_log))  (:567-571)
            const float bb = __bfloat162float(p.bproj[tok * p.ldba + head]);
            const float aa = __bfloat162float(p.aproj[tok * p.ldba + head]) + p.dt_bias[head];
            bi = 1.f / (1.f + expf(-bb));
            gi = (fmaxf(aa, 0.f) + logf(expf(-fabsf(aa)) + 1.f)) * p.neg_exp_a[head];
        } else {
            gi = p.g[tok * p.H + head];
            bi = p.beta[tok * p.H + head];
        }
    }
    float G = gi;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, G, o);
        if (lane >= o) G += t;
    }
    if (lane == 31) gsh[r] = G;  // warp total, parked in the slot of the warp's last row
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (q4 & 1) G += gsh[r - lane - 1];  // second warp of a chunk adds the first warp's total
    __syncthreads();
    gsh[r] = G;
    bsh[r] = bi;
    __syncthreads();
    S1_STAMP(3);   // gates
    const uint32_t tmem = *tmem_slot;
    const float Glast = gsh[half * 64 + 63];
    const float eG = __expf(G);
    const float eGl = __expf(Glast - G);
    if (slot_ok && i == 0 && fq == 0) p.decay[hs] = __expf(Glast);

    // ---- operands, one warp per row at a time (lane = 4 consecutive features), from the staged f32 rows:
    //      Q, K, beta e^G K as bf16 [token x feature] tiles; Q e^G and K e^{G_last - G} to the workspace
    //      (beta V is staged later, by the warps that are idle during the triangular solve)
    if (fq == 0) {
        egs[r] = eG;
        egl[r] = eGl;
    }
    cp_async_wait_all();
    __syncthreads();
    S1_STAMP(4);   // staged rows landed
    const int tile = lane >> 4, col = (4 * lane) & 63;
    // this lane's 4 features of a staged row
    auto fetch4 = [&](uint32_t stage, int row) -> float4 {
        if constexpr (FUSED) {
            uint32_t lo, hi;
            asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(lo), "=r"(hi) : "r"(stage + row * 256 + lane * 8) : "memory");
            const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&lo), b = *reinterpret_cast<const __nv_bfloat162*>(&hi);
            return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
        } else {
            const uint4 raw = ld_shared_v4(stage + row * 512 + lane * 16);
            return make_float4(__uint_as_float(raw.x), __uint_as_float(raw.y), __uint_as_float(raw.z), __uint_as_float(raw.w));
        }
    };
    // conv form: this lane's four channels' taps of one tensor as bf16x2 pairs of neighbouring channels, and the conv +
    // SiLU of eight consecutive rows of a chunk from the staged rows (or the history rows, for the chunk's first three):
    // the arithmetic of s1_conv_silu, tap by tap in bf16 (`__hmul2_rn` / `__hadd2_rn`, never contracted), SiLU in f32
    auto conv_taps = [&](int channel, uint32_t (&wt)[4][2]) {
        const uint4 a = __ldg(reinterpret_cast<const uint4*>(p.conv_w + static_cast<long long>(channel) * 4));
        const uint4 b = __ldg(reinterpret_cast<const uint4*>(p.conv_w + static_cast<long long>(channel) * 4) + 1);
        wt[0][0] = __byte_perm(a.x, a.z, 0x5410), wt[1][0] = __byte_perm(a.x, a.z, 0x7632);
        wt[2][0] = __byte_perm(a.y, a.w, 0x5410), wt[3][0] = __byte_perm(a.y, a.w, 0x7632);
        wt[0][1] = __byte_perm(b.x, b.z, 0x5410), wt[1][1] = __byte_perm(b.x, b.z, 0x7632);
        wt[2][1] = __byte_perm(b.y, b.w, 0x5410), wt[3][1] = __byte_perm(b.y, b.w, 0x7632);
    };
    auto ld2 = [&](uint32_t addr) -> uint2 {
        uint2 v;
        asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr) : "memory");
        return v;
    };
    // rows row0 .. row0 + 7 of the stacked pair (all in one chunk, whose history rows sit at `halo`); rows at or past `len`
    // come out as zero, like rows that were never staged
    auto conv8 = [&](uint32_t stage, uint32_t halo, int row0, int len, const uint32_t (&wt)[4][2], uint2 (&out)[8]) {
        const int ri0 = row0 & 63;
        uint2 x[11];
#pragma unroll
        for (int t = 0; t < 11; ++t) {
            const int idx = ri0 - 3 + t;
            x[t] = (idx >= 0) ? ld2(stage + (row0 - 3 + t) * 256 + lane * 8) : ld2(halo + (idx + 3) * 256 + lane * 8);
        }
        const __nv_bfloat162 zero2 = __floats2bfloat162_rn(0.f, 0.f);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            __nv_bfloat162 a0 = zero2, a1 = zero2;
#pragma unroll
            for (int tap = 0; tap < 4; ++tap) {
                a0 = __hadd2_rn(a0, __hmul2_rn(*reinterpret_cast<const __nv_bfloat162*>(&x[u + tap].x), *reinterpret_cast<const __nv_bfloat162*>(&wt[tap][0])));
                a1 = __hadd2_rn(a1, __hmul2_rn(*reinterpret_cast<const __nv_bfloat162*>(&x[u + tap].y), *reinterpret_cast<const __nv_bfloat162*>(&wt[tap][1])));
            }
            const float2 f0 = __bfloat1622float2(a0), f1 = __bfloat1622float2(a1);
            const bool live = ri0 + u < len;
            out[u].x = live ? pack2(silu_sfu(f0.x), silu_sfu(f0.y)) : 0u;
            out[u].y = live ? pack2(silu_sfu(f1.x), silu_sfu(f1.y)) : 0u;
        }
    };
    const uint32_t src_q = CONV ? post_q : stage_q, src_k = CONV ? post_k : stage_k;
    if constexpr (CONV) {
        const int row0 = warp * kPrepRowsPerWarp, hh = row0 >> 6;
        const int len = hh ? s1.len : s0.len;
        uint32_t wt[4][2];
        uint2 o8[8];
        conv_taps(hk * 128 + 4 * lane, wt);
        conv8(stage_q, halo_qk + hh * 768, row0, len, wt, o8);
#pragma unroll
        for (int u = 0; u < 8; ++u) st_shared_v2(post_q + (row0 + u) * 256 + lane * 8, o8[u].x, o8[u].y);
        conv_taps(kw + hk * 128 + 4 * lane, wt);
        conv8(stage_k, halo_qk + 1536 + hh * 768, row0, len, wt, o8);
#pragma unroll
        for (int u = 0; u < 8; ++u) st_shared_v2(post_k + (row0 + u) * 256 + lane * 8, o8[u].x, o8[u].y);
        // (every lane reads back only what it wrote itself: no barrier is needed before the loops below)
    }
    // fused form: L2 norms of this warp's q rows and k rows, all the warp reductions interleaved
    // (q = l2norm(q) * 128^-1/2, k = l2norm(k), 1e-6 inside the root: src/archs/qwen35_text.rs:560-565)
    float qsc[kPrepRowsPerWarp], ksc[kPrepRowsPerWarp];
    if constexpr (FUSED) {
#pragma unroll
        for (int u = 0; u < kPrepRowsPerWarp; ++u) {
            const float4 a = fetch4(src_q, warp * kPrepRowsPerWarp + u), b = fetch4(src_k, warp * kPrepRowsPerWarp + u);
            qsc[u] = a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
            ksc[u] = b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
            for (int u = 0; u < kPrepRowsPerWarp; ++u) {
                qsc[u] += __shfl_xor_sync(0xffffffffu, qsc[u], o);
                ksc[u] += __shfl_xor_sync(0xffffffffu, ksc[u], o);
            }
        }
#pragma unroll
        for (int u = 0; u < kPrepRowsPerWarp; ++u) {
            qsc[u] = 0.08838834764831845f * rsqrtf(qsc[u] + 1e-6f);
            ksc[u] = rsqrtf(ksc[u] + 1e-6f);
        }
    }
#pragma unroll
    for (int u = 0; u < kPrepRowsPerWarp; ++u) {  // Q first: its staging area is where beta e^G K goes next
        const int row = warp * kPrepRowsPerWarp + u, ri = row & 63;
        const int rslot = 2 * blockIdx.x + (row >> 6);
        float4 qq = fetch4(src_q, row);
        if constexpr (FUSED) qq.x *= qsc[u], qq.y *= qsc[u], qq.z *= qsc[u], qq.w *= qsc[u];
        const float eg = egs[row];
        st_shared_v2(qop + tile * kTileBytes + sw128(row, col), pack2(qq.x, qq.y), pack2(qq.z, qq.w));
        if (rslot < p.num_slots) {
            const long long hsr = static_cast<long long>(head) * p.num_slots + rslot;
            *reinterpret_cast<uint2*>(p.wq + (hsr * 128 + 64 + ri) * kD + 4 * lane) =
                make_uint2(pack2(qq.x * eg, qq.y * eg), pack2(qq.z * eg, qq.w * eg));
        }
    }
    __syncthreads();
    S1_STAMP(5);   // Q operands written
#pragma unroll
    for (int u = 0; u < kPrepRowsPerWarp; ++u) {
        const int row = warp * kPrepRowsPerWarp + u, ri = row & 63;
        const int rslot = 2 * blockIdx.x + (row >> 6);
        float4 kk = fetch4(src_k, row);
        if constexpr (FUSED) kk.x *= ksc[u], kk.y *= ksc[u], kk.z *= ksc[u], kk.w *= ksc[u];
        const float el = egl[row], sk = bsh[row] * egs[row];
        const uint32_t off = tile * kTileBytes + sw128(row, col);
        st_shared_v2(kop + off, pack2(kk.x, kk.y), pack2(kk.z, kk.w));
        st_shared_v2(xt + off, pack2(kk.x * sk, kk.y * sk), pack2(kk.z * sk, kk.w * sk));
        if (rslot < p.num_slots) {
            const long long hsr = static_cast<long long>(head) * p.num_slots + rslot;
            *reinterpret_cast<uint2*>(p.kn + (hsr * 64 + ri) * kD + 4 * lane) =
                make_uint2(pack2(kk.x * el, kk.y * el), pack2(kk.z * el, kk.w * el));
        }
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    S1_STAMP(6);   // K operands written

    // ---- K K^T -> TMEM columns 0..127, Q K^T -> 128..255 (both chunks at once; cross-chunk blocks are ignored)
    if (threadIdx.x == 0) {
        tc_fence_after();
        constexpr uint32_t idesc = make_idesc(1, 128, 128);
#pragma unroll
        for (int kt = 0; kt < 2; ++kt)
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                const uint64_t dk = make_sw128_kmajor_desc(kop + kt * kTileBytes) + 2u * kk;
                const uint64_t dq = make_sw128_kmajor_desc(qop + kt * kTileBytes) + 2u * kk;
                umma_bf16(tmem, dk, dk, idesc, (kt | kk) ? 1u : 0u);
                umma_bf16(tmem + 128, dq, dk, idesc, (kt | kk) ? 1u : 0u);
            }
        umma_commit(smem_u32(bar));
    }
    __syncwarp();
    bool ok = mbar_wait(smem_u32(bar), 0, abort_flag);
    S1_STAMP(7);   // first MMAs done
    ok = __all_sync(0xffffffffu, ok);
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>(q4 * 32) << 16);
    // K and Q tiles are consumed: their 64 KB now stage the raw V rows, in flight while A and P are formed
    if constexpr (FUSED) {
#pragma unroll 4
        for (int u = 0; u < kPrepRowsPerWarp / 2; ++u) {
            const int row = warp * kPrepRowsPerWarp + 2 * u + (lane >> 4), ri = row & 63;
            const SlotInfo sr = (row >> 6) ? s1 : s0;
            const bool rv = ok && ri < sr.len;
            const long long src = rv ? static_cast<long long>(sr.tok_start + ri) * p.ldm + 2 * kw + head * 128 + 8 * (lane & 15) : 0;
            cp_async16_zfill(stage_v + row * 256 + (lane & 15) * 16, p.mixed + src, rv ? 16u : 0u);
        }
        if constexpr (CONV) {
            if (warp < 3) {  // the three v rows before each chunk's first token, over the consumed Q tiles
                const int r6 = 2 * warp + (lane >> 4);
                const int hh = r6 / 3, back = 3 - r6 % 3;
                const SlotInfo sr = hh ? s1 : s0;
                const bool rv = ok && sr.len > 0 && pos0[hh] >= back;
                const long long src = rv ? static_cast<long long>(sr.tok_start - back) * p.ldm + 2 * kw + head * 128 + 8 * (lane & 15) : 0;
                cp_async16_zfill(halo_v + r6 * 256 + (lane & 15) * 16, p.mixed + src, rv ? 16u : 0u);
            }
        }
    } else {
#pragma unroll 4
        for (int u = 0; u < kPrepRowsPerWarp; ++u) {
            const int row = warp * kPrepRowsPerWarp + u, ri = row & 63;
            const SlotInfo sr = (row >> 6) ? s1 : s0;
            const bool rv = ok && ri < sr.len;
            const long long base_f = rv ? (static_cast<long long>(sr.tok_start + ri) * p.H + head) * kD + 4 * lane : 0;
            cp_async16_zfill(stage_v + row * 512 + lane * 16, p.v + base_f, rv ? 16u : 0u);
        }
    }
    cp_async_commit_group();
    if (ok) {
        tc_fence_after();
        // this thread's 16 of the own chunk's 64 columns of row r
        {
            const int c = fq;
            uint32_t kk[16], qk[16];
            tmem_ld_32x32b_x16(lane_addr + half * 64 + c * 16, kk);
            tmem_ld_32x32b_x16(lane_addr + 128 + half * 64 + c * 16, qk);
            tmem_ld_wait();
            uint32_t pp[8];
#pragma unroll
            for (int e = 0; e < 16; ++e) {
                const int j = c * 16 + e;
                const float dec = __expf(G - gsh[half * 64 + j]);  // <= 1 wherever it is used (j <= i)
                amat[(half * 64 + j) * kAStride + i] = (j < i) ? bi * __uint_as_float(kk[e]) * dec : 0.f;  // A^T[j][i]
                const float pv = (j <= i) ? __uint_as_float(qk[e]) * dec : 0.f;
                if (e & 1) pp[e >> 1] = pack2(__uint_as_float(pp[e >> 1]), pv);
                else pp[e >> 1] = __float_as_uint(pv);
            }
            if (slot_ok) {
#pragma unroll
                for (int e = 0; e < 2; ++e)
                    *reinterpret_cast<uint4*>(p.p + (hs * 64 + i) * kC + c * 16 + 8 * e) =
                        make_uint4(pp[4 * e], pp[4 * e + 1], pp[4 * e + 2], pp[4 * e + 3]);
            }
        }
    }
    cp_async_wait_all();
    tc_fence_before();
    __syncthreads();
    S1_STAMP(8);   // A, P formed; V rows landed
    tc_fence_after();

    // ---- Tm = (I + A)^-1 by forward substitution, one column per thread (columns are independent: the warps of column
    //      quarter 0 solve); the others meanwhile fill the zero blocks of the block-diagonal operand (quarter 1) and stage
    //      beta V (quarters 2 and 3)
    if (fq == 1) {
        const uint32_t ttile = top + half * kTileBytes;
#pragma unroll
        for (int ii = 0; ii < 64; ++ii) st_shared_b16(ttile + sw128((1 - half) * 64 + ii, i), __float2bfloat16_rn(0.f));
    } else if (fq >= 2) {
        // beta V rows (staged) -> tiles 2, 3 of the B operand: 8 warps x 16 rows
        if constexpr (CONV) {
            uint32_t wt[4][2];
            conv_taps(2 * kw + head * 128 + 4 * lane, wt);
#pragma unroll 1
            for (int part = 0; part < 2; ++part) {
                const int row0 = (warp - 8) * 16 + 8 * part, hh = row0 >> 6;
                uint2 o8[8];
                conv8(stage_v, halo_v + hh * 768, row0, hh ? s1.len : s0.len, wt, o8);
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int row = row0 + u;
                    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&o8[u].x), hi = *reinterpret_cast<const __nv_bfloat162*>(&o8[u].y);
                    const float be = bsh[row];
                    st_shared_v2(xt + (2 + tile) * kTileBytes + sw128(row, col), pack2(__low2float(lo) * be, __high2float(lo) * be),
                                 pack2(__low2float(hi) * be, __high2float(hi) * be));
                }
            }
        } else {
#pragma unroll 4
            for (int u = 0; u < 16; ++u) {
                const int row = (warp - 8) * 16 + u;
                const float4 vv = fetch4(stage_v, row);
                const float be = bsh[row];
                st_shared_v2(xt + (2 + tile) * kTileBytes + sw128(row, col), pack2(vv.x * be, vv.y * be), pack2(vv.z * be, vv.w * be));
            }
        }
    } else {
        // Column i of Tm = (I + A)^-1: t[ii] = [ii == i] - sum_{j < ii} A[ii][j] t[j], in blocks of 16 rows. A block first
        // takes the contributions of the rows solved before it (a run-time loop over j: one 4-byte load of t[j] from this
        // thread's own column in shared memory, four shared 16-byte loads of A^T[j][16 b ..], 16 fmas), then finishes its own
        // 16 x 16 triangle in registers. The code is a few hundred instructions that are re-used by every block; the fully
        // unrolled 64-step form was ten times slower (2000 fmas of straight-line code that each warp executes once: it
        // ran at the speed of instruction fetch).
        const float* at = amat + (half * 64) * kAStride;   // at[j * 64 + ii] = A[ii][j]
        float* tcol = tbuf + r;                              // tcol[j * 128] = t[j] of this column
        const uint32_t ttile = top + half * kTileBytes;
#pragma unroll 1
        for (int b = 0; b < 4; ++b) {
            float acc[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) acc[e] = (16 * b + e == i) ? 1.f : 0.f;
#pragma unroll 4
            for (int j = 0; j < 16 * b; ++j) {
                const float tj = tcol[j * 128];
                const float4* arow = reinterpret_cast<const float4*>(at + j * kAStride + 16 * b);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float4 a = arow[q];
                    acc[4 * q] = fmaf(-a.x, tj, acc[4 * q]);
                    acc[4 * q + 1] = fmaf(-a.y, tj, acc[4 * q + 1]);
                    acc[4 * q + 2] = fmaf(-a.z, tj, acc[4 * q + 2]);
                    acc[4 * q + 3] = fmaf(-a.w, tj, acc[4 * q + 3]);
                }
            }
#pragma unroll
            for (int e2 = 0; e2 < 15; ++e2) {  // acc[e2] is final here: fold it into the rows below it
                const float4* arow = reinterpret_cast<const float4*>(at + (16 * b + e2) * kAStride + 16 * b);
#pragma unroll
                for (int q = (e2 + 1) / 4; q < 4; ++q) {
                    const float4 a = arow[q];
                    if (4 * q > e2) acc[4 * q] = fmaf(-a.x, acc[e2], acc[4 * q]);
                    if (4 * q + 1 > e2) acc[4 * q + 1] = fmaf(-a.y, acc[e2], acc[4 * q + 1]);
                    if (4 * q + 2 > e2) acc[4 * q + 2] = fmaf(-a.z, acc[e2], acc[4 * q + 2]);
                    if (4 * q + 3 > e2) acc[4 * q + 3] = fmaf(-a.w, acc[e2], acc[4 * q + 3]);
                }
            }
            // column i of this chunk's Tm -> k-tile `half` of the block-diagonal A operand; and, for the blocks still to come,
            // into this thread's own column of the f32 buffer
#pragma unroll
            for (int e = 0; e < 16; ++e) {
                st_shared_b16(ttile + sw128(half * 64 + 16 * b + e, i), __float2bfloat16_rn(acc[e]));
                if (b < 3) tcol[(16 * b + e) * 128] = acc[e];
            }
        }
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    S1_STAMP(9);   // solve + beta V staged

    // ---- [W | U] = Tm [beta e^G K | beta V]  (M = 128 stacked rows, N = 256, K = 128 stacked tokens)
    if (threadIdx.x == 0) {
        tc_fence_after();
        // A = Tm (K-major: rows i, 64 j per tile); B = [beta e^G K | beta V] as stored, token rows x features (MN-major)
        constexpr uint32_t idesc = make_idesc(1, 128, 256) | kBMnMajor;
        const uint64_t bdesc = make_sw128_mnmajor_desc(xt, kTileBytes);
#pragma unroll
        for (int kt = 0; kt < 2; ++kt)
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
                umma_bf16(tmem, make_sw128_kmajor_desc(top + kt * kTileBytes) + 2u * kk, bdesc + 128u * (kt * 4 + kk), idesc,
                          (kt | kk) ? 1u : 0u);
        umma_commit(smem_u32(bar));
    }
    __syncwarp();
    ok = mbar_wait(smem_u32(bar), 1, abort_flag);
    S1_STAMP(10);  // second MMA done
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
        tc_fence_after();
        {  // W row: this thread's 32 of the 128 key features
            const int c = fq;
            uint32_t w[32];
            tmem_ld_32x32b_x32(lane_addr + c * 32, w);
            tmem_ld_wait();
            if (slot_ok) {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    *reinterpret_cast<uint4*>(p.wq + (hs * 128 + i) * kD + c * 32 + 8 * e) = make_uint4(
                        pack2(__uint_as_float(w[8 * e]), __uint_as_float(w[8 * e + 1])), pack2(__uint_as_float(w[8 * e + 2]), __uint_as_float(w[8 * e + 3])),
                        pack2(__uint_as_float(w[8 * e + 4]), __uint_as_float(w[8 * e + 5])), pack2(__uint_as_float(w[8 * e + 6]), __uint_as_float(w[8 * e + 7])));
            }
        }
        {  // U row -> transposed: ut[dv][token]; this thread's 32 of the 128 value columns
            const int c = fq;
            uint32_t u[32];
            tmem_ld_32x32b_x32(lane_addr + 128 + c * 32, u);
            tmem_ld_wait();
            if (slot_ok) {
#pragma unroll
                for (int e = 0; e < 32; ++e) p.ut[(hs * 128 + c * 32 + e) * kC + i] = __float2bfloat16_rn(__uint_as_float(u[e]));
            }
        }
    } else if (atomicCAS(p.status, 0, 2) == 0) {
        p.status[1] = blockIdx.x;
        p.status[2] = 10;
        p.status[3] = blockIdx.y;
    }
    tc_fence_before();
    __syncthreads();
    S1_STAMP(11);  // write-out done
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem, 256);
    }
}

// =====================================================================================================================
struct ScanParams {
    const SeqInfo* seqs;
    const SlotInfo* slots;
    const float* decay;
    float* out;  // [T, H, 128]
    int num_slots, H;
    int* status;
};

constexpr int kStageBytes = 2 * kTileBytes /*WQ*/ + kTileBytes /*UT*/ + kTileBytes /*K~*/ + kTileBytes / 2 /*P*/;  // 73728
constexpr int kScanSmem = 2 * kStageBytes + 2 * kTileBytes /*S^T*/ + 1024 + 160;

__global__ void __launch_bounds__(160, 1)
s1_delta_scan_kernel(const __grid_constant__ CUtensorMap tmWQ, const __grid_constant__ CUtensorMap tmUT,
                     const __grid_constant__ CUtensorMap tmKN, const __grid_constant__ CUtensorMap tmP, const ScanParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* al = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t sop = base + 2 * kStageBytes;  // S^T as bf16 A operand: 2 tiles [128 dv x 64 dk]
    uint64_t* bars = reinterpret_cast<uint64_t*>(al + 2 * kStageBytes + 2 * kTileBytes);
    // bars: 0,1 full; 2,3 empty; 4 (W S)^T done; 5 V' ready; 6 O^T done; 7 S ready; 8 dS^T done
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t b0 = smem_u32(bars);
    const uint32_t full0 = b0, empty0 = b0 + 16, bar_m1 = b0 + 32, bar_v = b0 + 40, bar_m2 = b0 + 48, bar_s = b0 + 56,
                   bar_m3 = b0 + 64;
    // TMEM columns: 0..63 (W S)^T, 64..127 / 128..191 O^T of even / odd chunks, 192..319 dS^T
    constexpr uint32_t kColO = 64, kColDS = 192;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.y;
    const SeqInfo sq = p.seqs[blockIdx.x];
    const int n = sq.num_chunks;
    if (n <= 0) return;

    if (threadIdx.x == 0) {
        mbar_init(full0, 1);
        mbar_init(full0 + 8, 1);
        mbar_init(empty0, 1);
        mbar_init(empty0 + 8, 1);
        mbar_init(bar_m1, 1);
        mbar_init(bar_v, 4);
        mbar_init(bar_m2, 1);
        mbar_init(bar_s, 4);
        mbar_init(bar_m3, 1);
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmWQ);
        tma_prefetch_desc(&tmUT);
        tma_prefetch_desc(&tmKN);
        tma_prefetch_desc(&tmP);
    }
    if (warp == 4) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    int fail = 0;

    if (warp == 4) {
        // ------------------------------------------------ TMA producer + MMA issuer (one thread)
        if (lane == 0) {
            auto load = [&](int c) {
                const int st = c & 1;
                const uint32_t sb = base + st * kStageBytes, fb = full0 + 8u * st;
                const int hs = head * p.num_slots + sq.first_slot + c;
                mbar_arrive_expect_tx(fb, kStageBytes);
                tma_load_2d(sb, &tmWQ, 0, hs * 128, fb);
                tma_load_2d(sb + kTileBytes, &tmWQ, 64, hs * 128, fb);
                tma_load_2d(sb + 2 * kTileBytes, &tmUT, 0, hs * 128, fb);
                tma_load_2d(sb + 3 * kTileBytes, &tmKN, 0, hs * 64, fb);               // dk 0..63  of 64 tokens (8 KB)
                tma_load_2d(sb + 3 * kTileBytes + kTileBytes / 2, &tmKN, 64, hs * 64, fb);  // dk 64..127
                tma_load_2d(sb + 4 * kTileBytes, &tmP, 0, hs * 64, fb);
            };
            load(0);
            for (int c = 0; c < n && !fail; ++c) {
                const int st = c & 1;
                const uint32_t sb = base + st * kStageBytes;
                if (c + 1 < n) {
                    if (c >= 1 && !mbar_wait(empty0 + 8u * ((c + 1) & 1), ((c - 1) >> 1) & 1, abort_flag)) { fail = 1; break; }
                    load(c + 1);
                }
                if (!mbar_wait(full0 + 8u * st, (c >> 1) & 1, abort_flag)) { fail = 2; break; }
                if (!mbar_wait(bar_s, c & 1, abort_flag)) { fail = 3; break; }
                tc_fence_after();
                const uint32_t o_col = kColO + 64u * (c & 1);
                {   // (W S)^T = S^T W^T, then the state part of the output O^T = S^T (Q e^G)^T : M = 128 (dv), N = 64, K = 128 (dk)
                    constexpr uint32_t idesc = make_idesc(1, 128, 64);
#pragma unroll
                    for (int kt = 0; kt < 2; ++kt)
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk)
                            umma_bf16(tmem, make_sw128_kmajor_desc(sop + kt * kTileBytes) + 2u * kk,
                                      make_sw128_kmajor_desc(sb + kt * kTileBytes) + 2u * kk, idesc, (kt | kk) ? 1u : 0u);
                    umma_commit(bar_m1);
#pragma unroll
                    for (int kt = 0; kt < 2; ++kt)
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk)  // rows 64..127 of the tile hold Q e^G (8192 bytes further)
                            umma_bf16(tmem + o_col, make_sw128_kmajor_desc(sop + kt * kTileBytes) + 2u * kk,
                                      make_sw128_kmajor_desc(sb + kt * kTileBytes + 8192) + 2u * kk, idesc, (kt | kk) ? 1u : 0u);
                }
                if (!mbar_wait(bar_v, c & 1, abort_flag)) { fail = 4; break; }
                tc_fence_after();
                {
                    constexpr uint32_t idesc_p = make_idesc(1, 128, 64), idesc_k = make_idesc(1, 128, 128) | kBMnMajor;
                    const uint32_t vt = sb + 2 * kTileBytes, ktile = sb + 3 * kTileBytes, ptile = sb + 4 * kTileBytes;
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)  // dS^T = V'^T K~ ; K~ as stored: token rows x dk (MN-major B, two 8 KB tiles)
                        umma_bf16(tmem + kColDS, make_sw128_kmajor_desc(vt) + 2u * kk,
                                  make_sw128_mnmajor_desc(ktile, kTileBytes / 2) + 128u * kk, idesc_k, kk ? 1u : 0u);
                    umma_commit(bar_m3);  // the state update (the critical path) can start
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)  // O^T += V'^T P^T  (K = 64 tokens j)
                        umma_bf16(tmem + o_col, make_sw128_kmajor_desc(vt) + 2u * kk, make_sw128_kmajor_desc(ptile) + 2u * kk, idesc_p, 1u);
                    umma_commit(bar_m2);
                    umma_commit(empty0 + 8u * st);
                }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------ state / V' / output warps: thread = value row d
        const int d = threadIdx.x;  // 0..127 = TMEM lane
        const uint32_t lane_addr = tmem + (static_cast<uint32_t>(warp * 32) << 16);
        float S[kD];
#pragma unroll
        for (int j = 0; j < kD; ++j) S[j] = 0.f;
#pragma unroll
        for (int c = 0; c < 16; ++c) st_shared_v4(sop + (c >> 3) * kTileBytes + sw128(d, (c & 7) * 8), make_uint4(0u, 0u, 0u, 0u));
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_s);

        for (int c = 0; c < n; ++c) {
            const int st = c & 1;
            const uint32_t sb = base + st * kStageBytes;
            const int slot = sq.first_slot + c;
            const SlotInfo si = p.slots[slot];
            const float dec = p.decay[head * p.num_slots + slot];
            bool ok = mbar_wait(full0 + 8u * st, (c >> 1) & 1, abort_flag);
            ok = ok && mbar_wait(bar_m1, c & 1, abort_flag);
            if (!__all_sync(0xffffffffu, ok)) { fail = 5; break; }
            tc_fence_after();
            // V'^T row: U^T row (shared memory) minus (W S)^T row (TMEM columns 0..63), back in place as bf16
            {
                uint32_t ws[2][32];
                tmem_ld_32x32b_x32(lane_addr, ws[0]);
                tmem_ld_32x32b_x32(lane_addr + 32, ws[1]);
                tmem_ld_wait();
                const uint32_t ut = sb + 2 * kTileBytes;
#pragma unroll
                for (int ch = 0; ch < 8; ++ch) {
                    const uint32_t addr = ut + sw128(d, ch * 8);
                    const uint4 u = ld_shared_v4(addr);
                    const uint32_t uu[4] = {u.x, u.y, u.z, u.w};
                    uint32_t o[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const __nv_bfloat162 t = *reinterpret_cast<const __nv_bfloat162*>(&uu[e]);
                        const int j = ch * 8 + 2 * e;
                        o[e] = pack2(__low2float(t) - __uint_as_float(ws[j >> 5][j & 31]), __high2float(t) - __uint_as_float(ws[(j + 1) >> 5][(j + 1) & 31]));
                    }
                    st_shared_v4(addr, make_uint4(o[0], o[1], o[2], o[3]));
                }
            }
            fence_proxy_async_smem();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_v);

            ok = mbar_wait(bar_m3, c & 1, abort_flag);
            if (!__all_sync(0xffffffffu, ok)) { fail = 6; break; }
            tc_fence_after();
            // state: S <- e^{G_last} S + dS ; refresh the bf16 operand copy (this is the chain the next chunk waits on)
#pragma unroll
            for (int cb = 0; cb < 4; ++cb) {
                uint32_t ds[32];
                tmem_ld_32x32b_x32(lane_addr + kColDS + cb * 32, ds);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 32; ++e) S[cb * 32 + e] = fmaf(dec, S[cb * 32 + e], __uint_as_float(ds[e]));
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = cb * 32 + 8 * e;
                    st_shared_v4(sop + (j >> 6) * kTileBytes + sw128(d, j & 63),
                                 make_uint4(pack2(S[j], S[j + 1]), pack2(S[j + 2], S[j + 3]), pack2(S[j + 4], S[j + 5]), pack2(S[j + 6], S[j + 7])));
                }
            }
            fence_proxy_async_smem();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_s);

            // output of this chunk, off the critical path: O^T row -> out[token j][head][d]
            ok = mbar_wait(bar_m2, c & 1, abort_flag);
            if (!__all_sync(0xffffffffu, ok)) { fail = 7; break; }
            tc_fence_after();
            {
                uint32_t o[2][32];
                const uint32_t o_col = kColO + 64u * (c & 1);
                tmem_ld_32x32b_x32(lane_addr + o_col, o[0]);
                tmem_ld_32x32b_x32(lane_addr + o_col + 32, o[1]);
                tmem_ld_wait();
                float* obase = p.out + (static_cast<long long>(si.tok_start) * p.H + head) * kD + d;
#pragma unroll
                for (int j = 0; j < 64; ++j)
                    if (j < si.len) obase[static_cast<long long>(j) * p.H * kD] = __uint_as_float(o[j >> 5][j & 31]);
            }
            tc_fence_before();
        }
        __syncwarp();
    }
    if (fail && atomicCAS(p.status, 0, 3) == 0) {
        p.status[1] = blockIdx.x;
        p.status[2] = 20 + fail;
        p.status[3] = blockIdx.y;
    }
    if (*abort_flag) __nanosleep(200000);
    tc_fence_before();
    __syncthreads();
    if (warp == 4) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct WorkspaceLayout {
    size_t slots_off, seqs_off, decay_off, wq_off, ut_off, kn_off, p_off, total;
};
WorkspaceLayout layout(int num_seqs, int max_slots, int heads) {
    WorkspaceLayout L;
    size_t o = 0;
    L.slots_off = o, o = align_up(o + sizeof(SlotInfo) * max_slots, 256);
    L.seqs_off = o, o = align_up(o + sizeof(SeqInfo) * (num_seqs > 0 ? num_seqs : 1), 256);
    L.decay_off = o, o = align_up(o + sizeof(float) * static_cast<size_t>(heads) * max_slots, 256);
    const size_t hs = static_cast<size_t>(heads) * max_slots;
    L.wq_off = o, o = align_up(o + hs * 128 * 128 * 2, 1024);
    L.ut_off = o, o = align_up(o + hs * 128 * 64 * 2, 1024);
    L.kn_off = o, o = align_up(o + hs * 64 * 128 * 2, 1024);
    L.p_off = o, o = align_up(o + hs * 64 * 64 * 2, 1024);
    L.total = o;
    return L;
}

}  // namespace

extern "C" size_t s1_delta_rule_chunked_workspace(int num_seqs, int total_tokens, int heads) {
    if (num_seqs < 0 || total_tokens < 0 || heads < 1) return 0;
    const int max_slots = total_tokens / kC + num_seqs + 1;  // every sequence may end in a partial chunk
    return layout(num_seqs, max_slots, heads).total;
}

// Shared host path of the two entry points: chunk tables, prep (FUSED or not), scan.
static int run_chunked(s1_ctx* ctx, const char* who, PrepParams pp, bool fused, const int32_t* cu_seqlens_host, int num_seqs,
                       int total_tokens, int heads, float* out, void* workspace, size_t workspace_bytes) {
    if (num_seqs == 0 || total_tokens == 0) return S1_OK;
    static_assert(sizeof(SlotInfo) == sizeof(S1ChunkSlot) && sizeof(SeqInfo) == sizeof(S1SeqChunks), "the plan's chunk tables have this kernel's layout");
    const S1BatchPlan* plan = cu_seqlens_host ? nullptr : ctx->active_plan(num_seqs, total_tokens);
    if (!cu_seqlens_host && !plan)
        return s1_fail(ctx, S1_EINVAL, "%s: cu_seqlens_host is NULL and no batch plan for this batch is in use", who);
    const int max_slots = total_tokens / kC + num_seqs + 1;
    const WorkspaceLayout L = layout(num_seqs, max_slots, heads);
    if (workspace_bytes < L.total) return s1_fail(ctx, S1_EINVAL, "%s: workspace of %zu bytes, %zu needed", who, workspace_bytes, L.total);
    if ((reinterpret_cast<uintptr_t>(workspace) & 1023u) != 0) return s1_fail(ctx, S1_EINVAL, "%s: the workspace must be 1024-byte aligned", who);
    S1_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    int num_slots = 0;
    const SlotInfo* slots_dev = nullptr;
    const SeqInfo* seqs_dev = nullptr;
    if (plan) {
        // chunk tables built and copied once for the whole batch (s1_batch_plan)
        num_slots = plan->num_slots;
        slots_dev = reinterpret_cast<const SlotInfo*>(plan->dev + plan->slots_off);
        seqs_dev = reinterpret_cast<const SeqInfo*>(plan->dev + plan->seqs_off);
    } else {
        if (cu_seqlens_host[0] != 0 || cu_seqlens_host[num_seqs] != total_tokens)
            return s1_fail(ctx, S1_EINVAL, "%s: cu_seqlens must run from 0 to total_tokens", who);
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(ctx->stream, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone)
            return s1_fail(ctx, S1_EINVAL, "%s: with cu_seqlens_host the call copies tables from host memory and cannot be "
                                           "captured; build a batch plan first (s1_batch_plan)", who);
        // chunk tables, built on the host from the host copy of the offsets
        ctx->host_scratch.resize(sizeof(SlotInfo) * max_slots + sizeof(SeqInfo) * num_seqs);
        SlotInfo* slots = reinterpret_cast<SlotInfo*>(ctx->host_scratch.data());
        SeqInfo* seqs = reinterpret_cast<SeqInfo*>(ctx->host_scratch.data() + sizeof(SlotInfo) * max_slots);
        for (int s = 0; s < num_seqs; ++s) {
            const int a = cu_seqlens_host[s], b = cu_seqlens_host[s + 1];
            if (b < a) return s1_fail(ctx, S1_EINVAL, "%s: cu_seqlens must not decrease", who);
            seqs[s].first_slot = num_slots;
            seqs[s].num_chunks = (b - a + kC - 1) / kC;
            for (int t = a; t < b; t += kC) slots[num_slots++] = SlotInfo{t, (b - t < kC) ? b - t : kC};
        }
        if (num_slots == 0) return S1_OK;
        // the scan kernel runs one CTA per (sequence, head): start the longest sequences first
        std::stable_sort(seqs, seqs + num_seqs, [](const SeqInfo& a, const SeqInfo& b) { return a.num_chunks > b.num_chunks; });
        // (copies from pageable memory are staged before the call returns, so the host buffer can be reused at once)
        S1_CUDA_OK(ctx, cudaMemcpyAsync(ws + L.slots_off, slots, sizeof(SlotInfo) * num_slots, cudaMemcpyHostToDevice, ctx->stream));
        S1_CUDA_OK(ctx, cudaMemcpyAsync(ws + L.seqs_off, seqs, sizeof(SeqInfo) * num_seqs, cudaMemcpyHostToDevice, ctx->stream));
        slots_dev = reinterpret_cast<const SlotInfo*>(ws + L.slots_off);
        seqs_dev = reinterpret_cast<const SeqInfo*>(ws + L.seqs_off);
    }
    if (num_slots == 0) return S1_OK;

    pp.slots = slots_dev;
    pp.num_slots = num_slots, pp.H = heads;
    pp.wq = reinterpret_cast<__nv_bfloat16*>(ws + L.wq_off);
    pp.ut = reinterpret_cast<__nv_bfloat16*>(ws + L.ut_off);
    pp.kn = reinterpret_cast<__nv_bfloat16*>(ws + L.kn_off);
    pp.p = reinterpret_cast<__nv_bfloat16*>(ws + L.p_off);
    pp.decay = reinterpret_cast<float*>(ws + L.decay_off);
    pp.status = ctx->status_dev;
    static thread_local int configured_device = -1;
    if (configured_device != ctx->device) {
        S1_CUDA_OK(ctx, cudaFuncSetAttribute(s1_delta_prep_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrepSmem));
        S1_CUDA_OK(ctx, cudaFuncSetAttribute(s1_delta_prep_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrepSmem));
        S1_CUDA_OK(ctx, cudaFuncSetAttribute(s1_delta_prep_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrepSmem));
        S1_CUDA_OK(ctx, cudaFuncSetAttribute(s1_delta_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kScanSmem));
        configured_device = ctx->device;
    }
    const dim3 pgrid((num_slots + 1) / 2, heads);
    if (fused && pp.conv_w) s1_delta_prep_kernel<true, true><<<pgrid, kPrepThreads, kPrepSmem, ctx->stream>>>(pp);
    else if (fused) s1_delta_prep_kernel<true><<<pgrid, kPrepThreads, kPrepSmem, ctx->stream>>>(pp);
    else s1_delta_prep_kernel<false><<<pgrid, kPrepThreads, kPrepSmem, ctx->stream>>>(pp);
    S1_CUDA_OK(ctx, cudaGetLastError());
    ctx->launches += 1;

    const long long hs_rows = static_cast<long long>(heads) * num_slots;
    CUtensorMap tWQ, tUT, tKN, tP;
    int rc = s1_get_tmap(ctx, pp.wq, hs_rows * 128, 128, 128, 128, 64, 2, 128, &tWQ);
    if (rc) return rc;
    rc = s1_get_tmap(ctx, pp.ut, hs_rows * 128, 64, 64, 128, 64, 2, 128, &tUT);
    if (rc) return rc;
    rc = s1_get_tmap(ctx, pp.kn, hs_rows * 64, 128, 128, 64, 64, 2, 128, &tKN);
    if (rc) return rc;
    rc = s1_get_tmap(ctx, pp.p, hs_rows * 64, 64, 64, 64, 64, 2, 128, &tP);
    if (rc) return rc;
    ScanParams sp;
    sp.seqs = seqs_dev;
    sp.slots = pp.slots;
    sp.decay = pp.decay;
    sp.out = out;
    sp.num_slots = num_slots, sp.H = heads;
    sp.status = ctx->status_dev;
    s1_delta_scan_kernel<<<dim3(num_seqs, heads), 160, kScanSmem, ctx->stream>>>(tWQ, tUT, tKN, tP, sp);
    S1_CUDA_OK(ctx, cudaGetLastError());
    ctx->launches += 1;
    return S1_OK;
}

extern "C" int s1_delta_rule_chunked(s1_ctx* ctx, const float* q, const float* k, const float* v, const float* g,
                                     const float* beta, const int32_t* cu_seqlens_host, int num_seqs, int total_tokens,
                                     int heads, int key_dim, int value_dim, float* out, void* workspace,
                                     size_t workspace_bytes) {
    if (!ctx) return S1_EINVAL;
    if (!q || !k || !v || !g || !beta || !out || !workspace)
        return s1_fail(ctx, S1_EINVAL, "s1_delta_rule_chunked: null pointer");
    if (key_dim != kD || value_dim != kD)
        return s1_fail(ctx, S1_EINVAL, "s1_delta_rule_chunked: key_dim and value_dim must be 128 (got %d, %d); use s1_delta_rule", key_dim, value_dim);
    if (num_seqs < 0 || heads < 1 || total_tokens < 0) return s1_fail(ctx, S1_EINVAL, "s1_delta_rule_chunked: bad sizes");
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15u)
        return s1_fail(ctx, S1_EINVAL, "s1_delta_rule_chunked: q, k, v must be 16-byte aligned");
    PrepParams pp = {};
    pp.q = q, pp.k = k, pp.v = v, pp.g = g, pp.beta = beta;
    return run_chunked(ctx, "s1_delta_rule_chunked", pp, false, cu_seqlens_host, num_seqs, total_tokens, heads, out, workspace, workspace_bytes);
}

extern "C" int s1_delta_finish(s1_ctx* ctx, const float* o, const void* z, long long ldz, const void* norm_weight, float eps,
                               int total_tokens, int value_heads, void* y, long long ldy);

extern "C" size_t s1_gated_delta_rule_workspace(int num_seqs, int total_tokens, int value_heads) {
    if (num_seqs < 0 || total_tokens < 0 || value_heads < 1) return 0;
    // the recurrence output o (f32 [T, Hv, 128]) + the chunk workspace
    return align_up(static_cast<size_t>(total_tokens) * value_heads * 128 * 4, 1024) +
           s1_delta_rule_chunked_workspace(num_seqs, total_tokens, value_heads);
}

// Shared body of s1_gated_delta_rule (conv_weight = NULL: `mixed` is the conv output) and s1_gated_delta_rule_conv.
static int gated_delta_rule(s1_ctx* ctx, const char* who, const void* mixed, long long ldm, const void* conv_weight,
                            const int32_t* positions, const void* b_proj, const void* a_proj, long long ldba, const float* dt_bias,
                            const float* neg_exp_a, const void* z, long long ldz, const void* norm_weight, float eps,
                            const int32_t* cu_seqlens_host, int num_seqs, int total_tokens, int key_heads, int value_heads, void* y,
                            long long ldy, void* workspace, size_t workspace_bytes) {
    if (!ctx) return S1_EINVAL;
    if (!mixed || !b_proj || !a_proj || !dt_bias || !neg_exp_a || !z || !norm_weight || !y || !workspace)
        return s1_fail(ctx, S1_EINVAL, "%s: null pointer", who);
    if (key_heads < 1 || value_heads < key_heads || value_heads % key_heads)
        return s1_fail(ctx, S1_EINVAL, "%s: value_heads must be a multiple of key_heads", who);
    const long long width = 2LL * key_heads * 128 + 1LL * value_heads * 128;
    if (ldm < width || (ldm % 8) || ldba < value_heads || (reinterpret_cast<uintptr_t>(mixed) & 15u))
        return s1_fail(ctx, S1_EINVAL, "%s: mixed needs %lld columns per row and 16-byte aligned rows", who, width);
    if (conv_weight && (reinterpret_cast<uintptr_t>(conv_weight) & 15u))
        return s1_fail(ctx, S1_EINVAL, "%s: the conv weight must be 16-byte aligned", who);
    if (reinterpret_cast<uintptr_t>(workspace) & 1023u)
        return s1_fail(ctx, S1_EINVAL, "%s: the workspace must be 1024-byte aligned device memory", who);
    if (workspace_bytes < s1_gated_delta_rule_workspace(num_seqs, total_tokens, value_heads))
        return s1_fail(ctx, S1_EINVAL, "%s: workspace of %zu bytes, %zu needed", who, workspace_bytes,
                       s1_gated_delta_rule_workspace(num_seqs, total_tokens, value_heads));
    if (total_tokens == 0) return S1_OK;
    const size_t obytes = align_up(static_cast<size_t>(total_tokens) * value_heads * 128 * 4, 1024);
    float* o = static_cast<float*>(workspace);
    PrepParams pp = {};
    pp.mixed = static_cast<const __nv_bfloat16*>(mixed), pp.ldm = ldm;
    pp.conv_w = static_cast<const __nv_bfloat16*>(conv_weight), pp.positions = positions;
    pp.bproj = static_cast<const __nv_bfloat16*>(b_proj), pp.aproj = static_cast<const __nv_bfloat16*>(a_proj), pp.ldba = ldba;
    pp.dt_bias = dt_bias, pp.neg_exp_a = neg_exp_a, pp.Hk = key_heads;
    int rc = run_chunked(ctx, who, pp, true, cu_seqlens_host, num_seqs, total_tokens, value_heads, o,
                         static_cast<uint8_t*>(workspace) + obytes, workspace_bytes - obytes);
    if (rc) return rc;
    return s1_delta_finish(ctx, o, z, ldz, norm_weight, eps, total_tokens, value_heads, y, ldy);
}

extern "C" int s1_gated_delta_rule(s1_ctx* ctx, const void* mixed, long long ldm, const void* b_proj, const void* a_proj,
                                   long long ldba, const float* dt_bias, const float* neg_exp_a, const void* z, long long ldz,
                                   const void* norm_weight, float eps, const int32_t* cu_seqlens_host, int num_seqs,
                                   int total_tokens, int key_heads, int value_heads, void* y, long long ldy, void* workspace,
                                   size_t workspace_bytes) {
    return gated_delta_rule(ctx, "s1_gated_delta_rule", mixed, ldm, nullptr, nullptr, b_proj, a_proj, ldba, dt_bias, neg_exp_a, z, ldz,
                            norm_weight, eps, cu_seqlens_host, num_seqs, total_tokens, key_heads, value_heads, y, ldy, workspace,
                            workspace_bytes);
}

extern "C" int s1_gated_delta_rule_conv(s1_ctx* ctx, const void* mixed_before_conv, long long ldm, const void* conv_weight,
                                        const int32_t* positions, const void* b_proj, const void* a_proj, long long ldba,
                                        const float* dt_bias, const float* neg_exp_a, const void* z, long long ldz,
                                        const void* norm_weight, float eps, const int32_t* cu_seqlens_host, int num_seqs,
                                        int total_tokens, int key_heads, int value_heads, void* y, long long ldy, void* workspace,
                                        size_t workspace_bytes) {
    if (ctx && (!conv_weight || !positions)) return s1_fail(ctx, S1_EINVAL, "s1_gated_delta_rule_conv: null pointer");
    return gated_delta_rule(ctx, "s1_gated_delta_rule_conv", mixed_before_conv, ldm, conv_weight, positions, b_proj, a_proj, ldba, dt_bias,
                            neg_exp_a, z, ldz, norm_weight, eps, cu_seqlens_host, num_seqs, total_tokens, key_heads, value_heads, y, ldy,
                            workspace, workspace_bytes);
}

#ifdef S1_MEASURE
extern "C" int s1_measure_read_stamps(long long* out, int n) {
    return cudaMemcpyFromSymbol(out, s1_phase_stamps, sizeof(long long) * (n < 64 ? n : 64)) == cudaSuccess ? 0 : -2;
}
#endif
