// C-ABI entry points: context management and the fused projection (s1_linear).
#include <string.h>

#include <new>

#include "context.h"
#include "gemm_sm100.cuh"

using namespace s1;

// ---------------------------------------------------------------------------------------------- context
extern "C" int s1_device_count(int* out) {
    if (!out) return S1_EINVAL;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) {
        *out = 0;
        return S1_EDEVICE;
    }
    *out = n;
    return S1_OK;
}

extern "C" int s1_ctx_create(int device_ordinal, void* cuda_stream, s1_ctx** out) {
    if (!out) return S1_EINVAL;
    *out = nullptr;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) return S1_EDEVICE;
    if (device_ordinal < 0 || device_ordinal >= n) return S1_EINVAL;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device_ordinal) != cudaSuccess) return S1_ECUDA;
    if (prop.major != 10) return S1_EDEVICE;  // the kernels are sm_100a only; there is no other path
    if (cudaSetDevice(device_ordinal) != cudaSuccess) return S1_ECUDA;

    s1_ctx* ctx = new (std::nothrow) s1_ctx();
    if (!ctx) return S1_ENOMEM;
    ctx->device = device_ordinal;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->stream = static_cast<cudaStream_t>(cuda_stream);  // NULL is CUDA's default stream
    // int[8]: words 0..3 the status record kernels fill when they give up, words 4..5 the projections' tile counters
    if (cudaMalloc(&ctx->status_dev, 8 * sizeof(int)) != cudaSuccess ||
        cudaMemset(ctx->status_dev, 0, 8 * sizeof(int)) != cudaSuccess) {
        delete ctx;
        return S1_ECUDA;
    }
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || !fn ||
        qres != cudaDriverEntryPointSuccess) {
        cudaFree(ctx->status_dev);
        delete ctx;
        return S1_ECUDA;
    }
    ctx->encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled>(fn);
    *out = ctx;
    return S1_OK;
}

extern "C" int s1_ctx_destroy(s1_ctx* ctx) {
    if (!ctx) return S1_EINVAL;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    s1_comm_destroy(ctx);
    if (ctx->status_dev) cudaFree(ctx->status_dev);
    delete ctx;
    return S1_OK;
}

extern "C" const char* s1_last_error(const s1_ctx* ctx) { return ctx ? ctx->err : "null context"; }

extern "C" long long s1_launch_count(const s1_ctx* ctx) { return ctx ? ctx->launches : 0; }

extern "C" int s1_set_option(s1_ctx* ctx, const char* name, long long value) {
    if (!ctx || !name) return S1_EINVAL;
    if (strcmp(name, "gemm_bn") == 0) {
        if (value != 0 && value != 128 && value != 256 && value != 512 && value != 384)
            return s1_fail(ctx, S1_EINVAL, "gemm_bn must be 0, 128, 256, 384 or 512 (got %lld)", value);
        ctx->opt_gemm_bn = static_cast<int>(value);
        return S1_OK;
    }
    if (strcmp(name, "gemm_sms") == 0) {  // SMs the projections may occupy (0 = all): leaves room for a concurrent collective
        if (value < 0 || (value != 0 && value < 2))
            return s1_fail(ctx, S1_EINVAL, "gemm_sms must be 0 (all) or at least 2 (got %lld)", value);
        ctx->opt_gemm_sms = static_cast<int>(value);
        return S1_OK;
    }
    if (strcmp(name, "comm_ctas") == 0) {  // set before s1_comm_init
        if (value < 0 || value > 64) return s1_fail(ctx, S1_EINVAL, "comm_ctas must be between 0 (default) and 64 (got %lld)", value);
        ctx->opt_comm_ctas = static_cast<int>(value);
        return S1_OK;
    }
    if (strcmp(name, "pdl") == 0) {  // programmatic dependent launch of the projections (default on)
        ctx->opt_pdl = value != 0;
        return S1_OK;
    }
    if (strcmp(name, "wait_limit_cycles") == 0) {  // longest single wait inside a projection kernel, in SM clock cycles
        if (value < 1000) return s1_fail(ctx, S1_EINVAL, "wait_limit_cycles must be at least 1000 (got %lld)", value);
        ctx->opt_wait_limit = value;
        return S1_OK;
    }
    if (strcmp(name, "comm_timeout_ms") == 0) {  // deadline of s1_comm_init (0 = wait for ever); set before s1_comm_init
        if (value < 0) return s1_fail(ctx, S1_EINVAL, "comm_timeout_ms must not be negative (got %lld)", value);
        ctx->opt_comm_timeout_ms = value;
        return S1_OK;
    }
    if (strcmp(name, "dynamic_tiles") == 0) {  // projections draw their tiles at run time instead of working through fixed shares
        ctx->opt_dynamic_tiles = value != 0;
        return S1_OK;
    }
    if (strcmp(name, "exchange_wait_ms") == 0) {  // longest the symmetric-memory exchange kernel waits for its peers
        if (value < 1 || value > 600000) return s1_fail(ctx, S1_EINVAL, "exchange_wait_ms must be between 1 and 600000 (got %lld)", value);
        ctx->opt_exchange_wait_ms = value;
        return S1_OK;
    }
#ifdef S1_MEASURE
    if (strcmp(name, "debug") == 0) {
        ctx->opt_debug = static_cast<int>(value);
        return S1_OK;
    }
#endif
    return s1_fail(ctx, S1_EINVAL, "unknown option '%s'", name);
}

extern "C" int s1_sync(s1_ctx* ctx) {
    if (!ctx) return S1_EINVAL;
    S1_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    S1_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    int st[4] = {0, 0, 0, 0};
    S1_CUDA_OK(ctx, cudaMemcpy(st, ctx->status_dev, sizeof(st), cudaMemcpyDeviceToHost));
    if (st[0] != 0) {
        cudaMemset(ctx->status_dev, 0, 8 * sizeof(int));  // the tile counters too: a kernel that gave up may have left them anywhere
        if (st[0] == 101 || st[0] == 102)
            return s1_fail(ctx, S1_EKERNEL, "%s: row %d has index %d outside the table", st[0] == 101 ? "s1_norm gather" : "s1_rope position",
                           st[2], st[3]);
        return s1_fail(ctx, S1_EKERNEL, "kernel gave up on a bounded wait: code %d block %d role %d tile %d", st[0],
                       st[1], st[2], st[3]);
    }
    return S1_OK;
}

// ---------------------------------------------------------------------------------------------- bounded-wait self test
namespace {
// One block whose only wait can never be satisfied: nothing (no copy, no MMA, no other thread) ever arrives on the
// barrier, so the bounded wait every kernel of this library uses runs out after `limit` cycles, the thread records the
// status the way the projection kernels do, and the kernel returns by itself.
__global__ void s1_wait_probe_kernel(int* status, long long limit) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        fence_mbar_init();
    }
    __syncthreads();
    bool ok = true;
    if (threadIdx.x == 0) ok = mbar_wait(smem_u32(&bar), 0, &abort_flag, limit);
    if (!ok && atomicCAS(status, 0, 1) == 0) {
        status[1] = static_cast<int>(blockIdx.x);
        status[2] = 99;  // role: the self test
        status[3] = -1;
    }
}
}  // namespace

extern "C" int s1_selftest_bounded_wait(s1_ctx* ctx) {
    if (!ctx) return S1_EINVAL;
    S1_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    s1_wait_probe_kernel<<<1, 32, 0, ctx->stream>>>(ctx->status_dev, ctx->opt_wait_limit);
    S1_CUDA_OK(ctx, cudaGetLastError());
    ctx->launches += 1;
    return S1_OK;
}

int s1_get_tmap(s1_ctx* ctx, const void* ptr, long long rows, long long cols, long long ld, int box_rows,
                int box_cols, int elem_bytes, int swizzle_bytes, CUtensorMap* out) {
    S1TmapKey key{ptr, rows, cols, ld, box_rows, box_cols + 1024 * swizzle_bytes, elem_bytes};
    auto it = ctx->tmaps.find(key);
    if (it != ctx->tmaps.end()) {
        *out = it->second;
        return S1_OK;
    }
    CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    cuuint64_t gdim[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    cuuint64_t gstr[1] = {static_cast<cuuint64_t>(ld) * elem_bytes};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
    cuuint32_t estr[2] = {1, 1};
    CUtensorMap m;
    CUresult r = ctx->encode(&m, dt, 2, const_cast<void*>(ptr), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                             : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                                   : CU_TENSOR_MAP_SWIZZLE_NONE,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return s1_fail(ctx, S1_ECUDA, "cuTensorMapEncodeTiled failed (%d) ptr=%p rows=%lld cols=%lld ld=%lld box=%dx%d",
                       static_cast<int>(r), ptr, rows, cols, ld, box_rows, box_cols);
    if (ctx->tmaps.size() > 4096) ctx->tmaps.clear();
    ctx->tmaps.emplace(key, m);
    *out = m;
    return S1_OK;
}

// ---------------------------------------------------------------------------------------------- s1_linear
template <int BN, int EPI, int MODE, int CTAS>
static int launch_gemm(s1_ctx* ctx, const CUtensorMap& a, const CUtensorMap& b0, const CUtensorMap& b1,
                       const CUtensorMap& ty, const GemmParams& p) {
    using Cfg = GemmCfg<BN, CTAS>;
    auto kern = s1_gemm_kernel<BN, EPI, MODE, CTAS>;
    // the kernel that draws its tiles at run time exists for the 256 x 256 pair tiles (the large projections a collective runs
    // beside); every other shape keeps its fixed shares whatever the option says
    constexpr bool kHasDyn = (BN == 256 && CTAS == 2);
    if constexpr (kHasDyn) {
        if (p.dynamic_tiles) kern = s1_gemm_kernel<BN, EPI, MODE, CTAS, true>;
    }
    static thread_local int configured_device = -1;
    if (configured_device != ctx->device) {
        const int smem = Cfg::smem_bytes(StoreCfg<BN, EPI, CTAS>::kStagingBytes);
        S1_CUDA_OK(ctx, cudaFuncSetAttribute(s1_gemm_kernel<BN, EPI, MODE, CTAS>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        if constexpr (kHasDyn)
            S1_CUDA_OK(ctx, cudaFuncSetAttribute(s1_gemm_kernel<BN, EPI, MODE, CTAS, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        configured_device = ctx->device;
    }
    const int tiles = p.tiles_m * p.tiles_n;
    const int sms = (ctx->opt_gemm_sms > 0 && ctx->opt_gemm_sms < ctx->sm_count) ? ctx->opt_gemm_sms : ctx->sm_count;
    const int units = sms / CTAS;  // CTAs, or CTA pairs
    const int grid = (tiles < units ? tiles : units) * CTAS;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(gemm_threads<BN, EPI>(), 1, 1);
    cfg.dynamicSmemBytes = Cfg::smem_bytes(StoreCfg<BN, EPI, CTAS>::kStagingBytes);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CTAS;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    // programmatic dependent launch: the set-up of this kernel overlaps the tail of the previous one in the stream
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = ctx->opt_pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    S1_CUDA_OK(ctx, cudaLaunchKernelEx(&cfg, kern, a, b0, b1, ty, p));
    ctx->launches += 1;
    return S1_OK;
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

namespace {
struct RopeArgs {  // rotary embedding fused into the epilogue of a plain projection (s1_linear_rope)
    const float* cos_table;
    const float* sin_table;
    const int32_t* positions;
    int max_positions;
    int rope_cols;  // output columns [0, rope_cols) are 64-column heads to rotate
    bool* fused;    // out: whether the fused kernel ran (otherwise the caller rotates afterwards)
};
}  // namespace

static int linear_impl(s1_ctx* ctx, const s1_linear_desc* lin, const void* x, long long ldx, const void* residual, long long ldr,
                       void* y, long long ldy, int T, const RopeArgs* rope) {
    if (!ctx) return S1_EINVAL;
    if (!lin || !x || !y || !lin->w) return s1_fail(ctx, S1_EINVAL, "s1_linear: null pointer");
    const int epi = lin->epilogue;
    if (epi != S1_EPI_NONE && epi != S1_EPI_GEGLU && epi != S1_EPI_SWIGLU)
        return s1_fail(ctx, S1_EINVAL, "s1_linear: unknown epilogue %d", epi);
    if (T < 1 || lin->N < 1 || lin->K < 1)
        return s1_fail(ctx, S1_EINVAL, "s1_linear: T=%d N=%d K=%d must be positive", T, lin->N, lin->K);
    if (epi == S1_EPI_GEGLU && (lin->N % 2)) return s1_fail(ctx, S1_EINVAL, "s1_linear: GEGLU needs even N");
    if (epi == S1_EPI_SWIGLU && !lin->w_up) return s1_fail(ctx, S1_EINVAL, "s1_linear: SWIGLU needs w_up");
    if (epi != S1_EPI_NONE && (lin->bias || lin->act != S1_ACT_NONE || residual))
        return s1_fail(ctx, S1_EINVAL, "s1_linear: bias / act / residual are not defined behind a gated epilogue");
    if (lin->act < S1_ACT_NONE || lin->act > S1_ACT_GELU)
        return s1_fail(ctx, S1_EINVAL, "s1_linear: unknown act %d", lin->act);
    const int n_out = (epi == S1_EPI_GEGLU) ? lin->N / 2 : lin->N;
    if ((lin->K % 8) || (n_out % 8))
        return s1_fail(ctx, S1_EINVAL, "s1_linear: K=%d and N_out=%d must be multiples of 8", lin->K, n_out);
    if (ldx < lin->K || lin->ldw < lin->K || ldy < n_out || (residual && ldr < n_out) ||
        (lin->w_up && lin->ldw_up < lin->K))
        return s1_fail(ctx, S1_EINVAL, "s1_linear: a leading dimension is smaller than its row");
    if ((ldx % 8) || (lin->ldw % 8) || (ldy % 8) || (residual && (ldr % 8)) || (lin->w_up && (lin->ldw_up % 8)))
        return s1_fail(ctx, S1_EINVAL, "s1_linear: leading dimensions must be multiples of 8 elements (16 bytes)");
    if (!aligned16(x) || !aligned16(lin->w) || !aligned16(y) || !aligned16(residual) || !aligned16(lin->w_up))
        return s1_fail(ctx, S1_EINVAL, "s1_linear: pointers must be 16-byte aligned");
    S1_CUDA_OK(ctx, cudaSetDevice(ctx->device));

    // Tile shape. A CTA pair (256 x 256 per pair) once there is at least a wave of pair-tiles; otherwise one CTA
    // per tile, 128 x 256, or 128 x 128 when that fills the SMs visibly better.
    // "gemm_bn": 0 = auto, 512 = force the pair kernel, 256 / 128 = force the single-CTA kernel of that width.
    const int out_w256 = (epi == S1_EPI_NONE) ? 256 : 128;
    const int n_tiles256 = (n_out + out_w256 - 1) / out_w256;
    auto wave_eff = [&](long long t, int units) {
        const long long waves = (t + units - 1) / units;
        return static_cast<double>(t) / static_cast<double>(waves * units);
    };
    int ctas = 1, bn = 256;
    const long long pair_tiles = static_cast<long long>((T + 2 * kBM - 1) / (2 * kBM)) * n_tiles256;
    const int tiles_m1 = (T + kBM - 1) / kBM;
    if (ctx->opt_gemm_bn == 512 || ctx->opt_gemm_bn == 384 || (ctx->opt_gemm_bn == 0 && pair_tiles >= ctx->sm_count / 2)) {
        ctas = 2;
        // 192-wide pair tiles: a quarter less work per tile at about 0.9 of the cost of a 256-wide one (measured on the N = 768
        // projections: 13.6 against 14.5 us and 17.0 against 18.2 us at T = 8192, where 96 tiles of 256 columns need two waves of
        // the 74 CTA pairs and 128 tiles of 192 columns need two shorter ones; slower at T = 16384 and 32768, where they need
        // a wave more). Taken when the wave count says so, for plain epilogues whose width is a multiple of 192.
        if (epi == S1_EPI_NONE) {
            if (ctx->opt_gemm_bn == 384) {
                bn = 192;
            } else if (ctx->opt_gemm_bn == 0 && !rope && !ctx->opt_dynamic_tiles && n_out % 192 == 0) {
                const long long m2 = (T + 2 * kBM - 1) / (2 * kBM);
                const int sms = (ctx->opt_gemm_sms > 0 && ctx->opt_gemm_sms < ctx->sm_count) ? ctx->opt_gemm_sms : ctx->sm_count;
                const long long pairs = sms / 2;
                const long long waves256 = (m2 * n_tiles256 + pairs - 1) / pairs;
                const long long waves192 = (m2 * (n_out / 192) + pairs - 1) / pairs;
                if (10 * waves256 > 9 * waves192) bn = 192;
            }
        }
    } else if (ctx->opt_gemm_bn == 128 || ctx->opt_gemm_bn == 256) {
        bn = ctx->opt_gemm_bn;
    } else {
        const int out_w128 = out_w256 / 2;
        const long long t256 = static_cast<long long>(tiles_m1) * n_tiles256;
        const long long t128 = static_cast<long long>(tiles_m1) * ((n_out + out_w128 - 1) / out_w128);
        bn = (wave_eff(t128, ctx->sm_count) > wave_eff(t256, ctx->sm_count) + 0.08) ? 128 : 256;
    }
    const int tiles_m = (ctas == 2) ? (T + 2 * kBM - 1) / (2 * kBM) : tiles_m1;
    auto n_tiles_for = [&](int bn_) {
        const int w = (epi == S1_EPI_NONE) ? bn_ : bn_ / 2;
        return (n_out + w - 1) / w;
    };

    GemmParams p{};
    p.M = T;
    p.n_out = n_out;
    p.K = lin->K;
    p.tiles_m = tiles_m;
    p.tiles_n = n_tiles_for(bn);
    p.act = lin->act;
    p.wait_limit = ctx->opt_wait_limit;
#ifdef S1_MEASURE
    p.debug = ctx->opt_debug;
#endif
    p.ldr = ldr;
    p.residual = static_cast<const __nv_bfloat16*>(residual);
    p.bias = static_cast<const __nv_bfloat16*>(lin->bias);
    p.status = ctx->status_dev;
    p.tile_counter = reinterpret_cast<unsigned int*>(ctx->status_dev + 4);
    p.dynamic_tiles = ctx->opt_dynamic_tiles ? 1 : 0;
    p.rope_cos = p.rope_sin = nullptr;
    p.rope_pos = nullptr;
    p.rope_max = p.rope_cols = 0;

    CUtensorMap ta, tb0, tb1, ty;
    int rc = s1_get_tmap(ctx, x, T, lin->K, ldx, kBM, kBK, 2, 128, &ta);
    if (rc) return rc;
    const bool wide_store = (epi == S1_EPI_NONE && bn == 256 && ctas == 2);  // StoreCfg::kWide
    rc = s1_get_tmap(ctx, y, T, n_out, ldy, 32, wide_store ? 64 : 32, 2, wide_store ? 128 : 64, &ty);
    if (rc) return rc;
    rc = s1_get_tmap(ctx, lin->w, lin->N, lin->K, lin->ldw, bn / 2, kBK, 2, 128, &tb0);
    if (rc) return rc;
    if (epi == S1_EPI_SWIGLU) {
        rc = s1_get_tmap(ctx, lin->w_up, lin->N, lin->K, lin->ldw_up, bn / 2, kBK, 2, 128, &tb1);
        if (rc) return rc;
        p.n_tile_stride = bn / 2;
        p.half1_base = 0;
    } else if (epi == S1_EPI_GEGLU) {
        tb1 = tb0;
        p.n_tile_stride = bn / 2;
        p.half1_base = n_out;  // gate rows follow the I activated rows
    } else {
        tb1 = tb0;
        p.n_tile_stride = bn;
        p.half1_base = bn / 2;
    }

    int mode = (residual ? 1 : 0) | ((lin->bias || lin->act != S1_ACT_NONE) ? 2 : 0);
    // residual stream updated in place (y is the residual buffer): no residual reads, the add happens in memory
    if (mode == 1 && residual == y && ldr == ldy) mode = 4;
    if (rope) {
        // the fused form exists for the CTA-pair tile (256 columns = 4 heads per tile, 128 per epilogue warp)
        *rope->fused = (epi == S1_EPI_NONE && mode == 0 && ctas == 2 && bn == 256 && (rope->rope_cols % 128) == 0);
        if (*rope->fused) {
            p.rope_cos = rope->cos_table;
            p.rope_sin = rope->sin_table;
            p.rope_pos = rope->positions;
            p.rope_max = rope->max_positions;
            p.rope_cols = rope->rope_cols;
            return launch_gemm<256, EPI_NONE, 8, 2>(ctx, ta, tb0, tb1, ty, p);
        }
    }
#define S1_LAUNCH(BN_, CTAS_)                                                                            \
    do {                                                                                                 \
        if (epi == S1_EPI_GEGLU) return launch_gemm<BN_, EPI_GEGLU, 0, CTAS_>(ctx, ta, tb0, tb1, ty, p);   \
        if (epi == S1_EPI_SWIGLU) return launch_gemm<BN_, EPI_SWIGLU, 0, CTAS_>(ctx, ta, tb0, tb1, ty, p); \
        switch (mode) {                                                                                  \
            case 0: return launch_gemm<BN_, EPI_NONE, 0, CTAS_>(ctx, ta, tb0, tb1, ty, p);                \
            case 1: return launch_gemm<BN_, EPI_NONE, 1, CTAS_>(ctx, ta, tb0, tb1, ty, p);                \
            case 2: return launch_gemm<BN_, EPI_NONE, 2, CTAS_>(ctx, ta, tb0, tb1, ty, p);                \
            case 4: return launch_gemm<BN_, EPI_NONE, 4, CTAS_>(ctx, ta, tb0, tb1, ty, p);                \
            default: return launch_gemm<BN_, EPI_NONE, 3, CTAS_>(ctx, ta, tb0, tb1, ty, p);               \
        }                                                                                                \
    } while (0)
    if (ctas == 2 && bn == 192) {
        switch (mode) {
            case 0: return launch_gemm<192, EPI_NONE, 0, 2>(ctx, ta, tb0, tb1, ty, p);
            case 1: return launch_gemm<192, EPI_NONE, 1, 2>(ctx, ta, tb0, tb1, ty, p);
            case 2: return launch_gemm<192, EPI_NONE, 2, 2>(ctx, ta, tb0, tb1, ty, p);
            case 4: return launch_gemm<192, EPI_NONE, 4, 2>(ctx, ta, tb0, tb1, ty, p);
            default: return launch_gemm<192, EPI_NONE, 3, 2>(ctx, ta, tb0, tb1, ty, p);
        }
    }
    if (ctas == 2) S1_LAUNCH(256, 2);
    if (bn == 256) S1_LAUNCH(256, 1);
    S1_LAUNCH(128, 1);
#undef S1_LAUNCH
}

extern "C" int s1_linear(s1_ctx* ctx, const s1_linear_desc* lin, const void* x, long long ldx, const void* residual,
                         long long ldr, void* y, long long ldy, int T) {
    return linear_impl(ctx, lin, x, ldx, residual, ldr, y, ldy, T, nullptr);
}

extern "C" int s1_linear_rope(s1_ctx* ctx, const s1_linear_desc* lin, const void* x, long long ldx, void* y, long long ldy, int T,
                              const float* cos_table, const float* sin_table, const int32_t* positions, int max_positions,
                              int rotated_heads) {
    if (!ctx) return S1_EINVAL;
    if (!lin || !cos_table || !sin_table || !positions) return s1_fail(ctx, S1_EINVAL, "s1_linear_rope: null pointer");
    if (lin->epilogue != S1_EPI_NONE || lin->bias || lin->act != S1_ACT_NONE)
        return s1_fail(ctx, S1_EINVAL, "s1_linear_rope: a plain projection only (no bias, activation or gating)");
    if (rotated_heads < 1 || max_positions < 1 || 64LL * rotated_heads > lin->N)
        return s1_fail(ctx, S1_EINVAL, "s1_linear_rope: %d heads of 64 columns do not fit N=%d", rotated_heads, lin->N);
    if ((reinterpret_cast<uintptr_t>(cos_table) | reinterpret_cast<uintptr_t>(sin_table)) & 15u)
        return s1_fail(ctx, S1_EINVAL, "s1_linear_rope: tables must be 16-byte aligned");
    bool fused = false;
    RopeArgs args{cos_table, sin_table, positions, max_positions, 64 * rotated_heads, &fused};
    const int rc = linear_impl(ctx, lin, x, ldx, nullptr, 0, y, ldy, T, &args);
    if (rc != S1_OK || fused) return rc;
    // small token counts and odd head counts run the projection's other tile shapes: rotate in a second pass
    return s1_rope(ctx, y, ldy, cos_table, sin_table, positions, max_positions, T, rotated_heads, 64, 64);
}
