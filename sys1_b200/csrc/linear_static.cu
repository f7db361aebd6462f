// s1_linear_static: the fused projection for callers that must not allocate device memory.
//
// Who needs it: a host whose device memory belongs to another allocator (sys1's Rust side hands every buffer
// out of candle's / cudarc's pool and wants no foreign cudaMalloc in its process), and code that runs while a
// stream is being captured or inside a latency-critical serving loop, where cudaMalloc is either illegal or an
// implicit device-wide synchronisation. The regular path needs an `s1_ctx`, and creating one allocates the
// kernel's status block with cudaMalloc. Here that block lives in a file-scope `__device__` array instead, so
// the whole call - set-up included - allocates nothing: no cudaMalloc / cudaFree, no context object, no cache of
// tensor maps (they are encoded on the stack for every call).
//
// The price: the array is one per GPU and shared by every call, so two calls whose kernels overlap on the GPU
// (different streams, different threads) race on it; run calls of this entry point on one stream at a time.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>
#include <stdarg.h>
#include <stdio.h>

#include <atomic>
#include <mutex>

#include "../../include/sys1_b200.h"
#include "gemm_sm100.cuh"

using namespace s1;

// The scratch itself: 256 bytes per GPU that loads the library, held until the process exits.
// Words 0..3 are the status record the GEMM kernel fills when one of its bounded waits runs out
// ({code, block, role, tile}), words 4..5 the counters its CTAs draw their tiles from; the rest is spare. Device code may name the array directly; host code may not -
// on the host this symbol is only a handle, the real address comes from cudaGetSymbolAddress (below).
#define S1_STATIC_SCRATCH_BYTES 256
static __device__ __align__(256) int s1_static_scratch[S1_STATIC_SCRATCH_BYTES / sizeof(int)];

namespace {

constexpr int kMaxDevices = 64;
struct PerDevice {
    // set (release) once every other field is final; read (acquire) by callers without the mutex
    std::atomic<bool> ready{false};
    int* scratch = nullptr;  // device address of s1_static_scratch on this GPU
    int sm_count = 0;
    PFN_cuTensorMapEncodeTiled encode = nullptr;
};
PerDevice g_dev[kMaxDevices];  // static storage: nothing here is heap-allocated
std::mutex g_setup_mutex;

int fail(char* err, size_t err_len, int code, const char* fmt, ...) {
    if (err && err_len) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(err, err_len, fmt, ap);
        va_end(ap);
    }
    return code;
}

template <int EPI, int MODE, int CTAS>
cudaError_t set_smem_attr() {
    return cudaFuncSetAttribute(s1_gemm_kernel<256, EPI, MODE, CTAS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                GemmCfg<256, CTAS>::smem_bytes(StoreCfg<256, EPI, CTAS>::kStagingBytes));
}

// Once per device, with that device current. Not to be run for the first time under stream capture.
int setup_device(int device, char* err, size_t err_len) {
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    PerDevice& d = g_dev[device];
    if (d.ready.load(std::memory_order_acquire)) return S1_OK;
    cudaDeviceProp prop;
    cudaError_t e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) return fail(err, err_len, S1_ECUDA, "cudaGetDeviceProperties: %s", cudaGetErrorString(e));
    if (prop.major != 10) return fail(err, err_len, S1_EDEVICE, "device %d is not compute capability 10.x", device);
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, s1_static_scratch);  // the device address; the bare symbol is a host-side stand-in
    if (e != cudaSuccess || !ptr)
        return fail(err, err_len, S1_ECUDA, "cudaGetSymbolAddress(s1_static_scratch): %s", cudaGetErrorString(e));
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || !fn || q != cudaDriverEntryPointSuccess)
        return fail(err, err_len, S1_ECUDA, "cuTensorMapEncodeTiled is not available");
    const cudaError_t attrs[] = {
        set_smem_attr<EPI_NONE, 0, 1>(),  set_smem_attr<EPI_NONE, 1, 1>(),  set_smem_attr<EPI_NONE, 4, 1>(),
        set_smem_attr<EPI_GEGLU, 0, 1>(), set_smem_attr<EPI_SWIGLU, 0, 1>(),
        set_smem_attr<EPI_NONE, 0, 2>(),  set_smem_attr<EPI_NONE, 1, 2>(),  set_smem_attr<EPI_NONE, 4, 2>(),
        set_smem_attr<EPI_GEGLU, 0, 2>(), set_smem_attr<EPI_SWIGLU, 0, 2>(),
    };
    for (cudaError_t a : attrs)
        if (a != cudaSuccess) return fail(err, err_len, S1_ECUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(a));
    d.scratch = static_cast<int*>(ptr);
    d.sm_count = prop.multiProcessorCount;
    d.encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled>(fn);
    d.ready.store(true, std::memory_order_release);
    return S1_OK;
}

bool encode_map(const PerDevice& d, CUtensorMap* out, const void* ptr, long long rows, long long cols, long long ld,
                int box_rows, int box_cols, bool swizzle128) {
    cuuint64_t gdim[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    cuuint64_t gstr[1] = {static_cast<cuuint64_t>(ld) * 2};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
    cuuint32_t estr[2] = {1, 1};
    return d.encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstr, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int EPI, int MODE, int CTAS>
cudaError_t launch(const PerDevice& d, cudaStream_t stream, const CUtensorMap& a, const CUtensorMap& b0,
                   const CUtensorMap& b1, const CUtensorMap& ty, const GemmParams& p) {
    const int tiles = p.tiles_m * p.tiles_n;
    const int units = d.sm_count / CTAS;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((tiles < units ? tiles : units) * CTAS, 1, 1);
    cfg.blockDim = dim3(gemm_threads<256, EPI>(), 1, 1);
    cfg.dynamicSmemBytes = GemmCfg<256, CTAS>::smem_bytes(StoreCfg<256, EPI, CTAS>::kStagingBytes);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CTAS;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, s1_gemm_kernel<256, EPI, MODE, CTAS>, a, b0, b1, ty, p);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Makes a device current for the length of one call and restores the one the caller had.
struct DeviceGuard {
    int previous = -1;
    bool switched = false;
    cudaError_t enter(int device) {
        cudaError_t e = cudaGetDevice(&previous);
        if (e != cudaSuccess) return e;
        if (previous == device) return cudaSuccess;
        e = cudaSetDevice(device);
        switched = (e == cudaSuccess);
        return e;
    }
    ~DeviceGuard() {
        if (switched) cudaSetDevice(previous);
    }
};

}  // namespace

extern "C" int s1_linear_static(int device_ordinal, void* cuda_stream, const s1_linear_desc* lin, const void* x,
                                long long ldx, const void* residual, long long ldr, void* y, long long ldy, int T,
                                int wait, char* err, size_t err_len) {
    if (err && err_len) err[0] = 0;
    if (device_ordinal < 0 || device_ordinal >= kMaxDevices) return fail(err, err_len, S1_EINVAL, "bad device ordinal %d", device_ordinal);
    if (!lin || !x || !y || !lin->w) return fail(err, err_len, S1_EINVAL, "s1_linear_static: null pointer");
    const int epi = lin->epilogue;
    if (epi != S1_EPI_NONE && epi != S1_EPI_GEGLU && epi != S1_EPI_SWIGLU)
        return fail(err, err_len, S1_EINVAL, "s1_linear_static: unknown epilogue %d", epi);
    if (lin->bias || lin->act != S1_ACT_NONE)
        return fail(err, err_len, S1_EINVAL, "s1_linear_static: bias / activation are only offered by s1_linear");
    if (T < 1 || lin->N < 1 || lin->K < 1) return fail(err, err_len, S1_EINVAL, "s1_linear_static: T, N, K must be positive");
    if (T > S1_STATIC_MAX_TOKENS || lin->N > S1_STATIC_MAX_FEATURES || lin->K > S1_STATIC_MAX_FEATURES)
        return fail(err, err_len, S1_ELIMIT,
                    "s1_linear_static: T=%d N=%d K=%d exceeds the supported maximum (T <= %d, N and K <= %d); "
                    "use s1_linear for larger problems",
                    T, lin->N, lin->K, S1_STATIC_MAX_TOKENS, S1_STATIC_MAX_FEATURES);
    if (epi == S1_EPI_GEGLU && (lin->N % 2)) return fail(err, err_len, S1_EINVAL, "s1_linear_static: GEGLU needs even N");
    if (epi == S1_EPI_SWIGLU && !lin->w_up) return fail(err, err_len, S1_EINVAL, "s1_linear_static: SWIGLU needs w_up");
    if (epi != S1_EPI_NONE && residual)
        return fail(err, err_len, S1_EINVAL, "s1_linear_static: no residual behind a gated epilogue");
    const int n_out = (epi == S1_EPI_GEGLU) ? lin->N / 2 : lin->N;
    if ((lin->K % 8) || (n_out % 8)) return fail(err, err_len, S1_EINVAL, "s1_linear_static: K and N_out must be multiples of 8");
    if (ldx < lin->K || lin->ldw < lin->K || ldy < n_out || (residual && ldr < n_out) || (lin->w_up && lin->ldw_up < lin->K))
        return fail(err, err_len, S1_EINVAL, "s1_linear_static: a leading dimension is smaller than its row");
    if ((ldx % 8) || (lin->ldw % 8) || (ldy % 8) || (residual && (ldr % 8)) || (lin->w_up && (lin->ldw_up % 8)))
        return fail(err, err_len, S1_EINVAL, "s1_linear_static: leading dimensions must be multiples of 8 elements");
    if (!aligned16(x) || !aligned16(lin->w) || !aligned16(y) || !aligned16(residual) || !aligned16(lin->w_up))
        return fail(err, err_len, S1_EINVAL, "s1_linear_static: pointers must be 16-byte aligned");

    // The call runs with `device_ordinal` current and puts the caller's device back before it returns.
    DeviceGuard guard;
    cudaError_t e = guard.enter(device_ordinal);
    if (e != cudaSuccess) return fail(err, err_len, S1_ECUDA, "cudaSetDevice: %s", cudaGetErrorString(e));
    if (!g_dev[device_ordinal].ready.load(std::memory_order_acquire)) {
        const int rc = setup_device(device_ordinal, err, err_len);
        if (rc != S1_OK) return rc;
    }
    const PerDevice& d = g_dev[device_ordinal];
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);

    const int out_w = (epi == S1_EPI_NONE) ? 256 : 128;
    const int tiles_n = (n_out + out_w - 1) / out_w;
    const long long pair_tiles = static_cast<long long>((T + 2 * kBM - 1) / (2 * kBM)) * tiles_n;
    const int ctas = (pair_tiles >= d.sm_count / 2) ? 2 : 1;

    GemmParams p{};
    p.M = T;
    p.n_out = n_out;
    p.K = lin->K;
    p.tiles_m = (T + ctas * kBM - 1) / (ctas * kBM);
    p.tiles_n = tiles_n;
    p.act = ACT_NONE;
    p.wait_limit = kWaitLimitCycles;
    p.ldr = ldr;
    p.residual = static_cast<const __nv_bfloat16*>(residual);
    p.bias = nullptr;
    p.status = d.scratch;  // the device address obtained at set-up, never the host-side symbol
    p.tile_counter = reinterpret_cast<unsigned int*>(d.scratch + 4);
    p.dynamic_tiles = 0;
    if (epi == S1_EPI_SWIGLU) {
        p.n_tile_stride = 128;
        p.half1_base = 0;
    } else if (epi == S1_EPI_GEGLU) {
        p.n_tile_stride = 128;
        p.half1_base = n_out;
    } else {
        p.n_tile_stride = 256;
        p.half1_base = 128;
    }

    CUtensorMap ta, tb0, tb1, ty;  // on the stack, re-encoded every call: no cache, no heap
    if (!encode_map(d, &ta, x, T, lin->K, ldx, kBM, kBK, true) || !encode_map(d, &ty, y, T, n_out, ldy, 32, (epi == S1_EPI_NONE && ctas == 2) ? 64 : 32, epi == S1_EPI_NONE && ctas == 2) ||
        !encode_map(d, &tb0, lin->w, lin->N, lin->K, lin->ldw, 128, kBK, true))
        return fail(err, err_len, S1_ECUDA, "s1_linear_static: cuTensorMapEncodeTiled failed");
    tb1 = tb0;
    if (epi == S1_EPI_SWIGLU && !encode_map(d, &tb1, lin->w_up, lin->N, lin->K, lin->ldw_up, 128, kBK, true))
        return fail(err, err_len, S1_ECUDA, "s1_linear_static: cuTensorMapEncodeTiled failed");

    // the array keeps whatever the last call left in it: the status record must start at zero
    e = cudaMemsetAsync(d.scratch, 0, 8 * sizeof(int), stream);  // and the two tile counters behind it
    if (e != cudaSuccess) return fail(err, err_len, S1_ECUDA, "cudaMemsetAsync: %s", cudaGetErrorString(e));

    int mode = residual ? 1 : 0;
    if (mode == 1 && residual == y && ldr == ldy) mode = 4;
#define S1_STATIC_LAUNCH(CTAS_)                                                                      \
    (epi == S1_EPI_GEGLU    ? launch<EPI_GEGLU, 0, CTAS_>(d, stream, ta, tb0, tb1, ty, p)            \
     : epi == S1_EPI_SWIGLU ? launch<EPI_SWIGLU, 0, CTAS_>(d, stream, ta, tb0, tb1, ty, p)           \
     : mode == 0            ? launch<EPI_NONE, 0, CTAS_>(d, stream, ta, tb0, tb1, ty, p)             \
     : mode == 1            ? launch<EPI_NONE, 1, CTAS_>(d, stream, ta, tb0, tb1, ty, p)             \
                            : launch<EPI_NONE, 4, CTAS_>(d, stream, ta, tb0, tb1, ty, p))
    e = (ctas == 2) ? S1_STATIC_LAUNCH(2) : S1_STATIC_LAUNCH(1);
#undef S1_STATIC_LAUNCH
    if (e != cudaSuccess) return fail(err, err_len, S1_ECUDA, "kernel launch: %s", cudaGetErrorString(e));

    if (wait) {
        e = cudaStreamSynchronize(stream);
        if (e != cudaSuccess) return fail(err, err_len, S1_ECUDA, "cudaStreamSynchronize: %s", cudaGetErrorString(e));
        int st[4] = {0, 0, 0, 0};
        e = cudaMemcpy(st, d.scratch, sizeof(st), cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) return fail(err, err_len, S1_ECUDA, "cudaMemcpy(status): %s", cudaGetErrorString(e));
        if (st[0] != 0)
            return fail(err, err_len, S1_EKERNEL, "kernel gave up on a bounded wait: block %d role %d tile %d", st[1], st[2], st[3]);
    }
    return S1_OK;
}
