// The sum over ranks of a row-parallel projection's partial outputs as one kernel of this library, over NVLink with the
// reduction done inside the NVSwitch (multimem): an alternative to the NCCL call behind s1_allreduce_bf16 for buffers that
// live in symmetric memory (the same virtual range mapped on every rank, plus a multicast mapping of it).
//
// Rank r owns the r-th slice of the buffer. Per 16 bytes of its slice it issues one `multimem.ld_reduce` (the switch
// fetches that location from every GPU, adds in f32 and returns the bf16 sum) and one `multimem.st` (the switch writes the
// sum into every GPU's copy). Per GPU that is (1 + 1 / ranks) buffers of NVLink traffic in each direction, whatever the
// number of ranks, and a handful of SMs: the projections of the next micro-batch keep the rest. Every rank ends with
// bit-identical values. The blocks are few and fat (1024 threads, 8 reductions in flight each): a projection CTA needs nearly
// all of an SM's shared memory, so an SM that holds a block of this kernel is lost to the projection beside it either way.
//
// Two flag exchanges bracket the data phase (every rank's partial is complete before anyone reduces; every rank's
// stores have landed before anyone reads): block b of rank r writes the call's epoch into slot (b, r) of every peer's flag
// array with a release store through the peer pointer, then polls its own slots. Every poll loop is bounded; a loop that runs
// out records a status the host reads (s1_sync -> S1_EKERNEL) and the kernel returns. No TMA, no cluster multicast loads:
// peer memory is touched only by multimem instructions and by the 4-byte flag stores.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "context.h"

namespace {

constexpr int kMaxRanks = 16;
constexpr int kThreads = 1024;  // few, fat blocks: an SM that holds one is lost to the projections' CTAs for as long as it runs
constexpr int kUnroll = 8;      // independent 16-byte reductions a thread keeps in flight

struct ExchangeParams {
    uint4* mc;                    // multicast address of the first 16-byte unit to reduce
    long long units;              // 16-byte units in the whole range
    uint32_t* peer_flags[kMaxRanks];  // flag array of every rank (peer pointers; [rank] is this GPU's own)
    int rank, size;
    uint32_t epoch;               // this call's first epoch value (the second flag exchange uses epoch + 1)
    unsigned long long wait_ns;   // longest a rank waits for its peers at one meeting point
    int* status;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// All ranks' block `blockIdx.x` meet: thread r < size tells peer r "rank `rank` reached `epoch`" and waits for peer r's word.
// Flags only grow (epochs are issued in order), so "at least epoch" is the test. Returns false if a peer never showed up.
// (The outcome travels through the barrier itself; the kernel uses no shared memory.)
__device__ __forceinline__ bool meet(const ExchangeParams& p, uint32_t epoch) {
    int timed_out = 0;
    __syncthreads();
    if (threadIdx.x < p.size) {
        const int peer = threadIdx.x;
        st_release_sys(p.peer_flags[peer] + blockIdx.x * kMaxRanks + p.rank, epoch);
        const uint32_t* mine = p.peer_flags[p.rank] + blockIdx.x * kMaxRanks + peer;
        const unsigned long long start = global_timer_ns();
        int polls = 0;
        while (static_cast<int32_t>(ld_acquire_sys(mine) - epoch) < 0) {
            if ((++polls & 63) == 0 && global_timer_ns() - start > p.wait_ns) {
                timed_out = 1;
                break;
            }
        }
    }
    return __syncthreads_or(timed_out) == 0;
}

__global__ void __launch_bounds__(kThreads, 1) s1_exchange_allreduce_kernel(const ExchangeParams p) {
    if (!meet(p, p.epoch)) {
        if (threadIdx.x == 0 && atomicCAS(p.status, 0, 6) == 0) p.status[1] = blockIdx.x, p.status[2] = 61, p.status[3] = p.rank;
        return;
    }
    // this rank's slice, split over the blocks; kUnroll independent 16-byte reductions in flight per thread
    const long long per_rank = (p.units + p.size - 1) / p.size;
    const long long lo = per_rank * p.rank, hi = (lo + per_rank < p.units) ? lo + per_rank : p.units;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long u = lo + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; u < hi; u += kUnroll * stride) {
        uint4 v[kUnroll];
#pragma unroll
        for (int k = 0; k < kUnroll; ++k) {
            const long long uu = u + k * stride;
            if (uu < hi)
                asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                             : "=r"(v[k].x), "=r"(v[k].y), "=r"(v[k].z), "=r"(v[k].w)
                             : "l"(p.mc + uu)
                             : "memory");
        }
#pragma unroll
        for (int k = 0; k < kUnroll; ++k) {
            const long long uu = u + k * stride;
            if (uu < hi)
                asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p.mc + uu), "r"(v[k].x), "r"(v[k].y),
                             "r"(v[k].z), "r"(v[k].w)
                             : "memory");
        }
    }
    __threadfence_system();  // this thread's stores are ordered before the flag the block raises next
    if (!meet(p, p.epoch + 1)) {
        if (threadIdx.x == 0 && atomicCAS(p.status, 0, 6) == 0) p.status[1] = blockIdx.x, p.status[2] = 62, p.status[3] = p.rank;
    }
}

}  // namespace

extern "C" int s1_exchange_register(s1_ctx* ctx, int rank, int size, void* local_base, void* multicast_base, size_t bytes,
                                    void* const* flag_arrays_host, size_t flag_bytes) {
    if (!ctx) return S1_EINVAL;
    if (size == 0) {  // forget the registration: sums go back to the communicator path
        ctx->xchg_local = ctx->xchg_mc = nullptr;
        ctx->xchg_bytes = 0;
        ctx->xchg_size = 0;
        return S1_OK;
    }
    if (size < 2 || size > kMaxRanks || rank < 0 || rank >= size)
        return s1_fail(ctx, S1_EINVAL, "s1_exchange_register: rank %d of %d (2 to %d ranks)", rank, size, kMaxRanks);
    if (!local_base || !multicast_base || !flag_arrays_host || bytes < 16)
        return s1_fail(ctx, S1_EINVAL, "s1_exchange_register: null pointer");
    if ((reinterpret_cast<uintptr_t>(local_base) | reinterpret_cast<uintptr_t>(multicast_base)) & 15u)
        return s1_fail(ctx, S1_EINVAL, "s1_exchange_register: the buffer must be 16-byte aligned");
    if (flag_bytes < sizeof(uint32_t) * kMaxRanks * S1_EXCHANGE_MAX_BLOCKS)
        return s1_fail(ctx, S1_EINVAL, "s1_exchange_register: flag arrays of %zu bytes, %zu needed", flag_bytes,
                       sizeof(uint32_t) * kMaxRanks * S1_EXCHANGE_MAX_BLOCKS);
    for (int r = 0; r < size; ++r)
        if (!flag_arrays_host[r]) return s1_fail(ctx, S1_EINVAL, "s1_exchange_register: null flag array of rank %d", r);
    ctx->xchg_local = static_cast<unsigned char*>(local_base);
    ctx->xchg_mc = static_cast<unsigned char*>(multicast_base);
    ctx->xchg_bytes = bytes;
    for (int r = 0; r < size; ++r) ctx->xchg_flags[r] = flag_arrays_host[r];
    ctx->xchg_rank = rank, ctx->xchg_size = size;
    ctx->xchg_epoch = 1;
    return S1_OK;
}

// Called by s1_allreduce_bf16 (comm.cu) for a buffer inside the registered range; enqueues on `stream`.
int s1_exchange_launch(s1_ctx* ctx, void* buf, size_t count, cudaStream_t stream) {
    const size_t off = static_cast<unsigned char*>(buf) - ctx->xchg_local;
    if ((off & 15u) || (count % 8)) return s1_fail(ctx, S1_EINVAL, "s1_allreduce_bf16: symmetric buffers are summed in 16-byte units");
    ExchangeParams p = {};
    p.mc = reinterpret_cast<uint4*>(ctx->xchg_mc + off);
    p.units = static_cast<long long>(count / 8);
    for (int r = 0; r < ctx->xchg_size; ++r) p.peer_flags[r] = static_cast<uint32_t*>(ctx->xchg_flags[r]);
    p.rank = ctx->xchg_rank, p.size = ctx->xchg_size;
    p.epoch = ctx->xchg_epoch;
    ctx->xchg_epoch += 2;
    p.status = ctx->status_dev;
    p.wait_ns = static_cast<unsigned long long>(ctx->opt_exchange_wait_ms) * 1000000ull;
    // a rank reduces 1 / size of the buffer: fewer ranks, more blocks (8 for four ranks and up, 16 for two)
    int blocks = ctx->opt_comm_ctas > 0 ? ctx->opt_comm_ctas : (32 / ctx->xchg_size > 8 ? 32 / ctx->xchg_size : 8);
    if (blocks > S1_EXCHANGE_MAX_BLOCKS) blocks = S1_EXCHANGE_MAX_BLOCKS;
    S1_KEEP_PROJECTION_SPLIT(s1_exchange_allreduce_kernel);  // or its blocks would keep the projections' CTAs off their SMs
    s1_exchange_allreduce_kernel<<<blocks, kThreads, 0, stream>>>(p);
    S1_CUDA_OK(ctx, cudaGetLastError());
    ctx->launches += 1;
    return S1_OK;
}
