// Host-side context shared by the C-ABI entry points: stream, device status word,
// tensor-map encoder entry point and a small cache of encoded maps.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cudaTypedefs.h>
#include <stdarg.h>
#include <stdio.h>

#include <unordered_map>
#include <vector>

#include "../../include/sys1_b200.h"

struct S1TmapKey {
    const void* ptr;
    long long rows, cols, ld;
    int box_rows, box_cols, elem_bytes;
    bool operator==(const S1TmapKey& o) const {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows &&
               box_cols == o.box_cols && elem_bytes == o.elem_bytes;
    }
};
struct S1TmapKeyHash {
    size_t operator()(const S1TmapKey& k) const {
        size_t h = reinterpret_cast<size_t>(k.ptr);
        auto mix = [&h](long long v) { h ^= static_cast<size_t>(v) + 0x9e3779b97f4a7c15ULL + (h << 6) + (h >> 2); };
        mix(k.rows);
        mix(k.cols);
        mix(k.ld);
        mix(k.box_rows);
        mix(k.box_cols);
        mix(k.elem_bytes);
        return h;
    }
};

// Tables of one packed batch that the attention and delta-rule kernels walk (s1_batch_plan): built once per batch on the
// host, copied to the device once, reused by every layer. The record below is the host's note of where they lie.
struct S1QBlock {      // one 128-query block of one sequence
    int seq_start;     // first token of the sequence
    int seq_len;
    int qb;            // query block inside the sequence
    int pad;
};
struct S1ChunkSlot {   // one 64-token chunk of the delta rule
    int tok_start;     // first token (row of the packed batch)
    int len;           // valid tokens in the chunk (1..64)
};
struct S1SeqChunks {
    int first_slot;
    int num_chunks;
};
struct S1BatchPlan {
    const unsigned char* dev = nullptr;
    int num_seqs = 0, total_tokens = 0;
    int num_blocks = 0;   // 128-query blocks (both attentions)
    int num_slots = 0;    // 64-token chunks
    size_t attn_global_off = 0, attn_local_off = 0, gqa_off = 0, slots_off = 0, seqs_off = 0;
};

struct s1_ctx {
    int device = 0;
    int sm_count = 0;
    cudaStream_t stream = nullptr;
    int* status_dev = nullptr;  // int[4], written by kernels on failure
    long long launches = 0;
    int opt_gemm_bn = 0;
    int opt_debug = 0;                          // only read by builds with -DS1_MEASURE (timing ablations)
    long long opt_wait_limit = 2000000000LL;    // SM clock cycles a wait inside a projection kernel may take (~1 s)
    long long opt_comm_timeout_ms = 120000;     // deadline of s1_comm_init; 0 = none
    long long opt_exchange_wait_ms = 10000;     // longest the symmetric-memory exchange kernel waits for its peers
    int opt_gemm_sms = 0;  // 0 = all SMs
    int opt_comm_ctas = 0;  // blocks the collective may use (0 = the library's default); read by s1_comm_init
    bool opt_dynamic_tiles = false;  // projections draw tiles from a counter at run time ("dynamic_tiles")
    bool opt_pdl = true;   // launch the projections with programmatic stream serialization
    PFN_cuTensorMapEncodeTiled encode = nullptr;
    std::unordered_map<S1TmapKey, CUtensorMap, S1TmapKeyHash> tmaps;
    std::vector<unsigned char> host_scratch;  // host staging for small tables copied to the device
    std::vector<S1BatchPlan> plans;           // plans built on this context (a few: one per batch in flight)
    int plan_in_use = -1;                     // index into `plans`, or -1
    // the plan in use if it describes this batch, else null
    const S1BatchPlan* active_plan(int num_seqs, int total_tokens) const {
        if (plan_in_use < 0 || plan_in_use >= static_cast<int>(plans.size())) return nullptr;
        const S1BatchPlan& p = plans[plan_in_use];
        return (p.num_seqs == num_seqs && p.total_tokens == total_tokens) ? &p : nullptr;
    }
    void* comm = nullptr;                     // ncclComm_t once s1_comm_init has run
    cudaStream_t comm_stream = nullptr;
    cudaEvent_t comm_ready = nullptr, comm_done = nullptr;
    static constexpr int kCommTickets = 64;
    cudaEvent_t comm_ticket[kCommTickets] = {};  // completion of the all-reduce with sequence number n sits in slot n % 64
    long long comm_issued = 0;                // all-reduces issued so far (the last one's ticket)
    // symmetric-memory exchange (s1_exchange_register): sums of buffers inside [xchg_local, xchg_local + xchg_bytes) run as
    // this library's own multimem kernel instead of the NCCL call
    unsigned char* xchg_local = nullptr;
    unsigned char* xchg_mc = nullptr;
    size_t xchg_bytes = 0;
    void* xchg_flags[16] = {};
    int xchg_rank = 0, xchg_size = 0;
    unsigned int xchg_epoch = 1;
    int comm_rank = 0, comm_size = 0;
    bool comm_pending = false;
    bool comm_blocking = true;                // false: created with a deadline (non-blocking NCCL communicator)
    char err[512] = {0};
};

inline int s1_fail(s1_ctx* ctx, int code, const char* fmt, ...) {
    if (ctx) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(ctx->err, sizeof(ctx->err), fmt, ap);
        va_end(ap);
    }
    return code;
}

// An SM changes its split between L1 and shared memory only while it is empty, and the projections need nearly all of it
// as shared memory. A kernel whose blocks sit beside the projections' CTAs (the exchange kernel) asks for the same split,
// so that an SM it reached first does not have to drain before a projection CTA can join. (The streaming kernels keep the
// default split: with the small L1 that goes with it they ran 10 to 50 % slower.) The hint is given once per kernel and device.
template <typename Kernel>
inline void s1_keep_projection_split(Kernel kernel) {
    cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, static_cast<int>(cudaSharedmemCarveoutMaxShared));
}
#define S1_KEEP_PROJECTION_SPLIT(kernel)                                          \
    do {                                                                          \
        static std::atomic<unsigned long long> told{0}; /* one bit per device */    \
        int dev_ = 0;                                                             \
        cudaGetDevice(&dev_);                                                     \
        const unsigned long long bit_ = 1ull << (dev_ & 63);                      \
        if (!(told.load(std::memory_order_relaxed) & bit_)) {                     \
            s1_keep_projection_split(kernel);                                     \
            told.fetch_or(bit_, std::memory_order_relaxed);                       \
        }                                                                         \
    } while (0)

#define S1_CUDA_OK(ctx, call)                                                                        \
    do {                                                                                             \
        cudaError_t e__ = (call);                                                                    \
        if (e__ != cudaSuccess)                                                                      \
            return s1_fail((ctx), S1_ECUDA, "%s failed: %s", #call, cudaGetErrorString(e__));         \
    } while (0)

// Encodes (or fetches from the cache) a 2-D tiled tensor map over a row-major matrix whose rows are `ld`
// elements apart: dim0 = cols (contiguous), dim1 = rows. swizzle_bytes is 0, 64 or 128.
// Blocks the exchange kernel may use at most (the flag arrays hold one slot per block and rank).
#define S1_EXCHANGE_MAX_BLOCKS 64
int s1_exchange_launch(s1_ctx* ctx, void* buf, size_t count, cudaStream_t stream);

int s1_get_tmap(s1_ctx* ctx, const void* ptr, long long rows, long long cols, long long ld, int box_rows,
                int box_cols, int elem_bytes, int swizzle_bytes, CUtensorMap* out);
