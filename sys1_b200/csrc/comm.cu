// The exchange step of tensor parallelism: an in-place bf16 sum over the ranks after a row-parallel projection
// (o_proj, out_proj, down_proj of the large hybrid model), on NCCL over NVLink. The reference has no multi-GPU
// path at all (`device::load` opens GPU 0 only, src/device.rs:43-56); this is the one collective the sharded
// projection path needs.
//
// NCCL is looked up at run time (dlopen of libnccl.so.2: in a PyTorch process that is the copy PyTorch has
// already loaded), so the library has no link-time dependency on it and single-GPU users never touch it.
// All-reduces run on a communication stream of the context's own, ordered after the work already queued on the
// context's stream; s1_allreduce_wait orders the context's stream after them. Issued slab by slab, the sum of one
// slab of rows travels while the projection of the next slab computes.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>
#include <stdio.h>
#include <string.h>

#include <mutex>

#include "sys1_b200.h"
#include "context.h"
#include "comm_init.h"

namespace {

using s1::NcclApi;

void load_nccl(NcclApi& api) {
    for (const char* name : {"libnccl.so.2", "libnccl.so"}) {
        api.handle = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
        if (api.handle) break;
    }
    if (!api.handle) {
        api.why = "libnccl.so.2 not found";
        return;
    }
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(dlsym(api.handle, "ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(dlsym(api.handle, "ncclCommInitRank"));
    api.CommInitRankConfig = reinterpret_cast<decltype(api.CommInitRankConfig)>(dlsym(api.handle, "ncclCommInitRankConfig"));
    api.CommGetAsyncError = reinterpret_cast<decltype(api.CommGetAsyncError)>(dlsym(api.handle, "ncclCommGetAsyncError"));
    api.CommAbort = reinterpret_cast<decltype(api.CommAbort)>(dlsym(api.handle, "ncclCommAbort"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(api.handle, "ncclCommDestroy"));
    api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(dlsym(api.handle, "ncclAllReduce"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(dlsym(api.handle, "ncclGetErrorString"));
    if (!api.GetUniqueId || !api.CommInitRank || !api.CommDestroy || !api.AllReduce || !api.GetErrorString) {
        api.why = "libnccl.so.2 lacks an expected symbol";
        api.handle = nullptr;
    }
}

NcclApi* nccl_api() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] { load_nccl(api); });
    return &api;
}

static_assert(sizeof(ncclUniqueId) == S1_COMM_ID_BYTES, "communicator id size");

}  // namespace

extern "C" int s1_comm_unique_id(void* id_out, char* err, size_t err_len) {
    auto say = [&](const char* msg) {
        if (err && err_len) snprintf(err, err_len, "%s", msg);
    };
    if (!id_out) {
        say("s1_comm_unique_id: null pointer");
        return S1_EINVAL;
    }
    NcclApi* api = nccl_api();
    if (!api->handle) {
        say(api->why);
        return S1_EDEVICE;
    }
    ncclUniqueId id;
    const ncclResult_t rc = api->GetUniqueId(&id);
    if (rc != ncclSuccess) {
        say(api->GetErrorString(rc));
        return S1_ECUDA;
    }
    memcpy(id_out, &id, sizeof(id));
    return S1_OK;
}

extern "C" int s1_comm_init(s1_ctx* ctx, const void* id, int rank, int size) {
    if (!ctx) return S1_EINVAL;
    if (!id || size < 1 || rank < 0 || rank >= size) return s1_fail(ctx, S1_EINVAL, "s1_comm_init: bad rank %d of %d", rank, size);
    if (ctx->comm) return s1_fail(ctx, S1_EINVAL, "s1_comm_init: the context already has a communicator");
    NcclApi* api = nccl_api();
    if (!api->handle) return s1_fail(ctx, S1_EDEVICE, "s1_comm_init: %s", api->why);
    S1_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    ncclUniqueId uid;
    memcpy(&uid, id, sizeof(uid));
    ncclComm_t comm = nullptr;
    bool blocking = true;
    // a bounded number of blocks for the collective ("comm_ctas"), so that it fits on the SMs the projections leave
    // free ("gemm_sms"); a deadline ("comm_timeout_ms") so that a rank that never joins does not block this one for ever
    const int st = s1::comm_init_with_deadline(*api, uid, rank, size, ctx->opt_comm_ctas, ctx->opt_comm_timeout_ms, &comm,
                                               &blocking, ctx->err, sizeof(ctx->err));
    if (st != S1_OK) return st;
    ctx->comm_blocking = blocking;
    int prio_low = 0, prio_high = 0;  // the collective's blocks go first when SMs free up
    cudaDeviceGetStreamPriorityRange(&prio_low, &prio_high);
    cudaError_t e = cudaSuccess;
    if (!ctx->comm_stream) {  // (a context that has already summed symmetric buffers has its stream and events)
        e = cudaStreamCreateWithPriority(&ctx->comm_stream, cudaStreamNonBlocking, prio_high);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ctx->comm_ready, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ctx->comm_done, cudaEventDisableTiming);
        for (int i = 0; i < s1_ctx::kCommTickets && e == cudaSuccess; ++i) e = cudaEventCreateWithFlags(&ctx->comm_ticket[i], cudaEventDisableTiming);
    }
    if (e != cudaSuccess) {
        api->CommDestroy(comm);
        return s1_fail(ctx, S1_ECUDA, "s1_comm_init: %s", cudaGetErrorString(e));
    }
    ctx->comm = comm;
    ctx->comm_rank = rank;
    ctx->comm_size = size;
    ctx->comm_pending = false;
    return S1_OK;
}

extern "C" int s1_comm_destroy(s1_ctx* ctx) {
    if (!ctx) return S1_EINVAL;
    if (!ctx->comm && !ctx->comm_stream) return S1_OK;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->comm_stream);
    if (ctx->comm) nccl_api()->CommDestroy(static_cast<ncclComm_t>(ctx->comm));
    cudaEventDestroy(ctx->comm_ready);
    cudaEventDestroy(ctx->comm_done);
    for (int i = 0; i < s1_ctx::kCommTickets; ++i)
        if (ctx->comm_ticket[i]) cudaEventDestroy(ctx->comm_ticket[i]), ctx->comm_ticket[i] = nullptr;
    cudaStreamDestroy(ctx->comm_stream);
    ctx->comm = nullptr;
    ctx->comm_stream = nullptr;
    ctx->comm_size = 0;
    return S1_OK;
}

extern "C" int s1_allreduce_bf16(s1_ctx* ctx, void* buf, size_t count) {
    if (!ctx) return S1_EINVAL;
    auto* b8 = static_cast<unsigned char*>(buf);
    const bool own = ctx->xchg_size > 1 && b8 >= ctx->xchg_local && b8 + 2 * count <= ctx->xchg_local + ctx->xchg_bytes;
    if (!ctx->comm && !own) return s1_fail(ctx, S1_EINVAL, "s1_allreduce_bf16: the context has no communicator (s1_comm_init)");
    if (!buf && count) return s1_fail(ctx, S1_EINVAL, "s1_allreduce_bf16: null pointer");
    if (count == 0) return S1_OK;
    S1_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    if (!ctx->comm_stream) {  // a context that only ever sums symmetric buffers has no NCCL communicator
        int prio_low = 0, prio_high = 0;
        cudaDeviceGetStreamPriorityRange(&prio_low, &prio_high);
        S1_CUDA_OK(ctx, cudaStreamCreateWithPriority(&ctx->comm_stream, cudaStreamNonBlocking, prio_high));
        S1_CUDA_OK(ctx, cudaEventCreateWithFlags(&ctx->comm_ready, cudaEventDisableTiming));
        S1_CUDA_OK(ctx, cudaEventCreateWithFlags(&ctx->comm_done, cudaEventDisableTiming));
        for (int i = 0; i < s1_ctx::kCommTickets; ++i) S1_CUDA_OK(ctx, cudaEventCreateWithFlags(&ctx->comm_ticket[i], cudaEventDisableTiming));
    }
    S1_CUDA_OK(ctx, cudaEventRecord(ctx->comm_ready, ctx->stream));
    S1_CUDA_OK(ctx, cudaStreamWaitEvent(ctx->comm_stream, ctx->comm_ready, 0));
    if (own) {
        // a buffer in registered symmetric memory: this library's own kernel, reduction inside the switch
        const int rc = s1_exchange_launch(ctx, buf, count, ctx->comm_stream);
        if (rc != S1_OK) return rc;
    } else {
        NcclApi* api = nccl_api();
        const ncclResult_t rc = api->AllReduce(buf, buf, count, ncclBfloat16, ncclSum, static_cast<ncclComm_t>(ctx->comm), ctx->comm_stream);
        if (rc == ncclInProgress && !ctx->comm_blocking) {
            // a communicator created with a deadline is non-blocking: the call is on the stream once its state says so
            char why[160] = {0};
            const int st = s1::comm_wait_enqueued(*api, static_cast<ncclComm_t>(ctx->comm), ctx->opt_comm_timeout_ms, why, sizeof(why));
            if (st != S1_OK) return s1_fail(ctx, st, "ncclAllReduce: %s", why);
        } else if (rc != ncclSuccess) {
            return s1_fail(ctx, S1_ECUDA, "ncclAllReduce failed: %s", api->GetErrorString(rc));
        }
    }
    S1_CUDA_OK(ctx, cudaEventRecord(ctx->comm_done, ctx->comm_stream));
    ctx->comm_issued += 1;
    S1_CUDA_OK(ctx, cudaEventRecord(ctx->comm_ticket[ctx->comm_issued % s1_ctx::kCommTickets], ctx->comm_stream));
    ctx->comm_pending = true;
    return S1_OK;
}

extern "C" long long s1_allreduce_ticket(const s1_ctx* ctx) { return ctx ? ctx->comm_issued : 0; }

extern "C" int s1_allreduce_wait_ticket(s1_ctx* ctx, long long ticket) {
    if (!ctx) return S1_EINVAL;
    if (!ctx->comm_stream) return s1_fail(ctx, S1_EINVAL, "s1_allreduce_wait_ticket: no all-reduce was ever issued on this context");
    if (ticket < 1 || ticket > ctx->comm_issued)
        return s1_fail(ctx, S1_EINVAL, "s1_allreduce_wait_ticket: ticket %lld was never issued (last: %lld)", ticket, ctx->comm_issued);
    S1_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    // a ticket older than the ring has been overwritten by a later all-reduce of the same (in-order) stream: waiting for
    // that later one covers it
    const long long t = (ctx->comm_issued - ticket >= s1_ctx::kCommTickets) ? ctx->comm_issued : ticket;
    S1_CUDA_OK(ctx, cudaStreamWaitEvent(ctx->stream, ctx->comm_ticket[t % s1_ctx::kCommTickets], 0));
    return S1_OK;
}

extern "C" int s1_allreduce_wait(s1_ctx* ctx) {
    if (!ctx) return S1_EINVAL;
    if (!ctx->comm_pending) return S1_OK;
    S1_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    S1_CUDA_OK(ctx, cudaStreamWaitEvent(ctx->stream, ctx->comm_done, 0));
    ctx->comm_pending = false;
    return S1_OK;
}
