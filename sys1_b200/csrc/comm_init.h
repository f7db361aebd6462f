// Communicator creation with a host-side deadline: a rank that never joins must not block the others for ever.
// Host-only code (no CUDA calls), so that the deadline logic can be driven on a CPU-only machine with a stand-in
// table of NCCL entry points (tests/native/comm_deadline_test.cc does that).
//
// NCCL is created non-blocking (`ncclConfig_t::blocking = 0`): ncclCommInitRankConfig returns at once and the
// communicator's state is polled with ncclCommGetAsyncError until it leaves ncclInProgress or the deadline passes;
// on expiry the half-built communicator is torn down with ncclCommAbort and the caller gets S1_ETIMEOUT.
// A non-blocking communicator may also answer ncclInProgress to a collective call; `comm_wait_enqueued` polls that
// out the same way before the caller records its events.
#pragma once
#include <nccl.h>
#include <stdio.h>

#include <chrono>
#include <thread>

#include "../../include/sys1_b200.h"

namespace s1 {

struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*) = nullptr;  // optional
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;                            // optional
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;                                                   // optional
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    const char* why = nullptr;
    bool can_deadline() const { return CommInitRankConfig && CommGetAsyncError && CommAbort; }
};

// Polls the communicator until its pending operation has completed. S1_OK, S1_ETIMEOUT (state still in progress at
// the deadline; the communicator is left as it is) or S1_ECUDA (NCCL reported a failure).
inline int comm_wait_enqueued(const NcclApi& api, ncclComm_t comm, long long timeout_ms, char* err, size_t err_len) {
    using clock = std::chrono::steady_clock;
    const auto start = clock::now();
    for (;;) {
        ncclResult_t state = ncclSuccess;
        const ncclResult_t rc = api.CommGetAsyncError(comm, &state);
        if (rc != ncclSuccess) state = rc;
        if (state == ncclSuccess) return S1_OK;
        if (state != ncclInProgress) {
            if (err && err_len) snprintf(err, err_len, "NCCL reported: %s", api.GetErrorString ? api.GetErrorString(state) : "error");
            return S1_ECUDA;
        }
        if (timeout_ms > 0 &&
            std::chrono::duration_cast<std::chrono::milliseconds>(clock::now() - start).count() >= timeout_ms) {
            if (err && err_len) snprintf(err, err_len, "still in progress after %lld ms", timeout_ms);
            return S1_ETIMEOUT;
        }
        std::this_thread::sleep_for(std::chrono::milliseconds(1));
    }
}

// Creates the communicator of `rank` among `size` ranks. `timeout_ms` > 0 bounds the wait for the other ranks;
// 0 (or an NCCL without the non-blocking entry points) waits for as long as NCCL does. `max_ctas` > 0 bounds the
// blocks the collectives may use. `*blocking_out` tells whether later collective calls return only once enqueued.
inline int comm_init_with_deadline(const NcclApi& api, const ncclUniqueId& uid, int rank, int size, int max_ctas,
                                   long long timeout_ms, ncclComm_t* out, bool* blocking_out, char* err, size_t err_len) {
    *out = nullptr;
    ncclComm_t comm = nullptr;
    const bool deadline = timeout_ms > 0 && api.can_deadline();
    *blocking_out = !deadline;
    ncclResult_t rc;
    if (deadline || (max_ctas > 0 && api.CommInitRankConfig)) {
        ncclConfig_t config = NCCL_CONFIG_INITIALIZER;
        if (max_ctas > 0) config.maxCTAs = max_ctas;
        if (deadline) config.blocking = 0;
        rc = api.CommInitRankConfig(&comm, size, uid, rank, &config);
    } else {
        rc = api.CommInitRank(&comm, size, uid, rank);
    }
    if (rc != ncclSuccess && !(deadline && rc == ncclInProgress)) {
        if (err && err_len) snprintf(err, err_len, "ncclCommInitRank failed: %s", api.GetErrorString ? api.GetErrorString(rc) : "error");
        if (comm && api.CommAbort) api.CommAbort(comm);
        return S1_ECUDA;
    }
    if (deadline) {
        char why[160] = {0};
        const int st = comm_wait_enqueued(api, comm, timeout_ms, why, sizeof(why));
        if (st != S1_OK) {
            api.CommAbort(comm);  // frees what the half-built communicator holds; the other ranks time out likewise
            if (err && err_len)
                snprintf(err, err_len, "s1_comm_init: rank %d of %d: communicator not ready (%s); aborted", rank, size, why);
            return st;
        }
    }
    *out = comm;
    return S1_OK;
}

}  // namespace s1
