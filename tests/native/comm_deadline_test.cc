// Drives s1::comm_init_with_deadline (sys1_b200/csrc/comm_init.h) with stand-in NCCL entry points, on the host only:
// no GPU, no NCCL. Each case prints one line "name: ok" or "name: FAILED ..."; the exit code is the number of failures.
// Built and run by tests/test_comm_deadline.py (g++, a few seconds).
#include <string.h>

#include <chrono>

#include "comm_init.h"

namespace {

int g_polls = 0, g_ready_after = -1, g_aborted = 0, g_destroyed = 0, g_blocking_seen = -1, g_max_ctas_seen = -1;
ncclResult_t g_final_state = ncclSuccess;
int g_fake_comm_storage;

ncclResult_t fake_init_config(ncclComm_t* comm, int, ncclUniqueId, int, ncclConfig_t* cfg) {
    g_blocking_seen = cfg->blocking;
    g_max_ctas_seen = cfg->maxCTAs;
    *comm = reinterpret_cast<ncclComm_t>(&g_fake_comm_storage);
    return cfg->blocking == 0 ? ncclInProgress : ncclSuccess;
}
ncclResult_t fake_init(ncclComm_t* comm, int, ncclUniqueId, int) {
    *comm = reinterpret_cast<ncclComm_t>(&g_fake_comm_storage);
    return ncclSuccess;
}
// the communicator becomes ready after g_ready_after polls; -1: a rank never joins, it stays in progress for ever
ncclResult_t fake_async_error(ncclComm_t, ncclResult_t* state) {
    ++g_polls;
    *state = (g_ready_after >= 0 && g_polls > g_ready_after) ? g_final_state : ncclInProgress;
    return ncclSuccess;
}
ncclResult_t fake_abort(ncclComm_t) { ++g_aborted; return ncclSuccess; }
ncclResult_t fake_destroy(ncclComm_t) { ++g_destroyed; return ncclSuccess; }
const char* fake_error_string(ncclResult_t r) { return r == ncclSystemError ? "system error" : "other"; }

s1::NcclApi fake_api(bool with_nonblocking) {
    s1::NcclApi api;
    api.handle = &g_fake_comm_storage;
    api.CommInitRank = fake_init;
    api.CommDestroy = fake_destroy;
    api.GetErrorString = fake_error_string;
    if (with_nonblocking) {
        api.CommInitRankConfig = fake_init_config;
        api.CommGetAsyncError = fake_async_error;
        api.CommAbort = fake_abort;
    }
    return api;
}

void reset(int ready_after, ncclResult_t final_state = ncclSuccess) {
    g_polls = g_aborted = g_destroyed = 0;
    g_blocking_seen = g_max_ctas_seen = -1;
    g_ready_after = ready_after;
    g_final_state = final_state;
}

int failures = 0;
void report(const char* name, bool ok, const char* detail = "") {
    printf("%s: %s %s\n", name, ok ? "ok" : "FAILED", ok ? "" : detail);
    if (!ok) ++failures;
}

}  // namespace

int main() {
    ncclUniqueId uid;
    memset(&uid, 0, sizeof(uid));
    char err[256];
    ncclComm_t comm;
    bool blocking;

    // 1. a rank never joins: the call gives up at the deadline, aborts the half-built communicator, reports S1_ETIMEOUT
    {
        reset(-1);
        s1::NcclApi api = fake_api(true);
        const auto t0 = std::chrono::steady_clock::now();
        const int rc = s1::comm_init_with_deadline(api, uid, 0, 2, 0, 150, &comm, &blocking, err, sizeof(err));
        const long long ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
        report("never_joins_times_out", rc == S1_ETIMEOUT && comm == nullptr && g_aborted == 1 && ms >= 150 && ms < 5000 &&
                                            g_blocking_seen == 0 && strstr(err, "rank 0 of 2") != nullptr, err);
    }
    // 2. the other ranks arrive after a few polls: success, nothing aborted, the communicator is marked non-blocking
    {
        reset(5);
        s1::NcclApi api = fake_api(true);
        const int rc = s1::comm_init_with_deadline(api, uid, 1, 2, 8, 2000, &comm, &blocking, err, sizeof(err));
        report("joins_late_succeeds", rc == S1_OK && comm != nullptr && g_aborted == 0 && !blocking && g_max_ctas_seen == 8 && g_polls == 6);
    }
    // 3. NCCL reports a failure while connecting: S1_ECUDA with NCCL's message, communicator aborted
    {
        reset(2, ncclSystemError);
        s1::NcclApi api = fake_api(true);
        const int rc = s1::comm_init_with_deadline(api, uid, 0, 2, 0, 2000, &comm, &blocking, err, sizeof(err));
        report("connect_failure_is_reported", rc == S1_ECUDA && comm == nullptr && g_aborted == 1 && strstr(err, "system error") != nullptr, err);
    }
    // 4. timeout 0, or an NCCL without the non-blocking entry points: the plain blocking call
    {
        reset(-1);
        s1::NcclApi api = fake_api(true);
        int rc = s1::comm_init_with_deadline(api, uid, 0, 2, 0, 0, &comm, &blocking, err, sizeof(err));
        bool ok = rc == S1_OK && blocking && g_polls == 0;
        s1::NcclApi old_api = fake_api(false);
        rc = s1::comm_init_with_deadline(old_api, uid, 0, 2, 4, 1000, &comm, &blocking, err, sizeof(err));
        report("no_deadline_is_blocking", ok && rc == S1_OK && blocking && g_polls == 0);
    }
    // 5. a collective call that answers "in progress" on a non-blocking communicator is polled out, with the same deadline
    {
        reset(3);
        s1::NcclApi api = fake_api(true);
        int rc = s1::comm_wait_enqueued(api, reinterpret_cast<ncclComm_t>(&g_fake_comm_storage), 1000, err, sizeof(err));
        bool ok = rc == S1_OK && g_polls == 4;
        reset(-1);
        rc = s1::comm_wait_enqueued(api, reinterpret_cast<ncclComm_t>(&g_fake_comm_storage), 50, err, sizeof(err));
        report("collective_in_progress_is_polled", ok && rc == S1_ETIMEOUT && g_aborted == 0);
    }
    return failures;
}
