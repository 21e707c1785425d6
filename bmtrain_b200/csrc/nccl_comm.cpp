// NCCL communicator wrapper with a plain C ABI (built into bmtrain_b200/_nccl.so, which links the NCCL library the
// process already uses).
//
// What it adds over calling NCCL directly:
//   * communicators are created NON-BLOCKING (ncclCommInitRankConfig with blocking = 0): every call returns at once and
//     completion / failure is observed with ncclCommGetAsyncError, so a peer that never shows up cannot wedge the caller
//     inside the library; initialisation and every collective poll with a time limit;
//   * an optional watchdog thread per communicator polls the asynchronous error state and aborts the communicator
//     (ncclCommAbort) when NCCL reports a failure, so that kernels waiting on a dead peer are released;
//   * all entry points take raw device pointers, element counts and a stream handle.
// The reference's wrapper (csrc/include/nccl.hpp:8-188) creates blocking communicators, has no error polling and no abort.
#include <nccl.h>

#include <atomic>
#include <chrono>
#include <cstring>
#include <mutex>
#include <thread>

namespace {

struct Comm {
    ncclComm_t comm = nullptr;
    int nranks = 0, rank = 0;
    std::atomic<int> async_error{0};     // last ncclResult_t seen by the watchdog (0 = none)
    std::atomic<bool> aborted{false}, stop{false};
    std::thread watchdog;
    std::mutex mu;                       // serialises abort / destroy against the watchdog
};

using Clock = std::chrono::steady_clock;

// Polls until the communicator leaves ncclInProgress; returns the final state, or -1000 when `timeout_s` passed.
int settle(Comm* c, double timeout_s) {
    const auto t0 = Clock::now();
    for (;;) {
        ncclResult_t st = ncclSuccess;
        const ncclResult_t q = ncclCommGetAsyncError(c->comm, &st);
        if (q != ncclSuccess) return (int)q;
        if (st != ncclInProgress) return (int)st;
        if (std::chrono::duration<double>(Clock::now() - t0).count() > timeout_s) return -1000;
        std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
}

// A call on a non-blocking communicator may answer ncclInProgress: that is not an error.
inline int launched(ncclResult_t r) { return (r == ncclSuccess || r == ncclInProgress) ? 0 : (int)r; }

}  // namespace

extern "C" {

int bmt_nccl_version(void) {
    int v = 0;
    return ncclGetVersion(&v) == ncclSuccess ? v : -1;
}

int bmt_nccl_unique_id_size(void) { return (int)sizeof(ncclUniqueId); }

int bmt_nccl_get_unique_id(void* out) {
    ncclUniqueId id;
    const ncclResult_t r = ncclGetUniqueId(&id);
    if (r != ncclSuccess) return (int)r;
    memcpy(out, &id, sizeof(id));
    return 0;
}

// Creates rank `rank` of an `nranks` communicator (the CUDA device must be current).  Non-blocking; waits up to
// `timeout_s` for the bootstrap to finish.  Returns 0 and the handle, an NCCL error code, or -1000 on time-out (the
// half-built communicator is aborted).
int bmt_nccl_comm_init(const void* unique_id, int nranks, int rank, double timeout_s, void** out) {
    ncclUniqueId id;
    memcpy(&id, unique_id, sizeof(id));
    ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
    cfg.blocking = 0;
    Comm* c = new Comm();
    c->nranks = nranks;
    c->rank = rank;
    const ncclResult_t r = ncclCommInitRankConfig(&c->comm, nranks, id, rank, &cfg);
    if (r != ncclSuccess && r != ncclInProgress) { delete c; return (int)r; }
    const int st = settle(c, timeout_s);
    if (st != 0) {
        if (c->comm) ncclCommAbort(c->comm);
        delete c;
        return st;
    }
    *out = c;
    return 0;
}

int bmt_nccl_comm_count(void* h) { return ((Comm*)h)->nranks; }
int bmt_nccl_comm_rank(void* h) { return ((Comm*)h)->rank; }

// Current asynchronous state: 0 fine, 7 (ncclInProgress) work pending, other NCCL codes = failure; -2000 after an abort.
int bmt_nccl_async_error(void* h) {
    Comm* c = (Comm*)h;
    if (c->aborted.load()) return -2000;
    const int seen = c->async_error.load();
    if (seen != 0) return seen;
    ncclResult_t st = ncclSuccess;
    const ncclResult_t q = ncclCommGetAsyncError(c->comm, &st);
    return q != ncclSuccess ? (int)q : (int)st;
}

// Blocks (polling) until queued NCCL calls have been issued or failed; -1000 on time-out.
int bmt_nccl_wait_issued(void* h, double timeout_s) {
    Comm* c = (Comm*)h;
    if (c->aborted.load()) return -2000;
    return settle(c, timeout_s);
}

int bmt_nccl_abort(void* h) {
    Comm* c = (Comm*)h;
    std::lock_guard<std::mutex> lk(c->mu);
    if (c->aborted.exchange(true)) return 0;
    return (int)ncclCommAbort(c->comm);
}

// Starts a thread that polls the asynchronous error state every `poll_ms` and aborts the communicator on failure.
int bmt_nccl_watchdog_start(void* h, int poll_ms) {
    Comm* c = (Comm*)h;
    if (c->watchdog.joinable()) return 0;
    c->watchdog = std::thread([c, poll_ms] {
        while (!c->stop.load()) {
            std::this_thread::sleep_for(std::chrono::milliseconds(poll_ms > 0 ? poll_ms : 100));
            std::lock_guard<std::mutex> lk(c->mu);
            if (c->stop.load() || c->aborted.load()) break;
            ncclResult_t st = ncclSuccess;
            if (ncclCommGetAsyncError(c->comm, &st) != ncclSuccess) continue;
            if (st != ncclSuccess && st != ncclInProgress) {
                c->async_error.store((int)st);
                c->aborted.store(true);
                ncclCommAbort(c->comm);
                break;
            }
        }
    });
    return 0;
}

int bmt_nccl_comm_destroy(void* h) {
    Comm* c = (Comm*)h;
    c->stop.store(true);
    if (c->watchdog.joinable()) c->watchdog.join();
    int rc = 0;
    if (!c->aborted.load()) {
        // finalize flushes outstanding work; on a non-blocking communicator it completes asynchronously
        ncclResult_t r = ncclCommFinalize(c->comm);
        if (r == ncclSuccess || r == ncclInProgress) settle(c, 30.0);
        r = ncclCommDestroy(c->comm);
        rc = launched(r);
    }
    delete c;
    return rc;
}

// ---- collectives: dtype / op are ncclDataType_t / ncclRedOp_t numbers, counts are in elements -----------------------
int bmt_nccl_all_reduce(void* h, const void* src, void* dst, int64_t count, int dtype, int op, void* stream) {
    return launched(ncclAllReduce(src, dst, (size_t)count, (ncclDataType_t)dtype, (ncclRedOp_t)op, ((Comm*)h)->comm, (cudaStream_t)stream));
}
int bmt_nccl_all_gather(void* h, const void* src, void* dst, int64_t send_count, int dtype, void* stream) {
    return launched(ncclAllGather(src, dst, (size_t)send_count, (ncclDataType_t)dtype, ((Comm*)h)->comm, (cudaStream_t)stream));
}
int bmt_nccl_reduce_scatter(void* h, const void* src, void* dst, int64_t recv_count, int dtype, int op, void* stream) {
    return launched(ncclReduceScatter(src, dst, (size_t)recv_count, (ncclDataType_t)dtype, (ncclRedOp_t)op, ((Comm*)h)->comm, (cudaStream_t)stream));
}
int bmt_nccl_broadcast(void* h, const void* src, void* dst, int64_t count, int dtype, int root, void* stream) {
    return launched(ncclBroadcast(src, dst, (size_t)count, (ncclDataType_t)dtype, root, ((Comm*)h)->comm, (cudaStream_t)stream));
}
int bmt_nccl_reduce(void* h, const void* src, void* dst, int64_t count, int dtype, int op, int root, void* stream) {
    return launched(ncclReduce(src, dst, (size_t)count, (ncclDataType_t)dtype, (ncclRedOp_t)op, root, ((Comm*)h)->comm, (cudaStream_t)stream));
}
int bmt_nccl_send(void* h, const void* src, int64_t count, int dtype, int peer, void* stream) {
    return launched(ncclSend(src, (size_t)count, (ncclDataType_t)dtype, peer, ((Comm*)h)->comm, (cudaStream_t)stream));
}
int bmt_nccl_recv(void* h, void* dst, int64_t count, int dtype, int peer, void* stream) {
    return launched(ncclRecv(dst, (size_t)count, (ncclDataType_t)dtype, peer, ((Comm*)h)->comm, (cudaStream_t)stream));
}
int bmt_nccl_group_start(void) { return launched(ncclGroupStart()); }
int bmt_nccl_group_end(void) { return launched(ncclGroupEnd()); }
const char* bmt_nccl_error_string(int code) {
    if (code == -1000) return "timed out waiting for NCCL";
    if (code == -2000) return "communicator was aborted";
    return ncclGetErrorString((ncclResult_t)code);
}

}  // extern "C"
