// Library-wide bookkeeping: launch counter and device probe.
#include <cuda.h>

#include <atomic>
#include <condition_variable>
#include <deque>
#include <mutex>
#include <thread>
#include <unordered_map>
#include <vector>

#include "api.h"
#include "common.cuh"

static std::atomic<int64_t> g_launches{0};

extern "C" void bmt_count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
extern "C" int64_t bmt_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

// 1 when the current device is a compute-capability 10.x part (tcgen05 / TMEM present).
extern "C" int bmt_device_is_sm100(void) {
    int dev = 0, major = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return 0;
    return major == 10 ? 1 : 0;
}

// ---------------------------------------------------------------------------------------------------------------
// Asynchronous offloaded Adam.  The training thread submits batches and returns to launching the next forward pass; one
// worker thread of this library runs them in order (gradient-copy event -> host Adam on the thread pool of the CPU
// library -> upload), and consumers of a parameter wait for the ticket of the batch that updates it.  Nothing here
// touches the interpreter, so the worker needs no lock of it.
namespace {

// The worker thread adopts the CUDA context that is current on the submitting thread (driver API, so that it does not
// matter which copy of the runtime library created it).
typedef CUresult (*CtxGetFn)(CUcontext*);
typedef CUresult (*CtxSetFn)(CUcontext);
void* driver_fn(const char* name) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) return nullptr;
    return fn;
}

struct Batch {
    int64_t ticket;
    CUcontext ctx;
    std::vector<BmtOffloadJob> jobs;
    BmtAdamCpuExFn fn;       // nullptr: uploads only
    cudaStream_t stream;
    cudaEvent_t uploaded;    // recorded on `stream` behind the batch's last upload
    int device;
};

struct Worker {
    std::mutex mu;
    std::condition_variable cv_work, cv_done;
    std::deque<Batch> queue;
    std::unordered_map<int64_t, std::pair<cudaEvent_t, int>> finished;   // ticket -> (event, error)
    int64_t next_ticket = 1;
    int64_t in_flight = 0;   // ticket the worker is running right now (0: none)
    bool started = false;
    std::vector<cudaEvent_t> spare_events;

    // under `mu`: the batch is still queued or being run
    bool pending(int64_t ticket) const {
        if (ticket == in_flight) return true;
        for (const Batch& b : queue)
            if (b.ticket == ticket) return true;
        return false;
    }

    void run() {
        int device = -1;
        CUcontext current = nullptr;
        CtxSetFn set_ctx = (CtxSetFn)driver_fn("cuCtxSetCurrent");
        for (;;) {
            Batch b;
            {
                std::unique_lock<std::mutex> lk(mu);
                cv_work.wait(lk, [&] { return !queue.empty(); });
                b = std::move(queue.front());
                queue.pop_front();
                in_flight = b.ticket;
            }
            // error word: (stage << 16) | CUDA error; stage 1 context, 2 gradient event, 3 upload, 4 completion event
            int err = 0;
            if (b.device != device || b.ctx != current) {
                if (b.ctx && set_ctx) {
                    const CUresult r = set_ctx(b.ctx);
                    if (r != CUDA_SUCCESS) err = (1 << 16) | (int)r;
                } else {
                    const cudaError_t e = cudaSetDevice(b.device);
                    if (e != cudaSuccess) err = (1 << 16) | (int)e;
                }
                device = b.device;
                current = b.ctx;
                cudaGetLastError();
            }
            for (const BmtOffloadJob& j : b.jobs) {
                if (j.n <= 0 || err) continue;
                if (b.fn) {
                    if (j.grad_ready) {
                        const cudaError_t e = cudaEventSynchronize((cudaEvent_t)j.grad_ready);
                        if (e != cudaSuccess) { err = (2 << 16) | (int)e; break; }
                    }
                    b.fn(j.n, j.p32, j.m, j.v, j.p32_out, j.m_out, j.v_out, j.p16_host, j.g16_host, j.beta1, j.beta2, j.eps, j.lr,
                         j.scale, j.wd, j.bc1, j.bc2, j.bf16);
                }
                if (j.upload) {
                    const cudaError_t e = cudaMemcpyAsync(j.p_dev, j.p16_host, (size_t)j.n * 2, cudaMemcpyHostToDevice, b.stream);
                    if (e != cudaSuccess) { err = (3 << 16) | (int)e; break; }
                }
            }
            const cudaError_t e = cudaEventRecord(b.uploaded, b.stream);
            if (e != cudaSuccess && err == 0) err = (4 << 16) | (int)e;
            {
                std::lock_guard<std::mutex> lk(mu);
                finished[b.ticket] = {b.uploaded, err};
                in_flight = 0;
            }
            cv_done.notify_all();
        }
    }
};

Worker& worker() {
    static Worker* w = new Worker();   // never destroyed: the thread may still be parked on it at process exit
    return *w;
}

int64_t submit_batch(const BmtOffloadJob* jobs, int n, BmtAdamCpuExFn fn, void* h2d_stream) {
    Worker& w = worker();
    Batch b;
    b.jobs.assign(jobs, jobs + n);
    b.fn = fn;
    b.stream = (cudaStream_t)h2d_stream;
    if (cudaGetDevice(&b.device) != cudaSuccess) return -1;
    b.ctx = nullptr;
    static CtxGetFn get_ctx = (CtxGetFn)driver_fn("cuCtxGetCurrent");
    if (get_ctx) get_ctx(&b.ctx);
    {
        std::lock_guard<std::mutex> lk(w.mu);
        if (!w.spare_events.empty()) { b.uploaded = w.spare_events.back(); w.spare_events.pop_back(); }
        else b.uploaded = nullptr;
    }
    if (!b.uploaded) {
        const cudaError_t e = cudaEventCreateWithFlags(&b.uploaded, cudaEventDisableTiming);
        if (e != cudaSuccess) return -(int64_t)e;
    }
    std::lock_guard<std::mutex> lk(w.mu);
    b.ticket = w.next_ticket++;
    const int64_t ticket = b.ticket;
    w.queue.push_back(std::move(b));
    if (!w.started) {
        w.started = true;
        std::thread([&w] { w.run(); }).detach();
    }
    w.cv_work.notify_one();
    return ticket;
}

}  // namespace

extern "C" int64_t bmt_offload_submit(const BmtOffloadJob* jobs, int n, BmtAdamCpuExFn fn, void* h2d_stream) {
    if (!fn || n < 0) return -1;
    return submit_batch(jobs, n, fn, h2d_stream);
}

extern "C" int64_t bmt_offload_submit_uploads(const BmtOffloadJob* jobs, int n, void* h2d_stream) {
    if (n < 0) return -1;
    return submit_batch(jobs, n, nullptr, h2d_stream);
}

extern "C" int bmt_offload_poll(int64_t ticket) {
    Worker& w = worker();
    std::lock_guard<std::mutex> lk(w.mu);
    return w.pending(ticket) ? 0 : 1;
}

extern "C" int bmt_offload_wait(int64_t ticket, void* stream) {
    Worker& w = worker();
    cudaEvent_t ev = nullptr;
    int err = 0;
    {
        std::unique_lock<std::mutex> lk(w.mu);
        if (ticket <= 0 || ticket >= w.next_ticket) return -1;
        w.cv_done.wait(lk, [&] { return !w.pending(ticket); });
        auto it = w.finished.find(ticket);
        if (it == w.finished.end()) return 0;   // cancelled, or already collected by an earlier wait
        ev = it->second.first;
        err = it->second.second;
        w.finished.erase(it);
    }
    if (stream && err == 0) {
        const cudaError_t e = cudaStreamWaitEvent((cudaStream_t)stream, ev, 0);
        if (e != cudaSuccess) err = (int)e;
    } else if (err == 0) {
        const cudaError_t e = cudaEventSynchronize(ev);
        if (e != cudaSuccess) err = (int)e;
    }
    // the wait above is queued (or over): the event may be recorded again by a later batch without disturbing it
    std::lock_guard<std::mutex> lk(w.mu);
    w.spare_events.push_back(ev);
    return err;
}

extern "C" int bmt_offload_cancel(int64_t ticket) {
    Worker& w = worker();
    std::lock_guard<std::mutex> lk(w.mu);
    for (auto it = w.queue.begin(); it != w.queue.end(); ++it) {
        if (it->ticket != ticket) continue;
        w.spare_events.push_back(it->uploaded);
        w.queue.erase(it);
        return 1;
    }
    return 0;
}

extern "C" int bmt_offload_drain(void) {
    Worker& w = worker();
    std::unique_lock<std::mutex> lk(w.mu);
    w.cv_done.wait(lk, [&] { return w.queue.empty() && w.in_flight == 0; });
    return 0;
}
