// Library-wide bookkeeping: launch counter and device probe.
#include <atomic>

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

// Offloaded Adam, chunk loop (see BmtOffloadChunk): event wait -> host math -> upload, without returning to the
// interpreter between chunks (the host threads would idle for the tens of microseconds each round trip takes).
extern "C" int bmt_offload_adam_run(const BmtOffloadChunk* chunks, int n, BmtAdamCpuFn fn_fp16, BmtAdamCpuFn fn_bf16, void* h2d_stream) {
    for (int i = 0; i < n; ++i) {
        const BmtOffloadChunk& c = chunks[i];
        if (c.grad_ready) {
            const cudaError_t e = cudaEventSynchronize((cudaEvent_t)c.grad_ready);
            if (e != cudaSuccess) return (int)e;
        }
        if (c.n <= 0) continue;
        (c.bf16 ? fn_bf16 : fn_fp16)(c.n, c.p32, c.p16_host, nullptr, c.g16_host, c.m, c.v, c.beta1, c.beta2, c.eps, c.lr, c.scale,
                                      c.wd, c.bc1, c.bc2);
        const cudaError_t e = cudaMemcpyAsync(c.p_dev, c.p16_host, (size_t)c.n * 2, cudaMemcpyHostToDevice, (cudaStream_t)h2d_stream);
        if (e != cudaSuccess) return (int)e;
    }
    return 0;
}
