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
