// Exercises the host-side native code under a sanitizer: the thread pool + AVX Adam (cpu_adam.cpp) and the shared-memory
// collectives (cpu_comm.cpp, ranks played by threads of this process that map the same segment).  Built and run by
// tests/test_native_sanitizers.py with -fsanitize=address,undefined and with -fsanitize=thread.
#include <unistd.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

extern "C" {
void bmt_adam_cpu_fp16(int64_t n, void* p32, void* p16, void* delta, const void* g16, void* m, void* v, float beta1, float beta2,
                       float eps, float lr, float scale, float wd, float bc1, float bc2);
void bmt_adam_cpu_bf16(int64_t n, void* p32, void* p16, void* delta, const void* g16, void* m, void* v, float beta1, float beta2,
                       float eps, float lr, float scale, float wd, float bc1, float bc2);
void* bmt_shm_open(const char* name, int world, int rank, uint64_t slot_bytes, double timeout_s);
void bmt_shm_close(void* handle);
int bmt_shm_barrier(void* handle);
int bmt_shm_all_reduce(void* handle, void* data, int64_t n, int dt, int op);
int bmt_shm_all_gather(void* handle, void* dst, const void* src, int64_t nbytes);
int bmt_shm_reduce_scatter(void* handle, void* dst, const void* src, int64_t n, int dt, int op);
int bmt_shm_broadcast(void* handle, void* data, int64_t nbytes, int root);
}

static int failures = 0;
#define CHECK(cond)                                                          \
    do {                                                                     \
        if (!(cond)) { std::printf("FAILED %s:%d %s\n", __FILE__, __LINE__, #cond); ++failures; } \
    } while (0)

static void test_adam() {
    // sizes around the vector widths and the pool's grain, odd offsets so the unaligned paths run
    for (int64_t n : {1, 15, 16, 33, 1000, 65536 + 17, 300000}) {
        std::vector<float> p(n + 3), m(n + 3, 0.f), v(n + 3, 0.f);
        std::vector<uint16_t> ph(n + 3, 0), g(n + 3);
        for (int64_t i = 0; i < n + 3; ++i) { p[i] = 0.01f * (float)(i % 97) - 0.4f; g[i] = (uint16_t)(0x3c00 + (i % 7)); }  // ~1.0 in fp16
        float delta[4] = {0, 0, 0, 0};
        for (int step = 1; step <= 2; ++step)
            bmt_adam_cpu_fp16(n, p.data() + 1, ph.data() + 1, step == 2 ? delta : nullptr, g.data() + 1, m.data() + 1, v.data() + 1,
                              0.9f, 0.999f, 1e-8f, 1e-3f, 2.0f, 0.01f, 1.f - std::pow(0.9f, step), 1.f - std::pow(0.999f, step));
        CHECK(std::isfinite(p[1]) && m[1] > 0.f && v[1] > 0.f);
        CHECK(p[0] == 0.01f * 0.f - 0.4f && m[0] == 0.f && ph[0] == 0);          // nothing before the range was touched
        CHECK(m[n + 1] == 0.f && ph[n + 1] == 0);                                  // nor behind it
        CHECK(std::isfinite(delta[0]) && delta[1] >= 0.f);
        std::vector<uint16_t> gb(n, 0x3f80);  // 1.0 in bf16
        bmt_adam_cpu_bf16(n, p.data() + 1, ph.data() + 1, nullptr, gb.data(), m.data() + 1, v.data() + 1, 0.9f, 0.999f, 1e-8f, 1e-3f,
                          1.0f, 0.0f, 0.1f, 0.001f);
        CHECK(std::isfinite(p[n]));
    }
}

static void shm_rank(const char* name, int world, int rank, int* errors) {
    void* h = bmt_shm_open(name, world, rank, 4096, 20.0);   // small slots: payloads span several pieces
    if (!h) { ++*errors; return; }
    for (int64_t n : {1, 5, 1000, 5000}) {
        std::vector<float> x(n);
        for (int64_t i = 0; i < n; ++i) x[i] = (float)(rank + 1) * (float)(i % 11);
        if (bmt_shm_all_reduce(h, x.data(), n, 0, 0)) ++*errors;
        const float tot = (float)(world * (world + 1) / 2);
        for (int64_t i = 0; i < n; ++i) if (x[i] != tot * (float)(i % 11)) { ++*errors; break; }
        std::vector<int64_t> mx(n, rank);
        if (bmt_shm_all_reduce(h, mx.data(), n, 3, 1)) ++*errors;
        if (mx[n - 1] != world - 1) ++*errors;
        std::vector<uint8_t> mine(n, (uint8_t)rank), all(n * world);
        if (bmt_shm_all_gather(h, all.data(), mine.data(), n)) ++*errors;
        for (int r = 0; r < world; ++r) if (all[(size_t)r * n] != r || all[(size_t)r * n + n - 1] != r) ++*errors;
        std::vector<double> src(n * world), dst(n);
        for (int64_t i = 0; i < n * world; ++i) src[i] = (double)(i % 13) + rank;
        if (bmt_shm_reduce_scatter(h, dst.data(), src.data(), n, 1, 0)) ++*errors;
        for (int64_t i = 0; i < n; ++i) {
            const double want = world * (double)((rank * n + i) % 13) + world * (world - 1) / 2.0;
            if (dst[i] != want) { ++*errors; break; }
        }
        std::vector<int32_t> b(n, rank == world - 1 ? 77 : -1);
        if (bmt_shm_broadcast(h, b.data(), n * 4, world - 1)) ++*errors;
        if (b[0] != 77 || b[n - 1] != 77) ++*errors;
    }
    if (bmt_shm_barrier(h)) ++*errors;
    bmt_shm_close(h);
}

static void test_shm() {
    for (int world : {1, 2, 3, 4}) {
        char name[64];
        std::snprintf(name, sizeof(name), "/bmt_san_%d_%d", (int)getpid(), world);
        std::vector<int> errors(world, 0);
        std::vector<std::thread> threads;
        for (int r = 0; r < world; ++r) threads.emplace_back(shm_rank, name, world, r, &errors[r]);
        for (auto& t : threads) t.join();
        for (int r = 0; r < world; ++r) CHECK(errors[r] == 0);
    }
    // a rank that never shows up: the others give up after the time limit instead of hanging
    char name[64];
    std::snprintf(name, sizeof(name), "/bmt_san_%d_missing", (int)getpid());
    CHECK(bmt_shm_open(name, 2, 0, 4096, 0.3) == nullptr);
}

int main() {
    test_adam();
    test_shm();
    if (failures) { std::printf("%d check(s) failed\n", failures); return 1; }
    std::printf("native host code: all checks passed\n");
    return 0;
}
