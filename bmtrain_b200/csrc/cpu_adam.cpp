// Host-side Adam for the offload optimizer, plus fp32 -> fp16/bf16 converters.
//
// * A persistent pool of worker threads (one per CPU the process may run on) is created once and
//   reused for every call; work is handed out in cache-friendly chunks from an atomic counter.
//   (The reference spawns fresh std::threads inside every call: csrc/include/adam_cpu.hpp:42-80.)
// * AVX-512 paths for fp16 AND bf16 (the reference's bf16 path is scalar and truncates; here bf16
//   is rounded to nearest even), AVX2+F16C path for fp16, scalar fall-back; dispatch at run time.
// * Math: g = g_half / scale; m = b1 m + (1-b1) g; v = b2 v + (1-b2) g^2;
//         p = p - lr * (m/bc1) / (sqrt(v/bc2) + eps) - lr * wd * p;  p_half = round(p).
// * Optional delta statistics (mean, variance, sum, sum of squares of p_new - p_old).
#include <immintrin.h>
#include <pthread.h>
#include <sched.h>
#include <stdint.h>
#include <string.h>

#include <atomic>
#include <cmath>
#include <condition_variable>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

namespace {

// ------------------------------------------------------------------------------------------ thread pool
class Pool {
  public:
    static Pool& get() {
        static Pool p;
        return p;
    }
    int size() const { return (int)workers_.size() + 1; }

    // Runs fn(begin, end, worker) over [0, n) in chunks; the caller participates.
    void parallel_for(int64_t n, int64_t chunk, const std::function<void(int64_t, int64_t, int)>& fn) {
        if (n <= 0) return;
        if (workers_.empty() || n <= chunk) { fn(0, n, 0); return; }
        std::unique_lock<std::mutex> call_lock(call_mu_);  // one parallel region at a time
        {
            std::lock_guard<std::mutex> lk(mu_);
            fn_ = &fn; n_ = n; chunk_ = chunk; next_.store(0); pending_ = (int)workers_.size(); ++epoch_;
        }
        cv_.notify_all();
        run_chunks(0);
        std::unique_lock<std::mutex> lk(mu_);
        done_cv_.wait(lk, [&] { return pending_ == 0; });
        fn_ = nullptr;
    }

  private:
    Pool() {
        cpu_set_t set;
        CPU_ZERO(&set);
        int ncpu = 1;
        std::vector<int> cpus;
        if (sched_getaffinity(0, sizeof(set), &set) == 0) {
            for (int c = 0; c < CPU_SETSIZE; ++c)
                if (CPU_ISSET(c, &set)) cpus.push_back(c);
            ncpu = (int)cpus.size();
        }
        const char* env = getenv("BMT_CPU_THREADS");
        int want = env ? atoi(env) : ncpu;
        if (want < 1) want = 1;
        if (want > 128) want = 128;
        for (int i = 1; i < want; ++i) workers_.emplace_back([this, i] { loop(i); });
    }
    ~Pool() {
        {
            std::lock_guard<std::mutex> lk(mu_);
            stop_ = true; ++epoch_;
        }
        cv_.notify_all();
        for (auto& t : workers_) t.join();
    }
    void run_chunks(int worker) {
        for (;;) {
            const int64_t b = next_.fetch_add(chunk_);
            if (b >= n_) break;
            const int64_t e = b + chunk_ < n_ ? b + chunk_ : n_;
            (*fn_)(b, e, worker);
        }
    }
    void loop(int worker) {
        uint64_t seen = 0;
        for (;;) {
            {
                std::unique_lock<std::mutex> lk(mu_);
                cv_.wait(lk, [&] { return epoch_ != seen; });
                seen = epoch_;
                if (stop_) return;
            }
            run_chunks(worker);
            std::lock_guard<std::mutex> lk(mu_);
            if (--pending_ == 0) done_cv_.notify_one();
        }
    }
    std::vector<std::thread> workers_;
    std::mutex mu_, call_mu_;
    std::condition_variable cv_, done_cv_;
    const std::function<void(int64_t, int64_t, int)>* fn_ = nullptr;
    int64_t n_ = 0, chunk_ = 1;
    std::atomic<int64_t> next_{0};
    int pending_ = 0;
    uint64_t epoch_ = 0;
    bool stop_ = false;
};

// --------------------------------------------------------------------------------------- scalar converters
inline float half_to_float(uint16_t h) { return _cvtsh_ss(h); }
inline uint16_t float_to_half(float f) { return _cvtss_sh(f, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC); }
inline float bf16_to_float(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
inline uint16_t float_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);  // quiet NaN
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

struct AdamConst {
    float beta1, beta2, eps, lr, inv_scale, wd, inv_bc1, inv_bc2;
};

template <bool BF16>
void adam_scalar(int64_t b, int64_t e, float* p, uint16_t* ph, const uint16_t* g, float* m, float* v, const AdamConst& c,
                 double* dsum, double* dsq) {
    for (int64_t i = b; i < e; ++i) {
        const float gf = (BF16 ? bf16_to_float(g[i]) : half_to_float(g[i])) * c.inv_scale;
        const float mm = c.beta1 * m[i] + (1.f - c.beta1) * gf;
        const float vv = c.beta2 * v[i] + (1.f - c.beta2) * gf * gf;
        const float old = p[i];
        const float np = old - c.lr * (mm * c.inv_bc1) / (std::sqrt(vv * c.inv_bc2) + c.eps) - c.lr * c.wd * old;
        m[i] = mm; v[i] = vv; p[i] = np;
        ph[i] = BF16 ? float_to_bf16(np) : float_to_half(np);
        if (dsum) { const double d = (double)np - old; *dsum += d; *dsq += d * d; }
    }
}

// ------------------------------------------------------------------------------------------------ AVX-512
__attribute__((target("avx512f,avx512bw,avx512vl"))) inline __m512 load_half16(const uint16_t* p, bool bf16) {
    const __m256i raw = _mm256_loadu_si256((const __m256i*)p);
    if (bf16) return _mm512_castsi512_ps(_mm512_slli_epi32(_mm512_cvtepu16_epi32(raw), 16));
    return _mm512_cvtph_ps(raw);
}
__attribute__((target("avx512f,avx512bw,avx512vl"))) inline __m256i to_half16(__m512 x, bool bf16) {
    if (!bf16) return _mm512_cvtps_ph(x, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC);
    const __m512i u = _mm512_castps_si512(x);
    const __m512i lsb = _mm512_and_si512(_mm512_srli_epi32(u, 16), _mm512_set1_epi32(1));
    const __m512i rounded = _mm512_add_epi32(u, _mm512_add_epi32(lsb, _mm512_set1_epi32(0x7fff)));
    const __mmask16 nan = _mm512_cmp_ps_mask(x, x, _CMP_UNORD_Q);
    const __m512i quiet = _mm512_or_si512(u, _mm512_set1_epi32(0x00400000));
    const __m512i sel = _mm512_mask_blend_epi32(nan, rounded, quiet);
    return _mm512_cvtepi32_epi16(_mm512_srli_epi32(sel, 16));
}
__attribute__((target("avx512f,avx512bw,avx512vl"))) inline void store_half16(uint16_t* p, __m512 x, bool bf16) {
    _mm256_storeu_si256((__m256i*)p, to_half16(x, bf16));
}

struct __attribute__((target("avx512f"))) AdamVec {
    __m512 b1, ob1, b2, ob2, eps, lr, isc, lrwd, ibc1, ibc2;
    __m512d s0, q0;
};

// Where the new fp32 state goes: back over the old one (in place) or into a second set of arrays.  Writing a second
// set with ordinary stores would read every destination line first; whole lines are written, so they go out with
// non-temporal stores and the memory traffic stays what the in-place form has.
struct StateOut {
    float *p, *m, *v;
    bool stream;   // destinations differ from the sources and are 64-byte aligned: non-temporal stores
};

// 16 elements at `at`: new m, v and fp32 parameters go to `o` (which may alias the inputs); returns the new parameters.
template <bool BF16>
__attribute__((target("avx512f,avx512bw,avx512vl"))) inline __m512 adam16(int64_t at, const float* p, const uint16_t* g, const float* m,
                                                                           const float* v, const StateOut& o, AdamVec& k, bool stats) {
    const __m512 gf = _mm512_mul_ps(load_half16(g + at, BF16), k.isc);
    const __m512 mm = _mm512_fmadd_ps(k.b1, _mm512_loadu_ps(m + at), _mm512_mul_ps(k.ob1, gf));
    const __m512 vv = _mm512_fmadd_ps(k.b2, _mm512_loadu_ps(v + at), _mm512_mul_ps(k.ob2, _mm512_mul_ps(gf, gf)));
    const __m512 old = _mm512_loadu_ps(p + at);
    const __m512 den = _mm512_add_ps(_mm512_sqrt_ps(_mm512_mul_ps(vv, k.ibc2)), k.eps);
    const __m512 upd = _mm512_div_ps(_mm512_mul_ps(mm, k.ibc1), den);
    __m512 np = _mm512_fnmadd_ps(k.lr, upd, old);
    np = _mm512_fnmadd_ps(k.lrwd, old, np);
    if (o.stream) {
        _mm512_stream_ps(o.m + at, mm);
        _mm512_stream_ps(o.v + at, vv);
        _mm512_stream_ps(o.p + at, np);
    } else {
        _mm512_storeu_ps(o.m + at, mm);
        _mm512_storeu_ps(o.v + at, vv);
        _mm512_storeu_ps(o.p + at, np);
    }
    if (stats) {
        const __m512 d = _mm512_sub_ps(np, old);
        const __m512d lo = _mm512_cvtps_pd(_mm512_castps512_ps256(d)), hi = _mm512_cvtps_pd(_mm256_castpd_ps(_mm512_extractf64x4_pd(_mm512_castps_pd(d), 1)));
        k.s0 = _mm512_add_pd(k.s0, _mm512_add_pd(lo, hi));
        k.q0 = _mm512_add_pd(k.q0, _mm512_fmadd_pd(lo, lo, _mm512_mul_pd(hi, hi)));
    }
    return np;
}

template <bool BF16>
void adam_scalar_out(int64_t b, int64_t e, const float* p, uint16_t* ph, const uint16_t* g, const float* m, const float* v,
                     const StateOut& o, const AdamConst& c) {
    for (int64_t i = b; i < e; ++i) {
        const float gf = (BF16 ? bf16_to_float(g[i]) : half_to_float(g[i])) * c.inv_scale;
        const float mm = c.beta1 * m[i] + (1.f - c.beta1) * gf;
        const float vv = c.beta2 * v[i] + (1.f - c.beta2) * gf * gf;
        const float old = p[i];
        const float np = old - c.lr * (mm * c.inv_bc1) / (std::sqrt(vv * c.inv_bc2) + c.eps) - c.lr * c.wd * old;
        o.m[i] = mm; o.v[i] = vv; o.p[i] = np;
        ph[i] = BF16 ? float_to_bf16(np) : float_to_half(np);
    }
}

template <bool BF16>
__attribute__((target("avx512f,avx512bw,avx512vl")))
void adam_avx512(int64_t b, int64_t e, const float* p, uint16_t* ph, const uint16_t* g, const float* m, const float* v,
                 const StateOut& out, const AdamConst& c, double* dsum, double* dsq) {
    AdamVec k;
    k.b1 = _mm512_set1_ps(c.beta1); k.ob1 = _mm512_set1_ps(1.f - c.beta1);
    k.b2 = _mm512_set1_ps(c.beta2); k.ob2 = _mm512_set1_ps(1.f - c.beta2);
    k.eps = _mm512_set1_ps(c.eps); k.lr = _mm512_set1_ps(c.lr); k.isc = _mm512_set1_ps(c.inv_scale);
    k.lrwd = _mm512_set1_ps(c.lr * c.wd); k.ibc1 = _mm512_set1_ps(c.inv_bc1); k.ibc2 = _mm512_set1_ps(c.inv_bc2);
    k.s0 = _mm512_setzero_pd(); k.q0 = _mm512_setzero_pd();
    const bool stats = dsum != nullptr;
    int64_t i = b;
    StateOut o = out;
    // non-temporal stores need 64-byte aligned destinations: the three arrays have to be aligned alike at `b`
    o.stream = out.stream && !((((uintptr_t)(out.p + b)) | ((uintptr_t)(out.m + b)) | ((uintptr_t)(out.v + b))) & 63);
    // the half-precision output is write-only: whole cache lines of it go out with non-temporal stores, which saves the
    // read-for-ownership of a line that would only be overwritten (the step is bound by host memory traffic)
    while (i + 16 <= e && (((uintptr_t)(ph + i)) & 63)) { store_half16(ph + i, adam16<BF16>(i, p, g, m, v, o, k, stats), BF16); i += 16; }
    for (; i + 32 <= e; i += 32) {
        const __m256i h0 = to_half16(adam16<BF16>(i, p, g, m, v, o, k, stats), BF16);
        const __m256i h1 = to_half16(adam16<BF16>(i + 16, p, g, m, v, o, k, stats), BF16);
        _mm512_stream_si512((__m512i*)(ph + i), _mm512_inserti64x4(_mm512_castsi256_si512(h0), h1, 1));
    }
    for (; i + 16 <= e; i += 16) store_half16(ph + i, adam16<BF16>(i, p, g, m, v, o, k, stats), BF16);
    _mm_sfence();   // non-temporal stores are ordered before whatever signals that this range is done
    const __m512d s0 = k.s0, q0 = k.q0;
    if (dsum) { *dsum += _mm512_reduce_add_pd(s0); *dsq += _mm512_reduce_add_pd(q0); }
    if (i < e) {
        if (out.p == p) adam_scalar<BF16>(i, e, out.p, ph, g, out.m, out.v, c, dsum, dsq);
        else adam_scalar_out<BF16>(i, e, p, ph, g, m, v, out, c);
    }
}

// --------------------------------------------------------------------------------------------------- AVX2
__attribute__((target("avx2,fma,f16c")))
void adam_avx2_fp16(int64_t b, int64_t e, float* p, uint16_t* ph, const uint16_t* g, float* m, float* v, const AdamConst& c,
                    double* dsum, double* dsq) {
    const __m256 b1 = _mm256_set1_ps(c.beta1), ob1 = _mm256_set1_ps(1.f - c.beta1);
    const __m256 b2 = _mm256_set1_ps(c.beta2), ob2 = _mm256_set1_ps(1.f - c.beta2);
    const __m256 eps = _mm256_set1_ps(c.eps), lr = _mm256_set1_ps(c.lr), isc = _mm256_set1_ps(c.inv_scale);
    const __m256 lrwd = _mm256_set1_ps(c.lr * c.wd), ibc1 = _mm256_set1_ps(c.inv_bc1), ibc2 = _mm256_set1_ps(c.inv_bc2);
    int64_t i = b;
    for (; i + 8 <= e; i += 8) {
        const __m256 gf = _mm256_mul_ps(_mm256_cvtph_ps(_mm_loadu_si128((const __m128i*)(g + i))), isc);
        const __m256 mm = _mm256_fmadd_ps(b1, _mm256_loadu_ps(m + i), _mm256_mul_ps(ob1, gf));
        const __m256 vv = _mm256_fmadd_ps(b2, _mm256_loadu_ps(v + i), _mm256_mul_ps(ob2, _mm256_mul_ps(gf, gf)));
        const __m256 old = _mm256_loadu_ps(p + i);
        const __m256 den = _mm256_add_ps(_mm256_sqrt_ps(_mm256_mul_ps(vv, ibc2)), eps);
        const __m256 upd = _mm256_div_ps(_mm256_mul_ps(mm, ibc1), den);
        __m256 np = _mm256_fnmadd_ps(lr, upd, old);
        np = _mm256_fnmadd_ps(lrwd, old, np);
        _mm256_storeu_ps(m + i, mm);
        _mm256_storeu_ps(v + i, vv);
        _mm256_storeu_ps(p + i, np);
        _mm_storeu_si128((__m128i*)(ph + i), _mm256_cvtps_ph(np, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC));
        if (dsum) {
            alignas(32) float dd[8];
            _mm256_store_ps(dd, _mm256_sub_ps(np, old));
            for (int k = 0; k < 8; ++k) { *dsum += dd[k]; *dsq += (double)dd[k] * dd[k]; }
        }
    }
    if (i < e) adam_scalar<false>(i, e, p, ph, g, m, v, c, dsum, dsq);
}

int cpu_level() {
    static int level = -1;
    if (level < 0) {
        __builtin_cpu_init();
        if (__builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512bw") && __builtin_cpu_supports("avx512vl")) level = 2;
        else if (__builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma") && __builtin_cpu_supports("f16c")) level = 1;
        else level = 0;
        const char* env = getenv("BMT_CPU_LEVEL");
        if (env && atoi(env) < level) level = atoi(env);
    }
    return level;
}

// State read from (p, m, v), new state written to (po, mo, vo); the two sets are either identical or disjoint.
template <bool BF16>
void adam_cpu_out(int64_t n, const float* p, const float* m, const float* v, float* po, float* mo, float* vo, uint16_t* ph,
                  const uint16_t* g, const AdamConst& c) {
    const int level = cpu_level();
    const StateOut out{po, mo, vo, po != p};
    Pool::get().parallel_for(n, 1 << 16, [&](int64_t b, int64_t e, int) {
        if (level == 2) adam_avx512<BF16>(b, e, p, ph, g, m, v, out, c, nullptr, nullptr);
        else if (po == p && level == 1 && !BF16) adam_avx2_fp16(b, e, po, ph, g, mo, vo, c, nullptr, nullptr);
        else if (po == p) adam_scalar<BF16>(b, e, po, ph, g, mo, vo, c, nullptr, nullptr);
        else adam_scalar_out<BF16>(b, e, p, ph, g, m, v, out, c);
    });
}

template <bool BF16>
void adam_cpu(int64_t n, float* p, uint16_t* ph, float* delta, const uint16_t* g, float* m, float* v, float beta1, float beta2,
              float eps, float lr, float scale, float wd, float bc1, float bc2) {
    const AdamConst c{beta1, beta2, eps, lr, 1.f / scale, wd, 1.f / bc1, 1.f / bc2};
    Pool& pool = Pool::get();
    const int level = cpu_level();
    std::vector<double> sums(delta ? pool.size() * 16 : 0, 0.0);  // padded to keep workers on separate cache lines
    const StateOut in_place{p, m, v, false};
    auto body = [&](int64_t b, int64_t e, int w) {
        double* ds = delta ? &sums[w * 16] : nullptr;
        double* dq = delta ? &sums[w * 16 + 1] : nullptr;
        if (level == 2) adam_avx512<BF16>(b, e, p, ph, g, m, v, in_place, c, ds, dq);
        else if (level == 1 && !BF16) adam_avx2_fp16(b, e, p, ph, g, m, v, c, ds, dq);
        else adam_scalar<BF16>(b, e, p, ph, g, m, v, c, ds, dq);
    };
    pool.parallel_for(n, 1 << 16, body);
    if (delta) {
        double s = 0, q = 0;
        for (int w = 0; w < pool.size(); ++w) { s += sums[w * 16]; q += sums[w * 16 + 1]; }
        const double mean = s / (double)n;
        delta[0] = (float)mean;
        delta[1] = (float)(q / (double)n - mean * mean);
        delta[2] = (float)s;
        delta[3] = (float)q;
    }
}

template <bool BF16>
__attribute__((target("avx512f,avx512bw,avx512vl"))) void convert_avx512(int64_t b, int64_t e, const float* src, uint16_t* dst) {
    int64_t i = b;
    for (; i + 16 <= e; i += 16) store_half16(dst + i, _mm512_loadu_ps(src + i), BF16);
    for (; i < e; ++i) dst[i] = BF16 ? float_to_bf16(src[i]) : float_to_half(src[i]);
}

template <bool BF16> void convert(int64_t n, const float* src, uint16_t* dst) {
    const int level = cpu_level();
    Pool::get().parallel_for(n, 1 << 17, [&](int64_t b, int64_t e, int) {
        if (level == 2) { convert_avx512<BF16>(b, e, src, dst); return; }
        for (int64_t i = b; i < e; ++i) dst[i] = BF16 ? float_to_bf16(src[i]) : float_to_half(src[i]);
    });
}

}  // namespace

extern "C" {

void bmt_adam_cpu_fp16(int64_t n, void* p32, void* p16, void* delta, const void* g16, void* m, void* v, float beta1, float beta2,
                       float eps, float lr, float scale, float wd, float bc1, float bc2) {
    adam_cpu<false>(n, (float*)p32, (uint16_t*)p16, (float*)delta, (const uint16_t*)g16, (float*)m, (float*)v, beta1, beta2, eps, lr,
                    scale, wd, bc1, bc2);
}

void bmt_adam_cpu_bf16(int64_t n, void* p32, void* p16, void* delta, const void* g16, void* m, void* v, float beta1, float beta2,
                       float eps, float lr, float scale, float wd, float bc1, float bc2) {
    adam_cpu<true>(n, (float*)p32, (uint16_t*)p16, (float*)delta, (const uint16_t*)g16, (float*)m, (float*)v, beta1, beta2, eps, lr,
                   scale, wd, bc1, bc2);
}

// Out-of-place capable form used by the offload worker: reads (p32, m, v), writes (p32_out, m_out, v_out) -- pass the
// same three pointers for an in-place step -- and the half-precision copy `p16`.
void bmt_adam_cpu_ex(int64_t n, const void* p32, const void* m, const void* v, void* p32_out, void* m_out, void* v_out, void* p16,
                     const void* g16, float beta1, float beta2, float eps, float lr, float scale, float wd, float bc1, float bc2,
                     int bf16) {
    const AdamConst c{beta1, beta2, eps, lr, 1.f / scale, wd, 1.f / bc1, 1.f / bc2};
    if (bf16) adam_cpu_out<true>(n, (const float*)p32, (const float*)m, (const float*)v, (float*)p32_out, (float*)m_out, (float*)v_out,
                                 (uint16_t*)p16, (const uint16_t*)g16, c);
    else adam_cpu_out<false>(n, (const float*)p32, (const float*)m, (const float*)v, (float*)p32_out, (float*)m_out, (float*)v_out,
                             (uint16_t*)p16, (const uint16_t*)g16, c);
}

void bmt_fp16_from_fp32(int64_t n, const void* src, void* dst) { convert<false>(n, (const float*)src, (uint16_t*)dst); }
void bmt_bf16_from_fp32(int64_t n, const void* src, void* dst) { convert<true>(n, (const float*)src, (uint16_t*)dst); }

// 0 = scalar, 1 = AVX2 + FMA + F16C, 2 = AVX-512 (F/BW/VL)
int bmt_cpu_level(void) { return cpu_level(); }
int bmt_cpu_threads(void) { return Pool::get().size(); }

}  // extern "C"
