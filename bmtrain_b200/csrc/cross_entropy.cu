// Cross-entropy for sm_100a: single-pass (online softmax) row statistics and a recomputing backward.
//
// bmt_ce_row_stats: per row i of logits (m x n) -> max_i, sum_j exp(x_ij - max_i), x[i, target_i - vocab_start]
//                   (0 when the target is outside [vocab_start, vocab_start + n)).  One read of the logits.
// bmt_ce_backward : out_ij = (exp(x_ij - lse_i) - [j == target_i - vocab_start]) * grad_i, 0 for ignored rows.
// The reference (csrc/cuda/cross_entropy.cu:9-199) makes three strided passes per row and stores the whole softmax.
#include "api.h"
#include "common.cuh"

namespace {

// 2^x on the special-function unit (one instruction; the C library's exp2f adds range handling around it)
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <typename T>
__global__ void __launch_bounds__(256) ce_row_stats_kernel(int64_t m, int64_t n, const T* __restrict__ x,
                                                           const int64_t* __restrict__ target, int64_t vocab_start,
                                                           float* __restrict__ out) {
    __shared__ float scratch[33];
    const int64_t row = blockIdx.x;
    const T* __restrict__ xr = x + row * n;
    constexpr int V = bmt::Vec16<T>::N;
    float mx = -INFINITY, se = 0.f;
    const bool vec_ok = (n % V == 0) && (((uintptr_t)xr & 15) == 0);
    if (vec_ok) {
        // U vectors per thread and trip: all loads are issued before the first use, the running maximum moves at most
        // once per trip, and every element costs one FMA and one ex2 (base-2 exponent of x * log2e - max * log2e)
        constexpr int U = 4;
        constexpr float L2E = 1.4426950408889634f;
        const int64_t nv = n / V;
        for (int64_t i0 = threadIdx.x; i0 < nv; i0 += (int64_t)blockDim.x * U) {
            bmt::Vec16<T> v[U];
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (i0 + (int64_t)u * blockDim.x < nv) v[u] = bmt::ld16(xr + (i0 + (int64_t)u * blockDim.x) * V);
            float lm = -INFINITY;
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (i0 + (int64_t)u * blockDim.x < nv) {
#pragma unroll
                    for (int k = 0; k < V; ++k) lm = fmaxf(lm, bmt::Cvt<T>::to_f(v[u].v[k]));
                }
            if (lm > mx) { se *= ex2((mx - lm) * L2E); mx = lm; }
            const float off = -mx * L2E;
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (i0 + (int64_t)u * blockDim.x < nv) {
#pragma unroll
                    for (int k = 0; k < V; ++k) se += ex2(fmaf(bmt::Cvt<T>::to_f(v[u].v[k]), L2E, off));
                }
        }
    } else {
        for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
            float f = bmt::Cvt<T>::to_f(xr[i]);
            if (f > mx) { se *= __expf(mx - f); mx = f; }
            se += __expf(f - mx);
        }
    }
    const float gmx = bmt::block_allreduce<true>(mx, scratch);
    const float contrib = (mx == -INFINITY) ? 0.f : se * __expf(mx - gmx);
    const float gse = bmt::block_allreduce<false>(contrib, scratch);
    if (threadIdx.x == 0) {
        const int64_t t = target[row] - vocab_start;
        out[row] = gmx;
        out[m + row] = gse;
        out[2 * m + row] = (t >= 0 && t < n) ? bmt::Cvt<T>::to_f(xr[t]) : 0.f;
    }
}

// Largest of the 8 values of a packet, found on packed pairs (no conversion to fp32 per element, so the compiler has no
// reason to keep 8 converted values per packet alive between the maximum pass and the exponent pass).
__device__ __forceinline__ float packet_max(const bmt::Vec16<__half>& v) {
    const __half2* h = reinterpret_cast<const __half2*>(v.v);
    const __half2 m = __hmax2(__hmax2(h[0], h[1]), __hmax2(h[2], h[3]));
    return __half2float(__hmax(__low2half(m), __high2half(m)));
}
__device__ __forceinline__ float packet_max(const bmt::Vec16<__nv_bfloat16>& v) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(v.v);
    const __nv_bfloat162 m = __hmax2(__hmax2(h[0], h[1]), __hmax2(h[2], h[3]));
    return __bfloat162float(__hmax(__low2bfloat16(m), __high2bfloat16(m)));
}

// (max, sum of exp relative to max) pairs combine associatively
__device__ __forceinline__ void lse_combine(float& m, float& s, float m2, float s2) {
    constexpr float L2E = 1.4426950408889634f;
    const float nm = fmaxf(m, m2);
    const float a = (m == -INFINITY) ? 0.f : s * ex2((m - nm) * L2E);
    const float b = (m2 == -INFINITY) ? 0.f : s2 * ex2((m2 - nm) * L2E);
    m = nm;
    s = a + b;
}

// Streaming form for rows of 16-byte vectors: a persistent grid walks over (row, trip) chunks of 256 * U vectors; the
// loads of the next chunk are issued before the arithmetic on the current one, so every thread has U loads in flight all
// the time.  One barrier per row: warps leave their (max, sum) pair in one of two alternating slot sets and thread 0
// combines them.
template <typename T, int U>
__global__ void __launch_bounds__(256) ce_row_stats_stream_kernel(int64_t m, int64_t n, int trips, const T* __restrict__ x,
                                                                  const int64_t* __restrict__ target, int64_t vocab_start,
                                                                  float* __restrict__ out) {
    constexpr int V = bmt::Vec16<T>::N;
    constexpr float L2E = 1.4426950408889634f;
    __shared__ float sm_m[2][8], sm_s[2][8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t nv = n / V;
    const int64_t my_rows = (int64_t)blockIdx.x < m ? (m - 1 - blockIdx.x) / gridDim.x + 1 : 0;
    const int64_t chunks = my_rows * trips;
    bmt::Vec16<T> a[U], b[U];
    const auto load = [&](bmt::Vec16<T>(&v)[U], int64_t c) {
        const int64_t row = blockIdx.x + (c / trips) * gridDim.x;
        const int64_t base = (c % trips) * (int64_t)U * 256 + threadIdx.x;
        const T* __restrict__ xr = x + row * n;
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (base + u * 256 < nv) v[u] = bmt::ld16(xr + (base + u * 256) * V);
    };
    float mx = -INFINITY, se = 0.f;
    int par = 0;
    const auto process = [&](bmt::Vec16<T>(&v)[U], int64_t c) {
        const int64_t row = blockIdx.x + (c / trips) * gridDim.x;
        const int trip = (int)(c % trips);
        const int64_t base = (int64_t)trip * U * 256 + threadIdx.x;
        float lm = -INFINITY;
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (base + u * 256 < nv) lm = fmaxf(lm, packet_max(v[u]));
        if (lm > mx) { se *= ex2((mx - lm) * L2E); mx = lm; }   // mx = -inf: se is 0 and stays 0 (0 * 2^-inf)
        const float off = -mx * L2E;
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (base + u * 256 < nv) {
#pragma unroll
                for (int k = 0; k < V; ++k) se += ex2(fmaf(bmt::Cvt<T>::to_f(v[u].v[k]), L2E, off));
            }
        if (trip == trips - 1) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float m2 = __shfl_xor_sync(0xffffffffu, mx, o), s2 = __shfl_xor_sync(0xffffffffu, se, o);
                lse_combine(mx, se, m2, s2);
            }
            if (lane == 0) { sm_m[par][warp] = mx; sm_s[par][warp] = se; }
            __syncthreads();
            if (threadIdx.x == 0) {
                float gm = sm_m[par][0], gs = sm_s[par][0];
#pragma unroll
                for (int i = 1; i < 8; ++i) lse_combine(gm, gs, sm_m[par][i], sm_s[par][i]);
                const int64_t t = target[row] - vocab_start;
                out[row] = gm;
                out[m + row] = gs;
                out[2 * m + row] = (t >= 0 && t < n) ? bmt::Cvt<T>::to_f(x[row * n + t]) : 0.f;
            }
            par ^= 1;
            mx = -INFINITY;
            se = 0.f;
        }
    };
    if (chunks > 0) load(a, 0);
    for (int64_t c = 0; c < chunks; c += 2) {
        if (c + 1 < chunks) load(b, c + 1);
        process(a, c);
        if (c + 1 < chunks) {
            if (c + 2 < chunks) load(a, c + 2);
            process(b, c + 1);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256) ce_backward_kernel(int64_t m, int64_t n, const T* __restrict__ x,
                                                          const int64_t* __restrict__ target, const float* __restrict__ lse,
                                                          const float* __restrict__ grad, int64_t vocab_start,
                                                          int64_t ignore_index, T* __restrict__ out) {
    const int64_t row = blockIdx.x;
    const T* __restrict__ xr = x + row * n;
    T* __restrict__ orow = out + row * n;
    const int64_t tg = target[row];
    const bool ignored = tg == ignore_index;
    const int64_t t = tg - vocab_start;
    const float l = lse[row];
    const float g = ignored ? 0.f : grad[row];
    constexpr int V = bmt::Vec16<T>::N;
    const bool vec_ok = (n % V == 0) && (((uintptr_t)xr & 15) == 0) && (((uintptr_t)orow & 15) == 0);
    if (vec_ok) {
        constexpr int U = 4;
        constexpr float L2E = 1.4426950408889634f;
        const int64_t nv = n / V;
        const float off = -l * L2E;
        for (int64_t i0 = threadIdx.x; i0 < nv; i0 += (int64_t)blockDim.x * U) {
            bmt::Vec16<T> v[U];
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (i0 + (int64_t)u * blockDim.x < nv) v[u] = bmt::ld16(xr + (i0 + (int64_t)u * blockDim.x) * V);
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t i = i0 + (int64_t)u * blockDim.x;
                if (i >= nv) continue;
                bmt::Vec16<T> o;
#pragma unroll
                for (int k = 0; k < V; ++k) {
                    float p = ex2(fmaf(bmt::Cvt<T>::to_f(v[u].v[k]), L2E, off));
                    if (i * V + k == t) p -= 1.f;
                    o.v[k] = bmt::Cvt<T>::from_f(p * g);
                }
                bmt::st16(orow + i * V, o);
            }
        }
    } else {
        for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
            float p = __expf(bmt::Cvt<T>::to_f(xr[i]) - l);
            if (i == t) p -= 1.f;
            orow[i] = bmt::Cvt<T>::from_f(p * g);
        }
    }
}

}  // namespace

extern "C" int bmt_ce_row_stats(int64_t m, int64_t n, const void* logits, int dtype, const void* target, int64_t vocab_start,
                                void* out, void* stream) {
    if (m <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    static const bool streaming = [] { const char* e = getenv("BMT_CE_STREAM"); return !(e && atoi(e) == 0); }();
    if (streaming && dtype != BMT_DT_F32 && n % 8 == 0 && n >= 2048 && ((uintptr_t)logits & 15) == 0) {
        const int64_t per_thread = (n / 8 + 255) / 256;
        const int u = per_thread <= 4 ? 4 : per_thread <= 5 ? 5 : per_thread <= 6 ? 6 : 8;
        const int trips = (int)((per_thread + u - 1) / u);
#define BMT_CE_STREAM(T, UU)                                                                                                   \
        do {                                                                                                                   \
            static int per_sm = 0;   /* resident CTAs per SM of this instantiation: the grid is exactly one wave */           \
            if (!per_sm && (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, ce_row_stats_stream_kernel<T, UU>, 256, 0) != cudaSuccess || per_sm < 1)) \
                per_sm = 2;                                                                                                    \
            const int64_t cap = (int64_t)148 * per_sm;                                                                         \
            ce_row_stats_stream_kernel<T, UU><<<(unsigned)(m < cap ? m : cap), 256, 0, s>>>(                                   \
                m, n, trips, (const T*)logits, (const int64_t*)target, vocab_start, (float*)out);                              \
        } while (0)
#define BMT_CE_STREAM_U(T) \
        do { if (u == 4) BMT_CE_STREAM(T, 4); else if (u == 5) BMT_CE_STREAM(T, 5); else if (u == 6) BMT_CE_STREAM(T, 6); else BMT_CE_STREAM(T, 8); } while (0)
        if (dtype == BMT_DT_F16) BMT_CE_STREAM_U(__half); else BMT_CE_STREAM_U(__nv_bfloat16);
#undef BMT_CE_STREAM_U
#undef BMT_CE_STREAM
        bmt_count_launch(1);
        return (int)cudaGetLastError();
    }
    if (dtype == BMT_DT_F16) ce_row_stats_kernel<__half><<<(unsigned)m, 256, 0, s>>>(m, n, (const __half*)logits, (const int64_t*)target, vocab_start, (float*)out);
    else if (dtype == BMT_DT_BF16) ce_row_stats_kernel<__nv_bfloat16><<<(unsigned)m, 256, 0, s>>>(m, n, (const __nv_bfloat16*)logits, (const int64_t*)target, vocab_start, (float*)out);
    else ce_row_stats_kernel<float><<<(unsigned)m, 256, 0, s>>>(m, n, (const float*)logits, (const int64_t*)target, vocab_start, (float*)out);
    bmt_count_launch(1);
    return (int)cudaGetLastError();
}

extern "C" int bmt_ce_backward(int64_t m, int64_t n, const void* logits, int dtype, const void* target, const void* lse,
                               const void* grad, int64_t vocab_start, int64_t ignore_index, void* out, void* stream) {
    if (m <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == BMT_DT_F16) ce_backward_kernel<__half><<<(unsigned)m, 256, 0, s>>>(m, n, (const __half*)logits, (const int64_t*)target, (const float*)lse, (const float*)grad, vocab_start, ignore_index, (__half*)out);
    else if (dtype == BMT_DT_BF16) ce_backward_kernel<__nv_bfloat16><<<(unsigned)m, 256, 0, s>>>(m, n, (const __nv_bfloat16*)logits, (const int64_t*)target, (const float*)lse, (const float*)grad, vocab_start, ignore_index, (__nv_bfloat16*)out);
    else ce_backward_kernel<float><<<(unsigned)m, 256, 0, s>>>(m, n, (const float*)logits, (const int64_t*)target, (const float*)lse, (const float*)grad, vocab_start, ignore_index, (float*)out);
    bmt_count_launch(1);
    return (int)cudaGetLastError();
}
