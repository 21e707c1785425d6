// Cross-entropy for sm_100a: single-pass (online softmax) row statistics and a recomputing backward.
//
// bmt_ce_row_stats: per row i of logits (m x n) -> max_i, sum_j exp(x_ij - max_i), x[i, target_i - vocab_start]
//                   (0 when the target is outside [vocab_start, vocab_start + n)).  One read of the logits.
// bmt_ce_backward : out_ij = (exp(x_ij - lse_i) - [j == target_i - vocab_start]) * grad_i, 0 for ignored rows.
// The reference (csrc/cuda/cross_entropy.cu:9-199) makes three strided passes per row and stores the whole softmax.
#include "api.h"
#include "common.cuh"

namespace {

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
            if (lm > mx) { se *= exp2f((mx - lm) * L2E); mx = lm; }
            const float off = -mx * L2E;
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (i0 + (int64_t)u * blockDim.x < nv) {
#pragma unroll
                    for (int k = 0; k < V; ++k) se += exp2f(fmaf(bmt::Cvt<T>::to_f(v[u].v[k]), L2E, off));
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
                    float p = exp2f(fmaf(bmt::Cvt<T>::to_f(v[u].v[k]), L2E, off));
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
