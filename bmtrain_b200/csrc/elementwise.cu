// SwiGLU forward/backward and column sums (bias gradient).
#include "api.h"
#include "common.cuh"

namespace {

template <typename T>
__global__ void __launch_bounds__(256) swiglu_fwd_kernel(int64_t rows, int64_t f, const T* __restrict__ x, T* __restrict__ out) {
    const int64_t per_row = f / 8;
    const int64_t total = rows * per_row;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / per_row, c = (i % per_row) * 8;
        bmt::Vec16<T> g = bmt::ld16(x + r * 2 * f + c), u = bmt::ld16(x + r * 2 * f + f + c), o;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float gv = bmt::Cvt<T>::to_f(g.v[k]);
            o.v[k] = bmt::Cvt<T>::from_f(gv / (1.f + __expf(-gv)) * bmt::Cvt<T>::to_f(u.v[k]));
        }
        bmt::st16(out + r * f + c, o);
    }
}

template <typename T>
__global__ void __launch_bounds__(256) swiglu_bwd_kernel(int64_t rows, int64_t f, const T* __restrict__ x, const T* __restrict__ go, T* __restrict__ dx) {
    const int64_t per_row = f / 8;
    const int64_t total = rows * per_row;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / per_row, c = (i % per_row) * 8;
        bmt::Vec16<T> g = bmt::ld16(x + r * 2 * f + c), u = bmt::ld16(x + r * 2 * f + f + c), d = bmt::ld16(go + r * f + c), dg, du;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float gv = bmt::Cvt<T>::to_f(g.v[k]), uv = bmt::Cvt<T>::to_f(u.v[k]), dv = bmt::Cvt<T>::to_f(d.v[k]);
            const float sg = 1.f / (1.f + __expf(-gv));
            const float silu = gv * sg;
            dg.v[k] = bmt::Cvt<T>::from_f(dv * uv * (sg + silu * (1.f - sg)));
            du.v[k] = bmt::Cvt<T>::from_f(dv * silu);
        }
        bmt::st16(dx + r * 2 * f + c, dg);
        bmt::st16(dx + r * 2 * f + f + c, du);
    }
}

// block = 8 column packets (64 columns) x 32 row lanes
template <typename T>
__global__ void __launch_bounds__(256) colsum_kernel(int64_t m, int64_t n, const T* __restrict__ x, T* __restrict__ out) {
    __shared__ float red[32][65];
    const int cv = threadIdx.x & 7, lane = threadIdx.x >> 3;
    const int64_t c = (int64_t)blockIdx.x * 64 + cv * 8;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (c < n) {
        for (int64_t r = lane; r < m; r += 32) {
            bmt::Vec16<T> v = bmt::ld16(x + r * n + c);
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[k] += bmt::Cvt<T>::to_f(v.v[k]);
        }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) red[lane][cv * 8 + k] = acc[k];
    __syncthreads();
    if (threadIdx.x < 64) {
        float s = 0.f;
#pragma unroll 8
        for (int l = 0; l < 32; ++l) s += red[l][threadIdx.x];
        const int64_t col = (int64_t)blockIdx.x * 64 + threadIdx.x;
        if (col < n) out[col] = bmt::Cvt<T>::from_f(s);
    }
}

template <typename T>
__global__ void __launch_bounds__(256) gelu_kernel(int64_t n8, const T* __restrict__ x, T* __restrict__ out) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (int64_t)gridDim.x * blockDim.x) {
        bmt::Vec16<T> v = bmt::ld16(x + i * 8), o;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float f = bmt::Cvt<T>::to_f(v.v[k]);
            o.v[k] = bmt::Cvt<T>::from_f(0.5f * f * (1.f + erff(f * 0.70710678118654752f)));
        }
        bmt::st16(out + i * 8, o);
    }
}

unsigned grid1d(int64_t work) {
    int64_t b = bmt::ceil_div64(work, 256);
    if (b > 148 * 8) b = 148 * 8;
    return (unsigned)(b < 1 ? 1 : b);
}

}  // namespace

extern "C" int bmt_swiglu_fwd(int64_t rows, int64_t f, const void* x, int dtype, void* out, void* stream) {
    if (rows <= 0) return 0;
    if (f % 8 || dtype == BMT_DT_F32) return -3;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == BMT_DT_F16) swiglu_fwd_kernel<__half><<<grid1d(rows * f / 8), 256, 0, s>>>(rows, f, (const __half*)x, (__half*)out);
    else swiglu_fwd_kernel<__nv_bfloat16><<<grid1d(rows * f / 8), 256, 0, s>>>(rows, f, (const __nv_bfloat16*)x, (__nv_bfloat16*)out);
    bmt_count_launch(1);
    return (int)cudaGetLastError();
}

extern "C" int bmt_swiglu_bwd(int64_t rows, int64_t f, const void* x, const void* g, int dtype, void* dx, void* stream) {
    if (rows <= 0) return 0;
    if (f % 8 || dtype == BMT_DT_F32) return -3;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == BMT_DT_F16) swiglu_bwd_kernel<__half><<<grid1d(rows * f / 8), 256, 0, s>>>(rows, f, (const __half*)x, (const __half*)g, (__half*)dx);
    else swiglu_bwd_kernel<__nv_bfloat16><<<grid1d(rows * f / 8), 256, 0, s>>>(rows, f, (const __nv_bfloat16*)x, (const __nv_bfloat16*)g, (__nv_bfloat16*)dx);
    bmt_count_launch(1);
    return (int)cudaGetLastError();
}

extern "C" int bmt_colsum(int64_t m, int64_t n, const void* x, int dtype, void* out, void* stream) {
    if (n <= 0) return 0;
    if (n % 8 || dtype == BMT_DT_F32) return -3;
    cudaStream_t s = (cudaStream_t)stream;
    const unsigned g = (unsigned)((n + 63) / 64);
    if (dtype == BMT_DT_F16) colsum_kernel<__half><<<g, 256, 0, s>>>(m, n, (const __half*)x, (__half*)out);
    else colsum_kernel<__nv_bfloat16><<<g, 256, 0, s>>>(m, n, (const __nv_bfloat16*)x, (__nv_bfloat16*)out);
    bmt_count_launch(1);
    return (int)cudaGetLastError();
}

// out = gelu(x), n elements (multiple of 8), exact erf form
extern "C" int bmt_gelu_fwd(int64_t n, const void* x, int dtype, void* out, void* stream) {
    if (n <= 0) return 0;
    if (n % 8 || dtype == BMT_DT_F32) return -3;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == BMT_DT_F16) gelu_kernel<__half><<<grid1d(n / 8), 256, 0, s>>>(n / 8, (const __half*)x, (__half*)out);
    else gelu_kernel<__nv_bfloat16><<<grid1d(n / 8), 256, 0, s>>>(n / 8, (const __nv_bfloat16*)x, (__nv_bfloat16*)out);
    bmt_count_launch(1);
    return (int)cudaGetLastError();
}
