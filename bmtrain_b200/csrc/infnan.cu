// Multi-tensor scans over gradient shards: inf/nan detection, sum of squares, in-place scaling.
// Replaces the reference's two-kernel-per-parameter any-reduce (csrc/cuda/has_inf_nan.cu:35-138) by one
// launch over up to 24 tensors with 128-bit loads; the flag is OR-ed with a single byte store.
#include "api.h"
#include "common.cuh"

namespace {

template <typename T> __device__ __forceinline__ bool bad(T v) {
    float f = bmt::Cvt<T>::to_f(v);
    return !(fabsf(f) <= 3.402823466e38f);  // true for inf and nan
}

template <typename T>
__global__ void __launch_bounds__(256) infnan_kernel(BmtPtrTable tab, unsigned char* out) {
    const int t = blockIdx.y;
    const T* __restrict__ p = (const T*)tab.p[t];
    const int64_t n = tab.n[t];
    constexpr int V = bmt::Vec16<T>::N;
    // peel to a 16-byte boundary so that arbitrary sub-slices can be scanned
    int64_t head = ((16 - ((uintptr_t)p & 15)) & 15) / sizeof(T);
    if (head > n) head = n;
    bool found = false;
    if (blockIdx.x == 0)
        for (int64_t i = threadIdx.x; i < head; i += blockDim.x) found |= bad(p[i]);
    const T* q = p + head;
    const int64_t nvec = (n - head) / V;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
        bmt::Vec16<T> x = bmt::ld16(q + i * V);
#pragma unroll
        for (int k = 0; k < V; ++k) found |= bad(x.v[k]);
    }
    if (blockIdx.x == 0)
        for (int64_t i = head + nvec * V + threadIdx.x; i < n; i += blockDim.x) found |= bad(p[i]);
    if (__syncthreads_or(found) && threadIdx.x == 0) *out = 1;
}

template <typename T>
__global__ void __launch_bounds__(256) sqnorm_kernel(BmtPtrTable tab, float* out) {
    __shared__ float scratch[33];
    const int t = blockIdx.y;
    const T* __restrict__ p = (const T*)tab.p[t];
    const int64_t n = tab.n[t];
    constexpr int V = bmt::Vec16<T>::N;
    int64_t head = ((16 - ((uintptr_t)p & 15)) & 15) / sizeof(T);
    if (head > n) head = n;
    float acc = 0.f;
    if (blockIdx.x == 0)
        for (int64_t i = threadIdx.x; i < head; i += blockDim.x) { float f = bmt::Cvt<T>::to_f(p[i]); acc += f * f; }
    const T* q = p + head;
    const int64_t nvec = (n - head) / V;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
        bmt::Vec16<T> x = bmt::ld16(q + i * V);
#pragma unroll
        for (int k = 0; k < V; ++k) { float f = bmt::Cvt<T>::to_f(x.v[k]); acc += f * f; }
    }
    if (blockIdx.x == 0)
        for (int64_t i = head + nvec * V + threadIdx.x; i < n; i += blockDim.x) { float f = bmt::Cvt<T>::to_f(p[i]); acc += f * f; }
    acc = bmt::block_allreduce<false>(acc, scratch);
    if (threadIdx.x == 0 && acc != 0.f) atomicAdd(out, acc);
}

template <typename T>
__global__ void __launch_bounds__(256) scale_kernel(BmtPtrTable tab, const float* coef) {
    const float c = fminf(*coef, 1.f);
    if (c >= 1.f) return;
    const int t = blockIdx.y;
    T* __restrict__ p = (T*)tab.p[t];
    const int64_t n = tab.n[t];
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        p[i] = bmt::Cvt<T>::from_f(bmt::Cvt<T>::to_f(p[i]) * c);
}

dim3 grid_for(const BmtPtrTable* tab, int per_thread) {
    int64_t maxn = 1;
    for (int i = 0; i < tab->count; ++i) maxn = tab->n[i] > maxn ? tab->n[i] : maxn;
    int64_t bx = bmt::ceil_div64(bmt::ceil_div64(maxn, per_thread), 256);
    if (bx > 148 * 4) bx = 148 * 4;
    if (bx < 1) bx = 1;
    return dim3((unsigned)bx, (unsigned)tab->count);
}

}  // namespace

extern "C" int bmt_has_inf_nan_multi(const BmtPtrTable* tab, int dtype, void* out, void* stream) {
    if (tab->count <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 g = grid_for(tab, 32);
    if (dtype == BMT_DT_F16) infnan_kernel<__half><<<g, 256, 0, s>>>(*tab, (unsigned char*)out);
    else if (dtype == BMT_DT_BF16) infnan_kernel<__nv_bfloat16><<<g, 256, 0, s>>>(*tab, (unsigned char*)out);
    else infnan_kernel<float><<<g, 256, 0, s>>>(*tab, (unsigned char*)out);
    bmt_count_launch(1);
    return (int)cudaGetLastError();
}

extern "C" int bmt_sq_norm_multi(const BmtPtrTable* tab, int dtype, void* out, void* stream) {
    if (tab->count <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 g = grid_for(tab, 32);
    if (dtype == BMT_DT_F16) sqnorm_kernel<__half><<<g, 256, 0, s>>>(*tab, (float*)out);
    else if (dtype == BMT_DT_BF16) sqnorm_kernel<__nv_bfloat16><<<g, 256, 0, s>>>(*tab, (float*)out);
    else sqnorm_kernel<float><<<g, 256, 0, s>>>(*tab, (float*)out);
    bmt_count_launch(1);
    return (int)cudaGetLastError();
}

extern "C" int bmt_scale_multi(const BmtPtrTable* tab, int dtype, const void* coef, void* stream) {
    if (tab->count <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 g = grid_for(tab, 8);
    if (dtype == BMT_DT_F16) scale_kernel<__half><<<g, 256, 0, s>>>(*tab, (const float*)coef);
    else if (dtype == BMT_DT_BF16) scale_kernel<__nv_bfloat16><<<g, 256, 0, s>>>(*tab, (const float*)coef);
    else scale_kernel<float><<<g, 256, 0, s>>>(*tab, (const float*)coef);
    bmt_count_launch(1);
    return (int)cudaGetLastError();
}
