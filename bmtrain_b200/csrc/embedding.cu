// Embedding gather and fp32 scatter-add (ids < 0: zeros in forward, skipped in backward).
#include "api.h"
#include "common.cuh"

namespace {

template <typename T>
__global__ void __launch_bounds__(128) emb_fwd_kernel(int64_t d, const int64_t* __restrict__ ids, const T* __restrict__ w, T* __restrict__ out) {
    const int64_t t = blockIdx.x;
    const int64_t id = ids[t];
    T* __restrict__ o = out + t * d;
    constexpr int V = bmt::Vec16<T>::N;
    if (id < 0) {
        bmt::Vec16<T> z;
#pragma unroll
        for (int k = 0; k < V; ++k) z.v[k] = bmt::Cvt<T>::from_f(0.f);
        for (int64_t c = threadIdx.x * V; c < d; c += blockDim.x * V) bmt::st16(o + c, z);
        return;
    }
    const T* __restrict__ src = w + id * d;
    for (int64_t c = threadIdx.x * V; c < d; c += blockDim.x * V) bmt::st16(o + c, bmt::ld16(src + c));
}

template <typename T>
__global__ void __launch_bounds__(128) emb_bwd_kernel(int64_t d, const int64_t* __restrict__ ids, const T* __restrict__ g, float* __restrict__ acc) {
    const int64_t t = blockIdx.x;
    const int64_t id = ids[t];
    if (id < 0) return;
    const T* __restrict__ gr = g + t * d;
    float* __restrict__ a = acc + id * d;
    constexpr int V = bmt::Vec16<T>::N;
    for (int64_t c = threadIdx.x * V; c < d; c += blockDim.x * V) {
        bmt::Vec16<T> v = bmt::ld16(gr + c);
#pragma unroll
        for (int k = 0; k < V; ++k) atomicAdd(a + c + k, bmt::Cvt<T>::to_f(v.v[k]));
    }
}

}  // namespace

extern "C" int bmt_embedding_fwd(int64_t tokens, int64_t d, const void* ids, const void* weight, int dtype, void* out, void* stream) {
    if (tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == BMT_DT_F32) { if (d % 4) return -3; emb_fwd_kernel<float><<<(unsigned)tokens, 128, 0, s>>>(d, (const int64_t*)ids, (const float*)weight, (float*)out); }
    else { if (d % 8) return -3;
        if (dtype == BMT_DT_F16) emb_fwd_kernel<__half><<<(unsigned)tokens, 128, 0, s>>>(d, (const int64_t*)ids, (const __half*)weight, (__half*)out);
        else emb_fwd_kernel<__nv_bfloat16><<<(unsigned)tokens, 128, 0, s>>>(d, (const int64_t*)ids, (const __nv_bfloat16*)weight, (__nv_bfloat16*)out); }
    bmt_count_launch(1);
    return (int)cudaGetLastError();
}

extern "C" int bmt_embedding_bwd(int64_t tokens, int64_t d, const void* ids, const void* grad, int dtype, void* acc, void* stream) {
    if (tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == BMT_DT_F32) { if (d % 4) return -3; emb_bwd_kernel<float><<<(unsigned)tokens, 128, 0, s>>>(d, (const int64_t*)ids, (const float*)grad, (float*)acc); }
    else { if (d % 8) return -3;
        if (dtype == BMT_DT_F16) emb_bwd_kernel<__half><<<(unsigned)tokens, 128, 0, s>>>(d, (const int64_t*)ids, (const __half*)grad, (float*)acc);
        else emb_bwd_kernel<__nv_bfloat16><<<(unsigned)tokens, 128, 0, s>>>(d, (const int64_t*)ids, (const __nv_bfloat16*)grad, (float*)acc); }
    bmt_count_launch(1);
    return (int)cudaGetLastError();
}
