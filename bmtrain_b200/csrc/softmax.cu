// Masked softmax over attention scores (in place) and its backward.
//
// Forward: scores (b, h, sq, sk) half; keep[b,q,k] = (!causal || k <= q + sk - sq) && (!mask || mask[b,q,k])
//          && (!kv_lens || k < kv_lens[b]); masked entries become 0, fully masked rows become all 0.
// Backward: dp <- p * (dp - sum_k dp*p) * scale, in place on dp.
// One CTA per row, the row is held in shared memory as fp32.  Rows are `ld` elements apart (ld >= sk).
#include "api.h"
#include "common.cuh"

namespace {

template <typename T>
__global__ void __launch_bounds__(128) masked_softmax_kernel(int64_t h, int64_t sq, int64_t sk, int64_t ld, T* __restrict__ s, int causal,
                                                             const unsigned char* __restrict__ mask, const int* __restrict__ kv_lens) {
    extern __shared__ float row[];
    __shared__ float scratch[33];
    const int64_t r = blockIdx.x;           // (b, h, q) flattened
    const int64_t q = r % sq;
    const int64_t b = r / (sq * h);
    T* __restrict__ sr = s + r * ld;
    const unsigned char* __restrict__ mr = mask ? mask + (b * sq + q) * sk : nullptr;
    int64_t limit = sk;
    if (causal) { int64_t c = q + sk - sq + 1; limit = c < limit ? c : limit; }
    if (kv_lens) { int64_t c = kv_lens[b]; limit = c < limit ? c : limit; }
    float mx = -INFINITY;
    for (int64_t k = threadIdx.x; k < sk; k += blockDim.x) {
        float f = -INFINITY;
        if (k < limit && (!mr || mr[k])) f = bmt::Cvt<T>::to_f(sr[k]);
        row[k] = f;
        mx = fmaxf(mx, f);
    }
    mx = bmt::block_allreduce<true>(mx, scratch);
    float sum = 0.f;
    if (mx != -INFINITY)
        for (int64_t k = threadIdx.x; k < sk; k += blockDim.x) { float e = __expf(row[k] - mx); row[k] = e; sum += e; }
    sum = bmt::block_allreduce<false>(sum, scratch);
    const float inv = (mx == -INFINITY || sum == 0.f) ? 0.f : 1.f / sum;
    for (int64_t k = threadIdx.x; k < sk; k += blockDim.x)
        sr[k] = bmt::Cvt<T>::from_f(mx == -INFINITY ? 0.f : row[k] * inv);
}

template <typename T>
__global__ void __launch_bounds__(128) softmax_bwd_kernel(int64_t cols, int64_t ld, const T* __restrict__ p, T* __restrict__ dp, float scale) {
    __shared__ float scratch[33];
    const int64_t r = blockIdx.x;
    const T* __restrict__ pr = p + r * ld;
    T* __restrict__ dr = dp + r * ld;
    float acc = 0.f;
    for (int64_t k = threadIdx.x; k < cols; k += blockDim.x) acc += bmt::Cvt<T>::to_f(pr[k]) * bmt::Cvt<T>::to_f(dr[k]);
    acc = bmt::block_allreduce<false>(acc, scratch);
    for (int64_t k = threadIdx.x; k < cols; k += blockDim.x) {
        const float pv = bmt::Cvt<T>::to_f(pr[k]);
        dr[k] = bmt::Cvt<T>::from_f(pv * (bmt::Cvt<T>::to_f(dr[k]) - acc) * scale);
    }
}

}  // namespace

extern "C" int bmt_masked_softmax(int64_t b, int64_t h, int64_t sq, int64_t sk, int64_t ld, void* scores, int dtype, int causal,
                                  const void* mask, const void* kv_lens, void* stream) {
    const int64_t rows = b * h * sq;
    if (rows <= 0) return 0;
    if (sk * 4 > 200 * 1024) return -3;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = sk * sizeof(float);
    if (dtype == BMT_DT_F16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(masked_softmax_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        masked_softmax_kernel<__half><<<(unsigned)rows, 128, smem, s>>>(h, sq, sk, ld, (__half*)scores, causal, (const unsigned char*)mask, (const int*)kv_lens);
    } else {
        if (smem > 48 * 1024) cudaFuncSetAttribute(masked_softmax_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        masked_softmax_kernel<__nv_bfloat16><<<(unsigned)rows, 128, smem, s>>>(h, sq, sk, ld, (__nv_bfloat16*)scores, causal, (const unsigned char*)mask, (const int*)kv_lens);
    }
    bmt_count_launch(1);
    return (int)cudaGetLastError();
}

extern "C" int bmt_softmax_bwd(int64_t rows, int64_t cols, int64_t ld, const void* p, void* dp, float scale, int dtype, void* stream) {
    if (rows <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == BMT_DT_F16) softmax_bwd_kernel<__half><<<(unsigned)rows, 128, 0, s>>>(cols, ld, (const __half*)p, (__half*)dp, scale);
    else softmax_bwd_kernel<__nv_bfloat16><<<(unsigned)rows, 128, 0, s>>>(cols, ld, (const __nv_bfloat16*)p, (__nv_bfloat16*)dp, scale);
    bmt_count_launch(1);
    return (int)cudaGetLastError();
}
