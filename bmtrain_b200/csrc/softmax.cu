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

// Warp-per-row variants for rows of up to 2048 elements whose pitch keeps 16-byte alignment: the row lives in
// registers (8-element packets per lane), reductions are shuffles only, no shared memory and no block barrier.
constexpr int WMAX = 8;  // packets per lane: 8 * 8 * 32 = 2048 columns

template <typename T>
__global__ void __launch_bounds__(128) masked_softmax_warp_kernel(int64_t rows, int64_t h, int64_t sq, int64_t sk, int64_t ld,
                                                                  T* __restrict__ s, int causal, const unsigned char* __restrict__ mask,
                                                                  const int* __restrict__ kv_lens) {
    const int lane = threadIdx.x & 31;
    const int64_t r = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (r >= rows) return;
    const int64_t q = r % sq, b = r / (sq * h);
    T* __restrict__ sr = s + r * ld;
    const unsigned char* __restrict__ mr = mask ? mask + (b * sq + q) * sk : nullptr;
    int64_t limit = sk;
    if (causal) { int64_t c = q + sk - sq + 1; limit = c < limit ? c : limit; }
    if (kv_lens) { int64_t c = kv_lens[b]; limit = c < limit ? c : limit; }
    float v[WMAX][8];
    float mx = -INFINITY;
    const bool mask_vec = mr && ((sk & 7) == 0);
#pragma unroll
    for (int it = 0; it < WMAX; ++it) {
        const int64_t c = ((int64_t)it * 32 + lane) * 8;
        if (c < sk) {
            bmt::Vec16<T> x = bmt::ld16(sr + c);
            unsigned long long mbits = ~0ull;
            if (mask_vec) mbits = *reinterpret_cast<const unsigned long long*>(mr + c);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                bool keep = (c + k) < limit;
                if (mr) keep = keep && (mask_vec ? ((mbits >> (8 * k)) & 0xff) != 0 : ((c + k) < sk && mr[c + k] != 0));
                v[it][k] = keep ? bmt::Cvt<T>::to_f(x.v[k]) : -INFINITY;
                mx = fmaxf(mx, v[it][k]);
            }
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) v[it][k] = -INFINITY;
        }
    }
    mx = bmt::warp_max(mx);
    float sum = 0.f;
    if (mx != -INFINITY) {
#pragma unroll
        for (int it = 0; it < WMAX; ++it)
#pragma unroll
            for (int k = 0; k < 8; ++k) { v[it][k] = __expf(v[it][k] - mx); sum += v[it][k]; }
    }
    sum = bmt::warp_sum(sum);
    const float inv = (mx == -INFINITY || sum == 0.f) ? 0.f : 1.f / sum;
#pragma unroll
    for (int it = 0; it < WMAX; ++it) {
        const int64_t c = ((int64_t)it * 32 + lane) * 8;
        if (c < sk) {
            bmt::Vec16<T> o;
#pragma unroll
            for (int k = 0; k < 8; ++k) o.v[k] = bmt::Cvt<T>::from_f(mx == -INFINITY ? 0.f : v[it][k] * inv);
            bmt::st16(sr + c, o);  // columns in [sk, ld) of the last packet are padding and may be written
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(128) softmax_bwd_warp_kernel(int64_t rows, int64_t cols, int64_t ld, const T* __restrict__ p,
                                                               T* __restrict__ dp, float scale) {
    const int lane = threadIdx.x & 31;
    const int64_t r = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (r >= rows) return;
    const T* __restrict__ pr = p + r * ld;
    T* __restrict__ dr = dp + r * ld;
    float pv[WMAX][8], dv[WMAX][8];
    float acc = 0.f;
#pragma unroll
    for (int it = 0; it < WMAX; ++it) {
        const int64_t c = ((int64_t)it * 32 + lane) * 8;
        if (c < cols) {
            bmt::Vec16<T> a = bmt::ld16(pr + c), g = bmt::ld16(dr + c);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const bool in = (c + k) < cols;
                pv[it][k] = in ? bmt::Cvt<T>::to_f(a.v[k]) : 0.f;
                dv[it][k] = in ? bmt::Cvt<T>::to_f(g.v[k]) : 0.f;
                acc += pv[it][k] * dv[it][k];
            }
        }
    }
    acc = bmt::warp_sum(acc);
#pragma unroll
    for (int it = 0; it < WMAX; ++it) {
        const int64_t c = ((int64_t)it * 32 + lane) * 8;
        if (c < cols) {
            bmt::Vec16<T> o;
#pragma unroll
            for (int k = 0; k < 8; ++k) o.v[k] = bmt::Cvt<T>::from_f(pv[it][k] * (dv[it][k] - acc) * scale);
            bmt::st16(dr + c, o);
        }
    }
}

}  // namespace

extern "C" int bmt_masked_softmax(int64_t b, int64_t h, int64_t sq, int64_t sk, int64_t ld, void* scores, int dtype, int causal,
                                  const void* mask, const void* kv_lens, void* stream) {
    const int64_t rows = b * h * sq;
    if (rows <= 0) return 0;
    if (sk * 4 > 200 * 1024) return -3;
    cudaStream_t s = (cudaStream_t)stream;
    if (sk <= WMAX * 256 && (ld & 7) == 0 && (((uintptr_t)scores) & 15) == 0 && ld >= ((sk + 7) / 8) * 8) {
        const unsigned g = (unsigned)((rows + 3) / 4);
        if (dtype == BMT_DT_F16) masked_softmax_warp_kernel<__half><<<g, 128, 0, s>>>(rows, h, sq, sk, ld, (__half*)scores, causal, (const unsigned char*)mask, (const int*)kv_lens);
        else masked_softmax_warp_kernel<__nv_bfloat16><<<g, 128, 0, s>>>(rows, h, sq, sk, ld, (__nv_bfloat16*)scores, causal, (const unsigned char*)mask, (const int*)kv_lens);
        bmt_count_launch(1);
        return (int)cudaGetLastError();
    }
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
    if (cols <= WMAX * 256 && (ld & 7) == 0 && ((((uintptr_t)p) | ((uintptr_t)dp)) & 15) == 0 && ld >= ((cols + 7) / 8) * 8) {
        const unsigned g = (unsigned)((rows + 3) / 4);
        if (dtype == BMT_DT_F16) softmax_bwd_warp_kernel<__half><<<g, 128, 0, s>>>(rows, cols, ld, (const __half*)p, (__half*)dp, scale);
        else softmax_bwd_warp_kernel<__nv_bfloat16><<<g, 128, 0, s>>>(rows, cols, ld, (const __nv_bfloat16*)p, (__nv_bfloat16*)dp, scale);
        bmt_count_launch(1);
        return (int)cudaGetLastError();
    }
    if (dtype == BMT_DT_F16) softmax_bwd_kernel<__half><<<(unsigned)rows, 128, 0, s>>>(cols, ld, (const __half*)p, (__half*)dp, scale);
    else softmax_bwd_kernel<__nv_bfloat16><<<(unsigned)rows, 128, 0, s>>>(cols, ld, (const __nv_bfloat16*)p, (__nv_bfloat16*)dp, scale);
    bmt_count_launch(1);
    return (int)cudaGetLastError();
}
