// Shared device helpers for the sm_100a kernels: dtype traits, 128-bit vector
// access, warp / block reductions.  (Reference counterpart: csrc/cuda/reduce.cuh,
// which offers shuffle + 32-float shared-memory block reductions only.)
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define BMT_DT_F16 0
#define BMT_DT_BF16 1
#define BMT_DT_F32 2

namespace bmt {

template <typename T> struct Cvt;
template <> struct Cvt<__half> {
    static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
};
template <> struct Cvt<__nv_bfloat16> {
    static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Cvt<float> {
    static __device__ __forceinline__ float to_f(float v) { return v; }
    static __device__ __forceinline__ float from_f(float v) { return v; }
};

// A 16-byte packet of T (8 halves or 4 floats).
template <typename T> struct alignas(16) Vec16 {
    static constexpr int N = 16 / sizeof(T);
    T v[N];
};

template <typename T> __device__ __forceinline__ Vec16<T> ld16(const T* p) {
    return *reinterpret_cast<const Vec16<T>*>(p);
}
template <typename T> __device__ __forceinline__ void st16(T* p, const Vec16<T>& x) {
    *reinterpret_cast<Vec16<T>*>(p) = x;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide all-reduce (every thread gets the result). `scratch` holds >= 33 floats.
template <bool IsMax> __device__ __forceinline__ float block_allreduce(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    v = IsMax ? warp_max(v) : warp_sum(v);
    __syncthreads();  // scratch may still be read from a previous call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nwarp) ? scratch[lane] : (IsMax ? -INFINITY : 0.f);
    r = IsMax ? warp_max(r) : warp_sum(r);
    return r;
}

__host__ __device__ __forceinline__ int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

}  // namespace bmt

#define BMT_CUDA_OK(expr)                        \
    do {                                         \
        cudaError_t _e = (expr);                 \
        if (_e != cudaSuccess) return (int)_e;   \
    } while (0)
