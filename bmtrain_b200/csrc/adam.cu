// Multi-tensor mixed-precision Adam for sm_100a.
//
// One launch updates up to 24 shards; the pointer table travels as a kernel
// argument, so nothing is copied to the device per step.  Each thread handles
// 8 elements with 128-bit loads/stores; every byte is read once and written
// once (fp16: 16 B in / 16 B out per element, bf16: 18 / 18), which makes the
// kernel a pure HBM-bandwidth problem.
//
// Math (same as the reference kernels csrc/cuda/adam_cuda.cu:8-72):
//   fp16: g stays loss-scaled; m (fp16) and v (fp32) are kept in scaled units
//         m = b1 m + (1-b1) g ; v = b2 v + (1-b2) g^2 / s
//         p -= lr * (m/bc1) / (sqrt(v s / bc2) + eps s) + lr wd p
//   bf16: g /= s first; m, v fp32 in true units; same update with s = 1.
#include "api.h"
#include "common.cuh"

namespace {

struct AdamArgs {
    float beta1, beta2, eps, lr, scale, wd, bc1, bc2;
};

template <typename T, typename M, bool SCALED_STATE>
__global__ void __launch_bounds__(256) adam_multi_kernel(BmtAdamTable tab, AdamArgs a, int64_t blocks_per_tensor_hint) {
    // grid: x = chunk within a tensor, y = tensor
    const int t = blockIdx.y;
    const int64_t n = tab.n[t];
    float* __restrict__ p32 = (float*)tab.p32[t];
    T* __restrict__ p16 = (T*)tab.p16[t];
    const T* __restrict__ g = (const T*)tab.g[t];
    M* __restrict__ m = (M*)tab.m[t];
    float* __restrict__ v = (float*)tab.v[t];

    const float inv_scale = 1.f / a.scale;
    const int64_t nvec = n / 8;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
        const int64_t e = i * 8;
        bmt::Vec16<T> gv = bmt::ld16(g + e);
        float4 pa = *reinterpret_cast<const float4*>(p32 + e), pb = *reinterpret_cast<const float4*>(p32 + e + 4);
        float4 va = *reinterpret_cast<const float4*>(v + e), vb = *reinterpret_cast<const float4*>(v + e + 4);
        float pf[8] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w};
        float vf[8] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
        float mf[8];
        if constexpr (sizeof(M) == 2) {
            bmt::Vec16<M> mv = bmt::ld16(m + e);
#pragma unroll
            for (int k = 0; k < 8; ++k) mf[k] = bmt::Cvt<M>::to_f(mv.v[k]);
        } else {
            float4 ma = *reinterpret_cast<const float4*>((const float*)m + e), mb = *reinterpret_cast<const float4*>((const float*)m + e + 4);
            mf[0] = ma.x; mf[1] = ma.y; mf[2] = ma.z; mf[3] = ma.w; mf[4] = mb.x; mf[5] = mb.y; mf[6] = mb.z; mf[7] = mb.w;
        }
        bmt::Vec16<T> po;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            float gf = bmt::Cvt<T>::to_f(gv.v[k]);
            float upd;
            if constexpr (SCALED_STATE) {
                mf[k] = a.beta1 * mf[k] + (1.f - a.beta1) * gf;
                vf[k] = a.beta2 * vf[k] + (1.f - a.beta2) * gf * gf * inv_scale;
                upd = (mf[k] / a.bc1) / (sqrtf(vf[k] * a.scale / a.bc2) + a.eps * a.scale);
            } else {
                gf *= inv_scale;
                mf[k] = a.beta1 * mf[k] + (1.f - a.beta1) * gf;
                vf[k] = a.beta2 * vf[k] + (1.f - a.beta2) * gf * gf;
                upd = (mf[k] / a.bc1) / (sqrtf(vf[k] / a.bc2) + a.eps);
            }
            pf[k] = pf[k] - a.lr * upd - a.lr * a.wd * pf[k];
            po.v[k] = bmt::Cvt<T>::from_f(pf[k]);
        }
        *reinterpret_cast<float4*>(p32 + e) = make_float4(pf[0], pf[1], pf[2], pf[3]);
        *reinterpret_cast<float4*>(p32 + e + 4) = make_float4(pf[4], pf[5], pf[6], pf[7]);
        *reinterpret_cast<float4*>(v + e) = make_float4(vf[0], vf[1], vf[2], vf[3]);
        *reinterpret_cast<float4*>(v + e + 4) = make_float4(vf[4], vf[5], vf[6], vf[7]);
        bmt::st16(p16 + e, po);
        if constexpr (sizeof(M) == 2) {
            bmt::Vec16<M> mo;
#pragma unroll
            for (int k = 0; k < 8; ++k) mo.v[k] = bmt::Cvt<M>::from_f(mf[k]);
            bmt::st16(m + e, mo);
        } else {
            *reinterpret_cast<float4*>((float*)m + e) = make_float4(mf[0], mf[1], mf[2], mf[3]);
            *reinterpret_cast<float4*>((float*)m + e + 4) = make_float4(mf[4], mf[5], mf[6], mf[7]);
        }
    }
    // scalar tail (n not a multiple of 8)
    if (blockIdx.x == 0) {
        for (int64_t e = nvec * 8 + threadIdx.x; e < n; e += blockDim.x) {
            float gf = bmt::Cvt<T>::to_f(g[e]);
            float mm = bmt::Cvt<M>::to_f(m[e]), vv = v[e], pp = p32[e], upd;
            if constexpr (SCALED_STATE) {
                mm = a.beta1 * mm + (1.f - a.beta1) * gf;
                vv = a.beta2 * vv + (1.f - a.beta2) * gf * gf * inv_scale;
                upd = (mm / a.bc1) / (sqrtf(vv * a.scale / a.bc2) + a.eps * a.scale);
            } else {
                gf *= inv_scale;
                mm = a.beta1 * mm + (1.f - a.beta1) * gf;
                vv = a.beta2 * vv + (1.f - a.beta2) * gf * gf;
                upd = (mm / a.bc1) / (sqrtf(vv / a.bc2) + a.eps);
            }
            pp = pp - a.lr * upd - a.lr * a.wd * pp;
            p32[e] = pp; p16[e] = bmt::Cvt<T>::from_f(pp); m[e] = bmt::Cvt<M>::from_f(mm); v[e] = vv;
        }
    }
}

template <typename T, typename M, bool S>
int launch(const BmtAdamTable* tab, AdamArgs a, cudaStream_t stream) {
    if (tab->count <= 0) return 0;
    int64_t maxn = 0;
    for (int i = 0; i < tab->count; ++i) {
        maxn = tab->n[i] > maxn ? tab->n[i] : maxn;
        // vector path needs 16-byte aligned bases
        if (((uintptr_t)tab->p32[i] | (uintptr_t)tab->p16[i] | (uintptr_t)tab->g[i] | (uintptr_t)tab->m[i] | (uintptr_t)tab->v[i]) & 15) return -2;
    }
    int64_t bx = bmt::ceil_div64(bmt::ceil_div64(maxn, 8), 256);
    if (bx < 1) bx = 1;
    if (bx > 148 * 8) bx = 148 * 8;
    dim3 grid((unsigned)bx, (unsigned)tab->count);
    adam_multi_kernel<T, M, S><<<grid, 256, 0, stream>>>(*tab, a, bx);
    bmt_count_launch(1);
    return (int)cudaGetLastError();
}

}  // namespace

extern "C" int bmt_adam_fp16_multi(const BmtAdamTable* tab, float beta1, float beta2, float eps, float lr, float scale,
                                   float wd, float bc1, float bc2, void* stream) {
    return launch<__half, __half, true>(tab, AdamArgs{beta1, beta2, eps, lr, scale, wd, bc1, bc2}, (cudaStream_t)stream);
}

// fp16 parameters with fp32 moments in true (unscaled) units: the layout of the host-offloaded optimizer state.
extern "C" int bmt_adam_fp16_f32state_multi(const BmtAdamTable* tab, float beta1, float beta2, float eps, float lr, float scale,
                                            float wd, float bc1, float bc2, void* stream) {
    return launch<__half, float, false>(tab, AdamArgs{beta1, beta2, eps, lr, scale, wd, bc1, bc2}, (cudaStream_t)stream);
}

extern "C" int bmt_adam_bf16_multi(const BmtAdamTable* tab, float beta1, float beta2, float eps, float lr, float scale,
                                   float wd, float bc1, float bc2, void* stream) {
    return launch<__nv_bfloat16, float, false>(tab, AdamArgs{beta1, beta2, eps, lr, scale, wd, bc1, bc2}, (cudaStream_t)stream);
}
