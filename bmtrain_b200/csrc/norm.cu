// LayerNorm / RMSNorm forward and backward for sm_100a.
//
// Forward: one CTA per row; the row is staged once in shared memory as fp32, mean and
// variance are exact two-pass statistics over that copy, the output is written with
// 128-bit stores.  Saves (mean, rstd) per row.
// Backward: a persistent grid (nblk CTAs) strides over the rows; each CTA produces dx for
// its rows and keeps per-thread partial dgamma / dbeta in registers, written once to a
// (nblk x d) fp32 scratch that a second kernel folds over nblk.
// (The reference calls F.layer_norm: example/layers/layernorm.py:29.)
#include <stdlib.h>

#include "api.h"
#include "common.cuh"

namespace {

constexpr int NT = 256;
constexpr int MAXIT = 8;  // d <= NT * 8 * MAXIT = 16384

template <typename T>
__global__ void __launch_bounds__(NT) norm_fwd_kernel(int64_t rows, int d, const T* __restrict__ x, const T* __restrict__ w,
                                                      const T* __restrict__ b, float eps, int rms, T* __restrict__ y,
                                                      float* __restrict__ stats) {
    extern __shared__ float row[];
    __shared__ float scratch[33];
    const int64_t r = blockIdx.x;
    const T* __restrict__ xr = x + r * d;
    float s = 0.f;
    for (int c = threadIdx.x * 8; c < d; c += NT * 8) {
        bmt::Vec16<T> v = bmt::ld16(xr + c);
#pragma unroll
        for (int k = 0; k < 8; ++k) { float f = bmt::Cvt<T>::to_f(v.v[k]); row[c + k] = f; s += f; }
    }
    float mean = 0.f;
    if (!rms) mean = bmt::block_allreduce<false>(s, scratch) / d;
    float q = 0.f;
    for (int c = threadIdx.x * 8; c < d; c += NT * 8) {
#pragma unroll
        for (int k = 0; k < 8; ++k) { float f = row[c + k] - mean; q += f * f; }
    }
    const float var = bmt::block_allreduce<false>(q, scratch) / d;
    const float rstd = rsqrtf(var + eps);
    if (threadIdx.x == 0) { stats[r] = mean; stats[rows + r] = rstd; }
    T* __restrict__ yr = y + r * d;
    for (int c = threadIdx.x * 8; c < d; c += NT * 8) {
        bmt::Vec16<T> wv = bmt::ld16(w + c), o;
        bmt::Vec16<T> bv;
        if (b) bv = bmt::ld16(b + c);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            float f = (row[c + k] - mean) * rstd * bmt::Cvt<T>::to_f(wv.v[k]);
            if (b) f += bmt::Cvt<T>::to_f(bv.v[k]);
            o.v[k] = bmt::Cvt<T>::from_f(f);
        }
        bmt::st16(yr + c, o);
    }
}

template <typename T>
__global__ void __launch_bounds__(NT) norm_bwd_kernel(int64_t rows, int d, const T* __restrict__ x, const T* __restrict__ dy,
                                                      const T* __restrict__ w, const float* __restrict__ stats, int rms,
                                                      T* __restrict__ dx, float* __restrict__ partial, const T* __restrict__ dres) {
    __shared__ float scratch[33];
    float dg[MAXIT][8], db[MAXIT][8];
#pragma unroll
    for (int it = 0; it < MAXIT; ++it)
#pragma unroll
        for (int k = 0; k < 8; ++k) dg[it][k] = db[it][k] = 0.f;

    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const float mean = stats[r], rstd = stats[rows + r];
        const T* __restrict__ xr = x + r * d;
        const T* __restrict__ gr = dy + r * d;
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int it = 0; it < MAXIT; ++it) {
            const int c = threadIdx.x * 8 + it * NT * 8;
            if (c < d) {
                bmt::Vec16<T> xv = bmt::ld16(xr + c), gv = bmt::ld16(gr + c), wv = bmt::ld16(w + c);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const float xh = (bmt::Cvt<T>::to_f(xv.v[k]) - mean) * rstd;
                    const float g = bmt::Cvt<T>::to_f(gv.v[k]);
                    const float wg = g * bmt::Cvt<T>::to_f(wv.v[k]);
                    s1 += wg; s2 += wg * xh;
                    dg[it][k] += g * xh; db[it][k] += g;
                }
            }
        }
        if (rms) s1 = 0.f; else s1 = bmt::block_allreduce<false>(s1, scratch) / d;
        s2 = bmt::block_allreduce<false>(s2, scratch) / d;
        T* __restrict__ dr = dx + r * d;
#pragma unroll
        for (int it = 0; it < MAXIT; ++it) {
            const int c = threadIdx.x * 8 + it * NT * 8;
            if (c < d) {
                bmt::Vec16<T> xv = bmt::ld16(xr + c), gv = bmt::ld16(gr + c), wv = bmt::ld16(w + c), o, rv;
                if (dres) rv = bmt::ld16(dres + r * d + c);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const float xh = (bmt::Cvt<T>::to_f(xv.v[k]) - mean) * rstd;
                    const float wg = bmt::Cvt<T>::to_f(gv.v[k]) * bmt::Cvt<T>::to_f(wv.v[k]);
                    float val = rstd * (wg - s1 - xh * s2);
                    if (dres) val += bmt::Cvt<T>::to_f(rv.v[k]);
                    o.v[k] = bmt::Cvt<T>::from_f(val);
                }
                bmt::st16(dr + c, o);
            }
        }
    }
    float* pg = partial + (int64_t)blockIdx.x * d;
    float* pb = partial + ((int64_t)gridDim.x + blockIdx.x) * d;
#pragma unroll
    for (int it = 0; it < MAXIT; ++it) {
        const int c = threadIdx.x * 8 + it * NT * 8;
        if (c < d) {
#pragma unroll
            for (int k = 0; k < 8; ++k) { pg[c + k] = dg[it][k]; pb[c + k] = db[it][k]; }
        }
    }
}

// Fold the per-CTA partial sums: block = 32 columns x 32 row lanes, rows strided over the lanes, smem tree at the end.
template <typename T, bool ACC = false>
__global__ void __launch_bounds__(1024) norm_fold_kernel(int d, int nblk, const float* __restrict__ partial, T* __restrict__ dw, T* __restrict__ db) {
    // ACC: dw / db already hold gradients of earlier passes and are added to
    __shared__ float sa[32][33], sb[32][33];
    const int tx = threadIdx.x, ty = threadIdx.y;
    const int c = blockIdx.x * 32 + tx;
    float a = 0.f, bsum = 0.f;
    if (c < d) {
        for (int i = ty; i < nblk; i += 32) {
            a += partial[(int64_t)i * d + c];
            bsum += partial[((int64_t)nblk + i) * d + c];
        }
    }
    sa[ty][tx] = a; sb[ty][tx] = bsum;
    __syncthreads();
    if (ty == 0 && c < d) {
        float ra = 0.f, rb = 0.f;
#pragma unroll 8
        for (int l = 0; l < 32; ++l) { ra += sa[l][tx]; rb += sb[l][tx]; }
        if (ACC) {
            ra += bmt::Cvt<T>::to_f(dw[c]);
            if (db) rb += bmt::Cvt<T>::to_f(db[c]);
        }
        dw[c] = bmt::Cvt<T>::from_f(ra);
        if (db) db[c] = bmt::Cvt<T>::from_f(rb);
    }
}

// Forward with the row held in registers: WPR warps share a row (8 / WPR rows per CTA at a time), every lane keeps VPL
// 16-byte vectors, all of whose loads are issued before the first use; statistics are exact two-pass sums over the
// registers, reduced with shuffles (and one shared-memory exchange when WPR > 1).  A persistent grid strides over the
// rows.
template <typename T, int VPL, int WPR>
__global__ void __launch_bounds__(NT, 2) norm_fwd_reg_kernel(int64_t rows, int d, const T* __restrict__ x, const T* __restrict__ w,
                                                          const T* __restrict__ b, float eps, int rms, T* __restrict__ y,
                                                          float* __restrict__ stats) {
    constexpr int RPC = 8 / WPR;                       // rows a CTA works on at a time
    __shared__ float ex[2][8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = warp % WPR, slot = warp / WPR;     // position inside the row's warp team, row slot inside the CTA
    const int64_t groups = (rows + RPC - 1) / RPC;
    for (int64_t gi = blockIdx.x; gi < groups; gi += gridDim.x) {
        const int64_t r = gi * RPC + slot;
        const bool live = r < rows;
        float f[VPL][8];
        float s = 0.f;
#pragma unroll
        for (int v = 0; v < VPL; ++v) {
            const int c = ((v * WPR + sub) * 32 + lane) * 8;
            if (live && c < d) {
                const bmt::Vec16<T> t = bmt::ld16(x + r * d + c);
#pragma unroll
                for (int k = 0; k < 8; ++k) { f[v][k] = bmt::Cvt<T>::to_f(t.v[k]); s += f[v][k]; }
            } else {
#pragma unroll
                for (int k = 0; k < 8; ++k) f[v][k] = 0.f;
            }
        }
        float mean = 0.f;
        if (!rms) {
            s = bmt::warp_sum(s);
            if (WPR > 1) {
                if (lane == 0) ex[0][warp] = s;
                __syncthreads();
                s = 0.f;
#pragma unroll
                for (int i = 0; i < WPR; ++i) s += ex[0][slot * WPR + i];
            }
            mean = s / d;
        }
        float q = 0.f;
#pragma unroll
        for (int v = 0; v < VPL; ++v) {
            const int c = ((v * WPR + sub) * 32 + lane) * 8;
            if (c < d) {
#pragma unroll
                for (int k = 0; k < 8; ++k) { const float t = f[v][k] - mean; q += t * t; }
            }
        }
        q = bmt::warp_sum(q);
        if (WPR > 1) {
            if (lane == 0) ex[1][warp] = q;
            __syncthreads();
            q = 0.f;
#pragma unroll
            for (int i = 0; i < WPR; ++i) q += ex[1][slot * WPR + i];
        }
        const float rstd = rsqrtf(q / d + eps);
        if (live && sub == 0 && lane == 0) { stats[r] = mean; stats[rows + r] = rstd; }
#pragma unroll
        for (int v = 0; v < VPL; ++v) {
            const int c = ((v * WPR + sub) * 32 + lane) * 8;
            if (live && c < d) {
                // weight and bias stay hot in L1 (a few KB re-read by every row); keeping them in registers instead would
                // halve the number of resident warps and with it the bytes in flight
                const bmt::Vec16<T> wv = bmt::ld16(w + c);
                bmt::Vec16<T> bv, o;
                if (b) bv = bmt::ld16(b + c);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    float t = (f[v][k] - mean) * rstd * bmt::Cvt<T>::to_f(wv.v[k]);
                    if (b) t += bmt::Cvt<T>::to_f(bv.v[k]);
                    o.v[k] = bmt::Cvt<T>::from_f(t);
                }
                bmt::st16(y + r * d + c, o);
            }
        }
        if (WPR > 1) __syncthreads();   // the exchange slots are reused by the next group
    }
}

// Streaming form of the kernel above: the row stays packed (16-byte vectors) in registers and the loads of the CTA's next
// group of rows are issued before the arithmetic on the current one starts, so every warp has VPL loads in flight all the
// time instead of only at the top of each row.  The exchange slots of a row's warp team alternate between two sets, which
// saves the barrier at the end of a group.
template <typename T, int VPL, int WPR>
__global__ void __launch_bounds__(NT, VPL <= 4 ? 3 : 2) norm_fwd_stream_kernel(int64_t rows, int d, const T* __restrict__ x, const T* __restrict__ w,
                                                             const T* __restrict__ b, float eps, int rms, T* __restrict__ y,
                                                             float* __restrict__ stats) {
    constexpr int RPC = 8 / WPR;
    __shared__ float ex[2][2][8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = warp % WPR, slot = warp / WPR;
    const int64_t groups = (rows + RPC - 1) / RPC;
    bmt::Vec16<T> cur[VPL], nxt[VPL];
    const auto load = [&](bmt::Vec16<T>(&v)[VPL], int64_t gi) {
        const int64_t r = gi * RPC + slot;
        if (r < rows) {
#pragma unroll
            for (int i = 0; i < VPL; ++i) {
                const int c = ((i * WPR + sub) * 32 + lane) * 8;
                if (c < d) v[i] = bmt::ld16(x + r * d + c);
            }
        }
    };
    int64_t gi = blockIdx.x;
    if (gi < groups) load(cur, gi);
    int par = 0;
    for (; gi < groups; gi += gridDim.x, par ^= 1) {
        if (gi + gridDim.x < groups) load(nxt, gi + gridDim.x);
        const int64_t r = gi * RPC + slot;
        const bool live = r < rows;
        float mean = 0.f;
        if (!rms) {
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < VPL; ++i) {
                const int c = ((i * WPR + sub) * 32 + lane) * 8;
                if (live && c < d) {
#pragma unroll
                    for (int k = 0; k < 8; ++k) s += bmt::Cvt<T>::to_f(cur[i].v[k]);
                }
            }
            s = bmt::warp_sum(s);
            if (WPR > 1) {
                if (lane == 0) ex[par][0][warp] = s;
                __syncthreads();
                s = 0.f;
#pragma unroll
                for (int i = 0; i < WPR; ++i) s += ex[par][0][slot * WPR + i];
            }
            mean = s / d;
        }
        float q = 0.f;
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            const int c = ((i * WPR + sub) * 32 + lane) * 8;
            if (live && c < d) {
#pragma unroll
                for (int k = 0; k < 8; ++k) { const float t = bmt::Cvt<T>::to_f(cur[i].v[k]) - mean; q += t * t; }
            }
        }
        q = bmt::warp_sum(q);
        if (WPR > 1) {
            if (lane == 0) ex[par][1][warp] = q;
            __syncthreads();
            q = 0.f;
#pragma unroll
            for (int i = 0; i < WPR; ++i) q += ex[par][1][slot * WPR + i];
        }
        const float rstd = rsqrtf(q / d + eps);
        if (live && sub == 0 && lane == 0) { stats[r] = mean; stats[rows + r] = rstd; }
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            const int c = ((i * WPR + sub) * 32 + lane) * 8;
            if (live && c < d) {
                const bmt::Vec16<T> wv = bmt::ld16(w + c);   // a few KB re-read by every row: stays in L1
                bmt::Vec16<T> bv, o;
                if (b) bv = bmt::ld16(b + c);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    float t = (bmt::Cvt<T>::to_f(cur[i].v[k]) - mean) * rstd * bmt::Cvt<T>::to_f(wv.v[k]);
                    if (b) t += bmt::Cvt<T>::to_f(bv.v[k]);
                    o.v[k] = bmt::Cvt<T>::from_f(t);
                }
                bmt::st16(y + r * d + c, o);
            }
        }
#pragma unroll
        for (int i = 0; i < VPL; ++i) cur[i] = nxt[i];
    }
}

template <typename T, int VPL, int WPR>
void launch_fwd_reg(int64_t rows, int d, const void* x, const void* w, const void* b, float eps, int rms, void* y, void* stats,
                    cudaStream_t s) {
    const int64_t groups = (rows + (8 / WPR) - 1) / (8 / WPR);
    static const bool stream = [] { const char* e = getenv("BMT_NORM_STAGED"); return !(e && atoi(e) == 2); }();
    if (stream) {
        const int64_t cap = 148 * (VPL <= 4 ? 3 : 2);
        const int64_t grid = groups < cap ? groups : cap;
        norm_fwd_stream_kernel<T, VPL, WPR><<<(unsigned)grid, NT, 0, s>>>(rows, d, (const T*)x, (const T*)w, (const T*)b, eps, rms,
                                                                           (T*)y, (float*)stats);
        return;
    }
    const int64_t grid = groups < 148 * 2 ? groups : 148 * 2;
    norm_fwd_reg_kernel<T, VPL, WPR><<<(unsigned)grid, NT, 0, s>>>(rows, d, (const T*)x, (const T*)w, (const T*)b, eps, rms, (T*)y,
                                                                    (float*)stats);
}

template <typename T, int WPR>
bool fwd_reg_vpl(int vpl, int64_t rows, int d, const void* x, const void* w, const void* b, float eps, int rms, void* y, void* stats,
                 cudaStream_t s) {
    if (vpl <= 2) launch_fwd_reg<T, 2, WPR>(rows, d, x, w, b, eps, rms, y, stats, s);
    else if (vpl <= 4) launch_fwd_reg<T, 4, WPR>(rows, d, x, w, b, eps, rms, y, stats, s);
    else if (vpl <= 6) launch_fwd_reg<T, 6, WPR>(rows, d, x, w, b, eps, rms, y, stats, s);
    else if (vpl <= 8) launch_fwd_reg<T, 8, WPR>(rows, d, x, w, b, eps, rms, y, stats, s);
    else return false;
    return true;
}

template <typename T>
int fwd(int64_t rows, int64_t d, const void* x, const void* w, const void* b, float eps, int rms, void* y, void* stats, cudaStream_t s) {
    // smallest warp team that keeps at most 8 vectors (64 values) per lane
    static const bool use_reg = [] { const char* e = getenv("BMT_NORM_STAGED"); return !(e && atoi(e) == 1); }();
    if (use_reg && d <= 16384) {
        const int wpr = d <= 2048 ? 1 : d <= 4096 ? 2 : d <= 8192 ? 4 : 8;
        const int vpl = (int)((d + 256 * wpr - 1) / (256 * wpr));
        bool done = false;
        if (wpr == 1) done = fwd_reg_vpl<T, 1>(vpl, rows, (int)d, x, w, b, eps, rms, y, stats, s);
        else if (wpr == 2) done = fwd_reg_vpl<T, 2>(vpl, rows, (int)d, x, w, b, eps, rms, y, stats, s);
        else if (wpr == 4) done = fwd_reg_vpl<T, 4>(vpl, rows, (int)d, x, w, b, eps, rms, y, stats, s);
        else done = fwd_reg_vpl<T, 8>(vpl, rows, (int)d, x, w, b, eps, rms, y, stats, s);
        if (done) {
            bmt_count_launch(1);
            return (int)cudaGetLastError();
        }
    }
    norm_fwd_kernel<T><<<(unsigned)rows, NT, d * sizeof(float), s>>>(rows, (int)d, (const T*)x, (const T*)w, (const T*)b, eps, rms, (T*)y, (float*)stats);
    bmt_count_launch(1);
    return (int)cudaGetLastError();
}

// Backward with the same work split as norm_fwd_reg_kernel: a team of WPR warps per row, every lane owns fixed columns.
// x and dy are read once (kept as packed 16-byte vectors in registers between the statistics and the dx pass), the
// per-column sums of dy * xhat and dy accumulate in registers over all rows a lane sees and are combined once per CTA
// through shared memory into the (nblk x d) scratch that norm_fold_kernel reduces.  No block-wide barrier per row
// unless a row is shared by several warps.
template <typename T, int VPL, int WPR>
__global__ void __launch_bounds__(NT, 1) norm_bwd_reg_kernel(int64_t rows, int d, const T* __restrict__ x, const T* __restrict__ dy,
                                                             const T* __restrict__ w, const float* __restrict__ stats, int rms,
                                                             T* __restrict__ dx, float* __restrict__ partial,
                                                             const T* __restrict__ dres) {
    constexpr int RPC = 8 / WPR;
    __shared__ float ex[2][8];
    extern __shared__ float fold[];                    // [RPC][2][d / ... ] reused for the final combination
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = warp % WPR, slot = warp / WPR;
    float dg[VPL][8], db[VPL][8];
#pragma unroll
    for (int v = 0; v < VPL; ++v)
#pragma unroll
        for (int k = 0; k < 8; ++k) dg[v][k] = db[v][k] = 0.f;
    const int64_t groups = (rows + RPC - 1) / RPC;
    for (int64_t gi = blockIdx.x; gi < groups; gi += gridDim.x) {
        const int64_t r = gi * RPC + slot;
        const bool live = r < rows;
        const float mean = live ? stats[r] : 0.f, rstd = live ? stats[rows + r] : 0.f;
        bmt::Vec16<T> xv[VPL], gv[VPL];
#pragma unroll
        for (int v = 0; v < VPL; ++v) {
            const int c = ((v * WPR + sub) * 32 + lane) * 8;
            if (live && c < d) { xv[v] = bmt::ld16(x + r * d + c); gv[v] = bmt::ld16(dy + r * d + c); }
        }
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int v = 0; v < VPL; ++v) {
            const int c = ((v * WPR + sub) * 32 + lane) * 8;
            if (live && c < d) {
                const bmt::Vec16<T> wv = bmt::ld16(w + c);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const float xh = (bmt::Cvt<T>::to_f(xv[v].v[k]) - mean) * rstd;
                    const float g = bmt::Cvt<T>::to_f(gv[v].v[k]);
                    const float wg = g * bmt::Cvt<T>::to_f(wv.v[k]);
                    s1 += wg; s2 += wg * xh;
                    dg[v][k] += g * xh; db[v][k] += g;
                }
            }
        }
        s1 = bmt::warp_sum(s1);
        s2 = bmt::warp_sum(s2);
        if (WPR > 1) {
            if (lane == 0) { ex[0][warp] = s1; ex[1][warp] = s2; }
            __syncthreads();
            s1 = s2 = 0.f;
#pragma unroll
            for (int i = 0; i < WPR; ++i) { s1 += ex[0][slot * WPR + i]; s2 += ex[1][slot * WPR + i]; }
        }
        s1 = rms ? 0.f : s1 / d;
        s2 = s2 / d;
#pragma unroll
        for (int v = 0; v < VPL; ++v) {
            const int c = ((v * WPR + sub) * 32 + lane) * 8;
            if (live && c < d) {
                const bmt::Vec16<T> wv = bmt::ld16(w + c);
                bmt::Vec16<T> o, rv;
                if (dres) rv = bmt::ld16(dres + r * d + c);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const float xh = (bmt::Cvt<T>::to_f(xv[v].v[k]) - mean) * rstd;
                    const float wg = bmt::Cvt<T>::to_f(gv[v].v[k]) * bmt::Cvt<T>::to_f(wv.v[k]);
                    float val = rstd * (wg - s1 - xh * s2);
                    if (dres) val += bmt::Cvt<T>::to_f(rv.v[k]);
                    o.v[k] = bmt::Cvt<T>::from_f(val);
                }
                bmt::st16(dx + r * d + c, o);
            }
        }
        if (WPR > 1) __syncthreads();
    }
    // combine the RPC row slots of this CTA: slot 0 ends up with the CTA's column sums
    float* pg = partial + (int64_t)blockIdx.x * d;
    float* pb = partial + ((int64_t)gridDim.x + blockIdx.x) * d;
    for (int s_ = 1; s_ < RPC; ++s_) {
        __syncthreads();
        if (slot == s_) {
#pragma unroll
            for (int v = 0; v < VPL; ++v) {
                const int c = ((v * WPR + sub) * 32 + lane) * 8;
                if (c < d) {
#pragma unroll
                    for (int k = 0; k < 8; ++k) { fold[c + k] = dg[v][k]; fold[d + c + k] = db[v][k]; }
                }
            }
        }
        __syncthreads();
        if (slot == 0) {
#pragma unroll
            for (int v = 0; v < VPL; ++v) {
                const int c = ((v * WPR + sub) * 32 + lane) * 8;
                if (c < d) {
#pragma unroll
                    for (int k = 0; k < 8; ++k) { dg[v][k] += fold[c + k]; db[v][k] += fold[d + c + k]; }
                }
            }
        }
    }
    if (slot == 0) {
#pragma unroll
        for (int v = 0; v < VPL; ++v) {
            const int c = ((v * WPR + sub) * 32 + lane) * 8;
            if (c < d) {
#pragma unroll
                for (int k = 0; k < 8; ++k) { pg[c + k] = dg[v][k]; pb[c + k] = db[v][k]; }
            }
        }
    }
}

template <typename T, int WPR>
bool bwd_reg_vpl(int vpl, int64_t rows, int d, const void* x, const void* dy, const void* w, const void* stats, int rms, int nblk,
                 void* dx, void* partial, const void* dres, cudaStream_t s) {
    const size_t smem = (size_t)2 * d * sizeof(float);
#define BMT_BWD_REG(V)                                                                                                          \
    do {                                                                                                                        \
        static bool cfg = false;                                                                                                \
        if (!cfg) { cudaFuncSetAttribute(norm_bwd_reg_kernel<T, V, WPR>, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * 16384 * 4); cfg = true; } \
        norm_bwd_reg_kernel<T, V, WPR><<<nblk, NT, smem, s>>>(rows, d, (const T*)x, (const T*)dy, (const T*)w, (const float*)stats, rms, \
                                                              (T*)dx, (float*)partial, (const T*)dres);                         \
    } while (0)
    if (vpl <= 2) BMT_BWD_REG(2);
    else if (vpl <= 4) BMT_BWD_REG(4);
    else if (vpl <= 6) BMT_BWD_REG(6);
    else if (vpl <= 8) BMT_BWD_REG(8);
    else return false;
#undef BMT_BWD_REG
    return true;
}

template <typename T>
int bwd(int64_t rows, int64_t d, const void* x, const void* dy, const void* w, const void* stats, int rms, int nblk, void* dx,
        void* partial, void* dw, void* db, cudaStream_t s, const void* dres = nullptr, bool acc = false) {
    const auto fold = [&] {
        const unsigned g = (unsigned)((d + 31) / 32);
        if (acc) norm_fold_kernel<T, true><<<g, dim3(32, 32), 0, s>>>((int)d, nblk, (const float*)partial, (T*)dw, (T*)db);
        else norm_fold_kernel<T><<<g, dim3(32, 32), 0, s>>>((int)d, nblk, (const float*)partial, (T*)dw, (T*)db);
    };
    static const bool use_reg = [] { const char* e = getenv("BMT_NORM_STAGED"); return !(e && atoi(e) == 1); }();
    if (use_reg && d <= 16384) {
        // the backward keeps two column-sum accumulators per value: at most 6 vectors per lane where the row length allows
        const int wpr = d <= 1536 ? 1 : d <= 3072 ? 2 : d <= 6144 ? 4 : 8;
        const int vpl = (int)((d + 256 * wpr - 1) / (256 * wpr));
        bool done = false;
        if (wpr == 1) done = bwd_reg_vpl<T, 1>(vpl, rows, (int)d, x, dy, w, stats, rms, nblk, dx, partial, dres, s);
        else if (wpr == 2) done = bwd_reg_vpl<T, 2>(vpl, rows, (int)d, x, dy, w, stats, rms, nblk, dx, partial, dres, s);
        else if (wpr == 4) done = bwd_reg_vpl<T, 4>(vpl, rows, (int)d, x, dy, w, stats, rms, nblk, dx, partial, dres, s);
        else done = bwd_reg_vpl<T, 8>(vpl, rows, (int)d, x, dy, w, stats, rms, nblk, dx, partial, dres, s);
        if (done) {
            fold();
            bmt_count_launch(2);
            return (int)cudaGetLastError();
        }
    }
    norm_bwd_kernel<T><<<nblk, NT, 0, s>>>(rows, (int)d, (const T*)x, (const T*)dy, (const T*)w, (const float*)stats, rms, (T*)dx, (float*)partial, (const T*)dres);
    fold();
    bmt_count_launch(2);
    return (int)cudaGetLastError();
}

}  // namespace

extern "C" int bmt_norm_fwd(int64_t rows, int64_t d, const void* x, const void* w, const void* b, float eps, int rms, int dtype,
                            void* y, void* stats, void* stream) {
    if (rows <= 0) return 0;
    if (d % 8 != 0 || d > 16384 || dtype == BMT_DT_F32) return -3;
    cudaStream_t s = (cudaStream_t)stream;
    return dtype == BMT_DT_F16 ? fwd<__half>(rows, d, x, w, b, eps, rms, y, stats, s)
                               : fwd<__nv_bfloat16>(rows, d, x, w, b, eps, rms, y, stats, s);
}

extern "C" int bmt_norm_bwd(int64_t rows, int64_t d, const void* x, const void* dy, const void* w, const void* stats, int rms,
                            int dtype, int nblk, void* dx, void* partial, void* dw, void* db, void* stream) {
    if (rows <= 0) return 0;
    if (d % 8 != 0 || d > NT * 8 * MAXIT || dtype == BMT_DT_F32) return -3;
    cudaStream_t s = (cudaStream_t)stream;
    return dtype == BMT_DT_F16 ? bwd<__half>(rows, d, x, dy, w, stats, rms, nblk, dx, partial, dw, db, s)
                               : bwd<__nv_bfloat16>(rows, d, x, dy, w, stats, rms, nblk, dx, partial, dw, db, s);
}

// Backward that also adds a residual-branch gradient: dx = dres + norm_backward(dy).
extern "C" int bmt_norm_bwd_res(int64_t rows, int64_t d, const void* x, const void* dy, const void* w, const void* stats, int rms,
                                int dtype, int nblk, void* dx, void* partial, void* dw, void* db, const void* dres, void* stream) {
    if (rows <= 0) return 0;
    if (d % 8 != 0 || d > NT * 8 * MAXIT || dtype == BMT_DT_F32) return -3;
    cudaStream_t s = (cudaStream_t)stream;
    return dtype == BMT_DT_F16 ? bwd<__half>(rows, d, x, dy, w, stats, rms, nblk, dx, partial, dw, db, s, dres)
                               : bwd<__nv_bfloat16>(rows, d, x, dy, w, stats, rms, nblk, dx, partial, dw, db, s, dres);
}

// Backward with residual-branch gradient and, when `accumulate` is set, dw / db += instead of =.
extern "C" int bmt_norm_bwd_ex(int64_t rows, int64_t d, const void* x, const void* dy, const void* w, const void* stats, int rms,
                               int dtype, int nblk, void* dx, void* partial, void* dw, void* db, const void* dres, int accumulate,
                               void* stream) {
    if (rows <= 0) return 0;
    if (d % 8 != 0 || d > NT * 8 * MAXIT || dtype == BMT_DT_F32) return -3;
    cudaStream_t s = (cudaStream_t)stream;
    return dtype == BMT_DT_F16 ? bwd<__half>(rows, d, x, dy, w, stats, rms, nblk, dx, partial, dw, db, s, dres, accumulate != 0)
                               : bwd<__nv_bfloat16>(rows, d, x, dy, w, stats, rms, nblk, dx, partial, dw, db, s, dres, accumulate != 0);
}

// ---------------------------------------------------------------------------------------------------------------
// Allocation-free variant (see norm_noalloc.h).  Same kernels as bmt_norm_bwd; the partial-sum scratch lives in a
// file-scope device array whose address is resolved once per device.
#include <mutex>
#include <stdio.h>

#include "norm_noalloc.h"

static __device__ __align__(256) float g_norm_noalloc_scratch[2 * BMT_NORM_NOALLOC_MAX_CTAS * BMT_NORM_NOALLOC_MAX_D];

namespace {
constexpr int kMaxDevices = 64;
float* g_noalloc_ptr[kMaxDevices] = {nullptr};
std::mutex g_noalloc_mu;

// Device address of the scratch array on the current device.  In host code the array's name is only a handle for
// the runtime, not a device address, so it is never passed to a kernel directly.
int noalloc_scratch(float** out) {
    int dev = 0;
    BMT_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return BMT_NORM_NOALLOC_BAD_ARG;
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    if (g_noalloc_ptr[dev] == nullptr) {
        float* p = nullptr;
        BMT_CUDA_OK(cudaGetSymbolAddress((void**)&p, g_norm_noalloc_scratch));
        g_noalloc_ptr[dev] = p;
    }
    *out = g_noalloc_ptr[dev];
    return 0;
}
}  // namespace

extern "C" int bmt_norm_bwd_noalloc(int64_t rows, int64_t d, const void* x, const void* dy, const void* w, const void* stats,
                                    int rms, int dtype, void* dx, void* dw, void* db, void* stream) {
    if (rows <= 0) return 0;
    if (d > BMT_NORM_NOALLOC_MAX_D) {
        fprintf(stderr, "bmt_norm_bwd_noalloc: d = %lld exceeds the built-in scratch (max d %d); use bmt_norm_bwd with your own scratch\n",
                (long long)d, BMT_NORM_NOALLOC_MAX_D);
        return BMT_NORM_NOALLOC_TOO_LARGE;
    }
    if (d <= 0 || d % 8 != 0 || (dtype != BMT_DT_F16 && dtype != BMT_DT_BF16) || (rms && db != nullptr)) {
        fprintf(stderr, "bmt_norm_bwd_noalloc: unsupported arguments (d = %lld must be a positive multiple of 8, dtype fp16/bf16, no bias gradient for RMSNorm)\n",
                (long long)d);
        return BMT_NORM_NOALLOC_BAD_ARG;
    }
    float* scratch = nullptr;
    const int rc = noalloc_scratch(&scratch);
    if (rc != 0) return rc;
    const int nblk = rows < BMT_NORM_NOALLOC_MAX_CTAS ? (int)rows : BMT_NORM_NOALLOC_MAX_CTAS;
    cudaStream_t s = (cudaStream_t)stream;
    return dtype == BMT_DT_F16 ? bwd<__half>(rows, d, x, dy, w, stats, rms, nblk, dx, scratch, dw, db, s)
                               : bwd<__nv_bfloat16>(rows, d, x, dy, w, stats, rms, nblk, dx, scratch, dw, db, s);
}
