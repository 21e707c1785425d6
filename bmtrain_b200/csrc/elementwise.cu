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

// Column sums of an (m, n) matrix (bias gradients).  Block = 8 column packets (64 columns) x 32 row lanes; grid =
// (column blocks, row splits): with `splits` > 1 every CTA writes its 64 fp32 partial sums to `scratch[split][n]`, and
// the CTA that finishes last in its column block (a ticket counter behind the partials, reset for the next call) adds
// the partials up in split order -- the result does not depend on the order in which CTAs run.  `acc`: out += sums.
template <typename T>
__global__ void __launch_bounds__(256) colsum_kernel(int64_t m, int64_t n, const T* __restrict__ x, T* __restrict__ out, int acc,
                                                     float* __restrict__ scratch, unsigned int* __restrict__ tickets) {
    __shared__ float red[32][65];
    __shared__ unsigned int last_s;
    const int cv = threadIdx.x & 7, lane = threadIdx.x >> 3;
    const int splits = gridDim.y, split = blockIdx.y;
    const int64_t c = (int64_t)blockIdx.x * 64 + cv * 8;
    float a0[8] = {0, 0, 0, 0, 0, 0, 0, 0}, a1[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (c < n) {
        const int64_t step = (int64_t)32 * splits;
        int64_t r = (int64_t)split * 32 + lane;
        for (; r + step < m; r += 2 * step) {          // two independent loads in flight per thread
            const bmt::Vec16<T> v0 = bmt::ld16(x + r * n + c), v1 = bmt::ld16(x + (r + step) * n + c);
#pragma unroll
            for (int k = 0; k < 8; ++k) { a0[k] += bmt::Cvt<T>::to_f(v0.v[k]); a1[k] += bmt::Cvt<T>::to_f(v1.v[k]); }
        }
        if (r < m) {
            const bmt::Vec16<T> v0 = bmt::ld16(x + r * n + c);
#pragma unroll
            for (int k = 0; k < 8; ++k) a0[k] += bmt::Cvt<T>::to_f(v0.v[k]);
        }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) red[lane][cv * 8 + k] = a0[k] + a1[k];
    __syncthreads();
    const int64_t col = (int64_t)blockIdx.x * 64 + threadIdx.x;
    float s = 0.f;
    if (threadIdx.x < 64) {
#pragma unroll 8
        for (int l = 0; l < 32; ++l) s += red[l][threadIdx.x];
    }
    if (splits == 1) {
        if (threadIdx.x < 64 && col < n) out[col] = bmt::Cvt<T>::from_f(acc ? s + bmt::Cvt<T>::to_f(out[col]) : s);
        return;
    }
    if (threadIdx.x < 64 && col < n) scratch[(int64_t)split * n + col] = s;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int t = atomicAdd(tickets + blockIdx.x, 1u);
        last_s = (t == (unsigned int)splits - 1) ? 1u : 0u;
        if (last_s) tickets[blockIdx.x] = 0;            // every CTA of this column block has taken its ticket
    }
    __syncthreads();
    if (!last_s) return;
    __threadfence();
    if (threadIdx.x < 64 && col < n) {
        float t = 0.f;
        for (int i = 0; i < splits; ++i) t += __ldcg(scratch + (int64_t)i * n + col);
        out[col] = bmt::Cvt<T>::from_f(acc ? t + bmt::Cvt<T>::to_f(out[col]) : t);
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

// Rotary position embedding on a packed projection.  `packed` is (b, s, hk, g + 2, d): per kv head g query heads, one key
// head, one value head ("half rotation" convention: element i pairs with i + d/2, angle = pos * theta^(-2i/d); `cs` holds
// (cos, sin) of every (position, i) as interleaved fp32 pairs, (pos0 + seq) x d/2 of them).
// SPLIT: packed -> q (b, s, hk*g, d) rotated, k (b, s, hk, d) rotated, v (b, s, hk, d) copied, all contiguous.
// !SPLIT (backward): gradients of q, k, v -> gradient of packed (contiguous), q and k parts rotated back.
// One thread moves 8 elements of the lower half of a head and their 8 partners of the upper half.
template <typename T, bool SPLIT>
__global__ void __launch_bounds__(256) rope_qkv_kernel(int64_t batch, int64_t seq, int hk, int g, int d, T* __restrict__ packed,
                                                       int64_t p_tok, int64_t p_batch, T* __restrict__ q, T* __restrict__ k,
                                                       T* __restrict__ v, const float* __restrict__ cs, int64_t pos0) {
    const int half = d / 2, vecs = half / 8, slots = hk * (g + 2);
    const int64_t total = batch * seq * slots * vecs;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % vecs) * 8;
        int64_t r = i / vecs;
        const int slot = (int)(r % slots);
        r /= slots;
        const int64_t t = r % seq, bb = r / seq;
        const int kvh = slot / (g + 2), j = slot % (g + 2);
        T* pin = packed + bb * p_batch + t * p_tok + (int64_t)slot * d;
        T* sep = j < g ? q + (((bb * seq + t) * hk + kvh) * g + j) * d : (j == g ? k : v) + ((bb * seq + t) * hk + kvh) * d;
        const T* src = SPLIT ? pin : sep;
        T* dst = SPLIT ? sep : pin;
        bmt::Vec16<T> lo = bmt::ld16(src + c), hi = bmt::ld16(src + half + c), olo, ohi;
        if (j <= g) {
            // (cos, sin) of position x frequency from the table (seq x d/2 pairs, built once per shape; it stays in L2)
            const float4* tab = reinterpret_cast<const float4*>(cs + ((pos0 + t) * half + c) * 2);
            float4 q4[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) q4[e] = tab[e];
            const float* f = reinterpret_cast<const float*>(q4);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float co = f[2 * e];
                const float sn = SPLIT ? f[2 * e + 1] : -f[2 * e + 1];
                const float a = bmt::Cvt<T>::to_f(lo.v[e]), b2 = bmt::Cvt<T>::to_f(hi.v[e]);
                olo.v[e] = bmt::Cvt<T>::from_f(a * co - b2 * sn);
                ohi.v[e] = bmt::Cvt<T>::from_f(a * sn + b2 * co);
            }
        } else {
            olo = lo;
            ohi = hi;
        }
        bmt::st16(dst + c, olo);
        bmt::st16(dst + half + c, ohi);
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

// `scratch` (optional): fp32 work space, `scratch_bytes` large; its first 4 KB hold the ticket counters and must be zero
// before the first call (the kernel leaves them zero), the rest takes the per-split partial sums.  Calls that share a
// scratch must be ordered on one stream.  Without scratch one CTA per 64 columns walks over all rows.
extern "C" int bmt_colsum_ex(int64_t m, int64_t n, const void* x, int dtype, void* out, int accumulate, void* scratch,
                             int64_t scratch_bytes, void* stream) {
    if (n <= 0) return 0;
    if (n % 8 || dtype == BMT_DT_F32) return -3;
    cudaStream_t s = (cudaStream_t)stream;
    const int64_t cb = (n + 63) / 64;
    int64_t splits = 1;
    if (scratch && cb <= 1024) {
        splits = (4 * 148 + cb - 1) / cb;                                  // about four CTAs per SM
        const int64_t by_rows = m / 128, by_mem = (scratch_bytes - 4096) / (n * 4);
        if (splits > by_rows) splits = by_rows;                            // at least four rows per lane
        if (splits > by_mem) splits = by_mem;
        if (splits > 64) splits = 64;
        if (splits < 1) splits = 1;
    }
    const dim3 g((unsigned)cb, (unsigned)splits);
    unsigned int* tickets = (unsigned int*)scratch;
    float* partial = scratch ? (float*)((char*)scratch + 4096) : nullptr;
    if (dtype == BMT_DT_F16) colsum_kernel<__half><<<g, 256, 0, s>>>(m, n, (const __half*)x, (__half*)out, accumulate, partial, tickets);
    else colsum_kernel<__nv_bfloat16><<<g, 256, 0, s>>>(m, n, (const __nv_bfloat16*)x, (__nv_bfloat16*)out, accumulate, partial, tickets);
    bmt_count_launch(1);
    return (int)cudaGetLastError();
}

extern "C" int bmt_colsum(int64_t m, int64_t n, const void* x, int dtype, void* out, void* stream) {
    return bmt_colsum_ex(m, n, x, dtype, out, 0, nullptr, 0, stream);
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

// Rotary embedding of a packed (b, s, hk, g + 2, d) projection (token / batch strides p_tok / p_batch, the last three
// dims contiguous).  split != 0: writes rotated q, k and the copied v (contiguous); split == 0: the backward, reads the
// three gradients and writes the packed gradient (contiguous, p_tok / p_batch describe it).  d: multiple of 16.
// cos_sin: fp32 table of (cos, sin) pairs, (pos0 + seq) x d/2, 16-byte aligned.
extern "C" int bmt_rope_qkv(int64_t batch, int64_t seq, int hk, int g, int d, void* packed, int64_t p_tok, int64_t p_batch, void* q,
                            void* k, void* v, const void* cos_sin, int64_t pos0, int split, int dtype, void* stream) {
    if (batch <= 0 || seq <= 0) return 0;
    if (d % 16 || dtype == BMT_DT_F32 || (p_tok & 7) || (p_batch & 7) || !cos_sin || ((uintptr_t)cos_sin & 15)) return -3;
    cudaStream_t s = (cudaStream_t)stream;
    const int64_t work = batch * seq * hk * (g + 2) * (d / 16);
    const float* table = (const float*)cos_sin;
    if (dtype == BMT_DT_F16) {
        if (split) rope_qkv_kernel<__half, true><<<grid1d(work), 256, 0, s>>>(batch, seq, hk, g, d, (__half*)packed, p_tok, p_batch, (__half*)q, (__half*)k, (__half*)v, table, pos0);
        else rope_qkv_kernel<__half, false><<<grid1d(work), 256, 0, s>>>(batch, seq, hk, g, d, (__half*)packed, p_tok, p_batch, (__half*)q, (__half*)k, (__half*)v, table, pos0);
    } else {
        if (split) rope_qkv_kernel<__nv_bfloat16, true><<<grid1d(work), 256, 0, s>>>(batch, seq, hk, g, d, (__nv_bfloat16*)packed, p_tok, p_batch, (__nv_bfloat16*)q, (__nv_bfloat16*)k, (__nv_bfloat16*)v, table, pos0);
        else rope_qkv_kernel<__nv_bfloat16, false><<<grid1d(work), 256, 0, s>>>(batch, seq, hk, g, d, (__nv_bfloat16*)packed, p_tok, p_batch, (__nv_bfloat16*)q, (__nv_bfloat16*)k, (__nv_bfloat16*)v, table, pos0);
    }
    bmt_count_launch(1);
    return (int)cudaGetLastError();
}
