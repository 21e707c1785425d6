// Peer-memory runtime for one NVLink / NVSwitch domain and the fused gradient reduce-scatter kernel.
//
// Symmetric buffers: every rank cudaMallocs a buffer of the same size, exports it with cudaIpcGetMemHandle and
// maps the buffers of its peers with cudaIpcOpenMemHandle (the handles travel through the Python side's process
// group).  Kernels then receive a table of W device pointers, one per rank, and read or write peers' memory with
// ordinary loads and stores that cross NVLink.  Synchronisation between ranks uses small flag arrays that live in
// the same kind of buffer: a rank publishes "epoch e reached" by storing e into its slot of every peer's flag
// array (st.release.sys); waiting is a bounded poll with ld.acquire.sys that gives up after a time limit and
// reports through a status word -- nothing spins forever and nothing traps.
// (The reference only has blocking NCCL wrappers: csrc/include/nccl.hpp:8-188.)
#include <stdio.h>
#include <string.h>

#include "api.h"
#include "common.cuh"

extern "C" int bmt_symm_alloc(int64_t bytes, void** out) {
    void* p = nullptr;
    BMT_CUDA_OK(cudaMalloc(&p, (size_t)bytes));
    BMT_CUDA_OK(cudaMemset(p, 0, (size_t)bytes));
    *out = p;
    return 0;
}
extern "C" int bmt_symm_free(void* p) { return (int)cudaFree(p); }
extern "C" int bmt_ipc_get_handle(void* p, void* handle64) {
    cudaIpcMemHandle_t h;
    BMT_CUDA_OK(cudaIpcGetMemHandle(&h, p));
    memcpy(handle64, &h, sizeof(h));
    return 0;
}
extern "C" int bmt_ipc_open_handle(const void* handle64, void** out) {
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    void* p = nullptr;
    BMT_CUDA_OK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *out = p;
    return 0;
}
extern "C" int bmt_ipc_close(void* p) { return (int)cudaIpcCloseMemHandle(p); }
extern "C" int bmt_ipc_handle_size(void) { return (int)sizeof(cudaIpcMemHandle_t); }

namespace {

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint64_t now_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Wait until flags[0..n) are all >= epoch (counters only grow); false after `limit_ns`.
__device__ bool wait_flags(const unsigned int* flags, int n, unsigned int epoch, uint64_t limit_ns) {
    const uint64_t t0 = now_ns();
    for (int j = 0; j < n; ++j) {
        unsigned int spins = 0;
        while ((int)(ld_acquire_sys(flags + j) - epoch) < 0) {
            if ((++spins & 255u) == 0 && now_ns() - t0 > limit_ns) return false;
        }
    }
    return true;
}

struct RsArgs {
    const void* peer[8];       // full gradient buffer of every rank (own rank included), `total` elements each
    unsigned int* peer_flags[8];  // flag array of every rank (own included): slot s*W + j = "rank j finished producing slot s"
    int world, rank, slot;
    unsigned int epoch;
    int64_t part;              // elements of one partition; this rank reduces [rank*part, (rank+1)*part)
    void* out;                 // partition gradient (param dtype)
    int accumulate;            // out += ...
    float scale;               // result multiplied by this (1/loss_scale, or 1)
    unsigned char* overflow;   // set to 1 when an inf/nan shows up in the reduced values
    int* status;               // set to a non-zero code when the wait ran out
    uint64_t limit_ns;
    float* acc32;              // optional fp32 copy of the partition gradient: with `accumulate` the sum is added to IT (not to
                               // the rounded `out`), so gradients accumulated over micro-steps are rounded once, at the end
    float* sqsum;              // optional: += sum of squares of the values written (for the gradient norm; zero it before)
};

// Σ v² of one CTA into *sqsum (one atomic per CTA; the order of the CTAs is not fixed, so the last bits may differ from
// run to run -- the gradient norm is a diagnostic / clipping quantity, the gradients themselves stay bit-reproducible)
__device__ __forceinline__ void add_sqsum(float* sqsum, float local) {
    __shared__ float sq_s[33];
    const float total = bmt::block_allreduce<false>(local, sq_s);
    if (threadIdx.x == 0 && sqsum) atomicAdd(sqsum, total);
}

// WMAX: upper bound of the group size (loads of all ranks are issued before the first add); U: vectors per thread per
// trip.  WMAX * U independent 16-byte loads are in flight per thread, which is what hides the NVLink round trip.
template <typename T, int WMAX, int U>
__global__ void __launch_bounds__(256, 2) fused_rs_kernel(RsArgs a) {
    __shared__ int ok_s;
    // epoch 0: the hand-shake (steps 1 and 2) was done by a one-CTA signal/wait kernel launched before this one, so that
    // this grid never holds SMs while it waits for another rank
    if (a.epoch != 0) {
        // 1. tell every rank that this rank's buffer (written by earlier kernels of this stream) is complete
        if (blockIdx.x == 0 && threadIdx.x < a.world) {
            __threadfence_system();
            st_release_sys(a.peer_flags[threadIdx.x] + a.slot * a.world + a.rank, a.epoch);
        }
        // 2. wait until every rank has said the same (bounded)
        if (threadIdx.x == 0) {
            const bool ok = wait_flags(a.peer_flags[a.rank] + a.slot * a.world, a.world, a.epoch, a.limit_ns);
            if (!ok) atomicCAS(a.status, 0, 0x100 | a.rank);
            ok_s = ok ? 1 : 0;
        }
        __syncthreads();
        if (!ok_s) return;
    }
    // 3. this rank's partition: sum over ranks in rank order (fp32), scale, accumulate, inf/nan, write
    const int64_t base = (int64_t)a.rank * a.part;
    const int64_t nvec = a.part / 8;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    T* __restrict__ out = (T*)a.out;
    bool bad = false;
    float sq = 0.f;
    const bool acc_half = a.accumulate && !a.acc32, acc_f32 = a.accumulate && a.acc32;
    for (int64_t i0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i0 < nvec; i0 += stride * U) {
        bmt::Vec16<T> v[U][WMAX];
        bmt::Vec16<T> old[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t i = i0 + u * stride;
            if (i < nvec) {
#pragma unroll
                for (int j = 0; j < WMAX; ++j)
                    if (j < a.world) v[u][j] = bmt::ld16((const T*)a.peer[j] + base + i * 8);
                if (acc_half) old[u] = bmt::ld16(out + i * 8);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t i = i0 + u * stride;
            if (i >= nvec) continue;
            float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
            for (int j = 0; j < WMAX; ++j)
                if (j < a.world) {
#pragma unroll
                    for (int k = 0; k < 8; ++k) acc[k] += bmt::Cvt<T>::to_f(v[u][j].v[k]);
                }
            bmt::Vec16<T> o;
            if (acc_half) {
#pragma unroll
                for (int k = 0; k < 8; ++k) acc[k] = acc[k] * a.scale + bmt::Cvt<T>::to_f(old[u].v[k]);
            } else if (acc_f32) {
                // local memory, read late on purpose: keeping it in registers next to the peer loads above would spill
                const float4 lo = *reinterpret_cast<const float4*>(a.acc32 + i * 8), hi = *reinterpret_cast<const float4*>(a.acc32 + i * 8 + 4);
                const float o32[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
                for (int k = 0; k < 8; ++k) acc[k] = acc[k] * a.scale + o32[k];
            } else {
#pragma unroll
                for (int k = 0; k < 8; ++k) acc[k] *= a.scale;
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                bad |= !(fabsf(acc[k]) <= 3.402823466e38f);
                o.v[k] = bmt::Cvt<T>::from_f(acc[k]);
                bad |= !(fabsf(bmt::Cvt<T>::to_f(o.v[k])) <= 3.402823466e38f);
                sq += acc[k] * acc[k];
            }
            bmt::st16(out + i * 8, o);
            if (a.acc32) {
                *reinterpret_cast<float4*>(a.acc32 + i * 8) = make_float4(acc[0], acc[1], acc[2], acc[3]);
                *reinterpret_cast<float4*>(a.acc32 + i * 8 + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
            }
        }
    }
    if (__syncthreads_or(bad) && threadIdx.x == 0 && a.overflow) *a.overflow = 1;
    if (a.sqsum) add_sqsum(a.sqsum, sq);
}

// ---- in-switch reduction (NVLS): one multimem.ld_reduce per 16 bytes reads the same offset of every rank's buffer through
// the NVSwitch multicast address and returns the sum (added up in fp32 inside the switch), so a rank pulls 1 / W of the
// bytes the plain peer loads above move.
template <typename T> __device__ __forceinline__ void mc_ld_reduce(const void* mc, uint32_t (&r)[4]);
template <> __device__ __forceinline__ void mc_ld_reduce<__nv_bfloat16>(const void* mc, uint32_t (&r)[4]) {
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "l"(mc) : "memory");
}
template <> __device__ __forceinline__ void mc_ld_reduce<__half>(const void* mc, uint32_t (&r)[4]) {
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "l"(mc) : "memory");
}

// Same contract as fused_rs_kernel; `mc` is the multicast address of the full gradient buffer (all ranks bound).
template <typename T, int U>
__global__ void __launch_bounds__(256, 2) fused_rs_mc_kernel(RsArgs a, const T* __restrict__ mc) {
    __shared__ int ok_s;
    if (a.epoch != 0) {
        if (blockIdx.x == 0 && threadIdx.x < a.world) {
            __threadfence_system();
            st_release_sys(a.peer_flags[threadIdx.x] + a.slot * a.world + a.rank, a.epoch);
        }
        if (threadIdx.x == 0) {
            const bool ok = wait_flags(a.peer_flags[a.rank] + a.slot * a.world, a.world, a.epoch, a.limit_ns);
            if (!ok) atomicCAS(a.status, 0, 0x100 | a.rank);
            ok_s = ok ? 1 : 0;
        }
        __syncthreads();
        if (!ok_s) return;
    }
    const int64_t base = (int64_t)a.rank * a.part;
    const int64_t nvec = a.part / 8;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    T* __restrict__ out = (T*)a.out;
    bool bad = false;
    float sq = 0.f;
    const bool acc_half = a.accumulate && !a.acc32, acc_f32 = a.accumulate && a.acc32;
    for (int64_t i0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i0 < nvec; i0 += stride * U) {
        uint32_t v[U][4];
        bmt::Vec16<T> old[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t i = i0 + u * stride;
            if (i < nvec) {
                mc_ld_reduce<T>(mc + base + i * 8, v[u]);
                if (acc_half) old[u] = bmt::ld16(out + i * 8);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t i = i0 + u * stride;
            if (i >= nvec) continue;
            bmt::Vec16<T> sum = *reinterpret_cast<bmt::Vec16<T>*>(v[u]), o;
            float o32[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            if (acc_f32) {
                const float4 lo = *reinterpret_cast<const float4*>(a.acc32 + i * 8), hi = *reinterpret_cast<const float4*>(a.acc32 + i * 8 + 4);
                o32[0] = lo.x; o32[1] = lo.y; o32[2] = lo.z; o32[3] = lo.w; o32[4] = hi.x; o32[5] = hi.y; o32[6] = hi.z; o32[7] = hi.w;
            }
            float f8[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                float f = bmt::Cvt<T>::to_f(sum.v[k]) * a.scale;
                if (acc_half) f += bmt::Cvt<T>::to_f(old[u].v[k]);
                if (acc_f32) f += o32[k];
                bad |= !(fabsf(f) <= 3.402823466e38f);
                o.v[k] = bmt::Cvt<T>::from_f(f);
                bad |= !(fabsf(bmt::Cvt<T>::to_f(o.v[k])) <= 3.402823466e38f);
                sq += f * f;
                f8[k] = f;
            }
            bmt::st16(out + i * 8, o);
            if (a.acc32) {
                *reinterpret_cast<float4*>(a.acc32 + i * 8) = make_float4(f8[0], f8[1], f8[2], f8[3]);
                *reinterpret_cast<float4*>(a.acc32 + i * 8 + 4) = make_float4(f8[4], f8[5], f8[6], f8[7]);
            }
        }
    }
    if (__syncthreads_or(bad) && threadIdx.x == 0 && a.overflow) *a.overflow = 1;
    if (a.sqsum) add_sqsum(a.sqsum, sq);
}

template <typename T>
static void launch_fused_rs(const RsArgs& a, unsigned blocks, cudaStream_t s) {
    if (a.world <= 2) fused_rs_kernel<T, 2, 4><<<blocks, 256, 0, s>>>(a);
    else if (a.world <= 4) fused_rs_kernel<T, 4, 2><<<blocks, 256, 0, s>>>(a);
    else fused_rs_kernel<T, 8, 1><<<blocks, 256, 0, s>>>(a);
}

__global__ void symm_signal_wait_kernel(unsigned int* const* peer_flags_table, unsigned int** unused, int world, int rank, int slot,
                                        unsigned int epoch, int do_signal, int do_wait, int* status, uint64_t limit_ns) {
    // grid of one block: publish and/or wait on a flag row (used as a cross-rank barrier on a stream)
    if (do_signal && threadIdx.x < world) {
        __threadfence_system();
        st_release_sys(peer_flags_table[threadIdx.x] + slot * world + rank, epoch);
    }
    if (do_wait && threadIdx.x == 0) {
        if (!wait_flags(peer_flags_table[rank] + slot * world, world, epoch, limit_ns)) atomicCAS(status, 0, 0x200 | rank);
    }
}

struct PushArgs {
    const char* src[16];     // local source of every range
    int64_t dst_off[16];     // byte offset inside every rank's destination buffer
    int64_t nbytes[16];      // multiple of 16
    int nranges;
    char* dst[8];            // destination buffer of every rank (own included)
    unsigned int* peer_flags[8];
    int world, rank, free_row, done_row;
    unsigned int epoch;
    unsigned int* counter;   // local, monotonic: CTAs finished
    int* status;
    uint64_t limit_ns;
};

// Push-style all-gather of a list of byte ranges: every rank writes its ranges to the same offsets of every rank's
// buffer (own first, then the peers in ring order).  A destination is only written after it published "free" for this
// epoch; when the whole grid is done the last CTA publishes "delivered" to every rank.
__global__ void __launch_bounds__(256) push_ranges_kernel(PushArgs a) {
    __shared__ int ok_s;
    const int64_t piece = 32768;
    for (int di = 0; di < a.world; ++di) {
        const int dst = (a.rank + di) % a.world;
        if (dst != a.rank) {
            if (threadIdx.x == 0) {
                const bool ok = wait_flags(a.peer_flags[a.rank] + a.free_row * a.world + dst, 1, a.epoch, a.limit_ns);
                if (!ok) atomicCAS(a.status, 0, 0x700 | a.rank);
                ok_s = ok ? 1 : 0;
            }
            __syncthreads();
            if (!ok_s) break;
        }
        int g0 = 0;  // (pieces of the earlier ranges) mod grid: pieces are dealt round-robin over the CTAs across ranges
        for (int r = 0; r < a.nranges; ++r) {
            const int64_t np = (a.nbytes[r] + piece - 1) / piece;
            // first piece of this range that belongs to this CTA, then every gridDim.x-th (no per-piece division)
            for (int64_t pi = ((int)blockIdx.x - g0 + (int)gridDim.x) % (int)gridDim.x; pi < np; pi += gridDim.x) {
                const int64_t b0 = pi * piece;
                const int64_t n = (a.nbytes[r] - b0 < piece ? a.nbytes[r] - b0 : piece) / 16;
                const int4* s = reinterpret_cast<const int4*>(a.src[r] + b0);
                int4* d = reinterpret_cast<int4*>(a.dst[dst] + a.dst_off[r] + b0);
                for (int64_t v = threadIdx.x; v < n; v += 256 * 8) {
                    int4 t[8];   // 128 bytes in flight per thread: the copy is bound by load latency, not by issue rate
#pragma unroll
                    for (int u = 0; u < 8; ++u) if (v + u * 256 < n) t[u] = s[v + u * 256];
#pragma unroll
                    for (int u = 0; u < 8; ++u) if (v + u * 256 < n) d[v + u * 256] = t[u];
                }
            }
            g0 = (int)((g0 + np) % (int64_t)gridDim.x);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        const unsigned int done = atomicAdd(a.counter, 1u) + 1u;
        if (done == a.epoch * gridDim.x) {
            __threadfence_system();
            for (int j = 0; j < a.world; ++j) st_release_sys(a.peer_flags[j] + a.done_row * a.world + a.rank, a.epoch);
        }
    }
}

}  // namespace

// Push-style all-gather of up to 16 byte ranges (see push_ranges_kernel).  `grid` CTAs; the caller's `counter` advances
// by `grid` per call, so it has to be dedicated to one (ranges, grid) configuration.
extern "C" int bmt_push_ranges(const void* const* src, const int64_t* dst_off, const int64_t* nbytes, int nranges,
                               void* const* dst, void* const* peer_flags, int world, int rank, int free_row, int done_row,
                               unsigned int epoch, void* counter_u32, void* status_i32, double timeout_s, int grid,
                               void* stream) {
    if (nranges < 0 || nranges > 16 || world < 1 || world > 8) return -33;
    PushArgs a;
    memset(&a, 0, sizeof(a));
    for (int r = 0; r < nranges; ++r) {
        if ((nbytes[r] & 15) || (dst_off[r] & 15) || ((uintptr_t)src[r] & 15)) return -34;
        a.src[r] = (const char*)src[r]; a.dst_off[r] = dst_off[r]; a.nbytes[r] = nbytes[r];
    }
    a.nranges = nranges;
    for (int j = 0; j < world; ++j) { a.dst[j] = (char*)dst[j]; a.peer_flags[j] = (unsigned int*)peer_flags[j]; }
    a.world = world; a.rank = rank; a.free_row = free_row; a.done_row = done_row; a.epoch = epoch;
    a.counter = (unsigned int*)counter_u32; a.status = (int*)status_i32; a.limit_ns = (uint64_t)(timeout_s * 1e9);
    push_ranges_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(a);
    bmt_count_launch(1);
    return (int)cudaGetLastError();
}

// Plain SM copy between two device pointers, either of which may be a mapped peer buffer (push: dst remote, pull: src remote).
__global__ void __launch_bounds__(256) peer_copy_kernel(int4* __restrict__ dst, const int4* __restrict__ src, int64_t nvec) {
    const int64_t stride = (int64_t)gridDim.x * 256;
    for (int64_t v0 = (int64_t)blockIdx.x * 256 + threadIdx.x; v0 < nvec; v0 += stride * 8) {
        int4 t[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) if (v0 + u * stride < nvec) t[u] = src[v0 + u * stride];
#pragma unroll
        for (int u = 0; u < 8; ++u) if (v0 + u * stride < nvec) dst[v0 + u * stride] = t[u];
    }
}

// Copies nbytes (multiple of 16, both pointers 16-byte aligned) with `grid` CTAs of 256 threads on `stream`.
extern "C" int bmt_peer_copy(void* dst, const void* src, int64_t nbytes, int grid, void* stream) {
    if ((nbytes & 15) || ((uintptr_t)dst & 15) || ((uintptr_t)src & 15) || grid < 1) return -35;
    peer_copy_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((int4*)dst, (const int4*)src, nbytes / 16);
    bmt_count_launch(1);
    return (int)cudaGetLastError();
}

// Fused reduce-scatter: out[0..part) (+)= scale * sum_j peer_j[rank*part + i], with inf/nan detection.
// peers / peer_flags: host arrays of `world` device pointers.  part must be a multiple of 8 elements and every
// buffer 16-byte aligned.  dtype: 0 fp16, 1 bf16, 2 fp32.
static int fused_reduce_scatter_impl(const void* const* peers, const void* multicast, void* const* peer_flags, int world, int rank,
                                     int slot, unsigned int epoch, int64_t part, void* out, int accumulate, float scale, int dtype,
                                     void* overflow_u8, void* status_i32, double timeout_s, void* stream, void* acc32 = nullptr,
                                     void* sqsum = nullptr);

// Same two reductions with the optional extras: `acc32` (fp32 partition gradient that accumulation goes through) and
// `sqsum_f32` (+= sum of squares of the values written); `multicast` null selects plain peer loads.
extern "C" int bmt_fused_reduce_scatter_ex(const void* const* peers, const void* multicast, void* const* peer_flags, int world,
                                           int rank, int slot, unsigned int epoch, int64_t part, void* out, int accumulate,
                                           float scale, int dtype, void* acc32, void* sqsum_f32, void* overflow_u8,
                                           void* status_i32, double timeout_s, void* stream) {
    return fused_reduce_scatter_impl(multicast ? nullptr : peers, multicast, peer_flags, world, rank, slot, epoch, part, out,
                                     accumulate, scale, dtype, overflow_u8, status_i32, timeout_s, stream, acc32, sqsum_f32);
}

extern "C" int bmt_fused_reduce_scatter(const void* const* peers, void* const* peer_flags, int world, int rank, int slot,
                                        unsigned int epoch, int64_t part, void* out, int accumulate, float scale, int dtype,
                                        void* overflow_u8, void* status_i32, double timeout_s, void* stream) {
    return fused_reduce_scatter_impl(peers, nullptr, peer_flags, world, rank, slot, epoch, part, out, accumulate, scale, dtype,
                                     overflow_u8, status_i32, timeout_s, stream);
}

// The same reduction through the NVSwitch multicast address `multicast` of the full buffers (multimem.ld_reduce).
extern "C" int bmt_fused_reduce_scatter_mc(const void* multicast, void* const* peer_flags, int world, int rank, int slot,
                                           unsigned int epoch, int64_t part, void* out, int accumulate, float scale, int dtype,
                                           void* overflow_u8, void* status_i32, double timeout_s, void* stream) {
    if (!multicast) return -33;
    return fused_reduce_scatter_impl(nullptr, multicast, peer_flags, world, rank, slot, epoch, part, out, accumulate, scale, dtype,
                                     overflow_u8, status_i32, timeout_s, stream);
}

static int fused_reduce_scatter_impl(const void* const* peers, const void* multicast, void* const* peer_flags, int world, int rank,
                                     int slot, unsigned int epoch, int64_t part, void* out, int accumulate, float scale, int dtype,
                                     void* overflow_u8, void* status_i32, double timeout_s, void* stream, void* acc32,
                                     void* sqsum) {
    if (world < 1 || world > 8) return -30;
    if (part % 8 != 0) return -31;
    RsArgs a;
    memset(&a, 0, sizeof(a));
    for (int j = 0; j < world; ++j) { a.peer[j] = peers ? peers[j] : nullptr; a.peer_flags[j] = (unsigned int*)peer_flags[j]; }
    a.world = world; a.rank = rank; a.slot = slot; a.epoch = epoch; a.part = part; a.out = out; a.accumulate = accumulate;
    a.scale = scale; a.overflow = (unsigned char*)overflow_u8; a.status = (int*)status_i32;
    a.limit_ns = (uint64_t)(timeout_s * 1e9);
    a.acc32 = (float*)acc32;
    a.sqsum = (float*)sqsum;
    int64_t blocks = bmt::ceil_div64(part / 8, 256);
    if (blocks > 148 * 4) blocks = 148 * 4;
    if (blocks < 1) blocks = 1;
    cudaStream_t s = (cudaStream_t)stream;
    if (multicast) {
        if (dtype == BMT_DT_F16) fused_rs_mc_kernel<__half, 4><<<(unsigned)blocks, 256, 0, s>>>(a, (const __half*)multicast);
        else if (dtype == BMT_DT_BF16) fused_rs_mc_kernel<__nv_bfloat16, 4><<<(unsigned)blocks, 256, 0, s>>>(a, (const __nv_bfloat16*)multicast);
        else return -32;
        bmt_count_launch(1);
        return (int)cudaGetLastError();
    }
    if (dtype == BMT_DT_F16) launch_fused_rs<__half>(a, (unsigned)blocks, s);
    else if (dtype == BMT_DT_BF16) launch_fused_rs<__nv_bfloat16>(a, (unsigned)blocks, s);
    else return -32;
    bmt_count_launch(1);
    return (int)cudaGetLastError();
}

// Stream-ordered cross-rank signal and/or bounded wait on flag row `slot` (device table of per-rank flag pointers).
extern "C" int bmt_symm_signal_wait(void* device_flag_table, int world, int rank, int slot, unsigned int epoch, int do_signal,
                                    int do_wait, void* status_i32, double timeout_s, void* stream) {
    symm_signal_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((unsigned int* const*)device_flag_table, nullptr, world, rank, slot,
                                                                epoch, do_signal, do_wait, (int*)status_i32,
                                                                (uint64_t)(timeout_s * 1e9));
    bmt_count_launch(1);
    return (int)cudaGetLastError();
}
