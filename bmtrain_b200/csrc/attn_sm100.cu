// Fused attention for sm_100a (B200): softmax(scale * Q K^T + mask) V without the score matrix ever leaving the SM.
//
// Forward, one CTA per (128 query rows, head, sample):
//   warp 0      TMA producer: Q once, then the K and V tiles of 128 keys through two-stage rings
//   warp 1      MMA issuer (one thread): S_j = Q K_j^T into tensor memory (two S buffers), O += P_j V_j into one fp32
//               accumulator in tensor memory; S_{j+1} is issued before P_j V_j so that the tensor core works while the
//               softmax warps are busy with S_j
//   warps 2..5  softmax: one thread per query row reads its whole row of S_j from tensor memory in one round trip
//               (tcgen05.ld), applies the masks, keeps the sum and a reference maximum, writes P_j = exp2(..) as
//               fp16/bf16 into shared memory in the 128-byte-swizzled K-major layout the MMA reads.  The reference
//               maximum follows the true one lazily; only when it moves is the accumulator rescaled (tcgen05.ld / st).
//               The epilogue normalises and stores the row and its log-sum-exp.
// Masks: causal (key j visible to query i iff j <= i + sk - sq), per-sample key counts, dense boolean (b, sq, sk).
// Grouped-query attention: kv head = head / (h / hk).  Head dims up to 128 (multiples of 16); tiles are padded with
// zeros by TMA.  Every mbarrier wait is bounded; on expiry a status word is set and the CTA winds down.
//
// The reference example materialises (b, h, s, s) scores and probabilities in HBM with two bmm calls
// (example/layers/attention.py:78-104).
#include <cuda.h>
#include <math.h>
#include <string.h>

#include "api.h"
#include "common.cuh"
#include "tcgen05.cuh"
#include "tma_host.h"

namespace {

using namespace bmt_tc;

constexpr int ATT_THREADS = 192;
constexpr int TILE = 128;                        // query rows per CTA and keys per step
constexpr uint32_t CHUNK = TILE * 64 * 2;        // one [128 rows][64 columns] swizzled chunk of 16-bit elements: 16 KiB

__device__ int g_attn_status = 0;                // 0, or (code << 16) | blockIdx.x of the first CTA whose wait ran out

struct AttnParams {
    int64_t sq, sk;
    int h, hk, d;
    float sl2;                  // scale * log2(e)
    int causal;
    int64_t causal_off;         // sk - sq
    const uint8_t* mask;        // (b, sq, sk) or null; non-zero = attend
    const int32_t* kv_lens;     // (b) or null
    void* o;                    // (b, sq, h, d) by strides
    int64_t o_tok, o_head, o_batch;
    float* lse;                 // (b, h, sq), natural log; -inf for rows without a visible key
    uint32_t idesc_s, idesc_pv;
};

struct AttnShared {
    uint64_t q_full, k_full[2], v_full[2], k_empty[2], v_empty[2];
    uint64_t s_full[2], s_free[2], p_ready, p_free, o_full;
    uint32_t tmem_base;
    int failed;
};

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void fail(AttnShared* sh, int code) {
    sh->failed = 1;
    atomicCAS(&g_attn_status, 0, (code << 16) | (int)(blockIdx.x & 0xffff));
}

// one lane polls, the warp follows
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, int lane) {
    int got = 1;
    if (lane == 0) got = mbar_wait(bar, parity) ? 1 : 0;
    return __shfl_sync(0xffffffffu, got, 0) != 0;
}

// Which of the 32 keys [col0, col0 + 32) one query row may attend to, as a bit mask: keys below `limit` (the smaller of
// the valid key count and the causal boundary + 1), and, with a dense mask row, keys whose mask byte is non-zero.
__device__ __forceinline__ uint32_t visible_bits(int64_t col0, int64_t limit, const uint8_t* mrow) {
    const int64_t n = limit - col0;
    uint32_t bits = n >= 32 ? 0xffffffffu : n <= 0 ? 0u : ((1u << (int)n) - 1u);
    if (mrow != nullptr && bits != 0u) {
        const uint8_t* m = mrow + col0;
        uint32_t mb = 0u;
        if ((((uintptr_t)m) & 15) == 0 && n >= 32) {
            const uint4 a = *reinterpret_cast<const uint4*>(m), b = *reinterpret_cast<const uint4*>(m + 16);
            const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint32_t nz = __vcmpne4(w[i], 0u);     // 0xff per non-zero byte
                mb |= ((nz & 1u) | ((nz >> 7) & 2u) | ((nz >> 14) & 4u) | ((nz >> 21) & 8u)) << (4 * i);
            }
        } else {
            for (int i = 0; i < 32 && i < n; ++i) mb |= (m[i] != 0 ? 1u : 0u) << i;
        }
        bits &= mb;
    }
    return bits;
}

template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

template <int HD, typename T>
__global__ void __launch_bounds__(ATT_THREADS, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk, const __grid_constant__ CUtensorMap tv,
                 const AttnParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    constexpr int DC = HD / 64;                     // 64-column chunks of the (padded) head dim
    constexpr uint32_t TB = DC * CHUNK;             // bytes of one Q / K / V tile
    const uint32_t sQ = smem_u32(smem), sK = sQ + TB, sV = sK + 2 * TB, sP = sV + 2 * TB;
    AttnShared* sh = (AttnShared*)(smem + 5 * TB + 2 * CHUNK);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qt = (int)gridDim.x - 1 - (int)blockIdx.x;       // under a causal mask the long rows start first
    const int head = blockIdx.y, b = blockIdx.z, kvh = head / (p.h / p.hk);
    const int64_t q0 = (int64_t)qt * TILE;
    int64_t kv_end = p.sk;
    if (p.causal && q0 + TILE + p.causal_off < kv_end) kv_end = q0 + TILE + p.causal_off;
    if (p.kv_lens && p.kv_lens[b] < kv_end) kv_end = p.kv_lens[b];
    if (kv_end < 0) kv_end = 0;
    const int J = (int)((kv_end + TILE - 1) / TILE);           // key tiles this CTA visits

    if (threadIdx.x == 0) {
        mbar_init(&sh->q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&sh->k_full[i], 1); mbar_init(&sh->v_full[i], 1); mbar_init(&sh->k_empty[i], 1); mbar_init(&sh->v_empty[i], 1);
            mbar_init(&sh->s_full[i], 1); mbar_init(&sh->s_free[i], 4);
        }
        mbar_init(&sh->p_ready, 4);
        mbar_init(&sh->p_free, 1);
        mbar_init(&sh->o_full, 1);
        sh->failed = 0;
        fence_barrier_init();
    }
    if (warp == 1) { tmem_alloc(&sh->tmem_base, 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;
    const uint32_t tmem_o = tmem + 256;             // S buffers: columns [0,128) and [128,256); the O accumulator behind them

    if (warp == 0) {
        // ------------------------------------------------------------------------------------------ TMA producer
        if (lane == 0 && J > 0) {
            const uint32_t qbar = smem_u32(&sh->q_full);
            mbar_expect_tx_u32(qbar, TB);
#pragma unroll
            for (int c = 0; c < DC; ++c) tma_load_4d_u32(&tq, qbar, sQ + c * CHUNK, c * 64, (int)q0, head, b);
            for (int j = 0; j < J; ++j) {
                const int st = j & 1;
                const uint32_t ph = (uint32_t)((j >> 1) & 1);
                if (!mbar_wait(&sh->k_empty[st], ph ^ 1)) { fail(sh, 1); break; }
                const uint32_t kbar = smem_u32(&sh->k_full[st]);
                mbar_expect_tx_u32(kbar, TB);
#pragma unroll
                for (int c = 0; c < DC; ++c) tma_load_4d_u32(&tk, kbar, sK + st * TB + c * CHUNK, c * 64, j * TILE, kvh, b);
                if (!mbar_wait(&sh->v_empty[st], ph ^ 1)) { fail(sh, 2); break; }
                const uint32_t vbar = smem_u32(&sh->v_full[st]);
                mbar_expect_tx_u32(vbar, TB);
#pragma unroll
                for (int c = 0; c < DC; ++c) tma_load_4d_u32(&tv, vbar, sV + st * TB + c * CHUNK, c * 64, j * TILE, kvh, b);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------------------------------ MMA issuer
        if (lane == 0 && J > 0) {
            const uint32_t hi = desc_hi(1024);
            const int ks_s = (p.d + 15) / 16;            // 16-deep steps of the Q K^T contraction
            bool ok = mbar_wait(&sh->q_full, 0);
            if (!ok) fail(sh, 3);
            auto issue_pv = [&](int i) -> bool {
                const int st = i & 1;
                const uint32_t ph = (uint32_t)((i >> 1) & 1);
                if (!mbar_wait(&sh->v_full[st], ph)) { fail(sh, 4); return false; }
                // P_i is in shared memory and, if the row maxima moved, the accumulator has been rescaled by its owners
                if (!mbar_wait(&sh->p_ready, (uint32_t)(i & 1))) { fail(sh, 5); return false; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_o;
#pragma unroll
                for (int ks = 0; ks < TILE / 16; ++ks) {
                    // A = P (128 x 128 keys, K-major): chunk ks / 4, 32 bytes per step inside the swizzle row
                    // B = V (128 keys x HD, head dim contiguous = MN-major): 16 key rows per step, chunks of 64 columns apart by CHUNK
                    const uint64_t ad = pack_desc(desc_lo(sP + (ks >> 2) * CHUNK + (ks & 3) * 32, 0), hi);
                    const uint64_t bd = pack_desc(desc_lo(sV + st * TB + ks * 2048, CHUNK), hi);
                    umma_f16(d_tmem, ad, bd, p.idesc_pv, (i | ks) != 0 ? 1u : 0u);   // O accumulates over all key tiles
                }
                umma_commit(&sh->v_empty[st]);
                umma_commit(&sh->p_free);
                umma_commit(&sh->o_full);
                return true;
            };
            for (int j = 0; j < J && ok; ++j) {
                const int st = j & 1;
                const uint32_t ph = (uint32_t)((j >> 1) & 1);
                if (!mbar_wait(&sh->k_full[st], ph)) { fail(sh, 7); ok = false; break; }
                if (!mbar_wait(&sh->s_free[st], ph ^ 1)) { fail(sh, 8); ok = false; break; }
                tc_fence_after();
                for (int ks = 0; ks < ks_s; ++ks) {
                    const uint32_t off = (uint32_t)((ks >> 2) * CHUNK + (ks & 3) * 32);
                    const uint64_t ad = pack_desc(desc_lo(sQ + off, 0), hi);
                    const uint64_t bd = pack_desc(desc_lo(sK + st * TB + off, 0), hi);
                    umma_f16(tmem + st * TILE, ad, bd, p.idesc_s, ks != 0 ? 1u : 0u);
                }
                umma_commit(&sh->k_empty[st]);
                umma_commit(&sh->s_full[st]);
                if (j >= 1) ok = issue_pv(j - 1);
            }
            if (ok) issue_pv(J - 1);
        }
    } else {
        // ------------------------------------------------------------------------------------------ softmax + epilogue
        const int quarter = warp & 3;                 // TMEM lanes [32 * quarter, 32 * quarter + 32) belong to this warp
        const int row = quarter * 32 + lane;
        const int64_t qi = q0 + row;                  // query index of this thread
        const bool row_ok = qi < p.sq;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const uint8_t* mrow = (p.mask && row_ok) ? p.mask + ((int64_t)b * p.sq + qi) * p.sk : nullptr;
        const int64_t causal_last = p.causal ? qi + p.causal_off : p.sk;   // last visible key of this row under the causal rule
        // m_ref: the maximum the exponents are taken against.  It follows the running maximum lazily: only when that
        // has grown by more than 8 (in base-2 exponent units) is the accumulator in tensor memory rescaled -- probabilities
        // stay below 2^8, sums are fp32 -- so that after the first few tiles a tile costs one round trip to tensor memory.
        float m_ref = -INFINITY, l_run = 0.f;
        bool ok = true;
        for (int j = 0; j < J && ok; ++j) {
            const int sb = j & 1;
            if (!warp_wait(&sh->s_full[sb], (uint32_t)((j >> 1) & 1), lane)) { if (lane == 0) fail(sh, 9); ok = false; break; }
            tc_fence_after();
            const int64_t kv0 = (int64_t)j * TILE;
            const bool need_mask = (kv0 + TILE > kv_end) || (p.causal && kv0 + TILE - 1 > q0 + p.causal_off) || mrow != nullptr;
            const uint32_t s_addr = tmem + lane_addr + sb * TILE;
            uint32_t r[TILE / 32][32];
#pragma unroll
            for (int c4 = 0; c4 < TILE / 32; ++c4) tmem_ld32(s_addr + c4 * 32, r[c4]);
            tmem_ld_wait();
            // the scores are in registers: the S buffer may take the tile after next
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh->s_free[sb]);
            uint32_t vis[TILE / 32];
#pragma unroll
            for (int c4 = 0; c4 < TILE / 32; ++c4) vis[c4] = 0xffffffffu;
            if (need_mask) {
                const int64_t limit = kv_end < causal_last + 1 ? kv_end : causal_last + 1;
#pragma unroll
                for (int c4 = 0; c4 < TILE / 32; ++c4) vis[c4] = visible_bits(kv0 + c4 * 32, limit, mrow);
            }
            // tiles away from the diagonal and the ragged edge (the common case) skip the per-element visibility tests
            float mt = -INFINITY;
            if (need_mask) {
#pragma unroll
                for (int c4 = 0; c4 < TILE / 32; ++c4)
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if ((vis[c4] >> i) & 1u) mt = fmaxf(mt, __uint_as_float(r[c4][i]));
            } else {
#pragma unroll
                for (int c4 = 0; c4 < TILE / 32; ++c4)
#pragma unroll
                    for (int i = 0; i < 32; ++i) mt = fmaxf(mt, __uint_as_float(r[c4][i]));
            }
            // move the reference maximum?  (first visible score of the row, or growth beyond the threshold)
            float alpha = 1.f;
            bool move = false;
            if (mt != -INFINITY) {
                if (m_ref == -INFINITY) { m_ref = mt; }               // nothing accumulated yet: O and l are zero
                else if ((mt - m_ref) * p.sl2 > 8.f) { alpha = ex2((m_ref - mt) * p.sl2); m_ref = mt; move = true; }
            }
            // the previous tile's MMAs have read P (and, when rescaling, must have finished adding into O)
            if (!warp_wait(&sh->p_free, (uint32_t)((j & 1) ^ 1), lane)) { if (lane == 0) fail(sh, 10); ok = false; break; }
            if (j > 0 && __any_sync(0xffffffffu, move)) {
                // rescale this warp's 32 rows of the accumulator (lanes whose maximum did not move multiply by one)
                tc_fence_after();
                l_run *= alpha;
#pragma unroll
                for (int c4 = 0; c4 < HD / 32; ++c4) {
                    uint32_t o[32];
                    tmem_ld32(tmem_o + lane_addr + c4 * 32, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tmem_st32(tmem_o + lane_addr + c4 * 32, o);
                }
                tmem_st_wait();
            } else {
                l_run *= alpha;
            }
            const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref * p.sl2;
            float rowsum = 0.f;
#pragma unroll
            for (int c4 = 0; c4 < TILE / 32; ++c4) {
                const uint32_t base = sP + (uint32_t)(c4 >> 1) * CHUNK + (uint32_t)row * 128;
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    float pv[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        float e = ex2(fmaf(__uint_as_float(r[c4][8 * t + i]), p.sl2, neg_m));
                        if (need_mask && !((vis[c4] >> (8 * t + i)) & 1u)) e = 0.f;
                        pv[i] = e;
                        rowsum += e;
                    }
                    const uint32_t piece = (uint32_t)(((c4 & 1) * 4 + t) ^ (row & 7));
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(base + (piece << 4)),
                                 "r"(pack2<T>(pv[0], pv[1])), "r"(pack2<T>(pv[2], pv[3])),
                                 "r"(pack2<T>(pv[4], pv[5])), "r"(pack2<T>(pv[6], pv[7])) : "memory");
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy stores before the MMA's async-proxy reads
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh->p_ready);
            l_run += rowsum;
        }
        if (ok && J > 0) {
            if (!warp_wait(&sh->o_full, (uint32_t)((J - 1) & 1), lane)) { if (lane == 0) fail(sh, 12); ok = false; }
        }
        if (ok) {
            // normalise and store the row (the tensor-memory loads are warp-wide; only the stores depend on the row)
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            T* orow = (T*)p.o + (int64_t)b * p.o_batch + qi * p.o_tok + (int64_t)head * p.o_head;
            tc_fence_after();
#pragma unroll
            for (int c4 = 0; c4 < HD / 32; ++c4) {
                uint32_t o[32];
                if (J > 0) {
                    tmem_ld32(tmem_o + lane_addr + c4 * 32, o);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = 0u;
                }
                if (row_ok) {
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        if (c4 * 32 + t * 8 < p.d) {
                            bmt::Vec16<T> ov;
#pragma unroll
                            for (int i = 0; i < 8; ++i) ov.v[i] = bmt::Cvt<T>::from_f(__uint_as_float(o[t * 8 + i]) * inv);
                            bmt::st16(orow + c4 * 32 + t * 8, ov);
                        }
                    }
                }
            }
            tc_fence_before();
            if (row_ok && p.lse)
                p.lse[((int64_t)b * p.h + head) * p.sq + qi] = l_run > 0.f ? (m_ref * p.sl2 + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
        }
    }

    // ---------------------------------------------------------------------------------------------- teardown
    __syncthreads();
    if (sh->failed) {
        // a wait ran out: give copies that are still in flight time to land before the shared memory goes away
        const uint64_t t0 = global_ns();
        while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
        __syncthreads();
    }
    tc_fence_after();
    if (warp == 1) tmem_dealloc(tmem, 512);
}

template <int HD, typename T>
int launch_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& p, int64_t batch, cudaStream_t stream) {
    constexpr uint32_t TB = (HD / 64) * CHUNK;
    const size_t smem = 5 * TB + 2 * CHUNK + sizeof(AttnShared) + 1024;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(flash_fwd_kernel<HD, T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return -30;
        configured = true;
    }
    dim3 grid((unsigned)((p.sq + TILE - 1) / TILE), (unsigned)p.h, (unsigned)batch);
    flash_fwd_kernel<HD, T><<<grid, ATT_THREADS, smem, stream>>>(tq, tk, tv, p);
    bmt_count_launch(1);
    return cudaGetLastError() == cudaSuccess ? 0 : -31;
}


// ================================================================================================ backward
// One CTA per (128 keys, kv head, sample).  K and V tiles stay in shared memory; the CTA walks over the query heads that
// share the kv head and over the query tiles that can see its keys.  Per (query tile, key tile) pair:
//   MMA   S = Q K^T and dP = dO V^T into tensor memory
//   warps P = exp2(S * scale * log2e - lse * log2e) (masked), dS = P * (dP - delta) * scale; both written to shared
//         memory as fp16/bf16 in the swizzled [query][key] layout, which serves as a K-major operand (dQ) and,
//         read "transposed", as an MN-major operand (dV, dK)
//   MMA   dV += P^T dO, dK += dS^T Q (accumulating in tensor memory over the whole walk), dQ = dS K
//   warps dQ rows are added to an fp32 accumulator in global memory (vector reductions); a small kernel converts it
// delta = rowsum(dO * O) comes from a pre-pass.  dK / dV are written once at the end, already summed over the group.
struct AttnBwdParams {
    int64_t sq, sk;
    int h, hk, d;
    float sl2, scale;
    int causal;
    int64_t causal_off;
    const uint8_t* mask;
    const int32_t* kv_lens;
    const float* lse;
    const float* delta;
    float* dq_acc;              // (b, sq, h, d) fp32, zero on entry
    void* dk; void* dv;         // (b, sk, hk, d) by strides {token, head, batch}
    int64_t dk_tok, dk_head, dk_batch, dv_tok, dv_head, dv_batch;
    uint32_t idesc_s, idesc_tn, idesc_dq;
};

struct BwdShared {
    uint64_t kv_full, qdo_full, qdo_empty, sdp_full, pds_ready, dq_full, tmem_free;
    uint32_t tmem_base;
    int failed;
};

__device__ __forceinline__ void fail_bwd(BwdShared* sh, int code) {
    sh->failed = 1;
    atomicCAS(&g_attn_status, 0, ((0x40 | code) << 16) | (int)(blockIdx.x & 0xffff));
}

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

template <int HD, typename T>
__global__ void __launch_bounds__(ATT_THREADS, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk, const __grid_constant__ CUtensorMap tv,
                 const __grid_constant__ CUtensorMap tdo, const AttnBwdParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    constexpr int DC = HD / 64;
    constexpr uint32_t TB = DC * CHUNK;
    const uint32_t sK = smem_u32(smem), sV = sK + TB, sQ = sV + TB, sdO = sQ + TB, sP = sdO + TB, sdS = sP + 2 * CHUNK;
    BwdShared* sh = (BwdShared*)(smem + 4 * TB + 4 * CHUNK);
    // tensor memory columns: S [0,128), dP [128,256), dV, dK behind them; dQ has columns of its own when they fit,
    // otherwise it reuses the S columns (S has been read by the time dS exists)
    constexpr uint32_t C_DP = 128, C_DV = 256, C_DK = 256 + HD, C_DQ = (256 + 3 * HD <= 512) ? 256 + 2 * HD : 0;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kt = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int group = p.h / p.hk;
    const int64_t kv0 = (int64_t)kt * TILE;
    int64_t kv_valid = p.sk;
    if (p.kv_lens && p.kv_lens[b] < kv_valid) kv_valid = p.kv_lens[b];
    const int n_qt = (int)((p.sq + TILE - 1) / TILE);
    int qt_first = 0;
    if (p.causal && kv0 - p.causal_off > 0) qt_first = (int)((kv0 - p.causal_off) / TILE);
    const int per_head = (kv0 < kv_valid && qt_first < n_qt) ? n_qt - qt_first : 0;
    const int n_it = per_head * group;

    if (threadIdx.x == 0) {
        mbar_init(&sh->kv_full, 1); mbar_init(&sh->qdo_full, 1); mbar_init(&sh->qdo_empty, 1); mbar_init(&sh->sdp_full, 1);
        mbar_init(&sh->pds_ready, 4); mbar_init(&sh->dq_full, 1); mbar_init(&sh->tmem_free, 4);
        sh->failed = 0;
        fence_barrier_init();
    }
    if (warp == 1) { tmem_alloc(&sh->tmem_base, 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;

    if (warp == 0) {
        if (lane == 0 && n_it > 0) {
            const uint32_t kvbar = smem_u32(&sh->kv_full);
            mbar_expect_tx_u32(kvbar, 2 * TB);
#pragma unroll
            for (int c = 0; c < DC; ++c) {
                tma_load_4d_u32(&tk, kvbar, sK + c * CHUNK, c * 64, (int)kv0, kvh, b);
                tma_load_4d_u32(&tv, kvbar, sV + c * CHUNK, c * 64, (int)kv0, kvh, b);
            }
            for (int it = 0; it < n_it; ++it) {
                const int head = kvh * group + it / per_head, qt = qt_first + it % per_head;
                if (!mbar_wait(&sh->qdo_empty, (uint32_t)((it & 1) ^ 1))) { fail_bwd(sh, 1); break; }
                const uint32_t bar = smem_u32(&sh->qdo_full);
                mbar_expect_tx_u32(bar, 2 * TB);
#pragma unroll
                for (int c = 0; c < DC; ++c) {
                    tma_load_4d_u32(&tq, bar, sQ + c * CHUNK, c * 64, qt * TILE, head, b);
                    tma_load_4d_u32(&tdo, bar, sdO + c * CHUNK, c * 64, qt * TILE, head, b);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && n_it > 0) {
            const uint32_t hi = desc_hi(1024);
            const int ks_d = (p.d + 15) / 16;
            bool ok = mbar_wait(&sh->kv_full, 0);
            if (!ok) fail_bwd(sh, 2);
            for (int it = 0; it < n_it && ok; ++it) {
                const uint32_t ph = (uint32_t)(it & 1);
                if (!mbar_wait(&sh->qdo_full, ph)) { fail_bwd(sh, 3); break; }
                if (!mbar_wait(&sh->tmem_free, ph ^ 1)) { fail_bwd(sh, 4); break; }
                tc_fence_after();
                for (int ks = 0; ks < ks_d; ++ks) {
                    const uint32_t off = (uint32_t)((ks >> 2) * CHUNK + (ks & 3) * 32);
                    umma_f16(tmem, pack_desc(desc_lo(sQ + off, 0), hi), pack_desc(desc_lo(sK + off, 0), hi), p.idesc_s, ks != 0 ? 1u : 0u);
                }
                for (int ks = 0; ks < ks_d; ++ks) {
                    const uint32_t off = (uint32_t)((ks >> 2) * CHUNK + (ks & 3) * 32);
                    umma_f16(tmem + C_DP, pack_desc(desc_lo(sdO + off, 0), hi), pack_desc(desc_lo(sV + off, 0), hi), p.idesc_s, ks != 0 ? 1u : 0u);
                }
                umma_commit(&sh->sdp_full);
                if (!mbar_wait(&sh->pds_ready, ph)) { fail_bwd(sh, 5); break; }
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < TILE / 16; ++ks)      // dV += P^T dO: 16 query rows per step, both operands MN-major
                    umma_f16(tmem + C_DV, pack_desc(desc_lo(sP + ks * 2048, CHUNK), hi), pack_desc(desc_lo(sdO + ks * 2048, CHUNK), hi),
                             p.idesc_tn, (it | ks) != 0 ? 1u : 0u);
#pragma unroll
                for (int ks = 0; ks < TILE / 16; ++ks)      // dK += dS^T Q
                    umma_f16(tmem + C_DK, pack_desc(desc_lo(sdS + ks * 2048, CHUNK), hi), pack_desc(desc_lo(sQ + ks * 2048, CHUNK), hi),
                             p.idesc_tn, (it | ks) != 0 ? 1u : 0u);
                umma_commit(&sh->qdo_empty);
#pragma unroll
                for (int ks = 0; ks < TILE / 16; ++ks)      // dQ = dS K: 16 keys per step, A K-major, B (K tile) MN-major
                    umma_f16(tmem + C_DQ, pack_desc(desc_lo(sdS + (ks >> 2) * CHUNK + (ks & 3) * 32, 0), hi),
                             pack_desc(desc_lo(sK + ks * 2048, CHUNK), hi), p.idesc_dq, ks != 0 ? 1u : 0u);
                umma_commit(&sh->dq_full);
            }
        }
    } else {
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        bool ok = true;
        for (int it = 0; it < n_it && ok; ++it) {
            const uint32_t ph = (uint32_t)(it & 1);
            const int head = kvh * group + it / per_head, qt = qt_first + it % per_head;
            const int64_t q0 = (int64_t)qt * TILE, qi = q0 + row;
            const bool row_ok = qi < p.sq;
            float lse_r = -INFINITY, delta_r = 0.f;
            if (row_ok) {
                lse_r = p.lse[((int64_t)b * p.h + head) * p.sq + qi];
                delta_r = p.delta[((int64_t)b * p.h + head) * p.sq + qi];
            }
            const bool alive = row_ok && lse_r != -INFINITY;
            const float nlse = alive ? -lse_r * 1.4426950408889634f : 0.f;
            const uint8_t* mrow = (p.mask && row_ok) ? p.mask + ((int64_t)b * p.sq + qi) * p.sk : nullptr;
            const int64_t causal_last = p.causal ? qi + p.causal_off : p.sk;
            const bool need_mask = (kv0 + TILE > kv_valid) || (p.causal && kv0 + TILE - 1 > q0 + p.causal_off) || mrow != nullptr;
            if (!warp_wait(&sh->sdp_full, ph, lane)) { if (lane == 0) fail_bwd(sh, 6); ok = false; break; }
            tc_fence_after();
            // A tensor-memory load costs a round trip of a few hundred nanoseconds however wide it is, so the loads of 64
            // columns of S and of dP are issued together and waited for once (two round trips per tile).
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                uint32_t rs[2][32], rd[2][32];
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    tmem_ld32(tmem + lane_addr + (half * 2 + u) * 32, rs[u]);
                    tmem_ld32(tmem + lane_addr + C_DP + (half * 2 + u) * 32, rd[u]);
                }
                tmem_ld_wait();
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const int c4 = half * 2 + u;
                    uint32_t bits = alive ? 0xffffffffu : 0u;
                    if (need_mask && alive) bits = visible_bits(kv0 + c4 * 32, kv_valid < causal_last + 1 ? kv_valid : causal_last + 1, mrow);
                    const uint32_t off = (uint32_t)half * CHUNK + (uint32_t)row * 128;
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        float pv[8], ds[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float e = ((bits >> (8 * t + i)) & 1u) ? ex2(fmaf(__uint_as_float(rs[u][8 * t + i]), p.sl2, nlse)) : 0.f;
                            pv[i] = e;
                            ds[i] = e * (__uint_as_float(rd[u][8 * t + i]) - delta_r) * p.scale;
                        }
                        const uint32_t piece = (uint32_t)((u * 4 + t) ^ (row & 7)) << 4;
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sP + off + piece),
                                     "r"(pack2<T>(pv[0], pv[1])), "r"(pack2<T>(pv[2], pv[3])),
                                     "r"(pack2<T>(pv[4], pv[5])), "r"(pack2<T>(pv[6], pv[7])) : "memory");
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sdS + off + piece),
                                     "r"(pack2<T>(ds[0], ds[1])), "r"(pack2<T>(ds[2], ds[3])),
                                     "r"(pack2<T>(ds[4], ds[5])), "r"(pack2<T>(ds[6], ds[7])) : "memory");
                    }
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh->pds_ready);
            if (!warp_wait(&sh->dq_full, ph, lane)) { if (lane == 0) fail_bwd(sh, 7); ok = false; break; }
            tc_fence_after();
            float* dq_row = p.dq_acc + (((int64_t)b * p.sq + qi) * p.h + head) * p.d;
            {
                uint32_t r[HD / 32][32];
#pragma unroll
                for (int c4 = 0; c4 < HD / 32; ++c4) tmem_ld32(tmem + lane_addr + C_DQ + c4 * 32, r[c4]);
                tmem_ld_wait();
                // the values are in registers: the tensor memory may be overwritten by the next tile's MMAs while the
                // reductions below are still being issued
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&sh->tmem_free);
                if (row_ok) {
#pragma unroll
                    for (int c4 = 0; c4 < HD / 32; ++c4)
#pragma unroll
                        for (int t = 0; t < 8; ++t)
                            if (c4 * 32 + t * 4 < p.d)
                                red_add_v4(dq_row + c4 * 32 + t * 4, __uint_as_float(r[c4][4 * t]), __uint_as_float(r[c4][4 * t + 1]),
                                           __uint_as_float(r[c4][4 * t + 2]), __uint_as_float(r[c4][4 * t + 3]));
                }
            }
        }
        // dK, dV rows of this CTA's keys (zeros when no query sees them).  The tensor-memory loads are warp-wide, so every
        // lane takes part in them; only the stores depend on the row.
        const int64_t kj = kv0 + row;
        if (ok) {
            T* dkr = (T*)p.dk + (int64_t)b * p.dk_batch + kj * p.dk_tok + (int64_t)kvh * p.dk_head;
            T* dvr = (T*)p.dv + (int64_t)b * p.dv_batch + kj * p.dv_tok + (int64_t)kvh * p.dv_head;
#pragma unroll
            for (int c4 = 0; c4 < HD / 32; ++c4) {
                uint32_t rk[32], rv[32];
                if (n_it > 0) {
                    tmem_ld32(tmem + lane_addr + C_DK + c4 * 32, rk);
                    tmem_ld32(tmem + lane_addr + C_DV + c4 * 32, rv);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) rk[i] = rv[i] = 0u;
                }
                if (kj < p.sk) {
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        if (c4 * 32 + t * 8 < p.d) {
                            bmt::Vec16<T> ok8, ov8;
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                ok8.v[i] = bmt::Cvt<T>::from_f(__uint_as_float(rk[t * 8 + i]));
                                ov8.v[i] = bmt::Cvt<T>::from_f(__uint_as_float(rv[t * 8 + i]));
                            }
                            bmt::st16(dkr + c4 * 32 + t * 8, ok8);
                            bmt::st16(dvr + c4 * 32 + t * 8, ov8);
                        }
                    }
                }
            }
        }
        tc_fence_before();
    }

    __syncthreads();
    if (sh->failed) {
        const uint64_t t0 = global_ns();
        while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
        __syncthreads();
    }
    tc_fence_after();
    if (warp == 1) tmem_dealloc(tmem, 512);
}

// delta[b, h, q] = sum_d dO[b, q, h, d] * O[b, q, h, d]; one warp per row
template <typename T>
__global__ void attn_delta_kernel(const T* o, int64_t o_tok, int64_t o_head, int64_t o_batch, const T* dout, int64_t g_tok, int64_t g_head,
                                  int64_t g_batch, float* delta, int64_t batch, int64_t sq, int h, int d) {
    const int64_t w = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (w >= batch * sq * h) return;
    const int head = (int)(w % h);
    const int64_t qi = (w / h) % sq, bb = w / ((int64_t)h * sq);
    const T* orow = o + bb * o_batch + qi * o_tok + head * o_head;
    const T* grow = dout + bb * g_batch + qi * g_tok + head * g_head;
    float acc = 0.f;
    for (int c = lane * 8; c < d; c += 256) {
        const bmt::Vec16<T> a = bmt::ld16(orow + c), g = bmt::ld16(grow + c);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc += bmt::Cvt<T>::to_f(a.v[i]) * bmt::Cvt<T>::to_f(g.v[i]);
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
    if (lane == 0) delta[(bb * h + head) * sq + qi] = acc;
}

// dq[b, q, h, :] (strided, T) <- dq_acc (b, sq, h, d) fp32
template <typename T>
__global__ void attn_dq_convert_kernel(const float* acc, T* dq, int64_t q_tok, int64_t q_head, int64_t q_batch, int64_t batch, int64_t sq,
                                       int h, int d) {
    const int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;   // one 8-element vector per thread
    const int per_row = d / 8;
    if (v >= batch * sq * h * per_row) return;
    const int c = (int)(v % per_row) * 8;
    const int64_t r = v / per_row;
    const int head = (int)(r % h);
    const int64_t qi = (r / h) % sq, bb = r / ((int64_t)h * sq);
    const float4 a0 = *reinterpret_cast<const float4*>(acc + r * d + c), a1 = *reinterpret_cast<const float4*>(acc + r * d + c + 4);
    bmt::Vec16<T> o;
    o.v[0] = bmt::Cvt<T>::from_f(a0.x); o.v[1] = bmt::Cvt<T>::from_f(a0.y); o.v[2] = bmt::Cvt<T>::from_f(a0.z); o.v[3] = bmt::Cvt<T>::from_f(a0.w);
    o.v[4] = bmt::Cvt<T>::from_f(a1.x); o.v[5] = bmt::Cvt<T>::from_f(a1.y); o.v[6] = bmt::Cvt<T>::from_f(a1.z); o.v[7] = bmt::Cvt<T>::from_f(a1.w);
    bmt::st16(dq + bb * q_batch + qi * q_tok + head * q_head + c, o);
}

template <int HD, typename T>
int launch_bwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo, const AttnBwdParams& p,
               int64_t batch, cudaStream_t stream) {
    constexpr uint32_t TB = (HD / 64) * CHUNK;
    const size_t smem = 4 * TB + 4 * CHUNK + sizeof(BwdShared) + 1024;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(flash_bwd_kernel<HD, T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return -30;
        configured = true;
    }
    dim3 grid((unsigned)((p.sk + TILE - 1) / TILE), (unsigned)p.hk, (unsigned)batch);
    flash_bwd_kernel<HD, T><<<grid, ATT_THREADS, smem, stream>>>(tq, tk, tv, tdo, p);
    bmt_count_launch(1);
    return cudaGetLastError() == cudaSuccess ? 0 : -31;
}

template <typename T>
int run_bwd(int64_t batch, int64_t sq, int64_t sk, int h, int hk, int d, const void* q, const int64_t* qs, const void* k, const int64_t* ks,
            const void* v, const int64_t* vs, const void* o, const int64_t* os, const void* dout, const int64_t* gs, const void* lse,
            void* dq, const int64_t* dqs, void* dk, const int64_t* dks, void* dv, const int64_t* dvs, void* dq_acc, void* delta, float scale,
            int causal, const void* mask, const void* kv_lens, int dtype, cudaStream_t st) {
    const int hd = d <= 64 ? 64 : 128;
    CUtensorMap tq, tk, tv, tdo;
    int rc;
    if ((rc = bmt_tma_map_4d(&tq, q, dtype, d, sq, qs[0], h, qs[1], batch, qs[2], 64, TILE)) != 0) return rc;
    if ((rc = bmt_tma_map_4d(&tk, k, dtype, d, sk, ks[0], hk, ks[1], batch, ks[2], 64, TILE)) != 0) return rc;
    if ((rc = bmt_tma_map_4d(&tv, v, dtype, d, sk, vs[0], hk, vs[1], batch, vs[2], 64, TILE)) != 0) return rc;
    if ((rc = bmt_tma_map_4d(&tdo, dout, dtype, d, sq, gs[0], h, gs[1], batch, gs[2], 64, TILE)) != 0) return rc;
    const int64_t rows = batch * sq * h;
    if (cudaMemsetAsync(dq_acc, 0, (size_t)rows * d * sizeof(float), st) != cudaSuccess) return -32;
    attn_delta_kernel<T><<<(unsigned)((rows * 32 + 255) / 256), 256, 0, st>>>((const T*)o, os[0], os[1], os[2], (const T*)dout, gs[0], gs[1],
                                                                                gs[2], (float*)delta, batch, sq, h, d);
    AttnBwdParams p;
    memset(&p, 0, sizeof(p));
    p.sq = sq; p.sk = sk; p.h = h; p.hk = hk; p.d = d;
    p.scale = scale; p.sl2 = scale * 1.4426950408889634f;
    p.causal = causal; p.causal_off = sk - sq;
    p.mask = (const uint8_t*)mask; p.kv_lens = (const int32_t*)kv_lens;
    p.lse = (const float*)lse; p.delta = (const float*)delta; p.dq_acc = (float*)dq_acc;
    p.dk = dk; p.dk_tok = dks[0]; p.dk_head = dks[1]; p.dk_batch = dks[2];
    p.dv = dv; p.dv_tok = dvs[0]; p.dv_head = dvs[1]; p.dv_batch = dvs[2];
    const uint32_t fmt = dtype == BMT_DT_F16 ? 0u : 1u;
    const uint32_t common = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(TILE >> 4) << 24);
    p.idesc_s = common | ((uint32_t)(TILE >> 3) << 17);
    p.idesc_tn = common | (1u << 15) | (1u << 16) | ((uint32_t)(hd >> 3) << 17);
    p.idesc_dq = common | (1u << 16) | ((uint32_t)(hd >> 3) << 17);
    rc = hd == 64 ? launch_bwd<64, T>(tq, tk, tv, tdo, p, batch, st) : launch_bwd<128, T>(tq, tk, tv, tdo, p, batch, st);
    if (rc != 0) return rc;
    const int64_t vecs = rows * (d / 8);
    attn_dq_convert_kernel<T><<<(unsigned)((vecs + 255) / 256), 256, 0, st>>>((const float*)dq_acc, (T*)dq, dqs[0], dqs[1], dqs[2], batch, sq, h, d);
    bmt_count_launch(3);
    return cudaGetLastError() == cudaSuccess ? 0 : -33;
}

}  // namespace

// q (b, sq, h, d), k / v (b, sk, hk, d), o (b, sq, h, d): element strides given per tensor as {token, head, batch}, the
// head dim is contiguous.  d: multiple of 16, at most 128; every stride a multiple of 8, pointers 16-byte aligned.
// lse (b, h, sq) fp32 or NULL.  mask: (b, sq, sk) bytes or NULL; kv_lens: (b) int32 or NULL.
extern "C" int bmt_flash_attn_fwd(int64_t batch, int64_t sq, int64_t sk, int h, int hk, int d, const void* q, const int64_t* q_strides,
                                  const void* k, const int64_t* k_strides, const void* v, const int64_t* v_strides, void* o,
                                  const int64_t* o_strides, void* lse, float scale, int causal, const void* mask, const void* kv_lens,
                                  int dtype, void* stream) {
    if (d <= 0 || d > 128 || (d & 15) || h % hk || batch <= 0 || sq <= 0 || sk <= 0) return -1;
    if (((uintptr_t)o & 15) || (o_strides[0] & 7) || (o_strides[1] & 7) || (o_strides[2] & 7)) return -2;
    const int hd = d <= 64 ? 64 : 128;
    CUtensorMap tq, tk, tv;
    int rc;
    if ((rc = bmt_tma_map_4d(&tq, q, dtype, d, sq, q_strides[0], h, q_strides[1], batch, q_strides[2], 64, TILE)) != 0) return rc;
    if ((rc = bmt_tma_map_4d(&tk, k, dtype, d, sk, k_strides[0], hk, k_strides[1], batch, k_strides[2], 64, TILE)) != 0) return rc;
    if ((rc = bmt_tma_map_4d(&tv, v, dtype, d, sk, v_strides[0], hk, v_strides[1], batch, v_strides[2], 64, TILE)) != 0) return rc;
    AttnParams p;
    memset(&p, 0, sizeof(p));
    p.sq = sq; p.sk = sk; p.h = h; p.hk = hk; p.d = d;
    p.sl2 = scale * 1.4426950408889634f;
    p.causal = causal; p.causal_off = sk - sq;
    p.mask = (const uint8_t*)mask; p.kv_lens = (const int32_t*)kv_lens;
    p.o = o; p.o_tok = o_strides[0]; p.o_head = o_strides[1]; p.o_batch = o_strides[2];
    p.lse = (float*)lse;
    const uint32_t fmt = dtype == BMT_DT_F16 ? 0u : 1u;
    const uint32_t common = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(TILE >> 4) << 24);
    p.idesc_s = common | ((uint32_t)(TILE >> 3) << 17);                       // A, B K-major; N = 128 keys
    p.idesc_pv = common | (1u << 16) | ((uint32_t)(hd >> 3) << 17);           // B (V) MN-major; N = padded head dim
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == BMT_DT_F16) return hd == 64 ? launch_fwd<64, __half>(tq, tk, tv, p, batch, st) : launch_fwd<128, __half>(tq, tk, tv, p, batch, st);
    if (dtype == BMT_DT_BF16) return hd == 64 ? launch_fwd<64, __nv_bfloat16>(tq, tk, tv, p, batch, st) : launch_fwd<128, __nv_bfloat16>(tq, tk, tv, p, batch, st);
    return -3;
}

// status of the attention kernels: 0, or (wait code << 16 | CTA) of the first CTA that gave up; reading clears it
extern "C" int bmt_attn_status(void) {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_attn_status, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_attn_status, &zero, sizeof(int));
    return v;
}

// Backward of bmt_flash_attn_fwd.  o / lse are the forward's results, dout the gradient of o; dq, dk, dv receive the
// gradients (strided like their operands).  dq_acc: scratch of batch * sq * h * d floats, delta: batch * h * sq floats.
// All tensors follow the forward's stride and alignment rules.
extern "C" int bmt_flash_attn_bwd(int64_t batch, int64_t sq, int64_t sk, int h, int hk, int d, const void* q, const int64_t* q_strides,
                                  const void* k, const int64_t* k_strides, const void* v, const int64_t* v_strides, const void* o,
                                  const int64_t* o_strides, const void* dout, const int64_t* do_strides, const void* lse, void* dq,
                                  const int64_t* dq_strides, void* dk, const int64_t* dk_strides, void* dv, const int64_t* dv_strides,
                                  void* dq_acc, void* delta, float scale, int causal, const void* mask, const void* kv_lens, int dtype,
                                  void* stream) {
    if (d <= 0 || d > 128 || (d & 15) || h % hk || batch <= 0 || sq <= 0 || sk <= 0) return -1;
    const int64_t* all[] = {o_strides, dq_strides, dk_strides, dv_strides};
    for (const int64_t* s3 : all)
        if ((s3[0] & 7) || (s3[1] & 7) || (s3[2] & 7)) return -2;
    if (((uintptr_t)o | (uintptr_t)dq | (uintptr_t)dk | (uintptr_t)dv | (uintptr_t)dq_acc) & 15) return -2;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == BMT_DT_F16)
        return run_bwd<__half>(batch, sq, sk, h, hk, d, q, q_strides, k, k_strides, v, v_strides, o, o_strides, dout, do_strides, lse, dq,
                               dq_strides, dk, dk_strides, dv, dv_strides, dq_acc, delta, scale, causal, mask, kv_lens, dtype, st);
    if (dtype == BMT_DT_BF16)
        return run_bwd<__nv_bfloat16>(batch, sq, sk, h, hk, d, q, q_strides, k, k_strides, v, v_strides, o, o_strides, dout, do_strides, lse,
                                      dq, dq_strides, dk, dk_strides, dv, dv_strides, dq_acc, delta, scale, causal, mask, kv_lens, dtype, st);
    return -3;
}
