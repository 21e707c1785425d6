// Persistent tcgen05 GEMM for sm_100a (B200).
//
//   C[b][M,N] (+)= alpha * op(A[b]) * op(B[b]) (+ bias[N]) , optional ReLU / GELU
//
// * fp16 / bf16 operands, fp32 accumulation in tensor memory (TMEM), output fp16 / bf16 / fp32.
// * Each operand may be "K-major" (reduction dim contiguous) or "MN-major" (output dim contiguous), so
//   forward (NT), dgrad (NN) and wgrad (TN) of a linear layer all run here without any transpose pass.
// * One CTA per SM, static persistent tile loop.  Warp roles:
//       warp 0      TMA producer  (cp.async.bulk.tensor, 128-byte swizzle, S-stage mbarrier pipeline)
//       warp 1      MMA issuer    (tcgen05.mma cta_group::1 kind::f16, 128 x BN x 16, one elected thread)
//       warps 2..5  epilogue      (tcgen05.ld 32x32b -> registers -> alpha/bias/activation -> global)
//   Two TMEM accumulator buffers let the epilogue of tile i overlap the main loop of tile i+1.
// * BN (16..256) is picked per problem to minimise wave quantisation on 148 SMs.
// * Every wait on an mbarrier is bounded (about two seconds of polling); on expiry the kernel records a code in a
//   device status word, lets in-flight copies land, frees its TMEM and returns.  Nothing traps.
// * No TMA multicast is used anywhere (every CTA loads its own tiles).
//
// The reference has no GEMM kernel: all matmuls go through cuBLAS (bmtrain/nn/linear.py:10-24).
#include <cuda.h>
#include <mutex>
#include <unordered_map>
#include <vector>
#include <stdio.h>
#include <string.h>

#include "api.h"
#include "common.cuh"
#include "tcgen05.cuh"

namespace {

using namespace bmt_tc;

constexpr int BM = 128;
constexpr int BK = 64;          // 64 halves = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;
constexpr int MAX_STAGES = 8;
constexpr uint32_t SMEM_BUDGET = 222 * 1024;  // tiles; header, alignment slack and the kernels' small static arrays fit below the 227 KiB limit

__device__ int g_gemm_status = 0;  // 0 = fine; otherwise (code << 16) | blockIdx of the first CTA that gave up
// Timing of the fused compute+collective kernels since the last read (nanoseconds of %globaltimer):
// [0] sum over the compute CTAs of the time their producer spent waiting for remote data, [1] longest pusher CTA,
// [2] longest CTA of any kind (main phase), [3] longest producer wait of one CTA, [4] kernels counted,
// [5] GEMM -> reduce-scatter: longest wait for the other ranks' deliveries, [6] longest CTA including its reduce phase,
// [7] sum over CTAs of that wait.
__device__ unsigned long long g_fused_stats[8] = {0, 0, 0, 0, 0, 0, 0, 0};

struct GemmParams {
    int64_t M, N, K;
    int bn;           // tile N
    int stages;
    uint32_t hdr_off;      // byte offset of the barrier header behind the tile stages (pusher CTAs need room for their ring)
    uint32_t out_stage_off;  // byte offset of the epilogue's row staging area (128 rows x OUT_PITCH) when rows go out as bulk copies
    int staged;              // plain GEMM: the epilogue stages rows in shared memory and writes them with bulk copies
    int a_mn, b_mn;   // 1 = MN-major operand
    int a_mn5, b_mn5; // the MN-major operand's tensor map has the 64-element chunks as a dimension of their own: one copy per
                      // stage brings all chunks of the tile (instead of one copy per chunk)
    int m_blocks, n_blocks;
    int64_t batch_inner, batch_outer, b_inner_div;
    void* c;
    int64_t ldc, c_bs0, c_bs1;
    int c_dtype;
    const void* bias;
    int bias_dtype;
    int act;
    int accumulate;
    float alpha;
    uint32_t idesc;
    const void* residual;  // optional (M x N, operand dtype, row pitch ldr): added after bias / activation
    int64_t ldr;
    const void* aux;       // optional (M x N, operand dtype, row pitch ld_aux) for the multiplicative epilogues
    int64_t ld_aux;
    int aux_mode;          // 0 none, 1: out *= (aux > 0)  (ReLU backward), 2: out *= gelu'(aux)
    int group_m;           // tile raster: consecutive tiles walk down `group_m` row blocks before moving to the next column block
    int debug;             // measurement only (BMT_GEMM_DEBUG): 1 = no TMA loads, 2 = no MMAs, 4 = no epilogue stores
};

__device__ __forceinline__ float gelu_f(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118654752f)); }

template <typename T> __device__ __forceinline__ void store8(T* dst, const float* v) {
    bmt::Vec16<T> o;
#pragma unroll
    for (int i = 0; i < 8; ++i) o.v[i] = bmt::Cvt<T>::from_f(v[i]);
    bmt::st16(dst, o);
}
template <typename T> __device__ __forceinline__ void load8(const T* src, float* v) {
    bmt::Vec16<T> o = bmt::ld16(src);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = bmt::Cvt<T>::to_f(o.v[i]);
}

// Sum of `world` inbox slots (+ bias) for the vectors [v0, v0 + U * stride) step stride: all U * world loads are issued
// before the first add so that enough bytes are in flight to stream from HBM.
template <typename T, int U, int WMAX>
__device__ __forceinline__ void rs_reduce_vectors(const T* inbox, int64_t slot_elems, int world, const T* bias, int64_t N, T* out,
                                                  int64_t v0, int64_t stride, int64_t nvec) {
    bmt::Vec16<T> t[U][WMAX];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int64_t v = v0 + u * stride;
        if (v < nvec) {
#pragma unroll
            for (int j = 0; j < WMAX; ++j)
                if (j < world) t[u][j] = bmt::ld16(inbox + j * slot_elems + v * 8);
        }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int64_t v = v0 + u * stride;
        if (v >= nvec) continue;
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
        for (int j = 0; j < WMAX; ++j)
            if (j < world) {
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] += bmt::Cvt<T>::to_f(t[u][j].v[i]);
            }
        if (bias) {
            float b[8];
            load8(bias + (v * 8) % N, b);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] += b[i];
        }
        store8(out + v * 8, acc);
    }
}

template <typename T>
__device__ __forceinline__ void rs_reduce_all(const void* inbox, int64_t slot_elems, int world, const void* bias, int64_t N, void* out,
                                              int64_t nvec) {
    const int64_t stride = (int64_t)gridDim.x * NUM_THREADS;
    const int64_t first = (int64_t)blockIdx.x * NUM_THREADS + threadIdx.x;
    if (world <= 2) {
        for (int64_t v = first; v < nvec; v += stride * 8)
            rs_reduce_vectors<T, 8, 2>((const T*)inbox, slot_elems, world, (const T*)bias, N, (T*)out, v, stride, nvec);
    } else if (world <= 4) {
        for (int64_t v = first; v < nvec; v += stride * 4)
            rs_reduce_vectors<T, 4, 4>((const T*)inbox, slot_elems, world, (const T*)bias, N, (T*)out, v, stride, nvec);
    } else {
        for (int64_t v = first; v < nvec; v += stride * 2)
            rs_reduce_vectors<T, 2, 8>((const T*)inbox, slot_elems, world, (const T*)bias, N, (T*)out, v, stride, nvec);
    }
}

// Grouped raster: the CTAs that run at the same time cover a compact (group_m x ~#SM/group_m) patch of output tiles, so
// every k-slice of A and B that one of them pulls from DRAM is found in L2 by the others.
__device__ __forceinline__ void tile_coords(const GemmParams& p, int64_t rem, int& m_blk, int& n_blk) {
    const int64_t per_group = (int64_t)p.group_m * p.n_blocks;
    const int64_t group = rem / per_group;
    const int first_m = (int)(group * p.group_m);
    const int rows = p.m_blocks - first_m < p.group_m ? p.m_blocks - first_m : p.group_m;
    const int64_t in_group = rem % per_group;
    m_blk = first_m + (int)(in_group % rows);
    n_blk = (int)(in_group / rows);
}

struct SharedHeader {
    uint64_t full[MAX_STAGES];
    uint64_t empty[MAX_STAGES];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    int failed;
};

__device__ __forceinline__ float gelu_grad_f(float x) {
    const float cdf = 0.5f * (1.f + erff(x * 0.70710678118654752f));
    return cdf + x * 0.3989422804014327f * __expf(-0.5f * x * x);
}
template <typename TA> __device__ __forceinline__ void apply_extras(const GemmParams& p, int64_t row, int64_t c, int64_t col_end, float* vv) {
    if (p.aux_mode) {
        const TA* ar = (const TA*)p.aux + row * p.ld_aux + c;
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (c + i < col_end) {
                const float a = bmt::Cvt<TA>::to_f(ar[i]);
                vv[i] = p.aux_mode == 1 ? (a > 0.f ? vv[i] : 0.f) : vv[i] * gelu_grad_f(a);
            }
    }
    if (p.residual) {
        const TA* rr = (const TA*)p.residual + row * p.ldr + c;
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (c + i < col_end) vv[i] += bmt::Cvt<TA>::to_f(rr[i]);
    }
}

// The arithmetic of epilogue_chunk without the store, for rows whose column count is a multiple of 8: v = final values of
// the columns [col0, min(col0 + 32, col_end)) of this thread's row (alpha, bias, activation, mask / residual, old C).
template <typename TC>
__device__ __forceinline__ void epilogue_math(const GemmParams& p, const TC* crow, int64_t row, int64_t col0, int64_t col_end,
                                              const uint32_t (&r)[32], float (&v)[32]) {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        const int64_t c = col0 + g * 8;
        if (c >= col_end) break;
        float* vv = v + g * 8;
        if (p.bias) {
            float b[8];
            if (p.bias_dtype == BMT_DT_F16) load8((const __half*)p.bias + c, b);
            else if (p.bias_dtype == BMT_DT_BF16) load8((const __nv_bfloat16*)p.bias + c, b);
            else {
#pragma unroll
                for (int i = 0; i < 8; ++i) b[i] = ((const float*)p.bias)[c + i];
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) vv[i] += b[i];
        }
        if (p.act == 1) {
#pragma unroll
            for (int i = 0; i < 8; ++i) vv[i] = fmaxf(vv[i], 0.f);
        } else if (p.act == 2) {
#pragma unroll
            for (int i = 0; i < 8; ++i) vv[i] = gelu_f(vv[i]);
        }
        if (p.aux_mode || p.residual) {
            if (p.bias_dtype == BMT_DT_F16) apply_extras<__half>(p, row, c, col_end, vv);
            else apply_extras<__nv_bfloat16>(p, row, c, col_end, vv);
        }
        if (p.accumulate) {
            float old[8];
            load8(crow + c, old);
#pragma unroll
            for (int i = 0; i < 8; ++i) vv[i] += old[i];
        }
    }
}

template <typename TC>
__device__ __forceinline__ void epilogue_chunk(const GemmParams& p, TC* crow, int64_t row, int64_t col0, int64_t col_end, const uint32_t (&r)[32], bool row_ok) {
    // this thread owns one output row and the columns [col0, min(col0 + 32, col_end))
    if (!row_ok) return;
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
    const bool vec = ((p.ldc & 7) == 0) && ((((uintptr_t)p.c) & 15) == 0) && (((p.c_bs0 | p.c_bs1) & 7) == 0) && sizeof(TC) == 2;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        const int64_t c = col0 + g * 8;
        if (c >= col_end) break;
        float* vv = v + g * 8;
        const bool full8 = c + 8 <= col_end;
        if (p.bias) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (c + i < col_end)
                    vv[i] += p.bias_dtype == BMT_DT_F16 ? __half2float(((const __half*)p.bias)[c + i])
                           : p.bias_dtype == BMT_DT_BF16 ? __bfloat162float(((const __nv_bfloat16*)p.bias)[c + i])
                                                         : ((const float*)p.bias)[c + i];
        }
        if (p.act == 1) {
#pragma unroll
            for (int i = 0; i < 8; ++i) vv[i] = fmaxf(vv[i], 0.f);
        } else if (p.act == 2) {
#pragma unroll
            for (int i = 0; i < 8; ++i) vv[i] = gelu_f(vv[i]);
        }
        if (p.aux_mode || p.residual) {
            if (p.bias_dtype == BMT_DT_F16) apply_extras<__half>(p, row, c, col_end, vv);
            else apply_extras<__nv_bfloat16>(p, row, c, col_end, vv);
        }
        if (full8 && vec) {
            if (p.accumulate) {
                float old[8];
                load8(crow + c, old);
#pragma unroll
                for (int i = 0; i < 8; ++i) vv[i] += old[i];
            }
            store8(crow + c, vv);
        } else if (full8 && sizeof(TC) == 4 && ((p.ldc & 3) == 0) && ((((uintptr_t)p.c) & 15) == 0)) {
            float4* d4 = reinterpret_cast<float4*>(crow + c);
            if (p.accumulate) {
                float4 o0 = d4[0], o1 = d4[1];
                vv[0] += o0.x; vv[1] += o0.y; vv[2] += o0.z; vv[3] += o0.w; vv[4] += o1.x; vv[5] += o1.y; vv[6] += o1.z; vv[7] += o1.w;
            }
            d4[0] = make_float4(vv[0], vv[1], vv[2], vv[3]);
            d4[1] = make_float4(vv[4], vv[5], vv[6], vv[7]);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (c + i < col_end) {
                    float o = vv[i];
                    if (p.accumulate) o += bmt::Cvt<TC>::to_f(crow[c + i]);
                    crow[c + i] = bmt::Cvt<TC>::from_f(o);
                }
        }
    }
}

// ---- two-CTA (cta_group::2) helpers: the pair shares one 256 x BN accumulator tile, each CTA feeds its own
// 128 rows of A and its own half of the B tile, the leader CTA (rank 0) issues the MMAs for both.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc_2cta(uint32_t* dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_2cta() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc_2cta(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16_2cta(uint32_t tmem_c, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_c), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrives on the barrier at the same shared-memory offset in both CTAs of the pair
__device__ __forceinline__ void umma_commit_2cta(uint64_t* bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(mask) : "memory");
}

// ---- fused collectives over peer memory (NVLink) ----------------------------------------------------------------
// mode 1, GEMM -> reduce-scatter: the epilogue stores every output row straight into the inbox of the rank that owns
//         the row (own rank: local memory, other ranks: P2P stores).  When all CTAs of this rank are done, the last one
//         publishes "rank r delivered" to every peer; each CTA then waits (bounded) for all ranks and sums the inbox
//         slots of its share of the local rows (+ bias) into the output.
// mode 2, all-gather -> GEMM: the first `ag_ctas` CTAs do no math; they push this rank's rows of A into the gathered
//         buffer of every rank (own first) in pieces and bump a per-128-row-block counter on the destination.  The
//         TMA producers of the compute CTAs visit local row blocks first and wait (bounded) on the counter of a block
//         before loading it, so the transfer overlaps the math block by block.
// Flags: `flags[j]` is rank j's flag array, row `x` of it has one counter per rank.  free_row: "my inbox / gathered
// buffer may be overwritten for this epoch" (published at kernel start); done_row: "my contributions are delivered".
struct FusedComm {
    int mode;                 // 0 none, 1 GEMM -> reduce-scatter, 2 all-gather -> GEMM
    int world, rank;
    unsigned int* flags[8];
    int free_row, done_row;
    unsigned int epoch;
    int* status;
    uint64_t limit_ns;
    // mode 1
    void* rs_inbox[8];        // destination j: base of slot `rank` inside j's inbox (rs_rows x N, pitch N)
    const void* rs_inbox_local;  // this rank's inbox: world slots of rs_rows x N
    int64_t rs_rows;          // rows per rank
    unsigned int* rs_counter; // local, monotonic: [0] epilogue warps that finished the tiles with rows of other ranks (early
                              // mode) or CTAs that finished all tiles; [1] early mode: CTAs that finished all tiles
    int rs_split;             // the kernel ends after publishing "delivered": waiting for the other ranks and summing the inbox
                              // are left to later launches (a one-CTA wait kernel and rs_reduce_kernel), so that no CTA of this
                              // grid holds an SM while it waits for another rank or for the rest of its own grid
    int rs_early;             // tiles with other ranks' rows come first and "delivered" is published when they are done
    int rs_bpr;               // early mode: tile rows per rank
    int64_t rs_remote_tiles;  // early mode: number of tiles (in raster order) that hold rows of other ranks
    void* rs_out;             // rs_rows x N
    const void* rs_bias;
    // mode 2
    int skip_local;           // modes 2/3: this rank's own part is already in its gathered buffer (copied before the launch)
    int ag_ctas;
    const void* ag_src;       // this rank's rows (ag_rows x K, pitch ag_ld_src)
    int64_t ag_ld_src, ag_rows;
    void* ag_dst[8];          // every rank's gathered buffer (world * ag_rows x K, pitch K)
    unsigned int* ag_count[8];// every rank's per-row-block counters
    int ag_piece_bytes;       // bytes per pushed piece: divides the bytes of a 128-row block, at most PUSH_PIECE_BYTES
    int ag_pieces_per_block;  // pieces per 128-row block
    int ag_runs_per_block;    // a block is pushed as this many runs of consecutive pieces, each by one CTA, each ending with
                              // one bump of the block's counter on the destination (what the counter grows by per epoch)
    // mode 3 (ZeRO weight gather -> GEMM): the B operand (N x K, rows contiguous) is cut over the ranks as a flat element
    // range; every rank pushes its part to all ranks in pieces and the TMA producer waits for the 128-row chunks it needs
    const char* bg_src;       // this rank's part (local shard memory)
    int64_t bg_first, bg_count;   // flat element range [bg_first, bg_first + bg_count) of the N*K weight elements
    void* bg_dst[8];          // start of the weight inside every rank's gathered buffer
    unsigned int* bg_cnt[8];  // every rank's per-chunk counters (chunk = 128 rows)
    const unsigned int* bg_expected;  // pieces a chunk receives in total, per chunk
    int bg_first_block;       // n-block at which this rank's own rows start (tile order is rotated to begin there)
    int bg_split;             // a rank's part of one 128-row chunk is pushed as up to this many runs (one counter bump each)
};
constexpr int64_t BG_PIECE = 16384;  // elements per pushed piece (32 KiB = one stage of the push pipeline)

__device__ __forceinline__ void st_release_sys_u32(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys_u32(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// Bounded poll until *p >= target (counters only grow).
__device__ __forceinline__ bool wait_counter(const unsigned int* p, unsigned int target, uint64_t limit_ns) {
    uint64_t t0 = 0;
    for (unsigned int spins = 0;; ++spins) {
        if ((int)(ld_acquire_sys_u32(p) - target) >= 0) return true;
        if ((spins & 255u) == 255u) {
            const uint64_t now = global_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > limit_ns) return false;
        }
    }
}

// ---- push pipeline of a pusher CTA ---------------------------------------------------------------------------------
// One thread moves pieces of local global memory to a (peer or local) destination through a ring of shared-memory
// stages with bulk asynchronous copies: global -> shared completes on an mbarrier, shared -> global is tracked in bulk
// groups.  Up to PUSH_AHEAD loads and PUSH_PENDING + 1 stores are in flight at a time; a piece's counter on the
// destination is bumped only after its store has completed (full wait_group, proxy fence, system fence).
// Epilogue staging of the GEMM -> reduce-scatter kernel: every thread packs up to OUT_CHUNK columns of its row into shared
// memory and sends them with one bulk copy (256-byte writes keep NVLink packets full; 16-byte scattered stores do not).
// The 16 bytes of padding per row spread the rows of a warp over all banks.
constexpr int OUT_CHUNK = 128, OUT_PITCH = OUT_CHUNK * 2 + 16;
constexpr int PUSH_STAGES = 6, PUSH_AHEAD = 3, PUSH_PENDING = 3;
constexpr uint32_t PUSH_PIECE_BYTES = 32768;

struct PushMeta {
    char* dst[PUSH_STAGES];
    unsigned int* cnt[PUSH_STAGES];
    uint32_t bytes[PUSH_STAGES];
};

struct PushPipe {
    uint32_t buf0, bar0;     // shared addresses: first stage, first mbarrier (8 bytes apart)
    PushMeta* meta;          // in shared memory
    int64_t n_loaded, n_stored, n_sig;

    __device__ __forceinline__ void init(uint32_t buf, uint32_t bar, PushMeta* m) {
        buf0 = buf; bar0 = bar; meta = m; n_loaded = n_stored = n_sig = 0;
    }
    __device__ __forceinline__ void retire(int64_t upto) {
        bool fenced = false;
        for (; n_sig < upto; ++n_sig) {
            unsigned int* c = meta->cnt[n_sig % PUSH_STAGES];
            if (!c) continue;
            if (!fenced) {
                asm volatile("fence.proxy.async.global;" ::: "memory");  // the stores went through the async proxy
                __threadfence_system();
                fenced = true;
            }
            atomicAdd_system(c, 1u);
        }
    }
    // Issue the store of the oldest loaded piece (if any) and retire stores beyond the pending limit.
    __device__ __forceinline__ bool advance() {
        if (n_stored < n_loaded) {
            const int s = (int)(n_stored % PUSH_STAGES);
            if (!mbar_wait_u32(bar0 + 8 * s, (uint32_t)((n_stored / PUSH_STAGES) & 1))) return false;
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                         ::"l"(meta->dst[s]), "r"(buf0 + s * PUSH_PIECE_BYTES), "r"(meta->bytes[s]) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            ++n_stored;
        }
        if (n_stored - n_sig > PUSH_PENDING) {
            asm volatile("cp.async.bulk.wait_group %0;" ::"n"(PUSH_PENDING) : "memory");
            retire(n_stored - PUSH_PENDING);
        }
        return true;
    }
    // Queue one piece: bytes is a multiple of 16 and at most PUSH_PIECE_BYTES, both addresses are 16-byte aligned.
    __device__ __forceinline__ bool submit(const char* src, char* dst, unsigned int* cnt, uint32_t bytes) {
        while (n_loaded - n_sig >= PUSH_STAGES || n_loaded - n_stored >= PUSH_AHEAD) {
            if (!advance()) return false;
        }
        const int s = (int)(n_loaded % PUSH_STAGES);
        meta->dst[s] = dst; meta->cnt[s] = cnt; meta->bytes[s] = bytes;
        mbar_expect_tx_u32(bar0 + 8 * s, bytes);
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(buf0 + s * PUSH_PIECE_BYTES), "l"(src), "r"(bytes), "r"(bar0 + 8 * s) : "memory");
        ++n_loaded;
        return true;
    }
    // Store what is loaded, wait for every store, signal the rest.  On a failed load wait the stores already issued are
    // still waited for (they read this CTA's shared memory).
    __device__ __forceinline__ bool drain() {
        bool ok = true;
        while (ok && n_stored < n_loaded) ok = advance();
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
        retire(n_stored);
        return ok;
    }
};

template <bool CTA2, int FUSED>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, const GemmParams p,
                    const FusedComm f) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // tiles first (1024-byte aligned for the 128-byte swizzle), bookkeeping after them
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    constexpr int NCTA = CTA2 ? 2 : 1;
    const uint32_t rank = CTA2 ? cluster_ctarank() : 0u;          // position inside the CTA pair
    const uint32_t bn_local = (uint32_t)p.bn / NCTA;               // rows of the B tile this CTA loads
    const uint32_t a_bytes = BM * BK * 2;
    const uint32_t b_bytes = bn_local * BK * 2;
    const uint32_t stage_bytes = a_bytes + b_bytes;
    SharedHeader* hdr = (SharedHeader*)(smem + p.hdr_off);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = (int)((p.K + BK - 1) / BK);
    const int64_t tiles_per_batch = (int64_t)p.m_blocks * p.n_blocks;   // m_blocks counts (BM * NCTA)-row tiles
    const int64_t num_tiles = tiles_per_batch * p.batch_inner * p.batch_outer;
    // The pusher CTAs are the first CTAs of the grid: CTAs are handed to SMs in index order, so when another kernel keeps
    // part of the GPU busy it is compute CTAs that wait for an SM, never the CTAs the other ranks depend on.
    const int comm_first = (FUSED == 2 || FUSED == 3) ? f.ag_ctas : 0;
    const int compute_ctas = (int)gridDim.x - comm_first;
    const bool comm_cta = (int)blockIdx.x < comm_first;
    const int64_t first_tile = comm_cta ? num_tiles : ((int)blockIdx.x - comm_first) / NCTA, tile_step = compute_ctas / NCTA;
    const int blocks_per_rank = FUSED == 2 ? (int)(f.ag_rows / (BM * NCTA)) : 0;   // in tile rows (256 rows for a CTA pair)
    const int row_blocks_per_rank = FUSED == 2 ? (int)(f.ag_rows / BM) : 1;          // in 128-row blocks (counter granularity)
    const uint32_t tmem_cols = 2 * p.bn <= 32 ? 32 : 2 * p.bn <= 64 ? 64 : 2 * p.bn <= 128 ? 128 : 2 * p.bn <= 256 ? 256 : 512;

    if (threadIdx.x == 0) {
        for (int s = 0; s < MAX_STAGES; ++s) { mbar_init(&hdr->full[s], 1); mbar_init(&hdr->empty[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&hdr->tmem_full[a], 1); mbar_init(&hdr->tmem_empty[a], 4 * NCTA); }
        hdr->failed = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        if (CTA2) { tmem_alloc_2cta(&hdr->tmem_base, tmem_cols); tmem_relinquish_2cta(); }
        else { tmem_alloc(&hdr->tmem_base, tmem_cols); tmem_relinquish(); }
    }
    tc_fence_before();
    __syncthreads();
    if (CTA2) cluster_sync();   // the peer's barriers must be initialised before anything is signalled across
    tc_fence_after();
    const uint32_t tmem_base = hdr->tmem_base;

    const uint64_t t_kernel0 = (FUSED != 0 && threadIdx.x == 0) ? global_ns() : 0;
    if (FUSED != 0 && blockIdx.x == 0 && threadIdx.x == 0) atomicAdd(&g_fused_stats[4], 1ull);
    if (FUSED != 0 && blockIdx.x == 0 && threadIdx.x < (unsigned)f.world) {
        // everything this rank did earlier on the stream is complete: peers may write into its buffers for this epoch
        st_release_sys_u32(f.flags[threadIdx.x] + f.free_row * f.world + f.rank, f.epoch);
    }

    if (comm_cta && threadIdx.x == 0) {
        // ------------------------------------------------------------------ pusher (one thread drives bulk copies)
        __shared__ PushMeta push_meta;
        PushPipe pipe;
        pipe.init(smem_u32(smem), smem_u32(&hdr->full[0]), &push_meta);
        const int n_pushers = f.ag_ctas, me = (int)blockIdx.x;
        bool ok = true;
        unsigned int free_seen = 1u << f.rank;   // destinations whose "free for this epoch" flag has been observed
        auto dst_free = [&](int dst) -> bool {
            if (free_seen & (1u << dst)) return true;
            if (!wait_counter(f.flags[f.rank] + f.free_row * f.world + dst, f.epoch, f.limit_ns)) {
                atomicCAS(f.status, 0, (FUSED == 3 ? 0x800 : 0x300) | f.rank);
                atomicCAS(&g_gemm_status, 0, ((FUSED == 3 ? 9 : 5) << 16) | (blockIdx.x & 0xffff));
                return false;
            }
            free_seen |= 1u << dst;
            return true;
        };
        if (FUSED == 3) {
            // weight pusher: this rank's flat element range, cut at 128-row chunk boundaries, to every rank (own first)
            const int64_t CK = (int64_t)BM * p.K;                       // elements per 128-row chunk
            const int64_t lo_all = f.bg_first, hi_all = f.bg_first + f.bg_count;
            for (int di = f.skip_local ? 1 : 0; di < f.world && ok && f.bg_count > 0; ++di) {
                // own copy first, then rank-1, rank-2, ...: a rank multiplies its own rows first and continues with the
                // rows of rank+1, rank+2, ..., so it should receive from those sources in that order
                const int dst = (f.rank - di + f.world) % f.world;
                int64_t g = 0;   // running index of runs
                for (int64_t c = lo_all / CK; c * CK < hi_all && ok; ++c) {
                    const int64_t lo = lo_all > c * CK ? lo_all : c * CK;
                    const int64_t hi = hi_all < (c + 1) * CK ? hi_all : (c + 1) * CK;
                    const int64_t np = (hi - lo + BG_PIECE - 1) / BG_PIECE;           // pieces of this rank in the chunk
                    const int64_t per_run = (np + f.bg_split - 1) / f.bg_split;       // pieces per run
                    for (int64_t r0 = 0; r0 < np && ok; r0 += per_run, ++g) {
                        if (g % n_pushers != me) continue;
                        if (!dst_free(dst)) { ok = false; break; }
                        const int64_t r1 = r0 + per_run < np ? r0 + per_run : np;
                        for (int64_t pi = r0; pi < r1 && ok; ++pi) {
                            const int64_t e0 = lo + pi * BG_PIECE;
                            const uint32_t bytes = (uint32_t)((hi - e0 < BG_PIECE ? hi - e0 : BG_PIECE) * 2);
                            // only the last piece of a run carries the counter: no fence between the pieces of a run
                            ok = pipe.submit(f.bg_src + (e0 - lo_all) * 2, (char*)f.bg_dst[dst] + e0 * 2,
                                             pi + 1 == r1 ? f.bg_cnt[dst] + c : nullptr, bytes);
                        }
                    }
                }
            }
        } else {
            // all-gather pusher: this rank's rows (contiguous) to every rank's gathered matrix, destination-major
            // starting with this rank itself, then rank-1, rank-2, ... (the order in which the consumers get to them)
            const int64_t block_bytes = (int64_t)BM * p.K * 2;
            const int64_t rpb = f.ag_runs_per_block, per_run = f.ag_pieces_per_block / rpb;
            const int64_t per_dst = (int64_t)row_blocks_per_rank * rpb;
            const int skip = f.skip_local ? 1 : 0;
            const int64_t total_runs = (int64_t)(f.world - skip) * per_dst;
            for (int64_t g = me; g < total_runs && ok; g += n_pushers) {
                const int dst = (f.rank - skip - (int)(g / per_dst) + 2 * f.world) % f.world;
                const int64_t rem = g % per_dst;
                const int64_t blk = rem / rpb, run = rem % rpb;
                if (!dst_free(dst)) { ok = false; break; }
                unsigned int* cnt = f.ag_count[dst] + (f.rank * row_blocks_per_rank + blk);
                char* dbase = (char*)f.ag_dst[dst] + (int64_t)f.rank * f.ag_rows * p.K * 2;
                for (int64_t pi = run * per_run; pi < (run + 1) * per_run && ok; ++pi) {
                    const int64_t off = blk * block_bytes + pi * (int64_t)f.ag_piece_bytes;
                    // only the last piece of a run carries the counter: no fence between the pieces of a run
                    ok = pipe.submit((const char*)f.ag_src + off, dbase + off, pi + 1 == (run + 1) * per_run ? cnt : nullptr,
                                     (uint32_t)f.ag_piece_bytes);
                }
            }
        }
        if (!pipe.drain()) ok = false;
        if (!ok) {
            hdr->failed = 1;
            atomicCAS(&g_gemm_status, 0, (11 << 16) | (blockIdx.x & 0xffff));
        }
        atomicMax(&g_fused_stats[1], (unsigned long long)(global_ns() - t_kernel0));
    } else if (comm_cta) {
        // the other threads of a pusher CTA have nothing to do
    } else if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (one per CTA)
        if (lane == 0) {
            bool ok = true;
            uint64_t waited = 0;        // time spent waiting for data of other ranks (fused modes)
            uint32_t ps = 0, pph = 0;   // ring position and phase, carried across tiles
            const uint32_t smem0 = smem_u32(smem), full0 = smem_u32(&hdr->full[0]), empty0 = smem_u32(&hdr->empty[0]);
            const uint32_t full_leader0 = CTA2 ? map_to_cta(full0, 0) : full0;
            for (int64_t tile = first_tile; tile < num_tiles && ok; tile += tile_step) {
                const int64_t batch = tile / tiles_per_batch;
                const int64_t rem = tile % tiles_per_batch;
                int m_blk, n_blk;
                tile_coords(p, rem, m_blk, n_blk);
                if (FUSED == 1 && f.rs_early) m_blk = (m_blk + (f.rank + 1) * f.rs_bpr) % p.m_blocks;   // own rows last
                if (FUSED == 3) {
                    // this rank's own rows first; wait for every 128-row chunk the B tile touches
                    n_blk = (n_blk + f.bg_first_block) % p.n_blocks;
                    const int64_t r0 = (int64_t)n_blk * p.bn;
                    const int64_t r1 = (r0 + p.bn < p.N ? r0 + p.bn : p.N) - 1;
                    const uint64_t tw0 = global_ns();
                    for (int64_t c = r0 / BM; c <= r1 / BM && ok; ++c) {
                        const unsigned int target = f.epoch * f.bg_expected[c];
                        if (!wait_counter(f.bg_cnt[f.rank] + c, target, f.limit_ns)) {
                            ok = false; atomicCAS(f.status, 0, 0x900 | f.rank); atomicCAS(&g_gemm_status, 0, (10 << 16) | (blockIdx.x & 0xffff)); hdr->failed = 1;
                        }
                    }
                    if (!ok) break;
                    waited += global_ns() - tw0;
                    asm volatile("fence.proxy.async.global;" ::: "memory");
                }
                if (FUSED == 2) {
                    // local row blocks first, then the peers' blocks in the order in which they are pushed
                    m_blk = (m_blk + f.rank * blocks_per_rank) % p.m_blocks;
                    const unsigned int target = f.epoch * (unsigned int)f.ag_runs_per_block;
                    const int row_block = m_blk * NCTA + (int)rank;
                    const bool mine = f.skip_local && row_block / row_blocks_per_rank == f.rank;   // copied before the launch
                    const uint64_t tw0 = global_ns();
                    if (!mine && !wait_counter(f.ag_count[f.rank] + row_block, target, f.limit_ns)) {
                        ok = false; atomicCAS(f.status, 0, 0x400 | f.rank); atomicCAS(&g_gemm_status, 0, (6 << 16) | (blockIdx.x & 0xffff)); hdr->failed = 1; break;
                    }
                    waited += global_ns() - tw0;
                    asm volatile("fence.proxy.async.global;" ::: "memory");  // the block was written by a peer's copies, TMA reads it
                }
                const int bi = (int)(batch % p.batch_inner), bo = (int)(batch / p.batch_inner);
                const int bib = (int)(bi / p.b_inner_div);
                const int m0 = m_blk * (BM * NCTA) + (int)rank * BM;            // this CTA's rows of A
                const int n0 = n_blk * p.bn + (int)(rank * bn_local);           // this CTA's rows of the B tile
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait_u32(empty0 + 8 * ps, pph ^ 1)) { ok = false; atomicCAS(&g_gemm_status, 0, (1 << 16) | (blockIdx.x & 0xffff)); hdr->failed = 1; break; }
                    const uint32_t sa = smem0 + ps * stage_bytes, sb = sa + a_bytes;
                    const int kx = kb * BK;
                    if (p.debug & 1) {
                        if (rank == 0) mbar_arrive_u32(full0 + 8 * ps);
                    } else if (!CTA2) {
                        const uint32_t bar = full0 + 8 * ps;
                        mbar_expect_tx_u32(bar, stage_bytes);
                        if (!p.a_mn) {
                            tma_load_4d_u32(&tma_a, bar, sa, kx, m0, bi, bo);
                        } else if (p.a_mn5) {
                            tma_load_5d_u32(&tma_a, bar, sa, 0, kx, m0 / 64, bi, bo);
                        } else {
#pragma unroll
                            for (int c = 0; c < BM / 64; ++c) tma_load_4d_u32(&tma_a, bar, sa + c * (64 * BK * 2), m0 + c * 64, kx, bi, bo);
                        }
                        if (!p.b_mn) {
                            tma_load_4d_u32(&tma_b, bar, sb, kx, n0, bib, bo);
                        } else if (p.b_mn5) {
                            tma_load_5d_u32(&tma_b, bar, sb, 0, kx, n0 / 64, bib, bo);
                        } else {
                            for (int c = 0; c < (int)bn_local / 64; ++c) tma_load_4d_u32(&tma_b, bar, sb + c * (64 * BK * 2), n0 + c * 64, kx, bib, bo);
                        }
                    } else {
                        // both CTAs report to the leader's barrier; the leader announces the bytes of the pair
                        const uint32_t bar = full_leader0 + 8 * ps;
                        if (rank == 0) mbar_expect_tx_u32(full0 + 8 * ps, 2 * stage_bytes);
                        if (!p.a_mn) {
                            tma_load_4d_2cta_u32(&tma_a, bar, sa, kx, m0, bi, bo);
                        } else if (p.a_mn5) {
                            tma_load_5d_2cta_u32(&tma_a, bar, sa, 0, kx, m0 / 64, bi, bo);
                        } else {
#pragma unroll
                            for (int c = 0; c < BM / 64; ++c) tma_load_4d_2cta_u32(&tma_a, bar, sa + c * (64 * BK * 2), m0 + c * 64, kx, bi, bo);
                        }
                        if (!p.b_mn) {
                            tma_load_4d_2cta_u32(&tma_b, bar, sb, kx, n0, bib, bo);
                        } else if (p.b_mn5) {
                            tma_load_5d_2cta_u32(&tma_b, bar, sb, 0, kx, n0 / 64, bib, bo);
                        } else {
                            for (int c = 0; c < (int)bn_local / 64; ++c) tma_load_4d_2cta_u32(&tma_b, bar, sb + c * (64 * BK * 2), n0 + c * 64, kx, bib, bo);
                        }
                    }
                    if (++ps == (uint32_t)p.stages) { ps = 0; pph ^= 1; }
                }
            }
            if (FUSED == 2 || FUSED == 3) {
                atomicAdd(&g_fused_stats[0], (unsigned long long)waited);
                atomicMax(&g_fused_stats[3], (unsigned long long)waited);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (leader CTA only in pair mode)
        if (lane == 0 && rank == 0) {
            uint32_t tcount = 0;
            bool ok = true;
            uint32_t cs = 0, cph = 0;
            const uint32_t smem0 = smem_u32(smem), full0 = smem_u32(&hdr->full[0]), empty0 = smem_u32(&hdr->empty[0]);
            // descriptor halves that never change; per MMA only the start address moves: K-major steps 32 bytes inside
            // the 128-byte swizzle row, MN-major steps 16 K rows (2 KiB)
            const uint32_t a_hi = desc_hi(1024), b_hi = desc_hi(1024);
            const uint32_t a_lbo = p.a_mn ? 64 * BK * 2 : 0, b_lbo = p.b_mn ? 64 * BK * 2 : 0;
            const uint32_t a_kstep = (p.a_mn ? UMMA_K * 128 : UMMA_K * 2) >> 4, b_kstep = (p.b_mn ? UMMA_K * 128 : UMMA_K * 2) >> 4;
            for (int64_t tile = first_tile; tile < num_tiles && ok; tile += tile_step, ++tcount) {
                const uint32_t acc = tcount & 1;
                const uint32_t acc_ph = (tcount >> 1) & 1;
                if (!mbar_wait(&hdr->tmem_empty[acc], acc_ph ^ 1)) { ok = false; atomicCAS(&g_gemm_status, 0, (2 << 16) | (blockIdx.x & 0xffff)); hdr->failed = 1; break; }
                tc_fence_after();
                const uint32_t tmem_c = tmem_base + acc * p.bn;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait_u32(full0 + 8 * cs, cph)) { ok = false; atomicCAS(&g_gemm_status, 0, (3 << 16) | (blockIdx.x & 0xffff)); hdr->failed = 1; break; }
                    tc_fence_after();
                    const uint32_t sa = smem0 + cs * stage_bytes;
                    const uint32_t a_lo = desc_lo(sa, a_lbo), b_lo = desc_lo(sa + a_bytes, b_lbo);
                    if (!(p.debug & 2)) {
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k) {
                            const uint64_t ad = pack_desc(a_lo + k * a_kstep, a_hi), bd = pack_desc(b_lo + k * b_kstep, b_hi);
                            if (CTA2) umma_f16_2cta(tmem_c, ad, bd, p.idesc, (kb | k) != 0 ? 1u : 0u);
                            else umma_f16(tmem_c, ad, bd, p.idesc, (kb | k) != 0 ? 1u : 0u);
                        }
                    }
                    // frees the smem stage (in both CTAs) once these MMAs have read it
                    if (CTA2) umma_commit_2cta_u32(empty0 + 8 * cs); else umma_commit_u32(empty0 + 8 * cs);
                    if (++cs == (uint32_t)p.stages) { cs = 0; cph ^= 1; }
                }
                if (ok) { if (CTA2) umma_commit_2cta(&hdr->tmem_full[acc]); else umma_commit(&hdr->tmem_full[acc]); }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5), own 128 rows
        const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter + 32) are visible to this warp
        uint32_t tcount = 0;
        uint32_t rs_free_mask = 0;     // destinations whose inbox is known to be free (mode 1)
        bool ok = true;
        bool remote_open = FUSED == 1 && f.rs_early;   // this warp has not yet reported its other-rank tiles as delivered
        auto report_remote_done = [&]() {
            // the warp's stores into other ranks' inboxes are all issued: make them visible and count the warp; the last
            // warp of the rank publishes "delivered" to every rank while the tiles with own rows are still being computed
            asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // this thread's row copies have completed
            asm volatile("fence.proxy.async.global;" ::: "memory");
            __threadfence_system();
            __syncwarp();
            if (lane == 0) {
                __threadfence_system();
                const unsigned int done = atomicAdd(f.rs_counter, 1u) + 1u;
                if (done == f.epoch * gridDim.x * 4u) {
                    __threadfence_system();
                    for (int j = 0; j < f.world; ++j) st_release_sys_u32(f.flags[j] + f.done_row * f.world + f.rank, f.epoch);
                }
            }
            remote_open = false;
        };
        for (int64_t tile = first_tile; tile < num_tiles && ok; tile += tile_step, ++tcount) {
            const int64_t batch = tile / tiles_per_batch;
            const int64_t rem = tile % tiles_per_batch;
            int m_blk, n_blk;
            tile_coords(p, rem, m_blk, n_blk);
            if (FUSED == 1 && f.rs_early) {
                if (remote_open && rem >= f.rs_remote_tiles) report_remote_done();
                m_blk = (m_blk + (f.rank + 1) * f.rs_bpr) % p.m_blocks;   // own rows last
            }
            if (FUSED == 2) m_blk = (m_blk + f.rank * blocks_per_rank) % p.m_blocks;
            if (FUSED == 3) n_blk = (n_blk + f.bg_first_block) % p.n_blocks;
            const int64_t bi = batch % p.batch_inner, bo = batch / p.batch_inner;
            const uint32_t acc = tcount & 1;
            const uint32_t acc_ph = (tcount >> 1) & 1;
            // one lane per warp polls the barrier (128 pollers would compete with the producer / MMA threads for the
            // barrier unit during the whole main loop); the warp then re-converges
            int got = 1;
            if (lane == 0) got = mbar_wait(&hdr->tmem_full[acc], acc_ph) ? 1 : 0;
            got = __shfl_sync(0xffffffffu, got, 0);
            if (!got) { ok = false; if (lane == 0) atomicCAS(&g_gemm_status, 0, (4 << 16) | (blockIdx.x & 0xffff)); break; }
            tc_fence_after();
            const int64_t row = (int64_t)m_blk * (BM * NCTA) + rank * BM + quarter * 32 + lane;
            const bool row_ok = row < p.M;
            int64_t coff = bi * p.c_bs0 + bo * p.c_bs1 + row * p.ldc;
            char* cbase = (char*)p.c;
            if (FUSED == 1 && row_ok) {
                // route the row to the inbox of its owner; wait once per destination until that rank freed the inbox
                const int owner = (int)(row / f.rs_rows);
                if (owner != f.rank && !((rs_free_mask >> owner) & 1u)) {
                    if (!wait_counter(f.flags[f.rank] + f.free_row * f.world + owner, f.epoch, f.limit_ns)) {
                        atomicCAS(f.status, 0, 0x500 | f.rank); atomicCAS(&g_gemm_status, 0, (7 << 16) | (blockIdx.x & 0xffff));
                    }
                    rs_free_mask |= 1u << owner;
                }
                cbase = (char*)f.rs_inbox[owner];
                coff = (row - (int64_t)owner * f.rs_rows) * p.N;
            }
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * p.bn;
            const int64_t tile_end = (int64_t)(n_blk + 1) * p.bn;
            const int64_t col_end = tile_end < p.N ? tile_end : p.N;
            if (FUSED == 1 || p.staged) {
                // staged bulk-store epilogue: pack OUT_CHUNK columns of the row in shared memory, one bulk copy per row chunk
                // (to the row's owner in the GEMM -> reduce-scatter kernel)
                const uint32_t srow = smem_u32(smem) + p.out_stage_off + (uint32_t)((quarter * 32 + lane) * OUT_PITCH);
                for (int c0 = 0; c0 < p.bn; c0 += OUT_CHUNK) {
                    const int64_t col0 = (int64_t)n_blk * p.bn + c0;
                    if (col0 >= col_end) break;
                    const int ncols = (int)(col_end - col0 < OUT_CHUNK ? col_end - col0 : OUT_CHUNK);
                    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the previous copy has read the row buffer
                    for (int sub = 0; sub < OUT_CHUNK; sub += 32) {
                        if (c0 + sub >= p.bn || col0 + sub >= col_end) break;
                        uint32_t r[32];
                        tmem_ld32(taddr + c0 + sub, r);
                        tmem_ld_wait();
                        float vals[32];
                        if (FUSED == 1) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) vals[i] = __uint_as_float(r[i]) * p.alpha;
                        } else if (row_ok) {
                            if (p.c_dtype == BMT_DT_F16) epilogue_math<__half>(p, (const __half*)cbase + coff, row, col0 + sub, col_end, r, vals);
                            else epilogue_math<__nv_bfloat16>(p, (const __nv_bfloat16*)cbase + coff, row, col0 + sub, col_end, r, vals);
                        }
                        uint32_t pk[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const float a = vals[2 * i], b = vals[2 * i + 1];
                            if (p.c_dtype == BMT_DT_F16) { __half2 h = __floats2half2_rn(a, b); pk[i] = *reinterpret_cast<uint32_t*>(&h); }
                            else { __nv_bfloat162 h = __floats2bfloat162_rn(a, b); pk[i] = *reinterpret_cast<uint32_t*>(&h); }
                        }
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(srow + sub * 2 + q * 16), "r"(pk[4 * q]),
                                         "r"(pk[4 * q + 1]), "r"(pk[4 * q + 2]), "r"(pk[4 * q + 3]) : "memory");
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    if (row_ok && !(p.debug & 4))
                        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                                     ::"l"(cbase + (coff + col0) * 2), "r"(srow), "r"(ncols * 2) : "memory");
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
            } else
            for (int c0 = 0; c0 < p.bn; c0 += 32) {
                const int64_t col0 = (int64_t)n_blk * p.bn + c0;
                if (col0 >= col_end) break;
                uint32_t r[32];
                tmem_ld32(taddr + c0, r);
                tmem_ld_wait();
                if (p.debug & 4) continue;
                if (p.c_dtype == BMT_DT_F16) epilogue_chunk<__half>(p, (__half*)cbase + coff, row, col0, col_end, r, row_ok);
                else if (p.c_dtype == BMT_DT_BF16) epilogue_chunk<__nv_bfloat16>(p, (__nv_bfloat16*)cbase + coff, row, col0, col_end, r, row_ok);
                else epilogue_chunk<float>(p, (float*)cbase + coff, row, col0, col_end, r, row_ok);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (CTA2) mbar_arrive_cluster(map_to_cta(smem_u32(&hdr->tmem_empty[acc]), 0));
                else mbar_arrive(&hdr->tmem_empty[acc]);
            }
        }
        if (remote_open) report_remote_done();
        if (FUSED == 1 || p.staged) {
            // row copies read this CTA's shared memory and write the inboxes: complete them before the teardown barrier
            asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
            asm volatile("fence.proxy.async.global;" ::: "memory");
            __threadfence_system();
        }
    }

    // ---------------------------------------------------------------------- teardown
    __syncthreads();
    if (FUSED != 0 && threadIdx.x == 0) atomicMax(&g_fused_stats[2], (unsigned long long)(global_ns() - t_kernel0));
    if (hdr->failed) {
        // a wait ran out: give copies that are still in flight time to land before the CTA's shared memory goes away
        const uint64_t t0 = global_ns();
        while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
        __syncthreads();
    }
    if (CTA2) cluster_sync();   // the peer may still be signalling barriers in this CTA's shared memory
    tc_fence_after();
    if (warp == 1) { if (CTA2) tmem_dealloc_2cta(tmem_base, tmem_cols); else tmem_dealloc(tmem_base, tmem_cols); }

    if (FUSED == 1) {
        // ---- reduce phase of GEMM -> reduce-scatter
        __shared__ int rs_ok;
        if (threadIdx.x == 0) {
            bool ok = true;
            if (!f.rs_early) {
                __threadfence_system();  // this CTA's inbox stores (ordered before by the barrier above) become visible system-wide
                const unsigned int done = atomicAdd(f.rs_counter, 1u) + 1u;
                if (done == f.epoch * gridDim.x) {
                    // last CTA of this rank: everything is delivered
                    __threadfence_system();
                    for (int j = 0; j < f.world; ++j) st_release_sys_u32(f.flags[j] + f.done_row * f.world + f.rank, f.epoch);
                }
            } else if (!f.rs_split) {
                // "delivered" went out when the other ranks' tiles were done; the tiles with own rows only have to be complete
                // on this GPU: count the CTA and wait (bounded) for the rest of the grid, all of which is resident
                __threadfence();
                atomicAdd(f.rs_counter + 1, 1u);
                ok = wait_counter(f.rs_counter + 1, f.epoch * gridDim.x, f.limit_ns);
            }
            if (!f.rs_split) {
                const uint64_t tw0 = global_ns();
                for (int j = 0; j < f.world && ok; ++j) ok = wait_counter(f.flags[f.rank] + f.done_row * f.world + j, f.epoch, f.limit_ns);
                atomicMax(&g_fused_stats[5], (unsigned long long)(global_ns() - tw0));
                atomicAdd(&g_fused_stats[7], (unsigned long long)(global_ns() - tw0));
                if (!ok) { atomicCAS(f.status, 0, 0x600 | f.rank); atomicCAS(&g_gemm_status, 0, (8 << 16) | (blockIdx.x & 0xffff)); }
            }
            rs_ok = (ok && !f.rs_split) ? 1 : 0;
        }
        __syncthreads();
        if (rs_ok) {
            const int64_t nvec = f.rs_rows * p.N / 8;
            const int64_t slot_elems = f.rs_rows * p.N;
            if (p.c_dtype == BMT_DT_F16) rs_reduce_all<__half>(f.rs_inbox_local, slot_elems, f.world, f.rs_bias, p.N, f.rs_out, nvec);
            else rs_reduce_all<__nv_bfloat16>(f.rs_inbox_local, slot_elems, f.world, f.rs_bias, p.N, f.rs_out, nvec);
            if (threadIdx.x == 0) atomicMax(&g_fused_stats[6], (unsigned long long)(global_ns() - t_kernel0));
        }
    }
}

// Second half of a split GEMM -> reduce-scatter: sums the inbox slots (+ bias) of this rank's rows once every rank's
// "delivered" flag has been seen by the wait kernel launched before it.  The last CTA tells every rank that this
// rank's inbox may be overwritten by the next use of the ring slot.
template <typename T>
__global__ void __launch_bounds__(NUM_THREADS) rs_reduce_kernel(const void* inbox, int64_t slot_elems, int world, const void* bias, int64_t N,
                                                                 void* out, int64_t nvec, FusedComm f, unsigned int next_epoch) {
    rs_reduce_all<T>(inbox, slot_elems, world, bias, N, out, nvec);
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned int done = atomicAdd(f.rs_counter + 1, 1u) + 1u;
        if (done == f.epoch * gridDim.x) {
            for (int j = 0; j < f.world; ++j) st_release_sys_u32(f.flags[j] + f.free_row * f.world + f.rank, next_epoch);
        }
    }
}

// ------------------------------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

struct MapKey {
    const void* ptr;
    int64_t d[4], s[3];
    int box0, box1, dtype;
    int chunks;   // 0: 4-D map; > 0: 5-D map of an MN-major operand with this many 64-element chunks per box
    bool operator==(const MapKey& o) const { return memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        const uint64_t* w = (const uint64_t*)&k;
        size_t h = 1469598103934665603ull;
        for (size_t i = 0; i < sizeof(MapKey) / 8; ++i) h = (h ^ w[i]) * 1099511628211ull;
        return h;
    }
};
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;
std::mutex g_maps_mu;

// 4-D map: dims {inner, rows, batch_inner, batch_outer}; element strides for dims 1..3.
int make_map(CUtensorMap* out, const void* ptr, int dtype, int64_t inner, int64_t rows, int64_t ld, int64_t nb0, int64_t bs0,
             int64_t nb1, int64_t bs1, int box_inner, int box_rows) {
    MapKey key;
    memset(&key, 0, sizeof(key));
    key.ptr = ptr; key.d[0] = inner; key.d[1] = rows; key.d[2] = nb0; key.d[3] = nb1;
    key.s[0] = ld; key.s[1] = bs0; key.s[2] = bs1; key.box0 = box_inner; key.box1 = box_rows; key.dtype = dtype;
    {
        std::lock_guard<std::mutex> lk(g_maps_mu);
        auto it = g_maps.find(key);
        if (it != g_maps.end()) { *out = it->second; return 0; }
    }
    EncodeTiledFn enc = get_encode();
    if (!enc) return -10;
    if (((uintptr_t)ptr & 15) || (ld & 7) || (nb0 > 1 && (bs0 & 7)) || (nb1 > 1 && (bs1 & 7))) return -11;
    cuuint64_t dims[4] = {(cuuint64_t)inner, (cuuint64_t)rows, (cuuint64_t)nb0, (cuuint64_t)nb1};
    // strides of unit-extent dims are irrelevant but must still be legal (multiple of 16 bytes, non-zero)
    cuuint64_t st[3] = {(cuuint64_t)ld * 2, (cuuint64_t)(nb0 > 1 ? bs0 : ld * rows) * 2, (cuuint64_t)(nb1 > 1 ? bs1 : ld * rows) * 2};
    if (st[1] == 0) st[1] = 16;
    if (st[2] == 0) st[2] = 16;
    cuuint32_t box[4] = {(cuuint32_t)box_inner, (cuuint32_t)box_rows, 1, 1};
    cuuint32_t es[4] = {1, 1, 1, 1};
    cudaFree(0);  // binds the primary context to this thread (autograd worker threads may not have one current yet)
    CUresult r = enc(out, dtype == BMT_DT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, (void*)ptr,
                     dims, st, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        fprintf(stderr, "bmtrain_b200: cuTensorMapEncodeTiled failed (%d): ptr=%p dims={%lld,%lld,%lld,%lld} strides={%lld,%lld,%lld} box={%d,%d}\n",
                (int)r, ptr, (long long)dims[0], (long long)dims[1], (long long)dims[2], (long long)dims[3], (long long)st[0],
                (long long)st[1], (long long)st[2], box_inner, box_rows);
        return -12;
    }
    std::lock_guard<std::mutex> lk(g_maps_mu);
    if (g_maps.size() > 8192) g_maps.clear();
    g_maps[key] = *out;
    return 0;
}

}  // namespace

// Cached 4-D tensor map {inner, rows, batch_inner, batch_outer} for the other tensor-core kernels of this library.
int bmt_tma_map_4d(CUtensorMap* out, const void* ptr, int dtype, int64_t inner, int64_t rows, int64_t ld, int64_t nb0, int64_t bs0,
                   int64_t nb1, int64_t bs1, int box_inner, int box_rows) {
    return make_map(out, ptr, dtype, inner, rows, ld, nb0, bs0, nb1, bs1, box_inner, box_rows);
}

namespace {

// 5-D map of an MN-major operand (element (k, mn) at ptr + k * ld + mn, mn contiguous): dims {64, k rows, mn / 64 chunks,
// batch_inner, batch_outer}; the chunk dimension has a stride of 64 elements, so one box {64, box_rows, chunks} lands in
// shared memory as `chunks` consecutive [box_rows][64] swizzled blocks -- the layout one copy per chunk produces, with one
// copy.  Only for mn extents that are multiples of 64 (the inner dimension is the fixed 64 of a chunk, so a ragged last
// chunk could not be bounds-checked by the copy engine).
int make_map_mn5(CUtensorMap* out, const void* ptr, int dtype, int64_t mn, int64_t rows, int64_t ld, int64_t nb0, int64_t bs0,
                 int64_t nb1, int64_t bs1, int box_rows, int chunks) {
    if (mn % 64 != 0) return -13;
    MapKey key;
    memset(&key, 0, sizeof(key));
    key.ptr = ptr; key.d[0] = mn; key.d[1] = rows; key.d[2] = nb0; key.d[3] = nb1;
    key.s[0] = ld; key.s[1] = bs0; key.s[2] = bs1; key.box0 = 64; key.box1 = box_rows; key.dtype = dtype; key.chunks = chunks;
    {
        std::lock_guard<std::mutex> lk(g_maps_mu);
        auto it = g_maps.find(key);
        if (it != g_maps.end()) { *out = it->second; return 0; }
    }
    EncodeTiledFn enc = get_encode();
    if (!enc) return -10;
    if (((uintptr_t)ptr & 15) || (ld & 7) || (nb0 > 1 && (bs0 & 7)) || (nb1 > 1 && (bs1 & 7))) return -11;
    cuuint64_t dims[5] = {64, (cuuint64_t)rows, (cuuint64_t)(mn / 64), (cuuint64_t)nb0, (cuuint64_t)nb1};
    cuuint64_t st[4] = {(cuuint64_t)ld * 2, 128, (cuuint64_t)(nb0 > 1 ? bs0 : ld * rows) * 2, (cuuint64_t)(nb1 > 1 ? bs1 : ld * rows) * 2};
    if (st[2] == 0) st[2] = 16;
    if (st[3] == 0) st[3] = 16;
    cuuint32_t box[5] = {64, (cuuint32_t)box_rows, (cuuint32_t)chunks, 1, 1};
    cuuint32_t es[5] = {1, 1, 1, 1, 1};
    cudaFree(0);
    CUresult r = enc(out, dtype == BMT_DT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, (void*)ptr,
                     dims, st, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return -12;   // the caller falls back to one 4-D copy per chunk
    std::lock_guard<std::mutex> lk(g_maps_mu);
    if (g_maps.size() > 8192) g_maps.clear();
    g_maps[key] = *out;
    return 0;
}

int g_num_sms = 0;
// SMs that fused (compute + collective) kernels leave free.  Their CTAs wait for other ranks while they hold their SM; when
// kernels of another parallel dimension (NCCL gathers of a ZeRO group) must be able to start next to them at any time, a
// few SMs stay out of the fused grids so that such a kernel always finds room (bmt_gemm_reserve_sms).
int g_reserved_sms = 0;

// Tile selection.  Per k-block (64 deep) an SM spends about 2.05 * BN clocks on the MMAs of its 128 accumulator rows
// and has to pull (128 + BN / ncta) * 128 bytes from L2 at about 64 bytes per clock; the slower of the two sets
// the pace.  A CTA pair (cta_group::2, 256 x BN tile) halves the B bytes per SM, which is what lifts large
// problems off the L2->SM limit.  The cost also counts waves on the available SMs and a fixed per-tile overhead.
struct TileChoice { int bn; int cta2; };

TileChoice pick_tile(int64_t M, int64_t N, int64_t K, int64_t batches, bool b_mn, int force_bn, int force_cta2) {
    TileChoice best{0, 0};
    double best_cost = 1e30;
    const double kblocks = (double)((K + BK - 1) / BK);
    for (int cta2 = 0; cta2 <= 1; ++cta2) {
        if (force_cta2 >= 0 && cta2 != force_cta2) continue;
        if (cta2 && M <= BM) continue;
        const int ncta = cta2 ? 2 : 1;
        const int step = (b_mn ? 64 : 16) * ncta;
        for (int bn = (b_mn ? 64 : 32) * ncta; bn <= 256; bn += step) {
            if (force_bn > 0 && bn != force_bn) continue;
            const int64_t tiles = ((M + BM * ncta - 1) / (BM * ncta)) * ((N + bn - 1) / bn) * batches;
            const int64_t slots = g_num_sms / ncta;
            const int64_t waves = (tiles + slots - 1) / slots;
            const double mma = 2.05 * bn, load = 2.0 * (128 + bn / ncta);
            const double per_tile = kblocks * (mma > load ? mma : load) + 600.0 + 6.0 * bn;  // + fill/drain and epilogue
            const double cost = (double)waves * per_tile;
            if (cost < best_cost * 0.999) { best_cost = cost; best = TileChoice{bn, cta2}; }
        }
    }
    return best;
}

int launch_gemm(const BmtGemmDesc& g, cudaStream_t stream, const FusedComm* fused = nullptr) {
    const int64_t m = g.m, n = g.n, k = g.k;
    const void* a = g.a; const void* b = g.b; void* c = g.c; const void* bias = g.bias;
    const int64_t lda = g.lda, ldb = g.ldb, ldc = g.ldc;
    const int a_major = g.a_major, b_major = g.b_major, c_dtype = g.c_dtype, act = g.act, accumulate = g.accumulate, ab_dtype = g.ab_dtype;
    const int64_t a_bs0 = g.a_bs0, a_bs1 = g.a_bs1, b_bs0 = g.b_bs0, b_bs1 = g.b_bs1, c_bs0 = g.c_bs0, c_bs1 = g.c_bs1;
    const int64_t batch_inner = g.batch_inner > 0 ? g.batch_inner : 1, batch_outer = g.batch_outer > 0 ? g.batch_outer : 1;
    const int64_t b_inner_div = g.b_inner_div;
    const float alpha = g.alpha;
    if (m <= 0 || n <= 0 || batch_inner <= 0 || batch_outer <= 0) return 0;
    if (k <= 0) return -20;
    if (g_num_sms == 0) {
        int dev = 0;
        BMT_CUDA_OK(cudaGetDevice(&dev));
        BMT_CUDA_OK(cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev));
        BMT_CUDA_OK(cudaFuncSetAttribute(gemm_tcgen05_kernel<false, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BUDGET + 2048));
        BMT_CUDA_OK(cudaFuncSetAttribute(gemm_tcgen05_kernel<true, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BUDGET + 2048));
        BMT_CUDA_OK(cudaFuncSetAttribute(gemm_tcgen05_kernel<false, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BUDGET + 2048));
        BMT_CUDA_OK(cudaFuncSetAttribute(gemm_tcgen05_kernel<false, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BUDGET + 2048));
        BMT_CUDA_OK(cudaFuncSetAttribute(gemm_tcgen05_kernel<false, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BUDGET + 2048));
        BMT_CUDA_OK(cudaFuncSetAttribute(gemm_tcgen05_kernel<true, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BUDGET + 2048));
        BMT_CUDA_OK(cudaFuncSetAttribute(gemm_tcgen05_kernel<true, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BUDGET + 2048));
        BMT_CUDA_OK(cudaFuncSetAttribute(gemm_tcgen05_kernel<true, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BUDGET + 2048));
    }
    static int force_bn = -1, force_cta2 = -2, debug_flags = -1;
    if (debug_flags < 0) { const char* e = getenv("BMT_GEMM_DEBUG"); debug_flags = e ? atoi(e) : 0; }
    if (force_bn < 0) { const char* e = getenv("BMT_GEMM_BN"); force_bn = e ? atoi(e) : 0; }
    if (force_cta2 == -2) { const char* e = getenv("BMT_GEMM_CTA2"); force_cta2 = e ? atoi(e) : -1; }

    GemmParams p;
    memset(&p, 0, sizeof(p));
    p.M = m; p.N = n; p.K = k;
    p.a_mn = a_major; p.b_mn = b_major;
    const int comm_ctas = (fused && (fused->mode == 2 || fused->mode == 3)) ? fused->ag_ctas : 0;
    const int held_back = fused ? comm_ctas + g_reserved_sms : 0;
    if (fused) g_num_sms -= held_back;  // tile choice for the CTAs that do math
    // a fused kernel can run as CTA pairs when its pusher CTAs pair up too and (mode 2) a rank's rows fill whole 256-row tiles
    const bool pair_ok = !fused || (comm_ctas % 2 == 0 && (fused->mode != 2 || fused->ag_rows % (2 * BM) == 0));
    TileChoice tc = pick_tile(m, n, k, batch_inner * batch_outer, b_major != 0, force_bn, pair_ok ? force_cta2 : 0);
    if (fused) g_num_sms += held_back;
    if (tc.bn == 0) tc = pick_tile(m, n, k, batch_inner * batch_outer, b_major != 0, 0, -1);  // forced shape not applicable here
    if (tc.bn == 0) return -22;
    p.bn = tc.bn;
    const int ncta = tc.cta2 ? 2 : 1;
    const uint32_t stage_bytes = BM * BK * 2 + (p.bn / ncta) * BK * 2;
    // The staged bulk-store epilogue of the GEMM -> reduce-scatter kernel can also serve plain GEMMs with 16-bit output
    // (BMT_GEMM_STAGED=1; =2: only for K <= 4096).  Off by default: measured on the transformer-block shapes it is slower
    // than the direct stores (797 vs 734 us over the 15 GEMMs of a block) because it costs a pipeline stage and local
    // stores do not need the 256-byte packets that peer stores do.
    static int staged_env = -1;
    if (staged_env < 0) { const char* e = getenv("BMT_GEMM_STAGED"); staged_env = e ? atoi(e) : 0; }
    const bool c16 = c_dtype == BMT_DT_F16 || c_dtype == BMT_DT_BF16;
    const bool can_stage = !fused && c16 && (ldc % 8 == 0) && (((uintptr_t)c & 15) == 0) && ((c_bs0 | c_bs1) % 8 == 0) && (n % 8 == 0) &&
                           (!bias || ((uintptr_t)bias & 15) == 0);
    p.staged = (can_stage && (staged_env == 1 || (staged_env == 2 && k <= 4096))) ? 1 : 0;
    const uint32_t out_stage_bytes = ((fused && fused->mode == 1) || p.staged) ? BM * OUT_PITCH : 0;
    int stages = (int)((SMEM_BUDGET - 1024 - out_stage_bytes) / stage_bytes);
    p.stages = stages > MAX_STAGES ? MAX_STAGES : stages;
    p.m_blocks = (int)((m + BM * ncta - 1) / (BM * ncta));
    p.n_blocks = (int)((n + p.bn - 1) / p.bn);
    p.batch_inner = batch_inner; p.batch_outer = batch_outer; p.b_inner_div = b_inner_div > 0 ? b_inner_div : 1;
    p.c = c; p.ldc = ldc; p.c_bs0 = c_bs0; p.c_bs1 = c_bs1; p.c_dtype = c_dtype;
    p.bias = bias; p.bias_dtype = ab_dtype; p.act = act; p.accumulate = accumulate; p.alpha = alpha;
    p.debug = debug_flags;
    static int group_env = -1;
    if (group_env < 0) { const char* e = getenv("BMT_GEMM_GROUP_M"); group_env = e ? atoi(e) : 0; }
    p.group_m = group_env > 0 ? group_env : 16;
    if (p.group_m > p.m_blocks) p.group_m = p.m_blocks;
    if (fused && fused->mode == 3) p.group_m = p.m_blocks;  // all row tiles of one weight chunk in a row: chunks are needed in order
    const bool rs_early = fused && fused->mode == 1 && fused->rs_rows % (BM * ncta) == 0;
    if (rs_early) {
        const int per_rank = (int)(fused->rs_rows / (BM * ncta));
        while (per_rank % p.group_m) --p.group_m;   // groups must not mix rows of this rank with rows of others
    }
    if (fused && fused->mode == 2) {
        // groups must not straddle the rows of two ranks (the tile order is rotated rank by rank)
        const int per_rank = (int)(fused->ag_rows / (BM * ncta));
        while (per_rank % p.group_m) --p.group_m;
    }
    p.residual = g.residual; p.ldr = g.ldr; p.aux = g.aux; p.ld_aux = g.ld_aux; p.aux_mode = g.aux ? g.aux_mode : 0;
    if ((p.residual || p.aux_mode) && batch_inner * batch_outer != 1) return -21;  // fused extras are for plain (unbatched) GEMMs
    const uint32_t fmt = ab_dtype == BMT_DT_F16 ? 0u : 1u;
    p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(a_major ? 1 : 0) << 15) | ((uint32_t)(b_major ? 1 : 0) << 16) |
              ((uint32_t)(p.bn >> 3) << 17) | ((uint32_t)((BM * ncta) >> 4) << 24);

    CUtensorMap ma, mb;
    int rc;
    const int64_t nb_b = (batch_inner + p.b_inner_div - 1) / p.b_inner_div;
    static int mn5_env = -1;
    if (mn5_env < 0) { const char* e = getenv("BMT_GEMM_MN5"); mn5_env = e ? atoi(e) : 1; }
    if (!a_major) rc = make_map(&ma, a, ab_dtype, k, m, lda, batch_inner, a_bs0, batch_outer, a_bs1, BK, BM);
    else {
        rc = mn5_env ? make_map_mn5(&ma, a, ab_dtype, m, k, lda, batch_inner, a_bs0, batch_outer, a_bs1, BK, BM / 64) : -1;
        p.a_mn5 = rc == 0 ? 1 : 0;
        if (rc) rc = make_map(&ma, a, ab_dtype, m, k, lda, batch_inner, a_bs0, batch_outer, a_bs1, 64, BK);
    }
    if (rc) return rc;
    if (!b_major) rc = make_map(&mb, b, ab_dtype, k, n, ldb, nb_b, b_bs0, batch_outer, b_bs1, BK, p.bn / ncta);
    else {
        rc = mn5_env ? make_map_mn5(&mb, b, ab_dtype, n, k, ldb, nb_b, b_bs0, batch_outer, b_bs1, BK, (p.bn / ncta) / 64) : -1;
        p.b_mn5 = rc == 0 ? 1 : 0;
        if (rc) rc = make_map(&mb, b, ab_dtype, n, k, ldb, nb_b, b_bs0, batch_outer, b_bs1, 64, BK);
    }
    if (rc) return rc;

    const int64_t tiles = (int64_t)p.m_blocks * p.n_blocks * batch_inner * batch_outer;
    p.out_stage_off = (uint32_t)p.stages * stage_bytes;
    p.hdr_off = p.out_stage_off + out_stage_bytes;
    if (comm_ctas > 0 && p.hdr_off < PUSH_STAGES * PUSH_PIECE_BYTES) p.hdr_off = PUSH_STAGES * PUSH_PIECE_BYTES;
    const size_t smem = (size_t)p.hdr_off + sizeof(SharedHeader) + 1024;
    FusedComm none;
    memset(&none, 0, sizeof(none));
    if (fused) {
        const int compute = (g_num_sms - held_back) / ncta;   // CTAs (or CTA pairs) that do math
        const unsigned grid = (unsigned)(ncta * (tiles < compute ? tiles : compute)) + comm_ctas;
        FusedComm fc = *fused;
        if (fc.mode == 3) fc.bg_first_block = (int)(((fc.bg_first / k) / p.bn) % p.n_blocks);
        if (fc.mode == 1) {
            fc.rs_early = rs_early ? 1 : 0;
            fc.rs_bpr = rs_early ? (int)(fc.rs_rows / (BM * ncta)) : 0;
            fc.rs_remote_tiles = rs_early ? (int64_t)(p.m_blocks - fc.rs_bpr) * p.n_blocks : 0;
        }
        if (!tc.cta2) {
            if (fc.mode == 1) gemm_tcgen05_kernel<false, 1><<<grid, NUM_THREADS, smem, stream>>>(ma, mb, p, fc);
            else if (fc.mode == 2) gemm_tcgen05_kernel<false, 2><<<grid, NUM_THREADS, smem, stream>>>(ma, mb, p, fc);
            else gemm_tcgen05_kernel<false, 3><<<grid, NUM_THREADS, smem, stream>>>(ma, mb, p, fc);
            bmt_count_launch(1);
            return (int)cudaGetLastError();
        }
        cudaLaunchConfig_t cfg;
        memset(&cfg, 0, sizeof(cfg));
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3(NUM_THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr; cfg.numAttrs = 1;
        cudaError_t e;
        if (fc.mode == 1) e = cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<true, 1>, ma, mb, p, fc);
        else if (fc.mode == 2) e = cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<true, 2>, ma, mb, p, fc);
        else e = cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<true, 3>, ma, mb, p, fc);
        bmt_count_launch(1);
        return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
    }
    if (!tc.cta2) {
        const unsigned grid = (unsigned)(tiles < g_num_sms ? tiles : g_num_sms);
        gemm_tcgen05_kernel<false, 0><<<grid, NUM_THREADS, smem, stream>>>(ma, mb, p, none);
        bmt_count_launch(1);
        return (int)cudaGetLastError();
    }
    const int64_t pairs = g_num_sms / 2;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)(2 * (tiles < pairs ? tiles : pairs)));
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<true, 0>, ma, mb, p, none);
    bmt_count_launch(1);
    return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

}  // namespace

extern "C" int bmt_gemm_reserve_sms(int n) {
    g_reserved_sms = n <= 0 ? 0 : (n > 64 ? 64 : (n & ~1));
    return 0;
}

extern "C" int bmt_gemm_ex(const BmtGemmDesc* desc, void* stream) { return launch_gemm(*desc, (cudaStream_t)stream); }

extern "C" int bmt_gemm(int64_t m, int64_t n, int64_t k, const void* a, int64_t lda, int a_major, const void* b, int64_t ldb,
                        int b_major, void* c, int64_t ldc, int c_dtype, const void* bias, int act, int accumulate, int ab_dtype,
                        void* stream) {
    BmtGemmDesc g;
    memset(&g, 0, sizeof(g));
    g.m = m; g.n = n; g.k = k; g.a = a; g.lda = lda; g.a_major = a_major; g.b = b; g.ldb = ldb; g.b_major = b_major;
    g.c = c; g.ldc = ldc; g.c_dtype = c_dtype; g.bias = bias; g.act = act; g.accumulate = accumulate; g.ab_dtype = ab_dtype;
    g.batch_inner = g.batch_outer = g.b_inner_div = 1; g.alpha = 1.0f;
    return launch_gemm(g, (cudaStream_t)stream);
}

extern "C" int bmt_gemm_batched(int64_t m, int64_t n, int64_t k, const void* a, int64_t lda, int a_major, int64_t a_bs0,
                                int64_t a_bs1, const void* b, int64_t ldb, int b_major, int64_t b_bs0, int64_t b_bs1, void* c,
                                int64_t ldc, int c_dtype, int64_t c_bs0, int64_t c_bs1, int64_t batch_inner, int64_t batch_outer,
                                int64_t b_inner_div, float alpha, int ab_dtype, void* stream) {
    BmtGemmDesc g;
    memset(&g, 0, sizeof(g));
    g.m = m; g.n = n; g.k = k; g.a = a; g.lda = lda; g.a_major = a_major; g.a_bs0 = a_bs0; g.a_bs1 = a_bs1;
    g.b = b; g.ldb = ldb; g.b_major = b_major; g.b_bs0 = b_bs0; g.b_bs1 = b_bs1;
    g.c = c; g.ldc = ldc; g.c_dtype = c_dtype; g.c_bs0 = c_bs0; g.c_bs1 = c_bs1;
    g.batch_inner = batch_inner; g.batch_outer = batch_outer; g.b_inner_div = b_inner_div; g.alpha = alpha; g.ab_dtype = ab_dtype;
    return launch_gemm(g, (cudaStream_t)stream);
}

// GEMM -> reduce-scatter over the rows of C (see FusedComm mode 1).  `inbox_slots[j]`: where this rank's slot starts in rank
// j's inbox; `grid_hint` receives the number of CTAs launched (the caller's counter advances by it per call).
// Reduce phase of a split GEMM -> reduce-scatter (bmt_gemm_reduce_scatter_main): to be launched after a wait kernel has
// seen every rank's "delivered" flag for `epoch`.  `counter_u32`: the same two counters the main kernel was given.
extern "C" int bmt_gemm_rs_reduce(const void* inbox_local, int64_t rows_per_rank, int64_t n, int world, int rank, void* const* flags,
                                  int free_row, unsigned int epoch, void* counter_u32, void* out, const void* bias, int dtype,
                                  void* stream) {
    if (world < 2 || world > 8 || n % 8 != 0) return -40;
    FusedComm f;
    memset(&f, 0, sizeof(f));
    f.world = world; f.rank = rank; f.free_row = free_row; f.epoch = epoch; f.rs_counter = (unsigned int*)counter_u32;
    for (int j = 0; j < world; ++j) f.flags[j] = (unsigned int*)flags[j];
    const int64_t nvec = rows_per_rank * n / 8, slot_elems = rows_per_rank * n;
    int64_t blocks = (nvec + NUM_THREADS * 4 - 1) / (NUM_THREADS * 4);
    if (blocks > 148) blocks = 148;
    if (blocks < 1) blocks = 1;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == BMT_DT_F16) rs_reduce_kernel<__half><<<(unsigned)blocks, NUM_THREADS, 0, st>>>(inbox_local, slot_elems, world, bias, n, out, nvec, f, epoch + 1);
    else rs_reduce_kernel<__nv_bfloat16><<<(unsigned)blocks, NUM_THREADS, 0, st>>>(inbox_local, slot_elems, world, bias, n, out, nvec, f, epoch + 1);
    bmt_count_launch(1);
    return (int)cudaGetLastError();
}

static int gemm_reduce_scatter_impl(const BmtGemmDesc* desc, int world, int rank, void* const* flags, int free_row, int done_row,
                                    unsigned int epoch, void* const* inbox_slots, const void* inbox_local, int64_t rows_per_rank,
                                    void* counter_u32, void* out, const void* bias, void* status_i32, double timeout_s,
                                    void* stream, int split);

// First half of a split GEMM -> reduce-scatter: the GEMM whose epilogue delivers every row to its owner's inbox and which
// publishes "delivered" when done.  No CTA waits for another rank's result or for its own grid.  Follow it with a wait
// on (done_row, epoch) and bmt_gemm_rs_reduce.
extern "C" int bmt_gemm_reduce_scatter_main(const BmtGemmDesc* desc, int world, int rank, void* const* flags, int free_row, int done_row,
                                            unsigned int epoch, void* const* inbox_slots, const void* inbox_local,
                                            int64_t rows_per_rank, void* counter_u32, void* status_i32, double timeout_s, void* stream) {
    return gemm_reduce_scatter_impl(desc, world, rank, flags, free_row, done_row, epoch, inbox_slots, inbox_local, rows_per_rank,
                                    counter_u32, nullptr, nullptr, status_i32, timeout_s, stream, 1);
}

extern "C" int bmt_gemm_reduce_scatter(const BmtGemmDesc* desc, int world, int rank, void* const* flags, int free_row, int done_row,
                                       unsigned int epoch, void* const* inbox_slots, const void* inbox_local, int64_t rows_per_rank,
                                       void* counter_u32, void* out, const void* bias, void* status_i32, double timeout_s,
                                       void* stream) {
    return gemm_reduce_scatter_impl(desc, world, rank, flags, free_row, done_row, epoch, inbox_slots, inbox_local, rows_per_rank,
                                    counter_u32, out, bias, status_i32, timeout_s, stream, 0);
}

static int gemm_reduce_scatter_impl(const BmtGemmDesc* desc, int world, int rank, void* const* flags, int free_row, int done_row,
                                    unsigned int epoch, void* const* inbox_slots, const void* inbox_local, int64_t rows_per_rank,
                                    void* counter_u32, void* out, const void* bias, void* status_i32, double timeout_s,
                                    void* stream, int split) {
    if (world < 2 || world > 8 || desc->m != rows_per_rank * world) return -40;
    if (desc->n % 8 != 0) return -41;
    FusedComm f;
    memset(&f, 0, sizeof(f));
    f.rs_split = split;
    f.mode = 1; f.world = world; f.rank = rank; f.free_row = free_row; f.done_row = done_row; f.epoch = epoch;
    f.status = (int*)status_i32; f.limit_ns = (uint64_t)(timeout_s * 1e9);
    for (int j = 0; j < world; ++j) { f.flags[j] = (unsigned int*)flags[j]; f.rs_inbox[j] = inbox_slots[j]; }
    f.rs_inbox_local = inbox_local; f.rs_rows = rows_per_rank; f.rs_counter = (unsigned int*)counter_u32; f.rs_out = out;
    f.rs_bias = bias;
    BmtGemmDesc g = *desc;
    g.bias = nullptr; g.residual = nullptr; g.aux = nullptr; g.accumulate = 0; g.act = 0;
    g.batch_inner = g.batch_outer = g.b_inner_div = 1;
    g.c = (void*)inbox_local; g.ldc = desc->n; g.c_dtype = desc->ab_dtype;
    return launch_gemm(g, (cudaStream_t)stream, &f);
}

// Number of CTAs the fused GEMM -> reduce-scatter launches for this problem (its completion counter advances by that much).
extern "C" int bmt_gemm_rs_grid(int64_t m, int64_t n, int64_t k, int b_major) {
    if (g_num_sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess) return -1;
        if (cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
    }
    const TileChoice tc = pick_tile(m, n, k, 1, b_major != 0, 0, 0);
    const int64_t tiles = ((m + BM - 1) / BM) * ((n + tc.bn - 1) / tc.bn);
    return (int)(tiles < g_num_sms ? tiles : g_num_sms);
}

// all-gather -> GEMM over the rows of A (see FusedComm mode 2).  The gathered matrix (world * rows x K, pitch K) lives in
// `gathered[rank]`; desc->a must point at it and desc->m = world * rows.  rows must be a multiple of 128.
extern "C" int bmt_all_gather_gemm(const BmtGemmDesc* desc, int world, int rank, void* const* flags, int free_row,
                                   unsigned int epoch, const void* src, int64_t ld_src, int64_t rows, void* const* gathered,
                                   void* const* counters, int comm_ctas, int skip_local, void* status_i32, double timeout_s,
                                   void* stream) {
    if (world < 2 || world > 8 || desc->m != rows * world || rows % BM != 0 || desc->a_major != 0) return -42;
    if (desc->k % 8 != 0 || desc->lda != desc->k || ld_src != desc->k || ((uintptr_t)src & 15)) return -43;
    FusedComm f;
    memset(&f, 0, sizeof(f));
    f.mode = 2; f.world = world; f.rank = rank; f.free_row = free_row; f.epoch = epoch;
    f.status = (int*)status_i32; f.limit_ns = (uint64_t)(timeout_s * 1e9);
    for (int j = 0; j < world; ++j) { f.flags[j] = (unsigned int*)flags[j]; f.ag_dst[j] = gathered[j]; f.ag_count[j] = (unsigned int*)counters[j]; }
    f.ag_ctas = comm_ctas; f.ag_src = src; f.ag_ld_src = ld_src; f.ag_rows = rows; f.skip_local = skip_local;
    // a 128-row block has 256 * K bytes = 2048 * (K / 8): pieces of 2048 * d bytes with d the largest divisor of K / 8 up to 16
    int d = 16;
    while ((desc->k / 8) % d) --d;
    f.ag_piece_bytes = 2048 * d; f.ag_pieces_per_block = (int)(desc->k / 8) / d;
    // runs: enough of them to keep every pusher CTA busy, otherwise one per block
    int rpb = 1;
    while ((int64_t)(world - (skip_local ? 1 : 0)) * (rows / BM) * rpb < 2 * (int64_t)comm_ctas && f.ag_pieces_per_block % (rpb * 2) == 0) rpb *= 2;
    f.ag_runs_per_block = rpb;
    BmtGemmDesc g = *desc;
    g.batch_inner = g.batch_outer = g.b_inner_div = 1;
    return launch_gemm(g, (cudaStream_t)stream, &f);
}

// How many CTAs of a fused kernel should push instead of multiply: the kernel ends when both the math (on the remaining
// SMs) and the pushes are done, so pick the even count that balances the two.  Rates are rough measured figures: a pusher
// CTA moves about 14 GB/s, all pushers together at most about 550 GB/s to remote destinations, and the math runs at
// about 1.1 PFLOP/s on a full GPU.  push_bytes counts every destination (own copy included), remote_bytes the peers only.
extern "C" int bmt_fused_comm_ctas(double flops, double push_bytes, double remote_bytes) {
    static int sms = 0;   // not g_num_sms: that one doubles as the "kernel attributes are set" marker of launch_gemm
    if (sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess) return 16;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 64) { sms = 0; return 16; }
    }
    int best = 8;
    double best_t = 1e30;
    for (int c = 8; c <= sms - 32; c += 4) {
        const double t_math = flops / (1.1e15 * (double)(sms - c) / (double)sms);
        double t_push = push_bytes / (c * 14e9);
        const double t_link = remote_bytes / 550e9;
        if (t_link > t_push) t_push = t_link;
        const double t = t_math > t_push ? t_math : t_push;
        if (t < best_t * 0.98) { best_t = t; best = c; }
    }
    return best;
}

static int zero_gather_split(int64_t n, int world, int comm_ctas);

// ZeRO weight gather -> GEMM (FusedComm mode 3).  desc->b points at the weight inside this rank's gathered buffer (N x K,
// rows contiguous, pitch K); this rank contributes the flat element range [first, first + count) of it, read from `src`.
// `expected` is a device array with the number of pieces every 128-row chunk receives from all ranks together
// (see bmt_zero_gather_expected).
extern "C" int bmt_zero_gather_gemm(const BmtGemmDesc* desc, int world, int rank, void* const* flags, int free_row,
                                    unsigned int epoch, const void* src, int64_t first, int64_t count, void* const* weight_on_rank,
                                    void* const* counters, const void* expected_u32, int comm_ctas, int skip_local,
                                    void* status_i32, double timeout_s, void* stream) {
    if (world < 2 || world > 8 || desc->b_major != 0 || desc->ldb != desc->k) return -44;
    if ((first & 7) || (count & 7) || ((uintptr_t)src & 15)) return -45;
    FusedComm f;
    memset(&f, 0, sizeof(f));
    f.mode = 3; f.world = world; f.rank = rank; f.free_row = free_row; f.epoch = epoch;
    f.status = (int*)status_i32; f.limit_ns = (uint64_t)(timeout_s * 1e9);
    for (int j = 0; j < world; ++j) { f.flags[j] = (unsigned int*)flags[j]; f.bg_dst[j] = weight_on_rank[j]; f.bg_cnt[j] = (unsigned int*)counters[j]; }
    f.ag_ctas = comm_ctas; f.bg_src = (const char*)src; f.bg_first = first; f.bg_count = count; f.skip_local = skip_local;
    f.bg_expected = (const unsigned int*)expected_u32;
    f.bg_split = zero_gather_split(desc->n, world, comm_ctas);
    BmtGemmDesc g = *desc;
    g.batch_inner = g.batch_outer = g.b_inner_div = 1;
    return launch_gemm(g, (cudaStream_t)stream, &f);
}

// Runs into which a rank's part of one chunk is cut: more when the weight has few chunks, so every pusher CTA has work.
static int zero_gather_split(int64_t n, int world, int comm_ctas) {
    const int64_t chunks = (n + BM - 1) / BM;
    int split = 1;
    while (chunks * world * split < 2 * (int64_t)comm_ctas && split < 8) split *= 2;
    return split;
}

// Host helper: counter bumps each 128-row chunk of an (n x k) weight receives when rank j owns the flat element range
// [first[j], first[j] + count[j]) and the kernel runs with `comm_ctas` pusher CTAs.  out has ceil(n / 128) entries.
extern "C" int bmt_zero_gather_expected(int64_t n, int64_t k, int world, const int64_t* first, const int64_t* count, int comm_ctas,
                                        unsigned int* out) {
    const int split = zero_gather_split(n, world, comm_ctas);
    const int64_t CK = (int64_t)BM * k;
    const int64_t chunks = (n + BM - 1) / BM;
    for (int64_t c = 0; c < chunks; ++c) out[c] = 0;
    for (int j = 0; j < world; ++j) {
        const int64_t lo_all = first[j], hi_all = first[j] + count[j];
        if (count[j] <= 0) continue;
        for (int64_t c = lo_all / CK; c * CK < hi_all && c < chunks; ++c) {
            const int64_t lo = lo_all > c * CK ? lo_all : c * CK;
            const int64_t hi = hi_all < (c + 1) * CK ? hi_all : (c + 1) * CK;
            const int64_t np = (hi - lo + BG_PIECE - 1) / BG_PIECE, per_run = (np + split - 1) / split;
            out[c] += (unsigned int)((np + per_run - 1) / per_run);
        }
    }
    return 0;
}

// Timing counters of the fused kernels launched on the current device since the last call (see g_fused_stats); the
// counters are cleared.  out: 8 values.  Synchronises with the device.
extern "C" int bmt_fused_stats(unsigned long long* out) {
    unsigned long long v[8], zero[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (cudaMemcpyFromSymbol(v, g_fused_stats, sizeof(v)) != cudaSuccess) return -1;
    if (cudaMemcpyToSymbol(g_fused_stats, zero, sizeof(zero)) != cudaSuccess) return -1;
    for (int i = 0; i < 8; ++i) out[i] = v[i];
    return 0;
}

// Status word of the GEMM kernels: 0, or (role << 16 | cta) of the first CTA whose bounded wait ran out.  Reading clears it.
extern "C" int bmt_gemm_status(void) {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemm_status, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_gemm_status, &zero, sizeof(int));
    return v;
}
