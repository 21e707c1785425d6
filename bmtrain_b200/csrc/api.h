// C ABI of the CUDA kernel library (_C.so).  Every entry point takes raw device
// pointers and a CUDA stream handle, returns 0 on success (a cudaError_t value or
// a negative library code otherwise) and never allocates device memory.
// The reference exposes its kernels the same way -- pointers as integers through
// pybind (csrc/bind.cpp:3-35) -- here the boundary is plain C so that ctypes can load it.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BMT_MAX_TENSORS 24

typedef struct {
    void* p32[BMT_MAX_TENSORS];
    void* p16[BMT_MAX_TENSORS];
    void* g[BMT_MAX_TENSORS];
    void* m[BMT_MAX_TENSORS];
    void* v[BMT_MAX_TENSORS];
    int64_t n[BMT_MAX_TENSORS];
    int32_t count;
} BmtAdamTable;

typedef struct {
    void* p[BMT_MAX_TENSORS];
    int64_t n[BMT_MAX_TENSORS];
    int32_t count;
} BmtPtrTable;

// dtype codes: 0 = fp16, 1 = bf16, 2 = fp32
int bmt_adam_fp16_multi(const BmtAdamTable* tab, float beta1, float beta2, float eps, float lr, float scale, float wd,
                        float bc1, float bc2, void* stream);
int bmt_adam_fp16_f32state_multi(const BmtAdamTable* tab, float beta1, float beta2, float eps, float lr, float scale, float wd,
                                 float bc1, float bc2, void* stream);
int bmt_adam_bf16_multi(const BmtAdamTable* tab, float beta1, float beta2, float eps, float lr, float scale, float wd,
                        float bc1, float bc2, void* stream);

int bmt_has_inf_nan_multi(const BmtPtrTable* tab, int dtype, void* out_flag_u8, void* stream);
int bmt_sq_norm_multi(const BmtPtrTable* tab, int dtype, void* out_f32, void* stream);
int bmt_scale_multi(const BmtPtrTable* tab, int dtype, const void* coef_f32, void* stream);

int bmt_ce_row_stats(int64_t m, int64_t n, const void* logits, int dtype, const void* target_i64, int64_t vocab_start,
                     void* out_3xm_f32, void* stream);
int bmt_ce_backward(int64_t m, int64_t n, const void* logits, int dtype, const void* target_i64, const void* lse_f32,
                    const void* grad_loss_f32, int64_t vocab_start, int64_t ignore_index, void* out, void* stream);

int bmt_norm_fwd(int64_t rows, int64_t d, const void* x, const void* w, const void* b, float eps, int rms, int dtype,
                 void* y, void* stats_2xrows_f32, void* stream);
int bmt_norm_bwd(int64_t rows, int64_t d, const void* x, const void* dy, const void* w, const void* stats, int rms,
                 int dtype, int nblk, void* dx, void* partial_2xnblkxd_f32, void* dw, void* db, void* stream);

int bmt_norm_bwd_res(int64_t rows, int64_t d, const void* x, const void* dy, const void* w, const void* stats, int rms,
                     int dtype, int nblk, void* dx, void* partial_2xnblkxd_f32, void* dw, void* db, const void* dres, void* stream);

int bmt_norm_bwd_ex(int64_t rows, int64_t d, const void* x, const void* dy, const void* w, const void* stats, int rms,
                    int dtype, int nblk, void* dx, void* partial_2xnblkxd_f32, void* dw, void* db, const void* dres,
                    int accumulate, void* stream);

int bmt_embedding_fwd(int64_t tokens, int64_t d, const void* ids_i64, const void* weight, int dtype, void* out, void* stream);
int bmt_embedding_bwd(int64_t tokens, int64_t d, const void* ids_i64, const void* grad, int dtype, void* acc_f32, void* stream);

int bmt_masked_softmax(int64_t b, int64_t h, int64_t sq, int64_t sk, int64_t ld, void* scores, int dtype, int causal,
                       const void* mask_u8_b_sq_sk, const void* kv_lens_i32, void* stream);
int bmt_softmax_bwd(int64_t rows, int64_t cols, int64_t ld, const void* p, void* dp_inout, float scale, int dtype, void* stream);

int bmt_swiglu_fwd(int64_t rows, int64_t f, const void* x, int dtype, void* out, void* stream);
int bmt_swiglu_bwd(int64_t rows, int64_t f, const void* x, const void* g, int dtype, void* dx, void* stream);
int bmt_gelu_fwd(int64_t n, const void* x, int dtype, void* out, void* stream);
int bmt_colsum(int64_t m, int64_t n, const void* x, int dtype, void* out, void* stream);
// Same with a row-split grid: `scratch` = 4 KB of zero-initialised ticket counters followed by room for the partial sums
// (splits x n floats; the split count adapts to `scratch_bytes`); `accumulate`: out += column sums.
int bmt_colsum_ex(int64_t m, int64_t n, const void* x, int dtype, void* out, int accumulate, void* scratch,
                  int64_t scratch_bytes, void* stream);

// Full description of one (optionally batched) GEMM launch; zero-initialise, then fill what is needed.
typedef struct {
    int64_t m, n, k;
    const void* a; int64_t lda; int a_major; int64_t a_bs0, a_bs1;   // majors: 0 = reduction dim contiguous, 1 = output dim contiguous
    const void* b; int64_t ldb; int b_major; int64_t b_bs0, b_bs1;
    void* c; int64_t ldc; int c_dtype; int64_t c_bs0, c_bs1;
    int64_t batch_inner, batch_outer, b_inner_div;                    // B's inner batch index = inner index / b_inner_div
    const void* bias;                                                 // length n, operand dtype
    int act;                                                          // 0 none, 1 ReLU, 2 GELU
    int accumulate;                                                   // C += result
    float alpha;
    int ab_dtype;
    const void* residual; int64_t ldr;                                // + residual (m x n, operand dtype)
    const void* aux; int64_t ld_aux; int aux_mode;                    // 1: *= (aux > 0), 2: *= gelu'(aux)
} BmtGemmDesc;
// Fused GEMM + collective kernels launched from now on leave `n` SMs (even, at most 64) out of their grids, so that a kernel
// of another parallel dimension can start while their CTAs wait for other ranks; 0 restores full grids.
int bmt_gemm_reserve_sms(int n);
int bmt_gemm_ex(const BmtGemmDesc* desc, void* stream);

// C[M,N] (+)= alpha * op(A) op(B) (+ bias) with optional activation; majors: 0 = reduction dim contiguous, 1 = output dim contiguous.
int bmt_gemm(int64_t m, int64_t n, int64_t k, const void* a, int64_t lda, int a_major, const void* b, int64_t ldb,
             int b_major, void* c, int64_t ldc, int c_dtype, const void* bias, int act, int accumulate, int ab_dtype,
             void* stream);
int bmt_gemm_batched(int64_t m, int64_t n, int64_t k, const void* a, int64_t lda, int a_major, int64_t a_bs0, int64_t a_bs1,
                     const void* b, int64_t ldb, int b_major, int64_t b_bs0, int64_t b_bs1, void* c, int64_t ldc,
                     int c_dtype, int64_t c_bs0, int64_t c_bs1, int64_t batch_inner, int64_t batch_outer,
                     int64_t b_inner_div, float alpha, int ab_dtype, void* stream);
// ---- whole transformer block (pre-LN GPT layout) executed as one native call ---------------------------------
// y = h1 + fc2(act(fc1(LN2(h1)))),  h1 = x + out(attention(qkv(LN1(x))))
// All activations are caller-provided buffers; forward fills the "saved" ones, backward consumes them.
typedef struct {
    int64_t batch, seq, d_model, n_heads, d_head, d_ff;
    int dtype;   // 0 fp16, 1 bf16
    int act;     // 1 ReLU, 2 GELU
    float eps;
    int causal;
    const void* mask;  // uint8 (batch, seq, seq), 1 = attend; may be NULL
    const void *ln1_w, *ln1_b, *qkv_w, *qkv_b, *out_w, *out_b, *ln2_w, *ln2_b, *fc1_w, *fc1_b, *fc2_w, *fc2_b;
    const void* x;   // (batch*seq, d_model)
    void* y;         // (batch*seq, d_model)
    // saved activations
    void* ln1;       // (T, d)
    void* stats1;    // (2, T) fp32
    void* qkv;       // (T, heads, 3, d_head)
    void* probs;     // (batch, heads, seq, probs_ld)
    int64_t probs_ld;
    void* ctx;       // (T, heads*d_head)
    void* h1;        // (T, d)
    void* ln2;       // (T, d)
    void* stats2;    // (2, T) fp32
    void* ff;        // (T, d_ff) post-activation
    void* pre;       // (T, d_ff) pre-activation, GELU only (NULL for ReLU)
    // fused attention (csrc/attn_sm100.cu): non-NULL lse selects it; probs is then unused and may be NULL
    void* lse;       // (batch, heads, seq) fp32
} BmtGptBlock;

typedef struct {
    const void* dy;  // (T, d)
    void* dx;        // (T, d)
    void *d_ln1_w, *d_ln1_b, *d_qkv_w, *d_qkv_b, *d_out_w, *d_out_b, *d_ln2_w, *d_ln2_b, *d_fc1_w, *d_fc1_b, *d_fc2_w, *d_fc2_b;
    int acc_w;       // 1: the four weight-matrix gradients are accumulated into (C += ...), 0: overwritten
    // workspace
    void* d_ff;      // (T, d_ff)
    void* d_ln2;     // (T, d)   also reused for d_ln1
    void* d_h1;      // (T, d)
    void* d_ctx;     // (T, heads*d_head)
    void* d_probs;   // like probs
    void* d_qkv;     // like qkv
    void* norm_partial;  // (2, nblk, d) fp32
    int nblk;
    // fused attention backward scratch (used when the block carries lse): fp32, T*heads*d_head and batch*heads*seq
    void* dq_acc;
    void* delta;
    int acc_small;            // bias and norm gradients are added to what d_*_b / d_ln*_w already hold
    void* colsum_scratch;     // optional work space of bmt_colsum_ex (zero-initialised once), colsum_scratch_bytes large
    int64_t colsum_scratch_bytes;
} BmtGptBlockGrad;

int bmt_gpt_block_forward(const BmtGptBlock* blk, void* stream);
int bmt_gpt_block_forward_steps(const BmtGptBlock* blk, int first_step, int last_step, void* stream);
int bmt_gpt_block_backward(const BmtGptBlock* blk, const BmtGptBlockGrad* g, void* stream);

// ---- peer memory (one NVLink domain) ------------------------------------------------------------------------------
int bmt_symm_alloc(int64_t bytes, void** out);
int bmt_symm_free(void* p);
int bmt_ipc_get_handle(void* p, void* handle64);
int bmt_ipc_open_handle(const void* handle64, void** out);
int bmt_ipc_close(void* p);
int bmt_ipc_handle_size(void);
int bmt_fused_reduce_scatter(const void* const* peers, void* const* peer_flags, int world, int rank, int slot,
                             unsigned int epoch, int64_t part, void* out, int accumulate, float scale, int dtype,
                             void* overflow_u8, void* status_i32, double timeout_s, void* stream);
// Same reduction with one multimem.ld_reduce per 16 bytes through the NVSwitch multicast address of the full buffers.
int bmt_fused_reduce_scatter_mc(const void* multicast, void* const* peer_flags, int world, int rank, int slot,
                                unsigned int epoch, int64_t part, void* out, int accumulate, float scale, int dtype,
                                void* overflow_u8, void* status_i32, double timeout_s, void* stream);
// Both forms with the optional extras (`multicast` null: plain peer loads): `acc32` = fp32 partition gradient through which
// accumulation over micro-steps goes (rounded to `out` once per call), `sqsum_f32` += sum of squares of the values written.
int bmt_fused_reduce_scatter_ex(const void* const* peers, const void* multicast, void* const* peer_flags, int world, int rank,
                                int slot, unsigned int epoch, int64_t part, void* out, int accumulate, float scale, int dtype,
                                void* acc32, void* sqsum_f32, void* overflow_u8, void* status_i32, double timeout_s,
                                void* stream);
int bmt_push_ranges(const void* const* src, const int64_t* dst_off, const int64_t* nbytes, int nranges, void* const* dst,
                    void* const* peer_flags, int world, int rank, int free_row, int done_row, unsigned int epoch,
                    void* counter_u32, void* status_i32, double timeout_s, int grid, void* stream);
int bmt_symm_signal_wait(void* device_flag_table, int world, int rank, int slot, unsigned int epoch, int do_signal,
                         int do_wait, void* status_i32, double timeout_s, void* stream);

// fused tensor-parallel operators: one kernel does the GEMM and the collective over peer memory
int bmt_gemm_reduce_scatter(const BmtGemmDesc* desc, int world, int rank, void* const* flags, int free_row, int done_row,
                            unsigned int epoch, void* const* inbox_slots, const void* inbox_local, int64_t rows_per_rank,
                            void* counter_u32, void* out, const void* bias, void* status_i32, double timeout_s, void* stream);
int bmt_gemm_rs_grid(int64_t m, int64_t n, int64_t k, int b_major);
// The same operator as three launches, for jobs in which other kernels that wait for other ranks (ZeRO gathers and
// reductions) run next to the tensor-parallel ones: (1) the GEMM that delivers every row to its owner and publishes
// "delivered", none of whose CTAs waits for another rank's result or for its own grid; (2) a one-CTA wait on
// (done_row, epoch), e.g. bmt_symm_signal_wait; (3) the sum over the inbox slots (+ bias).
int bmt_gemm_reduce_scatter_main(const BmtGemmDesc* desc, int world, int rank, void* const* flags, int free_row, int done_row,
                                 unsigned int epoch, void* const* inbox_slots, const void* inbox_local, int64_t rows_per_rank,
                                 void* counter_u32, void* status_i32, double timeout_s, void* stream);
int bmt_gemm_rs_reduce(const void* inbox_local, int64_t rows_per_rank, int64_t n, int world, int rank, void* const* flags,
                       int free_row, unsigned int epoch, void* counter_u32, void* out, const void* bias, int dtype, void* stream);
int bmt_all_gather_gemm(const BmtGemmDesc* desc, int world, int rank, void* const* flags, int free_row, unsigned int epoch,
                        const void* src, int64_t ld_src, int64_t rows, void* const* gathered, void* const* counters,
                        int comm_ctas, int skip_local, void* status_i32, double timeout_s, void* stream);

// skip_local != 0 (both kernels): the caller has already copied this rank's own part into its gathered buffer, the pusher
// CTAs only serve the peers and the math does not wait for the own part.  bmt_zero_gather_expected must then be given
// count[rank] = 0 on that rank.
int bmt_zero_gather_gemm(const BmtGemmDesc* desc, int world, int rank, void* const* flags, int free_row, unsigned int epoch,
                         const void* src, int64_t first, int64_t count, void* const* weight_on_rank, void* const* counters,
                         const void* expected_u32, int comm_ctas, int skip_local, void* status_i32, double timeout_s,
                         void* stream);
int bmt_zero_gather_expected(int64_t n, int64_t k, int world, const int64_t* first, const int64_t* count, int comm_ctas,
                             unsigned int* out);

// number of kernel launches issued by this library since load (for launch accounting)
int64_t bmt_launch_count(void);
void bmt_count_launch(int n);
// SM copy of nbytes (multiple of 16) between device pointers, either of which may be a mapped peer buffer.
int bmt_peer_copy(void* dst, const void* src, int64_t nbytes, int grid, void* stream);
// Number of pusher CTAs that balances math and transfer of a fused all-gather -> GEMM / ZeRO gather -> GEMM kernel.
int bmt_fused_comm_ctas(double flops, double push_bytes, double remote_bytes);

// ---- asynchronous offloaded Adam: a worker thread of this library runs batches of jobs in submission order ---------
// One job = one contiguous range of one parameter shard.  The fp32 state is read from (p32, m, v) and written to
// (p32_out, m_out, v_out); pass the same pointers for an in-place step, a second set of arrays for a step that can
// still be discarded.  `upload` != 0: the new half parameters are copied to the device when the math is done.
typedef struct {
    void* grad_ready;                       // cudaEvent_t of the gradient's copy to the host, or NULL
    const void* p32; const void* m; const void* v;
    void* p32_out; void* m_out; void* v_out;
    void* p16_host; const void* g16_host; void* p_dev;
    int64_t n;
    float beta1, beta2, eps, lr, scale, wd, bc1, bc2;
    int bf16, upload;
} BmtOffloadJob;
typedef void (*BmtAdamCpuExFn)(int64_t n, const void* p32, const void* m, const void* v, void* p32_out, void* m_out, void* v_out,
                               void* p16, const void* g16, float beta1, float beta2, float eps, float lr, float scale, float wd,
                               float bc1, float bc2, int bf16);
// Queue a batch (the jobs are copied); returns a ticket > 0, or a negative CUDA error.  Uploads go to `h2d_stream`.
int64_t bmt_offload_submit(const BmtOffloadJob* jobs, int n, BmtAdamCpuExFn fn, void* h2d_stream);
// Block until the batch has been processed (math done, uploads queued).  With `stream` != NULL that stream is then made
// to wait for the batch's uploads.  Returns 0 or the CUDA error the batch ran into.
int bmt_offload_wait(int64_t ticket, void* stream);
// 1 when the batch has been processed, 0 while it is queued or running.
int bmt_offload_poll(int64_t ticket);
// Take a batch that has not been started out of the queue: 1 = removed (it will never run), 0 = running or finished.
int bmt_offload_cancel(int64_t ticket);
// Block until every batch submitted so far has been processed.
int bmt_offload_drain(void);
// Queue only the uploads of the jobs (no math): used to publish results that were computed ahead of time.
int64_t bmt_offload_submit_uploads(const BmtOffloadJob* jobs, int n, void* h2d_stream);

// Rotary position embedding on a packed (b, s, hk, g + 2, d) projection (csrc/elementwise.cu): split != 0 writes rotated q
// (b, s, hk*g, d), rotated k and copied v (b, s, hk, d); split == 0 is the backward (q, k, v gradients -> packed gradient).
// cos_sin: fp32 (cos, sin) pairs for every (position, frequency), (pos0 + s) x d/2 of them.
int bmt_rope_qkv(int64_t batch, int64_t seq, int hk, int g, int d, void* packed, int64_t p_tok, int64_t p_batch, void* q, void* k,
                 void* v, const void* cos_sin, int64_t pos0, int split, int dtype, void* stream);

// Fused attention forward (csrc/attn_sm100.cu): o = softmax(scale * q k^T + masks) v, lse = log-sum-exp per row.
// q (b, sq, h, d), k / v (b, sk, hk, d), o (b, sq, h, d); *_strides = element strides {token, head, batch}, head dim
// contiguous; d a multiple of 16 up to 128; strides multiples of 8; pointers 16-byte aligned.  lse (b, h, sq) fp32 or
// NULL; mask (b, sq, sk) bytes (non-zero = attend) or NULL; kv_lens (b) int32 or NULL.
int bmt_flash_attn_fwd(int64_t batch, int64_t sq, int64_t sk, int h, int hk, int d, const void* q, const int64_t* q_strides,
                       const void* k, const int64_t* k_strides, const void* v, const int64_t* v_strides, void* o,
                       const int64_t* o_strides, void* lse, float scale, int causal, const void* mask, const void* kv_lens,
                       int dtype, void* stream);
// Backward of bmt_flash_attn_fwd: o / lse from the forward, dout = gradient of o; dq, dk, dv receive the gradients (strided
// like q, k, v).  Scratch from the caller: dq_acc = batch * sq * h * d floats, delta = batch * h * sq floats.
int bmt_flash_attn_bwd(int64_t batch, int64_t sq, int64_t sk, int h, int hk, int d, const void* q, const int64_t* q_strides,
                       const void* k, const int64_t* k_strides, const void* v, const int64_t* v_strides, const void* o,
                       const int64_t* o_strides, const void* dout, const int64_t* do_strides, const void* lse, void* dq,
                       const int64_t* dq_strides, void* dk, const int64_t* dk_strides, void* dv, const int64_t* dv_strides,
                       void* dq_acc, void* delta, float scale, int causal, const void* mask, const void* kv_lens, int dtype,
                       void* stream);
// 0, or (wait code << 16 | CTA) of the first attention CTA whose bounded wait ran out; reading clears it
int bmt_attn_status(void);

// status word of the GEMM kernels: 0, or (role << 16 | cta) of the first CTA whose bounded wait ran out; reading clears it
int bmt_gemm_status(void);
// Timing counters of the fused compute+collective GEMM kernels since the last call, in nanoseconds: out[0] sum over
// compute CTAs of producer time spent waiting for other ranks' data, out[1] longest pusher CTA, out[2] longest CTA,
// out[3] longest producer wait of one CTA, out[4] kernels counted, out[5] (GEMM -> reduce-scatter) longest wait for the
// other ranks' deliveries, out[6] longest CTA including the reduce phase, out[7] sum over CTAs of the out[5] wait.
// Reading clears the counters.
int bmt_fused_stats(unsigned long long* out);

#ifdef __cplusplus
}
#endif
