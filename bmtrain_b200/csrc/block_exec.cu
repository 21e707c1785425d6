// Native executor for one pre-LN GPT block: the whole forward (9 launches) or backward (21 launches) of a
// transformer layer is issued from C++ by a single call, so the host cost per layer is a few microseconds instead
// of one Python/autograd round trip per operator.  Every contraction goes to the tcgen05 GEMM (gemm_sm100.cu) with
// fused epilogues: bias, ReLU, residual add, ReLU-mask / GELU-derivative on the dgrad path.
// (The reference runs a block as ~40 separate PyTorch ops: example/layers/transformer.py:19-33.)
#include <math.h>
#include <string.h>

#include "api.h"
#include "common.cuh"

namespace {

#define RUN(expr)                 \
    do {                          \
        int _rc = (expr);         \
        if (_rc != 0) return _rc; \
    } while (0)

BmtGemmDesc plain(int64_t m, int64_t n, int64_t k, const void* a, int64_t lda, int a_major, const void* b, int64_t ldb, int b_major,
                  void* c, int64_t ldc, int dtype) {
    BmtGemmDesc g;
    memset(&g, 0, sizeof(g));
    g.m = m; g.n = n; g.k = k; g.a = a; g.lda = lda; g.a_major = a_major; g.b = b; g.ldb = ldb; g.b_major = b_major;
    g.c = c; g.ldc = ldc; g.c_dtype = dtype; g.ab_dtype = dtype; g.alpha = 1.f;
    g.batch_inner = g.batch_outer = g.b_inner_div = 1;
    return g;
}

struct Dims {
    int64_t T, d, h, dh, hd, dff, s, b, es;  // es = element size
};

Dims dims_of(const BmtGptBlock& k) {
    Dims q;
    q.b = k.batch; q.s = k.seq; q.T = k.batch * k.seq; q.d = k.d_model; q.h = k.n_heads; q.dh = k.d_head; q.hd = q.h * q.dh;
    q.dff = k.d_ff; q.es = 2;
    return q;
}

const char* off(const void* p, int64_t elems) { return (const char*)p + elems * 2; }
char* off(void* p, int64_t elems) { return (char*)p + elems * 2; }

}  // namespace

// Steps [first_step, last_step] of the forward (1 = LN1, 2 = QKV projection, 3..5 attention core, 6 = output
// projection + residual, 7 = LN2, 8 = first FFN GEMM, 9 = second FFN GEMM + residual).  Running a sub-range lets the
// caller put its own QKV GEMM (fused with the parameter gather) or a stream wait between the steps.
extern "C" int bmt_gpt_block_forward_steps(const BmtGptBlock* blk, int first_step, int last_step, void* stream) {
    const BmtGptBlock& k = *blk;
    const Dims q = dims_of(k);
    const int dt = k.dtype;
#define STEP(n) if (first_step <= (n) && (n) <= last_step)
    // 1. LN1
    STEP(1) RUN(bmt_norm_fwd(q.T, q.d, k.x, k.ln1_w, k.ln1_b, k.eps, 0, dt, k.ln1, k.stats1, stream));
    // 2. fused QKV projection (+ bias): qkv laid out (token, head, {q,k,v}, d_head)
    STEP(2) {
        BmtGemmDesc g = plain(q.T, 3 * q.hd, q.d, k.ln1, q.d, 0, k.qkv_w, q.d, 0, k.qkv, 3 * q.hd, dt);
        g.bias = k.qkv_b;
        RUN(bmt_gemm_ex(&g, stream));
    }
    const int64_t tok = 3 * q.hd, head = 3 * q.dh;
    // 3-5 as one fused attention kernel: q, k, v are strided views of the packed projection, nothing of size s x s is stored
    if (k.lse) {
        STEP(3) {
            const int64_t in_str[3] = {tok, head, q.s * tok}, out_str[3] = {q.hd, q.dh, q.s * q.hd};
            RUN(bmt_flash_attn_fwd(q.b, q.s, q.s, (int)q.h, (int)q.h, (int)q.dh, k.qkv, in_str, off(k.qkv, q.dh), in_str,
                                   off(k.qkv, 2 * q.dh), in_str, k.ctx, out_str, k.lse, 1.f / sqrtf((float)q.dh), k.causal, k.mask,
                                   nullptr, dt, stream));
        }
    } else {
    // 3. scores = q k^T / sqrt(d_head)   -> probs (b, h, s, ld)
    STEP(3) {
        BmtGemmDesc g = plain(q.s, q.s, q.dh, k.qkv, tok, 0, off(k.qkv, q.dh), tok, 0, k.probs, k.probs_ld, dt);
        g.a_bs0 = head; g.a_bs1 = q.s * tok; g.b_bs0 = head; g.b_bs1 = q.s * tok;
        g.c_bs0 = q.s * k.probs_ld; g.c_bs1 = q.h * q.s * k.probs_ld;
        g.batch_inner = q.h; g.batch_outer = q.b; g.alpha = 1.f / sqrtf((float)q.dh);
        RUN(bmt_gemm_ex(&g, stream));
    }
    // 4. masked softmax in place
    STEP(4) RUN(bmt_masked_softmax(q.b, q.h, q.s, q.s, k.probs_ld, k.probs, dt, k.causal, k.mask, nullptr, stream));
    // 5. ctx = probs v  -> (token, head, d_head)
    STEP(5) {
        BmtGemmDesc g = plain(q.s, q.dh, q.s, k.probs, k.probs_ld, 0, off(k.qkv, 2 * q.dh), tok, 1, k.ctx, q.hd, dt);
        g.a_bs0 = q.s * k.probs_ld; g.a_bs1 = q.h * q.s * k.probs_ld; g.b_bs0 = head; g.b_bs1 = q.s * tok;
        g.c_bs0 = q.dh; g.c_bs1 = q.s * q.hd;
        g.batch_inner = q.h; g.batch_outer = q.b;
        RUN(bmt_gemm_ex(&g, stream));
    }
    }
    // 6. h1 = ctx W_o^T + b_o + x
    STEP(6) {
        BmtGemmDesc g = plain(q.T, q.d, q.hd, k.ctx, q.hd, 0, k.out_w, q.hd, 0, k.h1, q.d, dt);
        g.bias = k.out_b; g.residual = k.x; g.ldr = q.d;
        RUN(bmt_gemm_ex(&g, stream));
    }
    // 7. LN2
    STEP(7) RUN(bmt_norm_fwd(q.T, q.d, k.h1, k.ln2_w, k.ln2_b, k.eps, 0, dt, k.ln2, k.stats2, stream));
    // 8. ff = act(ln2 W_1^T + b_1)
    STEP(8) {
        BmtGemmDesc g = plain(q.T, q.dff, q.d, k.ln2, q.d, 0, k.fc1_w, q.d, 0, k.act == 2 ? k.pre : k.ff, q.dff, dt);
        g.bias = k.fc1_b; g.act = k.act == 1 ? 1 : 0;
        RUN(bmt_gemm_ex(&g, stream));
        if (k.act == 2) RUN(bmt_gelu_fwd(q.T * q.dff, k.pre, dt, k.ff, stream));
    }
    // 9. y = ff W_2^T + b_2 + h1
    STEP(9) {
        BmtGemmDesc g = plain(q.T, q.d, q.dff, k.ff, q.dff, 0, k.fc2_w, q.dff, 0, k.y, q.d, dt);
        g.bias = k.fc2_b; g.residual = k.h1; g.ldr = q.d;
        RUN(bmt_gemm_ex(&g, stream));
    }
#undef STEP
    return 0;
}

extern "C" int bmt_gpt_block_forward(const BmtGptBlock* blk, void* stream) { return bmt_gpt_block_forward_steps(blk, 1, 9, stream); }

extern "C" int bmt_gpt_block_backward(const BmtGptBlock* blk, const BmtGptBlockGrad* grad, void* stream) {
    const BmtGptBlock& k = *blk;
    const BmtGptBlockGrad& w = *grad;
    const Dims q = dims_of(k);
    const int dt = k.dtype;
    const int64_t tok = 3 * q.hd, head = 3 * q.dh;
    // ---- FFN
    {   // d_ff = (dy W_2) * act'(.)
        BmtGemmDesc g = plain(q.T, q.dff, q.d, w.dy, q.d, 0, k.fc2_w, q.dff, 1, w.d_ff, q.dff, dt);
        g.aux = k.act == 2 ? k.pre : k.ff; g.ld_aux = q.dff; g.aux_mode = k.act == 2 ? 2 : 1;
        RUN(bmt_gemm_ex(&g, stream));
    }
    {   // dW_2 = dy^T ff
        BmtGemmDesc g = plain(q.d, q.dff, q.T, w.dy, q.d, 1, k.ff, q.dff, 1, w.d_fc2_w, q.dff, dt);
        g.accumulate = w.acc_w;
        RUN(bmt_gemm_ex(&g, stream));
    }
    RUN(bmt_colsum_ex(q.T, q.d, w.dy, dt, w.d_fc2_b, w.acc_small, w.colsum_scratch, w.colsum_scratch_bytes, stream));
    {   // d_ln2 = d_ff W_1
        BmtGemmDesc g = plain(q.T, q.d, q.dff, w.d_ff, q.dff, 0, k.fc1_w, q.d, 1, w.d_ln2, q.d, dt);
        RUN(bmt_gemm_ex(&g, stream));
    }
    {   // dW_1 = d_ff^T ln2
        BmtGemmDesc g = plain(q.dff, q.d, q.T, w.d_ff, q.dff, 1, k.ln2, q.d, 1, w.d_fc1_w, q.d, dt);
        g.accumulate = w.acc_w;
        RUN(bmt_gemm_ex(&g, stream));
    }
    RUN(bmt_colsum_ex(q.T, q.dff, w.d_ff, dt, w.d_fc1_b, w.acc_small, w.colsum_scratch, w.colsum_scratch_bytes, stream));
    // d_h1 = dy + LN2'(d_ln2)
    RUN(bmt_norm_bwd_ex(q.T, q.d, k.h1, w.d_ln2, k.ln2_w, k.stats2, 0, dt, w.nblk, w.d_h1, w.norm_partial, w.d_ln2_w, w.d_ln2_b,
                        w.dy, w.acc_small, stream));
    // ---- attention output projection
    {   // d_ctx = d_h1 W_o
        BmtGemmDesc g = plain(q.T, q.hd, q.d, w.d_h1, q.d, 0, k.out_w, q.hd, 1, w.d_ctx, q.hd, dt);
        RUN(bmt_gemm_ex(&g, stream));
    }
    {   // dW_o = d_h1^T ctx
        BmtGemmDesc g = plain(q.d, q.hd, q.T, w.d_h1, q.d, 1, k.ctx, q.hd, 1, w.d_out_w, q.hd, dt);
        g.accumulate = w.acc_w;
        RUN(bmt_gemm_ex(&g, stream));
    }
    RUN(bmt_colsum_ex(q.T, q.d, w.d_h1, dt, w.d_out_b, w.acc_small, w.colsum_scratch, w.colsum_scratch_bytes, stream));
    // ---- attention core
    const int64_t pl = k.probs_ld;
    if (k.lse) {
        // fused backward: dq, dk, dv go straight into the packed d_qkv buffer
        const int64_t in_str[3] = {tok, head, q.s * tok}, out_str[3] = {q.hd, q.dh, q.s * q.hd};
        RUN(bmt_flash_attn_bwd(q.b, q.s, q.s, (int)q.h, (int)q.h, (int)q.dh, k.qkv, in_str, off(k.qkv, q.dh), in_str,
                               off(k.qkv, 2 * q.dh), in_str, k.ctx, out_str, w.d_ctx, out_str, k.lse, w.d_qkv, in_str,
                               off(w.d_qkv, q.dh), in_str, off(w.d_qkv, 2 * q.dh), in_str, w.dq_acc, w.delta,
                               1.f / sqrtf((float)q.dh), k.causal, k.mask, nullptr, dt, stream));
    } else {
    {   // dP = d_ctx v^T
        BmtGemmDesc g = plain(q.s, q.s, q.dh, w.d_ctx, q.hd, 0, off(k.qkv, 2 * q.dh), tok, 0, w.d_probs, pl, dt);
        g.a_bs0 = q.dh; g.a_bs1 = q.s * q.hd; g.b_bs0 = head; g.b_bs1 = q.s * tok;
        g.c_bs0 = q.s * pl; g.c_bs1 = q.h * q.s * pl; g.batch_inner = q.h; g.batch_outer = q.b;
        RUN(bmt_gemm_ex(&g, stream));
    }
    RUN(bmt_softmax_bwd(q.b * q.h * q.s, q.s, pl, k.probs, w.d_probs, 1.f / sqrtf((float)q.dh), dt, stream));
    {   // dq = dS k
        BmtGemmDesc g = plain(q.s, q.dh, q.s, w.d_probs, pl, 0, off(k.qkv, q.dh), tok, 1, w.d_qkv, tok, dt);
        g.a_bs0 = q.s * pl; g.a_bs1 = q.h * q.s * pl; g.b_bs0 = head; g.b_bs1 = q.s * tok;
        g.c_bs0 = head; g.c_bs1 = q.s * tok; g.batch_inner = q.h; g.batch_outer = q.b;
        RUN(bmt_gemm_ex(&g, stream));
    }
    {   // dk = dS^T q
        BmtGemmDesc g = plain(q.s, q.dh, q.s, w.d_probs, pl, 1, k.qkv, tok, 1, off(w.d_qkv, q.dh), tok, dt);
        g.a_bs0 = q.s * pl; g.a_bs1 = q.h * q.s * pl; g.b_bs0 = head; g.b_bs1 = q.s * tok;
        g.c_bs0 = head; g.c_bs1 = q.s * tok; g.batch_inner = q.h; g.batch_outer = q.b;
        RUN(bmt_gemm_ex(&g, stream));
    }
    {   // dv = P^T d_ctx
        BmtGemmDesc g = plain(q.s, q.dh, q.s, k.probs, pl, 1, w.d_ctx, q.hd, 1, off(w.d_qkv, 2 * q.dh), tok, dt);
        g.a_bs0 = q.s * pl; g.a_bs1 = q.h * q.s * pl; g.b_bs0 = q.dh; g.b_bs1 = q.s * q.hd;
        g.c_bs0 = head; g.c_bs1 = q.s * tok; g.batch_inner = q.h; g.batch_outer = q.b;
        RUN(bmt_gemm_ex(&g, stream));
    }
    }
    // ---- QKV projection
    {   // d_ln1 = d_qkv W_qkv   (reuses the d_ln2 buffer)
        BmtGemmDesc g = plain(q.T, q.d, 3 * q.hd, w.d_qkv, tok, 0, k.qkv_w, q.d, 1, w.d_ln2, q.d, dt);
        RUN(bmt_gemm_ex(&g, stream));
    }
    {   // dW_qkv = d_qkv^T ln1
        BmtGemmDesc g = plain(3 * q.hd, q.d, q.T, w.d_qkv, tok, 1, k.ln1, q.d, 1, w.d_qkv_w, q.d, dt);
        g.accumulate = w.acc_w;
        RUN(bmt_gemm_ex(&g, stream));
    }
    RUN(bmt_colsum_ex(q.T, 3 * q.hd, w.d_qkv, dt, w.d_qkv_b, w.acc_small, w.colsum_scratch, w.colsum_scratch_bytes, stream));
    // dx = d_h1 + LN1'(d_ln1)
    RUN(bmt_norm_bwd_ex(q.T, q.d, k.x, w.d_ln2, k.ln1_w, k.stats1, 0, dt, w.nblk, w.dx, w.norm_partial, w.d_ln1_w, w.d_ln1_b,
                        w.d_h1, w.acc_small, stream));
    return 0;
}
