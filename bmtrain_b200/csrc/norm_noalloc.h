// Allocation-free LayerNorm / RMSNorm backward.
//
// This entry point has no counterpart in the reference (OpenBMB/BMTrain has no norm kernel at all and every one of
// its launchers works on buffers the Python side allocated).
//
// Who needs it: code that drives the norm backward but is not allowed to obtain device memory at that moment --
// for example a host that embeds this library without PyTorch's caching allocator, a real-time or signal-handling
// path where cudaMalloc's implicit device synchronisation is unacceptable, or a process whose memory budget was
// handed out completely up front.  The regular entry point (bmt_norm_bwd in api.h) needs a caller-provided fp32
// scratch of 2 * nblk * d floats for the per-CTA partial sums of the weight / bias gradients; this variant keeps
// that scratch inside the library instead.
//
// How: the scratch is a file-scope `static __device__` array of fixed size (BMT_NORM_NOALLOC_SCRATCH_BYTES, 4 MiB;
// every GPU that loads the library holds it until the process exits).  Its device address is looked up with
// cudaGetSymbolAddress the first time the entry point runs on a given device (with that device current) and cached
// per device.  Because that first call performs this set-up, make it before any CUDA stream capture begins.
//
// Limits and rules:
//   * d must be a multiple of 8 and at most BMT_NORM_NOALLOC_MAX_D (4096); fp16 or bf16 only.  Anything else is
//     refused: the function prints one line to stderr and returns BMT_NORM_NOALLOC_TOO_LARGE (or
//     BMT_NORM_NOALLOC_BAD_ARG) without launching anything.
//   * rows is unlimited: the kernel uses at most BMT_NORM_NOALLOC_MAX_CTAS (128) CTAs that stride over the rows.
//   * The function calls no cudaMalloc / cudaFree and no allocating library routine; inputs and outputs are the
//     caller's.
//   * All calls share the one scratch array and it keeps the previous call's contents.  Nothing in it has to start
//     at zero (every slot that is read was written earlier in the same call), but two calls that overlap in time on
//     the same GPU (different streams, or different host threads) race on it: serialise them.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BMT_NORM_NOALLOC_MAX_D 4096
#define BMT_NORM_NOALLOC_MAX_CTAS 128
#define BMT_NORM_NOALLOC_SCRATCH_BYTES (2 * BMT_NORM_NOALLOC_MAX_CTAS * BMT_NORM_NOALLOC_MAX_D * 4)
#define BMT_NORM_NOALLOC_TOO_LARGE (-100)
#define BMT_NORM_NOALLOC_BAD_ARG (-101)

// dx, dw (and db when not NULL) <- backward of y = norm(x) * w (+ b) given dy and the saved (mean, rstd) rows.
// x, dy, dx: rows x d; w, dw, db: d; stats: 2 x rows fp32 (mean then rstd) as written by bmt_norm_fwd.
// dtype: 0 = fp16, 1 = bf16.  rms != 0 selects RMSNorm (db must be NULL).  Returns 0, a cudaError_t, or one of
// the negative codes above.
int bmt_norm_bwd_noalloc(int64_t rows, int64_t d, const void* x, const void* dy, const void* w, const void* stats,
                         int rms, int dtype, void* dx, void* dw, void* db, void* stream);

#ifdef __cplusplus
}
#endif
