// RMSNorm backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference implementation.
//
// Who needs it: code that runs where cudaMalloc is off limits - inside a region whose memory
// plan is frozen (a captured or replayed launch sequence, a pre-sized arena owned by another
// runtime), in a plug-in that is handed device pointers but no allocator, or in a process that
// runs close to the memory limit and must not fragment it.  The regular path
// (olb_rmsnorm_bwd + olb_colsum_finalize) needs a caller-provided fp32 scratch buffer for the
// per-block partial sums of the weight gradient; here that scratch is a file-scope device array
// that lives in the library image, so the call itself allocates nothing: no cudaMalloc, no
// cudaFree, no allocating library routine.
//
// Cost and limits:
//  * every GPU that loads the library holds the array until the process exits:
//    OLB_NOALLOC_MAX_PARTS x OLB_NOALLOC_MAX_COLS floats = 296 x 8192 x 4 B = 9.25 MiB;
//  * cols must be a multiple of 8 and <= OLB_NOALLOC_MAX_COLS; larger sizes are rejected with
//    OLB_NOALLOC_ERR_TOO_LARGE (use olb_noalloc_strerror for the text);
//  * the first call on a device looks up the array's device address (cudaGetSymbolAddress, with
//    that device current) and raises the kernel's shared-memory limit if the row is wide; make
//    this first call before any stream capture begins on that device;
//  * all calls on one device share the one array.  It keeps the previous call's contents; this
//    kernel overwrites every partial it later reads, so nothing needs clearing.  Two calls that
//    overlap on the GPU (different streams, no ordering between them) race on the array and
//    give wrong weight gradients: order them.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OLB_NOALLOC_MAX_COLS 8192
#define OLB_NOALLOC_MAX_PARTS 296

enum {
  OLB_NOALLOC_OK = 0,
  OLB_NOALLOC_ERR_BAD_COLS = -1,      // cols not a multiple of 8
  OLB_NOALLOC_ERR_LAUNCH = -2,        // a kernel launch failed
  OLB_NOALLOC_ERR_TOO_LARGE = -20,    // cols > OLB_NOALLOC_MAX_COLS
  OLB_NOALLOC_ERR_SYMBOL = -21,       // cudaGetSymbolAddress / attribute set-up failed
  OLB_NOALLOC_ERR_DEVICE = -22,       // no current device / device index out of range
  OLB_NOALLOC_ERR_NULL = -23,         // dy, x, rstd, dx or dw is null while rows > 0
};

// dx [rows, cols] (bf16) = RMSNorm input gradient; dw [cols] (bf16, or fp32 when dw_fp32) = weight
// gradient (overwritten).  dy, x: bf16 [rows, cols]; w: bf16 [cols]; rstd: fp32 [rows] as saved by
// olb_rmsnorm_fwd.  Work is enqueued on `stream`.  Returns OLB_NOALLOC_OK or a negative code.
int olb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx, void* dw,
                            int dw_fp32, int rows, int cols, cudaStream_t stream);

// Human-readable text for a return code of olb_rmsnorm_bwd_noalloc.
const char* olb_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
