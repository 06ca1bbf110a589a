// Allocation-free entry point of the kernel library.  (This entry point has no counterpart in the
// reference project, which ships no native code at all.)
//
// Who needs it: code that must not – or cannot – call the CUDA allocator around a kernel launch.
// Examples are hosts that hand this library a fixed memory budget up front (inference servers and
// embedded runtimes with their own arena), plugins running inside another framework's stream
// callbacks where cudaMalloc would synchronise the device, and real-time loops where an allocator
// call is an unbounded stall.  Such callers can still pass input and output buffers they own,
// but they have nowhere to get the kernel's fp32 work buffer from.
//
// What it is: RMSNorm backward, exactly as apb_rms_norm_bwd computes it, except that the fp32
// accumulator for the weight gradient lives in a fixed array inside the loaded library instead of
// being passed in.  The array holds APB_NOALLOC_MAX_D floats (64 KiB) and is held by every GPU
// that loads the library until the process exits.
//
// Rules for callers:
//   * D (the normalised width) must be a multiple of 8 and at most APB_NOALLOC_MAX_D; larger
//     widths are refused with APB_NOALLOC_ERR_TOO_LARGE and nothing is launched.
//   * The first call on each device looks up the array's device address (one-time set-up, done
//     with that device current).  Make that first call outside of any stream capture.
//   * All calls on one GPU share the one array.  It is cleared at the start of every call, so
//     calls may follow each other freely on one stream; two calls that can overlap on the GPU
//     (different streams without an ordering between them) race on it and give wrong dw.
//   * No cudaMalloc / cudaFree / allocating library routine is called, here or by the kernel.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define APB_NOALLOC_MAX_D 16384

#define APB_NOALLOC_OK 0
#define APB_NOALLOC_ERR_BAD_SHAPE 3   /* D not a multiple of 8, or negative sizes */
#define APB_NOALLOC_ERR_LAUNCH 4      /* the CUDA launch itself failed */
#define APB_NOALLOC_ERR_TOO_LARGE 7   /* D exceeds APB_NOALLOC_MAX_D */
#define APB_NOALLOC_ERR_SETUP 8       /* the scratch array's address could not be obtained */

// dy, x, dx: [rows, D]; w, dw: [D] (bf16 if is_bf16 else fp32); rstd: fp32 [rows].
int apb_rms_norm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx, void* dw,
                             long long rows, int D, int is_bf16, cudaStream_t stream);

// Human-readable text for a return code of the function above.
const char* apb_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
