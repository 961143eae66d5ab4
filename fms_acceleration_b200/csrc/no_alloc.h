// Allocation-free entry point.  This has no counterpart in the reference project: it exists for callers of this
// library that must not allocate device memory when they call into it.
//
// Who that is: code that runs inside a region where the CUDA allocator may not be touched - for example a host
// program that has handed all device memory to its own arena and forbids cudaMalloc afterwards, a plugin loaded by
// an inference server whose memory budget is fixed at start-up, or a caller on a latency-critical path that cannot
// afford the implicit device synchronisation a cudaMalloc / cudaFree can cause.  The regular entry points of this
// library leave scratch allocation to the caller (the Python front-end uses torch's allocator); this one needs no
// scratch from anybody.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest row width (elements) and largest number of partial-sum rows the built-in scratch can hold.
#define FMSB_NOALLOC_MAX_H 8192
#define FMSB_NOALLOC_PARTIAL_ROWS 128

// RMSNorm backward with weight gradient, same math as fmsb_rmsnorm_bwd:
//   dx = inv_rms/H * (H * dy*w - xhat * sum(dy*w*xhat)) [+ dres_in],   dw[c] = sum_rows dy[r,c] * xhat[r,c]
// The per-CTA partial sums of dw live in a scratch array that is part of the library image (a file-scope
// __device__ array of FMSB_NOALLOC_PARTIAL_ROWS x FMSB_NOALLOC_MAX_H floats = 4 MiB; every GPU that loads the
// library holds it until the process exits).  The caller passes only inputs and outputs.
//
//   * H must be a multiple of 8 and at most FMSB_NOALLOC_MAX_H; larger rows are rejected with
//     FMSB_NOALLOC_ERR_TOO_LARGE and a message retrievable through fmsb_noalloc_last_error().
//   * dy, x, w, dres_in (when given) and dx must be 16-byte aligned (the kernels use 16-byte accesses; rows are
//     H elements apart, so with H a multiple of 8 every row is aligned when the base is); inv_rms and dw 4-byte
//     aligned.  A pointer off these boundaries is rejected with FMSB_NOALLOC_ERR_BAD_ARG; nothing is launched.
//   * The first call on a device looks up the device address of the scratch array (cudaGetSymbolAddress, with
//     that device current).  Make that first call outside of any stream capture.
//   * The entry point itself calls no cudaMalloc / cudaFree / allocating library routine, on any path.  What it
//     cannot control is the CUDA runtime's own module loading: with lazy loading (the default) the library's
//     device code, this 4 MiB array included, is placed on a device the first time something from the library is
//     used there, which can be this entry point's first call.  A caller with a no-allocation region should
//     therefore make one warm-up call per device (any small valid input) before entering that region; from then
//     on nothing is reserved or released.
//   * All calls on one device share the one scratch array and it keeps whatever the last call left in it.
//     Nothing in it has to start at zero: a call overwrites every partial row before it reads it.  Two calls
//     that overlap on the GPU (different streams, or one stream per thread) race on the scratch: serialise them.
//
// dtype: 0 = fp16, 1 = bf16.  dres_in may be null.  Returns 0, a CUDA error code (> 0) or one of the codes below.
#define FMSB_NOALLOC_ERR_BAD_ARG (-2)
#define FMSB_NOALLOC_ERR_TOO_LARGE (-3)
#define FMSB_NOALLOC_ERR_SETUP (-4)
int fmsb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* inv_rms, const void* dres_in,
                             void* dx, float* dw, int rows, int H, int gemma, int dtype, cudaStream_t stream);

// Text of the last error reported by fmsb_rmsnorm_bwd_noalloc on the calling thread ("" if none).
const char* fmsb_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
