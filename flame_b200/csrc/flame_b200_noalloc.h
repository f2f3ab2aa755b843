// Allocation-free entry point of libflame_b200.
//
// This function has no counterpart in the reference project; it exists for callers of this library that are not
// allowed to allocate device memory at the time they need the result - for example code running inside a
// framework's own memory pool where a stray cudaMalloc would fragment or deadlock the pool, a latency-critical
// loop that must not hit the driver's allocator lock, or a host process that was started with all device memory
// already handed out.  Such callers pass only their input and output buffers; the scratch space the kernel needs
// is a fixed array that lives inside the library image on every GPU that loads it.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest hidden size accepted by fb_rmsnorm_bwd_noalloc.  The built-in scratch array holds
// 592 x FB_NOALLOC_MAX_D floats (about 9.7 MB per GPU, resident until the process exits).
#define FB_NOALLOC_MAX_D 4096

// RMSNorm backward without any allocation.
//
//   dx[rows, D] (bf16) = rstd * (dy * w - xhat * mean(dy * w * xhat)),  xhat = xin * rstd
//   dw[D]       (fp32) = sum over rows of dy * xhat      (added to dw when accumulate_dw != 0, else stored)
//
// dy, xin: bf16 [rows, D]; w: bf16 [D]; rstd: fp32 [rows] as written by the forward.  D must be a multiple of 8 and at
// most FB_NOALLOC_MAX_D; larger sizes are rejected with an error message and a non-zero return value.
//
// The function calls no cudaMalloc / cudaFree and no allocating library routine.  Its scratch (per-CTA partial sums
// of dw) is a file-scope device array; the first call on each device looks up that array's device address
// (cudaGetSymbolAddress) and therefore should happen before any stream capture on that device.  All calls on one
// device share the array: the kernels fully overwrite the part they read, so nothing needs clearing between calls,
// but two calls that overlap on the GPU (different streams without ordering) race on it.
//
// Returns 0 on success, a negative value for rejected arguments, or the CUDA error code of a failed launch.
int fb_rmsnorm_bwd_noalloc(const void* dy, const void* xin, const void* w, const float* rstd, void* dx, float* dw,
                           long long rows, int D, int accumulate_dw, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
