// Host-side helpers: tensor-map (TMA descriptor) construction through the driver entry point,
// the library status word, and launch-error plumbing.  Nothing here allocates device memory.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

namespace fb {

// Library-wide status word written by kernels whose bounded waits run out or that reject an argument.
// It lives in mapped pinned host memory, so the host reads it without touching the stream and a kernel
// writes it through the same (unified) address.  Read with fb_status_read(); clear with fb_status_clear().
int* status_ptr();
// Limit (ns) of waits on flags raised by another GPU; set with fb_set_peer_wait_seconds().
unsigned long long peer_wait_ns();

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn();

// 2-D row-major tensor [rows, cols] with `ld` elements between rows; box = [box_rows, box_cols].
// elem_bytes 2 (bf16) or 4 (fp32).  Returns 0 on success.
int make_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint64_t cols, uint64_t ld,
                 uint32_t box_rows, uint32_t box_cols, bool swizzle128);
// 3-D tensor [d2, d1, d0] (d0 innermost) with strides in elements; box = [b2, b1, b0].  `swizzle`: 0 none, 1 the
// 128-byte pattern (so `true` keeps its meaning), kSwizzle64 the 64-byte pattern.
constexpr int kSwizzle64 = 64;
int make_tmap_3d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t d2, uint64_t d1, uint64_t d0,
                 uint64_t stride2, uint64_t stride1, uint32_t b2, uint32_t b1, uint32_t b0, int swizzle);

// 4-D tensor [d3, d2, d1, d0] (d0 innermost, contiguous) with strides in elements; box = [1, 1, b1, b0].
int make_tmap_4d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t d3, uint64_t d2, uint64_t d1, uint64_t d0,
                 uint64_t stride3, uint64_t stride2, uint64_t stride1, uint32_t b1, uint32_t b0, bool swizzle128);

inline int launch_ok(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    fprintf(stderr, "[flame_b200] launch of %s failed: %s\n", what, cudaGetErrorString(e));
    return (int)e;
  }
  return 0;
}

}  // namespace fb
