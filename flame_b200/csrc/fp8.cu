// Tensor-wise dynamic float8 quantisation for the fp8 GEMM (gemm2.cu, kind::f8f6f4).
//
// One call turns a bf16 matrix into an 8-bit copy, optionally a transposed 8-bit copy as well (the GEMM reads both
// operands K-major, so the backward products need the transposes), and the factor that undoes the scaling:
//   amax = max |x|,  scale = FMAX / amax,  q = sat(x * scale),  inv_scale = amax / FMAX
// with FMAX = 448 (e4m3) or 57344 (e5m2).  This is the "tensorwise" recipe of torchao's Float8Linear as configured by
// torchtitan/components/quantization/float8.py.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "host_utils.cuh"

namespace {

constexpr int TILE = 64;

__global__ void fp8_amax_kernel(const __nv_bfloat16* __restrict__ x, long long rows, int cols, long long ld,
                                unsigned int* __restrict__ amax_bits) {
  const int vec_per_row = cols >> 3;
  const long long total = rows * vec_per_row;
  float m = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vec_per_row;
    const int c = (int)(i - r * vec_per_row) << 3;
    const uint4 v = *reinterpret_cast<const uint4*>(x + r * ld + c);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(h[k]);
      m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, s));
  __shared__ float warp_max[8];
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) m = fmaxf(m, warp_max[w]);
    // non-negative floats order like their bit patterns; NaN (a larger pattern) propagates into the scale
    atomicMax(amax_bits, __float_as_uint(m));
  }
}

template <bool E5M2>
__device__ __forceinline__ uint32_t cvt4(float a, float b, float c, float d) {
  constexpr __nv_fp8_interpretation_t kind = E5M2 ? __NV_E5M2 : __NV_E4M3;
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, kind);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, kind);
  return lo | (hi << 16);
}

// One block converts a 64 x 64 tile: thread t owns 16 consecutive columns of row t / 4, writes them to q as one
// 16-byte store, and the tile goes through shared memory once more for the transposed copy.
template <bool E5M2, bool TRANSPOSE>
__global__ void __launch_bounds__(256)
fp8_cast_kernel(const __nv_bfloat16* __restrict__ x, long long rows, int cols, long long ld,
                const float* __restrict__ amax, uint8_t* __restrict__ q, uint8_t* __restrict__ qT,
                float* __restrict__ inv_scale) {
  constexpr float FMAX = E5M2 ? 57344.f : 448.f;
  const float a = fmaxf(*amax, 1e-12f);
  const float scale = FMAX / a;
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) *inv_scale = a / FMAX;
  __shared__ __align__(16) uint8_t tile[TILE][TILE + 16];
  const long long row0 = (long long)blockIdx.y * TILE;
  const int col0 = blockIdx.x * TILE;
  {
    const int r = threadIdx.x >> 2, cg = (threadIdx.x & 3) << 4;
    const long long row = row0 + r;
    const int col = col0 + cg;
    uint4 out = make_uint4(0, 0, 0, 0);
    if (row < rows && col < cols) {
      const uint4 v0 = *reinterpret_cast<const uint4*>(x + row * ld + col);
      const uint4 v1 = *reinterpret_cast<const uint4*>(x + row * ld + col + 8);
      const __nv_bfloat162* h0 = reinterpret_cast<const __nv_bfloat162*>(&v0);
      const __nv_bfloat162* h1 = reinterpret_cast<const __nv_bfloat162*>(&v1);
      float2 f[8];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        f[k] = __bfloat1622float2(h0[k]);
        f[4 + k] = __bfloat1622float2(h1[k]);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        f[k].x *= scale;
        f[k].y *= scale;
      }
      out.x = cvt4<E5M2>(f[0].x, f[0].y, f[1].x, f[1].y);
      out.y = cvt4<E5M2>(f[2].x, f[2].y, f[3].x, f[3].y);
      out.z = cvt4<E5M2>(f[4].x, f[4].y, f[5].x, f[5].y);
      out.w = cvt4<E5M2>(f[6].x, f[6].y, f[7].x, f[7].y);
      *reinterpret_cast<uint4*>(q + row * (long long)cols + col) = out;
    }
    if (TRANSPOSE) *reinterpret_cast<uint4*>(&tile[r][cg]) = out;
  }
  if (TRANSPOSE) {
    __syncthreads();
    const int c = threadIdx.x >> 2, rg = (threadIdx.x & 3) << 4;
    const int col = col0 + c;
    const long long row = row0 + rg;
    if (col < cols && row < rows) {
      uint32_t w[4];
#pragma unroll
      for (int k = 0; k < 4; ++k)
        w[k] = (uint32_t)tile[rg + 4 * k][c] | ((uint32_t)tile[rg + 4 * k + 1][c] << 8) |
               ((uint32_t)tile[rg + 4 * k + 2][c] << 16) | ((uint32_t)tile[rg + 4 * k + 3][c] << 24);
      *reinterpret_cast<uint4*>(qT + (long long)col * rows + row) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

}  // namespace

extern "C" {

// x: bf16 [rows, cols] with row stride ld (elements); rows and cols multiples of 16, ld a multiple of 8, x 16-byte
// aligned.  q: [rows, cols] bytes; qT: [cols, rows] bytes or null; amax: one float of scratch; inv_scale: one float.
int fb_fp8_quantize(const void* x, long long rows, int cols, long long ld, int e5m2, void* q, void* qT, float* amax,
                    float* inv_scale, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if ((rows & 15) || (cols & 15) || (ld & 7) || ((uintptr_t)x & 15) || ((uintptr_t)q & 15) || ((uintptr_t)qT & 15)) return -2;
  cudaError_t e = cudaMemsetAsync(amax, 0, sizeof(float), stream);
  if (e != cudaSuccess) return (int)e;
  const long long vecs = rows * (cols >> 3);
  long long blocks = (vecs + 256 * 8 - 1) / (256 * 8);
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  fp8_amax_kernel<<<(unsigned)blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, rows, cols, ld, (unsigned int*)amax);
  dim3 grid((cols + TILE - 1) / TILE, (unsigned)((rows + TILE - 1) / TILE));
  const __nv_bfloat16* xb = (const __nv_bfloat16*)x;
  if (e5m2) {
    if (qT) fp8_cast_kernel<true, true><<<grid, 256, 0, stream>>>(xb, rows, cols, ld, amax, (uint8_t*)q, (uint8_t*)qT, inv_scale);
    else    fp8_cast_kernel<true, false><<<grid, 256, 0, stream>>>(xb, rows, cols, ld, amax, (uint8_t*)q, nullptr, inv_scale);
  } else {
    if (qT) fp8_cast_kernel<false, true><<<grid, 256, 0, stream>>>(xb, rows, cols, ld, amax, (uint8_t*)q, (uint8_t*)qT, inv_scale);
    else    fp8_cast_kernel<false, false><<<grid, 256, 0, stream>>>(xb, rows, cols, ld, amax, (uint8_t*)q, nullptr, inv_scale);
  }
  return fb::launch_ok("fp8_cast_kernel");
}

}  // extern "C"
