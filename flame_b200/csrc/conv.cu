// Depthwise causal short convolution (kernel width <= 8) over packed sequences, with optional bias and SiLU.
//   pre[t, d] = b[d] + sum_{j < W, j <= pos[t]} w[d, W-1-j] * x[t-j, d];   y = act(pre)
// `pos[t]` is the token's offset inside its document, so taps never reach into the previous document.
// Backward runs as: (1) dpre = dy * act'(pre) with pre recomputed, (2) dx[t] = sum_j w[., W-1-j] dpre[t+j] (same
// document only) together with per-CTA partial sums of dw / db, (3) a fixed-order reduction of the partials.
// Semantics of fla/modules/conv/triton/kernels.py:37-345; the row-strip partial reduction replaces its atomics.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include "host_utils.cuh"

namespace {

constexpr int MAXW = 8;

__device__ __forceinline__ void unpack8(const uint4& q, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 q;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return q;
}
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// weights are read as bf16 [D, W]; one thread = one token x 8 channels
template <bool SILU, bool WRITE_DPRE>
__global__ void conv_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                const __nv_bfloat16* __restrict__ b, const int* __restrict__ pos,
                                const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ out, long long T,
                                int D, int W, long long ldx, long long ldo) {
  const int vec = D >> 3;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= T * vec) return;
  const long long t = idx / vec;
  const int d0 = (int)(idx - t * vec) * 8;
  const int p = pos[t];
  float acc[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) acc[c] = b ? __bfloat162float(b[d0 + c]) : 0.f;
  for (int j = 0; j < W && j <= p; ++j) {
    float xv[8];
    unpack8(*reinterpret_cast<const uint4*>(x + (t - j) * ldx + d0), xv);
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[c] += __bfloat162float(w[(d0 + c) * W + (W - 1 - j)]) * xv[c];
  }
  float o[8];
  if (WRITE_DPRE) {
    float g[8];
    unpack8(*reinterpret_cast<const uint4*>(dy + t * ldo + d0), g);
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      if (SILU) {
        const float s = sigmoidf_(acc[c]);
        o[c] = g[c] * s * (1.f + acc[c] * (1.f - s));
      } else {
        o[c] = g[c];
      }
    }
  } else {
#pragma unroll
    for (int c = 0; c < 8; ++c) o[c] = SILU ? acc[c] * sigmoidf_(acc[c]) : acc[c];
  }
  *reinterpret_cast<uint4*>(out + t * ldo + d0) = pack8(o);
}

// dx and per-strip partial sums of dw (and db).  grid = (channel vectors / 32, strips); a warp's lanes cover 32
// consecutive channel vectors, each thread walks its strip of rows.
__global__ void conv_bwd_kernel(const __nv_bfloat16* __restrict__ dpre, const __nv_bfloat16* __restrict__ x,
                                const __nv_bfloat16* __restrict__ w, const int* __restrict__ pos,
                                __nv_bfloat16* __restrict__ dx, float* __restrict__ part, long long T, int D, int W,
                                long long ldx, long long ldd, int rows_per_strip) {
  const int vec = D >> 3;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= vec) return;
  const int d0 = v * 8;
  const long long r0 = (long long)blockIdx.y * rows_per_strip;
  const long long r1 = min(T, r0 + rows_per_strip);
  float wv[MAXW][8];
  for (int j = 0; j < W; ++j)
#pragma unroll
    for (int c = 0; c < 8; ++c) wv[j][c] = __bfloat162float(w[(d0 + c) * W + (W - 1 - j)]);  // tap at distance j
  float dw[MAXW][8], db[8];
  for (int j = 0; j < MAXW; ++j)
#pragma unroll
    for (int c = 0; c < 8; ++c) dw[j][c] = 0.f;
#pragma unroll
  for (int c = 0; c < 8; ++c) db[c] = 0.f;
  for (long long t = r0; t < r1; ++t) {
    float g[8];
    unpack8(*reinterpret_cast<const uint4*>(dpre + t * ldd + d0), g);
    const int p = pos[t];
    // weight / bias gradients: dw[tap j] += dpre[t] * x[t - j]
#pragma unroll
    for (int c = 0; c < 8; ++c) db[c] += g[c];
    for (int j = 0; j < W && j <= p; ++j) {
      float xv[8];
      unpack8(*reinterpret_cast<const uint4*>(x + (t - j) * ldx + d0), xv);
#pragma unroll
      for (int c = 0; c < 8; ++c) dw[j][c] += g[c] * xv[c];
    }
    // input gradient: dx[t] = sum_j w[tap j] * dpre[t + j] while t + j is in the same document
    float acc[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[c] = wv[0][c] * g[c];
    for (int j = 1; j < W; ++j) {
      const long long tj = t + j;
      if (tj >= T || pos[tj] < j) break;  // crossed into the next document (positions restart at 0)
      float gj[8];
      unpack8(*reinterpret_cast<const uint4*>(dpre + tj * ldd + d0), gj);
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[c] += wv[j][c] * gj[c];
    }
    *reinterpret_cast<uint4*>(dx + t * ldx + d0) = pack8(acc);
  }
  // partial layout: [strip][D][W + 1]
  float* dst = part + ((long long)blockIdx.y * D + d0) * (W + 1);
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    for (int j = 0; j < W; ++j) dst[c * (W + 1) + (W - 1 - j)] = dw[j][c];
    dst[c * (W + 1) + W] = db[c];
  }
}

__global__ void conv_reduce_kernel(const float* __restrict__ part, int strips, int D, int W, float* __restrict__ dw,
                                   float* __restrict__ db, int accumulate) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;  // over D * (W + 1)
  if (i >= D * (W + 1)) return;
  float s = 0.f;
  for (int k = 0; k < strips; ++k) s += part[(long long)k * D * (W + 1) + i];
  const int d = i / (W + 1), j = i % (W + 1);
  if (j < W) {
    float* o = dw + d * W + j;
    *o = accumulate ? *o + s : s;
  } else if (db != nullptr) {
    float* o = db + d;
    *o = accumulate ? *o + s : s;
  }
}

}  // namespace

extern "C" {

int fb_short_conv_strips(long long T) {
  long long s = (T + 255) / 256;
  return (int)(s < 1 ? 1 : (s > 512 ? 512 : s));
}

int fb_short_conv_fwd(const void* x, const void* w, const void* b, const int* pos, void* y, long long T, int D, int W,
                      long long ldx, long long ldy, int silu, cudaStream_t stream) {
  if (T == 0) return 0;
  if ((D % 8) || W > MAXW || (ldx % 8) || (ldy % 8)) return -2;
  const unsigned blocks = (unsigned)((T * (D / 8) + 255) / 256);
  if (silu)
    conv_fwd_kernel<true, false><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
                                                             (const __nv_bfloat16*)b, pos, nullptr, (__nv_bfloat16*)y, T,
                                                             D, W, ldx, ldy);
  else
    conv_fwd_kernel<false, false><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
                                                              (const __nv_bfloat16*)b, pos, nullptr, (__nv_bfloat16*)y,
                                                              T, D, W, ldx, ldy);
  return fb::launch_ok("conv_fwd_kernel");
}

// dpre: bf16 [T, D] scratch; part: fp32 [fb_short_conv_strips(T), D, W + 1] scratch; dw: fp32 [D, W]; db: fp32 [D] or null
int fb_short_conv_bwd(const void* dy, const void* x, const void* w, const void* b, const int* pos, void* dx, void* dpre,
                      float* part, float* dw, float* db, long long T, int D, int W, long long ldx, long long ldy, int silu,
                      int accumulate, cudaStream_t stream) {
  if (T == 0) return 0;
  if ((D % 8) || W > MAXW || (ldx % 8) || (ldy % 8)) return -2;
  const unsigned blocks = (unsigned)((T * (D / 8) + 255) / 256);
  if (silu)
    conv_fwd_kernel<true, true><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
                                                            (const __nv_bfloat16*)b, pos, (const __nv_bfloat16*)dy,
                                                            (__nv_bfloat16*)dpre, T, D, W, ldx, ldy);
  else
    conv_fwd_kernel<false, true><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
                                                             (const __nv_bfloat16*)b, pos, (const __nv_bfloat16*)dy,
                                                             (__nv_bfloat16*)dpre, T, D, W, ldx, ldy);
  int rc = fb::launch_ok("conv_fwd_kernel(dpre)");
  if (rc) return rc;
  const int strips = fb_short_conv_strips(T);
  const int rows_per_strip = (int)((T + strips - 1) / strips);
  dim3 grid((D / 8 + 63) / 64, strips);
  conv_bwd_kernel<<<grid, 64, 0, stream>>>((const __nv_bfloat16*)dpre, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
                                           pos, (__nv_bfloat16*)dx, part, T, D, W, ldx, ldy, rows_per_strip);
  rc = fb::launch_ok("conv_bwd_kernel");
  if (rc) return rc;
  conv_reduce_kernel<<<(D * (W + 1) + 255) / 256, 256, 0, stream>>>(part, strips, D, W, dw, db, accumulate);
  return fb::launch_ok("conv_reduce_kernel");
}

}  // extern "C"
