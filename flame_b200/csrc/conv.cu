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

// Width-specialised forward (and dpre) kernel: a thread owns 8 channels and walks a strip of consecutive tokens with the
// last W-1 inputs in registers, so every input row is read once and the taps are read once per strip.
// grid = (channel vectors / 64, strips of `rows` tokens).
template <bool SILU, bool WRITE_DPRE, int W>
__global__ void __launch_bounds__(64) conv_strip_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                        const __nv_bfloat16* __restrict__ b, const int* __restrict__ pos,
                                                        const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ out,
                                                        long long T, int D, long long ldx, long long ldo, int rows) {
  const int v = blockIdx.x * 64 + threadIdx.x;
  if (v >= (D >> 3)) return;
  const int d0 = v * 8;
  const long long r0 = (long long)blockIdx.y * rows;
  const long long r1 = min(T, r0 + rows);
  float wv[W][8], bias[8], win[W > 1 ? W - 1 : 1][8];
#pragma unroll
  for (int j = 0; j < W; ++j)
#pragma unroll
    for (int c = 0; c < 8; ++c) wv[j][c] = __bfloat162float(w[(d0 + c) * W + (W - 1 - j)]);  // tap at distance j
#pragma unroll
  for (int c = 0; c < 8; ++c) bias[c] = b ? __bfloat162float(b[d0 + c]) : 0.f;
#pragma unroll
  for (int j = 1; j < W; ++j) {
    if (r0 - j >= 0) {
      unpack8(*reinterpret_cast<const uint4*>(x + (r0 - j) * ldx + d0), win[j - 1]);
    } else {
#pragma unroll
      for (int c = 0; c < 8; ++c) win[j - 1][c] = 0.f;
    }
  }
#pragma unroll 4
  for (long long t = r0; t < r1; ++t) {
    float xc[8], acc[8];
    unpack8(*reinterpret_cast<const uint4*>(x + t * ldx + d0), xc);
    const int p = pos[t];
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[c] = fmaf(wv[0][c], xc[c], bias[c]);
#pragma unroll
    for (int j = 1; j < W; ++j) {
      if (j <= p) {
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[c] = fmaf(wv[j][c], win[j - 1][c], acc[c]);
      }
    }
#pragma unroll
    for (int j = W - 2; j >= 1; --j)
#pragma unroll
      for (int c = 0; c < 8; ++c) win[j][c] = win[j - 1][c];
    if (W > 1) {
#pragma unroll
      for (int c = 0; c < 8; ++c) win[0][c] = xc[c];
    }
    float o[8];
    if (WRITE_DPRE) {
      float g[8];
      unpack8(*reinterpret_cast<const uint4*>(dy + t * ldo + d0), g);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        if (SILU) {
          const float sg = sigmoidf_(acc[c]);
          o[c] = g[c] * sg * (1.f + acc[c] * (1.f - sg));
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
}

template <bool SILU, bool WRITE_DPRE>
int launch_conv_point(const void* x, const void* w, const void* b, const int* pos, const void* dy, void* out, long long T, int D,
                      int W, long long ldx, long long ldo, cudaStream_t stream) {
  const __nv_bfloat16 *xx = (const __nv_bfloat16*)x, *ww = (const __nv_bfloat16*)w, *bb = (const __nv_bfloat16*)b,
                      *gg = (const __nv_bfloat16*)dy;
  __nv_bfloat16* oo = (__nv_bfloat16*)out;
  if (W == 4 || W == 2 || W == 3) {
    const int rows = 32;
    dim3 grid((D / 8 + 63) / 64, (unsigned)((T + rows - 1) / rows));
    if (W == 4) conv_strip_kernel<SILU, WRITE_DPRE, 4><<<grid, 64, 0, stream>>>(xx, ww, bb, pos, gg, oo, T, D, ldx, ldo, rows);
    else if (W == 3) conv_strip_kernel<SILU, WRITE_DPRE, 3><<<grid, 64, 0, stream>>>(xx, ww, bb, pos, gg, oo, T, D, ldx, ldo, rows);
    else conv_strip_kernel<SILU, WRITE_DPRE, 2><<<grid, 64, 0, stream>>>(xx, ww, bb, pos, gg, oo, T, D, ldx, ldo, rows);
    return fb::launch_ok("conv_strip_kernel");
  }
  const unsigned blocks = (unsigned)((T * (D / 8) + 255) / 256);
  conv_fwd_kernel<SILU, WRITE_DPRE><<<blocks, 256, 0, stream>>>(xx, ww, bb, pos, gg, oo, T, D, W, ldx, ldo);
  return fb::launch_ok("conv_fwd_kernel");
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

// Width-specialised backward: one pass over the strip with register windows of the last W inputs (for dw) and the last W
// dpre rows (for dx, written W-1 rows behind the read position), so dpre and x are each read once.
template <int W>
__global__ void __launch_bounds__(64) conv_bwd_strip_kernel(const __nv_bfloat16* __restrict__ dpre, const __nv_bfloat16* __restrict__ x,
                                                            const __nv_bfloat16* __restrict__ w, const int* __restrict__ pos,
                                                            __nv_bfloat16* __restrict__ dx, float* __restrict__ part, long long T,
                                                            int D, long long ldx, long long ldd, int rows_per_strip) {
  const int v = blockIdx.x * 64 + threadIdx.x;
  if (v >= (D >> 3)) return;
  const int d0 = v * 8;
  const long long r0 = (long long)blockIdx.y * rows_per_strip;
  const long long r1 = min(T, r0 + rows_per_strip);
  float wv[W][8], dw[W][8], db[8], xwin[W][8], gwin[W][8];
  int pwin[W];
#pragma unroll
  for (int j = 0; j < W; ++j) {
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      wv[j][c] = __bfloat162float(w[(d0 + c) * W + (W - 1 - j)]);  // tap at distance j
      dw[j][c] = 0.f;
      gwin[j][c] = 0.f;
    }
    pwin[j] = -1;
  }
#pragma unroll
  for (int c = 0; c < 8; ++c) db[c] = 0.f;
  // xwin[j] = x[u - j] at the top of iteration u (xwin[0] is loaded inside)
#pragma unroll
  for (int j = 1; j < W; ++j) {
    if (r0 - j >= 0) {
      unpack8(*reinterpret_cast<const uint4*>(x + (r0 - j) * ldx + d0), xwin[j]);
    } else {
#pragma unroll
      for (int c = 0; c < 8; ++c) xwin[j][c] = 0.f;
    }
  }
  const long long u_end = r1 + (W - 1);
  // Four rows per trip: their dpre / x / position loads are issued together before any of them is used, so a thread
  // keeps eight 16-byte loads in flight instead of two (the walk is serial per thread and latency-bound otherwise).
  for (long long ub = r0; ub < u_end; ub += 4) {
    uint4 gq[4], xq[4];
    int pq[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const long long u = ub + i;
      const bool in_t = u < T && u < u_end;
      gq[i] = in_t ? *reinterpret_cast<const uint4*>(dpre + u * ldd + d0) : make_uint4(0, 0, 0, 0);
      pq[i] = in_t ? pos[u] : -1;
      xq[i] = u < r1 ? *reinterpret_cast<const uint4*>(x + u * ldx + d0) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const long long u = ub + i;
      if (u >= u_end) break;
      // shift the dpre / position windows and take row u (zero / invalid past the end of the tensor)
#pragma unroll
      for (int j = W - 1; j >= 1; --j) {
#pragma unroll
        for (int c = 0; c < 8; ++c) gwin[j][c] = gwin[j - 1][c];
        pwin[j] = pwin[j - 1];
      }
      unpack8(gq[i], gwin[0]);
      pwin[0] = pq[i];
      if (u < r1) {
        // weight / bias gradients of row u: dw[tap j] += dpre[u] * x[u - j]
        unpack8(xq[i], xwin[0]);
#pragma unroll
        for (int c = 0; c < 8; ++c) db[c] += gwin[0][c];
#pragma unroll
        for (int j = 0; j < W; ++j) {
          if (j <= pwin[0]) {
#pragma unroll
            for (int c = 0; c < 8; ++c) dw[j][c] = fmaf(gwin[0][c], xwin[j][c], dw[j][c]);
          }
        }
#pragma unroll
        for (int j = W - 1; j >= 1; --j)
#pragma unroll
          for (int c = 0; c < 8; ++c) xwin[j][c] = xwin[j - 1][c];
      }
      // input gradient of row s = u - (W-1): dx[s] = sum_j w[tap j] dpre[s + j] while s + j stays in the same document
      const long long srow = u - (W - 1);
      if (srow >= r0) {
        float acc[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[c] = wv[0][c] * gwin[W - 1][c];
        bool alive = true;
#pragma unroll
        for (int j = 1; j < W; ++j) {
          alive = alive && (pwin[W - 1 - j] >= j);  // row s + j exists and is at least j tokens into the same document
          if (alive) {
#pragma unroll
            for (int c = 0; c < 8; ++c) acc[c] = fmaf(wv[j][c], gwin[W - 1 - j][c], acc[c]);
          }
        }
        *reinterpret_cast<uint4*>(dx + srow * ldx + d0) = pack8(acc);
      }
    }
  }
  float* dst = part + ((long long)blockIdx.y * D + d0) * (W + 1);
#pragma unroll
  for (int c = 0; c < 8; ++c) {
#pragma unroll
    for (int j = 0; j < W; ++j) dst[c * (W + 1) + (W - 1 - j)] = dw[j][c];
    dst[c * (W + 1) + W] = db[c];
  }
}

// Sums the per-strip partials in a fixed order: a block of 32 outputs x 8 strip groups reads coalesced rows of partials.
__global__ void conv_reduce_kernel(const float* __restrict__ part, int strips, int D, int W, float* __restrict__ dw,
                                   float* __restrict__ db, int accumulate) {
  __shared__ float red[8][32];
  const int n = D * (W + 1);
  const int ix = threadIdx.x & 31, ky = threadIdx.x >> 5;
  const int i = blockIdx.x * 32 + ix;
  float s = 0.f;
  if (i < n)
    for (int k = ky; k < strips; k += 8) s += part[(long long)k * n + i];
  red[ky][ix] = s;
  __syncthreads();
  if (ky != 0 || i >= n) return;
#pragma unroll
  for (int k = 1; k < 8; ++k) s += red[k][ix];
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

// 64-row strips: the backward walks a strip serially per thread, so the strip count is what gives it parallelism
// (65,536 tokens x 1024 channels -> 1024 strips x 128 threads)
int fb_short_conv_strips(long long T) {
  long long s = (T + 63) / 64;
  return (int)(s < 1 ? 1 : (s > 2048 ? 2048 : s));
}

int fb_short_conv_fwd(const void* x, const void* w, const void* b, const int* pos, void* y, long long T, int D, int W,
                      long long ldx, long long ldy, int silu, cudaStream_t stream) {
  if (T == 0) return 0;
  if ((D % 8) || W > MAXW || (ldx % 8) || (ldy % 8)) return -2;
  return silu ? launch_conv_point<true, false>(x, w, b, pos, nullptr, y, T, D, W, ldx, ldy, stream)
              : launch_conv_point<false, false>(x, w, b, pos, nullptr, y, T, D, W, ldx, ldy, stream);
}

// dpre: bf16 [T, D] scratch; part: fp32 [fb_short_conv_strips(T), D, W + 1] scratch; dw: fp32 [D, W]; db: fp32 [D] or null
int fb_short_conv_bwd(const void* dy, const void* x, const void* w, const void* b, const int* pos, void* dx, void* dpre,
                      float* part, float* dw, float* db, long long T, int D, int W, long long ldx, long long ldy, int silu,
                      int accumulate, cudaStream_t stream) {
  if (T == 0) return 0;
  if ((D % 8) || W > MAXW || (ldx % 8) || (ldy % 8)) return -2;
  int rc = silu ? launch_conv_point<true, true>(x, w, b, pos, dy, dpre, T, D, W, ldx, ldy, stream)
                : launch_conv_point<false, true>(x, w, b, pos, dy, dpre, T, D, W, ldx, ldy, stream);
  if (rc) return rc;
  const int strips = fb_short_conv_strips(T);
  const int rows_per_strip = (int)((T + strips - 1) / strips);
  dim3 grid((D / 8 + 63) / 64, strips);
  if (W == 4)
    conv_bwd_strip_kernel<4><<<grid, 64, 0, stream>>>((const __nv_bfloat16*)dpre, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
                                                      pos, (__nv_bfloat16*)dx, part, T, D, ldx, ldy, rows_per_strip);
  else
    conv_bwd_kernel<<<grid, 64, 0, stream>>>((const __nv_bfloat16*)dpre, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
                                             pos, (__nv_bfloat16*)dx, part, T, D, W, ldx, ldy, rows_per_strip);
  rc = fb::launch_ok("conv_bwd_kernel");
  if (rc) return rc;
  conv_reduce_kernel<<<(D * (W + 1) + 31) / 32, 256, 0, stream>>>(part, strips, D, W, dw, db, accumulate);
  return fb::launch_ok("conv_reduce_kernel");
}

}  // extern "C"
