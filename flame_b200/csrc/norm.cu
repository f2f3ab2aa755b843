// Fused RMSNorm (+ residual add) forward and backward, and the gated variant used by the linear-attention
// layers.  Bandwidth-bound: one warp owns a row, 16-byte loads, fp32 math, a single pass over HBM
// (the second sweep over the row hits L1).
//
//   forward :  r = x (+ residual_in);  y = r * rsqrt(mean(r^2) + eps) * w;   optionally writes r and rstd
//   backward:  dx = rstd * (dy*w - xhat * mean(dy*w*xhat)) (+ d_residual);   dw = sum_rows dy * xhat
//
// Semantics follow fla/modules/layernorm.py:1084-1134 (RMSNorm with prenorm residual) and
// fla/modules/fused_norm_gate.py:992 (norm(x) * w * g * sigmoid(g)); the row-parallel design, the fixed-order
// two-stage dw reduction and the fused residual-gradient add are this library's own.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include "host_utils.cuh"
#include "flame_b200_noalloc.h"

namespace {

constexpr int WARPS = 8;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
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

// gate_mode: 0 none, 1 swish (g * sigmoid(g)), 2 sigmoid
template <bool HAS_RES, bool WRITE_RES, int GATE>
__global__ void __launch_bounds__(WARPS * 32)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res_in,
                   const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ gate,
                   __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ res_out, float* __restrict__ rstd,
                   long long rows, int D, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * WARPS + warp;
  if (row >= rows) return;
  const int nvec = D >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * D);
  const uint4* rr = HAS_RES ? reinterpret_cast<const uint4*>(res_in + row * D) : nullptr;
  uint4* ro = WRITE_RES ? reinterpret_cast<uint4*>(res_out + row * D) : nullptr;
  float ss = 0.f;
  for (int i = lane; i < nvec; i += 32) {
    float a[8];
    unpack8(xr[i], a);
    if (HAS_RES) {
      float b[8];
      unpack8(rr[i], b);
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] += b[j];
    }
    if (WRITE_RES) {
      uint4 q = pack8(a);
      ro[i] = q;
      unpack8(q, a);  // normalise what was stored, so backward sees identical values
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += a[j] * a[j];
  }
  ss = warp_sum(ss);
  const float rs = rsqrtf(ss / (float)D + eps);
  if (lane == 0 && rstd != nullptr) rstd[row] = rs;
  const uint4* src = WRITE_RES ? reinterpret_cast<const uint4*>(res_out + row * D) : xr;
  const uint4* wv = reinterpret_cast<const uint4*>(w);
  const uint4* gv = GATE ? reinterpret_cast<const uint4*>(gate + row * D) : nullptr;
  uint4* yo = reinterpret_cast<uint4*>(y + row * D);
  for (int i = lane; i < nvec; i += 32) {
    float a[8], ww[8];
    unpack8(src[i], a);
    if (HAS_RES && !WRITE_RES) {
      float b[8];
      unpack8(rr[i], b);
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] += b[j];
    }
    if (w != nullptr) unpack8(wv[i], ww);
    float o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = a[j] * rs * (w != nullptr ? ww[j] : 1.f);
    if (GATE) {
      float g[8];
      unpack8(gv[i], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] *= (GATE == 1) ? g[j] * sigmoidf_(g[j]) : sigmoidf_(g[j]);
    }
    yo[i] = pack8(o);
  }
}

__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// Backward.  `xin` is the tensor that was normalised (the stored residual sum when a residual was fused).
// dw partials: each CTA reduces its rows into dw_part[blockIdx.x, :]; a second kernel sums the CTAs in order.
template <bool HAS_DRES, int GATE, int NITER>
__global__ void __launch_bounds__(WARPS * 32, 2)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ xin,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                   const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ dres,
                   __nv_bfloat16* __restrict__ dx, __nv_bfloat16* __restrict__ dgate, float* __restrict__ dw_part,
                   long long rows, int D, int rows_per_cta) {
  extern __shared__ float s_dw_all[];  // [WARPS][D]: every warp owns a private row, so no atomics and a fixed order
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = D >> 3;
  float* s_dw = s_dw_all + (size_t)warp * D;
  for (int i = threadIdx.x; i < WARPS * D; i += blockDim.x) s_dw_all[i] = 0.f;
  __syncthreads();
  const long long row0 = (long long)blockIdx.x * rows_per_cta;
  const long long row1 = min(rows, row0 + rows_per_cta);
  const uint4* wv = reinterpret_cast<const uint4*>(w);
  // NITER > 0: D == 256 * NITER and each lane keeps its dw columns in registers across all of its rows
  float dw_reg[NITER > 0 ? NITER : 1][8];
#pragma unroll
  for (int a = 0; a < (NITER > 0 ? NITER : 1); ++a)
#pragma unroll
    for (int j = 0; j < 8; ++j) dw_reg[a][j] = 0.f;
  if constexpr (NITER > 0) {
    // D == 256 * NITER: a lane owns NITER vectors of 8 columns.  x, dy (and the residual gradient, the gate) of a row are
    // read ONCE and stay in registers as packed bf16 for both passes, so a row costs one round trip and half the L1
    // traffic of re-reading; only the 2 KB weight vector is re-read (L1 resident).
    for (long long row = row0 + warp; row < row1; row += WARPS) {
      const uint4* dyr = reinterpret_cast<const uint4*>(dy + row * D);
      const uint4* xr = reinterpret_cast<const uint4*>(xin + row * D);
      uint4 xa[NITER], ga[NITER], ra[HAS_DRES ? NITER : 1], ta[GATE ? NITER : 1];
#pragma unroll
      for (int it = 0; it < NITER; ++it) {
        // streaming loads: every operand row is read exactly once, so it should not displace the weight vector in L1
        xa[it] = __ldcs(&xr[lane + it * 32]);
        ga[it] = __ldcs(&dyr[lane + it * 32]);
        if (HAS_DRES) ra[it] = __ldcs(&reinterpret_cast<const uint4*>(dres + row * D)[lane + it * 32]);
        if (GATE) ta[it] = __ldcs(&reinterpret_cast<const uint4*>(gate + row * D)[lane + it * 32]);
      }
      const float rs = rstd[row];
      float c = 0.f;
#pragma unroll
      for (int it = 0; it < NITER; ++it) {
        float a[8], g[8], ww[8];
        unpack8(xa[it], a);
        unpack8(ga[it], g);
        if (w != nullptr) unpack8(wv[lane + it * 32], ww);
        if (GATE) {
          float gt[8];
          unpack8(ta[it], gt);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float sg = sigmoidf_(gt[j]);
            g[j] *= (GATE == 1) ? gt[j] * sg : sg;
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) c += g[j] * (w != nullptr ? ww[j] : 1.f) * a[j] * rs;
      }
      c = warp_sum(c) / (float)D;
      // keep the compiler from carrying the unpacked fp32 values of the first pass (twice the registers) into the second
#pragma unroll
      for (int it = 0; it < NITER; ++it) {
        asm volatile("" : "+r"(xa[it].x), "+r"(xa[it].y), "+r"(xa[it].z), "+r"(xa[it].w));
        asm volatile("" : "+r"(ga[it].x), "+r"(ga[it].y), "+r"(ga[it].z), "+r"(ga[it].w));
      }
      uint4* dxr = reinterpret_cast<uint4*>(dx + row * D);
      uint4* dgr = GATE ? reinterpret_cast<uint4*>(dgate + row * D) : nullptr;
#pragma unroll
      for (int it = 0; it < NITER; ++it) {
        float a[8], g[8], ww[8], o[8], gt[8], dgo[8];
        unpack8(xa[it], a);
        unpack8(ga[it], g);
        if (w != nullptr) unpack8(wv[lane + it * 32], ww);
        if (GATE) unpack8(ta[it], gt);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xhat = a[j] * rs;
          const float wj = (w != nullptr ? ww[j] : 1.f);
          float gy = g[j];
          if (GATE) {
            const float sg = sigmoidf_(gt[j]);
            const float act = (GATE == 1) ? gt[j] * sg : sg;
            const float dact = (GATE == 1) ? sg * (1.f + gt[j] * (1.f - sg)) : sg * (1.f - sg);
            dgo[j] = g[j] * xhat * wj * dact;
            gy = g[j] * act;
          }
          o[j] = rs * (gy * wj - xhat * c);
          if (w != nullptr) dw_reg[it][j] += gy * xhat;
        }
        if (HAS_DRES) {
          float b[8];
          unpack8(ra[it], b);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += b[j];
        }
        __stcs(&dxr[lane + it * 32], pack8(o));
        if (GATE) __stcs(&dgr[lane + it * 32], pack8(dgo));
      }
    }
  } else {
    for (long long row = row0 + warp; row < row1; row += WARPS) {
      const uint4* dyr = reinterpret_cast<const uint4*>(dy + row * D);
      const uint4* xr = reinterpret_cast<const uint4*>(xin + row * D);
      const uint4* gr = GATE ? reinterpret_cast<const uint4*>(gate + row * D) : nullptr;
      if (row + WARPS < row1) {
        // pull this warp's NEXT row into L2 while the current one is processed: the row's two passes then see cache latency
        const long long nrow = row + WARPS;
        for (int i = lane; i < nvec; i += 32) {
          prefetch_l2(dy + nrow * D + i * 8);
          prefetch_l2(xin + nrow * D + i * 8);
          if (HAS_DRES) prefetch_l2(dres + nrow * D + i * 8);
          if (GATE) prefetch_l2(gate + nrow * D + i * 8);
        }
      }
      const float rs = rstd[row];
      float c = 0.f;
      for (int i = lane; i < nvec; i += 32) {
        float a[8], g[8], ww[8];
        unpack8(xr[i], a);
        unpack8(dyr[i], g);
        if (w != nullptr) unpack8(wv[i], ww);
        if (GATE) {
          float gt[8];
          unpack8(gr[i], gt);
  #pragma unroll
          for (int j = 0; j < 8; ++j) {
            float s = sigmoidf_(gt[j]);
            g[j] *= (GATE == 1) ? gt[j] * s : s;
          }
        }
  #pragma unroll
        for (int j = 0; j < 8; ++j) c += g[j] * (w != nullptr ? ww[j] : 1.f) * a[j] * rs;
      }
      c = warp_sum(c) / (float)D;
      uint4* dxr = reinterpret_cast<uint4*>(dx + row * D);
      const uint4* drr = HAS_DRES ? reinterpret_cast<const uint4*>(dres + row * D) : nullptr;
      uint4* dgr = GATE ? reinterpret_cast<uint4*>(dgate + row * D) : nullptr;
  #pragma unroll
      for (int it = 0; it < (NITER > 0 ? NITER : 64); ++it) {
        const int i = lane + it * 32;
        if (NITER == 0 && i >= nvec) break;
        float a[8], g[8], ww[8], o[8];
        unpack8(xr[i], a);
        unpack8(dyr[i], g);
        if (w != nullptr) unpack8(wv[i], ww);
        float gt[8], dgo[8];
        if (GATE) unpack8(gr[i], gt);
  #pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xhat = a[j] * rs;
          const float wj = (w != nullptr ? ww[j] : 1.f);
          float gy = g[j];
          if (GATE) {
            const float s = sigmoidf_(gt[j]);
            const float act = (GATE == 1) ? gt[j] * s : s;
            const float dact = (GATE == 1) ? s * (1.f + gt[j] * (1.f - s)) : s * (1.f - s);
            dgo[j] = g[j] * xhat * wj * dact;
            gy = g[j] * act;
          }
          o[j] = rs * (gy * wj - xhat * c);
          if (w != nullptr) {
            if (NITER > 0) dw_reg[NITER > 0 ? it : 0][j] += gy * xhat;
            else s_dw[i * 8 + j] += gy * xhat;
          }
        }
        if (HAS_DRES) {
          float b[8];
          unpack8(drr[i], b);
  #pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += b[j];
        }
        dxr[i] = pack8(o);
        if (GATE) dgr[i] = pack8(dgo);
      }
    }
}
  if (NITER > 0 && w != nullptr) {
#pragma unroll
    for (int it = 0; it < (NITER > 0 ? NITER : 1); ++it)
#pragma unroll
      for (int j = 0; j < 8; ++j) s_dw[(lane + it * 32) * 8 + j] = dw_reg[it][j];
  }
  __syncthreads();
  if (w != nullptr)
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
      float t = 0.f;
#pragma unroll
      for (int k = 0; k < WARPS; ++k) t += s_dw_all[(size_t)k * D + i];
      dw_part[(long long)blockIdx.x * D + i] = t;
    }
}

__global__ void colsum_partials_kernel(const float* __restrict__ part, int nparts, int D, float* __restrict__ out,
                                       int accumulate) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= D) return;
  float s = 0.f;
  for (int p = 0; p < nparts; ++p) s += part[(long long)p * D + i];
  out[i] = accumulate ? out[i] + s : s;
}

}  // namespace

extern "C" {

// Number of CTAs (= rows of the dw partial buffer) the backward launches for `rows` rows.
int fb_rmsnorm_bwd_parts(long long rows) {
  long long want = (rows + WARPS - 1) / WARPS;
  return (int)(want < 592 ? (want < 1 ? 1 : want) : 592);  // two resident CTAs on each of 148 SMs: two full waves
}

int fb_rmsnorm_fwd(const void* x, const void* res_in, const void* w, const void* gate, void* y, void* res_out,
                   float* rstd, long long rows, int D, float eps, int gate_mode, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (D % 8) return -2;
  const unsigned grid = (unsigned)((rows + WARPS - 1) / WARPS);
  const auto X = (const __nv_bfloat16*)x;
  const auto R = (const __nv_bfloat16*)res_in;
  const auto W = (const __nv_bfloat16*)w;
  const auto G = (const __nv_bfloat16*)gate;
  auto Y = (__nv_bfloat16*)y;
  auto RO = (__nv_bfloat16*)res_out;
#define FWD(HR, WR, GM) \
  rmsnorm_fwd_kernel<HR, WR, GM><<<grid, WARPS * 32, 0, stream>>>(X, R, W, G, Y, RO, rstd, rows, D, eps)
  if (gate_mode == 0) {
    if (res_in && res_out) FWD(true, true, 0);
    else if (res_in) FWD(true, false, 0);
    else FWD(false, false, 0);
  } else if (gate_mode == 1) {
    FWD(false, false, 1);
  } else {
    FWD(false, false, 2);
  }
#undef FWD
  return fb::launch_ok("rmsnorm_fwd_kernel");
}

// dw_part: fp32 [fb_rmsnorm_bwd_parts(rows), D] scratch; dw: fp32 [D] (accumulated when accumulate_dw != 0).
int fb_rmsnorm_bwd(const void* dy, const void* xin, const void* w, const float* rstd, const void* gate,
                   const void* dres, void* dx, void* dgate, float* dw_part, float* dw, long long rows, int D,
                   int gate_mode, int accumulate_dw, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (D % 8) return -2;
  const int parts = fb_rmsnorm_bwd_parts(rows);
  const int rows_per_cta = (int)((rows + parts - 1) / parts);
  const size_t smem = (size_t)WARPS * D * sizeof(float);
  if (smem > 220 * 1024) return -3;
#define BWD_N(HD, GM, NI)                                                                                         \
  do {                                                                                                            \
    if (smem > 48 * 1024)                                                                                         \
      cudaFuncSetAttribute(rmsnorm_bwd_kernel<HD, GM, NI>, cudaFuncAttributeMaxDynamicSharedMemorySize,           \
                           (int)smem);                                                                            \
    rmsnorm_bwd_kernel<HD, GM, NI><<<parts, WARPS * 32, smem, stream>>>(                                          \
        (const __nv_bfloat16*)dy, (const __nv_bfloat16*)xin, (const __nv_bfloat16*)w, rstd,                       \
        (const __nv_bfloat16*)gate, (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, (__nv_bfloat16*)dgate,        \
        dw_part, rows, D, rows_per_cta);                                                                          \
  } while (0)
#define BWD(HD, GM)                                                                                               \
  do {                                                                                                            \
    if (D == 256) BWD_N(HD, GM, 1);                                                                               \
    else if (D == 512) BWD_N(HD, GM, 2);                                                                          \
    else if (D == 1024) BWD_N(HD, GM, 4);                                                                         \
    else if (D == 2048) BWD_N(HD, GM, 0); /* eight vectors per lane would spill */                                \
    else BWD_N(HD, GM, 0);                                                                                        \
  } while (0)
  if (gate_mode == 0) {
    if (dres) { BWD(true, 0); } else { BWD(false, 0); }
  } else if (gate_mode == 1) {
    BWD(false, 1);
  } else {
    BWD(false, 2);
  }
#undef BWD
#undef BWD_N
  int rc = fb::launch_ok("rmsnorm_bwd_kernel");
  if (rc) return rc;
  if (w != nullptr) {
    colsum_partials_kernel<<<(D + 255) / 256, 256, 0, stream>>>(dw_part, parts, D, dw, accumulate_dw);
    rc = fb::launch_ok("colsum_partials_kernel");
  }
  return rc;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// Allocation-free variant (declared in flame_b200_noalloc.h)
// ------------------------------------------------------------------------------------------------
namespace {
constexpr int kNoAllocParts = 592;   // upper bound of fb_rmsnorm_bwd_parts()
constexpr int kNoAllocMaxDevices = 64;
// Scratch for the per-CTA dw partial sums.  In host code this name is only a stand-in for the symbol; the
// address a kernel can use is obtained once per device with cudaGetSymbolAddress below.
static __device__ __align__(256) float g_noalloc_dw_part[(size_t)kNoAllocParts * FB_NOALLOC_MAX_D];
static float* g_noalloc_dw_part_addr[kNoAllocMaxDevices] = {nullptr};
}  // namespace

extern "C" int fb_rmsnorm_bwd_noalloc(const void* dy, const void* xin, const void* w, const float* rstd, void* dx,
                                      float* dw, long long rows, int D, int accumulate_dw, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (D <= 0 || (D % 8) != 0) {
    fprintf(stderr, "[flame_b200] fb_rmsnorm_bwd_noalloc: D=%d must be a positive multiple of 8\n", D);
    return -2;
  }
  if (D > FB_NOALLOC_MAX_D) {
    fprintf(stderr,
            "[flame_b200] fb_rmsnorm_bwd_noalloc: D=%d exceeds the built-in scratch (max D = %d); use fb_rmsnorm_bwd "
            "with caller-provided scratch instead\n", D, FB_NOALLOC_MAX_D);
    return -3;
  }
  if (w == nullptr || dw == nullptr) {
    fprintf(stderr, "[flame_b200] fb_rmsnorm_bwd_noalloc: w and dw are required\n");
    return -4;
  }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kNoAllocMaxDevices) {
    fprintf(stderr, "[flame_b200] fb_rmsnorm_bwd_noalloc: cannot identify the current device\n");
    return -5;
  }
  if (g_noalloc_dw_part_addr[dev] == nullptr) {
    // one-time set-up for this device, with this device current
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_dw_part);
    if (e != cudaSuccess || p == nullptr) {
      fprintf(stderr, "[flame_b200] fb_rmsnorm_bwd_noalloc: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(e));
      return (int)(e != cudaSuccess ? e : cudaErrorInvalidSymbol);
    }
    g_noalloc_dw_part_addr[dev] = p;
  }
  // same kernels and launch shape as fb_rmsnorm_bwd; only the origin of the scratch differs
  return fb_rmsnorm_bwd(dy, xin, w, rstd, nullptr, nullptr, dx, nullptr, g_noalloc_dw_part_addr[dev], dw, rows, D, 0,
                        accumulate_dw, stream);
}

