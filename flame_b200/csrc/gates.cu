// Fused gate arithmetic of the linear-attention layers: what the reference leaves to a chain of elementwise framework
// kernels (ten passes forward, fifteen backward over [tokens, hidden] fp32 tensors for HGRN2), one pass each way.
//
// HGRN2 (fla/layers/hgrn2.py:160-190):
//   q = silu(q_raw)
//   g = logsigmoid(f_raw)                                        (no lower bound)
//   g = log(lb + (1 - lb) sigmoid(f_raw))                        (with a per-channel lower bound lb in (0, 1))
//   k = 1 - exp(g)
// Outputs: q, k in bf16, g in fp32 (the log decay the chunk kernels consume).  The backward takes dq, dk (bf16) and dg
// (fp32), recomputes the gate from f_raw and returns dq_raw, df_raw and the per-channel sum of dlb.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "host_utils.cuh"

namespace {

__device__ __forceinline__ void unpack8(const uint4& q, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __bfloat1622float2(h[i]);
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
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
// log(sigmoid(x)) without cancellation or underflow
__device__ __forceinline__ float logsigmoidf_(float x) { return fminf(x, 0.f) - log1pf(__expf(-fabsf(x))); }

// one thread per (row, 8 channels)
template <bool HAS_LB>
__global__ void hgrn2_gate_fwd_kernel(const __nv_bfloat16* __restrict__ qr, const __nv_bfloat16* __restrict__ fr,
                                      const float* __restrict__ lb, __nv_bfloat16* __restrict__ q,
                                      __nv_bfloat16* __restrict__ k, float* __restrict__ g, long long rows, int D) {
  const int vecs = D >> 3;
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long row = gid / vecs;
  if (row >= rows) return;
  const int d0 = (int)(gid - row * vecs) * 8;
  const long long off = row * D + d0;
  float a[8], f[8], qo[8], ko[8], go[8];
  unpack8(*reinterpret_cast<const uint4*>(qr + off), a);
  unpack8(*reinterpret_cast<const uint4*>(fr + off), f);
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    qo[c] = a[c] * sigmoidf_(a[c]);
    float gs = logsigmoidf_(f[c]);
    if (HAS_LB) {
      const float l = lb[d0 + c];
      gs = __logf(l + (1.f - l) * __expf(gs));
    }
    go[c] = gs;
    ko[c] = 1.f - __expf(gs);
  }
  *reinterpret_cast<uint4*>(q + off) = pack8(qo);
  *reinterpret_cast<uint4*>(k + off) = pack8(ko);
  *reinterpret_cast<float4*>(g + off) = make_float4(go[0], go[1], go[2], go[3]);
  *reinterpret_cast<float4*>(g + off + 4) = make_float4(go[4], go[5], go[6], go[7]);
}

constexpr int GATE_TILE_ROWS = 64;  // rows per block of the backward; a block covers 256 channels

// block = 32 channel vectors x 8 row lanes; a block walks 64 rows and leaves one partial row of dlb sums
template <bool HAS_LB>
__global__ void __launch_bounds__(256)
hgrn2_gate_bwd_kernel(const __nv_bfloat16* __restrict__ qr, const __nv_bfloat16* __restrict__ fr, const float* __restrict__ lb,
                      const __nv_bfloat16* __restrict__ dq, const __nv_bfloat16* __restrict__ dk, const float* __restrict__ dg,
                      __nv_bfloat16* __restrict__ dqr, __nv_bfloat16* __restrict__ dfr, float* __restrict__ dlb_part,
                      long long rows, int D) {
  __shared__ float red[8][256];
  const int vx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int d0 = (blockIdx.x * 32 + vx) * 8;
  const bool col_ok = d0 < D;
  const long long r0 = (long long)blockIdx.y * GATE_TILE_ROWS;
  float lbv[8], acc[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    lbv[c] = (HAS_LB && col_ok) ? lb[d0 + c] : 0.f;
    acc[c] = 0.f;
  }
  if (col_ok) {
#pragma unroll 2
    for (int i = ry; i < GATE_TILE_ROWS; i += 8) {
      const long long row = r0 + i;
      if (row >= rows) break;
      const long long off = row * D + d0;
      float a[8], f[8], gq[8], gk[8], gg[8], oq[8], of[8];
      unpack8(*reinterpret_cast<const uint4*>(qr + off), a);
      unpack8(*reinterpret_cast<const uint4*>(fr + off), f);
      unpack8(*reinterpret_cast<const uint4*>(dq + off), gq);
      unpack8(*reinterpret_cast<const uint4*>(dk + off), gk);
      const float4 g0 = *reinterpret_cast<const float4*>(dg + off), g1 = *reinterpret_cast<const float4*>(dg + off + 4);
      gg[0] = g0.x; gg[1] = g0.y; gg[2] = g0.z; gg[3] = g0.w;
      gg[4] = g1.x; gg[5] = g1.y; gg[6] = g1.z; gg[7] = g1.w;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const float sq = sigmoidf_(a[c]);
        oq[c] = gq[c] * sq * (1.f + a[c] * (1.f - sq));
        const float s = sigmoidf_(f[c]);
        if (HAS_LB) {
          const float l = lbv[c];
          const float e = l + (1.f - l) * s;           // exp(g), at least l > 0
          const float de = gg[c] / e - gk[c];          // g = log e, k = 1 - e
          of[c] = de * (1.f - l) * s * (1.f - s);
          acc[c] += de * (1.f - s);
        } else {
          // e = s: dg / s * s (1 - s) = dg (1 - s), which stays finite where s underflows
          of[c] = (gg[c] - gk[c] * s) * (1.f - s);
        }
      }
      *reinterpret_cast<uint4*>(dqr + off) = pack8(oq);
      *reinterpret_cast<uint4*>(dfr + off) = pack8(of);
    }
  }
  if (!HAS_LB) return;
#pragma unroll
  for (int c = 0; c < 8; ++c) red[ry][vx * 8 + c] = acc[c];
  __syncthreads();
  const int ch = threadIdx.x;  // one of the block's 256 channels
  const int d = blockIdx.x * 256 + ch;
  if (d < D) {
    float s = 0.f;
#pragma unroll
    for (int y = 0; y < 8; ++y) s += red[y][ch];
    dlb_part[(long long)blockIdx.y * D + d] = s;
  }
}

// out[d] = sum over `parts` partial rows, in a fixed order; block = 32 channels x 8 part lanes
__global__ void colsum_rows_kernel(const float* __restrict__ part, int parts, int D, float* __restrict__ out) {
  __shared__ float red[8][32];
  const int ix = threadIdx.x & 31, ky = threadIdx.x >> 5;
  const int d = blockIdx.x * 32 + ix;
  float s = 0.f;
  if (d < D)
    for (int k = ky; k < parts; k += 8) s += part[(long long)k * D + d];
  red[ky][ix] = s;
  __syncthreads();
  if (ky != 0 || d >= D) return;
#pragma unroll
  for (int k = 1; k < 8; ++k) s += red[k][ix];
  out[d] = s;
}

// ---------------------------------------------------------------------------------------------------------------
// Mamba2 (fla/layers/mamba2.py:241-331): the elementwise work around the SSD core, H heads of P channels.
//   pre :  dt = softplus(dt_raw + dt_bias),  g = -exp(A_log) dt,  xv = x dt                 (x, dt_raw: strided views)
//   post:  out = (y + D x) silu(z)                                                           (z: strided view)
// A thread owns 8 channels of one token; the P / 8 threads of a head reduce over the head with shuffles.
__device__ __forceinline__ float softplusf_(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

template <int LANES>  // LANES = P / 8 threads per head: 8, 16 or 32
__global__ void mamba2_pre_fwd_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const __nv_bfloat16* __restrict__ dt_raw,
                                      long long ld_dt, const float* __restrict__ dt_bias, const float* __restrict__ A_log,
                                      __nv_bfloat16* __restrict__ xv, float* __restrict__ dt_out, float* __restrict__ g_out,
                                      long long T, int H) {
  const int vecs = H * LANES;
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long t = gid / vecs;
  if (t >= T) return;
  const int v = (int)(gid - t * vecs);
  const int h = v / LANES;
  const float dt = softplusf_(__bfloat162float(dt_raw[t * ld_dt + h]) + dt_bias[h]);
  float a[8];
  unpack8(*reinterpret_cast<const uint4*>(x + t * ldx + v * 8), a);
#pragma unroll
  for (int c = 0; c < 8; ++c) a[c] *= dt;
  *reinterpret_cast<uint4*>(xv + (t * vecs + v) * 8) = pack8(a);
  if (v % LANES == 0) {
    dt_out[t * H + h] = dt;
    g_out[t * H + h] = -__expf(A_log[h]) * dt;
  }
}

// dx = dxv dt;  d_raw = (sum_p dxv x + dg A + ddt) sigmoid(dt_raw + bias)   (ddt: gradient reaching dt directly, may be null)
template <int LANES>
__global__ void mamba2_pre_bwd_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const __nv_bfloat16* __restrict__ dt_raw,
                                      long long ld_dt, const float* __restrict__ dt_bias, const float* __restrict__ A_log,
                                      const __nv_bfloat16* __restrict__ dxv, const float* __restrict__ dg,
                                      const float* __restrict__ ddt, __nv_bfloat16* __restrict__ dx, float* __restrict__ d_raw,
                                      long long T, int H) {
  const int vecs = H * LANES;
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long t = gid / vecs;
  const bool live = t < T;
  const int v = live ? (int)(gid - t * vecs) : 0;
  const int h = v / LANES;
  float part = 0.f, pre = 0.f;
  if (live) {
    pre = __bfloat162float(dt_raw[t * ld_dt + h]) + dt_bias[h];
    const float dt = softplusf_(pre);
    float a[8], g[8], o[8];
    unpack8(*reinterpret_cast<const uint4*>(x + t * ldx + v * 8), a);
    unpack8(*reinterpret_cast<const uint4*>(dxv + (t * vecs + v) * 8), g);
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      part = fmaf(g[c], a[c], part);
      o[c] = g[c] * dt;
    }
    *reinterpret_cast<uint4*>(dx + (t * vecs + v) * 8) = pack8(o);
  }
  // blockDim is a multiple of 32 and LANES divides 32, so a head's threads sit in one warp; dead threads add zero
#pragma unroll
  for (int o = LANES / 2; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
  if (live && v % LANES == 0) {
    float total = part + dg[t * H + h] * (-__expf(A_log[h]));
    if (ddt != nullptr) total += ddt[t * H + h];
    d_raw[t * H + h] = total * sigmoidf_(pre);
  }
}

template <int LANES>
__global__ void mamba2_post_fwd_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ x, long long ldx,
                                       const __nv_bfloat16* __restrict__ z, long long ldz, const float* __restrict__ D,
                                       __nv_bfloat16* __restrict__ out, long long T, int H) {
  const int vecs = H * LANES;
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long t = gid / vecs;
  if (t >= T) return;
  const int v = (int)(gid - t * vecs);
  const float d = D[v / LANES];
  float a[8], b[8], g[8], o[8];
  unpack8(*reinterpret_cast<const uint4*>(y + (t * vecs + v) * 8), a);
  unpack8(*reinterpret_cast<const uint4*>(x + t * ldx + v * 8), b);
  unpack8(*reinterpret_cast<const uint4*>(z + t * ldz + v * 8), g);
#pragma unroll
  for (int c = 0; c < 8; ++c) o[c] = fmaf(d, b[c], a[c]) * g[c] * sigmoidf_(g[c]);
  *reinterpret_cast<uint4*>(out + (t * vecs + v) * 8) = pack8(o);
}

// du = dout silu(z): dy = du, dx = du D, dz = dout (y + D x) silu'(z), dD_part[t, h] = sum_p du x
template <int LANES>
__global__ void mamba2_post_bwd_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ x, long long ldx,
                                       const __nv_bfloat16* __restrict__ z, long long ldz, const float* __restrict__ D,
                                       const __nv_bfloat16* __restrict__ dout, __nv_bfloat16* __restrict__ dy,
                                       __nv_bfloat16* __restrict__ dx, __nv_bfloat16* __restrict__ dz,
                                       float* __restrict__ dD_part, long long T, int H) {
  const int vecs = H * LANES;
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long t = gid / vecs;
  const bool live = t < T;
  const int v = live ? (int)(gid - t * vecs) : 0;
  const int h = v / LANES;
  float part = 0.f;
  if (live) {
    const float d = D[h];
    float a[8], b[8], g[8], go[8], oy[8], ox[8], oz[8];
    const long long off = (t * vecs + v) * 8;
    unpack8(*reinterpret_cast<const uint4*>(y + off), a);
    unpack8(*reinterpret_cast<const uint4*>(x + t * ldx + v * 8), b);
    unpack8(*reinterpret_cast<const uint4*>(z + t * ldz + v * 8), g);
    unpack8(*reinterpret_cast<const uint4*>(dout + off), go);
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const float sg = sigmoidf_(g[c]);
      const float du = go[c] * g[c] * sg;
      oy[c] = du;
      ox[c] = du * d;
      oz[c] = go[c] * fmaf(d, b[c], a[c]) * sg * (1.f + g[c] * (1.f - sg));
      part = fmaf(du, b[c], part);
    }
    *reinterpret_cast<uint4*>(dy + off) = pack8(oy);
    *reinterpret_cast<uint4*>(dx + off) = pack8(ox);
    *reinterpret_cast<uint4*>(dz + off) = pack8(oz);
  }
#pragma unroll
  for (int o = LANES / 2; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
  if (live && v % LANES == 0) dD_part[t * H + h] = part;
}

}  // namespace

extern "C" {

// x: bf16 [T, H * P] view with row stride ldx (elements); dt_raw: bf16 [T, H] view with row stride ld_dt; dt_bias, A_log: fp32 [H]
// xv: bf16 [T, H, P]; dt, g: fp32 [T, H].  P in {64, 128, 256}; ldx a multiple of 8, x 16-byte aligned.
int fb_mamba2_pre_fwd(const void* x, long long ldx, const void* dt_raw, long long ld_dt, const float* dt_bias, const float* A_log,
                      void* xv, float* dt, float* g, long long T, int H, int P, cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((P != 64 && P != 128 && P != 256) || (ldx % 8) || ((uintptr_t)x & 15)) return -2;
  const long long threads = T * H * (P / 8);
  const unsigned blocks = (unsigned)((threads + 255) / 256);
#define FB_PRE_FWD(L) mamba2_pre_fwd_kernel<L><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)dt_raw, \
      ld_dt, dt_bias, A_log, (__nv_bfloat16*)xv, dt, g, T, H)
  if (P == 64) FB_PRE_FWD(8); else if (P == 128) FB_PRE_FWD(16); else FB_PRE_FWD(32);
#undef FB_PRE_FWD
  return fb::launch_ok("mamba2_pre_fwd_kernel");
}

// dxv: bf16 [T, H, P]; dg: fp32 [T, H]; ddt: fp32 [T, H] or null; dx: bf16 [T, H, P]; d_raw: fp32 [T, H]
int fb_mamba2_pre_bwd(const void* x, long long ldx, const void* dt_raw, long long ld_dt, const float* dt_bias, const float* A_log,
                      const void* dxv, const float* dg, const float* ddt, void* dx, float* d_raw, long long T, int H, int P,
                      cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((P != 64 && P != 128 && P != 256) || (ldx % 8) || ((uintptr_t)x & 15)) return -2;
  const long long threads = T * H * (P / 8);
  const unsigned blocks = (unsigned)((threads + 255) / 256);
#define FB_PRE_BWD(L) mamba2_pre_bwd_kernel<L><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)dt_raw, \
      ld_dt, dt_bias, A_log, (const __nv_bfloat16*)dxv, dg, ddt, (__nv_bfloat16*)dx, d_raw, T, H)
  if (P == 64) FB_PRE_BWD(8); else if (P == 128) FB_PRE_BWD(16); else FB_PRE_BWD(32);
#undef FB_PRE_BWD
  return fb::launch_ok("mamba2_pre_bwd_kernel");
}

// y: bf16 [T, H, P]; x, z: bf16 views with row strides ldx / ldz; D: fp32 [H]; out: bf16 [T, H * P]
int fb_mamba2_post_fwd(const void* y, const void* x, long long ldx, const void* z, long long ldz, const float* D, void* out,
                       long long T, int H, int P, cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((P != 64 && P != 128 && P != 256) || (ldx % 8) || (ldz % 8) || ((uintptr_t)x & 15) || ((uintptr_t)z & 15)) return -2;
  const long long threads = T * H * (P / 8);
  const unsigned blocks = (unsigned)((threads + 255) / 256);
#define FB_POST_FWD(L) mamba2_post_fwd_kernel<L><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)y, (const __nv_bfloat16*)x, ldx, \
      (const __nv_bfloat16*)z, ldz, D, (__nv_bfloat16*)out, T, H)
  if (P == 64) FB_POST_FWD(8); else if (P == 128) FB_POST_FWD(16); else FB_POST_FWD(32);
#undef FB_POST_FWD
  return fb::launch_ok("mamba2_post_fwd_kernel");
}

// dout: bf16 [T, H * P]; dy, dx, dz: bf16 [T, H * P]; dD_part: fp32 [T, H] (summed over T by the caller)
int fb_mamba2_post_bwd(const void* y, const void* x, long long ldx, const void* z, long long ldz, const float* D, const void* dout,
                       void* dy, void* dx, void* dz, float* dD_part, long long T, int H, int P, cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((P != 64 && P != 128 && P != 256) || (ldx % 8) || (ldz % 8) || ((uintptr_t)x & 15) || ((uintptr_t)z & 15)) return -2;
  const long long threads = T * H * (P / 8);
  const unsigned blocks = (unsigned)((threads + 255) / 256);
#define FB_POST_BWD(L) mamba2_post_bwd_kernel<L><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)y, (const __nv_bfloat16*)x, ldx, \
      (const __nv_bfloat16*)z, ldz, D, (const __nv_bfloat16*)dout, (__nv_bfloat16*)dy, (__nv_bfloat16*)dx, (__nv_bfloat16*)dz, \
      dD_part, T, H)
  if (P == 64) FB_POST_BWD(8); else if (P == 128) FB_POST_BWD(16); else FB_POST_BWD(32);
#undef FB_POST_BWD
  return fb::launch_ok("mamba2_post_bwd_kernel");
}

int fb_hgrn2_gate_tiles(long long rows) { return (int)((rows + GATE_TILE_ROWS - 1) / GATE_TILE_ROWS); }

// q_raw, f_raw, q, k: bf16 [rows, D]; g: fp32 [rows, D]; lb: fp32 [D] or null.  D a multiple of 8.
int fb_hgrn2_gate_fwd(const void* q_raw, const void* f_raw, const float* lb, void* q, void* k, float* g, long long rows, int D,
                      cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (D % 8) return -2;
  const long long threads = rows * (D / 8);
  const unsigned blocks = (unsigned)((threads + 255) / 256);
  if (lb)
    hgrn2_gate_fwd_kernel<true><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)q_raw, (const __nv_bfloat16*)f_raw, lb,
                                                            (__nv_bfloat16*)q, (__nv_bfloat16*)k, g, rows, D);
  else
    hgrn2_gate_fwd_kernel<false><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)q_raw, (const __nv_bfloat16*)f_raw, lb,
                                                             (__nv_bfloat16*)q, (__nv_bfloat16*)k, g, rows, D);
  return fb::launch_ok("hgrn2_gate_fwd_kernel");
}

// dlb_part: fp32 [fb_hgrn2_gate_tiles(rows), D] scratch and dlb: fp32 [D], both only read / written when lb is given
int fb_hgrn2_gate_bwd(const void* q_raw, const void* f_raw, const float* lb, const void* dq, const void* dk, const float* dg,
                      void* dq_raw, void* df_raw, float* dlb_part, float* dlb, long long rows, int D, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (D % 8) return -2;
  const int tiles = fb_hgrn2_gate_tiles(rows);
  dim3 grid((D + 255) / 256, tiles);
  if (lb) {
    hgrn2_gate_bwd_kernel<true><<<grid, 256, 0, stream>>>(
        (const __nv_bfloat16*)q_raw, (const __nv_bfloat16*)f_raw, lb, (const __nv_bfloat16*)dq, (const __nv_bfloat16*)dk, dg,
        (__nv_bfloat16*)dq_raw, (__nv_bfloat16*)df_raw, dlb_part, rows, D);
    int rc = fb::launch_ok("hgrn2_gate_bwd_kernel");
    if (rc) return rc;
    colsum_rows_kernel<<<(D + 31) / 32, 256, 0, stream>>>(dlb_part, tiles, D, dlb);
    return fb::launch_ok("colsum_rows_kernel");
  }
  hgrn2_gate_bwd_kernel<false><<<grid, 256, 0, stream>>>(
      (const __nv_bfloat16*)q_raw, (const __nv_bfloat16*)f_raw, lb, (const __nv_bfloat16*)dq, (const __nv_bfloat16*)dk, dg,
      (__nv_bfloat16*)dq_raw, (__nv_bfloat16*)df_raw, dlb_part, rows, D);
  return fb::launch_ok("hgrn2_gate_bwd_kernel");
}

}  // extern "C"
