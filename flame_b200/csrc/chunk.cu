// Small CUDA-core kernels of the chunk-parallel token mixers (everything GEMM-shaped runs on bgemm.cu).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "host_utils.cuh"

namespace {

// T = (I + A)^-1 for a strictly lower-triangular 64 x 64 A (the WY "solve" of the delta rule; the reference does it by
// blockwise forward substitution in fla/ops/utils/solve_tril.py).  One 64-thread block per matrix: thread c solves
// (I + A) x = e_c by forward substitution with x in registers; every A element is a shared-memory broadcast.
__global__ void __launch_bounds__(64) tri_inverse_kernel(const float* __restrict__ A, __nv_bfloat16* __restrict__ out16,
                                                         float* __restrict__ out32, long long n) {
  __shared__ float sA[64 * 64];
  const long long m = blockIdx.x;
  if (m >= n) return;
  const float* a = A + m * 4096;
  for (int i = threadIdx.x; i < 4096 / 4; i += 64)
    reinterpret_cast<float4*>(sA)[i] = reinterpret_cast<const float4*>(a)[i];
  __syncthreads();
  const int c = threadIdx.x;
  float x[64];
#pragma unroll
  for (int i = 0; i < 64; ++i) {
    float s = (i == c) ? 1.f : 0.f;
#pragma unroll
    for (int j = 0; j < i; ++j) s = fmaf(-sA[i * 64 + j], x[j], s);
    x[i] = s;
  }
  if (out16 != nullptr) {
    __nv_bfloat16* o = out16 + m * 4096;
#pragma unroll
    for (int i = 0; i < 64; ++i) o[i * 64 + c] = __float2bfloat16(x[i]);
  }
  if (out32 != nullptr) {
    float* o = out32 + m * 4096;
#pragma unroll
    for (int i = 0; i < 64; ++i) o[i * 64 + c] = x[i];
  }
}

// Elementwise chunk-state recurrence without a transition matrix:
//   forward  X[c+1] = alpha[c] * X[c] + X[c+1]      reverse  X[c] = alpha[c] * X[c+1] + X[c]
// over the chunks listed for one chunk position; alpha is [NC, H] (per_row = 0) or [NC, H, rows] (per_row = 1).
// X is [NC + 1, H, rows, cols] fp32 with a bf16 mirror.
__global__ void state_step_kernel(const int* __restrict__ idx, int n_idx, const float* __restrict__ alpha, int per_row,
                                  float* __restrict__ X, __nv_bfloat16* __restrict__ X16, int H, int rows, int cols,
                                  int reverse) {
  const long long per_chunk = (long long)H * rows * cols;
  const long long total = (long long)n_idx * per_chunk / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long e = i * 4;
    const int b = (int)(e / per_chunk);
    const long long r = e - (long long)b * per_chunk;
    const int c = idx[b];
    const int h = (int)(r / ((long long)rows * cols));
    const int row = (int)((r / cols) % rows);
    const float al = per_row ? alpha[((long long)c * H + h) * rows + row] : alpha[(long long)c * H + h];
    const long long src = (long long)(reverse ? c + 1 : c) * per_chunk + r;
    const long long dst = (long long)(reverse ? c : c + 1) * per_chunk + r;
    const float4 s = *reinterpret_cast<const float4*>(X + src);
    float4 d = *reinterpret_cast<float4*>(X + dst);
    d.x = fmaf(al, s.x, d.x); d.y = fmaf(al, s.y, d.y); d.z = fmaf(al, s.z, d.z); d.w = fmaf(al, s.w, d.w);
    *reinterpret_cast<float4*>(X + dst) = d;
    __nv_bfloat162 lo = __floats2bfloat162_rn(d.x, d.y), hi = __floats2bfloat162_rn(d.z, d.w);
    uint2 q;
    q.x = *reinterpret_cast<uint32_t*>(&lo);
    q.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(X16 + dst) = q;
  }
}

}  // namespace

extern "C" {

int fb_tri_inverse(const float* A, void* out16, float* out32, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  tri_inverse_kernel<<<(unsigned)n, 64, 0, stream>>>(A, (__nv_bfloat16*)out16, out32, n);
  return fb::launch_ok("tri_inverse_kernel");
}

int fb_state_step(const int* idx, int n_idx, const float* alpha, int per_row, float* X, void* X16, int H, int rows, int cols,
                  int reverse, cudaStream_t stream) {
  if (n_idx <= 0) return 0;
  if (cols & 3) return -2;
  const long long total = (long long)n_idx * H * rows * cols / 4;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  state_step_kernel<<<(unsigned)blocks, 256, 0, stream>>>(idx, n_idx, alpha, per_row, X, (__nv_bfloat16*)X16, H, rows, cols,
                                                          reverse);
  return fb::launch_ok("state_step_kernel");
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------------------
// GLA intra-chunk scores, diagonal 16 x 16 sub-blocks:  A_ij = scale * sum_d q_id k_jd exp(b_id - b_jd),  j <= i,
// evaluated pairwise so that no exponent is positive whatever the gates are (the "secondary chunking" of
// fla/ops/gla/chunk.py:88-170; the off-diagonal sub-blocks are re-based products on the batched GEMM).
// q, k: [NC, 64, H, dk] bf16; b: [NC, 64, H, dk] fp32 (within-chunk cumulative log decay); A: [NC, H, 64, 64].
// Grid (NC * H, 4); 256 threads = one (i, j) pair each.
namespace {

__global__ void __launch_bounds__(256) gla_diag_fwd_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                                           const float* __restrict__ b, float* __restrict__ A, int H, int dk,
                                                           float scale) {
  extern __shared__ float sm[];
  const int ld = dk + 1;
  float* sq = sm;
  float* sk = sq + 16 * ld;
  float* sb = sk + 16 * ld;
  const int ch = blockIdx.x, c = ch / H, h = ch - c * H, blk = blockIdx.y;
  const long long row0 = ((long long)c * 64 + blk * 16);
  for (int idx = threadIdx.x; idx < 16 * dk; idx += 256) {
    const int r = idx / dk, d = idx - r * dk;
    const long long g = ((row0 + r) * H + h) * dk + d;
    sq[r * ld + d] = __bfloat162float(q[g]);
    sk[r * ld + d] = __bfloat162float(k[g]);
    sb[r * ld + d] = b[g];
  }
  __syncthreads();
  const int i = threadIdx.x >> 4, j = threadIdx.x & 15;
  float acc = 0.f;
  if (j <= i) {
    for (int d = 0; d < dk; ++d) acc = fmaf(sq[i * ld + d] * sk[j * ld + d], __expf(sb[i * ld + d] - sb[j * ld + d]), acc);
  }
  A[((long long)ch * 64 + blk * 16 + i) * 64 + blk * 16 + j] = acc * scale;
}

// Backward of the diagonal sub-blocks: dq_id = scale sum_{j<=i} dA_ij k_jd e^{b_id-b_jd}, dk_jd = scale sum_{i>=j} dA_ij q_id e^{b_id-b_jd},
// db = q dq - k dk (all ADDED into fp32 [NC, 64, H, dk] buffers).
__global__ void __launch_bounds__(256) gla_diag_bwd_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                                           const float* __restrict__ b, const float* __restrict__ dA,
                                                           float* __restrict__ dq, float* __restrict__ dk_, float* __restrict__ db,
                                                           int H, int dk, float scale) {
  extern __shared__ float sm[];
  const int ld = dk + 1;
  float* sq = sm;
  float* sk = sq + 16 * ld;
  float* sb = sk + 16 * ld;
  float* sdA = sb + 16 * ld;  // 16 x 16
  const int ch = blockIdx.x, c = ch / H, h = ch - c * H, blk = blockIdx.y;
  const long long row0 = ((long long)c * 64 + blk * 16);
  for (int idx = threadIdx.x; idx < 16 * dk; idx += 256) {
    const int r = idx / dk, d = idx - r * dk;
    const long long g = ((row0 + r) * H + h) * dk + d;
    sq[r * ld + d] = __bfloat162float(q[g]);
    sk[r * ld + d] = __bfloat162float(k[g]);
    sb[r * ld + d] = b[g];
  }
  {
    const int i = threadIdx.x >> 4, j = threadIdx.x & 15;
    sdA[threadIdx.x] = (j <= i) ? dA[((long long)ch * 64 + blk * 16 + i) * 64 + blk * 16 + j] * scale : 0.f;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < 16 * dk; idx += 256) {
    const int r = idx / dk, d = idx - r * dk;
    const float br = sb[r * ld + d];
    float gq = 0.f, gk = 0.f;
    for (int j = 0; j <= r; ++j) gq = fmaf(sdA[r * 16 + j] * sk[j * ld + d], __expf(br - sb[j * ld + d]), gq);
    for (int i = r; i < 16; ++i) gk = fmaf(sdA[i * 16 + r] * sq[i * ld + d], __expf(sb[i * ld + d] - br), gk);
    const long long g = ((row0 + r) * H + h) * dk + d;
    dq[g] += gq;
    dk_[g] += gk;
    db[g] += sq[r * ld + d] * gq - sk[r * ld + d] * gk;
  }
}

}  // namespace

extern "C" {

int fb_gla_diag_fwd(const void* q, const void* k, const float* b, float* A, int NC, int H, int dk, float scale,
                    cudaStream_t stream) {
  if (NC <= 0) return 0;
  const int smem = 3 * 16 * (dk + 1) * 4;
  static int configured = 0;
  if (smem > configured) {
    if (cudaFuncSetAttribute(gla_diag_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -2;
    configured = smem;
  }
  gla_diag_fwd_kernel<<<dim3(NC * H, 4), 256, smem, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k, b, A, H, dk, scale);
  return fb::launch_ok("gla_diag_fwd_kernel");
}

int fb_gla_diag_bwd(const void* q, const void* k, const float* b, const float* dA, float* dq, float* dk_, float* db, int NC,
                    int H, int dk, float scale, cudaStream_t stream) {
  if (NC <= 0) return 0;
  const int smem = 3 * 16 * (dk + 1) * 4 + 256 * 4;
  static int configured = 0;
  if (smem > configured) {
    if (cudaFuncSetAttribute(gla_diag_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -2;
    configured = smem;
  }
  gla_diag_bwd_kernel<<<dim3(NC * H, 4), 256, smem, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k, b, dA, dq, dk_, db,
                                                             H, dk, scale);
  return fb::launch_ok("gla_diag_bwd_kernel");
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------------------
// L2 normalisation of q / k heads (fla/modules/l2norm.py): y = x * rsqrt(sum x^2 + eps); one warp per row of D <= 1024.
namespace {

__global__ void l2norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, float* __restrict__ rstd,
                                  long long rows, int D, float eps) {
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const __nv_bfloat16* xr = x + row * D;
  float v[32];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const int d = lane + i * 32;
    v[i] = d < D ? __bfloat162float(xr[d]) : 0.f;
    ss = fmaf(v[i], v[i], ss);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float r = rsqrtf(ss + eps);
  if (lane == 0) rstd[row] = r;
  __nv_bfloat16* yr = y + row * D;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const int d = lane + i * 32;
    if (d < D) yr[d] = __float2bfloat16(v[i] * r);
  }
}

__global__ void l2norm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ rstd,
                                  const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dx, long long rows, int D) {
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const __nv_bfloat16* xr = x + row * D;
  const __nv_bfloat16* gr = dy + row * D;
  const float r = rstd[row];
  float y[32], g[32];
  float dot = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const int d = lane + i * 32;
    y[i] = d < D ? __bfloat162float(xr[d]) * r : 0.f;
    g[i] = d < D ? __bfloat162float(gr[d]) : 0.f;
    dot = fmaf(y[i], g[i], dot);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
  __nv_bfloat16* dr = dx + row * D;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const int d = lane + i * 32;
    if (d < D) dr[d] = __float2bfloat16(r * (g[i] - y[i] * dot));
  }
}

// The same two kernels for head dims that are a multiple of 64: LANES threads share a row and move 8 bf16 per access,
// so a warp covers 32 / LANES rows with 16-byte loads (the one-warp-per-row kernels above spend most of their 32
// predicated 2-byte accesses idle at the usual head dims of 64..256).
template <int LANES, int ITERS>
__global__ void l2norm_fwd_vec_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                      float* __restrict__ rstd, long long rows, float eps) {
  constexpr int D = LANES * ITERS * 8;
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long row = gid / LANES;
  const int sub = (int)(gid % LANES);
  const bool live = row < rows;
  uint4 v[ITERS];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    v[it] = live ? *reinterpret_cast<const uint4*>(x + row * D + (it * LANES + sub) * 8) : make_uint4(0, 0, 0, 0);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[it]);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(h[e]);
      ss = fmaf(f.x, f.x, fmaf(f.y, f.y, ss));
    }
  }
#pragma unroll
  for (int o = LANES / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float r = rsqrtf(ss + eps);
  if (!live) return;
  if (sub == 0) rstd[row] = r;
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[it]);
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(h[e]);
      oh[e] = __floats2bfloat162_rn(f.x * r, f.y * r);
    }
    *reinterpret_cast<uint4*>(y + row * D + (it * LANES + sub) * 8) = o;
  }
}

template <int LANES, int ITERS>
__global__ void l2norm_bwd_vec_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ rstd,
                                      const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dx, long long rows) {
  constexpr int D = LANES * ITERS * 8;
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long row = gid / LANES;
  const int sub = (int)(gid % LANES);
  const bool live = row < rows;
  const float r = live ? rstd[row] : 0.f;
  uint4 xv[ITERS], gv[ITERS];
  float dot = 0.f;
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const long long off = row * D + (it * LANES + sub) * 8;
    xv[it] = live ? *reinterpret_cast<const uint4*>(x + off) : make_uint4(0, 0, 0, 0);
    gv[it] = live ? *reinterpret_cast<const uint4*>(dy + off) : make_uint4(0, 0, 0, 0);
    const __nv_bfloat162* xh = reinterpret_cast<const __nv_bfloat162*>(&xv[it]);
    const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gv[it]);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 a = __bfloat1622float2(xh[e]), g = __bfloat1622float2(gh[e]);
      dot = fmaf(a.x * r, g.x, fmaf(a.y * r, g.y, dot));
    }
  }
#pragma unroll
  for (int o = LANES / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
  if (!live) return;
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const __nv_bfloat162* xh = reinterpret_cast<const __nv_bfloat162*>(&xv[it]);
    const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gv[it]);
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 a = __bfloat1622float2(xh[e]), g = __bfloat1622float2(gh[e]);
      oh[e] = __floats2bfloat162_rn(r * (g.x - a.x * r * dot), r * (g.y - a.y * r * dot));
    }
    *reinterpret_cast<uint4*>(dx + row * D + (it * LANES + sub) * 8) = o;
  }
}

template <int LANES, int ITERS>
void l2norm_fwd_vec(const void* x, void* y, float* rstd, long long rows, float eps, cudaStream_t stream) {
  const long long threads = rows * LANES;
  l2norm_fwd_vec_kernel<LANES, ITERS><<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>(
      (const __nv_bfloat16*)x, (__nv_bfloat16*)y, rstd, rows, eps);
}
template <int LANES, int ITERS>
void l2norm_bwd_vec(const void* x, const float* rstd, const void* dy, void* dx, long long rows, cudaStream_t stream) {
  const long long threads = rows * LANES;
  l2norm_bwd_vec_kernel<LANES, ITERS><<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>(
      (const __nv_bfloat16*)x, rstd, (const __nv_bfloat16*)dy, (__nv_bfloat16*)dx, rows);
}
bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

}  // namespace

extern "C" {

int fb_l2norm_fwd(const void* x, void* y, float* rstd, long long rows, int D, float eps, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (D > 1024) return -2;
  if (aligned16(x) && aligned16(y)) {
    switch (D) {
      case 64: l2norm_fwd_vec<8, 1>(x, y, rstd, rows, eps, stream); return fb::launch_ok("l2norm_fwd_vec_kernel");
      case 128: l2norm_fwd_vec<16, 1>(x, y, rstd, rows, eps, stream); return fb::launch_ok("l2norm_fwd_vec_kernel");
      case 256: l2norm_fwd_vec<32, 1>(x, y, rstd, rows, eps, stream); return fb::launch_ok("l2norm_fwd_vec_kernel");
      case 512: l2norm_fwd_vec<32, 2>(x, y, rstd, rows, eps, stream); return fb::launch_ok("l2norm_fwd_vec_kernel");
      case 1024: l2norm_fwd_vec<32, 4>(x, y, rstd, rows, eps, stream); return fb::launch_ok("l2norm_fwd_vec_kernel");
      default: break;
    }
  }
  l2norm_fwd_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, rstd, rows, D, eps);
  return fb::launch_ok("l2norm_fwd_kernel");
}

int fb_l2norm_bwd(const void* x, const float* rstd, const void* dy, void* dx, long long rows, int D, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (D > 1024) return -2;
  if (aligned16(x) && aligned16(dy) && aligned16(dx)) {
    switch (D) {
      case 64: l2norm_bwd_vec<8, 1>(x, rstd, dy, dx, rows, stream); return fb::launch_ok("l2norm_bwd_vec_kernel");
      case 128: l2norm_bwd_vec<16, 1>(x, rstd, dy, dx, rows, stream); return fb::launch_ok("l2norm_bwd_vec_kernel");
      case 256: l2norm_bwd_vec<32, 1>(x, rstd, dy, dx, rows, stream); return fb::launch_ok("l2norm_bwd_vec_kernel");
      case 512: l2norm_bwd_vec<32, 2>(x, rstd, dy, dx, rows, stream); return fb::launch_ok("l2norm_bwd_vec_kernel");
      case 1024: l2norm_bwd_vec<32, 4>(x, rstd, dy, dx, rows, stream); return fb::launch_ok("l2norm_bwd_vec_kernel");
      default: break;
    }
  }
  l2norm_bwd_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, stream>>>((const __nv_bfloat16*)x, rstd, (const __nv_bfloat16*)dy,
                                                                   (__nv_bfloat16*)dx, rows, D);
  return fb::launch_ok("l2norm_bwd_kernel");
}

}  // extern "C"

// out[b (, r)] = sum x[b, ...] * y[b, ...] in fp32 for bf16 x, y of shape [B, R, C]: per_row = 0 sums over R x C (one
// value per batch), per_row = 1 sums over C (one value per row).  One block per batch.
namespace {
__global__ void __launch_bounds__(256) pair_dot_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ y,
                                                       float* __restrict__ out, int R, int C, int per_row) {
  const long long b = blockIdx.x;
  const __nv_bfloat16* xb = x + b * (long long)R * C;
  const __nv_bfloat16* yb = y + b * (long long)R * C;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __shared__ float red[8];
  float total = 0.f;
  for (int r = warp; r < R; r += 8) {
    float s = 0.f;
    for (int c = lane * 8; c < C; c += 256) {
      const uint4 a = *reinterpret_cast<const uint4*>(xb + (long long)r * C + c);
      const uint4 d = *reinterpret_cast<const uint4*>(yb + (long long)r * C + c);
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, dw[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        s = fmaf(__uint_as_float(aw[t] << 16), __uint_as_float(dw[t] << 16), s);
        s = fmaf(__uint_as_float(aw[t] & 0xffff0000u), __uint_as_float(dw[t] & 0xffff0000u), s);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (per_row) {
      if (lane == 0) out[b * R + r] = s;
    } else {
      total += s;
    }
  }
  if (!per_row) {
    if (lane == 0) red[warp] = total;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int i = 0; i < 8; ++i) t += red[i];
      out[b] = t;
    }
  }
}
}  // namespace

extern "C" int fb_pair_dot(const void* x, const void* y, float* out, long long B, int R, int C, int per_row, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (C & 7) return -2;
  pair_dot_kernel<<<(unsigned)B, 256, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)y, out, R, C, per_row);
  return fb::launch_ok("pair_dot_kernel");
}

// Whole elementwise chunk-state recurrence of one document in ONE launch (no transition matrix):
//   forward  X[c+1] = alpha[c] * X[c] + X[c+1]   for c = first .. last-1        (X[first] is the zero initial state)
//   reverse  X[c]   = alpha[c] * X[c+1] + X[c]   for c = last-1 .. first
// Each thread owns four state elements of one (document, head) and carries them in registers across the chunks, so the
// fp32 array is read once and written once.  X: [NC + 1, H, rows, cols] fp32, X16 its bf16 mirror;
// alpha: [NC, H] (per_row = 0) or [NC, H, rows] (per_row = 1).  Grid: (ceil(H*rows*cols/4 / 256), documents).
namespace {
__global__ void __launch_bounds__(256) state_scan_kernel(const long long* __restrict__ first, const long long* __restrict__ last,
                                                         const float* __restrict__ alpha, int per_row, float* __restrict__ X,
                                                         __nv_bfloat16* __restrict__ X16, int H, int rows, int cols, int reverse) {
  const long long per_chunk = (long long)H * rows * cols;
  const long long e = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (e >= per_chunk) return;
  const int doc = blockIdx.y;
  const long long c0 = first[doc], c1 = last[doc];
  const int h = (int)(e / ((long long)rows * cols));
  const int row = (int)((e / cols) % rows);
  auto a_of = [&](long long c) { return per_row ? alpha[(c * H + h) * rows + row] : alpha[c * H + h]; };
  auto store16 = [&](long long off, const float4& v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 q;
    q.x = *reinterpret_cast<uint32_t*>(&lo);
    q.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(X16 + off) = q;
  };
  if (!reverse) {
    float4 s = *reinterpret_cast<const float4*>(X + c0 * per_chunk + e);
    for (long long c = c0; c < c1; ++c) {
      const float al = a_of(c);
      const long long off = (c + 1) * per_chunk + e;
      float4 d = *reinterpret_cast<const float4*>(X + off);
      s.x = fmaf(al, s.x, d.x); s.y = fmaf(al, s.y, d.y); s.z = fmaf(al, s.z, d.z); s.w = fmaf(al, s.w, d.w);
      *reinterpret_cast<float4*>(X + off) = s;
      store16(off, s);
    }
  } else {
    float4 s = *reinterpret_cast<const float4*>(X + c1 * per_chunk + e);
    for (long long c = c1 - 1; c >= c0; --c) {
      const float al = a_of(c);
      const long long off = c * per_chunk + e;
      float4 d = *reinterpret_cast<const float4*>(X + off);
      s.x = fmaf(al, s.x, d.x); s.y = fmaf(al, s.y, d.y); s.z = fmaf(al, s.z, d.z); s.w = fmaf(al, s.w, d.w);
      *reinterpret_cast<float4*>(X + off) = s;
      store16(off, s);
    }
  }
}
}  // namespace

extern "C" int fb_state_scan(const long long* first, const long long* last, int n_docs, const float* alpha, int per_row, float* X,
                             void* X16, int H, int rows, int cols, int reverse, cudaStream_t stream) {
  if (n_docs <= 0) return 0;
  if (cols & 3) return -2;
  const long long per_chunk = (long long)H * rows * cols;
  dim3 grid((unsigned)((per_chunk / 4 + 255) / 256), (unsigned)n_docs);
  state_scan_kernel<<<grid, 256, 0, stream>>>(first, last, alpha, per_row, X, (__nv_bfloat16*)X16, H, rows, cols, reverse);
  return fb::launch_ok("state_scan_kernel");
}

// ---------------------------------------------------------------------------------------------------------------
// GLA chunk preparation (one pass over q, k, g of a chunk; stands in for fla/ops/utils/cumsum.py and the scaling
// prologues of fla/ops/gla/chunk.py).  Chunk layout [NC, 64, H, dk]; a thread owns one channel of one (chunk, head).
//   b     = within-chunk cumulative sum of the log decay g                      (fp32)
//   khat  = k * exp(b_last - b)        key decayed to the end of its chunk      (state update operand)
//   qbar  = q * exp(b) * scale         query against the state entering the chunk
//   qt    = q * exp(b - r_I)           query re-based on the first row of its 16-row sub-block I
//   k3[I-1, j] = k_j * exp(r_I - b_j)  for j < 16 I, zero otherwise (I = 1..3; 48 rows): keys re-based for sub-block I
//   alpha = exp(b_last)                per-channel decay of the state across the chunk
// Every exponent is <= 0.
namespace {

__global__ void __launch_bounds__(128) gla_prep_fwd_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                                           const float* __restrict__ g, float* __restrict__ b,
                                                           __nv_bfloat16* __restrict__ khat, __nv_bfloat16* __restrict__ qbar,
                                                           __nv_bfloat16* __restrict__ qt, __nv_bfloat16* __restrict__ k3,
                                                           float* __restrict__ alpha, int H, int dk, float scale) {
  const int d = blockIdx.y * 128 + threadIdx.x;
  if (d >= dk) return;
  const int ch = blockIdx.x, c = ch / H, h = ch - c * H;
  const long long rs = (long long)H * dk;                       // row stride
  const long long base = ((long long)c * 64 * H + h) * dk + d;  // element (c, row 0, h, d)
  float run = 0.f, r[4];
#pragma unroll 8
  for (int i = 0; i < 64; ++i) {
    run += g[base + i * rs];
    b[base + i * rs] = run;
    if ((i & 15) == 0) r[i >> 4] = run;
  }
  const float b_last = run;
  alpha[(long long)ch * dk + d] = __expf(b_last);
  const long long k3base = (((long long)c * 3) * 48 * H + h) * dk + d;  // element (c, I-1 = 0, row 0, h, d)
#pragma unroll 4
  for (int i = 0; i < 64; ++i) {
    const long long off = base + i * rs;
    const float bi = b[off];
    const float qi = __bfloat162float(q[off]), ki = __bfloat162float(k[off]);
    khat[off] = __float2bfloat16(ki * __expf(b_last - bi));
    qbar[off] = __float2bfloat16(qi * __expf(bi) * scale);
    qt[off] = __float2bfloat16(qi * __expf(bi - r[i >> 4]));
    if (i < 48) {
#pragma unroll
      for (int I = 1; I <= 3; ++I) {
        const float v = (i < 16 * I) ? ki * __expf(r[I] - bi) : 0.f;
        k3[k3base + ((long long)(I - 1) * 48 + i) * rs] = __float2bfloat16(v);
      }
    }
  }
}

// Backward of the preparation.  Null gradient pointers count as zero.  dg receives the gradient of the log decay:
// db_i collects every use of b_i, and g_j feeds b_i for all i >= j (and b_last), hence the reverse cumulative sum.
__global__ void __launch_bounds__(128) gla_prep_bwd_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                                           const float* __restrict__ b, const __nv_bfloat16* __restrict__ dkhat,
                                                           const __nv_bfloat16* __restrict__ dqbar, const __nv_bfloat16* __restrict__ dqt,
                                                           const __nv_bfloat16* __restrict__ dk3, const float* __restrict__ dalpha,
                                                           const float* __restrict__ db_in, __nv_bfloat16* __restrict__ dq,
                                                           __nv_bfloat16* __restrict__ dk_, float* __restrict__ dg, int H, int dk,
                                                           float scale) {
  const int d = blockIdx.y * 128 + threadIdx.x;
  if (d >= dk) return;
  const int ch = blockIdx.x, c = ch / H, h = ch - c * H;
  const long long rs = (long long)H * dk;
  const long long base = ((long long)c * 64 * H + h) * dk + d;
  const long long k3base = (((long long)c * 3) * 48 * H + h) * dk + d;
  float r[4];
#pragma unroll
  for (int I = 0; I < 4; ++I) r[I] = b[base + (long long)(16 * I) * rs];
  const float b_last = b[base + 63 * rs];
  float acc_last = 0.f;
#pragma unroll 4
  for (int i = 0; i < 64; ++i) {
    const long long off = base + i * rs;
    const float bi = b[off];
    const float qi = __bfloat162float(q[off]), ki = __bfloat162float(k[off]);
    const float e = __expf(bi) * scale, ek = __expf(b_last - bi), et = __expf(bi - r[i >> 4]);
    const float g_qbar = dqbar ? __bfloat162float(dqbar[off]) : 0.f;
    const float g_qt = dqt ? __bfloat162float(dqt[off]) : 0.f;
    const float g_khat = dkhat ? __bfloat162float(dkhat[off]) : 0.f;
    float gq = g_qbar * e + g_qt * et;
    float gk = g_khat * ek;
    float gb = qi * gq - g_khat * ek * ki;
    acc_last += g_khat * ek * ki;
    if (dk3 != nullptr && i < 48) {
#pragma unroll
      for (int I = 1; I <= 3; ++I) {
        if (i < 16 * I) {
          const float t = __bfloat162float(dk3[k3base + ((long long)(I - 1) * 48 + i) * rs]) * __expf(r[I] - bi);
          gk += t;
          gb -= t * ki;
        }
      }
    }
    if (db_in != nullptr) gb += db_in[off];
    dq[off] = __float2bfloat16(gq);
    dk_[off] = __float2bfloat16(gk);
    dg[off] = gb;
  }
  float tail = acc_last + (dalpha ? dalpha[(long long)ch * dk + d] * __expf(b_last) : 0.f);  // gradient of b_last
#pragma unroll 8
  for (int i = 63; i >= 0; --i) {
    const long long off = base + i * rs;
    tail += dg[off];
    dg[off] = tail;
  }
}

}  // namespace

extern "C" {

int fb_gla_prep_fwd(const void* q, const void* k, const float* g, float* b, void* khat, void* qbar, void* qt, void* k3,
                    float* alpha, int NC, int H, int dk, float scale, cudaStream_t stream) {
  if (NC <= 0) return 0;
  dim3 grid(NC * H, (dk + 127) / 128);
  gla_prep_fwd_kernel<<<grid, 128, 0, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k, g, b, (__nv_bfloat16*)khat,
                                                (__nv_bfloat16*)qbar, (__nv_bfloat16*)qt, (__nv_bfloat16*)k3, alpha, H, dk, scale);
  return fb::launch_ok("gla_prep_fwd_kernel");
}

int fb_gla_prep_bwd(const void* q, const void* k, const float* b, const void* dkhat, const void* dqbar, const void* dqt,
                    const void* dk3, const float* dalpha, const float* db_in, void* dq, void* dk_, float* dg, int NC, int H,
                    int dk, float scale, cudaStream_t stream) {
  if (NC <= 0) return 0;
  dim3 grid(NC * H, (dk + 127) / 128);
  gla_prep_bwd_kernel<<<grid, 128, 0, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k, b, (const __nv_bfloat16*)dkhat,
                                                (const __nv_bfloat16*)dqbar, (const __nv_bfloat16*)dqt, (const __nv_bfloat16*)dk3,
                                                dalpha, db_in, (__nv_bfloat16*)dq, (__nv_bfloat16*)dk_, dg, H, dk, scale);
  return fb::launch_ok("gla_prep_bwd_kernel");
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------------------
// Preparation of the scalar-gated chunk algorithms (gated delta rule, SSD): one log decay per token and head.
//   b = within-chunk cumulative sum of g,  khat = k * exp(b_last - b),  qbar = q * exp(b) * scale,  alpha = exp(b_last)
// q, k: [NC, C, H, dk] bf16 (C = 64 or 128); g, b: [NC, C, H] fp32; alpha: [NC, H].  One block per (chunk, head).
namespace {

__global__ void __launch_bounds__(256) scalar_prep_fwd_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                                              const float* __restrict__ g, float* __restrict__ b,
                                                              __nv_bfloat16* __restrict__ khat, __nv_bfloat16* __restrict__ qbar,
                                                              float* __restrict__ alpha, int C, int H, int dk, float scale) {
  __shared__ float sb[128];
  const int ch = blockIdx.x, c = ch / H, h = ch - c * H;
  for (int i = threadIdx.x; i < C; i += blockDim.x) sb[i] = g != nullptr ? g[((long long)c * C + i) * H + h] : 0.f;
  __syncthreads();
  if (threadIdx.x == 0) {
    float run = 0.f;
    for (int i = 0; i < C; ++i) {
      run += sb[i];
      sb[i] = run;
    }
    alpha[ch] = __expf(run);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < C; i += blockDim.x) b[((long long)c * C + i) * H + h] = sb[i];
  const float b_last = sb[C - 1];
  const int nv = dk >> 3;  // 8 channels per thread and row
  for (int idx = threadIdx.x; idx < C * nv; idx += blockDim.x) {
    const int i = idx / nv, v = idx - i * nv;
    const long long off = (((long long)c * C + i) * H + h) * dk + v * 8;
    const float ek = __expf(b_last - sb[i]), eq = __expf(sb[i]) * scale;
    const uint4 qa = *reinterpret_cast<const uint4*>(q + off), ka = *reinterpret_cast<const uint4*>(k + off);
    const __nv_bfloat162* q2 = reinterpret_cast<const __nv_bfloat162*>(&qa);
    const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&ka);
    uint4 qo, ko;
    __nv_bfloat162* qo2 = reinterpret_cast<__nv_bfloat162*>(&qo);
    __nv_bfloat162* ko2 = reinterpret_cast<__nv_bfloat162*>(&ko);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 qf = __bfloat1622float2(q2[j]), kf = __bfloat1622float2(k2[j]);
      qo2[j] = __floats2bfloat162_rn(qf.x * eq, qf.y * eq);
      ko2[j] = __floats2bfloat162_rn(kf.x * ek, kf.y * ek);
    }
    *reinterpret_cast<uint4*>(qbar + off) = qo;
    *reinterpret_cast<uint4*>(khat + off) = ko;
  }
}

// Backward: dq = dqbar e^{b} scale, dk = dkhat e^{b_last - b}; db_i = sum_d (q dq - k dk) + db_in_i, the b_last uses
// (sum_i sum_d k dk, and alpha) go to the last row, and dg is the reverse cumulative sum of db.
__global__ void __launch_bounds__(256) scalar_prep_bwd_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                                              const float* __restrict__ b, const __nv_bfloat16* __restrict__ dkhat,
                                                              const __nv_bfloat16* __restrict__ dqbar, const float* __restrict__ dalpha,
                                                              const float* __restrict__ db_in, __nv_bfloat16* __restrict__ dq,
                                                              __nv_bfloat16* __restrict__ dk_, float* __restrict__ dg, int C, int H,
                                                              int dk, float scale) {
  __shared__ float sb[128], sdb[128];
  __shared__ float slast;
  const int ch = blockIdx.x, c = ch / H, h = ch - c * H;
  for (int i = threadIdx.x; i < C; i += blockDim.x) {
    sb[i] = b[((long long)c * C + i) * H + h];
    sdb[i] = db_in != nullptr ? db_in[((long long)c * C + i) * H + h] : 0.f;
  }
  if (threadIdx.x == 0) slast = 0.f;
  __syncthreads();
  const float b_last = sb[C - 1];
  const int nv = dk >> 3;
  // dk / 8 is a power of two for every supported head size, so a row's vectors sit in aligned lane groups
  for (int idx = threadIdx.x; idx < C * nv; idx += blockDim.x) {
    const int i = idx / nv, v = idx - i * nv;
    const long long off = (((long long)c * C + i) * H + h) * dk + v * 8;
    const float ek = __expf(b_last - sb[i]), eq = __expf(sb[i]) * scale;
    const uint4 qa = *reinterpret_cast<const uint4*>(q + off), ka = *reinterpret_cast<const uint4*>(k + off);
    uint4 gqa = make_uint4(0, 0, 0, 0), gka = make_uint4(0, 0, 0, 0);
    if (dqbar != nullptr) gqa = *reinterpret_cast<const uint4*>(dqbar + off);
    if (dkhat != nullptr) gka = *reinterpret_cast<const uint4*>(dkhat + off);
    const __nv_bfloat162* q2 = reinterpret_cast<const __nv_bfloat162*>(&qa);
    const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&ka);
    const __nv_bfloat162* gq2 = reinterpret_cast<const __nv_bfloat162*>(&gqa);
    const __nv_bfloat162* gk2 = reinterpret_cast<const __nv_bfloat162*>(&gka);
    uint4 qo, ko;
    __nv_bfloat162* qo2 = reinterpret_cast<__nv_bfloat162*>(&qo);
    __nv_bfloat162* ko2 = reinterpret_cast<__nv_bfloat162*>(&ko);
    float tq = 0.f, tk = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 qf = __bfloat1622float2(q2[j]), kf = __bfloat1622float2(k2[j]);
      const float2 gq = __bfloat1622float2(gq2[j]), gk = __bfloat1622float2(gk2[j]);
      const float dqx = gq.x * eq, dqy = gq.y * eq, dkx = gk.x * ek, dky = gk.y * ek;
      qo2[j] = __floats2bfloat162_rn(dqx, dqy);
      ko2[j] = __floats2bfloat162_rn(dkx, dky);
      tq += qf.x * dqx + qf.y * dqy;
      tk += kf.x * dkx + kf.y * dky;
    }
    *reinterpret_cast<uint4*>(dq + off) = qo;
    *reinterpret_cast<uint4*>(dk_ + off) = ko;
    // reduce over the lanes that share the row (a row's vectors are consecutive lanes), then one atomic per group
    const int grp = nv < 32 ? nv : 32;
    float s1 = tq - tk, s2 = tk;
    for (int o = grp >> 1; o > 0; o >>= 1) s1 += __shfl_xor_sync(0xffffffffu, s1, o);
    for (int o = 16; o > 0; o >>= 1) s2 += __shfl_xor_sync(0xffffffffu, s2, o);
    if ((threadIdx.x & (grp - 1)) == 0) atomicAdd(&sdb[i], s1);
    if ((threadIdx.x & 31) == 0) atomicAdd(&slast, s2);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float tail = slast + (dalpha != nullptr ? dalpha[ch] * __expf(b_last) : 0.f);
    for (int i = C - 1; i >= 0; --i) {
      tail += sdb[i];
      sdb[i] = tail;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < C; i += blockDim.x) dg[((long long)c * C + i) * H + h] = sdb[i];
}

}  // namespace

extern "C" {

int fb_scalar_prep_fwd(const void* q, const void* k, const float* g, float* b, void* khat, void* qbar, float* alpha, int NC,
                       int C, int H, int dk, float scale, cudaStream_t stream) {
  if (NC <= 0) return 0;
  if (C > 128 || (dk & 7)) return -2;
  scalar_prep_fwd_kernel<<<NC * H, 256, 0, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k, g, b, (__nv_bfloat16*)khat,
                                                     (__nv_bfloat16*)qbar, alpha, C, H, dk, scale);
  return fb::launch_ok("scalar_prep_fwd_kernel");
}

int fb_scalar_prep_bwd(const void* q, const void* k, const float* b, const void* dkhat, const void* dqbar, const float* dalpha,
                       const float* db_in, void* dq, void* dk_, float* dg, int NC, int C, int H, int dk, float scale,
                       cudaStream_t stream) {
  if (NC <= 0) return 0;
  if (C > 128 || (dk & 7) || ((dk >> 3) & ((dk >> 3) - 1))) return -2;  // dk / 8 must be a power of two
  scalar_prep_bwd_kernel<<<NC * H, 256, 0, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k, b, (const __nv_bfloat16*)dkhat,
                                                     (const __nv_bfloat16*)dqbar, dalpha, db_in, (__nv_bfloat16*)dq,
                                                     (__nv_bfloat16*)dk_, dg, C, H, dk, scale);
  return fb::launch_ok("scalar_prep_bwd_kernel");
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------------------
// Value-side decay (first pass of gated slot attention), diagonal 16 x 16 sub-blocks evaluated pairwise:
//   o[i, c] = sum_{j <= i, same sub-block} P[i, j] v[j, c] exp(b[i, c] - b[j, c])
// P: [NC, H, 64, 64] fp32 (causal scores), v: [NC, 64, H, M] bf16, b: [NC, 64, H, M] fp32, o: [NC, 64, H, M] fp32.
// Grid (NC * H, 4), 256 threads.  (fla/ops/gsa/chunk.py evaluates the same sub-blocks inside its intra-chunk kernel.)
namespace {

__global__ void __launch_bounds__(256) vdecay_diag_fwd_kernel(const float* __restrict__ P, const __nv_bfloat16* __restrict__ v,
                                                              const float* __restrict__ b, float* __restrict__ o, int H, int M) {
  extern __shared__ float sm[];
  float* sP = sm;            // 16 x 16
  float* sv = sP + 256;      // 16 x M
  float* sb = sv + 16 * M;   // 16 x M
  const int ch = blockIdx.x, c = ch / H, h = ch - c * H, blk = blockIdx.y;
  const long long row0 = (long long)c * 64 + blk * 16;
  sP[threadIdx.x] = P[((long long)ch * 64 + blk * 16 + (threadIdx.x >> 4)) * 64 + blk * 16 + (threadIdx.x & 15)];
  for (int idx = threadIdx.x; idx < 16 * M; idx += 256) {
    const int r = idx / M, cc = idx - r * M;
    const long long g = ((row0 + r) * H + h) * M + cc;
    sv[idx] = __bfloat162float(v[g]);
    sb[idx] = b[g];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < 16 * M; idx += 256) {
    const int r = idx / M, cc = idx - r * M;
    const float br = sb[idx];
    float acc = 0.f;
    for (int j = 0; j <= r; ++j) acc = fmaf(sP[r * 16 + j] * sv[j * M + cc], __expf(br - sb[j * M + cc]), acc);
    o[((row0 + r) * H + h) * M + cc] = acc;
  }
}

// dP (diagonal sub-blocks, lower triangle), dv and db of the forward above; dout: [NC, 64, H, M] fp32.
__global__ void __launch_bounds__(256) vdecay_diag_bwd_kernel(const float* __restrict__ P, const __nv_bfloat16* __restrict__ v,
                                                              const float* __restrict__ b, const float* __restrict__ dout,
                                                              float* __restrict__ dP, float* __restrict__ dv, float* __restrict__ db,
                                                              int H, int M) {
  extern __shared__ float sm[];
  float* sP = sm;
  float* sv = sP + 256;
  float* sb = sv + 16 * M;
  float* sd = sb + 16 * M;   // 16 x M
  const int ch = blockIdx.x, c = ch / H, h = ch - c * H, blk = blockIdx.y;
  const long long row0 = (long long)c * 64 + blk * 16;
  const int pi = threadIdx.x >> 4, pj = threadIdx.x & 15;
  const long long pidx = ((long long)ch * 64 + blk * 16 + pi) * 64 + blk * 16 + pj;
  sP[threadIdx.x] = P[pidx];
  for (int idx = threadIdx.x; idx < 16 * M; idx += 256) {
    const int r = idx / M, cc = idx - r * M;
    const long long g = ((row0 + r) * H + h) * M + cc;
    sv[idx] = __bfloat162float(v[g]);
    sb[idx] = b[g];
    sd[idx] = dout[g];
  }
  __syncthreads();
  float gp = 0.f;
  if (pj <= pi) {
    for (int cc = 0; cc < M; ++cc)
      gp = fmaf(sd[pi * M + cc] * sv[pj * M + cc], __expf(sb[pi * M + cc] - sb[pj * M + cc]), gp);
  }
  dP[pidx] = gp;
  for (int idx = threadIdx.x; idx < 16 * M; idx += 256) {
    const int r = idx / M, cc = idx - r * M;
    const float br = sb[idx];
    float orc = 0.f, gv = 0.f;
    for (int j = 0; j <= r; ++j) orc = fmaf(sP[r * 16 + j] * sv[j * M + cc], __expf(br - sb[j * M + cc]), orc);
    for (int i = r; i < 16; ++i) gv = fmaf(sP[i * 16 + r] * sd[i * M + cc], __expf(sb[i * M + cc] - br), gv);
    const long long g = ((row0 + r) * H + h) * M + cc;
    dv[g] = gv;
    db[g] = sd[idx] * orc - sv[idx] * gv;
  }
}

}  // namespace

extern "C" {

int fb_vdecay_diag_fwd(const float* P, const void* v, const float* b, float* o, int NC, int H, int M, cudaStream_t stream) {
  if (NC <= 0) return 0;
  const int smem = (256 + 2 * 16 * M) * 4;
  static int configured = 0;
  if (smem > configured) {
    if (cudaFuncSetAttribute(vdecay_diag_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -2;
    configured = smem;
  }
  vdecay_diag_fwd_kernel<<<dim3(NC * H, 4), 256, smem, stream>>>(P, (const __nv_bfloat16*)v, b, o, H, M);
  return fb::launch_ok("vdecay_diag_fwd_kernel");
}

int fb_vdecay_diag_bwd(const float* P, const void* v, const float* b, const float* dout, float* dP, float* dv, float* db, int NC,
                       int H, int M, cudaStream_t stream) {
  if (NC <= 0) return 0;
  const int smem = (256 + 3 * 16 * M) * 4;
  static int configured = 0;
  if (smem > configured) {
    if (cudaFuncSetAttribute(vdecay_diag_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -2;
    configured = smem;
  }
  vdecay_diag_bwd_kernel<<<dim3(NC * H, 4), 256, smem, stream>>>(P, (const __nv_bfloat16*)v, b, dout, dP, dv, db, H, M);
  return fb::launch_ok("vdecay_diag_bwd_kernel");
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------------------
// Backward helper of the decayed / masked score blocks C_ij = alpha (a_i . b_j) exp(d_i - d_j):
//   g_ij  = dC_ij * keep_ij * exp(d_i - d_j)      (bf16, the operand of the two gradient GEMMs)
//   dd_i  = sum_j dC_ij C_ij - sum_j dC_ji C_ji    (gradient of the cumulative log decay)
// dC and C may each be fp32 or bf16 (exactly one pointer of each pair is non-null).  One block per (chunk, head).
namespace {

__global__ void __launch_bounds__(256) scores_bwd_prep_kernel(const float* __restrict__ dc32, const __nv_bfloat16* __restrict__ dc16,
                                                              const float* __restrict__ c32, const __nv_bfloat16* __restrict__ c16,
                                                              const float* __restrict__ d, long long d_hi, long long d_lo,
                                                              long long d_r, int H, int C, int mask_mode,
                                                              __nv_bfloat16* __restrict__ g, float* __restrict__ dd) {
  __shared__ float sd[128], srow[128], scol[128];
  const int ch = blockIdx.x, c = ch / H, h = ch - c * H;
  const float* dv = d + (long long)c * d_hi + (long long)h * d_lo;
  for (int i = threadIdx.x; i < C; i += 256) {
    sd[i] = dv[(long long)i * d_r];
    srow[i] = 0.f;
    scol[i] = 0.f;
  }
  __syncthreads();
  const long long base = (long long)ch * C * C;
  for (int idx = threadIdx.x; idx < C * C; idx += 256) {
    const int i = idx / C, j = idx - i * C;  // a warp covers 32 consecutive j of one row (C is a multiple of 32)
    const bool keep = mask_mode == 0 || (mask_mode == 1 ? j <= i : j < i);
    const float dcv = dc32 != nullptr ? dc32[base + idx] : __bfloat162float(dc16[base + idx]);
    const float cv = c32 != nullptr ? c32[base + idx] : __bfloat162float(c16[base + idx]);
    g[base + idx] = __float2bfloat16(keep ? dcv * __expf(sd[i] - sd[j]) : 0.f);
    const float e = dcv * cv;  // C is zero where masked
    float r = e;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
    if ((threadIdx.x & 31) == 0) atomicAdd(&srow[i], r);
    atomicAdd(&scol[j], e);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < C; i += 256) dd[(long long)ch * C + i] = srow[i] - scol[i];
}

}  // namespace

extern "C" int fb_scores_bwd_prep(const float* dc32, const void* dc16, const float* c32, const void* c16, const float* d,
                                  long long d_hi, long long d_lo, long long d_r, int NC, int H, int C, int mask_mode, void* g,
                                  float* dd, cudaStream_t stream) {
  if (NC <= 0) return 0;
  if (C > 128 || (C & 31)) return -2;
  scores_bwd_prep_kernel<<<NC * H, 256, 0, stream>>>(dc32, (const __nv_bfloat16*)dc16, c32, (const __nv_bfloat16*)c16, d, d_hi, d_lo,
                                                     d_r, H, C, mask_mode, (__nv_bfloat16*)g, dd);
  return fb::launch_ok("scores_bwd_prep_kernel");
}
