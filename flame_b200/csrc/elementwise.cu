// Bandwidth-bound training kernels: rotary embedding (varlen), SwiGLU, row-wise cross-entropy with in-place
// gradient, embedding gather / scatter-add, flat AdamW with clipping and skip-on-NaN, sum-of-squares partials,
// and the device-side builders for position ids.  All use 16-byte accesses and fp32 math.
//
// Reference semantics: fla/modules/rotary.py:29-43 (NeoX rotation, positions restart at cu_seqlens
// boundaries), fla/modules/activations.py:553-628 (swiglu), fla/modules/fused_cross_entropy.py:31-156
// (loss = lse - logit[target], dlogits = softmax - onehot, ignore_index rows give zero), torch AdamW.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <math.h>
#include <stdint.h>
#include "host_utils.cuh"

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
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

// ------------------------------------------------------------------------------------------------
// position ids from cu_seqlens: pos[t] = t - cu[doc(t)], seq_id[t] = doc(t)
// ------------------------------------------------------------------------------------------------
__global__ void position_ids_kernel(const int* __restrict__ cu, int nseq, int* __restrict__ pos,
                                    int* __restrict__ seq_id, int total) {
  int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= total) return;
  int lo = 0, hi = nseq;  // find largest i with cu[i] <= t
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (cu[mid] <= t) lo = mid; else hi = mid;
  }
  pos[t] = t - cu[lo];
  if (seq_id) seq_id[t] = lo;
}

// ------------------------------------------------------------------------------------------------
// RoPE, NeoX (half-split) layout, in place or out of place, on rows of [T, H, Dh] with a row stride.
// cos/sin tables are fp32 [max_pos, rot/2].  conj = 1 applies the inverse rotation (backward).
// ------------------------------------------------------------------------------------------------
template <bool IN_F32>
__global__ void rope_kernel(const void* __restrict__ xin, __nv_bfloat16* __restrict__ y,
                            const int* __restrict__ pos, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, long long T, int H, int Dh, int rot,
                            long long x_stride_t, long long y_stride_t, int seq_len_mod, int conj) {
  // one thread handles 8 consecutive elements of the first half and their partners in the second half
  const int half = rot >> 1;
  const int vec_per_head = half >> 3;
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  long long total = T * H * vec_per_head;
  if (idx >= total) return;
  int v = (int)(idx % vec_per_head);
  long long th = idx / vec_per_head;
  int h = (int)(th % H);
  long long t = th / H;
  int p = pos ? pos[t] : (int)(seq_len_mod > 0 ? (t % seq_len_mod) : t);
  __nv_bfloat16* yd = y + t * y_stride_t + (long long)h * Dh + v * 8;
  float a[8], b[8];
  if (IN_F32) {
    const float* xs = reinterpret_cast<const float*>(xin) + t * x_stride_t + (long long)h * Dh + v * 8;
    *reinterpret_cast<float4*>(&a[0]) = *reinterpret_cast<const float4*>(xs);
    *reinterpret_cast<float4*>(&a[4]) = *reinterpret_cast<const float4*>(xs + 4);
    *reinterpret_cast<float4*>(&b[0]) = *reinterpret_cast<const float4*>(xs + half);
    *reinterpret_cast<float4*>(&b[4]) = *reinterpret_cast<const float4*>(xs + half + 4);
  } else {
    const __nv_bfloat16* xs = reinterpret_cast<const __nv_bfloat16*>(xin) + t * x_stride_t + (long long)h * Dh + v * 8;
    unpack8(*reinterpret_cast<const uint4*>(xs), a);
    unpack8(*reinterpret_cast<const uint4*>(xs + half), b);
  }
  const float4* c4 = reinterpret_cast<const float4*>(cos_t + (long long)p * half + v * 8);
  const float4* s4 = reinterpret_cast<const float4*>(sin_t + (long long)p * half + v * 8);
  float c[8], s[8];
  *reinterpret_cast<float4*>(&c[0]) = c4[0];
  *reinterpret_cast<float4*>(&c[4]) = c4[1];
  *reinterpret_cast<float4*>(&s[0]) = s4[0];
  *reinterpret_cast<float4*>(&s[4]) = s4[1];
  float o1[8], o2[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float sj = conj ? -s[j] : s[j];
    o1[j] = a[j] * c[j] - b[j] * sj;
    o2[j] = a[j] * sj + b[j] * c[j];
  }
  *reinterpret_cast<uint4*>(yd) = pack8(o1);
  *reinterpret_cast<uint4*>(yd + half) = pack8(o2);
}

// ------------------------------------------------------------------------------------------------
// SwiGLU: a = silu(g) * u.  g and u are column blocks of one [T, 2I] buffer or separate tensors.
// ------------------------------------------------------------------------------------------------
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ u,
                                  __nv_bfloat16* __restrict__ a, long long T, int I, long long ld_g, long long ld_u,
                                  long long ld_a) {
  const int vec = I >> 3;
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= T * vec) return;
  long long t = idx / vec;
  int v = (int)(idx - t * vec);
  float gg[8], uu[8], o[8];
  unpack8(*reinterpret_cast<const uint4*>(g + t * ld_g + v * 8), gg);
  unpack8(*reinterpret_cast<const uint4*>(u + t * ld_u + v * 8), uu);
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j] = gg[j] * sigmoidf_(gg[j]) * uu[j];
  *reinterpret_cast<uint4*>(a + t * ld_a + v * 8) = pack8(o);
}
// dg = da * u * s * (1 + g (1 - s)),  du = da * g * s;  optionally re-emits a (needed by the down-proj wgrad)
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ da, const __nv_bfloat16* __restrict__ g,
                                  const __nv_bfloat16* __restrict__ u, __nv_bfloat16* __restrict__ dg,
                                  __nv_bfloat16* __restrict__ du, __nv_bfloat16* __restrict__ a_out, long long T,
                                  int I, long long ld_da, long long ld_g, long long ld_u, long long ld_dg,
                                  long long ld_du, long long ld_a) {
  const int vec = I >> 3;
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= T * vec) return;
  long long t = idx / vec;
  int v = (int)(idx - t * vec);
  float d[8], gg[8], uu[8], o1[8], o2[8], aa[8];
  unpack8(*reinterpret_cast<const uint4*>(da + t * ld_da + v * 8), d);
  unpack8(*reinterpret_cast<const uint4*>(g + t * ld_g + v * 8), gg);
  unpack8(*reinterpret_cast<const uint4*>(u + t * ld_u + v * 8), uu);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float s = sigmoidf_(gg[j]);
    o1[j] = d[j] * uu[j] * s * (1.f + gg[j] * (1.f - s));
    o2[j] = d[j] * gg[j] * s;
    aa[j] = gg[j] * s * uu[j];
  }
  *reinterpret_cast<uint4*>(dg + t * ld_dg + v * 8) = pack8(o1);
  *reinterpret_cast<uint4*>(du + t * ld_du + v * 8) = pack8(o2);
  if (a_out) *reinterpret_cast<uint4*>(a_out + t * ld_a + v * 8) = pack8(aa);
}

// ------------------------------------------------------------------------------------------------
// Cross-entropy over bf16 logits [rows, V]: one CTA per row.
//   loss_row = lse - logit[target];  dlogits = (softmax - onehot) * grad_scale, written in place.
//   grad_scale = scale_num / max(n_valid, 1) with n_valid read from device memory (no host sync).
//   Rows whose target == ignore_index produce loss 0 and zero gradient.
// ------------------------------------------------------------------------------------------------
// Options of fla's FusedCrossEntropyLoss (fla/modules/fused_cross_entropy.py:374-400): the loss is taken on
//   z = softcap * tanh(logit_scale * x / softcap)   (softcap <= 0: z = logit_scale * x)
//   loss = lse(z) - smoothing * mean(z) - (1 - smoothing) * z_target + lse_square_scale * lse(z)^2
struct CeOptions {
  float label_smoothing, logit_scale, lse_square_scale, softcap;
};
__device__ __forceinline__ float ce_z(float x, const CeOptions& o) {
  x *= o.logit_scale;
  return o.softcap > 0.f ? o.softcap * tanhf(x / o.softcap) : x;
}
constexpr int CE_THREADS = 512;
__global__ void __launch_bounds__(CE_THREADS)
cross_entropy_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ targets,
                     float* __restrict__ loss_rows, float* __restrict__ lse_rows, const int* __restrict__ n_valid,
                     float scale_num, int V, long long ld, int ignore_index, int write_grad, CeOptions opt) {
  __shared__ float s_red[CE_THREADS / 32];
  __shared__ float s_bcast[2];
  const long long row = blockIdx.x;
  __nv_bfloat16* lr = logits + row * ld;
  const long long tgt = targets[row];
  const int nvec = V >> 3;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // pass 1: online max / sum-exp
  const bool plain = opt.logit_scale == 1.f && opt.softcap <= 0.f;
  float m = -INFINITY, s = 0.f, zsum = 0.f;
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    float f[8];
    unpack8(reinterpret_cast<const uint4*>(lr)[i], f);
    if (!plain) {
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = ce_z(f[j], opt);
    }
    if (opt.label_smoothing > 0.f) {
#pragma unroll
      for (int j = 0; j < 8; ++j) zsum += f[j];
    }
    float lm = f[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
    float nm = fmaxf(m, lm);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += __expf(f[j] - nm);
    s = s * __expf(m - nm) + acc;
    m = nm;
  }
  for (int i = (nvec << 3) + threadIdx.x; i < V; i += CE_THREADS) {
    float f = ce_z(__bfloat162float(lr[i]), opt);
    zsum += f;
    float nm = fmaxf(m, f);
    s = s * __expf(m - nm) + __expf(f - nm);
    m = nm;
  }
  float gm = warp_max(m);
  if (lane == 0) s_red[warp] = gm;
  __syncthreads();
  if (warp == 0) {
    float t = lane < CE_THREADS / 32 ? s_red[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) s_bcast[0] = t;
  }
  __syncthreads();
  gm = s_bcast[0];
  s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  s = warp_sum(s);
  __syncthreads();
  if (lane == 0) s_red[warp] = s;
  __syncthreads();
  if (warp == 0) {
    float t = lane < CE_THREADS / 32 ? s_red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) s_bcast[1] = t;
  }
  __syncthreads();
  const float sum = s_bcast[1];
  const float lse = gm + __logf(sum);
  const bool ignored = (tgt == (long long)ignore_index);
  float zmean = 0.f;
  if (opt.label_smoothing > 0.f) {  // block-wide sum of z for the smoothing term
    __syncthreads();
    zsum = warp_sum(zsum);
    if (lane == 0) s_red[warp] = zsum;
    __syncthreads();
    if (warp == 0) {
      float t = lane < CE_THREADS / 32 ? s_red[lane] : 0.f;
      t = warp_sum(t);
      if (lane == 0) s_bcast[0] = t;
    }
    __syncthreads();
    zmean = s_bcast[0] / (float)V;
  }
  if (threadIdx.x == 0) {
    float l = 0.f;
    if (!ignored) {
      const float zt = ce_z(__bfloat162float(lr[tgt]), opt);
      l = lse - opt.label_smoothing * zmean - (1.f - opt.label_smoothing) * zt + opt.lse_square_scale * lse * lse;
    }
    loss_rows[row] = l;
    if (lse_rows) lse_rows[row] = lse;
  }
  if (!write_grad) return;
  __syncthreads();  // the target logit was read above before anyone overwrites it
  const float nv = (float)max(*n_valid, 1);
  const float gs = ignored ? 0.f : scale_num / nv;
  const float inv = 1.f / sum;
  // d loss / d z_j = p_j (1 + 2 zl lse) - smoothing / V - (1 - smoothing) [j == target];   d z / d x = scale (1 - tanh^2)
  const float pmul = 1.f + 2.f * opt.lse_square_scale * lse;
  const float sm = opt.label_smoothing / (float)V;
  const float hit = 1.f - opt.label_smoothing;
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    float f[8];
    uint4* p = reinterpret_cast<uint4*>(lr) + i;
    unpack8(*p, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float z = f[j], dz = 1.f;
      if (!plain) {
        z = ce_z(f[j], opt);
        dz = opt.softcap > 0.f ? opt.logit_scale * (1.f - (z / opt.softcap) * (z / opt.softcap)) : opt.logit_scale;
      }
      float pr = __expf(z - gm) * inv * pmul - sm;
      if ((long long)(i * 8 + j) == tgt) pr -= hit;
      f[j] = pr * gs * dz;
    }
    *p = pack8(f);
  }
  for (int i = (nvec << 3) + threadIdx.x; i < V; i += CE_THREADS) {
    const float z = ce_z(__bfloat162float(lr[i]), opt);
    const float dz = opt.softcap > 0.f ? opt.logit_scale * (1.f - (z / opt.softcap) * (z / opt.softcap)) : opt.logit_scale;
    float pr = __expf(z - gm) * inv * pmul - sm;
    if ((long long)i == tgt) pr -= hit;
    lr[i] = __float2bfloat16(pr * gs * dz);
  }
}

// ------------------------------------------------------------------------------------------------
// Vocabulary-parallel cross-entropy (tensor parallelism): every rank holds a column slice of the logits.
//   stats kernel : per row the slice's max, its sum of exp(x - max) and the target logit if the target falls in the slice
//   (host)       : the [ranks, rows, 3] statistics are all-gathered and folded into the global log-sum-exp per row
//   grad kernel  : in place, logits <- (exp(x - lse) - [column == target]) * grad_scale / n_valid   (0 for ignored rows)
// One block per row, the slice is read once per kernel; no fp32 copy of the logits is ever made.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(CE_THREADS)
ce_vp_stats_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ targets,
                   float* __restrict__ stats, int V, long long ld, long long vocab_start, int ignore_index) {
  __shared__ float s_red[CE_THREADS / 32];
  __shared__ float s_bcast;
  const long long row = blockIdx.x;
  const __nv_bfloat16* lr = logits + row * ld;
  const int nvec = V >> 3;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    float f[8];
    unpack8(reinterpret_cast<const uint4*>(lr)[i], f);
    float lm = f[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
    const float nm = fmaxf(m, lm);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += __expf(f[j] - nm);
    s = s * __expf(m - nm) + acc;
    m = nm;
  }
  for (int i = (nvec << 3) + threadIdx.x; i < V; i += CE_THREADS) {
    const float f = __bfloat162float(lr[i]);
    const float nm = fmaxf(m, f);
    s = s * __expf(m - nm) + __expf(f - nm);
    m = nm;
  }
  float gm = warp_max(m);
  if (lane == 0) s_red[warp] = gm;
  __syncthreads();
  if (warp == 0) {
    float t = lane < CE_THREADS / 32 ? s_red[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) s_bcast = t;
  }
  __syncthreads();
  gm = s_bcast;
  s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  s = warp_sum(s);
  __syncthreads();
  if (lane == 0) s_red[warp] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < CE_THREADS / 32; ++w) t += s_red[w];
    const long long tgt = targets[row];
    const long long local = tgt - vocab_start;
    float tv = 0.f;
    if (tgt != (long long)ignore_index && local >= 0 && local < V) tv = __bfloat162float(lr[local]);
    stats[row * 3 + 0] = gm;
    stats[row * 3 + 1] = t;
    stats[row * 3 + 2] = tv;
  }
}

__global__ void __launch_bounds__(CE_THREADS)
ce_vp_grad_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ targets, const float* __restrict__ lse,
                  const int* __restrict__ n_valid, float scale_num, int V, long long ld, long long vocab_start,
                  int ignore_index) {
  const long long row = blockIdx.x;
  __nv_bfloat16* lr = logits + row * ld;
  const long long tgt = targets[row];
  const long long local = tgt - vocab_start;
  const float gs = (tgt == (long long)ignore_index) ? 0.f : scale_num / (float)max(*n_valid, 1);
  const float l = lse[row];
  const int nvec = V >> 3;
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    float f[8];
    uint4* p = reinterpret_cast<uint4*>(lr) + i;
    unpack8(*p, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float pr = __expf(f[j] - l);
      if ((long long)(i * 8 + j) == local) pr -= 1.f;
      f[j] = pr * gs;
    }
    *p = pack8(f);
  }
  for (int i = (nvec << 3) + threadIdx.x; i < V; i += CE_THREADS) {
    float pr = __expf(__bfloat162float(lr[i]) - l);
    if ((long long)i == local) pr -= 1.f;
    lr[i] = __float2bfloat16(pr * gs);
  }
}

// counts targets != ignore_index into *n_valid (single CTA, fixed order)
__global__ void count_valid_kernel(const long long* __restrict__ targets, long long n, int ignore_index,
                                   int* __restrict__ n_valid) {
  __shared__ int s[32];
  int c = 0;
  for (long long i = threadIdx.x; i < n; i += blockDim.x) c += targets[i] != (long long)ignore_index;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x < 32) {
    int t = threadIdx.x < (blockDim.x >> 5) ? s[threadIdx.x] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (threadIdx.x == 0) *n_valid = t;
  }
}

// out[0] (+)= sum(rows) / max(n_valid,1) in a fixed order (single CTA)
__global__ void mean_loss_kernel(const float* __restrict__ rows, long long n, const int* __restrict__ n_valid,
                                 float* __restrict__ out, int accumulate) {
  __shared__ float s[32];
  float c = 0.f;
  for (long long i = threadIdx.x; i < n; i += blockDim.x) c += rows[i];
  c = warp_sum(c);
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? s[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) {
      float v = t / (float)max(*n_valid, 1);
      out[0] = accumulate ? out[0] + v : v;
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Embedding
// ------------------------------------------------------------------------------------------------
__global__ void embedding_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                     __nv_bfloat16* __restrict__ out, long long T, int D, long long V) {
  const int vec = D >> 3;
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= T * vec) return;
  long long t = idx / vec;
  int v = (int)(idx - t * vec);
  long long id = ids[t];
  uint4 q = make_uint4(0, 0, 0, 0);
  if (id >= 0 && id < V) q = reinterpret_cast<const uint4*>(table + id * D)[v];
  reinterpret_cast<uint4*>(out + t * D)[v] = q;
}
// Deterministic scatter-add: tokens are pre-sorted by id (perm), seg_start marks runs of equal ids.
// One warp per unique id sums its rows in sorted order and adds them to the fp32 gradient row.
__global__ void embedding_bwd_sorted_kernel(const long long* __restrict__ sorted_ids,
                                            const long long* __restrict__ perm, const int* __restrict__ seg_start,
                                            int nseg, long long T, const __nv_bfloat16* __restrict__ dout,
                                            float* __restrict__ dtable, int D, long long V) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= nseg) return;
  const long long b = seg_start[warp];
  const long long e = (warp + 1 < nseg) ? (long long)seg_start[warp + 1] : T;
  const long long id = sorted_ids[b];
  if (id < 0 || id >= V) return;
  const int vec = D >> 3;
  for (int v = lane; v < vec; v += 32) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (long long r = b; r < e; ++r) {
      float f[8];
      unpack8(reinterpret_cast<const uint4*>(dout + perm[r] * D)[v], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
    float4* dst = reinterpret_cast<float4*>(dtable + id * D + v * 8);
    float4 o0 = dst[0], o1 = dst[1];
    o0.x += acc[0]; o0.y += acc[1]; o0.z += acc[2]; o0.w += acc[3];
    o1.x += acc[4]; o1.y += acc[5]; o1.z += acc[6]; o1.w += acc[7];
    dst[0] = o0;
    dst[1] = o1;
  }
}

// ------------------------------------------------------------------------------------------------
// sum of squares partials (grad-norm) and flat AdamW
// ------------------------------------------------------------------------------------------------
constexpr int SQ_THREADS = 512;
__global__ void __launch_bounds__(SQ_THREADS)
sumsq_partials_kernel(const float* __restrict__ x, long long n, float* __restrict__ partials) {
  __shared__ float s[SQ_THREADS / 32];
  float acc = 0.f;
  const long long nvec = n >> 2;
  for (long long i = (long long)blockIdx.x * SQ_THREADS + threadIdx.x; i < nvec; i += (long long)gridDim.x * SQ_THREADS) {
    float4 v = reinterpret_cast<const float4*>(x)[i];
    acc += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  if (blockIdx.x == 0)
    for (long long i = (nvec << 2) + threadIdx.x; i < n; i += SQ_THREADS) acc += x[i] * x[i];
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < SQ_THREADS / 32 ? s[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) partials[blockIdx.x] = t;
  }
}
// out[0] (+)= sum(partials) in a fixed order
__global__ void sum_partials_kernel(const float* __restrict__ partials, int n, float* __restrict__ out,
                                    int accumulate) {
  __shared__ float s[32];
  float c = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) c += partials[i];
  c = warp_sum(c);
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? s[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) out[0] = accumulate ? out[0] + t : t;
  }
}

// AdamW on a flat fp32 shard.  `ctrl` lives on the device:
//   ctrl[0] = total grad-norm squared (all ranks, all params)   ctrl[1] = (float) applied step count
//   ctrl[2] = skipped-step counter                               ctrl[3] = last clip coefficient
//   ctrl[5] = abort flag of this step (set from the library status word: a bounded wait ran out, so gradients or
//             parameters may be incomplete; no update is applied, whatever skip_nan_inf says)   ctrl[6] = aborted steps
// If the norm is NaN/Inf and skip_nan_inf is set the parameters, moments and step count stay untouched.
// The update follows torch.optim.AdamW (decoupled weight decay, bias correction) with grad * clip_coef.
// A single thread of the launch (block 0, thread 0 of the LAST shard launch, flagged by `finalize`) advances the counters.
__global__ void adamw_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                             const float* __restrict__ g, __nv_bfloat16* __restrict__ p_bf16, long long n, float lr,
                             float beta1, float beta2, float eps, float wd, float max_norm, int skip_nan_inf,
                             const float* __restrict__ ctrl, float grad_scale) {
  // wd >= 0: decoupled weight decay (AdamW).  wd < 0: plain Adam, the decay |wd| * p is added to the gradient instead.
  const float wd_l2 = wd < 0.f ? -wd : 0.f;
  wd = wd < 0.f ? 0.f : wd;
  if (ctrl[5] != 0.f) return;
  const float norm = sqrtf(ctrl[0]) * grad_scale;
  const bool bad = !isfinite(norm);
  if (bad && skip_nan_inf) return;
  float coef = 1.f;
  if (max_norm > 0.f) coef = fminf(1.f, max_norm / (norm + 1e-6f));
  coef *= grad_scale;
  const float step = ctrl[1] + 1.f;
  const float bc1 = 1.f - powf(beta1, step);
  const float bc2 = 1.f - powf(beta2, step);
  const float step_size = lr / bc1;
  const float inv_sqrt_bc2 = rsqrtf(bc2);
  long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= n) return;
  if (i + 4 <= n) {
    float4 pp = *reinterpret_cast<float4*>(p + i);
    float4 mm = *reinterpret_cast<float4*>(m + i);
    float4 vv = *reinterpret_cast<float4*>(v + i);
    float4 gg = *reinterpret_cast<const float4*>(g + i);
    float P[4] = {pp.x, pp.y, pp.z, pp.w}, M[4] = {mm.x, mm.y, mm.z, mm.w}, V[4] = {vv.x, vv.y, vv.z, vv.w},
          G[4] = {gg.x, gg.y, gg.z, gg.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float gr = G[j] * coef + wd_l2 * P[j];
      P[j] *= (1.f - lr * wd);
      M[j] = beta1 * M[j] + (1.f - beta1) * gr;
      V[j] = beta2 * V[j] + (1.f - beta2) * gr * gr;
      float denom = sqrtf(V[j]) * inv_sqrt_bc2 + eps;
      P[j] -= step_size * M[j] / denom;
    }
    *reinterpret_cast<float4*>(p + i) = make_float4(P[0], P[1], P[2], P[3]);
    *reinterpret_cast<float4*>(m + i) = make_float4(M[0], M[1], M[2], M[3]);
    *reinterpret_cast<float4*>(v + i) = make_float4(V[0], V[1], V[2], V[3]);
    if (p_bf16) {
      uint2 q;
      __nv_bfloat162 a = __floats2bfloat162_rn(P[0], P[1]), b = __floats2bfloat162_rn(P[2], P[3]);
      q.x = *reinterpret_cast<uint32_t*>(&a);
      q.y = *reinterpret_cast<uint32_t*>(&b);
      *reinterpret_cast<uint2*>(p_bf16 + i) = q;
    }
  } else {
    for (long long k = i; k < n; ++k) {
      float gr = g[k] * coef + wd_l2 * p[k];
      float P = p[k] * (1.f - lr * wd);
      float M = beta1 * m[k] + (1.f - beta1) * gr;
      float V = beta2 * v[k] + (1.f - beta2) * gr * gr;
      P -= step_size * M / (sqrtf(V) * inv_sqrt_bc2 + eps);
      p[k] = P; m[k] = M; v[k] = V;
      if (p_bf16) p_bf16[k] = __float2bfloat16(P);
    }
  }
}
// Advances the optimizer counters after all shards were updated: step += 1 unless skipped.
__global__ void adamw_finalize_kernel(float* __restrict__ ctrl, float max_norm, int skip_nan_inf, float grad_scale) {
  const float norm = sqrtf(ctrl[0]) * grad_scale;
  const bool bad = !isfinite(norm);
  if (ctrl[5] != 0.f) {
    ctrl[6] += 1.f;
    ctrl[3] = 0.f;
  } else if (bad && skip_nan_inf) {
    ctrl[2] += 1.f;
    ctrl[3] = 0.f;
  } else {
    ctrl[1] += 1.f;
    ctrl[3] = max_norm > 0.f ? fminf(1.f, max_norm / (norm + 1e-6f)) : 1.f;
  }
  ctrl[4] = norm;
}

// Latches the library status word (mapped host memory) into the step's abort flag on the device, so that the update
// kernels of this step read it from device memory.
__global__ void status_to_ctrl_kernel(const int* __restrict__ status, float* __restrict__ ctrl) {
  ctrl[5] = (status != nullptr && *reinterpret_cast<const volatile int*>(status) != 0) ? 1.f : 0.f;
}

__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y, long long n) {
  long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= n) return;
  if (i + 4 <= n) {
    float4 v = *reinterpret_cast<const float4*>(x + i);
    uint2 q;
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    q.x = *reinterpret_cast<uint32_t*>(&a);
    q.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(y + i) = q;
  } else {
    for (long long k = i; k < n; ++k) y[k] = __float2bfloat16(x[k]);
  }
}

inline unsigned blocks_for(long long n, int threads) { return (unsigned)((n + threads - 1) / threads); }

}  // namespace

namespace {
// dst[r, :] = idx[r] >= 0 ? src[idx[r], :] : 0 for rows of `vecs` 16-byte vectors: the padded-chunk pack (rows that pad a
// document come out zero) and its backward in one pass, instead of a fill plus an indexed copy.
__global__ void gather_rows_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, const int* __restrict__ idx,
                                   long long n_dst, int vecs) {
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long r = gid / vecs;
  if (r >= n_dst) return;
  const int v = (int)(gid - r * vecs);
  const int s = idx[r];
  dst[r * vecs + v] = s >= 0 ? src[(long long)s * vecs + v] : make_uint4(0, 0, 0, 0);
}
}  // namespace

extern "C" {

int fb_position_ids(const int* cu_seqlens, int nseq, int* pos, int* seq_id, int total, cudaStream_t stream) {
  if (total == 0) return 0;
  position_ids_kernel<<<blocks_for(total, 256), 256, 0, stream>>>(cu_seqlens, nseq, pos, seq_id, total);
  return fb::launch_ok("position_ids_kernel");
}

// x: bf16 (x_fp32 = 0) or fp32 (x_fp32 = 1) rows of H heads; y: bf16.  Strides are in elements of the own dtype.
// With rot < Dh the features beyond `rot` are left untouched (x and y must then alias or be pre-copied).
int fb_rope(const void* x, void* y, const int* pos, const float* cos_t, const float* sin_t, long long T, int H, int Dh,
            int rot, long long x_stride_t, long long y_stride_t, int seq_len_mod, int conj, int x_fp32,
            cudaStream_t stream) {
  if (T == 0) return 0;
  if ((rot % 16) || (Dh % 8) || (x_stride_t % 8) || (y_stride_t % 8)) return -2;
  long long total = T * H * (rot / 16);
  if (x_fp32)
    rope_kernel<true><<<blocks_for(total, 256), 256, 0, stream>>>(x, (__nv_bfloat16*)y, pos, cos_t, sin_t, T, H, Dh, rot,
                                                                  x_stride_t, y_stride_t, seq_len_mod, conj);
  else
    rope_kernel<false><<<blocks_for(total, 256), 256, 0, stream>>>(x, (__nv_bfloat16*)y, pos, cos_t, sin_t, T, H, Dh, rot,
                                                                   x_stride_t, y_stride_t, seq_len_mod, conj);
  return fb::launch_ok("rope_kernel");
}

int fb_swiglu_fwd(const void* g, const void* u, void* a, long long T, int I, long long ld_g, long long ld_u,
                  long long ld_a, cudaStream_t stream) {
  if (T == 0) return 0;
  if ((I % 8) || (ld_g % 8) || (ld_u % 8) || (ld_a % 8)) return -2;
  swiglu_fwd_kernel<<<blocks_for(T * (I / 8), 256), 256, 0, stream>>>(
      (const __nv_bfloat16*)g, (const __nv_bfloat16*)u, (__nv_bfloat16*)a, T, I, ld_g, ld_u, ld_a);
  return fb::launch_ok("swiglu_fwd_kernel");
}
int fb_swiglu_bwd(const void* da, const void* g, const void* u, void* dg, void* du, void* a_out, long long T, int I,
                  long long ld_da, long long ld_g, long long ld_u, long long ld_dg, long long ld_du, long long ld_a,
                  cudaStream_t stream) {
  if (T == 0) return 0;
  if ((I % 8) || (ld_da % 8) || (ld_g % 8) || (ld_u % 8) || (ld_dg % 8) || (ld_du % 8) || (ld_a % 8)) return -2;
  swiglu_bwd_kernel<<<blocks_for(T * (I / 8), 256), 256, 0, stream>>>(
      (const __nv_bfloat16*)da, (const __nv_bfloat16*)g, (const __nv_bfloat16*)u, (__nv_bfloat16*)dg,
      (__nv_bfloat16*)du, (__nv_bfloat16*)a_out, T, I, ld_da, ld_g, ld_u, ld_dg, ld_du, ld_a);
  return fb::launch_ok("swiglu_bwd_kernel");
}

int fb_count_valid(const long long* targets, long long n, int ignore_index, int* n_valid, cudaStream_t stream) {
  count_valid_kernel<<<1, 1024, 0, stream>>>(targets, n, ignore_index, n_valid);
  return fb::launch_ok("count_valid_kernel");
}
int fb_cross_entropy_opt(void* logits, const long long* targets, float* loss_rows, float* lse_rows, const int* n_valid,
                         float scale_num, long long rows, int V, long long ld, int ignore_index, int write_grad,
                         float label_smoothing, float logit_scale, float lse_square_scale, float softcap,
                         cudaStream_t stream) {
  if (rows == 0) return 0;
  if ((ld % 8) || ((uintptr_t)logits & 15)) return -2;
  CeOptions opt = {label_smoothing, logit_scale, lse_square_scale, softcap};
  cross_entropy_kernel<<<(unsigned)rows, CE_THREADS, 0, stream>>>((__nv_bfloat16*)logits, targets, loss_rows, lse_rows,
                                                                  n_valid, scale_num, V, ld, ignore_index, write_grad, opt);
  return fb::launch_ok("cross_entropy_kernel");
}
int fb_cross_entropy(void* logits, const long long* targets, float* loss_rows, float* lse_rows, const int* n_valid,
                     float scale_num, long long rows, int V, long long ld, int ignore_index, int write_grad,
                     cudaStream_t stream) {
  return fb_cross_entropy_opt(logits, targets, loss_rows, lse_rows, n_valid, scale_num, rows, V, ld, ignore_index,
                              write_grad, 0.f, 1.f, 0.f, 0.f, stream);
}
// stats: fp32 [rows, 3] = (slice max, slice sum of exp(x - max), target logit or 0)
int fb_ce_vp_stats(const void* logits, const long long* targets, float* stats, long long rows, int V, long long ld,
                   long long vocab_start, int ignore_index, cudaStream_t stream) {
  if (rows == 0) return 0;
  if ((ld % 8) || ((uintptr_t)logits & 15)) return -2;
  ce_vp_stats_kernel<<<(unsigned)rows, CE_THREADS, 0, stream>>>((const __nv_bfloat16*)logits, targets, stats, V, ld,
                                                                vocab_start, ignore_index);
  return fb::launch_ok("ce_vp_stats_kernel");
}
// lse: fp32 [rows] global log-sum-exp; logits become the gradient of the mean loss times scale_num
int fb_ce_vp_grad(void* logits, const long long* targets, const float* lse, const int* n_valid, float scale_num,
                  long long rows, int V, long long ld, long long vocab_start, int ignore_index, cudaStream_t stream) {
  if (rows == 0) return 0;
  if ((ld % 8) || ((uintptr_t)logits & 15)) return -2;
  ce_vp_grad_kernel<<<(unsigned)rows, CE_THREADS, 0, stream>>>((__nv_bfloat16*)logits, targets, lse, n_valid, scale_num, V,
                                                               ld, vocab_start, ignore_index);
  return fb::launch_ok("ce_vp_grad_kernel");
}
int fb_mean_loss(const float* rows, long long n, const int* n_valid, float* out, int accumulate, cudaStream_t stream) {
  mean_loss_kernel<<<1, 1024, 0, stream>>>(rows, n, n_valid, out, accumulate);
  return fb::launch_ok("mean_loss_kernel");
}

int fb_embedding_fwd(const long long* ids, const void* table, void* out, long long T, int D, long long V,
                     cudaStream_t stream) {
  if (T == 0) return 0;
  if (D % 8) return -2;
  embedding_fwd_kernel<<<blocks_for(T * (D / 8), 256), 256, 0, stream>>>(ids, (const __nv_bfloat16*)table,
                                                                        (__nv_bfloat16*)out, T, D, V);
  return fb::launch_ok("embedding_fwd_kernel");
}
int fb_embedding_bwd_sorted(const long long* sorted_ids, const long long* perm, const int* seg_start, int nseg,
                            long long T, const void* dout, float* dtable, int D, long long V, cudaStream_t stream) {
  if (nseg == 0) return 0;
  if (D % 8) return -2;
  embedding_bwd_sorted_kernel<<<blocks_for((long long)nseg * 32, 256), 256, 0, stream>>>(
      sorted_ids, perm, seg_start, nseg, T, (const __nv_bfloat16*)dout, dtable, D, V);
  return fb::launch_ok("embedding_bwd_sorted_kernel");
}

// partials must hold fb_sumsq_parts() floats
int fb_sumsq_parts() { return 1184; }
int fb_sumsq(const float* x, long long n, float* partials, float* out, int accumulate, cudaStream_t stream) {
  const int parts = fb_sumsq_parts();
  sumsq_partials_kernel<<<parts, SQ_THREADS, 0, stream>>>(x, n, partials);
  int rc = fb::launch_ok("sumsq_partials_kernel");
  if (rc) return rc;
  sum_partials_kernel<<<1, 1024, 0, stream>>>(partials, parts, out, accumulate);
  return fb::launch_ok("sum_partials_kernel");
}

int fb_adamw(float* p, float* m, float* v, const float* g, void* p_bf16, long long n, float lr, float beta1,
             float beta2, float eps, float wd, float max_norm, int skip_nan_inf, const float* ctrl, float grad_scale,
             cudaStream_t stream) {
  if (n == 0) return 0;
  adamw_kernel<<<blocks_for((n + 3) / 4, 256), 256, 0, stream>>>(p, m, v, g, (__nv_bfloat16*)p_bf16, n, lr, beta1,
                                                                 beta2, eps, wd, max_norm, skip_nan_inf, ctrl,
                                                                 grad_scale);
  return fb::launch_ok("adamw_kernel");
}
int fb_status_to_ctrl(float* ctrl, cudaStream_t stream) {
  status_to_ctrl_kernel<<<1, 1, 0, stream>>>(fb::status_ptr(), ctrl);
  return fb::launch_ok("status_to_ctrl_kernel");
}

int fb_adamw_finalize(float* ctrl, float max_norm, int skip_nan_inf, float grad_scale, cudaStream_t stream) {
  adamw_finalize_kernel<<<1, 1, 0, stream>>>(ctrl, max_norm, skip_nan_inf, grad_scale);
  return fb::launch_ok("adamw_finalize_kernel");
}
int fb_cast_f32_bf16(const float* x, void* y, long long n, cudaStream_t stream) {
  if (n == 0) return 0;
  cast_f32_to_bf16_kernel<<<blocks_for((n + 3) / 4, 256), 256, 0, stream>>>(x, (__nv_bfloat16*)y, n);
  return fb::launch_ok("cast_f32_to_bf16_kernel");
}

// row_bytes must be a multiple of 16 and both buffers 16-byte aligned; idx: int32 [n_dst], -1 = zero row
int fb_gather_rows(const void* src, void* dst, const int* idx, long long n_dst, long long row_bytes, cudaStream_t stream) {
  if (n_dst <= 0 || row_bytes <= 0) return 0;
  if ((row_bytes % 16) || ((uintptr_t)src & 15) || ((uintptr_t)dst & 15)) return -2;
  const int vecs = (int)(row_bytes / 16);
  const long long threads = n_dst * vecs;
  gather_rows_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>((const uint4*)src, (uint4*)dst, idx, n_dst, vecs);
  return fb::launch_ok("gather_rows_kernel");
}

}  // extern "C"
