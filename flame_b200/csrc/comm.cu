// Data-parallel gradient reduction and parameter publication over NVLink peer memory (one process per GPU).
//
// Every rank maps every peer's flat gradient buffer (fp32) and flat parameter buffer (bf16).  Per unit:
//   peer_signal          : "my gradients of unit u are final" -> one flag word on every peer (release, system scope)
//   peer_wait            : bounded spin until all peers raised that flag (acquire, system scope)
//   peer_reduce_scatter  : this rank's 1/N slice = mean over ranks, read straight from the peers' buffers in rank order
//                          (deterministic), written as fp32 together with per-CTA sums of squares (gradient norm)
//   peer_adamw_push      : AdamW on the slice (clip coefficient and NaN/Inf skip decided on the device), bf16 result
//                          stored into EVERY rank's parameter buffer - the all-gather is the optimizer's epilogue
// Plain peer loads/stores only (no multimem, no TMA), so a rank that leaves between steps cannot fault the others.
// These kernels replace FSDP2's NCCL all-gather / reduce-scatter plus its copy-in/copy-out kernels and the separate
// foreach-norm and fused-AdamW launches (torch/distributed/fsdp/_fully_shard/_fsdp_collectives.py:89-146, 448-665).
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <math.h>
#include <stdint.h>
#include "host_utils.cuh"
#include "tc05.cuh"

namespace {

constexpr int MAX_RANKS = 16;
struct PeerPtrs {
  void* p[MAX_RANKS];
};

__device__ __forceinline__ void st_release_sys(int* addr, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* addr) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_peer_f4(const float* addr) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(addr)
               : "memory");
  return v;
}

// flags layout on every rank: [slot][source rank]
__global__ void peer_signal_kernel(PeerPtrs flags, int world, int my_rank, int slot, int value) {
  const int r = threadIdx.x;
  if (r < world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<int*>(flags.p[r]) + slot * MAX_RANKS + my_rank, value);
  }
}

__global__ void peer_wait_kernel(const int* __restrict__ my_flags, int world, int slot, int value, int* status,
                                 unsigned long long limit_ns) {
  const int r = threadIdx.x;
  if (r >= world) return;
  const int* f = my_flags + slot * MAX_RANKS + r;
  const unsigned long long t0 = tc05::globaltimer_ns();
  unsigned spins = 0;
  while (ld_acquire_sys(f) < value) {
    if ((++spins & 0x3FF) == 0 && tc05::globaltimer_ns() - t0 > limit_ns) {
      volatile int* s = status;
      if (*s == 0) *s = (tc05::ERR_WAIT_PEER << 16) | (r & 0xFFFF);
      return;
    }
    __nanosleep(64);
  }
}

// Gather of a flat, evenly sharded byte range: dst[b] = shard_{b / shard_bytes}[b % shard_bytes] for b in [lo, hi), 16
// bytes per thread and step, plain peer loads.  The stand-alone form of the all-gather (small parameters that are needed
// before the first GEMM of a block, the root unit, and every case the fused GEMM does not cover).
__global__ void __launch_bounds__(256)
peer_gather_flat_kernel(PeerPtrs shards, long long shard_bytes, uint8_t* __restrict__ dst, long long lo, long long hi) {
  const long long nvec = (hi - lo) >> 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const long long b = lo + (i << 4);
    const int r = (int)(b / shard_bytes);
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(shards.p[r]) + (b - (long long)r * shard_bytes));
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(src)
                 : "memory");
    *reinterpret_cast<uint4*>(dst + b) = v;
  }
}

constexpr int RS_THREADS = 256;
__global__ void __launch_bounds__(RS_THREADS)
peer_reduce_scatter_kernel(PeerPtrs grads, int world, long long slice_off, long long n, float inv_world,
                           float* __restrict__ out, float* __restrict__ partials, int accumulate) {
  __shared__ float s[RS_THREADS / 32];
  float acc = 0.f;
  const long long nvec = n >> 2;
  for (long long i = (long long)blockIdx.x * RS_THREADS + threadIdx.x; i < nvec; i += (long long)gridDim.x * RS_THREADS) {
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < world; ++r) {
      const float4 v = ld_peer_f4(reinterpret_cast<const float*>(grads.p[r]) + slice_off + i * 4);
      sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
    }
    sum.x *= inv_world; sum.y *= inv_world; sum.z *= inv_world; sum.w *= inv_world;
    if (accumulate) {  // a later micro-batch of the same step: add to what the earlier ones left in the slice
      const float4 o = reinterpret_cast<const float4*>(out)[i];
      sum.x += o.x; sum.y += o.y; sum.z += o.z; sum.w += o.w;
    }
    reinterpret_cast<float4*>(out)[i] = sum;
    acc += sum.x * sum.x + sum.y * sum.y + sum.z * sum.z + sum.w * sum.w;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < RS_THREADS / 32 ? s[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (threadIdx.x == 0) partials[blockIdx.x] = t;
  }
}

__global__ void sum_partials_acc_kernel(const float* __restrict__ partials, int n, float* __restrict__ out) {
  __shared__ float s[32];
  float c = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) c += partials[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? s[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (threadIdx.x == 0) out[0] += t;
  }
}

// AdamW on the local slice; 8 elements per thread; the bf16 result goes to every rank's parameter buffer.
__global__ void peer_adamw_push_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                                       const float* __restrict__ g, PeerPtrs params, int world, long long slice_off,
                                       long long n, float lr, float beta1, float beta2, float eps, float wd,
                                       float max_norm, int skip_nan_inf, const float* __restrict__ ctrl,
                                       float grad_scale) {
  if (ctrl[5] != 0.f) return;  // a bounded wait ran out during this step: the gradients may be incomplete
  const float wd_l2 = wd < 0.f ? -wd : 0.f;  // wd < 0 selects plain Adam: the decay enters through the gradient
  wd = wd < 0.f ? 0.f : wd;
  const float norm = sqrtf(ctrl[0]) * grad_scale;
  const bool bad = !isfinite(norm);
  if (bad && skip_nan_inf) return;  // parameters unchanged everywhere: nothing to publish
  float coef = 1.f;
  if (max_norm > 0.f) coef = fminf(1.f, max_norm / (norm + 1e-6f));
  coef *= grad_scale;
  const float step = ctrl[1] + 1.f;
  const float bc1 = 1.f - powf(beta1, step);
  const float bc2 = 1.f - powf(beta2, step);
  const float step_size = lr / bc1;
  const float inv_sqrt_bc2 = rsqrtf(bc2);
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i >= n) return;  // n is a multiple of 8 (units are padded)
  float P[8], M[8], V[8], G[8];
  *reinterpret_cast<float4*>(&P[0]) = *reinterpret_cast<const float4*>(p + i);
  *reinterpret_cast<float4*>(&P[4]) = *reinterpret_cast<const float4*>(p + i + 4);
  *reinterpret_cast<float4*>(&M[0]) = *reinterpret_cast<const float4*>(m + i);
  *reinterpret_cast<float4*>(&M[4]) = *reinterpret_cast<const float4*>(m + i + 4);
  *reinterpret_cast<float4*>(&V[0]) = *reinterpret_cast<const float4*>(v + i);
  *reinterpret_cast<float4*>(&V[4]) = *reinterpret_cast<const float4*>(v + i + 4);
  *reinterpret_cast<float4*>(&G[0]) = *reinterpret_cast<const float4*>(g + i);
  *reinterpret_cast<float4*>(&G[4]) = *reinterpret_cast<const float4*>(g + i + 4);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float gr = G[j] * coef + wd_l2 * P[j];
    P[j] *= (1.f - lr * wd);
    M[j] = beta1 * M[j] + (1.f - beta1) * gr;
    V[j] = beta2 * V[j] + (1.f - beta2) * gr * gr;
    P[j] -= step_size * M[j] / (sqrtf(V[j]) * inv_sqrt_bc2 + eps);
  }
  *reinterpret_cast<float4*>(p + i) = *reinterpret_cast<float4*>(&P[0]);
  *reinterpret_cast<float4*>(p + i + 4) = *reinterpret_cast<float4*>(&P[4]);
  *reinterpret_cast<float4*>(m + i) = *reinterpret_cast<float4*>(&M[0]);
  *reinterpret_cast<float4*>(m + i + 4) = *reinterpret_cast<float4*>(&M[4]);
  *reinterpret_cast<float4*>(v + i) = *reinterpret_cast<float4*>(&V[0]);
  *reinterpret_cast<float4*>(v + i + 4) = *reinterpret_cast<float4*>(&V[4]);
  uint4 q;
  q.x = tc05::pack_bf16(P[0], P[1]);
  q.y = tc05::pack_bf16(P[2], P[3]);
  q.z = tc05::pack_bf16(P[4], P[5]);
  q.w = tc05::pack_bf16(P[6], P[7]);
  for (int r = 0; r < world; ++r)
    *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(params.p[r]) + slice_off + i) = q;
}

PeerPtrs to_ptrs(const unsigned long long* ptrs, int world) {
  PeerPtrs pp;
  for (int r = 0; r < MAX_RANKS; ++r) pp.p[r] = r < world ? (void*)ptrs[r] : nullptr;
  return pp;
}

}  // namespace

extern "C" {

int fb_peer_reduce_scatter_acc(const unsigned long long* grad_ptrs, int world, long long slice_off, long long n, float* out,
                               float* partials, float* norm_sq_out, int accumulate, cudaStream_t stream);
int fb_peer_max_ranks() { return MAX_RANKS; }
int fb_peer_rs_parts() { return 592; }

int fb_peer_signal(const unsigned long long* flag_ptrs, int world, int my_rank, int slot, int value,
                   cudaStream_t stream) {
  if (world > MAX_RANKS) return -2;
  peer_signal_kernel<<<1, 32, 0, stream>>>(to_ptrs(flag_ptrs, world), world, my_rank, slot, value);
  return fb::launch_ok("peer_signal_kernel");
}

int fb_peer_wait(const int* my_flags, int world, int slot, int value, double limit_seconds, cudaStream_t stream) {
  if (world > MAX_RANKS) return -2;
  peer_wait_kernel<<<1, 32, 0, stream>>>(my_flags, world, slot, value, fb::status_ptr(),
                                         (unsigned long long)(limit_seconds * 1e9));
  return fb::launch_ok("peer_wait_kernel");
}

// out[n] = mean_r grads_r[slice_off + i]; norm_sq_out[0] += sum(out^2).  n must be a multiple of 4.
int fb_peer_reduce_scatter(const unsigned long long* grad_ptrs, int world, long long slice_off, long long n, float* out,
                           float* partials, float* norm_sq_out, cudaStream_t stream) {
  return fb_peer_reduce_scatter_acc(grad_ptrs, world, slice_off, n, out, partials, norm_sq_out, 0, stream);
}

// As above; with `accumulate` the mean is added to `out` (gradient accumulation over micro-batches when the full
// gradient buffer is recycled between them), and norm_sq_out may be null (only the last micro-batch contributes the
// norm of the accumulated slice).
int fb_peer_reduce_scatter_acc(const unsigned long long* grad_ptrs, int world, long long slice_off, long long n, float* out,
                               float* partials, float* norm_sq_out, int accumulate, cudaStream_t stream) {
  if (world > MAX_RANKS || (n & 3)) return -2;
  const int parts = fb_peer_rs_parts();
  peer_reduce_scatter_kernel<<<parts, RS_THREADS, 0, stream>>>(to_ptrs(grad_ptrs, world), world, slice_off, n,
                                                               1.f / (float)world, out, partials, accumulate);
  int rc = fb::launch_ok("peer_reduce_scatter_kernel");
  if (rc || norm_sq_out == nullptr) return rc;
  sum_partials_acc_kernel<<<1, 1024, 0, stream>>>(partials, parts, norm_sq_out);
  return fb::launch_ok("sum_partials_acc_kernel");
}

// dst[lo, hi) of a flat buffer <- the ranks' shards (see peer_gather_flat_kernel); lo, hi, shard_bytes multiples of 16.
int fb_peer_gather_flat(const unsigned long long* shard_ptrs, int world, long long shard_bytes, void* dst, long long lo,
                        long long hi, cudaStream_t stream) {
  if (world > MAX_RANKS || (lo & 15) || (hi & 15) || (shard_bytes & 15) || hi > shard_bytes * world || lo < 0) return -2;
  if (hi <= lo) return 0;
  const long long nvec = (hi - lo) >> 4;
  long long blocks = (nvec + 255) / 256;
  if (blocks > 1184) blocks = 1184;  // 8 CTAs of 256 threads per SM
  peer_gather_flat_kernel<<<(unsigned)blocks, 256, 0, stream>>>(to_ptrs(shard_ptrs, world), shard_bytes, (uint8_t*)dst, lo, hi);
  return fb::launch_ok("peer_gather_flat_kernel");
}

int fb_peer_adamw_push(float* p, float* m, float* v, const float* g, const unsigned long long* param_ptrs, int world,
                       long long slice_off, long long n, float lr, float beta1, float beta2, float eps, float wd,
                       float max_norm, int skip_nan_inf, const float* ctrl, float grad_scale, cudaStream_t stream) {
  if (world > MAX_RANKS || (n & 7)) return -2;
  const long long threads = n / 8;
  peer_adamw_push_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>(
      p, m, v, g, to_ptrs(param_ptrs, world), world, slice_off, n, lr, beta1, beta2, eps, wd, max_norm, skip_nan_inf,
      ctrl, grad_scale);
  return fb::launch_ok("peer_adamw_push_kernel");
}

}  // extern "C"
