// Mamba-1 selective scan, forward and backward, chunk-parallel (state size N = 16).
//
//   h_t[d, n] = exp(delta_t[d] A[d, n]) h_{t-1}[d, n] + delta_t[d] B_t[n] u_t[d],     y_t[d] = sum_n h_t[d, n] C_t[n] + D[d] u_t[d]
//
// Tokens are laid out in 64-token chunks that never straddle a document ([NC, 64, ...], zero rows as padding: delta = 0
// leaves the state untouched).  A thread owns ONE state element (d, n) of one chunk, so the 64 states of a chunk fit in
// registers for the backward pass and every reduction over n is a 16-lane shuffle.
//   forward:  (1) chunk-local end state from a zero start and the chunk's total decay P = exp(A sum delta)
//             (2) carry across the chunks of each document: h_in[c+1] = P[c] h_in[c] + h_loc[c]
//             (3) outputs from the true chunk-start state
//   backward: (4) chunk-local adjoint of the chunk-start state, (5) reverse carry, (6) all gradients with the states of
//             the chunk recomputed into registers.
// Replaces the sequential loop of fla/layers/mamba.py:361-397 (the reference's fast path, mamba_ssm's CUDA scan, is not
// installed in the reference environment).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "host_utils.cuh"

namespace {

constexpr int N = 16;    // state size
constexpr int L = 64;    // chunk length
constexpr int DB = 32;   // channels per block
constexpr int THREADS = DB * N;

struct ScanArgs {
  const __nv_bfloat16* u;   // [NC, L, Di]
  const float* dl;          // [NC, L, Di]
  const float* A;           // [Di, N]
  const float* B;           // [NC, L, N]
  const float* C;           // [NC, L, N]
  const float* Dv;          // [Di]
  int Di;
};

// (1) and (4): one sweep over the chunk from a zero state / zero adjoint
template <bool REVERSE>
__global__ void __launch_bounds__(THREADS) sscan_local_kernel(ScanArgs a, const __nv_bfloat16* __restrict__ dy,
                                                              float* __restrict__ loc, float* __restrict__ P) {
  const int n = threadIdx.x & (N - 1);
  const int d = blockIdx.y * DB + (threadIdx.x >> 4);
  const long long c = blockIdx.x;
  if (d >= a.Di) return;
  const float An = a.A[(long long)d * N + n];
  const long long row0 = c * L;
  if (!REVERSE) {
    float h = 0.f, sdl = 0.f;
#pragma unroll 8
    for (int t = 0; t < L; ++t) {
      const float dlt = a.dl[(row0 + t) * a.Di + d];
      const float uu = __bfloat162float(a.u[(row0 + t) * a.Di + d]);
      h = fmaf(__expf(dlt * An), h, dlt * uu * a.B[(row0 + t) * N + n]);
      sdl += dlt;
    }
    loc[(c * a.Di + d) * N + n] = h;
    P[(c * a.Di + d) * N + n] = __expf(An * sdl);
  } else {
    // g_t = C_t dy_t + a_{t+1} g_{t+1}; result: adjoint of the state entering the chunk = a_0 g_0
    float g = 0.f, a_next = 0.f;
#pragma unroll 8
    for (int t = L - 1; t >= 0; --t) {
      const float dlt = a.dl[(row0 + t) * a.Di + d];
      const float dyv = __bfloat162float(dy[(row0 + t) * a.Di + d]);
      g = fmaf(a_next, g, a.C[(row0 + t) * N + n] * dyv);
      a_next = __expf(dlt * An);
    }
    loc[(c * a.Di + d) * N + n] = a_next * g;
  }
}

// (2) and (5): carry over the chunks of each document.  forward: in[c] = state entering chunk c; reverse: in[c] = adjoint
// of the state leaving chunk c.
__global__ void sscan_carry_kernel(const long long* __restrict__ first, const long long* __restrict__ last,
                                   const float* __restrict__ loc, const float* __restrict__ P, float* __restrict__ in, int DiN,
                                   int reverse) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= DiN) return;
  const int doc = blockIdx.y;
  const long long c0 = first[doc], c1 = last[doc];
  float s = 0.f;
  if (!reverse) {
    for (long long c = c0; c <= c1; ++c) {
      in[c * DiN + e] = s;
      s = fmaf(P[c * DiN + e], s, loc[c * DiN + e]);
    }
  } else {
    for (long long c = c1; c >= c0; --c) {
      in[c * DiN + e] = s;
      s = fmaf(P[c * DiN + e], s, loc[c * DiN + e]);
    }
  }
}

// (3): outputs from the true chunk-start state
__global__ void __launch_bounds__(THREADS) sscan_out_kernel(ScanArgs a, const float* __restrict__ hin, __nv_bfloat16* __restrict__ y) {
  const int n = threadIdx.x & (N - 1);
  const int d = blockIdx.y * DB + (threadIdx.x >> 4);
  const long long c = blockIdx.x;
  if (d >= a.Di) return;
  const float An = a.A[(long long)d * N + n];
  const float Dd = a.Dv[d];
  const long long row0 = c * L;
  float h = hin[(c * a.Di + d) * N + n];
#pragma unroll 8
  for (int t = 0; t < L; ++t) {
    const float dlt = a.dl[(row0 + t) * a.Di + d];
    const float uu = __bfloat162float(a.u[(row0 + t) * a.Di + d]);
    h = fmaf(__expf(dlt * An), h, dlt * uu * a.B[(row0 + t) * N + n]);
    float yv = h * a.C[(row0 + t) * N + n];
#pragma unroll
    for (int o = N / 2; o > 0; o >>= 1) yv += __shfl_xor_sync(0xffffffffu, yv, o);
    if (n == 0) y[(row0 + t) * a.Di + d] = __float2bfloat16(fmaf(Dd, uu, yv));
  }
}

// (6): all gradients of one chunk.  gout[c] is the adjoint of the state leaving the chunk.
__global__ void __launch_bounds__(THREADS) sscan_bwd_kernel(ScanArgs a, const __nv_bfloat16* __restrict__ dy,
                                                            const float* __restrict__ hin, const float* __restrict__ gout,
                                                            float* __restrict__ du, float* __restrict__ ddl, float* __restrict__ dA,
                                                            float* __restrict__ dB, float* __restrict__ dC, float* __restrict__ dD) {
  __shared__ float sB[L * N], sC[L * N];
  const int n = threadIdx.x & (N - 1);
  const int d = blockIdx.y * DB + (threadIdx.x >> 4);
  const long long c = blockIdx.x;
  for (int i = threadIdx.x; i < L * N; i += THREADS) {
    sB[i] = 0.f;
    sC[i] = 0.f;
  }
  __syncthreads();
  const bool live = d < a.Di;
  const int dd = live ? d : a.Di - 1;  // dead threads shadow a live channel and contribute nothing
  const float An = a.A[(long long)dd * N + n];
  const float Dd = a.Dv[dd];
  const long long row0 = c * L;
  float hprev[L];
  float h = hin[(c * a.Di + dd) * N + n];
#pragma unroll
  for (int t = 0; t < L; ++t) {
    hprev[t] = h;
    const float dlt = a.dl[(row0 + t) * a.Di + dd];
    const float uu = __bfloat162float(a.u[(row0 + t) * a.Di + dd]);
    h = fmaf(__expf(dlt * An), h, dlt * uu * a.B[(row0 + t) * N + n]);
  }
  float carry = gout[(c * a.Di + dd) * N + n];  // a_{t+1} g_{t+1} for t = L-1
  float dA_acc = 0.f, dD_acc = 0.f;
#pragma unroll
  for (int t = L - 1; t >= 0; --t) {
    const float dlt = a.dl[(row0 + t) * a.Di + dd];
    const float uu = __bfloat162float(a.u[(row0 + t) * a.Di + dd]);
    const float bt = a.B[(row0 + t) * N + n], ct = a.C[(row0 + t) * N + n];
    const float dyv = live ? __bfloat162float(dy[(row0 + t) * a.Di + dd]) : 0.f;
    const float at = __expf(dlt * An);
    const float g = live ? fmaf(ct, dyv, carry) : 0.f;
    const float ht = fmaf(at, hprev[t], dlt * uu * bt);
    const float ah = at * hprev[t];
    float vb = g * dlt * uu, vc = ht * dyv;
    float vdl = g * fmaf(An, ah, bt * uu), vdu = g * dlt * bt;
    dA_acc = fmaf(g * dlt, ah, dA_acc);
    carry = at * g;
    // over the 16 states of this channel
#pragma unroll
    for (int o = N / 2; o > 0; o >>= 1) {
      vdl += __shfl_xor_sync(0xffffffffu, vdl, o);
      vdu += __shfl_xor_sync(0xffffffffu, vdu, o);
    }
    if (n == 0 && live) {
      ddl[(row0 + t) * a.Di + d] = vdl;
      du[(row0 + t) * a.Di + d] = fmaf(Dd, dyv, vdu);
      dD_acc = fmaf(dyv, uu, dD_acc);
    }
    // over the channels: the two channels of the warp, then the block through shared memory
    vb += __shfl_xor_sync(0xffffffffu, vb, 16);
    vc += __shfl_xor_sync(0xffffffffu, vc, 16);
    if ((threadIdx.x & 31) < N) {
      atomicAdd(&sB[t * N + n], vb);
      atomicAdd(&sC[t * N + n], vc);
    }
  }
  if (live) {
    atomicAdd(&dA[(long long)d * N + n], dA_acc);
    if (n == 0) atomicAdd(&dD[d], dD_acc);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < L * N; i += THREADS) {
    atomicAdd(&dB[row0 * N + i], sB[i]);
    atomicAdd(&dC[row0 * N + i], sC[i]);
  }
}

}  // namespace

extern "C" {

// Forward.  hloc, P, hin: fp32 [NC, Di, 16] scratch (hin and P are kept for the backward); y: bf16 [NC, 64, Di].
int fb_sscan_fwd(const void* u, const float* dl, const float* A, const float* B, const float* C, const float* Dv,
                 const long long* first, const long long* last, int n_docs, float* hloc, float* P, float* hin, void* y, int NC,
                 int Di, int n_state, cudaStream_t stream) {
  if (NC <= 0) return 0;
  if (n_state != N) return -2;
  ScanArgs a{(const __nv_bfloat16*)u, dl, A, B, C, Dv, Di};
  dim3 grid(NC, (Di + DB - 1) / DB);
  sscan_local_kernel<false><<<grid, THREADS, 0, stream>>>(a, nullptr, hloc, P);
  int rc = fb::launch_ok("sscan_local_kernel");
  if (rc) return rc;
  const int DiN = Di * N;
  sscan_carry_kernel<<<dim3((DiN + 255) / 256, n_docs), 256, 0, stream>>>(first, last, hloc, P, hin, DiN, 0);
  rc = fb::launch_ok("sscan_carry_kernel");
  if (rc) return rc;
  sscan_out_kernel<<<grid, THREADS, 0, stream>>>(a, hin, (__nv_bfloat16*)y);
  return fb::launch_ok("sscan_out_kernel");
}

// Backward.  gloc, gout: fp32 [NC, Di, 16] scratch; du, ddl: fp32 [NC, 64, Di]; dA [Di, 16], dB, dC [NC, 64, 16], dD [Di]
// must be zero on entry (they are accumulated into).
int fb_sscan_bwd(const void* u, const float* dl, const float* A, const float* B, const float* C, const float* Dv, const void* dy,
                 const long long* first, const long long* last, int n_docs, const float* P, const float* hin, float* gloc,
                 float* gout, float* du, float* ddl, float* dA, float* dB, float* dC, float* dD, int NC, int Di, int n_state,
                 cudaStream_t stream) {
  if (NC <= 0) return 0;
  if (n_state != N) return -2;
  ScanArgs a{(const __nv_bfloat16*)u, dl, A, B, C, Dv, Di};
  dim3 grid(NC, (Di + DB - 1) / DB);
  sscan_local_kernel<true><<<grid, THREADS, 0, stream>>>(a, (const __nv_bfloat16*)dy, gloc, nullptr);
  int rc = fb::launch_ok("sscan_local_kernel(reverse)");
  if (rc) return rc;
  const int DiN = Di * N;
  sscan_carry_kernel<<<dim3((DiN + 255) / 256, n_docs), 256, 0, stream>>>(first, last, gloc, P, gout, DiN, 1);
  rc = fb::launch_ok("sscan_carry_kernel(reverse)");
  if (rc) return rc;
  sscan_bwd_kernel<<<grid, THREADS, 0, stream>>>(a, (const __nv_bfloat16*)dy, hin, gout, du, ddl, dA, dB, dC, dD);
  return fb::launch_ok("sscan_bwd_kernel");
}

}  // extern "C"
