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

// Stages a chunk's operands of the block's 32 channels in shared memory with coalesced loads; the time loops then read
// broadcast values from shared memory instead of issuing two-address global loads at every step.
struct Tile {
  float* dl;  // [L][DB]
  float* u;   // [L][DB]
  float* dy;  // [L][DB]
  float* B;   // [L][N]
  float* C;   // [L][N]
};
__device__ __forceinline__ Tile carve(float* sm) { return Tile{sm, sm + L * DB, sm + 2 * L * DB, sm + 3 * L * DB, sm + 3 * L * DB + L * N}; }
constexpr int TILE_FLOATS = 3 * L * DB + 2 * L * N;

__device__ __forceinline__ void stage(const ScanArgs& a, const __nv_bfloat16* dy, long long row0, int d0, const Tile& s, bool want_u,
                                      bool want_dy, bool want_B, bool want_C) {
  for (int idx = threadIdx.x; idx < L * DB; idx += THREADS) {
    const int t = idx / DB, dd = idx - t * DB;
    const int d = d0 + dd;
    const bool ok = d < a.Di;
    const long long g = (row0 + t) * a.Di + d;
    s.dl[idx] = ok ? a.dl[g] : 0.f;
    if (want_u) s.u[idx] = ok ? __bfloat162float(a.u[g]) : 0.f;
    if (want_dy) s.dy[idx] = ok ? __bfloat162float(dy[g]) : 0.f;
  }
  for (int idx = threadIdx.x; idx < L * N; idx += THREADS) {
    if (want_B) s.B[idx] = a.B[row0 * N + idx];
    if (want_C) s.C[idx] = a.C[row0 * N + idx];
  }
  __syncthreads();
}

// (1) and (4): one sweep over the chunk from a zero state / zero adjoint
template <bool REVERSE>
__global__ void __launch_bounds__(THREADS) sscan_local_kernel(ScanArgs a, const __nv_bfloat16* __restrict__ dy,
                                                              float* __restrict__ loc, float* __restrict__ P) {
  extern __shared__ float sm[];
  const Tile s = carve(sm);
  const int n = threadIdx.x & (N - 1);
  const int dloc = threadIdx.x >> 4;
  const int d = blockIdx.y * DB + dloc;
  const long long c = blockIdx.x;
  stage(a, dy, c * L, blockIdx.y * DB, s, !REVERSE, REVERSE, !REVERSE, REVERSE);
  if (d >= a.Di) return;
  const float An = a.A[(long long)d * N + n];
  if (!REVERSE) {
    float h = 0.f, sdl = 0.f;
#pragma unroll 8
    for (int t = 0; t < L; ++t) {
      const float dlt = s.dl[t * DB + dloc];
      h = fmaf(__expf(dlt * An), h, dlt * s.u[t * DB + dloc] * s.B[t * N + n]);
      sdl += dlt;
    }
    loc[(c * a.Di + d) * N + n] = h;
    P[(c * a.Di + d) * N + n] = __expf(An * sdl);
  } else {
    // g_t = C_t dy_t + a_{t+1} g_{t+1}; result: adjoint of the state entering the chunk = a_0 g_0
    float g = 0.f, a_next = 0.f;
#pragma unroll 8
    for (int t = L - 1; t >= 0; --t) {
      g = fmaf(a_next, g, s.C[t * N + n] * s.dy[t * DB + dloc]);
      a_next = __expf(s.dl[t * DB + dloc] * An);
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
  extern __shared__ float sm[];
  const Tile s = carve(sm);
  const int n = threadIdx.x & (N - 1);
  const int dloc = threadIdx.x >> 4;
  const int d = blockIdx.y * DB + dloc;
  const long long c = blockIdx.x;
  const long long row0 = c * L;
  stage(a, nullptr, row0, blockIdx.y * DB, s, true, false, true, true);
  if (d >= a.Di) return;
  const float An = a.A[(long long)d * N + n];
  const float Dd = a.Dv[d];
  float h = hin[(c * a.Di + d) * N + n];
#pragma unroll 8
  for (int t = 0; t < L; ++t) {
    const float dlt = s.dl[t * DB + dloc], uu = s.u[t * DB + dloc];
    h = fmaf(__expf(dlt * An), h, dlt * uu * s.B[t * N + n]);
    float yv = h * s.C[t * N + n];
#pragma unroll
    for (int o = N / 2; o > 0; o >>= 1) yv += __shfl_xor_sync(0xffffffffu, yv, o);
    if (n == 0) y[(row0 + t) * a.Di + d] = __float2bfloat16(fmaf(Dd, uu, yv));
  }
}

// (6): all gradients of one chunk.  gout[c] is the adjoint of the state leaving the chunk.  The sums over the block's
// channels (dB, dC) go through per-warp private slices of shared memory: a warp visits every (t, n) exactly once, so it
// stores instead of accumulating and no atomics are needed; the slices are added at the end.
constexpr int WARPS_PER_BLOCK = THREADS / 32;
constexpr int BWD_SMEM_FLOATS = TILE_FLOATS + 2 * WARPS_PER_BLOCK * L * N;
__global__ void __launch_bounds__(THREADS, 1) sscan_bwd_kernel(ScanArgs a, const __nv_bfloat16* __restrict__ dy,
                                                            const float* __restrict__ hin, const float* __restrict__ gout,
                                                            float* __restrict__ du, float* __restrict__ ddl, float* __restrict__ dA,
                                                            float* __restrict__ dB, float* __restrict__ dC, float* __restrict__ dD) {
  extern __shared__ float sm[];
  const Tile s = carve(sm);
  float* wB = sm + TILE_FLOATS;                       // [WARPS][L][N]
  float* wC = wB + WARPS_PER_BLOCK * L * N;
  const int n = threadIdx.x & (N - 1);
  const int dloc = threadIdx.x >> 4;
  const int warp = threadIdx.x >> 5;
  const int d = blockIdx.y * DB + dloc;
  const long long c = blockIdx.x;
  const long long row0 = c * L;
  stage(a, dy, row0, blockIdx.y * DB, s, true, true, true, true);
  const bool live = d < a.Di;
  const int dd = live ? d : a.Di - 1;  // dead channels were staged as zeros (delta = u = dy = 0): they contribute nothing
  const float An = a.A[(long long)dd * N + n];
  const float Dd = a.Dv[dd];
  // The chunk is differentiated in two halves of 32 steps so that only 32 recomputed states live in registers: the
  // second half first (its entering state comes from a forward sweep over the first half), then the first half.
  constexpr int HL = L / 2;
  const float h0 = live ? hin[(c * a.Di + dd) * N + n] : 0.f;
  float carry = live ? gout[(c * a.Di + dd) * N + n] : 0.f;  // a_{t+1} g_{t+1} for t = L-1
  float dA_acc = 0.f, dD_acc = 0.f;
  auto fwd_step = [&](float h, int t) {
    const float dlt = s.dl[t * DB + dloc];
    return fmaf(__expf(dlt * An), h, dlt * s.u[t * DB + dloc] * s.B[t * N + n]);
  };
  auto rev_step = [&](int t, float hp) {
    const float dlt = s.dl[t * DB + dloc], uu = s.u[t * DB + dloc], dyv = s.dy[t * DB + dloc];
    const float bt = s.B[t * N + n], ct = s.C[t * N + n];
    const float at = __expf(dlt * An);
    const float g = fmaf(ct, dyv, carry);
    const float ah = at * hp;
    const float ht = fmaf(dlt * uu, bt, ah);
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
    // over the channels: the two channels of the warp by shuffle, the warps through their private slices
    vb += __shfl_xor_sync(0xffffffffu, vb, 16);
    vc += __shfl_xor_sync(0xffffffffu, vc, 16);
    if ((threadIdx.x & 31) < N) {
      wB[(warp * L + t) * N + n] = vb;
      wC[(warp * L + t) * N + n] = vc;
    }
  };
  float hp[HL];
  {
    float h = h0;
#pragma unroll 8
    for (int t = 0; t < HL; ++t) h = fwd_step(h, t);
#pragma unroll
    for (int t = 0; t < HL; ++t) {
      hp[t] = h;
      h = fwd_step(h, HL + t);
    }
#pragma unroll
    for (int t = HL - 1; t >= 0; --t) rev_step(HL + t, hp[t]);
  }
  {
    float h = h0;
#pragma unroll
    for (int t = 0; t < HL; ++t) {
      hp[t] = h;
      h = fwd_step(h, t);
    }
#pragma unroll
    for (int t = HL - 1; t >= 0; --t) rev_step(t, hp[t]);
  }
  // partial results without global atomics: dA / dD per chunk, dB / dC per (channel block, chunk); the host sums them
  if (live) {
    dA[(c * a.Di + d) * N + n] = dA_acc;
    if (n == 0) dD[c * a.Di + d] = dD_acc;
  }
  __syncthreads();
  const long long part = ((long long)blockIdx.y * gridDim.x + c) * (L * N);
  for (int i = threadIdx.x; i < L * N; i += THREADS) {
    float sb = 0.f, sc = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS_PER_BLOCK; ++w) {
      sb += wB[w * L * N + i];
      sc += wC[w * L * N + i];
    }
    dB[part + i] = sb;
    dC[part + i] = sc;
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
  const int tile_bytes = TILE_FLOATS * 4;
  sscan_local_kernel<false><<<grid, THREADS, tile_bytes, stream>>>(a, nullptr, hloc, P);
  int rc = fb::launch_ok("sscan_local_kernel");
  if (rc) return rc;
  const int DiN = Di * N;
  sscan_carry_kernel<<<dim3((DiN + 255) / 256, n_docs), 256, 0, stream>>>(first, last, hloc, P, hin, DiN, 0);
  rc = fb::launch_ok("sscan_carry_kernel");
  if (rc) return rc;
  sscan_out_kernel<<<grid, THREADS, tile_bytes, stream>>>(a, hin, (__nv_bfloat16*)y);
  return fb::launch_ok("sscan_out_kernel");
}

// Backward.  gloc, gout: fp32 [NC, Di, 16] scratch; du, ddl: fp32 [NC, 64, Di].  Partial sums for the caller to reduce over
// their leading dimension: dA [NC, Di, 16], dD [NC, Di], dB, dC [fb_sscan_channel_blocks(Di), NC, 64, 16].
int fb_sscan_bwd(const void* u, const float* dl, const float* A, const float* B, const float* C, const float* Dv, const void* dy,
                 const long long* first, const long long* last, int n_docs, const float* P, const float* hin, float* gloc,
                 float* gout, float* du, float* ddl, float* dA, float* dB, float* dC, float* dD, int NC, int Di, int n_state,
                 cudaStream_t stream) {
  if (NC <= 0) return 0;
  if (n_state != N) return -2;
  ScanArgs a{(const __nv_bfloat16*)u, dl, A, B, C, Dv, Di};
  dim3 grid(NC, (Di + DB - 1) / DB);
  const int tile_bytes = TILE_FLOATS * 4;
  sscan_local_kernel<true><<<grid, THREADS, tile_bytes, stream>>>(a, (const __nv_bfloat16*)dy, gloc, nullptr);
  int rc = fb::launch_ok("sscan_local_kernel(reverse)");
  if (rc) return rc;
  const int DiN = Di * N;
  sscan_carry_kernel<<<dim3((DiN + 255) / 256, n_docs), 256, 0, stream>>>(first, last, gloc, P, gout, DiN, 1);
  rc = fb::launch_ok("sscan_carry_kernel(reverse)");
  if (rc) return rc;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(sscan_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BWD_SMEM_FLOATS * 4) != cudaSuccess) return -3;
    configured = true;
  }
  sscan_bwd_kernel<<<grid, THREADS, BWD_SMEM_FLOATS * 4, stream>>>(a, (const __nv_bfloat16*)dy, hin, gout, du, ddl, dA, dB, dC, dD);
  return fb::launch_ok("sscan_bwd_kernel");
}

int fb_sscan_channel_blocks(int Di) { return (Di + DB - 1) / DB; }

}  // extern "C"
