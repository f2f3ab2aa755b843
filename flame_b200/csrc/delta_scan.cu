// Chunk-state recurrence of the (gated) delta rule as ONE persistent launch per direction (sm_100a).
//
//   forward :  S_{c+1} = alpha_c S_c - M_c   S_c     + B_c      S = 0 at the first chunk of a document
//   reverse :  L_c     = alpha_c L_{c+1} - M_c^T L_{c+1} + G_c  L = G at the last chunk of a document
//
// with M_c = khat_c^T w_c  [dk, dk] (the chunk transition), B_c = khat_c^T u_c  [dk, dv], G_c = dL/dS_c, all bf16 and
// produced by batched GEMMs.  The recurrence is sequential along the chunks of one document but independent across
// (document, head, 128-wide slice of dv), so each CTA owns one such triple and walks its chunks with the state resident:
// fp32 in tensor memory, a bf16 copy in shared memory as the B operand of the next step's MMA.  One step is
//   T = op(M_c) S16          one tcgen05 product, A tiles streamed by TMA through a two-stage ring
//   S = alpha_c S - T + add  by the four epilogue warps (a thread owns state rows r and r + 128), written back to tensor
//                            memory, to shared memory (bf16, the MN-major B layout) and to global memory (bf16: the state
//                            that the output stage and the backward pass read).
// It replaces one batched-GEMM launch per chunk position (about 20 us each, 2 x 63 of them per layer at 4096-token
// documents) by a walk that costs a few microseconds per step.  Role of the reference's chunk_gated_delta_rule_fwd_h /
// bwd_dhu kernels (fla/ops/common/chunk_delta_h.py:41-313), in the chunk-transition-matrix form of this library.
#include "tc05.cuh"
#include "host_utils.cuh"

using namespace tc05;

namespace {

constexpr int BN = 128;     // dv columns per CTA
constexpr int STAGES = 2;

struct ScanParams {
  const int* first;        // [n_docs] first chunk of every document
  const int* last;         // [n_docs] last chunk
  int n_docs, H, NC, dk, dv;
  int reverse;
  const float* alpha;      // [NC, H]
  const __nv_bfloat16* add;  // forward: B [NC, H, dk, dv]; reverse: G [NC (+1), H, dk, dv]
  __nv_bfloat16* out;      // forward: S16 [NC + 1, H, dk, dv] (chunk c + 1 receives the state after chunk c);
                           // reverse: L16 [NC + 1, H, dk, dv] (chunk c receives L_c; L16[last] = G[last] is the caller's)
  int* status;
};

template <int DK>
struct Smem {
  static constexpr int S_BYTES = DK * BN * 2;          // bf16 state: 2 column groups of [DK rows][64]
  static constexpr int STAGE_BYTES = DK * 64 * 2;      // one 64-wide k-block of M (either orientation)
  static constexpr int S_OFF = 0;
  static constexpr int RING_OFF = S_BYTES;
  static constexpr int BAR_OFF = RING_OFF + STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFF + 128 + 1024;
};

__device__ __forceinline__ uint32_t sw128(int row, int col) {  // byte offset inside a [rows][64] bf16 group, 128-byte swizzle
  return (uint32_t)(row * 128 + (((col >> 3) ^ (row & 7)) << 4) + (col & 7) * 2);
}

template <int DK>
__global__ void __launch_bounds__(192, DK == 128 ? 2 : 1)
delta_scan_kernel(const __grid_constant__ CUtensorMap tmM, ScanParams p) {
  using L = Smem<DK>;
  constexpr int HALVES = DK / 128;
  constexpr int KB = DK / 64;
  constexpr uint32_t TCOLS = HALVES * 2 * BN;  // T and the fp32 state, per half
  const int vt = blockIdx.x, head = blockIdx.y, doc = blockIdx.z;
  const int c_first = p.first[doc], c_last = p.last[doc];
  const int n_steps = c_last - c_first;   // chunks that have a successor
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sS = smem + L::S_OFF;
  uint64_t* full_bar = (uint64_t*)(smem + L::BAR_OFF);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* t_full = empty_bar + STAGES;
  uint64_t* s_ready = t_full + 1;
  uint32_t* tmem_slot = (uint32_t*)(s_ready + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const long long mat = (long long)DK * p.dv;                        // elements of one [dk, dv] state
  const long long col0 = (long long)vt * BN;
  auto state_ptr = [&](const __nv_bfloat16* base, int chunk, int row) {
    return base + ((long long)chunk * p.H + head) * mat + (long long)row * p.dv + col0;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(t_full, 1);
    mbar_init(s_ready, 128);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmM);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TCOLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // per half h: T at columns [h * 2 * BN, +BN), fp32 state at [h * 2 * BN + BN, +BN)

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      int n = 0;
      for (int s = 0; s < n_steps && ok; ++s) {
        const int c = p.reverse ? c_last - 1 - s : c_first + s;
        const int row_base = (c * p.H + head) * DK;
        for (int kb = 0; kb < KB && ok; ++kb, ++n) {
          const int stage = n % STAGES;
          if (!mbar_wait(&empty_bar[stage], ((n / STAGES) & 1) ^ 1, p.status, abort_flag, ERR_WAIT_EMPTY)) { ok = false; break; }
          uint8_t* dst = smem + L::RING_OFF + stage * L::STAGE_BYTES;
          mbar_expect_tx(&full_bar[stage], L::STAGE_BYTES);
          // forward: A = M (K-major): rows i in blocks of 64, columns j = kb * 64 ..   -> block b at dst + b * 8 KB
          // reverse: A = M^T (MN-major): rows j = kb * 64 .., columns i in groups of 64 -> group g at dst + g * 8 KB
#pragma unroll
          for (int b = 0; b < KB; ++b) {
            if (!p.reverse) tma_load_2d(dst + b * 8192, &tmM, &full_bar[stage], kb * 64, row_base + b * 64);
            else            tma_load_2d(dst + b * 8192, &tmM, &full_bar[stage], b * 64, row_base + kb * 64);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_f = make_idesc_bf16(128, BN, 0, 1);   // A = M K-major, B = S16 MN-major
      const uint32_t idesc_r = make_idesc_bf16(128, BN, 1, 1);   // A = M^T MN-major
      const uint32_t idesc = p.reverse ? idesc_r : idesc_f;
      const uint32_t sSa = smem_u32(sS);
      bool ok = true;
      int n = 0;
      for (int s = 0; s < n_steps && ok; ++s) {
        // the state of the previous step (or the initial state) is in shared memory and in tensor memory
        if (!mbar_wait(s_ready, s & 1, p.status, abort_flag, ERR_WAIT_MISC)) { ok = false; break; }
        tc_fence_after();
        for (int kb = 0; kb < KB && ok; ++kb, ++n) {
          const int stage = n % STAGES;
          if (!mbar_wait(&full_bar[stage], (n / STAGES) & 1, p.status, abort_flag, ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + L::RING_OFF + stage * L::STAGE_BYTES);
          // B: K = state rows (this k-block's 64), N = 128 columns in two groups DK * 128 bytes apart
          const uint64_t bd = make_smem_desc(sSa + kb * 8192, DK * 128, 1024);
#pragma unroll
          for (int h = 0; h < HALVES; ++h) {
            const uint64_t ad = p.reverse ? make_smem_desc(sA + h * 2 * 8192, 8192, 1024)
                                          : make_smem_desc(sA + h * 2 * 8192, 16, 1024);
            const uint32_t d_tmem = tmem_base + h * 2 * BN;
#pragma unroll
            for (int k = 0; k < 4; ++k)
              mma_ss(d_tmem, desc_advance(ad, p.reverse ? k * 2048 : k * 32), desc_advance(bd, k * 2048), idesc,
                     (kb | k) ? 1u : 0u);
          }
          mma_commit(&empty_bar[stage]);
        }
        if (ok) mma_commit(t_full);
      }
    }
  } else {
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t lane_sel = (uint32_t)(quarter * 32) << 16;
    bool ok = true;
    // initial state: forward 0; reverse G[last] (which is also what L16[last] holds)
    {
      const int c_init = c_last;
#pragma unroll
      for (int h = 0; h < HALVES; ++h) {
        const int row = h * 128 + r;
        const __nv_bfloat16* src = p.reverse ? state_ptr(p.add, c_init, row) : nullptr;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t st[32];
          uint4 packed[4];
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            packed[g] = p.reverse ? *reinterpret_cast<const uint4*>(src + c0 + g * 8) : make_uint4(0u, 0u, 0u, 0u);
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&packed[g]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = __bfloat1622float2(h2[e]);
              st[g * 8 + 2 * e] = __float_as_uint(f.x);
              st[g * 8 + 2 * e + 1] = __float_as_uint(f.y);
            }
            const int col = c0 + g * 8;
            *reinterpret_cast<uint4*>(sS + (col >> 6) * (DK * 128) + sw128(row, col & 63)) = packed[g];
          }
          tmem_st_32x32(tmem_base + h * 2 * BN + BN + lane_sel + c0, st);
        }
      }
      tmem_st_wait();
      if (!p.reverse) {  // the state entering the first chunk is zero
        __nv_bfloat16* dst0 = const_cast<__nv_bfloat16*>(state_ptr(p.out, c_first, 0));
#pragma unroll
        for (int h = 0; h < HALVES; ++h)
          for (int c0 = 0; c0 < BN; c0 += 8)
            *reinterpret_cast<uint4*>(dst0 + (long long)(h * 128 + r) * p.dv + c0) = make_uint4(0u, 0u, 0u, 0u);
      }
      tc_fence_before();
      fence_async_smem();
      mbar_arrive(s_ready);
    }
    for (int s = 0; s < n_steps && ok; ++s) {
      const int c = p.reverse ? c_last - 1 - s : c_first + s;
      const int c_out = p.reverse ? c : c + 1;
      const float a = __ldg(p.alpha + (long long)c * p.H + head);
      // the addend rows of this step are fetched BEFORE waiting for the product: their global-memory latency (they are
      // read once, from L2 or HBM) then overlaps the tensor-core work instead of adding to every 32-column piece
      // (the second half of a 256-row state fetches its row when its turn comes: 64 more registers would spill)
      uint4 ad[BN / 8];
      {
        const __nv_bfloat16* addrow = state_ptr(p.add, c, r);
#pragma unroll
        for (int g = 0; g < BN / 8; ++g) ad[g] = __ldg(reinterpret_cast<const uint4*>(addrow + g * 8));
      }
      if (!mbar_wait_warp(t_full, s & 1, p.status, abort_flag, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
#pragma unroll
      for (int h = 0; h < HALVES; ++h) {
        const int row = h * 128 + r;
        if (h > 0) {
          const __nv_bfloat16* addrow = state_ptr(p.add, c, row);
#pragma unroll
          for (int g = 0; g < BN / 8; ++g) ad[g] = __ldg(reinterpret_cast<const uint4*>(addrow + g * 8));
        }
        __nv_bfloat16* outrow = const_cast<__nv_bfloat16*>(state_ptr(p.out, c_out, row));
#pragma unroll
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t t[32], st[32];
          tmem_ld_32x32(tmem_base + h * 2 * BN + lane_sel + c0, t);
          tmem_ld_32x32(tmem_base + h * 2 * BN + BN + lane_sel + c0, st);
          tmem_ld_wait();
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&ad[(c0 >> 3) + g]);
            uint4 q;
            uint32_t* qw = reinterpret_cast<uint32_t*>(&q);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = __bfloat1622float2(a2[e]);
              const int i = g * 8 + 2 * e;
              const float x0 = fmaf(a, __uint_as_float(st[i]), f.x - __uint_as_float(t[i]));
              const float x1 = fmaf(a, __uint_as_float(st[i + 1]), f.y - __uint_as_float(t[i + 1]));
              st[i] = __float_as_uint(x0);
              st[i + 1] = __float_as_uint(x1);
              qw[e] = pack_bf16(x0, x1);
            }
            const int col = c0 + g * 8;
            *reinterpret_cast<uint4*>(sS + (col >> 6) * (DK * 128) + sw128(row, col & 63)) = q;
            *reinterpret_cast<uint4*>(outrow + col) = q;
          }
          tmem_st_32x32(tmem_base + h * 2 * BN + BN + lane_sel + c0, st);
        }
      }
      tmem_st_wait();
      tc_fence_before();
      fence_async_smem();
      mbar_arrive(s_ready);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TCOLS);
  }
}

template <int DK>
int launch_scan(const CUtensorMap& tm, const ScanParams& p, cudaStream_t stream) {
  auto kern = delta_scan_kernel<DK>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<DK>::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(p.dv / BN, p.H, p.n_docs);
  kern<<<grid, 192, Smem<DK>::TOTAL, stream>>>(tm, p);
  return fb::launch_ok("delta_scan_kernel");
}

}  // namespace

extern "C" {

// M [NC, H, dk, dk], add [>= NC, H, dk, dv], out [NC + 1, H, dk, dv] bf16 contiguous; alpha [NC, H] fp32; first / last
// [n_docs] chunk indices.  dk in {128, 256}, dv a multiple of 128.  reverse = 0 / 1 as described at the top of the file.
int fb_delta_scan(const void* M, const void* add, const float* alpha, void* out, const int* first, const int* last,
                  int n_docs, int H, int NC, int dk, int dv, int reverse, cudaStream_t stream) {
  if (n_docs <= 0 || NC <= 0) return 0;
  if ((dk != 128 && dk != 256) || (dv % BN) != 0) return -2;
  CUtensorMap tm;
  int rc = fb::make_tmap_2d(&tm, M, 2, (uint64_t)NC * H * dk, (uint64_t)dk, (uint64_t)dk, 64, 64, true);
  if (rc) return rc;
  ScanParams p;
  p.first = first; p.last = last; p.n_docs = n_docs; p.H = H; p.NC = NC; p.dk = dk; p.dv = dv; p.reverse = reverse;
  p.alpha = alpha; p.add = (const __nv_bfloat16*)add; p.out = (__nv_bfloat16*)out;
  p.status = fb::status_ptr();
  return dk == 128 ? launch_scan<128>(tm, p, stream) : launch_scan<256>(tm, p, stream);
}

}  // extern "C"
