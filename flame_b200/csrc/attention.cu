// Variable-length causal softmax attention (optionally sliding-window) for sm_100a, forward and backward.
//
// Packed layout: q [T, H, Dh], k/v [T, Hkv, Dh] with arbitrary token strides (so they may be column blocks of
// one fused qkv buffer); documents are delimited by cu_seqlens and never attend across boundaries.
//
// Forward: one CTA per (128-query tile of one document, head).  Warp 0 feeds K/V tiles through a 3-slot TMA
// ring, warp 1 issues tcgen05 MMAs (S = Q K^T into TMEM, O += P V with V read MN-major), warps 2-5 own one
// query row per thread: two sweeps over S in TMEM (row max, then exp2 / row sum / bf16 P written to swizzled
// shared memory).  O stays in TMEM and is rescaled only when the running max grows by more than 2^8, so the
// correction is rare.  Two CTAs fit per SM (256 TMEM columns, ~100 KB smem each), which is what overlaps one
// CTA's exponentials with the other's MMAs.
//
// Backward: one CTA per (128-key tile, kv head); it walks the query tiles that see those keys, recomputes
// P = exp2(S - lse), forms dS = P * (dP - delta), and accumulates dV += P^T dO, dK += dS^T Q in TMEM; dQ tiles
// are reduced into an fp32 buffer with TMA reduce-adds.  Head dim 64 and head dim 128 are two kernels: the second
// works on the transposed score tile (see attn_bwd128_kernel).
//
// Takes the place of flash_attn_varlen_func as called by fla/layers/attn.py:146-174.
#include "tc05.cuh"
#include "host_utils.cuh"
#include <math.h>
#include <stdlib.h>

using namespace tc05;


namespace {

constexpr int BQ = 128;   // query rows per tile
constexpr int BKV = 128;  // keys per tile
constexpr float kLog2e = 1.4426950408889634f;

struct AttnParams {
  const int* cu_seqlens;    // [nseq + 1]
  const int* tile_offsets;  // [nseq + 1] prefix sum of ceil(len / 128)
  int nseq;
  int H, Hkv;
  int total_tokens;
  int window;  // 0 = full causal, else keys in (q - window, q]
  float scale;       // softmax scale
  float scale_log2;  // scale * log2(e)
  __nv_bfloat16* O;
  long long o_stride_t;
  // Optional second output [T, H, Dh] (contiguous): the bf16 rounding of (O_fp32 - O), i.e. the low half of a two-term
  // bf16 split of the fp32 result.  The stick-breaking backward needs do . o to fp32 accuracy (see sb_attention.cu).
  __nv_bfloat16* O_lo;
  float* lse;  // [H, T] in log2 domain of the scaled logits
  int* status;
};

// 2^x on the MUFU unit without the range fix-up of exp2f: results below 2^-126 flush to 0, -inf gives 0
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 2^x on the FMA pipe: Cody-Waite split x = n + f with f in [-0.5, 0.5], a degree-3 minimax polynomial for 2^f
// (relative error 7.5e-5, far inside the 2^-9 of the bf16 value the result is rounded to) and n added into the exponent
// field.  Inputs below -125 (masked scores are -inf) give 2^-125, which is zero for every purpose here.  A share of the
// exponentials of a score tile goes this way because the SM's 16 MUFU results per clock are what bounds the softmax.
__device__ __forceinline__ float poly_exp2(float x) {
  x = fmaxf(x, -125.f);
  const float t = x + 12582912.f;  // 1.5 * 2^23: round(x) lands in the low mantissa bits
  const float f = x - (t - 12582912.f);
  float p = fmaf(f, 0.05517146f, 0.24261086f);
  p = fmaf(p, f, 0.69326099f);
  p = fmaf(p, f, 0.99992809f);
  return __uint_as_float(__float_as_uint(p) + (__float_as_uint(t) << 23));
}

// largest i in [0, n) with offs[i] <= x
__device__ __forceinline__ int upper_doc(const int* __restrict__ offs, int n, int x) {
  int lo = 0, hi = n;
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (offs[mid] <= x) lo = mid; else hi = mid;
  }
  return lo;
}

// byte offset of element (row, col) in a [rows][64]-bf16 tile stored with the 128-byte swizzle
__device__ __forceinline__ uint32_t sw128_offset(int row, int col) {
  const int chunk = (col >> 3) ^ (row & 7);
  return (uint32_t)(row * 128 + chunk * 16 + (col & 7) * 2);
}

template <int DH>
struct FwdSmem {
  static constexpr int KB = DH / 64;               // 64-column k-blocks per head dim
  static constexpr int TILE_BYTES = BKV * DH * 2;  // one Q / K / V tile
  static constexpr int NSLOT = 3;
  static constexpr int Q_OFF = 0;
  static constexpr int RING_OFF = TILE_BYTES;
  static constexpr int P_OFF = RING_OFF + NSLOT * TILE_BYTES;
  static constexpr int P_BYTES = BQ * BKV * 2;
  static constexpr int BAR_OFF = P_OFF + P_BYTES;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

// MODE 0: softmax attention.  MODE 1: stick-breaking attention (strictly causal; key tiles are walked from the diagonal
// backwards so that each row can carry the running sum of log(1 - sigmoid) over the keys already seen; weights never
// exceed one, so there is no running maximum and O is never rescaled; `lse` receives the remainder 1 - sum_j att_ij).
template <int DH, int MODE>
__global__ void __launch_bounds__(192, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, AttnParams p) {
  using L = FwdSmem<DH>;
  const int total_tiles = p.tile_offsets[p.nseq];
  // heavier tiles (late in their document) are scheduled first
  const int tile_id = total_tiles - 1 - (int)blockIdx.x;
  if (tile_id < 0) return;
  const int head = blockIdx.y;
  const int kv_head = head / (p.H / p.Hkv);
  const int doc = upper_doc(p.tile_offsets, p.nseq + 1, tile_id);
  const int tile_in_doc = tile_id - p.tile_offsets[doc];
  const int doc_start = p.cu_seqlens[doc];
  const int doc_len = p.cu_seqlens[doc + 1] - doc_start;
  const int q0 = tile_in_doc * BQ;
  int j_start = 0;
  if (p.window > 0) {
    int lo = q0 - p.window + 1;
    j_start = lo > 0 ? lo / BKV : 0;
  }
  const int j_end = tile_in_doc;  // inclusive (BQ == BKV)
  const int nblk = j_end - j_start + 1;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = (uint64_t*)(smem + L::BAR_OFF);  // [NSLOT]
  uint64_t* empty_bar = full_bar + L::NSLOT;            // [NSLOT]
  uint64_t* q_full = empty_bar + L::NSLOT;
  uint64_t* s_full = q_full + 1;
  uint64_t* p_ready = s_full + 1;
  uint64_t* pv_done = p_ready + 1;
  uint64_t* s_free = pv_done + 1;
  uint32_t* tmem_slot = (uint32_t*)(s_free + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < L::NSLOT; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(q_full, 1);
    mbar_init(s_full, 1);
    mbar_init(p_ready, 128);
    mbar_init(pv_done, 1);
    mbar_init(s_free, 128);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base;
  const uint32_t tmem_O = tmem_base + 128;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, L::TILE_BYTES);
#pragma unroll
      for (int kb = 0; kb < L::KB; ++kb)
        tma_load_3d(smem + L::Q_OFF + kb * (BQ * 128), &tmQ, q_full, kb * 64, head, doc_start + q0);
      bool ok = true;
      for (int n = 0; n < 2 * nblk && ok; ++n) {
        const int slot = n % L::NSLOT;
        const uint32_t par = ((n / L::NSLOT) & 1) ^ 1;
        if (!mbar_wait(&empty_bar[slot], par, p.status, abort_flag, ERR_WAIT_EMPTY)) { ok = false; break; }
        const int j = MODE == 0 ? j_start + (n >> 1) : j_end - (n >> 1);
        uint8_t* dst = smem + L::RING_OFF + slot * L::TILE_BYTES;
        mbar_expect_tx(&full_bar[slot], L::TILE_BYTES);
        const CUtensorMap* tm = (n & 1) ? &tmV : &tmK;
#pragma unroll
        for (int kb = 0; kb < L::KB; ++kb)
          tma_load_3d(dst + kb * (BKV * 128), tm, &full_bar[slot], kb * 64, kv_head, doc_start + j * BKV);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BQ, BKV, 0, 0);
      constexpr uint32_t idesc_o = make_idesc_bf16(BQ, DH, 0, 1);
      const uint32_t sQ = smem_u32(smem + L::Q_OFF);
      const uint32_t sP = smem_u32(smem + L::P_OFF);
      bool ok = mbar_wait(q_full, 0, p.status, abort_flag, ERR_WAIT_FULL);
      auto issue_qk = [&](int jj) -> bool {
        const int n = 2 * jj, slot = n % L::NSLOT;
        if (!mbar_wait(&full_bar[slot], (n / L::NSLOT) & 1, p.status, abort_flag, ERR_WAIT_FULL)) return false;
        tc_fence_after();
        const uint32_t sK = smem_u32(smem + L::RING_OFF + slot * L::TILE_BYTES);
#pragma unroll
        for (int kb = 0; kb < L::KB; ++kb) {
          const uint64_t ad = make_smem_desc(sQ + kb * (BQ * 128), 16, 1024);
          const uint64_t bd = make_smem_desc(sK + kb * (BKV * 128), 16, 1024);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            mma_ss(tmem_S, desc_advance(ad, k * 32), desc_advance(bd, k * 32), idesc_s, (kb | k) ? 1u : 0u);
        }
        mma_commit(&empty_bar[slot]);
        mma_commit(s_full);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int jj = 0; jj < nblk && ok; ++jj) {
        if (jj + 1 < nblk) {
          // S_jj has been copied to registers: the next score tile may overwrite it while the softmax runs
          if (!mbar_wait(s_free, jj & 1, p.status, abort_flag, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
          tc_fence_after();
          if (!issue_qk(jj + 1)) { ok = false; break; }
        }
        if (!mbar_wait(p_ready, jj & 1, p.status, abort_flag, ERR_WAIT_MISC)) { ok = false; break; }
        tc_fence_after();
        const int n = 2 * jj + 1, slot = n % L::NSLOT;
        if (!mbar_wait(&full_bar[slot], (n / L::NSLOT) & 1, p.status, abort_flag, ERR_WAIT_FULL)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sV = smem_u32(smem + L::RING_OFF + slot * L::TILE_BYTES);
        // P: K-major, two 64-key k-blocks; V: MN-major, DH/64 groups of 64 head-dim columns
        const uint64_t bd = make_smem_desc(sV, BKV * 128, 1024);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
          const uint64_t ad = make_smem_desc(sP + kb * (BQ * 128), 16, 1024);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            mma_ss(tmem_O, desc_advance(ad, k * 32), desc_advance(bd, (kb * 4 + k) * 2048), idesc_o,
                   (jj > 0 || kb > 0 || k > 0) ? 1u : 0u);
        }
        mma_commit(&empty_bar[slot]);
        mma_commit(pv_done);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax / correction / epilogue
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;  // query row inside the tile
    const int q_idx = q0 + r;           // position inside the document
    const uint32_t lane_sel = (uint32_t)(quarter * 32) << 16;
    uint8_t* sP = smem + L::P_OFF;
    float m_run = MODE == 0 ? -INFINITY : 1.f;  // stale running max (log2 domain, scaled) / carried remainder product
    float l_run = 0.f;
    bool ok = true;
    for (int jj = 0; jj < nblk && ok; ++jj) {
      const int kv0 = (MODE == 0 ? j_start + jj : j_end - jj) * BKV;
      const bool mask_causal = (kv0 + BKV - 1 > q0);
      const bool mask_window = (p.window > 0) && (kv0 <= q0 + BQ - 1 - p.window);
      const bool need_mask = mask_causal || mask_window;
      if (!mbar_wait_warp(s_full, jj & 1, p.status, abort_flag, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      if (MODE == 1) {
        // stick-breaking: sigma = t / (1 + t) with t = 2^x, x the logit in log2 units; att_j = sigma_j * E_j with
        // E_j = prod (1 - sigma) over the later keys of this row, carried from tile to tile (two MUFU ops per element,
        // no logarithm).  The row is consumed in four 32-column pieces from the right.
        const bool diag = (jj == 0);
        if (jj > 0) {
          if (!mbar_wait_warp(pv_done, (jj - 1) & 1, p.status, abort_flag, ERR_WAIT_MISC)) { ok = false; break; }
          tc_fence_after();
        }
        float E = m_run;  // m_run doubles as the carried product (starts at 1 for this mode)
#pragma unroll 1
        for (int c0 = BKV - 32; c0 >= 0; c0 -= 32) {
          uint32_t xr[32];
          tmem_ld_32x32(tmem_S + lane_sel + c0, xr);
          tmem_ld_wait();
#pragma unroll
          for (int c = 24; c >= 0; c -= 8) {
            float e[8];
#pragma unroll
            for (int i = 7; i >= 0; --i) {
              const bool dead = diag && (kv0 + c0 + c + i >= q_idx);
              float x = __uint_as_float(xr[c + i]) * p.scale_log2;
              x = fminf(fmaxf(x, -100.f), 100.f);
              const float t = fast_exp2(x);
              const float inv = __frcp_rn(1.f + t);
              e[i] = dead ? 0.f : t * inv * E;
              E = dead ? E : E * inv;
            }
            uint4 q;
            q.x = pack_bf16(e[0], e[1]);
            q.y = pack_bf16(e[2], e[3]);
            q.z = pack_bf16(e[4], e[5]);
            q.w = pack_bf16(e[6], e[7]);
            const int cc = c0 + c;
            *reinterpret_cast<uint4*>(sP + (cc >> 6) * (BQ * 128) + sw128_offset(r, cc & 63)) = q;
          }
        }
        m_run = E;
        tc_fence_before();
        mbar_arrive(s_free);
      } else {
      // the whole score row moves to registers in one go, which frees S for the next tile right away
      uint32_t sr[BKV];
      tmem_ld_32x32(tmem_S + lane_sel + 0, *reinterpret_cast<uint32_t(*)[32]>(&sr[0]));
      tmem_ld_32x32(tmem_S + lane_sel + 32, *reinterpret_cast<uint32_t(*)[32]>(&sr[32]));
      tmem_ld_32x32(tmem_S + lane_sel + 64, *reinterpret_cast<uint32_t(*)[32]>(&sr[64]));
      tmem_ld_32x32(tmem_S + lane_sel + 96, *reinterpret_cast<uint32_t(*)[32]>(&sr[96]));
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(s_free);
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < BKV; ++i) {
          const int kv = kv0 + i;
          const bool dead = (kv > q_idx) || (p.window > 0 && kv <= q_idx - p.window);
          if (dead) sr[i] = 0xff800000u;  // -inf
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < BKV; i += 4) {
        mx0 = fmaxf(mx0, __uint_as_float(sr[i]));
        mx1 = fmaxf(mx1, __uint_as_float(sr[i + 1]));
        mx2 = fmaxf(mx2, __uint_as_float(sr[i + 2]));
        mx3 = fmaxf(mx3, __uint_as_float(sr[i + 3]));
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2;
      if (jj > 0) {
        if (!mbar_wait_warp(pv_done, (jj - 1) & 1, p.status, abort_flag, ERR_WAIT_MISC)) { ok = false; break; }
        tc_fence_after();
      }
      const float m_new = fmaxf(m_run, mx);
      const bool grow = (m_new > m_run + 8.f) || (m_run == -INFINITY && m_new != -INFINITY);
      if (__any_sync(0xffffffffu, grow)) {
        const float factor = (m_run == -INFINITY) ? 0.f : fast_exp2(m_run - m_new);
        if (jj > 0) {
#pragma unroll 1
          for (int c = 0; c < DH; c += 32) {
            uint32_t v[32];
            tmem_ld_32x32(tmem_O + lane_sel + c, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * factor);
            tmem_st_32x32(tmem_O + lane_sel + c, v);
          }
          tmem_st_wait();
        }
        l_run *= factor;
        m_run = m_new;
      }
      const float m_use = (m_run == -INFINITY) ? 0.f : m_run;
      // p = exp2(s * scale - m); masked scores are -inf and give exactly 0
      float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
#pragma unroll
      for (int c = 0; c < BKV; c += 8) {
        float e[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) e[i] = fast_exp2(fmaf(__uint_as_float(sr[c + i]), p.scale_log2, -m_use));
        l0 += e[0] + e[4];
        l1 += e[1] + e[5];
        l2 += e[2] + e[6];
        l3 += e[3] + e[7];
        uint4 q;
        q.x = pack_bf16(e[0], e[1]);
        q.y = pack_bf16(e[2], e[3]);
        q.z = pack_bf16(e[4], e[5]);
        q.w = pack_bf16(e[6], e[7]);
        *reinterpret_cast<uint4*>(sP + (c >> 6) * (BQ * 128) + sw128_offset(r, c & 63)) = q;
      }
      l_run += (l0 + l1) + (l2 + l3);
      }
      tc_fence_before();
      fence_async_smem();
      mbar_arrive(p_ready);
    }
    if (ok) ok = mbar_wait_warp(pv_done, (nblk - 1) & 1, p.status, abort_flag, ERR_WAIT_MISC);
    if (ok) {
      tc_fence_after();
      const bool valid = q_idx < doc_len;
      const float inv_l = MODE == 0 ? (l_run > 0.f ? 1.f / l_run : 0.f) : 1.f;
      const long long tok = (long long)doc_start + q_idx;
      __nv_bfloat16* orow = p.O + tok * p.o_stride_t + (long long)head * DH;
#pragma unroll 1
      for (int c = 0; c < DH; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_O + lane_sel + c, v);
        tmem_ld_wait();
        if (valid) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 q;
            q.x = pack_bf16(__uint_as_float(v[g * 8 + 0]) * inv_l, __uint_as_float(v[g * 8 + 1]) * inv_l);
            q.y = pack_bf16(__uint_as_float(v[g * 8 + 2]) * inv_l, __uint_as_float(v[g * 8 + 3]) * inv_l);
            q.z = pack_bf16(__uint_as_float(v[g * 8 + 4]) * inv_l, __uint_as_float(v[g * 8 + 5]) * inv_l);
            q.w = pack_bf16(__uint_as_float(v[g * 8 + 6]) * inv_l, __uint_as_float(v[g * 8 + 7]) * inv_l);
            *reinterpret_cast<uint4*>(orow + c + g * 8) = q;
            if (MODE == 1 && p.O_lo != nullptr) {
              const __nv_bfloat162* hi = reinterpret_cast<const __nv_bfloat162*>(&q);
              uint4 lo;
              uint32_t* lw = reinterpret_cast<uint32_t*>(&lo);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 h = __bfloat1622float2(hi[e]);
                lw[e] = pack_bf16(__uint_as_float(v[g * 8 + 2 * e]) * inv_l - h.x, __uint_as_float(v[g * 8 + 2 * e + 1]) * inv_l - h.y);
              }
              *reinterpret_cast<uint4*>(p.O_lo + (tok * p.H + head) * DH + c + g * 8) = lo;
            }
          }
        }
      }
      if (valid) p.lse[(long long)head * p.total_tokens + tok] = MODE == 0 ? m_run + log2f(l_run) : m_run;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

// ------------------------------------------------------------------------------------------------
// forward, head dim 64, softmax mode, P in tensor memory
// ------------------------------------------------------------------------------------------------
// Same tiling and roles as attn_fwd_kernel<64, 0>, with two changes that take the probability tile off shared memory:
// (1) P is written as bf16 pairs into 64 TMEM columns and read from there as the A operand of O += P V, so a tile no
//     longer costs 32 KB of shared-memory stores, a proxy fence and 32 KB of operand reads by the tensor core;
// (2) P is handed over in two halves of 64 keys with a barrier pair each, so the PV product of the first half runs while
//     the second half is exponentiated, and the next tile's first half only waits for the first half's product.
// TMEM (256 columns, two CTAs per SM): S 128 | O 64 | P 64.
struct FwdPtSmem {
  static constexpr int TILE_BYTES = BKV * 64 * 2;
  static constexpr int NSLOT = 4;
  static constexpr int Q_OFF = 0;
  static constexpr int RING_OFF = TILE_BYTES;
  static constexpr int BAR_OFF = RING_OFF + NSLOT * TILE_BYTES;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__global__ void __launch_bounds__(192, 2)
attn_fwd_pt_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, AttnParams p) {
  using L = FwdPtSmem;
  constexpr int DH = 64;
  const int total_tiles = p.tile_offsets[p.nseq];
  const int tile_id = total_tiles - 1 - (int)blockIdx.x;  // heavier tiles first
  if (tile_id < 0) return;
  const int head = blockIdx.y;
  const int kv_head = head / (p.H / p.Hkv);
  const int doc = upper_doc(p.tile_offsets, p.nseq + 1, tile_id);
  const int tile_in_doc = tile_id - p.tile_offsets[doc];
  const int doc_start = p.cu_seqlens[doc];
  const int doc_len = p.cu_seqlens[doc + 1] - doc_start;
  const int q0 = tile_in_doc * BQ;
  int j_start = 0;
  if (p.window > 0) {
    int lo = q0 - p.window + 1;
    j_start = lo > 0 ? lo / BKV : 0;
  }
  const int j_end = tile_in_doc;
  const int nblk = j_end - j_start + 1;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = (uint64_t*)(smem + L::BAR_OFF);  // [NSLOT]
  uint64_t* empty_bar = full_bar + L::NSLOT;            // [NSLOT]
  uint64_t* q_full = empty_bar + L::NSLOT;
  uint64_t* s_full = q_full + 1;
  uint64_t* s_free = s_full + 1;
  uint64_t* p_ready = s_free + 1;  // [2]
  uint64_t* pv_done = p_ready + 2;  // [2]
  uint32_t* tmem_slot = (uint32_t*)(pv_done + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < L::NSLOT; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(q_full, 1);
    mbar_init(s_full, 1);
    mbar_init(s_free, 128);
    for (int h = 0; h < 2; ++h) {
      mbar_init(&p_ready[h], 128);
      mbar_init(&pv_done[h], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base;
  const uint32_t tmem_O = tmem_base + 128;
  const uint32_t tmem_P = tmem_base + 192;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, L::TILE_BYTES);
      tma_load_3d(smem + L::Q_OFF, &tmQ, q_full, 0, head, doc_start + q0);
      for (int n = 0; n < 2 * nblk; ++n) {
        const int slot = n % L::NSLOT;
        const uint32_t par = ((n / L::NSLOT) & 1) ^ 1;
        if (!mbar_wait(&empty_bar[slot], par, p.status, abort_flag, ERR_WAIT_EMPTY)) break;
        const int j = j_start + (n >> 1);
        mbar_expect_tx(&full_bar[slot], L::TILE_BYTES);
        tma_load_3d(smem + L::RING_OFF + slot * L::TILE_BYTES, (n & 1) ? &tmV : &tmK, &full_bar[slot], 0, kv_head,
                    doc_start + j * BKV);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BQ, BKV, 0, 0);
      constexpr uint32_t idesc_o = make_idesc_bf16(BQ, DH, 0, 1);
      const uint32_t sQ = smem_u32(smem + L::Q_OFF);
      bool ok = mbar_wait(q_full, 0, p.status, abort_flag, ERR_WAIT_FULL);
      auto issue_qk = [&](int jj) -> bool {
        const int n = 2 * jj, slot = n % L::NSLOT;
        if (!mbar_wait(&full_bar[slot], (n / L::NSLOT) & 1, p.status, abort_flag, ERR_WAIT_FULL)) return false;
        tc_fence_after();
        const uint64_t ad = make_smem_desc(sQ, 16, 1024);
        const uint64_t bd = make_smem_desc(smem_u32(smem + L::RING_OFF + slot * L::TILE_BYTES), 16, 1024);
#pragma unroll
        for (int k = 0; k < 4; ++k) mma_ss(tmem_S, desc_advance(ad, k * 32), desc_advance(bd, k * 32), idesc_s, k ? 1u : 0u);
        mma_commit(&empty_bar[slot]);
        mma_commit(s_full);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int jj = 0; jj < nblk && ok; ++jj) {
        if (jj + 1 < nblk) {
          if (!mbar_wait(s_free, jj & 1, p.status, abort_flag, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
          tc_fence_after();
          if (!issue_qk(jj + 1)) { ok = false; break; }
        }
        const int n = 2 * jj + 1, slot = n % L::NSLOT;
        const uint64_t bd = make_smem_desc(smem_u32(smem + L::RING_OFF + slot * L::TILE_BYTES), BKV * 128, 1024);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (!mbar_wait(&p_ready[h], jj & 1, p.status, abort_flag, ERR_WAIT_MISC)) { ok = false; break; }
          if (h == 0 && !mbar_wait(&full_bar[slot], (n / L::NSLOT) & 1, p.status, abort_flag, ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          // P: bf16 pairs in tensor memory, 8 columns per 16 keys; V: MN-major, 16 keys = 2048 bytes
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int kk = h * 4 + k;
            mma_ts(tmem_O, tmem_P + kk * 8, desc_advance(bd, kk * 2048), idesc_o, (jj > 0 || kk > 0) ? 1u : 0u);
          }
          if (h == 1) mma_commit(&empty_bar[slot]);
          mma_commit(&pv_done[h]);
        }
      }
    }
  } else {
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int q_idx = q0 + r;
    const uint32_t lane_sel = (uint32_t)(quarter * 32) << 16;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int jj = 0; jj < nblk && ok; ++jj) {
      const int kv0 = (j_start + jj) * BKV;
      const bool mask_causal = (kv0 + BKV - 1 > q0);
      const bool mask_window = (p.window > 0) && (kv0 <= q0 + BQ - 1 - p.window);
      if (!mbar_wait_warp(s_full, jj & 1, p.status, abort_flag, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      uint32_t sr[BKV];
      tmem_ld_32x32(tmem_S + lane_sel + 0, *reinterpret_cast<uint32_t(*)[32]>(&sr[0]));
      tmem_ld_32x32(tmem_S + lane_sel + 32, *reinterpret_cast<uint32_t(*)[32]>(&sr[32]));
      tmem_ld_32x32(tmem_S + lane_sel + 64, *reinterpret_cast<uint32_t(*)[32]>(&sr[64]));
      tmem_ld_32x32(tmem_S + lane_sel + 96, *reinterpret_cast<uint32_t(*)[32]>(&sr[96]));
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(s_free);
      // Without a window only the diagonal tile has dead entries: row r of the tile sees its columns 0..r.  
      const bool diag = (p.window == 0) && mask_causal;
      if (diag) {
#pragma unroll
        for (int i = 0; i < BKV; ++i)
          if (i > r) sr[i] = 0xff800000u;
      } else if (mask_causal || mask_window) {
#pragma unroll
        for (int i = 0; i < BKV; ++i) {
          const int kv = kv0 + i;
          const bool dead = (kv > q_idx) || (kv <= q_idx - p.window);
          if (dead) sr[i] = 0xff800000u;
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < BKV; i += 8) {
        mx0 = fmax3(mx0, __uint_as_float(sr[i]), __uint_as_float(sr[i + 1]));
        mx1 = fmax3(mx1, __uint_as_float(sr[i + 2]), __uint_as_float(sr[i + 3]));
        mx2 = fmax3(mx2, __uint_as_float(sr[i + 4]), __uint_as_float(sr[i + 5]));
        mx3 = fmax3(mx3, __uint_as_float(sr[i + 6]), __uint_as_float(sr[i + 7]));
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2;
      const float m_new = fmaxf(m_run, mx);
      const bool grow = (m_new > m_run + 8.f) || (m_run == -INFINITY && m_new != -INFINITY);
      if (__any_sync(0xffffffffu, grow)) {
        const float factor = (m_run == -INFINITY) ? 0.f : fast_exp2(m_run - m_new);
        if (jj > 0) {
          // O is rescaled in place: every product of the previous tile must have landed
          if (!mbar_wait_warp(&pv_done[1], (jj - 1) & 1, p.status, abort_flag, ERR_WAIT_MISC)) { ok = false; break; }
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < DH; c += 32) {
            uint32_t v[32];
            tmem_ld_32x32(tmem_O + lane_sel + c, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * factor);
            tmem_st_32x32(tmem_O + lane_sel + c, v);
          }
          tmem_st_wait();
        }
        l_run *= factor;
        m_run = m_new;
      }
      const float m_use = (m_run == -INFINITY) ? 0.f : m_run;
      float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        // packed in place: the bf16 pairs of columns [64 h, 64 h + 64) go to sr[32 h .. 32 h + 31], all already consumed
#pragma unroll
        for (int hb = 0; hb < 2; ++hb) {
          const int b = h * 2 + hb;  // 32-column block of the tile
          {
#pragma unroll
            for (int c = 0; c < 32; c += 4) {
              // three exponentials on the MUFU, the fourth on the FMA pipe
              const float e0 = fast_exp2(fmaf(__uint_as_float(sr[b * 32 + c]), p.scale_log2, -m_use));
              const float e1 = fast_exp2(fmaf(__uint_as_float(sr[b * 32 + c + 1]), p.scale_log2, -m_use));
              const float e2 = fast_exp2(fmaf(__uint_as_float(sr[b * 32 + c + 2]), p.scale_log2, -m_use));
              const float e3 = poly_exp2(fmaf(__uint_as_float(sr[b * 32 + c + 3]), p.scale_log2, -m_use));
              l0 += e0;
              l1 += e1;
              l2 += e2;
              l3 += e3;
              sr[h * 32 + hb * 16 + (c >> 1)] = pack_bf16(e0, e1);
              sr[h * 32 + hb * 16 + (c >> 1) + 1] = pack_bf16(e2, e3);
            }
          }
        }
        // the half's P columns are free once the previous tile's product over them has finished
        if (jj > 0) {
          if (!mbar_wait_warp(&pv_done[h], (jj - 1) & 1, p.status, abort_flag, ERR_WAIT_MISC)) { ok = false; break; }
          tc_fence_after();
        }
        tmem_st_32x32(tmem_P + lane_sel + h * 32, *reinterpret_cast<uint32_t(*)[32]>(&sr[h * 32]));
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(&p_ready[h]);
      }
      l_run += (l0 + l1) + (l2 + l3);
    }
    if (ok) ok = mbar_wait_warp(&pv_done[1], (nblk - 1) & 1, p.status, abort_flag, ERR_WAIT_MISC);
    if (ok) {
      tc_fence_after();
      const bool valid = q_idx < doc_len;
      const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
      const long long tok = (long long)doc_start + q_idx;
      __nv_bfloat16* orow = p.O + tok * p.o_stride_t + (long long)head * DH;
#pragma unroll 1
      for (int c = 0; c < DH; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_O + lane_sel + c, v);
        tmem_ld_wait();
        if (valid) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 q;
            q.x = pack_bf16(__uint_as_float(v[g * 8 + 0]) * inv_l, __uint_as_float(v[g * 8 + 1]) * inv_l);
            q.y = pack_bf16(__uint_as_float(v[g * 8 + 2]) * inv_l, __uint_as_float(v[g * 8 + 3]) * inv_l);
            q.z = pack_bf16(__uint_as_float(v[g * 8 + 4]) * inv_l, __uint_as_float(v[g * 8 + 5]) * inv_l);
            q.w = pack_bf16(__uint_as_float(v[g * 8 + 6]) * inv_l, __uint_as_float(v[g * 8 + 7]) * inv_l);
            *reinterpret_cast<uint4*>(orow + c + g * 8) = q;
          }
        }
      }
      if (valid) p.lse[(long long)head * p.total_tokens + tok] = m_run + log2f(l_run);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

// ------------------------------------------------------------------------------------------------
// backward
// ------------------------------------------------------------------------------------------------
struct AttnBwdParams {
  const int* cu_seqlens;
  const int* tile_offsets;
  int nseq;
  int H, Hkv;
  int total_tokens;
  int window;
  float scale;
  float scale_log2;
  const float* lse;    // [H, T]
  const float* delta;  // [H, T]  rowsum(dO * O)
  float* dQ;           // fp32 [T, H, DH], zero-initialised by the caller
  __nv_bfloat16* dK;   // [T, Hkv, DH] with token stride dk_stride_t
  __nv_bfloat16* dV;
  long long dk_stride_t, dv_stride_t;
  int* status;
};

template <int DH>
struct BwdSmem {
  static constexpr int TILE_BYTES = 128 * DH * 2;
  static constexpr int K_OFF = 0;
  static constexpr int V_OFF = TILE_BYTES;
  static constexpr int NSTAGE = 3;  // Q + dO tiles arrive two iterations ahead of their S / dP products
  static constexpr int RING_OFF = 2 * TILE_BYTES;  // stage = Q tile + dO tile
  static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  static constexpr int P_OFF = RING_OFF + NSTAGE * STAGE_BYTES;
  static constexpr int PD_BYTES = BQ * BKV * 2;
  static constexpr int DS_OFF = P_OFF + PD_BYTES;
  static constexpr int DQ_OFF = DS_OFF + PD_BYTES;  // fp32 staging tile for the dQ reduce: 2 x [128][32]
  static constexpr int DQ_BYTES = BQ * DH * 4;
  static constexpr int BAR_OFF = DQ_OFF + DQ_BYTES;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

// dO·O row sums: delta[h, t] = sum_d dO[t,h,d] * O[t,h,d].  DH / 8 lanes cooperate on one (t, h) row with 16-byte loads.
template <int DH>
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ O, const __nv_bfloat16* __restrict__ dO,
                                  float* __restrict__ delta, long long T, int H, long long o_stride_t,
                                  long long do_stride_t) {
  constexpr int LANES = DH / 8;  // 8 (DH = 64) or 16 (DH = 128)
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long row = gid / LANES;
  const int sub = (int)(gid % LANES);
  float acc = 0.f;
  long long t = 0;
  int h = 0;
  const bool live = row < T * H;
  if (live) {
    t = row / H;
    h = (int)(row - t * H);
    const uint4 a = *reinterpret_cast<const uint4*>(O + t * o_stride_t + (long long)h * DH + sub * 8);
    const uint4 b = *reinterpret_cast<const uint4*>(dO + t * do_stride_t + (long long)h * DH + sub * 8);
    const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 x = __bfloat1622float2(pa[i]), y = __bfloat1622float2(pb[i]);
      acc += x.x * y.x + x.y * y.y;
    }
  }
#pragma unroll
  for (int s = LANES / 2; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (live && sub == 0) delta[(long long)h * T + t] = acc;
}

constexpr int BWD_THREADS = 576;  // warp 0 TMA, warp 1 MMA, warps 2..17 softmax (four warps per TMEM lane quarter)

template <int DH>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                const __grid_constant__ CUtensorMap tmdQ, AttnBwdParams p) {
  static_assert(DH == 64, "the backward kernel is laid out for head dim 64");
  using L = BwdSmem<DH>;
  const int total_tiles = p.tile_offsets[p.nseq];
  const int tile_id = (int)blockIdx.x;  // early key tiles see the most queries and come first
  if (tile_id >= total_tiles) return;
  const int kv_head = blockIdx.y;
  const int group = p.H / p.Hkv;
  const int doc = upper_doc(p.tile_offsets, p.nseq + 1, tile_id);
  const int j = tile_id - p.tile_offsets[doc];
  const int doc_start = p.cu_seqlens[doc];
  const int doc_len = p.cu_seqlens[doc + 1] - doc_start;
  const int n_qt = (doc_len + BQ - 1) / BQ;
  const int kv0 = j * BKV;
  int i_end = n_qt - 1;
  if (p.window > 0) {
    int hi = (kv0 + BKV - 1 + p.window - 1) / BQ;
    if (hi < i_end) i_end = hi;
  }
  const int n_i = i_end - j + 1;   // query tiles per head
  const int n_iter = n_i * group;  // (head in group, query tile)

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = (uint64_t*)(smem + L::BAR_OFF);  // [NSTAGE]
  uint64_t* empty_bar = full_bar + L::NSTAGE;
  uint64_t* kv_full = empty_bar + L::NSTAGE;
  uint64_t* sdp_full = kv_full + 1;
  uint64_t* pds_ready = sdp_full + 1;
  uint64_t* dq_full = pds_ready + 1;
  uint64_t* dq_free = dq_full + 1;
  uint64_t* sdp_free = dq_free + 1;  // S and dP were read out of TMEM: the next pair may overwrite them
  uint32_t* tmem_slot = (uint32_t*)(sdp_free + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < L::NSTAGE; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(kv_full, 1);
    mbar_init(sdp_full, 1);
    mbar_init(pds_ready, BWD_THREADS - 64);
    mbar_init(dq_full, 1);
    mbar_init(dq_free, BWD_THREADS - 64);
    mbar_init(sdp_free, BWD_THREADS - 64);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmdO);
    tma_prefetch_desc(&tmdQ);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base, tmem_dP = tmem_base + 128, tmem_dV = tmem_base + 256,
                 tmem_dK = tmem_base + 320, tmem_dQ = tmem_base + 384,
                 tmem_dS16 = tmem_base + 448;  // dS as bf16 pairs (64 columns): the A operand of dQ = dS K

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * L::TILE_BYTES);
      tma_load_3d(smem + L::K_OFF, &tmK, kv_full, 0, kv_head, doc_start + kv0);
      tma_load_3d(smem + L::V_OFF, &tmV, kv_full, 0, kv_head, doc_start + kv0);
      int head = kv_head * group, i = j;  // iteration = (head of the group, query tile), query tiles innermost
      for (int it = 0; it < n_iter; ++it) {
        const int stage = it % L::NSTAGE;
        const uint32_t par = ((it / L::NSTAGE) & 1) ^ 1;
        if (!mbar_wait(&empty_bar[stage], par, p.status, abort_flag, ERR_WAIT_EMPTY)) break;
        uint8_t* dst = smem + L::RING_OFF + stage * L::STAGE_BYTES;
        mbar_expect_tx(&full_bar[stage], L::STAGE_BYTES);
        tma_load_3d(dst, &tmQ, &full_bar[stage], 0, head, doc_start + i * BQ);
        tma_load_3d(dst + L::TILE_BYTES, &tmdO, &full_bar[stage], 0, head, doc_start + i * BQ);
        if (++i > i_end) { i = j; ++head; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BQ, BKV, 0, 0);    // S, dP
      constexpr uint32_t idesc_kv = make_idesc_bf16(BKV, DH, 1, 1);   // dV, dK: A = P^T / dS^T, B = dO / Q
      constexpr uint32_t idesc_dq = make_idesc_bf16(BQ, DH, 0, 1);    // dQ: A = dS, B = K
      const uint32_t sK = smem_u32(smem + L::K_OFF), sV = smem_u32(smem + L::V_OFF);
      const uint32_t sP = smem_u32(smem + L::P_OFF), sDS = smem_u32(smem + L::DS_OFF);
      bool ok = mbar_wait(kv_full, 0, p.status, abort_flag, ERR_WAIT_FULL);
      auto issue_sdp = [&](int it) -> bool {
        const int stage = it % L::NSTAGE;
        if (!mbar_wait(&full_bar[stage], (it / L::NSTAGE) & 1, p.status, abort_flag, ERR_WAIT_FULL)) return false;
        tc_fence_after();
        const uint32_t sQ = smem_u32(smem + L::RING_OFF + stage * L::STAGE_BYTES);
        const uint32_t sdO = sQ + L::TILE_BYTES;
        const uint64_t aq = make_smem_desc(sQ, 16, 1024), bk = make_smem_desc(sK, 16, 1024);
        const uint64_t ad = make_smem_desc(sdO, 16, 1024), bv = make_smem_desc(sV, 16, 1024);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          mma_ss(tmem_S, desc_advance(aq, k * 32), desc_advance(bk, k * 32), idesc_s, k ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          mma_ss(tmem_dP, desc_advance(ad, k * 32), desc_advance(bv, k * 32), idesc_s, k ? 1u : 0u);
        mma_commit(sdp_full);
        return true;
      };
      if (ok && n_iter > 0) ok = issue_sdp(0);
      for (int it = 0; it < n_iter && ok; ++it) {
        const int stage = it % L::NSTAGE;
        const uint32_t sQ = smem_u32(smem + L::RING_OFF + stage * L::STAGE_BYTES);
        const uint32_t sdO = sQ + L::TILE_BYTES;
        // The next S / dP pair goes to the tensor pipe as soon as this one was read out of TMEM, ahead of this tile's
        // dV / dK / dQ: it runs while the softmax warps form P and dS, and the three products below run while they
        // work on the next pair, so the tensor pipe (bound here by its shared-memory operand reads) never idles.
        if (it + 1 < n_iter) {
          if (!mbar_wait(sdp_free, it & 1, p.status, abort_flag, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
          tc_fence_after();
          if (!issue_sdp(it + 1)) { ok = false; break; }
        }
        if (!mbar_wait(pds_ready, it & 1, p.status, abort_flag, ERR_WAIT_MISC)) { ok = false; break; }
        tc_fence_after();
        {
          // A = P / dS read MN-major (M = keys): two 64-key groups 16 KB apart; K = query rows, 2048 B per 16
          const uint64_t ap = make_smem_desc(sP, BQ * 128, 1024), ads = make_smem_desc(sDS, BQ * 128, 1024);
          const uint64_t bdo = make_smem_desc(sdO, 16, 1024), bq = make_smem_desc(sQ, 16, 1024);
#pragma unroll
          for (int k = 0; k < 8; ++k)
            mma_ss(tmem_dV, desc_advance(ap, k * 2048), desc_advance(bdo, k * 2048), idesc_kv, (it > 0 || k > 0) ? 1u : 0u);
#pragma unroll
          for (int k = 0; k < 8; ++k)
            mma_ss(tmem_dK, desc_advance(ads, k * 2048), desc_advance(bq, k * 2048), idesc_kv, (it > 0 || k > 0) ? 1u : 0u);
        }
        // dQ tile: wait until the previous one was drained from TMEM
        if (it > 0) {
          if (!mbar_wait(dq_free, (it - 1) & 1, p.status, abort_flag, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
          tc_fence_after();
        }
        {
          const uint64_t bk = make_smem_desc(sK, 16, 1024);  // MN-major B: N = head dim (one group), K = keys
#pragma unroll
          for (int k = 0; k < 8; ++k)  // A = dS straight from TMEM (8 packed columns per 16 keys): no shared-memory read
            mma_ts(tmem_dQ, tmem_dS16 + k * 8, desc_advance(bk, k * 2048), idesc_dq, k ? 1u : 0u);
        }
        mma_commit(&empty_bar[stage]);
        mma_commit(dq_full);  // also: P and dS in shared memory may be overwritten
      }
    }
  } else {
    // ---------------------------------------------------------------- 512 softmax threads (16 warps)
    // The chain tcgen05.ld -> fma -> ex2 -> mul -> cvt -> st.shared is bound by latency, not by any pipe, so it is
    // spread over four warps per scheduler: a thread owns one query row and 32 of the tile's 128 key columns.
    const int sw = warp - 2;
    const int quarter = warp & 3;  // the TMEM lane quarter this warp may read
    const int cq = sw >> 2;        // which 32 of the 128 key columns (and which 16 of the 64 head-dim columns)
    const int hf = cq >> 1, c0 = (cq & 1) * 32;
    const int r = quarter * 32 + lane;
    const uint32_t lane_sel = (uint32_t)(quarter * 32) << 16;
    uint8_t* sP = smem + L::P_OFF + hf * (BQ * 128);
    uint8_t* sDS = smem + L::DS_OFF + hf * (BQ * 128);
    bool ok = true;
    uint32_t dq_regs[16];
    int dq_head = 0, dq_row0 = 0;
    // Publishes this warp's 32 x 16 block of the dQ tile held in registers: fp32 staging slab (64-byte rows, 64-byte
    // swizzle) -> one TMA reduce-add per warp, so the warps never wait for one another here.  (Per-thread 16-byte vector
    // reductions straight to global memory were measured slower: a warp's 32 rows are 32 separate L2 requests each.)
    uint8_t* slab = smem + L::DQ_OFF + sw * 2048;
    auto flush_dq = [&]() {
      if (lane == 0) tma_store_wait_read<0>();  // this warp's previous reduce has finished reading the slab
      __syncwarp();
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        float4 q = make_float4(__uint_as_float(dq_regs[g * 4 + 0]) * p.scale, __uint_as_float(dq_regs[g * 4 + 1]) * p.scale,
                               __uint_as_float(dq_regs[g * 4 + 2]) * p.scale, __uint_as_float(dq_regs[g * 4 + 3]) * p.scale);
        *reinterpret_cast<float4*>(slab + lane * 64 + ((g ^ ((lane >> 1) & 3)) << 4)) = q;
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0 && dq_row0 + quarter * 32 < p.total_tokens) {
        tma_reduce_add_3d(&tmdQ, slab, cq * 16, dq_head, dq_row0 + quarter * 32);
        tma_store_commit();
      }
    };
    // lse and delta of a tile are fetched one iteration ahead, off the critical path
    float lse_next = INFINITY, dlt_next = 0.f;
    auto fetch_row_stats = [&](int head, int i) {
      const int q_idx = i * BQ + r;
      if (q_idx < doc_len) {
        const long long tok = (long long)doc_start + q_idx;
        lse_next = __ldg(p.lse + (long long)head * p.total_tokens + tok);
        dlt_next = __ldg(p.delta + (long long)head * p.total_tokens + tok);
      } else {
        lse_next = INFINITY;
        dlt_next = 0.f;
      }
    };
    int head = kv_head * group, i = j;
    if (n_iter > 0) fetch_row_stats(head, i);
    for (int it = 0; it < n_iter && ok; ++it) {
      const int q_idx = i * BQ + r;
      const float lse = lse_next, dlt = dlt_next;
      int head_n = head, i_n = i + 1;
      if (i_n > i_end) { i_n = j; ++head_n; }
      if (it + 1 < n_iter) fetch_row_stats(head_n, i_n);
      const bool need_mask = (kv0 + BKV - 1 > i * BQ) || (p.window > 0 && kv0 <= i * BQ + BQ - 1 - p.window);
      if (!mbar_wait_warp(sdp_full, it & 1, p.status, abort_flag, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      uint32_t sv[32], dv[32];
      tmem_ld_32x32(tmem_S + lane_sel + cq * 32, sv);
      tmem_ld_32x32(tmem_dP + lane_sel + cq * 32, dv);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(sdp_free);
      if (need_mask) {
#pragma unroll
        for (int x = 0; x < 32; ++x) {
          const int kv = kv0 + cq * 32 + x;
          if ((kv > q_idx) || (p.window > 0 && kv <= q_idx - p.window)) sv[x] = 0xff800000u;
        }
      }
      // P and dS as packed bf16 pairs, in place: sv[0..15] holds P, dv[0..15] holds dS
#pragma unroll
      for (int x = 0; x < 32; x += 2) {
        const float e0 = fast_exp2(fmaf(__uint_as_float(sv[x]), p.scale_log2, -lse));
        const float e1 = fast_exp2(fmaf(__uint_as_float(sv[x + 1]), p.scale_log2, -lse));
        const float d0 = e0 * (__uint_as_float(dv[x]) - dlt);
        const float d1 = e1 * (__uint_as_float(dv[x + 1]) - dlt);
        sv[x >> 1] = pack_bf16(e0, e1);
        dv[x >> 1] = pack_bf16(d0, d1);
      }
      // The previous tile's dV / dK / dQ products read P and dS (shared memory, tensor memory); they were issued while
      // this tile's exponentials ran.
      if (it > 0) {
        if (!mbar_wait_warp(dq_full, (it - 1) & 1, p.status, abort_flag, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
        tc_fence_after();
      }
#pragma unroll
      for (int c = 0; c < 32; c += 8) {
        const uint32_t off = sw128_offset(r, c0 + c);
        *reinterpret_cast<uint4*>(sP + off) = make_uint4(sv[c / 2], sv[c / 2 + 1], sv[c / 2 + 2], sv[c / 2 + 3]);
        *reinterpret_cast<uint4*>(sDS + off) = make_uint4(dv[c / 2], dv[c / 2 + 1], dv[c / 2 + 2], dv[c / 2 + 3]);
      }
      tmem_st_32x16(tmem_dS16 + lane_sel + cq * 16, *reinterpret_cast<uint32_t(*)[16]>(&dv[0]));
      tmem_st_wait();
      tc_fence_before();
      fence_async_smem();
      mbar_arrive(pds_ready);
      // The previous tile's dQ leaves while the tensor core works on this tile's dV and dK: the MMA thread only asks
      // for the dQ columns back before this tile's dQ product, which it issues after those two.
      if (it > 0) {
        tmem_ld_32x16(tmem_dQ + lane_sel + cq * 16, dq_regs);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(dq_free);
        flush_dq();
      }
      dq_head = head;
      dq_row0 = doc_start + i * BQ;
      head = head_n;
      i = i_n;
    }
    if (ok && n_iter > 0) ok = mbar_wait_warp(dq_full, (n_iter - 1) & 1, p.status, abort_flag, ERR_WAIT_TMEM_FULL);
    if (ok && n_iter > 0) {
      tc_fence_after();
      tmem_ld_32x16(tmem_dQ + lane_sel + cq * 16, dq_regs);
      tmem_ld_wait();
      flush_dq();
      // dK, dV for key row r of this tile; this thread owns 16 of the 64 head-dim columns
      const int kv_idx = kv0 + r;
      const bool kvalid = kv_idx < doc_len;
      const long long ktok = (long long)doc_start + kv_idx;
      __nv_bfloat16* dkrow = p.dK + ktok * p.dk_stride_t + (long long)kv_head * DH + cq * 16;
      __nv_bfloat16* dvrow = p.dV + ktok * p.dv_stride_t + (long long)kv_head * DH + cq * 16;
      uint32_t a[16], b[16];
      tmem_ld_32x16(tmem_dK + lane_sel + cq * 16, a);
      tmem_ld_32x16(tmem_dV + lane_sel + cq * 16, b);
      tmem_ld_wait();
      if (kvalid) {
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          uint4 q;
          q.x = pack_bf16(__uint_as_float(a[g * 8 + 0]) * p.scale, __uint_as_float(a[g * 8 + 1]) * p.scale);
          q.y = pack_bf16(__uint_as_float(a[g * 8 + 2]) * p.scale, __uint_as_float(a[g * 8 + 3]) * p.scale);
          q.z = pack_bf16(__uint_as_float(a[g * 8 + 4]) * p.scale, __uint_as_float(a[g * 8 + 5]) * p.scale);
          q.w = pack_bf16(__uint_as_float(a[g * 8 + 6]) * p.scale, __uint_as_float(a[g * 8 + 7]) * p.scale);
          *reinterpret_cast<uint4*>(dkrow + g * 8) = q;
          q.x = pack_bf16(__uint_as_float(b[g * 8 + 0]), __uint_as_float(b[g * 8 + 1]));
          q.y = pack_bf16(__uint_as_float(b[g * 8 + 2]), __uint_as_float(b[g * 8 + 3]));
          q.z = pack_bf16(__uint_as_float(b[g * 8 + 4]), __uint_as_float(b[g * 8 + 5]));
          q.w = pack_bf16(__uint_as_float(b[g * 8 + 6]), __uint_as_float(b[g * 8 + 7]));
          *reinterpret_cast<uint4*>(dvrow + g * 8) = q;
        }
      }
    }
    if (lane == 0) tma_store_wait_all<0>();  // also on the failure path: the reduces read this CTA's shared memory
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------------------
// backward, head dim 128
// ------------------------------------------------------------------------------------------------
// With 128-wide heads every operand tile doubles, and S / dP / dV / dK / dQ no longer fit the 512 TMEM columns next to
// each other in the layout of the head-dim-64 kernel.  This kernel therefore works on the TRANSPOSED score tile: one CTA
// per (128-key tile, kv head) walks the query tiles 64 rows at a time and forms
//     S^T  = K Q^T   and  dP^T = V dO^T        (M = 128 keys, N = 64 queries: 64 TMEM columns each)
// so that a softmax thread owns one KEY row.  P^T and dS^T are then already laid out as the A operand of
//     dV  += P^T dO  and  dK  += dS^T Q        (A read from tensor memory, never through shared memory)
// and only dS^T is also written to shared memory (16 KB), where it is the MN-major B operand of
//     dQ^T = K^T dS^T                           (M = 128 head-dim rows, N = 64 queries).
// dQ^T leaves through an fp32 slab (transposed on the way, conflict-free) and one TMA reduce-add per warp.
// TMEM: S^T 64 | dP^T 64 | dV 128 | dK 128 | dQ^T 64 | P^T bf16 32 | dS^T bf16 32 = 512 columns.
// The per-query statistics (lse, delta) vary along the columns here, so they are staged in shared memory per tile.
struct Bwd128Smem {
  static constexpr int BQ2 = 64;
  static constexpr int KV_BYTES = 128 * 128 * 2;      // K or V tile: 2 k-blocks of [128 keys][64]
  static constexpr int QT_BYTES = BQ2 * 128 * 2;      // Q or dO tile: 2 k-blocks of [64 queries][64]
  static constexpr int K_OFF = 0;
  static constexpr int V_OFF = KV_BYTES;
  static constexpr int NSTAGE = 3;
  static constexpr int RING_OFF = 2 * KV_BYTES;
  static constexpr int STAGE_BYTES = 2 * QT_BYTES;    // Q + dO
  static constexpr int DS_OFF = RING_OFF + NSTAGE * STAGE_BYTES;   // dS^T [128 keys][64 queries] bf16, swizzled
  static constexpr int DS_BYTES = 128 * BQ2 * 2;
  static constexpr int DQ_OFF = DS_OFF + DS_BYTES;    // fp32 slab: 8 regions of [32 queries][32 head-dim columns]
  static constexpr int DQ_BYTES = 8 * 32 * 32 * 4;
  static constexpr int STAT_OFF = DQ_OFF + DQ_BYTES;  // 2 buffers x (lse[64], delta[64])
  static constexpr int STAT_BYTES = 2 * 2 * BQ2 * 4;
  static constexpr int BAR_OFF = STAT_OFF + STAT_BYTES;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

constexpr int BWD128_SOFTMAX = 256;                  // warps 2..9: a thread owns one key row and 32 of the 64 query columns
constexpr int BWD128_THREADS = 64 + BWD128_SOFTMAX;  // warp 0 TMA, warp 1 MMA

__global__ void __launch_bounds__(BWD128_THREADS, 1)
attn_bwd128_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                   const __grid_constant__ CUtensorMap tmdQ, AttnBwdParams p) {
  using L = Bwd128Smem;
  constexpr int DH = 128, BQ2 = L::BQ2;
  const int total_tiles = p.tile_offsets[p.nseq];
  const int tile_id = (int)blockIdx.x;
  if (tile_id >= total_tiles) return;
  const int kv_head = blockIdx.y;
  const int group = p.H / p.Hkv;
  const int doc = upper_doc(p.tile_offsets, p.nseq + 1, tile_id);
  const int j = tile_id - p.tile_offsets[doc];
  const int doc_start = p.cu_seqlens[doc];
  const int doc_len = p.cu_seqlens[doc + 1] - doc_start;
  const int kv0 = j * BKV;
  const int i_first = 2 * j;  // first 64-row query tile that sees this key tile
  int i_last = (doc_len + BQ2 - 1) / BQ2 - 1;
  if (p.window > 0) {
    const int hi = (kv0 + BKV - 1 + p.window - 1) / BQ2;
    if (hi < i_last) i_last = hi;
  }
  const int n_i = i_last - i_first + 1;
  const int n_iter = n_i > 0 ? n_i * group : 0;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = (uint64_t*)(smem + L::BAR_OFF);
  uint64_t* empty_bar = full_bar + L::NSTAGE;
  uint64_t* kv_full = empty_bar + L::NSTAGE;
  uint64_t* sdp_full = kv_full + 1;
  uint64_t* pds_ready = sdp_full + 1;
  uint64_t* dq_full = pds_ready + 1;
  uint64_t* dq_free = dq_full + 1;
  uint64_t* sdp_free = dq_free + 1;
  uint64_t* stat_ready = sdp_free + 1;  // lse / delta of the current query tile are in shared memory
  uint32_t* tmem_slot = (uint32_t*)(stat_ready + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < L::NSTAGE; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(kv_full, 1);
    mbar_init(sdp_full, 1);
    mbar_init(stat_ready, 2 * Bwd128Smem::BQ2);
    mbar_init(pds_ready, BWD128_SOFTMAX);
    mbar_init(dq_full, 1);
    mbar_init(dq_free, BWD128_SOFTMAX);
    mbar_init(sdp_free, BWD128_SOFTMAX);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmdO);
    tma_prefetch_desc(&tmdQ);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base, tmem_dP = tmem_base + 64, tmem_dV = tmem_base + 128, tmem_dK = tmem_base + 256,
                 tmem_dQ = tmem_base + 384, tmem_P16 = tmem_base + 448, tmem_dS16 = tmem_base + 480;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * L::KV_BYTES);
#pragma unroll
      for (int kb = 0; kb < 2; ++kb) {
        tma_load_3d(smem + L::K_OFF + kb * (BKV * 128), &tmK, kv_full, kb * 64, kv_head, doc_start + kv0);
        tma_load_3d(smem + L::V_OFF + kb * (BKV * 128), &tmV, kv_full, kb * 64, kv_head, doc_start + kv0);
      }
      bool ok = true;
      for (int it = 0; it < n_iter && ok; ++it) {
        const int stage = it % L::NSTAGE;
        const uint32_t par = ((it / L::NSTAGE) & 1) ^ 1;
        if (!mbar_wait(&empty_bar[stage], par, p.status, abort_flag, ERR_WAIT_EMPTY)) { ok = false; break; }
        const int head = kv_head * group + it / n_i;
        const int row0 = doc_start + (i_first + it % n_i) * BQ2;
        uint8_t* dst = smem + L::RING_OFF + stage * L::STAGE_BYTES;
        mbar_expect_tx(&full_bar[stage], L::STAGE_BYTES);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
          tma_load_3d(dst + kb * (BQ2 * 128), &tmQ, &full_bar[stage], kb * 64, head, row0);
          tma_load_3d(dst + L::QT_BYTES + kb * (BQ2 * 128), &tmdO, &full_bar[stage], kb * 64, head, row0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_st = make_idesc_bf16(BKV, BQ2, 0, 0);  // S^T, dP^T: A = K / V (K-major), B = Q / dO (K-major)
      constexpr uint32_t idesc_kv = make_idesc_bf16(BKV, DH, 0, 1);   // dV, dK: A = P^T / dS^T in TMEM, B = dO / Q MN-major
      constexpr uint32_t idesc_dq = make_idesc_bf16(DH, BQ2, 1, 1);   // dQ^T: A = K^T (MN-major), B = dS^T (MN-major)
      const uint32_t sK = smem_u32(smem + L::K_OFF), sV = smem_u32(smem + L::V_OFF);
      const uint32_t sDS = smem_u32(smem + L::DS_OFF);
      bool ok = mbar_wait(kv_full, 0, p.status, abort_flag, ERR_WAIT_FULL);
      auto issue_sdp = [&](int it) -> bool {
        const int stage = it % L::NSTAGE;
        if (!mbar_wait(&full_bar[stage], (it / L::NSTAGE) & 1, p.status, abort_flag, ERR_WAIT_FULL)) return false;
        tc_fence_after();
        const uint32_t sQ = smem_u32(smem + L::RING_OFF + stage * L::STAGE_BYTES);
        const uint32_t sdO = sQ + L::QT_BYTES;
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
          const uint64_t ak = make_smem_desc(sK + kb * (BKV * 128), 16, 1024);
          const uint64_t bq = make_smem_desc(sQ + kb * (BQ2 * 128), 16, 1024);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            mma_ss(tmem_S, desc_advance(ak, k * 32), desc_advance(bq, k * 32), idesc_st, (kb | k) ? 1u : 0u);
        }
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
          const uint64_t av = make_smem_desc(sV + kb * (BKV * 128), 16, 1024);
          const uint64_t bd = make_smem_desc(sdO + kb * (BQ2 * 128), 16, 1024);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            mma_ss(tmem_dP, desc_advance(av, k * 32), desc_advance(bd, k * 32), idesc_st, (kb | k) ? 1u : 0u);
        }
        mma_commit(sdp_full);
        return true;
      };
      if (ok && n_iter > 0) ok = issue_sdp(0);
      for (int it = 0; it < n_iter && ok; ++it) {
        const int stage = it % L::NSTAGE;
        const uint32_t sQ = smem_u32(smem + L::RING_OFF + stage * L::STAGE_BYTES);
        const uint32_t sdO = sQ + L::QT_BYTES;
        if (it + 1 < n_iter) {
          if (!mbar_wait(sdp_free, it & 1, p.status, abort_flag, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
          tc_fence_after();
          if (!issue_sdp(it + 1)) { ok = false; break; }
        }
        if (!mbar_wait(pds_ready, it & 1, p.status, abort_flag, ERR_WAIT_MISC)) { ok = false; break; }
        tc_fence_after();
        {
          // B = dO / Q read MN-major: N = 128 head-dim columns in two 64-wide groups 8 KB apart, K = 64 query rows
          const uint64_t bdo = make_smem_desc(sdO, BQ2 * 128, 1024), bq = make_smem_desc(sQ, BQ2 * 128, 1024);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            mma_ts(tmem_dV, tmem_P16 + k * 8, desc_advance(bdo, k * 2048), idesc_kv, (it > 0 || k > 0) ? 1u : 0u);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            mma_ts(tmem_dK, tmem_dS16 + k * 8, desc_advance(bq, k * 2048), idesc_kv, (it > 0 || k > 0) ? 1u : 0u);
        }
        if (it > 0) {
          if (!mbar_wait(dq_free, (it - 1) & 1, p.status, abort_flag, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
          tc_fence_after();
        }
        {
          // A = K^T: M = 128 head-dim rows in two 64-wide groups 16 KB apart, K = 128 keys (2 KB per 16);
          // B = dS^T: N = 64 queries (one group), K = 128 keys
          const uint64_t akt = make_smem_desc(sK, BKV * 128, 1024), bds = make_smem_desc(sDS, 16, 1024);
#pragma unroll
          for (int k = 0; k < 8; ++k)
            mma_ss(tmem_dQ, desc_advance(akt, k * 2048), desc_advance(bds, k * 2048), idesc_dq, k ? 1u : 0u);
        }
        mma_commit(&empty_bar[stage]);
        mma_commit(dq_full);  // also: P^T / dS^T in tensor memory and dS^T in shared memory may be overwritten
      }
    }
  } else {
    const int sw = warp - 2;        // 0..7
    const int quarter = warp & 3;   // TMEM lane quarter this warp may access
    const int half = sw >> 2;       // which 32 of the 64 query columns
    const int r = quarter * 32 + lane;  // key row inside the tile (also: head-dim row of dQ^T)
    const int st_tid = sw * 32 + lane;  // 0..255 inside the softmax group
    const uint32_t lane_sel = (uint32_t)(quarter * 32) << 16;
    uint8_t* sDS = smem + L::DS_OFF;
    float* stats = reinterpret_cast<float*>(smem + L::STAT_OFF);
    uint8_t* slab = smem + L::DQ_OFF + (quarter * 2 + half) * 4096;  // [32 queries][32 head-dim columns] fp32
    bool ok = true;
    uint32_t dq_regs[32];
    bool have_dq = false;
    int dq_head = 0, dq_row0 = 0;
    auto flush_dq = [&]() {
      if (lane == 0) tma_store_wait_read<0>();
      __syncwarp();
#pragma unroll
      for (int x = 0; x < 32; ++x)
        *reinterpret_cast<float*>(slab + x * 128 + lane * 4) = __uint_as_float(dq_regs[x]) * p.scale;
      fence_async_smem();
      __syncwarp();
      if (lane == 0 && dq_row0 + half * 32 < p.total_tokens) {
        tma_reduce_add_3d(&tmdQ, slab, quarter * 32, dq_head, dq_row0 + half * 32);
        tma_store_commit();
      }
      have_dq = false;
    };
    // row statistics of the NEXT query tile: threads 0..63 fetch lse, 64..127 fetch delta
    float stat_next = 0.f;
    auto fetch_stat = [&](int it) {
      if (st_tid < 2 * BQ2) {
        const int head = kv_head * group + it / n_i;
        const int q_idx = (i_first + it % n_i) * BQ2 + (st_tid & (BQ2 - 1));
        const bool is_lse = st_tid < BQ2;
        if (q_idx < doc_len) {
          const long long tok = (long long)doc_start + q_idx;
          stat_next = __ldg((is_lse ? p.lse : p.delta) + (long long)head * p.total_tokens + tok);
        } else {
          stat_next = is_lse ? INFINITY : 0.f;
        }
      }
    };
    if (n_iter > 0) fetch_stat(0);
    for (int it = 0; it < n_iter && ok; ++it) {
      const int head = kv_head * group + it / n_i;
      const int i = i_first + it % n_i;
      float* st = stats + (it & 1) * (2 * BQ2);
      // Buffer (it & 1) was last read for tile it - 2; every thread finished those reads before it arrived on
      // pds_ready(it - 2), which the products awaited through dq_full(it - 2) depend on: the writers are past that wait.
      if (st_tid < 2 * BQ2) {
        st[st_tid] = stat_next;
        mbar_arrive(stat_ready);
      }
      if (it + 1 < n_iter) fetch_stat(it + 1);
      if (!mbar_wait_warp(stat_ready, it & 1, p.status, abort_flag, ERR_WAIT_MISC)) { ok = false; break; }
      const int q_base = i * BQ2 + half * 32;  // document position of this thread's first query column
      const int kv = kv0 + r;
      const bool need_mask = (kv0 + BKV - 1 > i * BQ2) || (p.window > 0 && kv0 <= i * BQ2 + BQ2 - 1 - p.window);
      if (!mbar_wait_warp(sdp_full, it & 1, p.status, abort_flag, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      uint32_t sv[32], dv[32];
      tmem_ld_32x32(tmem_S + lane_sel + half * 32, sv);
      tmem_ld_32x32(tmem_dP + lane_sel + half * 32, dv);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(sdp_free);
      if (need_mask) {
#pragma unroll
        for (int x = 0; x < 32; ++x) {
          const int q_idx = q_base + x;
          if ((kv > q_idx) || (p.window > 0 && kv <= q_idx - p.window)) sv[x] = 0xff800000u;
        }
      }
      const float4* lse4 = reinterpret_cast<const float4*>(st + half * 32);
      const float4* dlt4 = reinterpret_cast<const float4*>(st + BQ2 + half * 32);
#pragma unroll
      for (int x = 0; x < 32; x += 4) {
        const float4 l = lse4[x >> 2], d = dlt4[x >> 2];
        const float e0 = fast_exp2(fmaf(__uint_as_float(sv[x]), p.scale_log2, -l.x));
        const float e1 = fast_exp2(fmaf(__uint_as_float(sv[x + 1]), p.scale_log2, -l.y));
        const float e2 = fast_exp2(fmaf(__uint_as_float(sv[x + 2]), p.scale_log2, -l.z));
        const float e3 = fast_exp2(fmaf(__uint_as_float(sv[x + 3]), p.scale_log2, -l.w));
        const float g0 = e0 * (__uint_as_float(dv[x]) - d.x);
        const float g1 = e1 * (__uint_as_float(dv[x + 1]) - d.y);
        const float g2 = e2 * (__uint_as_float(dv[x + 2]) - d.z);
        const float g3 = e3 * (__uint_as_float(dv[x + 3]) - d.w);
        sv[x >> 1] = pack_bf16(e0, e1);
        sv[(x >> 1) + 1] = pack_bf16(e2, e3);
        dv[x >> 1] = pack_bf16(g0, g1);
        dv[(x >> 1) + 1] = pack_bf16(g2, g3);
      }
      // the previous tile's dV / dK / dQ^T products read P^T / dS^T and fill the dQ^T columns
      if (it > 0) {
        if (!mbar_wait_warp(dq_full, (it - 1) & 1, p.status, abort_flag, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
        tc_fence_after();
        tmem_ld_32x32(tmem_dQ + lane_sel + half * 32, dq_regs);
        tmem_ld_wait();
        have_dq = true;
        tc_fence_before();
        mbar_arrive(dq_free);
      }
      tmem_st_32x16(tmem_P16 + lane_sel + half * 16, *reinterpret_cast<uint32_t(*)[16]>(&sv[0]));
      tmem_st_32x16(tmem_dS16 + lane_sel + half * 16, *reinterpret_cast<uint32_t(*)[16]>(&dv[0]));
#pragma unroll
      for (int c = 0; c < 32; c += 8)
        *reinterpret_cast<uint4*>(sDS + sw128_offset(r, half * 32 + c)) =
            make_uint4(dv[c / 2], dv[c / 2 + 1], dv[c / 2 + 2], dv[c / 2 + 3]);
      tmem_st_wait();
      tc_fence_before();
      fence_async_smem();
      mbar_arrive(pds_ready);
      if (have_dq) flush_dq();
      dq_head = head;
      dq_row0 = doc_start + i * BQ2;
    }
    if (ok && n_iter > 0) ok = mbar_wait_warp(dq_full, (n_iter - 1) & 1, p.status, abort_flag, ERR_WAIT_TMEM_FULL);
    if (ok && n_iter > 0) {
      tc_fence_after();
      tmem_ld_32x32(tmem_dQ + lane_sel + half * 32, dq_regs);
      tmem_ld_wait();
      have_dq = true;
      flush_dq();
      // dK, dV of key row r; this thread owns 64 of the 128 head-dim columns
      const int kv_idx = kv0 + r;
      const bool kvalid = kv_idx < doc_len;
      const long long ktok = (long long)doc_start + kv_idx;
      __nv_bfloat16* dkrow = p.dK + ktok * p.dk_stride_t + (long long)kv_head * DH + half * 64;
      __nv_bfloat16* dvrow = p.dV + ktok * p.dv_stride_t + (long long)kv_head * DH + half * 64;
#pragma unroll 1
      for (int c = 0; c < 64; c += 32) {
        uint32_t a[32], b[32];
        tmem_ld_32x32(tmem_dK + lane_sel + half * 64 + c, a);
        tmem_ld_32x32(tmem_dV + lane_sel + half * 64 + c, b);
        tmem_ld_wait();
        if (kvalid) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 q;
            q.x = pack_bf16(__uint_as_float(a[g * 8 + 0]) * p.scale, __uint_as_float(a[g * 8 + 1]) * p.scale);
            q.y = pack_bf16(__uint_as_float(a[g * 8 + 2]) * p.scale, __uint_as_float(a[g * 8 + 3]) * p.scale);
            q.z = pack_bf16(__uint_as_float(a[g * 8 + 4]) * p.scale, __uint_as_float(a[g * 8 + 5]) * p.scale);
            q.w = pack_bf16(__uint_as_float(a[g * 8 + 6]) * p.scale, __uint_as_float(a[g * 8 + 7]) * p.scale);
            *reinterpret_cast<uint4*>(dkrow + c + g * 8) = q;
            q.x = pack_bf16(__uint_as_float(b[g * 8 + 0]), __uint_as_float(b[g * 8 + 1]));
            q.y = pack_bf16(__uint_as_float(b[g * 8 + 2]), __uint_as_float(b[g * 8 + 3]));
            q.z = pack_bf16(__uint_as_float(b[g * 8 + 4]), __uint_as_float(b[g * 8 + 5]));
            q.w = pack_bf16(__uint_as_float(b[g * 8 + 6]), __uint_as_float(b[g * 8 + 7]));
            *reinterpret_cast<uint4*>(dvrow + c + g * 8) = q;
          }
        }
      }
    }
    if (lane == 0) tma_store_wait_all<0>();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// tile_offsets[i] = sum_{d < i} ceil(len_d / 128); single CTA, sequential over documents in chunks
__global__ void attn_tile_offsets_kernel(const int* __restrict__ cu, int nseq, int* __restrict__ offs) {
  if (threadIdx.x == 0) {
    int acc = 0;
    offs[0] = 0;
    for (int d = 0; d < nseq; ++d) {
      acc += (cu[d + 1] - cu[d] + BQ - 1) / BQ;
      offs[d + 1] = acc;
    }
  }
}

template <typename K>
int set_smem(K kern, int bytes) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) {
    fprintf(stderr, "[flame_b200] attention: cannot opt in to %d bytes of shared memory: %s\n", bytes,
            cudaGetErrorString(e));
    return (int)e;
  }
  return 0;
}

int make_qkv_map(CUtensorMap* m, const void* base, long long T, int H, int DH, long long stride_t, int box_rows = 128) {
  // dims (inner to outer): [DH, H, T]; box [64, 1, box_rows]
  return fb::make_tmap_3d(m, base, 2, (uint64_t)T, (uint64_t)H, (uint64_t)DH, (uint64_t)stride_t, (uint64_t)DH,
                          (uint32_t)box_rows, 1, 64, true);
}

}  // namespace

extern "C" {


int fb_attn_tile_offsets(const int* cu_seqlens, int nseq, int* tile_offsets, cudaStream_t stream) {
  attn_tile_offsets_kernel<<<1, 32, 0, stream>>>(cu_seqlens, nseq, tile_offsets);
  return fb::launch_ok("attn_tile_offsets_kernel");
}

// max_tiles: an upper bound on the number of 128-row tiles (T / 128 + nseq is always enough).
int fb_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int* cu_seqlens,
                const int* tile_offsets, int nseq, int max_tiles, long long T, int H, int Hkv, int DH,
                long long q_stride_t, long long k_stride_t, long long v_stride_t, long long o_stride_t, float scale,
                int window, cudaStream_t stream) {
  if (T == 0) return 0;
  if (DH != 64 && DH != 128) return -2;
  if ((q_stride_t % 8) || (k_stride_t % 8) || (v_stride_t % 8) || (o_stride_t % 8)) return -3;
  CUtensorMap tmQ, tmK, tmV;
  int rc = make_qkv_map(&tmQ, q, T, H, DH, q_stride_t);
  if (!rc) rc = make_qkv_map(&tmK, k, T, Hkv, DH, k_stride_t);
  if (!rc) rc = make_qkv_map(&tmV, v, T, Hkv, DH, v_stride_t);
  if (rc) return rc;
  AttnParams p;
  p.cu_seqlens = cu_seqlens;
  p.tile_offsets = tile_offsets;
  p.nseq = nseq;
  p.H = H;
  p.Hkv = Hkv;
  p.total_tokens = (int)T;
  p.window = window;
  p.scale = scale;
  p.scale_log2 = scale * kLog2e;
  p.O = (__nv_bfloat16*)o;
  p.o_stride_t = o_stride_t;
  p.O_lo = nullptr;
  p.lse = lse;
  p.status = fb::status_ptr();
  dim3 grid(max_tiles, H);
  static const bool p_in_tmem = []() {
    const char* e = getenv("FLAME_B200_ATTN_FWD_PT");  // 0: the version of the kernel that stages P in shared memory
    return !(e && e[0] == '0');
  }();
  if (DH == 64 && p_in_tmem) {
    static bool done = false;
    if (!done) { rc = set_smem(attn_fwd_pt_kernel, FwdPtSmem::TOTAL); if (rc) return rc; done = true; }
    attn_fwd_pt_kernel<<<grid, 192, FwdPtSmem::TOTAL, stream>>>(tmQ, tmK, tmV, p);
  } else if (DH == 64) {
    static bool done = false;
    if (!done) { rc = set_smem(attn_fwd_kernel<64, 0>, FwdSmem<64>::TOTAL); if (rc) return rc; done = true; }
    attn_fwd_kernel<64, 0><<<grid, 192, FwdSmem<64>::TOTAL, stream>>>(tmQ, tmK, tmV, p);
  } else {
    static bool done = false;
    if (!done) { rc = set_smem(attn_fwd_kernel<128, 0>, FwdSmem<128>::TOTAL); if (rc) return rc; done = true; }
    attn_fwd_kernel<128, 0><<<grid, 192, FwdSmem<128>::TOTAL, stream>>>(tmQ, tmK, tmV, p);
  }
  return fb::launch_ok("attn_fwd_kernel");
}

// Stick-breaking attention forward (head dim 64): o = sum_j att_ij v_j without normalisation, rem[h, t] = 1 - sum_j att_ij.
// o_lo: optional bf16 [T, H, 64] that receives the part of the fp32 result the bf16 output lost (null: not written).
int fb_sb_attn_fwd(const void* q, const void* k, const void* v, void* o, void* o_lo, float* rem, const int* cu_seqlens,
                   const int* tile_offsets, int nseq, int max_tiles, long long T, int H, int DH, long long q_stride_t,
                   long long k_stride_t, long long v_stride_t, long long o_stride_t, float scale, cudaStream_t stream) {
  if (T == 0) return 0;
  if (DH != 64) return -2;
  if ((q_stride_t % 8) || (k_stride_t % 8) || (v_stride_t % 8) || (o_stride_t % 8)) return -3;
  CUtensorMap tmQ, tmK, tmV;
  int rc = make_qkv_map(&tmQ, q, T, H, DH, q_stride_t);
  if (!rc) rc = make_qkv_map(&tmK, k, T, H, DH, k_stride_t);
  if (!rc) rc = make_qkv_map(&tmV, v, T, H, DH, v_stride_t);
  if (rc) return rc;
  AttnParams p;
  p.cu_seqlens = cu_seqlens;
  p.tile_offsets = tile_offsets;
  p.nseq = nseq;
  p.H = H;
  p.Hkv = H;
  p.total_tokens = (int)T;
  p.window = 0;
  p.scale = scale;
  p.scale_log2 = scale * kLog2e;
  p.O = (__nv_bfloat16*)o;
  p.o_stride_t = o_stride_t;
  p.O_lo = (__nv_bfloat16*)o_lo;
  p.lse = rem;
  p.status = fb::status_ptr();
  static bool done = false;
  if (!done) { rc = set_smem(attn_fwd_kernel<64, 1>, FwdSmem<64>::TOTAL); if (rc) return rc; done = true; }
  dim3 grid(max_tiles, H);
  attn_fwd_kernel<64, 1><<<grid, 192, FwdSmem<64>::TOTAL, stream>>>(tmQ, tmK, tmV, p);
  return fb::launch_ok("attn_fwd_kernel<sb>");
}

int fb_attn_delta(const void* o, const void* dout, float* delta, long long T, int H, int DH, long long o_stride_t,
                  long long do_stride_t, cudaStream_t stream) {
  if (T == 0) return 0;
  if (DH != 64 && DH != 128) return -2;
  const long long threads = T * H * (DH / 8);
  const unsigned blocks = (unsigned)((threads + 255) / 256);
  if (DH == 64)
    attn_delta_kernel<64><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, delta, T, H,
                                                      o_stride_t, do_stride_t);
  else
    attn_delta_kernel<128><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, delta, T, H,
                                                       o_stride_t, do_stride_t);
  return fb::launch_ok("attn_delta_kernel");
}

// dq_accum: fp32 [T, H, DH], must be zero on entry.  Head dims 64 and 128 (two kernels, see above).
int fb_attn_bwd(const void* q, const void* k, const void* v, const void* dout, const float* lse, const float* delta,
                float* dq_accum, void* dk, void* dv, const int* cu_seqlens, const int* tile_offsets, int nseq,
                int max_tiles, long long T, int H, int Hkv, int DH, long long q_stride_t, long long k_stride_t,
                long long v_stride_t, long long do_stride_t, long long dk_stride_t, long long dv_stride_t, float scale,
                int window, cudaStream_t stream) {
  if (T == 0) return 0;
  if (DH != 64 && DH != 128) return -2;
  if ((q_stride_t % 8) || (k_stride_t % 8) || (v_stride_t % 8) || (do_stride_t % 8) || (dk_stride_t % 8) ||
      (dv_stride_t % 8))
    return -3;
  CUtensorMap tmQ, tmK, tmV, tmdO, tmdQ;
  const int q_rows = DH == 64 ? 128 : Bwd128Smem::BQ2;  // query rows per Q / dO box
  int rc = make_qkv_map(&tmQ, q, T, H, DH, q_stride_t, q_rows);
  if (!rc) rc = make_qkv_map(&tmK, k, T, Hkv, DH, k_stride_t);
  if (!rc) rc = make_qkv_map(&tmV, v, T, Hkv, DH, v_stride_t);
  if (!rc) rc = make_qkv_map(&tmdO, dout, T, H, DH, do_stride_t, q_rows);
  // fp32 dQ accumulator [T, H, DH], reduced into with TMA adds.  Head dim 64: boxes of 32 rows x 16 columns (64 bytes,
  // 64-byte swizzle); head dim 128: boxes of 32 rows x 32 columns (128 bytes, no swizzle)
  if (!rc && DH == 64)
    rc = fb::make_tmap_3d(&tmdQ, dq_accum, 4, (uint64_t)T, (uint64_t)H, (uint64_t)DH, (uint64_t)H * DH, (uint64_t)DH,
                          32, 1, 16, fb::kSwizzle64);
  if (!rc && DH == 128)
    rc = fb::make_tmap_3d(&tmdQ, dq_accum, 4, (uint64_t)T, (uint64_t)H, (uint64_t)DH, (uint64_t)H * DH, (uint64_t)DH,
                          32, 1, 32, 0);
  if (rc) return rc;
  AttnBwdParams p;
  p.cu_seqlens = cu_seqlens;
  p.tile_offsets = tile_offsets;
  p.nseq = nseq;
  p.H = H;
  p.Hkv = Hkv;
  p.total_tokens = (int)T;
  p.window = window;
  p.scale = scale;
  p.scale_log2 = scale * kLog2e;
  p.lse = lse;
  p.delta = delta;
  p.dQ = dq_accum;
  p.dK = (__nv_bfloat16*)dk;
  p.dV = (__nv_bfloat16*)dv;
  p.dk_stride_t = dk_stride_t;
  p.dv_stride_t = dv_stride_t;
  p.status = fb::status_ptr();
  dim3 grid(max_tiles, Hkv);
  if (DH == 128) {
    static bool done128 = false;
    if (!done128) { rc = set_smem(attn_bwd128_kernel, Bwd128Smem::TOTAL); if (rc) return rc; done128 = true; }
    attn_bwd128_kernel<<<grid, BWD128_THREADS, Bwd128Smem::TOTAL, stream>>>(tmQ, tmK, tmV, tmdO, tmdQ, p);
    return fb::launch_ok("attn_bwd128_kernel");
  }
  static bool done = false;
  if (!done) { rc = set_smem(attn_bwd_kernel<64>, BwdSmem<64>::TOTAL); if (rc) return rc; done = true; }
  attn_bwd_kernel<64><<<grid, BWD_THREADS, BwdSmem<64>::TOTAL, stream>>>(tmQ, tmK, tmV, tmdO, tmdQ, p);
  return fb::launch_ok("attn_bwd_kernel");
}

}  // extern "C"
