// Stick-breaking attention backward for sm_100a (head dim 64), packed variable-length documents.
//
//   att_ij = sigma_ij * prod_{j<m<i} (1 - sigma_im)   (j < i),   o_i = sum_j att_ij v_j,   rem_i = 1 - sum_j att_ij
//   g_ij   = do_i . v_j - drem_i,   dA = att * g,   dl_ij = dA_ij - sigma_ij * sum_{k<=j} dA_ik
//   dq_i = scale sum_j dl_ij k_j,   dk_j = scale sum_i dl_ij q_i,   dv_j = sum_i att_ij do_i
//
// One CTA owns a 128-query tile of one (document, head) and walks the key tiles from the diagonal backwards - the
// direction in which both running quantities of a row are available: E = prod (1 - sigma) over the keys already
// seen (so att = sigma * E) and R = sum of dA over the keys already seen; the prefix sum the gradient needs is
// Tot_i - R with Tot_i = do_i . o_i - drem_i (1 - rem_i), known up front.  Per key tile the tensor core forms S and dP,
// one thread per query row turns them into P = att and dS = dl (bf16, swizzled smem), and three more MMAs produce the
// tile's dV, dK (fresh each tile, added to fp32 accumulators in global memory by TMA reduce) and dQ (accumulated in
// TMEM across the whole walk, no atomics).  The reference reaches the same sums with spin-locked adds
// (custom_models/sba/stickbreaking_attention/sb_varlen/sb_varlen_bwd.py:13-52); here nothing spins unbounded.
#include "tc05.cuh"
#include "host_utils.cuh"
#include <math.h>

using namespace tc05;

namespace {

constexpr int BQ = 128, BKV = 128, DH = 64;
constexpr float kLog2e = 1.4426950408889634f;

struct SbBwdParams {
  const int* cu_seqlens;
  const int* tile_offsets;
  int nseq, H, total_tokens;
  float scale, scale_log2;
  const float* tot;    // [H, T]  do.o - drem (1 - rem)
  const float* drem;   // [H, T] or null
  __nv_bfloat16* dQ;   // [T, H, DH] with token stride dq_stride_t
  long long dq_stride_t;
  int* status;
};

__device__ __forceinline__ int upper_doc(const int* __restrict__ offs, int n, int x) {
  int lo = 0, hi = n;
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (offs[mid] <= x) lo = mid; else hi = mid;
  }
  return lo;
}
__device__ __forceinline__ uint32_t sw128_offset(int row, int col) {
  const int chunk = (col >> 3) ^ (row & 7);
  return (uint32_t)(row * 128 + chunk * 16 + (col & 7) * 2);
}

struct Smem {
  static constexpr int TILE = 128 * DH * 2;          // 16 KB
  static constexpr int Q_OFF = 0, DO_OFF = TILE;
  static constexpr int NSTAGE = 2;
  static constexpr int RING_OFF = 2 * TILE;          // stage = K tile + V tile
  static constexpr int STAGE = 2 * TILE;
  static constexpr int P_OFF = RING_OFF + NSTAGE * STAGE;
  static constexpr int PD = BQ * BKV * 2;            // 32 KB
  static constexpr int DS_OFF = P_OFF + PD;
  static constexpr int STG_OFF = DS_OFF + PD;        // fp32 staging for the dK / dV reduce: 2 x [128][32]
  static constexpr int STG = 128 * DH * 4;
  static constexpr int BAR_OFF = STG_OFF + STG;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

__global__ void __launch_bounds__(192, 1)
sb_attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                   const __grid_constant__ CUtensorMap tmdK, const __grid_constant__ CUtensorMap tmdV, SbBwdParams p) {
  using L = Smem;
  const int total_tiles = p.tile_offsets[p.nseq];
  const int tile_id = total_tiles - 1 - (int)blockIdx.x;  // long walks first
  if (tile_id < 0) return;
  const int head = blockIdx.y;
  const int doc = upper_doc(p.tile_offsets, p.nseq + 1, tile_id);
  const int ti = tile_id - p.tile_offsets[doc];
  const int doc_start = p.cu_seqlens[doc];
  const int doc_len = p.cu_seqlens[doc + 1] - doc_start;
  const int q0 = ti * BQ;
  const int n_iter = ti + 1;  // key tiles ti, ti-1, ..., 0

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = (uint64_t*)(smem + L::BAR_OFF);
  uint64_t* empty_bar = full_bar + L::NSTAGE;
  uint64_t* q_full = empty_bar + L::NSTAGE;
  uint64_t* sdp_full = q_full + 1;
  uint64_t* pds_ready = sdp_full + 1;
  uint64_t* dkv_full = pds_ready + 1;
  uint64_t* dkv_free = dkv_full + 1;
  uint64_t* grp_bar = dkv_free + 1;
  uint32_t* tmem_slot = (uint32_t*)(grp_bar + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < L::NSTAGE; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(q_full, 1);
    mbar_init(sdp_full, 1);
    mbar_init(pds_ready, 128);
    mbar_init(dkv_full, 1);
    mbar_init(dkv_free, 128);
    mbar_init(grp_bar, 128);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmdO);
    tma_prefetch_desc(&tmdK);
    tma_prefetch_desc(&tmdV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base, tmem_dP = tmem_base + 128, tmem_dV = tmem_base + 256, tmem_dK = tmem_base + 320,
                 tmem_dQ = tmem_base + 384;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, 2 * L::TILE);
      tma_load_3d(smem + L::Q_OFF, &tmQ, q_full, 0, head, doc_start + q0);
      tma_load_3d(smem + L::DO_OFF, &tmdO, q_full, 0, head, doc_start + q0);
      bool ok = true;
      for (int it = 0; it < n_iter && ok; ++it) {
        const int stage = it % L::NSTAGE;
        if (!mbar_wait(&empty_bar[stage], ((it / L::NSTAGE) & 1) ^ 1, p.status, abort_flag, ERR_WAIT_EMPTY)) { ok = false; break; }
        const int j = ti - it;
        uint8_t* dst = smem + L::RING_OFF + stage * L::STAGE;
        mbar_expect_tx(&full_bar[stage], L::STAGE);
        tma_load_3d(dst, &tmK, &full_bar[stage], 0, head, doc_start + j * BKV);
        tma_load_3d(dst + L::TILE, &tmV, &full_bar[stage], 0, head, doc_start + j * BKV);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BQ, BKV, 0, 0);
      constexpr uint32_t idesc_kv = make_idesc_bf16(BKV, DH, 1, 1);
      constexpr uint32_t idesc_dq = make_idesc_bf16(BQ, DH, 0, 1);
      const uint32_t sQ = smem_u32(smem + L::Q_OFF), sdO = smem_u32(smem + L::DO_OFF);
      const uint32_t sP = smem_u32(smem + L::P_OFF), sDS = smem_u32(smem + L::DS_OFF);
      bool ok = mbar_wait(q_full, 0, p.status, abort_flag, ERR_WAIT_FULL);
      auto issue_sdp = [&](int it) -> bool {
        const int stage = it % L::NSTAGE;
        if (!mbar_wait(&full_bar[stage], (it / L::NSTAGE) & 1, p.status, abort_flag, ERR_WAIT_FULL)) return false;
        tc_fence_after();
        const uint32_t sK = smem_u32(smem + L::RING_OFF + stage * L::STAGE), sV = sK + L::TILE;
        const uint64_t aq = make_smem_desc(sQ, 16, 1024), bk = make_smem_desc(sK, 16, 1024);
        const uint64_t ad = make_smem_desc(sdO, 16, 1024), bv = make_smem_desc(sV, 16, 1024);
#pragma unroll
        for (int k = 0; k < 4; ++k) mma_ss(tmem_S, desc_advance(aq, k * 32), desc_advance(bk, k * 32), idesc_s, k ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < 4; ++k) mma_ss(tmem_dP, desc_advance(ad, k * 32), desc_advance(bv, k * 32), idesc_s, k ? 1u : 0u);
        mma_commit(sdp_full);
        return true;
      };
      if (ok) ok = issue_sdp(0);
      for (int it = 0; it < n_iter && ok; ++it) {
        const int stage = it % L::NSTAGE;
        const uint32_t sK = smem_u32(smem + L::RING_OFF + stage * L::STAGE);
        if (!mbar_wait(pds_ready, it & 1, p.status, abort_flag, ERR_WAIT_MISC)) { ok = false; break; }
        tc_fence_after();
        if (it > 0) {  // the previous tile's dK / dV must have left TMEM
          if (!mbar_wait(dkv_free, (it - 1) & 1, p.status, abort_flag, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
          tc_fence_after();
        }
        {
          const uint64_t ap = make_smem_desc(sP, BQ * 128, 1024), ads = make_smem_desc(sDS, BQ * 128, 1024);
          const uint64_t bdo = make_smem_desc(sdO, 16, 1024), bq = make_smem_desc(sQ, 16, 1024);
#pragma unroll
          for (int k = 0; k < 8; ++k)
            mma_ss(tmem_dV, desc_advance(ap, k * 2048), desc_advance(bdo, k * 2048), idesc_kv, k ? 1u : 0u);
#pragma unroll
          for (int k = 0; k < 8; ++k)
            mma_ss(tmem_dK, desc_advance(ads, k * 2048), desc_advance(bq, k * 2048), idesc_kv, k ? 1u : 0u);
          const uint64_t bk = make_smem_desc(sK, 16, 1024);
#pragma unroll
          for (int kb = 0; kb < 2; ++kb) {
            const uint64_t a2 = make_smem_desc(sDS + kb * (BQ * 128), 16, 1024);
#pragma unroll
            for (int k = 0; k < 4; ++k)
              mma_ss(tmem_dQ, desc_advance(a2, k * 32), desc_advance(bk, (kb * 4 + k) * 2048), idesc_dq,
                     (it > 0 || kb > 0 || k > 0) ? 1u : 0u);
          }
        }
        mma_commit(&empty_bar[stage]);
        mma_commit(dkv_full);
        if (it + 1 < n_iter) {
          if (!issue_sdp(it + 1)) { ok = false; break; }
        }
      }
    }
  } else {
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t lane_sel = (uint32_t)(quarter * 32) << 16;
    uint8_t* sP = smem + L::P_OFF;
    uint8_t* sDS = smem + L::DS_OFF;
    uint8_t* sSTG = smem + L::STG_OFF;
    const bool issuer = (warp == 2 && lane == 0);
    const int q_idx = q0 + r;
    const bool valid = q_idx < doc_len;
    const long long tok = (long long)doc_start + q_idx;
    const float tot = valid ? p.tot[(long long)head * p.total_tokens + tok] : 0.f;
    const float drem = (valid && p.drem != nullptr) ? p.drem[(long long)head * p.total_tokens + tok] : 0.f;
    float E = 1.f;  // product of (1 - sigma) over the keys already seen
    float R = 0.f;  // sum of dA over the keys already seen
    bool ok = true;
    uint32_t grp_phase = 0;
    auto group_sync = [&]() -> bool {
      mbar_arrive(grp_bar);
      const bool done = mbar_wait_warp(grp_bar, grp_phase, p.status, abort_flag, ERR_WAIT_MISC);
      grp_phase ^= 1;
      return done;
    };
    // adds one [128 keys][64] fp32 tile (TMEM columns at `taddr`, scaled) to the global accumulator behind `tm`
    auto flush_tile = [&](uint32_t taddr, const CUtensorMap* tm, float mul, int row0) -> bool {
      if (issuer) tma_store_wait_read<0>();
      if (!group_sync()) return false;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t v[32];
        tmem_ld_32x32(taddr + lane_sel + half * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          float4 q = make_float4(__uint_as_float(v[g * 4 + 0]) * mul, __uint_as_float(v[g * 4 + 1]) * mul,
                                 __uint_as_float(v[g * 4 + 2]) * mul, __uint_as_float(v[g * 4 + 3]) * mul);
          *reinterpret_cast<float4*>(sSTG + half * (128 * 128) + r * 128 + ((g ^ (r & 7)) << 4)) = q;
        }
      }
      fence_async_smem();
      if (!group_sync()) return false;
      if (issuer) {
        tma_reduce_add_3d(tm, sSTG, 0, head, row0);
        tma_reduce_add_3d(tm, sSTG + 128 * 128, 32, head, row0);
        tma_store_commit();
      }
      return true;
    };
    for (int it = 0; it < n_iter && ok; ++it) {
      const int j = ti - it;
      const int kv0 = j * BKV;
      const bool diag = (it == 0);
      if (!mbar_wait_warp(sdp_full, it & 1, p.status, abort_flag, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
#pragma unroll 1
      for (int c0 = BKV - 32; c0 >= 0; c0 -= 32) {
        uint32_t xr[32], dr[32];
        tmem_ld_32x32(tmem_S + lane_sel + c0, xr);
        tmem_ld_32x32(tmem_dP + lane_sel + c0, dr);
        tmem_ld_wait();
#pragma unroll
        for (int c = 24; c >= 0; c -= 8) {
          float a[8], d[8];
#pragma unroll
          for (int i = 7; i >= 0; --i) {
            const bool dead = !valid || (diag && (kv0 + c0 + c + i >= q_idx));
            float x = __uint_as_float(xr[c + i]) * p.scale_log2;
            x = fminf(fmaxf(x, -100.f), 100.f);
            const float t = exp2f(x);
            const float inv = __frcp_rn(1.f + t);
            const float sig = t * inv;
            const float att = dead ? 0.f : sig * E;
            // The forward formed o from the bf16 rounding of att, and tot = do . o is the total the running sum R has to
            // meet exactly at the end of the walk: the same rounded weight enters dA here (the remainder term keeps the
            // fp32 weight, as rem was formed from it).  With fp32 att in this place the mismatch of the two roundings,
            // multiplied by sigma for every key of the row, was a 20 % error in dq at 4096-token rows.
            const float att16 = __bfloat162float(__float2bfloat16(att));
            const float dA = att16 * __uint_as_float(dr[c + i]) - att * drem;
            a[i] = att;
            d[i] = dead ? 0.f : dA - sig * (tot - R);
            R += dA;
            E = dead ? E : E * inv;
          }
          const int cc = c0 + c;
          const uint32_t off = (cc >> 6) * (BQ * 128) + sw128_offset(r, cc & 63);
          uint4 q;
          q.x = pack_bf16(a[0], a[1]); q.y = pack_bf16(a[2], a[3]); q.z = pack_bf16(a[4], a[5]); q.w = pack_bf16(a[6], a[7]);
          *reinterpret_cast<uint4*>(sP + off) = q;
          q.x = pack_bf16(d[0], d[1]); q.y = pack_bf16(d[2], d[3]); q.z = pack_bf16(d[4], d[5]); q.w = pack_bf16(d[6], d[7]);
          *reinterpret_cast<uint4*>(sDS + off) = q;
        }
      }
      tc_fence_before();
      fence_async_smem();
      mbar_arrive(pds_ready);
      // this tile's dV and dK: wait for the MMAs, move them out through the staging tile, release TMEM
      if (!mbar_wait_warp(dkv_full, it & 1, p.status, abort_flag, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      if (!flush_tile(tmem_dV, &tmdV, 1.f, doc_start + kv0)) { ok = false; break; }
      if (!flush_tile(tmem_dK, &tmdK, p.scale, doc_start + kv0)) { ok = false; break; }
      tc_fence_before();
      mbar_arrive(dkv_free);
    }
    if (ok) {
      // dQ of this query tile: all MMAs are complete (dkv_full of the last tile covered them)
      tc_fence_after();
      __nv_bfloat16* dqrow = p.dQ + tok * p.dq_stride_t + (long long)head * DH;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_dQ + lane_sel + half * 32, v);
        tmem_ld_wait();
        if (valid) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 q;
            q.x = pack_bf16(__uint_as_float(v[g * 8 + 0]) * p.scale, __uint_as_float(v[g * 8 + 1]) * p.scale);
            q.y = pack_bf16(__uint_as_float(v[g * 8 + 2]) * p.scale, __uint_as_float(v[g * 8 + 3]) * p.scale);
            q.z = pack_bf16(__uint_as_float(v[g * 8 + 4]) * p.scale, __uint_as_float(v[g * 8 + 5]) * p.scale);
            q.w = pack_bf16(__uint_as_float(v[g * 8 + 6]) * p.scale, __uint_as_float(v[g * 8 + 7]) * p.scale);
            *reinterpret_cast<uint4*>(dqrow + half * 32 + g * 8) = q;
          }
        }
      }
      if (issuer) tma_store_wait_all<0>();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// tot[h, t] = do.o - drem * (1 - rem).  The prefix sums the gradient needs are formed as tot - (running sum of dA), a
// difference of nearly equal numbers for the far keys, and every key's dl carries sigma times its error: with o rounded
// to bf16 the error of dq / dk grows with the row length (7 % at 1000 tokens, 22 % at 4096).  So o enters as the
// two-term split o + o_lo that the forward kernel writes (16 mantissa bits), which makes tot agree with the running sum
// to fp32 accuracy.
__global__ void sb_tot_kernel(const __nv_bfloat16* __restrict__ O, const __nv_bfloat16* __restrict__ O_lo,
                              const __nv_bfloat16* __restrict__ dO,
                              const float* __restrict__ rem, const float* __restrict__ drem, float* __restrict__ tot,
                              long long T, int H, long long o_stride_t, long long do_stride_t) {
  constexpr int LANES = DH / 8;
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
    uint4 l = make_uint4(0u, 0u, 0u, 0u);
    if (O_lo != nullptr) l = *reinterpret_cast<const uint4*>(O_lo + (t * H + h) * DH + sub * 8);
    const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
    const __nv_bfloat162* pl = reinterpret_cast<const __nv_bfloat162*>(&l);
    float lo_acc = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 x = __bfloat1622float2(pa[i]), y = __bfloat1622float2(pb[i]), z = __bfloat1622float2(pl[i]);
      acc += x.x * y.x + x.y * y.y;
      lo_acc += z.x * y.x + z.y * y.y;
    }
    acc += lo_acc;
  }
#pragma unroll
  for (int s = LANES / 2; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (live && sub == 0) {
    const long long i = (long long)h * T + t;
    tot[i] = acc - (drem ? drem[i] * (1.f - rem[i]) : 0.f);
  }
}

}  // namespace

extern "C" {

// dk_acc, dv_acc: fp32 [T, H, 64], zero on entry (reduced into with TMA adds); dq: bf16 [T, H, 64] (token stride given).
// tot: fp32 [H, T] scratch.  rem: fp32 [H, T] from the forward; drem may be null.  o_lo: the forward's second output
// (bf16 [T, H, 64], contiguous) or null.
int fb_sb_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* o_lo, const void* dout, const float* rem,
                   const float* drem, float* tot, void* dq, float* dk_acc, float* dv_acc, const int* cu_seqlens,
                   const int* tile_offsets, int nseq, int max_tiles, long long T, int H, long long q_stride_t,
                   long long k_stride_t, long long v_stride_t, long long o_stride_t, long long do_stride_t,
                   long long dq_stride_t, float scale, cudaStream_t stream) {
  if (T == 0) return 0;
  if ((q_stride_t % 8) || (k_stride_t % 8) || (v_stride_t % 8) || (o_stride_t % 8) || (do_stride_t % 8) || (dq_stride_t % 8))
    return -3;
  {
    const long long threads = T * H * (DH / 8);
    sb_tot_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)o_lo,
                                                                       (const __nv_bfloat16*)dout, rem, drem, tot, T, H,
                                                                       o_stride_t, do_stride_t);
    int rc = fb::launch_ok("sb_tot_kernel");
    if (rc) return rc;
  }
  CUtensorMap tmQ, tmK, tmV, tmdO, tmdK, tmdV;
  auto qkv_map = [&](CUtensorMap* m, const void* base, long long stride) {
    return fb::make_tmap_3d(m, base, 2, (uint64_t)T, (uint64_t)H, (uint64_t)DH, (uint64_t)stride, (uint64_t)DH, 128, 1, 64, true);
  };
  int rc = qkv_map(&tmQ, q, q_stride_t);
  if (!rc) rc = qkv_map(&tmK, k, k_stride_t);
  if (!rc) rc = qkv_map(&tmV, v, v_stride_t);
  if (!rc) rc = qkv_map(&tmdO, dout, do_stride_t);
  if (!rc) rc = fb::make_tmap_3d(&tmdK, dk_acc, 4, (uint64_t)T, (uint64_t)H, (uint64_t)DH, (uint64_t)H * DH, (uint64_t)DH, 128, 1, 32, true);
  if (!rc) rc = fb::make_tmap_3d(&tmdV, dv_acc, 4, (uint64_t)T, (uint64_t)H, (uint64_t)DH, (uint64_t)H * DH, (uint64_t)DH, 128, 1, 32, true);
  if (rc) return rc;
  SbBwdParams p;
  p.cu_seqlens = cu_seqlens;
  p.tile_offsets = tile_offsets;
  p.nseq = nseq;
  p.H = H;
  p.total_tokens = (int)T;
  p.scale = scale;
  p.scale_log2 = scale * kLog2e;
  p.tot = tot;
  p.drem = drem;
  p.dQ = (__nv_bfloat16*)dq;
  p.dq_stride_t = dq_stride_t;
  p.status = fb::status_ptr();
  static bool done = false;
  if (!done) {
    cudaError_t e = cudaFuncSetAttribute(sb_attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::TOTAL);
    if (e != cudaSuccess) return (int)e;
    done = true;
  }
  dim3 grid(max_tiles, H);
  sb_attn_bwd_kernel<<<grid, 192, Smem::TOTAL, stream>>>(tmQ, tmK, tmV, tmdO, tmdK, tmdV, p);
  return fb::launch_ok("sb_attn_bwd_kernel");
}

}  // extern "C"
