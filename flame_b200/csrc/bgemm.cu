// Batched bf16 GEMM for the chunk-parallel token mixers (linear attention, delta rule, SSD):
//
//   C[b] = epilogue( alpha * A[b] * B[b]^T )      b = (hi, lo) = (chunk, head)
//
// Thousands of small problems (64 x 64 x dk score blocks, dk x dv chunk states, 64 x dv outputs) run as ONE persistent
// launch: every operand is a 4-D tensor map (inner, row, lo, hi), so a tile of any batch is a TMA box and the batch
// coordinates come from the work-unit index (optionally through an index table, which is how the chunk-by-chunk state
// recurrence of documents with different lengths addresses "chunk s of every document that has one").  The main loop is
// the single-CTA tcgen05 pipeline of gemm.cu (TMA warp, MMA warp, four epilogue warps, two TMEM accumulators); the
// epilogue adds what the chunk algorithms need so no elementwise pass follows the GEMM:
//   * causal masks (keep col <= row, or col < row),
//   * a decay factor exp(d[row] - d[col]) from a per-batch fp32 vector (scalar-gated attention scores),
//   * the state step   C = alpha * acc + gamma[b] * Cin[b'] + add16[b''] (+ C)   with a bf16 copy of the result written
//     to a batch of its own (C may be its own Cin: an fp32 state updated in place, small enough to stay in L2).
//
// Stands in for the tl.dot bodies of the reference's Triton chunk kernels (fla/ops/common/chunk_h.py,
// fla/ops/common/chunk_o.py, fla/ops/gated_delta_rule/wy_fast.py, fla/ops/common/chunk_scaled_dot_kkt.py).
#include <stdlib.h>

#include "tc05.cuh"
#include "host_utils.cuh"

using namespace tc05;

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int MAX_BN = 256;
// warp 0 TMA, warp 1 MMA, warps 2..9 epilogue: two warps per TMEM lane quarter, each taking half of the tile's columns.
// The chunk algorithms' problems mostly have 64 rows, which live in two lane quarters only; with one warp per quarter
// two warps would drain every accumulator and the epilogue, not memory, would set the pace.
constexpr int BGEMM_THREADS = 320;

struct BOperandIdx {
  const int* hi_index;  // optional: hi coordinate = hi_index[hi_raw]
  int hi_offset;        // added to the hi coordinate
  int lo_div;           // lo coordinate = lo / lo_div (grouped value heads)
};

struct BGemmParams {
  int M, N, K;
  int tiles_m, tiles_n, num_kb, bn;
  int n_lo, n_batch;
  BOperandIdx a, b, c, cin, c16i, add16i;
  void* C;
  long long ldc, c_stride_lo, c_stride_hi;
  const float* Cin;    // optional fp32 addend, same layout as C (may BE C: in-place state), scaled by gamma[hi(A) * n_lo + lo]
  const float* gamma;
  // bf16 side tensors of the fp32 modes, sharing one layout (ld16, stride_lo16, stride_hi16) but with hi coordinates of
  // their own: C16 receives a bf16 copy of the result, add16 is added to it
  __nv_bfloat16* C16;
  const __nv_bfloat16* add16;
  long long ld16, stride_lo16, stride_hi16;
  const float* decay;  // optional: value *= exp(decay[row] - decay[col]); element (hi, lo, r) at hi*d_hi + lo*d_lo + r*d_r
  long long d_hi, d_lo, d_r;
  float alpha;
  int out_mode;        // 0 bf16 store, 1 fp32 store, 2 fp32 accumulate
  int mask_mode;       // 0 none, 1 keep col <= row, 2 keep col < row
  int* status;
};

struct Smem {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = MAX_BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;
};

struct Unit {
  int hi_raw, lo, tm, tn;
};

__device__ __forceinline__ Unit decode(const BGemmParams& p, int unit) {
  Unit u;
  const int per_batch = p.tiles_m * p.tiles_n;
  const int batch = unit / per_batch;
  const int r = unit - batch * per_batch;
  u.tn = r / p.tiles_m;
  u.tm = r - u.tn * p.tiles_m;
  u.hi_raw = batch / p.n_lo;
  u.lo = batch - u.hi_raw * p.n_lo;
  return u;
}
__device__ __forceinline__ int hi_of(const BOperandIdx& o, int hi_raw) {
  return (o.hi_index != nullptr ? o.hi_index[hi_raw] : hi_raw) + o.hi_offset;
}

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(BGEMM_THREADS, 1)
bgemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, BGemmParams p) {
  using L = Smem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = (uint64_t*)(smem + L::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = (uint32_t*)(tempty_bar + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_units = p.n_batch * p.tiles_m * p.tiles_n;
  const int BN = p.bn;
  const uint32_t stage_tx = (uint32_t)(L::A_BYTES + BN * BK * 2);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], (blockDim.x >> 5) - 2);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * MAX_BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
        const Unit u = decode(p, unit);
        const int a_hi = hi_of(p.a, u.hi_raw), a_lo = u.lo / p.a.lo_div;
        const int b_hi = hi_of(p.b, u.hi_raw), b_lo = u.lo / p.b.lo_div;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, abort_flag, ERR_WAIT_EMPTY)) { ok = false; break; }
          uint8_t* sA = smem + stage * L::STAGE_BYTES;
          uint8_t* sB = sA + L::A_BYTES;
          mbar_expect_tx(&full_bar[stage], stage_tx);
          if (!A_MN) {
            tma_load_4d(sA, &tmA, &full_bar[stage], kb * BK, u.tm * BM, a_lo, a_hi);
          } else {
#pragma unroll
            for (int g = 0; g < BM / 64; ++g)
              tma_load_4d(sA + g * (64 * BK * 2), &tmA, &full_bar[stage], u.tm * BM + g * 64, kb * BK, a_lo, a_hi);
          }
          if (!B_MN) {
            tma_load_4d(sB, &tmB, &full_bar[stage], kb * BK, u.tn * BN, b_lo, b_hi);
          } else {
            for (int g = 0; g < BN / 64; ++g)
              tma_load_4d(sB + g * (64 * BK * 2), &tmB, &full_bar[stage], u.tn * BN + g * 64, kb * BK, b_lo, b_hi);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      constexpr uint32_t A_LBO = A_MN ? 64 * BK * 2 : 16;
      constexpr uint32_t B_LBO = B_MN ? 64 * BK * 2 : 16;
      constexpr uint32_t A_KSTEP = A_MN ? 16 * 128 : 32;
      constexpr uint32_t B_KSTEP = B_MN ? 16 * 128 : 32;
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x, ++it) {
        const int acc = it & 1;
        if (!mbar_wait(&tempty_bar[acc], ((it >> 1) & 1) ^ 1, p.status, abort_flag, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * MAX_BN;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, p.status, abort_flag, ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + stage * L::STAGE_BYTES);
          const uint32_t sB = sA + L::A_BYTES;
          const uint64_t adesc = make_smem_desc(sA, A_LBO, 1024);
          const uint64_t bdesc = make_smem_desc(sB, B_LBO, 1024);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            mma_ss(d_tmem, desc_advance(adesc, k * A_KSTEP), desc_advance(bdesc, k * B_KSTEP), idesc,
                   (kb > 0 || k > 0) ? 1u : 0u);
          mma_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) mma_commit(&tfull_bar[acc]);
      }
    }
  } else {
    const int quarter = warp & 3;
    // eight epilogue warps: two per lane quarter, each takes half of the tile's columns (tiles are 64..256 wide);
    // four: one per quarter takes them all
    const bool split = blockDim.x == BGEMM_THREADS;
    const int half = (warp - 2) >> 2;
    const int c_begin = split ? half * (BN / 2) : 0;
    const int c_end = split ? c_begin + BN / 2 : BN;
    int it = 0;
    bool ok = true;
    for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x, ++it) {
      const Unit u = decode(p, unit);
      const int acc = it & 1;
      if (!mbar_wait_warp(&tfull_bar[acc], (it >> 1) & 1, p.status, abort_flag, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int row = u.tm * BM + quarter * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t t_row = tmem_base + acc * MAX_BN + ((uint32_t)(quarter * 32) << 16);
      const long long c_base = (long long)hi_of(p.c, u.hi_raw) * p.c_stride_hi + (long long)(u.lo / p.c.lo_div) * p.c_stride_lo +
                               (long long)row * p.ldc;
      const float* cin_row = nullptr;
      float gamma = 0.f;
      if (p.Cin != nullptr) {
        cin_row = p.Cin + (long long)hi_of(p.cin, u.hi_raw) * p.c_stride_hi + (long long)(u.lo / p.cin.lo_div) * p.c_stride_lo +
                  (long long)row * p.ldc;
        gamma = p.gamma != nullptr ? p.gamma[(long long)hi_of(p.a, u.hi_raw) * p.n_lo + u.lo] : 1.f;
      }
      const long long lo16 = (long long)(u.lo / p.c.lo_div) * p.stride_lo16 + (long long)row * p.ld16;
      __nv_bfloat16* c16_row = p.C16 != nullptr ? p.C16 + (long long)hi_of(p.c16i, u.hi_raw) * p.stride_hi16 + lo16 : nullptr;
      const __nv_bfloat16* add_row = p.add16 != nullptr ? p.add16 + (long long)hi_of(p.add16i, u.hi_raw) * p.stride_hi16 + lo16 : nullptr;
      const float* dec = nullptr;
      float dec_row = 0.f;
      if (p.decay != nullptr) {
        dec = p.decay + (long long)u.hi_raw * p.d_hi + (long long)u.lo * p.d_lo;
        if (row_ok) dec_row = dec[(long long)row * p.d_r];
      }
#pragma unroll 1
      for (int c = c_begin; c < c_end; c += 32) {
        const int col0 = u.tn * BN + c;
        if (col0 >= p.N) break;  // warp-uniform
        uint32_t r[32];
        tmem_ld_32x32(t_row + c, r);
        const bool full = (col0 + 32 <= p.N);
        const bool vec = full && row_ok && p.out_mode != 0;
        // every global read of this piece is issued before any store, so the loads overlap (one round trip per piece)
        float4 o_acc[8], o_cin[8];
        uint4 o_add[4];
        if (vec) {
          const float* dst = (const float*)p.C + c_base + col0;
          if (p.out_mode == 2) {
#pragma unroll
            for (int j = 0; j < 8; ++j) o_acc[j] = *reinterpret_cast<const float4*>(dst + 4 * j);
          }
          if (cin_row != nullptr) {
#pragma unroll
            for (int j = 0; j < 8; ++j) o_cin[j] = *reinterpret_cast<const float4*>(cin_row + col0 + 4 * j);
          }
          if (add_row != nullptr) {
#pragma unroll
            for (int j = 0; j < 4; ++j) o_add[j] = *reinterpret_cast<const uint4*>(add_row + col0 + 8 * j);
          }
        }
        tmem_ld_wait();
        if (!row_ok) continue;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
        if (dec != nullptr) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int col = col0 + j;
            // masked entries may have a positive exponent: they are dropped, never multiplied
            const bool keep = col < p.N && (p.mask_mode == 0 || (p.mask_mode == 1 ? col <= row : col < row));
            v[j] = keep ? v[j] * __expf(dec_row - dec[(long long)col * p.d_r]) : 0.f;
          }
        } else if (p.mask_mode != 0) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int col = col0 + j;
            if (!(p.mask_mode == 1 ? col <= row : col < row)) v[j] = 0.f;
          }
        }
        if (p.out_mode == 0) {
          __nv_bfloat16* dst = (__nv_bfloat16*)p.C + c_base + col0;
          if (add_row != nullptr) {  // bf16 result with a bf16 addend (v_new = u - w S, o = q S + A v)
            if (full) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const uint4 a4 = *reinterpret_cast<const uint4*>(add_row + col0 + 8 * j);
                const uint32_t w4[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                  v[8 * j + 2 * t] += __uint_as_float(w4[t] << 16);
                  v[8 * j + 2 * t + 1] += __uint_as_float(w4[t] & 0xffff0000u);
                }
              }
            } else {
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) v[j] += __bfloat162float(add_row[col0 + j]);
            }
          }
          if (full) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint4 q;
              q.x = pack_bf16(v[j], v[j + 1]);
              q.y = pack_bf16(v[j + 2], v[j + 3]);
              q.z = pack_bf16(v[j + 4], v[j + 5]);
              q.w = pack_bf16(v[j + 6], v[j + 7]);
              *reinterpret_cast<uint4*>(dst + j) = q;
            }
          } else {
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) dst[j] = __float2bfloat16(v[j]);
          }
        } else if (vec) {
          float* dst = (float*)p.C + c_base + col0;
          if (p.out_mode == 2) {
#pragma unroll
            for (int j = 0; j < 8; ++j) { v[4 * j] += o_acc[j].x; v[4 * j + 1] += o_acc[j].y; v[4 * j + 2] += o_acc[j].z; v[4 * j + 3] += o_acc[j].w; }
          }
          if (cin_row != nullptr) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              v[4 * j] = fmaf(gamma, o_cin[j].x, v[4 * j]); v[4 * j + 1] = fmaf(gamma, o_cin[j].y, v[4 * j + 1]);
              v[4 * j + 2] = fmaf(gamma, o_cin[j].z, v[4 * j + 2]); v[4 * j + 3] = fmaf(gamma, o_cin[j].w, v[4 * j + 3]);
            }
          }
          if (add_row != nullptr) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t w4[4] = {o_add[j].x, o_add[j].y, o_add[j].z, o_add[j].w};
#pragma unroll
              for (int t = 0; t < 4; ++t) {
                v[8 * j + 2 * t] += __uint_as_float(w4[t] << 16);
                v[8 * j + 2 * t + 1] += __uint_as_float(w4[t] & 0xffff0000u);
              }
            }
          }
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<float4*>(dst + 4 * j) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          if (c16_row != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint4 q;
              q.x = pack_bf16(v[j], v[j + 1]);
              q.y = pack_bf16(v[j + 2], v[j + 3]);
              q.z = pack_bf16(v[j + 4], v[j + 5]);
              q.w = pack_bf16(v[j + 6], v[j + 7]);
              *reinterpret_cast<uint4*>(c16_row + col0 + j) = q;
            }
          }
        } else {
          float* dst = (float*)p.C + c_base + col0;
          for (int j = 0; j < 32; ++j) {
            if (col0 + j >= p.N) continue;
            float x = v[j];
            if (p.out_mode == 2) x += dst[j];
            if (cin_row != nullptr) x += gamma * cin_row[col0 + j];
            if (add_row != nullptr) x += __bfloat162float(add_row[col0 + j]);
            dst[j] = x;
            if (c16_row != nullptr) c16_row[col0 + j] = __float2bfloat16(x);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * MAX_BN);
  }
}

template <bool A_MN, bool B_MN>
int launch_b(const CUtensorMap& tmA, const CUtensorMap& tmB, const BGemmParams& p, cudaStream_t stream) {
  auto kern = bgemm_bf16_kernel<A_MN, B_MN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  const long long units = (long long)p.n_batch * p.tiles_m * p.tiles_n;
  const int grid = (int)(units < sms ? units : sms);
  static const int threads = []() {
    const char* e = getenv("FLAME_B200_BGEMM_EPI_WARPS");  // 4: one epilogue warp per TMEM lane quarter
    return (e && e[0] == '4') ? 192 : BGEMM_THREADS;
  }();
  kern<<<grid, threads, Smem::TOTAL, stream>>>(tmA, tmB, p);
  return fb::launch_ok("bgemm_bf16_kernel");
}

}  // namespace

extern "C" {

// Operand of a batched GEMM: a [rows, inner] bf16 matrix per batch (hi, lo) at ptr + hi*stride_hi + lo*stride_lo, `ld`
// elements between rows, inner contiguous.  `mn` = 0: rows are the M (or N) dimension and inner is K; `mn` = 1: rows are K
// and inner is the M (or N) dimension.  n_hi / n_lo are the EXTENTS of the storage (coordinates may come from an index).
struct FbBOperand {
  const void* ptr;
  long long ld, stride_lo, stride_hi;
  int n_lo, n_hi;
  int mn;
  int lo_div;
  int hi_offset;
  const int* hi_index;
};

struct FbBEpilogue {
  void* C;             // [.., M, N] bf16 (out_mode 0) or fp32 (1 store, 2 accumulate)
  long long ldc, stride_lo, stride_hi;
  int c_lo_div, c_hi_offset;
  const int* c_hi_index;
  const float* Cin;    // optional fp32 addend (layout of C; may be C itself), scaled by gamma[hi coordinate of A * n_lo_batch + lo] (null = 1)
  int cin_hi_offset;
  const int* cin_hi_index;
  const float* gamma;
  void* C16;           // optional bf16 copy of the result (fp32 modes), own hi coordinate
  int c16_hi_offset;
  const int* c16_hi_index;
  const void* add16;   // optional bf16 addend (fp32 modes), own hi coordinate; shares the layout below with C16
  int add16_hi_offset;
  const int* add16_hi_index;
  long long ld16, stride_lo16, stride_hi16;
  const float* decay;  // optional fp32 vector per batch, see bgemm.cu header
  long long d_hi, d_lo, d_r;
  float alpha;
  int out_mode, mask_mode;
};

// n_hi_batch x n_lo_batch problems of size M x N x K.  Returns 0 on success.
int fb_bgemm_bf16(const FbBOperand* a, const FbBOperand* b, const FbBEpilogue* e, int n_hi_batch, int n_lo_batch, int M,
                  int N, int K, cudaStream_t stream) {
  if (n_hi_batch <= 0 || n_lo_batch <= 0 || M <= 0 || N <= 0 || K <= 0) return 0;
  if ((a->ld & 7) || (b->ld & 7) || (a->stride_lo & 7) || (b->stride_lo & 7) || (a->stride_hi & 7) || (b->stride_hi & 7) ||
      ((uintptr_t)a->ptr & 15) || ((uintptr_t)b->ptr & 15)) {
    fprintf(stderr, "[flame_b200] bgemm: operand bases and strides must be multiples of 16 bytes\n");
    return -2;
  }
  if ((e->ldc & 7) || (e->stride_lo & 7) || (e->stride_hi & 7) || ((uintptr_t)e->C & 15)) {
    fprintf(stderr, "[flame_b200] bgemm: output base and strides must be multiples of 8 elements\n");
    return -2;
  }
  BGemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.bn = N <= 64 ? 64 : (N <= 128 ? 128 : 256);
  p.tiles_m = (M + BM - 1) / BM;
  p.tiles_n = (N + p.bn - 1) / p.bn;
  p.num_kb = (K + BK - 1) / BK;
  p.n_lo = n_lo_batch;
  p.n_batch = n_hi_batch * n_lo_batch;
  p.a = {a->hi_index, a->hi_offset, a->lo_div > 0 ? a->lo_div : 1};
  p.b = {b->hi_index, b->hi_offset, b->lo_div > 0 ? b->lo_div : 1};
  p.c = {e->c_hi_index, e->c_hi_offset, e->c_lo_div > 0 ? e->c_lo_div : 1};
  p.cin = {e->cin_hi_index, e->cin_hi_offset, p.c.lo_div};
  p.C = e->C; p.ldc = e->ldc; p.c_stride_lo = e->stride_lo; p.c_stride_hi = e->stride_hi;
  p.c16i = {e->c16_hi_index, e->c16_hi_offset, p.c.lo_div};
  p.add16i = {e->add16_hi_index, e->add16_hi_offset, p.c.lo_div};
  p.C16 = (__nv_bfloat16*)e->C16;
  p.add16 = (const __nv_bfloat16*)e->add16;
  p.ld16 = e->ld16; p.stride_lo16 = e->stride_lo16; p.stride_hi16 = e->stride_hi16;
  p.Cin = e->Cin; p.gamma = e->gamma;
  p.decay = e->decay; p.d_hi = e->d_hi; p.d_lo = e->d_lo; p.d_r = e->d_r;
  p.alpha = e->alpha; p.out_mode = e->out_mode; p.mask_mode = e->mask_mode;
  p.status = fb::status_ptr();
  if ((p.C16 != nullptr || p.Cin != nullptr) && p.out_mode == 0) return -3;
  if ((p.C16 != nullptr || p.add16 != nullptr) && ((p.ld16 & 7) || (p.stride_lo16 & 7) || (p.stride_hi16 & 7))) return -2;
  CUtensorMap tmA, tmB;
  int rc;
  // dims: (inner, rows, lo, hi)
  if (!a->mn) rc = fb::make_tmap_4d(&tmA, a->ptr, 2, a->n_hi, a->n_lo, M, K, a->stride_hi, a->stride_lo, a->ld, BM, BK, true);
  else        rc = fb::make_tmap_4d(&tmA, a->ptr, 2, a->n_hi, a->n_lo, K, M, a->stride_hi, a->stride_lo, a->ld, BK, 64, true);
  if (rc) return rc;
  if (!b->mn) rc = fb::make_tmap_4d(&tmB, b->ptr, 2, b->n_hi, b->n_lo, N, K, b->stride_hi, b->stride_lo, b->ld, p.bn, BK, true);
  else        rc = fb::make_tmap_4d(&tmB, b->ptr, 2, b->n_hi, b->n_lo, K, N, b->stride_hi, b->stride_lo, b->ld, BK, 64, true);
  if (rc) return rc;
  if (!a->mn && !b->mn) return launch_b<false, false>(tmA, tmB, p, stream);
  if (!a->mn && b->mn)  return launch_b<false, true>(tmA, tmB, p, stream);
  if (a->mn && !b->mn)  return launch_b<true, false>(tmA, tmB, p, stream);
  return launch_b<true, true>(tmA, tmB, p, stream);
}

}  // extern "C"
