// bf16 GEMM for sm_100a: TMA -> shared memory -> tcgen05.mma with fp32 accumulators in TMEM.
//
//   C[M,N] = A[M,K] * B[N,K]^T        (both operands may be stored K-major or MN-major)
//
// One persistent CTA per SM.  Warp roles: warp 0 = TMA producer, warp 1 = MMA issuer (owns TMEM),
// warps 2..5 = epilogue (each reads its 32-lane quarter of the accumulator with tcgen05.ld).
// The accumulator is double buffered in TMEM (2 x BN columns), so the epilogue of tile i runs
// under the main loop of tile i+1.  Shared-memory operands use the 128-byte swizzle; a K-major
// tile is one TMA box, an MN-major tile is one box per 64 MN elements.
//
// Replaces the cuBLAS calls behind every nn.Linear of the reference (fla/modules/mlp.py:58-73,
// fla/layers/attn.py:73-82, fla/modules/fused_linear_cross_entropy.py:330-397).
#include "tc05.cuh"
#include "host_utils.cuh"

using namespace tc05;

namespace {

constexpr int BM = 128;
constexpr int BK = 64;

enum EpiMode : int {
  EPI_BF16 = 0,     // C(bf16)  = alpha * acc (+ bias)
  EPI_F32 = 1,      // C(fp32)  = alpha * acc
  EPI_F32_ACC = 2,  // C(fp32) += alpha * acc
};

struct GemmParams {
  int M, N, K;
  int tiles_m, tiles_n;
  int num_kb;       // K blocks in total
  int splits;       // split-K factor (units = tiles * splits)
  int kb_per_split;
  void* C;
  long long ldc;
  long long split_stride;  // elements between split partials (EPI_F32 with splits > 1)
  const __nv_bfloat16* bias;
  float alpha;
  int epi;
  int group_m;
  int* status;
};

template <int BN, int STAGES>
struct SmemLayout {
  static constexpr int A_BYTES = BM * BK * 2;  // 16 KB
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;  // barriers + alignment slack
};

__device__ __forceinline__ void unit_to_tile(const GemmParams& p, int unit, int& tm, int& tn, int& split) {
  int tile = unit / p.splits;
  split = unit - tile * p.splits;
  // grouped raster: GROUP_M tiles of M share each sweep over N so concurrently running CTAs reuse A and B in L2
  int per_group = p.group_m * p.tiles_n;
  int g = tile / per_group;
  int first_m = g * p.group_m;
  int gsz = min(p.tiles_m - first_m, p.group_m);
  int r = tile - g * per_group;
  tm = first_m + (r % gsz);
  tn = r / gsz;
}

template <int BN, int STAGES, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmParams p) {
  using L = SmemLayout<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = (uint64_t*)(smem + L::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = (uint32_t*)(tempty_bar + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int total_units = p.tiles_m * p.tiles_n * p.splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 4);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
        int tm, tn, split;
        unit_to_tile(p, unit, tm, tn, split);
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(p.num_kb, kb0 + p.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, abort_flag, ERR_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* sA = smem + stage * L::STAGE_BYTES;
          uint8_t* sB = sA + L::A_BYTES;
          mbar_expect_tx(&full_bar[stage], L::STAGE_BYTES);
          if (!A_MN) {
            tma_load_2d(sA, &tmA, &full_bar[stage], kb * BK, tm * BM);
          } else {
#pragma unroll
            for (int g = 0; g < BM / 64; ++g)
              tma_load_2d(sA + g * (64 * BK * 2), &tmA, &full_bar[stage], tm * BM + g * 64, kb * BK);
          }
          if (!B_MN) {
            tma_load_2d(sB, &tmB, &full_bar[stage], kb * BK, tn * BN);
          } else {
#pragma unroll
            for (int g = 0; g < BN / 64; ++g)
              tma_load_2d(sB + g * (64 * BK * 2), &tmB, &full_bar[stage], tn * BN + g * 64, kb * BK);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      constexpr uint32_t A_LBO = A_MN ? 64 * BK * 2 : 16;
      constexpr uint32_t B_LBO = B_MN ? 64 * BK * 2 : 16;
      constexpr uint32_t A_KSTEP = A_MN ? 16 * 128 : 32;  // bytes per UMMA_K = 16
      constexpr uint32_t B_KSTEP = B_MN ? 16 * 128 : 32;
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x, ++it) {
        int tm, tn, split;
        unit_to_tile(p, unit, tm, tn, split);
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(p.num_kb, kb0 + p.kb_per_split);
        const int acc = it & 1;
        if (!mbar_wait(&tempty_bar[acc], ((it >> 1) & 1) ^ 1, p.status, abort_flag, ERR_WAIT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, p.status, abort_flag, ERR_WAIT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + stage * L::STAGE_BYTES);
          const uint32_t sB = sA + L::A_BYTES;
          const uint64_t adesc = make_smem_desc(sA, A_LBO, 1024);
          const uint64_t bdesc = make_smem_desc(sB, B_LBO, 1024);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            mma_ss(d_tmem, desc_advance(adesc, k * A_KSTEP), desc_advance(bdesc, k * B_KSTEP), idesc,
                   (kb > kb0 || k > 0) ? 1u : 0u);
          }
          mma_commit(&empty_bar[stage]);  // stage reusable once these MMAs have read it
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) mma_commit(&tfull_bar[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter + 32)
    int it = 0;
    bool ok = true;
    for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x, ++it) {
      int tm, tn, split;
      unit_to_tile(p, unit, tm, tn, split);
      const int acc = it & 1;
      if (!mbar_wait_warp(&tfull_bar[acc], (it >> 1) & 1, p.status, abort_flag, ERR_WAIT_TMEM_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int row = tm * BM + quarter * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t t_row = tmem_base + acc * BN + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        const int col0 = tn * BN + c;
        if (col0 >= p.N) break;  // warp-uniform
        uint32_t r[32];
        tmem_ld_32x32(t_row + c, r);
        tmem_ld_wait();
        if (!row_ok) continue;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
        const bool full = (col0 + 32 <= p.N);
        if (p.epi == EPI_BF16) {
          if (p.bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) v[j] += __bfloat162float(p.bias[col0 + j]);
          }
          __nv_bfloat16* dst = (__nv_bfloat16*)p.C + (long long)row * p.ldc + col0;
          if (full && ((p.ldc & 7) == 0)) {
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
        } else {
          float* dst = (float*)p.C + (long long)split * p.split_stride + (long long)row * p.ldc + col0;
          const bool accumulate = (p.epi == EPI_F32_ACC);
          if (full && ((p.ldc & 3) == 0)) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              float4 q = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
              if (accumulate) {
                float4 o = *reinterpret_cast<float4*>(dst + j);
                q.x += o.x; q.y += o.y; q.z += o.z; q.w += o.w;
              }
              *reinterpret_cast<float4*>(dst + j) = q;
            }
          } else {
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) dst[j] = accumulate ? dst[j] + v[j] : v[j];
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
    }
  }

  // ------------------------------------------------------------------ tear-down
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

// Deterministic split-K reduction: out = sum_s partial[s] in a fixed order (optionally accumulated).
__global__ void splitk_reduce_kernel(const float* __restrict__ part, int splits, long long split_stride, long long n,
                                     void* out, int out_fp32, int accumulate) {
  long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= n) return;
  float4 s = *reinterpret_cast<const float4*>(part + i);
  for (int k = 1; k < splits; ++k) {
    float4 t = *reinterpret_cast<const float4*>(part + (long long)k * split_stride + i);
    s.x += t.x; s.y += t.y; s.z += t.z; s.w += t.w;
  }
  if (out_fp32) {
    float4* o = reinterpret_cast<float4*>((float*)out + i);
    if (accumulate) {
      float4 t = *o;
      s.x += t.x; s.y += t.y; s.z += t.z; s.w += t.w;
    }
    *o = s;
  } else {
    uint2 q;
    q.x = pack_bf16(s.x, s.y);
    q.y = pack_bf16(s.z, s.w);
    *reinterpret_cast<uint2*>((__nv_bfloat16*)out + i) = q;
  }
}

template <int BN, int STAGES, bool A_MN, bool B_MN>
int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int sm_count,
                cudaStream_t stream) {
  using L = SmemLayout<BN, STAGES>;
  auto kern = gemm_bf16_kernel<BN, STAGES, A_MN, B_MN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) {
      fprintf(stderr, "[flame_b200] gemm: cannot opt in to %d bytes of shared memory: %s\n", L::TOTAL,
              cudaGetErrorString(e));
      return (int)e;
    }
    configured = true;
  }
  int units = p.tiles_m * p.tiles_n * p.splits;
  int grid = units < sm_count ? units : sm_count;
  kern<<<grid, 192, L::TOTAL, stream>>>(tmA, tmB, p);
  return fb::launch_ok("gemm_bf16_kernel");
}

int sm_count_cached() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

}  // namespace

extern "C" {

// Bytes of fp32 workspace a split-K call needs (0 when splits <= 1).
long long fb_gemm_workspace_bytes(int M, int N, int splits) {
  return splits > 1 ? (long long)splits * M * N * 4 : 0;
}

// Chooses a split-K factor with a small cost model: waves of work units times K blocks per unit, plus the
// traffic of writing and re-reading the fp32 partials.  Few-tile, long-K GEMMs (weight gradients) gain most.
int fb_gemm_pick_splits(int M, int N, int K) {
  const long long tiles = (long long)((M + BM - 1) / BM) * ((N + 255) / 256);
  const int sms = sm_count_cached();
  const int num_kb = (K + BK - 1) / BK;
  if (tiles >= 2 * sms || num_kb < 16) return 1;
  const double t_kb = 0.30;                                    // microseconds per 128x256x64 block
  const double bytes_per_split = (double)M * N * 8.0;          // fp32 write + read
  double best = 1e30;
  int best_s = 1;
  for (int s = 1; s <= 16 && s * 4 <= num_kb; ++s) {
    const long long waves = (tiles * s + sms - 1) / sms;
    const int kb = (num_kb + s - 1) / s;
    double c = (double)waves * kb * t_kb + 2.0;
    if (s > 1) c += bytes_per_split * s / 5.0e6 + 3.0;         // 5 TB/s effective, plus a launch
    if (c < best * 0.97) {
      best = c;
      best_s = s;
    }
  }
  return best_s;
}

// C[M,N] = alpha * A[M,K] * B[N,K]^T (+ bias)
//  a_mn: 0 -> A stored [M, lda] (K contiguous); 1 -> A stored [K, lda] (M contiguous)
//  b_mn: 0 -> B stored [N, ldb] (K contiguous); 1 -> B stored [K, ldb] (N contiguous)
//  out_mode: 0 bf16 store, 1 fp32 store, 2 fp32 accumulate
//  splits > 1 needs `workspace` of fb_gemm_workspace_bytes(); the partial sums are reduced in a fixed order.
// Returns 0 on success.
int fb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                 long long ldc, int a_mn, int b_mn, int out_mode, float alpha, const void* bias, int splits,
                 void* workspace, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda & 7) || (ldb & 7) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15)) {
    fprintf(stderr, "[flame_b200] gemm: operands need 16-byte aligned bases and leading dimensions (lda=%lld ldb=%lld)\n",
            lda, ldb);
    return -2;
  }
  constexpr int BN = 256;
  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.tiles_m = (M + BM - 1) / BM;
  p.tiles_n = (N + BN - 1) / BN;
  p.num_kb = (K + BK - 1) / BK;
  if (splits < 1) splits = 1;
  if (splits > p.num_kb) splits = p.num_kb;
  p.kb_per_split = (p.num_kb + splits - 1) / splits;
  splits = (p.num_kb + p.kb_per_split - 1) / p.kb_per_split;
  p.splits = splits;
  p.bias = (const __nv_bfloat16*)bias;
  p.alpha = alpha;
  p.group_m = 16;
  p.status = fb::status_ptr();
  if (splits > 1) {
    if (workspace == nullptr) return -3;
    p.C = workspace;
    p.ldc = N;
    p.split_stride = (long long)M * N;
    p.epi = EPI_F32;
    p.alpha = alpha;
  } else {
    p.C = C;
    p.ldc = ldc;
    p.split_stride = 0;
    p.epi = out_mode;
  }
  CUtensorMap tmA, tmB;
  int rc;
  if (!a_mn) rc = fb::make_tmap_2d(&tmA, A, 2, M, K, lda, BM, BK, true);
  else       rc = fb::make_tmap_2d(&tmA, A, 2, K, M, lda, BK, 64, true);
  if (rc) return rc;
  if (!b_mn) rc = fb::make_tmap_2d(&tmB, B, 2, N, K, ldb, BN, BK, true);
  else       rc = fb::make_tmap_2d(&tmB, B, 2, K, N, ldb, BK, 64, true);
  if (rc) return rc;
  const int sms = sm_count_cached();
  constexpr int STAGES = 4;
  if (!a_mn && !b_mn)      rc = launch_gemm<BN, STAGES, false, false>(tmA, tmB, p, sms, stream);
  else if (!a_mn && b_mn)  rc = launch_gemm<BN, STAGES, false, true>(tmA, tmB, p, sms, stream);
  else if (a_mn && !b_mn)  rc = launch_gemm<BN, STAGES, true, false>(tmA, tmB, p, sms, stream);
  else                     rc = launch_gemm<BN, STAGES, true, true>(tmA, tmB, p, sms, stream);
  if (rc) return rc;
  if (splits > 1) {
    if (ldc != N) {
      fprintf(stderr, "[flame_b200] gemm: split-K needs a contiguous output (ldc == N)\n");
      return -4;
    }
    long long n = (long long)M * N;
    if (n & 3) return -5;
    int threads = 256;
    long long blocks = (n / 4 + threads - 1) / threads;
    splitk_reduce_kernel<<<(unsigned)blocks, threads, 0, stream>>>((const float*)workspace, splits, p.split_stride, n,
                                                                    C, out_mode != 0, out_mode == 2);
    rc = fb::launch_ok("splitk_reduce_kernel");
  }
  return rc;
}

}  // extern "C"
