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
#include <cstdlib>
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
  // --- fused collective modes (tensor parallelism over NVLink peer memory) ---
  // gather: the first g_ncopy CTAs copy every rank's [rows_per_rank, K] activation shard into the local full
  //   matrix A (g_dst) chunk by chunk and publish a flag per chunk; GEMM producers wait for the chunk they need.
  // scatter: the epilogue stores each output row into the buffer of the rank that owns the row (reduce-scatter by
  //   "everyone writes its partial into slot [my rank] of the owner"); a follow-up kernel sums the slots.
  int m_rot;            // tile rows are visited starting at this M tile (local shard first / remote shards first)
  int g_ncopy;          // > 0 enables gather mode
  int g_world, g_rank, g_rows_per_rank, g_chunk_rows, g_epoch;
  unsigned long long g_wait_ns;  // limit of the waits on flags another GPU raises
  long long g_ld;       // leading dimension of the shards and of g_dst (elements)
  const void* g_src[16];
  __nv_bfloat16* g_dst;
  int* g_flags;         // local: one word per chunk of the full matrix
  const int* g_ready;   // local: ready[src rank] >= epoch once that rank's shard may be read
  int s_world;          // > 0 enables scatter mode (bf16 output only)
  int s_rank, s_rows_per_rank;
  void* s_dst[16];      // per owner rank: base of its [world][rows_per_rank, ldc] receive buffer
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
  if (p.m_rot) {
    tm += p.m_rot;
    if (tm >= p.tiles_m) tm -= p.tiles_m;
  }
}

__device__ __forceinline__ int ld_acquire_gpu(const int* addr) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
__device__ __forceinline__ int ld_acquire_sys(const int* addr) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(int* addr, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
// bounded spin on a flag word; false (and the status word set) when the limit passes
template <bool SYS>
__device__ __forceinline__ bool wait_flag(const int* addr, int value, int* status, unsigned long long limit_ns) {
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while ((SYS ? ld_acquire_sys(addr) : ld_acquire_gpu(addr)) < value) {
    if ((++spins & 0xFF) == 0 && globaltimer_ns() - t0 > limit_ns) {
      report(status, ERR_WAIT_PEER);
      return false;
    }
    __nanosleep(32);
  }
  return true;
}

// Copy role of the gather mode: shard chunks are fetched in ring order starting with the local shard.
__device__ void gather_copy_role(const GemmParams& p) {
  const int cpr = p.g_rows_per_rank / p.g_chunk_rows;  // chunks per rank
  const int total = cpr * p.g_world;
  const int vec_per_row = p.K >> 3;
  __shared__ int s_ok;
  for (int c = blockIdx.x; c < total; c += p.g_ncopy) {
    const int src = (p.g_rank + c / cpr) % p.g_world;
    const int cc = c % cpr;
    if (threadIdx.x == 0) s_ok = (src == p.g_rank) ? 1 : (wait_flag<true>(p.g_ready + src, p.g_epoch, p.status, p.g_wait_ns) ? 1 : 0);
    __syncthreads();
    const bool ok = s_ok != 0;
    const long long src_row0 = (long long)cc * p.g_chunk_rows;
    const long long dst_row0 = (long long)src * p.g_rows_per_rank + src_row0;
    if (ok) {
      const uint4* sp = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.g_src[src]) + src_row0 * p.g_ld);
      uint4* dp = reinterpret_cast<uint4*>(p.g_dst + dst_row0 * p.g_ld);
      const long long ld_vec = p.g_ld >> 3;
      const long long n = (long long)p.g_chunk_rows * vec_per_row;
      // sixteen independent 16-byte loads per thread are in flight before the first store: a peer load takes a few
      // microseconds over NVLink, so the copy rate is (bytes in flight) / latency
      constexpr int U = 16;
      for (long long i0 = threadIdx.x; i0 < n; i0 += (long long)blockDim.x * U) {
        uint4 q[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i = i0 + (long long)u * blockDim.x;
          if (i < n) {
            const long long r = i / vec_per_row, v = i - r * vec_per_row;
            const uint4* a = sp + r * ld_vec + v;
            asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(q[u].x), "=r"(q[u].y), "=r"(q[u].z), "=r"(q[u].w)
                         : "l"(a)
                         : "memory");
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i = i0 + (long long)u * blockDim.x;
          if (i < n) {
            const long long r = i / vec_per_row, v = i - r * vec_per_row;
            dp[r * ld_vec + v] = q[u];
          }
        }
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      st_release_gpu(p.g_flags + dst_row0 / p.g_chunk_rows, p.g_epoch);  // published even after a time-out: nobody hangs
    }
  }
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

  if (p.g_ncopy > 0 && (int)blockIdx.x < p.g_ncopy) {
    gather_copy_role(p);
    return;
  }
  const int bid = (int)blockIdx.x - p.g_ncopy;
  const int nctas = (int)gridDim.x - p.g_ncopy;
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
      for (int unit = bid; unit < total_units && ok; unit += nctas) {
        int tm, tn, split;
        unit_to_tile(p, unit, tm, tn, split);
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(p.num_kb, kb0 + p.kb_per_split);
        if (p.g_ncopy > 0) {
          // rows of this tile come from one gathered chunk: wait until the copy CTAs published it, then order the
          // generic-proxy writes before the TMA reads of the async proxy
          if (!wait_flag<false>(p.g_flags + (tm * BM) / p.g_chunk_rows, p.g_epoch, p.status, p.g_wait_ns + kWaitLimitNs)) *abort_flag = 1;
          asm volatile("fence.proxy.async.global;" ::: "memory");
        }
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
      for (int unit = bid; unit < total_units && ok; unit += nctas, ++it) {
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
    for (int unit = bid; unit < total_units && ok; unit += nctas, ++it) {
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
          if (p.s_world > 0) {
            const int owner = row / p.s_rows_per_rank;
            const long long lrow = (long long)p.s_rank * p.s_rows_per_rank + (row - owner * p.s_rows_per_rank);
            dst = (__nv_bfloat16*)p.s_dst[owner] + lrow * p.ldc + col0;
          }
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
  // the copy CTAs of the gather mode occupy SMs of their own; the persistent GEMM CTAs share the rest
  const int gemm_ctas = sm_count - p.g_ncopy;
  int grid = (units < gemm_ctas ? units : gemm_ctas) + p.g_ncopy;
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

// 1: one CTA per 128x256 tile; 2: CTA pairs on 256x256 tiles (gemm2.cu, the default: 10-19 % faster on the shapes of a
// training step).  FLAME_B200_GEMM_VARIANT=1 in the environment selects the single-CTA kernel.
int initial_variant() {
  const char* e = getenv("FLAME_B200_GEMM_VARIANT");
  return (e != nullptr && e[0] == '1') ? 1 : 2;
}
int g_variant = initial_variant();

}  // namespace

extern "C" int fb_gemm2_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                             long long ldc, int a_mn, int b_mn, int out_mode, float alpha, int splits, void* workspace,
                             int sm_count, cudaStream_t stream);

extern "C" int fb_gemm2_allgather_a(const unsigned long long* shard_ptrs, int world, int rank, int rows_per_rank, long long ld,
                                    void* a_full, int* chunk_flags, const int* ready, int epoch, const void* B, void* C, int N,
                                    int K, long long ldb, long long ldc, int b_mn, int sm_count, cudaStream_t stream);
extern "C" int fb_gemm2_scatter_rows(const void* A, const void* B, const unsigned long long* recv_ptrs, int world, int rank,
                                     int rows_per_rank, int N, int K, long long lda, long long ldb, long long ldc, int b_mn,
                                     int sm_count, cudaStream_t stream);

extern "C" {

// Selects the kernel behind fb_gemm_bf16 for calls without bias: 1 = single-CTA tiles, 2 = CTA pairs.  Returns the old value.
int fb_gemm_set_variant(int v) {
  int old = g_variant;
  if (v == 1 || v == 2) g_variant = v;
  return old;
}

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
  p.m_rot = 0;
  p.g_ncopy = 0;
  p.s_world = 0;
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
  const int sms = sm_count_cached();
  int rc;
  if (g_variant == 2 && bias == nullptr) {
    rc = fb_gemm2_bf16(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, out_mode, alpha, splits, workspace, sms, stream);
  } else {
    CUtensorMap tmA, tmB;
    if (!a_mn) rc = fb::make_tmap_2d(&tmA, A, 2, M, K, lda, BM, BK, true);
    else       rc = fb::make_tmap_2d(&tmA, A, 2, K, M, lda, BK, 64, true);
    if (rc) return rc;
    if (!b_mn) rc = fb::make_tmap_2d(&tmB, B, 2, N, K, ldb, BN, BK, true);
    else       rc = fb::make_tmap_2d(&tmB, B, 2, K, N, ldb, BK, 64, true);
    if (rc) return rc;
    constexpr int STAGES = 4;
    if (!a_mn && !b_mn)      rc = launch_gemm<BN, STAGES, false, false>(tmA, tmB, p, sms, stream);
    else if (!a_mn && b_mn)  rc = launch_gemm<BN, STAGES, false, true>(tmA, tmB, p, sms, stream);
    else if (a_mn && !b_mn)  rc = launch_gemm<BN, STAGES, true, false>(tmA, tmB, p, sms, stream);
    else                     rc = launch_gemm<BN, STAGES, true, true>(tmA, tmB, p, sms, stream);
  }
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


// C[M,N] = allgather_rows(A_shards)[M,K] * B[N,K]^T in ONE kernel.  Every rank holds a [rows_per_rank, K] shard (peer
// pointers in `shard_ptrs`, leading dimension ld); M = world * rows_per_rank.  `a_full` ([M, ld], local) receives the
// gathered matrix (kept for the weight-gradient GEMM of the backward pass); `chunk_flags` (local, M / chunk_rows ints) and
// `ready` (local, written by the peers: ready[r] >= epoch when rank r's shard is final) carry the hand-off; `epoch` must
// grow from call to call on the same flag arrays.  b_mn selects the storage of B as in fb_gemm_bf16.
int fb_gemm_allgather_a(const unsigned long long* shard_ptrs, int world, int rank, int rows_per_rank, long long ld,
                        void* a_full, int* chunk_flags, const int* ready, int epoch, const void* B, void* C, int N, int K,
                        long long ldb, long long ldc, int b_mn, cudaStream_t stream) {
  constexpr int BN = 256;
  const int M = world * rows_per_rank;
  if (g_variant == 2 && (M % 256) == 0 && world <= 16 && (rows_per_rank % BM) == 0)
    return fb_gemm2_allgather_a(shard_ptrs, world, rank, rows_per_rank, ld, a_full, chunk_flags, ready, epoch, B, C, N, K, ldb,
                                ldc, b_mn, sm_count_cached(), stream);
  if (world > 16 || (rows_per_rank % BM) || (ld & 7) || (ldb & 7) || (K & 7)) {
    fprintf(stderr, "[flame_b200] gemm_allgather_a: rows per rank must be a multiple of %d and K, ld, ldb multiples of 8\n", BM);
    return -2;
  }
  int chunk_rows = 1024;
  while (rows_per_rank % chunk_rows) chunk_rows >>= 1;  // >= 128 because rows_per_rank % 128 == 0
  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.tiles_m = M / BM;
  p.tiles_n = (N + BN - 1) / BN;
  p.num_kb = (K + BK - 1) / BK;
  p.splits = 1;
  p.kb_per_split = p.num_kb;
  p.C = C; p.ldc = ldc; p.split_stride = 0;
  p.bias = nullptr; p.alpha = 1.f; p.epi = EPI_BF16;
  p.group_m = 16;
  p.status = fb::status_ptr();
  p.m_rot = rank * (rows_per_rank / BM);  // local shard first, then the ring
  p.g_ncopy = 16;
  p.g_world = world; p.g_rank = rank; p.g_rows_per_rank = rows_per_rank; p.g_chunk_rows = chunk_rows; p.g_epoch = epoch;
  p.g_wait_ns = fb::peer_wait_ns();
  p.g_ld = ld;
  for (int r = 0; r < 16; ++r) p.g_src[r] = r < world ? (const void*)shard_ptrs[r] : nullptr;
  p.g_dst = (__nv_bfloat16*)a_full;
  p.g_flags = chunk_flags;
  p.g_ready = ready;
  p.s_world = 0;
  CUtensorMap tmA, tmB;
  int rc = fb::make_tmap_2d(&tmA, a_full, 2, M, K, ld, BM, BK, true);
  if (rc) return rc;
  if (!b_mn) rc = fb::make_tmap_2d(&tmB, B, 2, N, K, ldb, BN, BK, true);
  else       rc = fb::make_tmap_2d(&tmB, B, 2, K, N, ldb, BK, 64, true);
  if (rc) return rc;
  const int sms = sm_count_cached();
  if (!b_mn) return launch_gemm<BN, 4, false, false>(tmA, tmB, p, sms, stream);
  return launch_gemm<BN, 4, false, true>(tmA, tmB, p, sms, stream);
}

// Partial product for a reduce-scatter over rows: computes A[M,K] * B[N,K]^T and stores row m into slot `rank` of the
// receive buffer of the rank that owns row m (recv_ptrs[owner] points at [world][rows_per_rank, ldc] bf16).  Remote
// rows are produced first so their NVLink traffic overlaps the remaining tiles.  Sum the slots with fb_sum_slots once
// every rank has signalled completion.
int fb_gemm_scatter_rows(const void* A, const void* B, const unsigned long long* recv_ptrs, int world, int rank,
                         int rows_per_rank, int N, int K, long long lda, long long ldb, long long ldc, int b_mn,
                         cudaStream_t stream) {
  constexpr int BN = 256;
  const int M = world * rows_per_rank;
  if (g_variant == 2 && (M % 256) == 0 && world <= 16 && (rows_per_rank % BM) == 0)
    return fb_gemm2_scatter_rows(A, B, recv_ptrs, world, rank, rows_per_rank, N, K, lda, ldb, ldc, b_mn, sm_count_cached(),
                                 stream);
  if (world > 16 || (rows_per_rank % BM) || (lda & 7) || (ldb & 7) || (ldc & 7)) return -2;
  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.tiles_m = M / BM;
  p.tiles_n = (N + BN - 1) / BN;
  p.num_kb = (K + BK - 1) / BK;
  p.splits = 1;
  p.kb_per_split = p.num_kb;
  p.C = nullptr; p.ldc = ldc; p.split_stride = 0;
  p.bias = nullptr; p.alpha = 1.f; p.epi = EPI_BF16;
  p.group_m = 16;
  p.status = fb::status_ptr();
  p.m_rot = ((rank + 1) % world) * (rows_per_rank / BM);  // next rank's rows first, own rows last
  p.g_ncopy = 0;
  p.s_world = world; p.s_rank = rank; p.s_rows_per_rank = rows_per_rank;
  for (int r = 0; r < 16; ++r) p.s_dst[r] = r < world ? (void*)recv_ptrs[r] : nullptr;
  CUtensorMap tmA, tmB;
  int rc = fb::make_tmap_2d(&tmA, A, 2, M, K, lda, BM, BK, true);
  if (rc) return rc;
  if (!b_mn) rc = fb::make_tmap_2d(&tmB, B, 2, N, K, ldb, BN, BK, true);
  else       rc = fb::make_tmap_2d(&tmB, B, 2, K, N, ldb, BK, 64, true);
  if (rc) return rc;
  const int sms = sm_count_cached();
  if (!b_mn) return launch_gemm<BN, 4, false, false>(tmA, tmB, p, sms, stream);
  return launch_gemm<BN, 4, false, true>(tmA, tmB, p, sms, stream);
}

// out[n] (bf16) = sum over `world` slots (fixed order, fp32) of slots[s * slot_stride + i]; optional residual addend.
int fb_sum_slots(const void* slots, int world, long long slot_stride, long long n, void* out, cudaStream_t stream);

}  // extern "C"

namespace {
__global__ void sum_slots_kernel(const __nv_bfloat16* __restrict__ slots, int world, long long slot_stride, long long n,
                                 __nv_bfloat16* __restrict__ out) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i >= n) return;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int s = 0; s < world; ++s) {
    const uint4 q = *reinterpret_cast<const uint4*>(slots + (long long)s * slot_stride + i);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 t = __bfloat1622float2(h[j]);
      acc[2 * j] += t.x;
      acc[2 * j + 1] += t.y;
    }
  }
  uint4 o;
  o.x = pack_bf16(acc[0], acc[1]);
  o.y = pack_bf16(acc[2], acc[3]);
  o.z = pack_bf16(acc[4], acc[5]);
  o.w = pack_bf16(acc[6], acc[7]);
  *reinterpret_cast<uint4*>(out + i) = o;
}
}  // namespace

extern "C" int fb_sum_slots(const void* slots, int world, long long slot_stride, long long n, void* out,
                            cudaStream_t stream) {
  if (n == 0) return 0;
  if (n & 7) return -2;
  sum_slots_kernel<<<(unsigned)((n / 8 + 255) / 256), 256, 0, stream>>>((const __nv_bfloat16*)slots, world, slot_stride, n,
                                                                      (__nv_bfloat16*)out);
  return fb::launch_ok("sum_slots_kernel");
}
