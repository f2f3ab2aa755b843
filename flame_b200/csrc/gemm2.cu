// bf16 GEMM on CTA pairs (tcgen05 cta_group::2): C[M,N] = A[M,K] * B[N,K]^T with 256 x 256 output tiles.
//
// Two CTAs of a cluster share one tile: each loads its own 128 rows of A and ONE HALF (128 of the 256 N rows) of the
// B tile; the leader CTA issues a single M=256 MMA that reads both shared memories and writes 128 accumulator rows
// into each CTA's TMEM.  Compared with the single-CTA kernel (gemm.cu) every SM pulls one third fewer operand bytes
// per FLOP from L2 (64 instead of 96 bytes per clock at full tensor rate), and the freed shared memory deepens the
// TMA pipeline from four to six stages - both matter because the single-CTA kernel is L2-latency/bandwidth limited.
// Every TMA load is a plain per-CTA copy: the two B halves are different data.
//
// Barrier protocol (all waits bounded):
//   full[s]   leader CTA, 2 arrivals (one expect_tx per CTA's producer) + the bytes of both CTAs' TMA loads
//   empty[s]  each CTA, released by the leader's tcgen05.commit (one commit per CTA of the pair)
//   tfull[a]  each CTA, accumulator a complete (same two commits); tempty[a] leader, 8 arrivals (4 epilogue warps x 2)
#include "tc05.cuh"
#include "host_utils.cuh"

using namespace tc05;

namespace {

constexpr int BMH = 128;   // rows per CTA
constexpr int BM2 = 256;   // rows per pair
constexpr int BN = 256;
constexpr int BNH = 128;   // B rows loaded per CTA
constexpr int BK = 64;
constexpr int STAGES = 6;

struct Gemm2Params {
  int M, N, K;
  int tiles_m, tiles_n, num_kb, splits, kb_per_split;
  void* C;
  long long ldc, split_stride;
  float alpha;
  const float* alpha_a;  // optional device scalars multiplied into alpha (the fp8 operands' inverse scales)
  const float* alpha_b;
  uint32_t fp8_formats;  // instruction-descriptor format bits of the fp8 operands (A at bit 7, B at bit 10: 0 e4m3, 1 e5m2)
  int epi;  // 0 bf16, 1 fp32 store, 2 fp32 accumulate
  int group_m;
  int* status;
  // fused tensor-parallel collectives (same protocol as the single-CTA kernel in gemm.cu)
  int m_rot;            // tile rows (of 256) are visited starting here
  int g_ncopy;          // > 0: gather mode, this many leading CTAs (whole pairs) copy the peers' shards
  int g_world, g_rank, g_rows_per_rank, g_chunk_rows, g_epoch;
  unsigned long long g_wait_ns;  // limit of the waits on flags another GPU raises
  long long g_ld;
  const void* g_src[16];
  __nv_bfloat16* g_dst;
  int* g_flags;
  const int* g_ready;
  // g_mode 1: the copy CTAs gather a FLAT byte range that is sharded evenly over the ranks (a unit of sharded
  // parameters) into g_dst, and the B operand of this GEMM lies inside that range: an MMA CTA waits for the chunks that
  // hold its B rows instead of for a chunk of A rows
  int g_mode;
  int gb_chunk_shift;                 // log2 of the chunk size in bytes; a chunk never straddles two shards
  int gb_first_chunk;                 // chunks are fetched starting here (the one that holds the start of B), wrapping
  long long gb_shard_bytes;           // bytes of one rank's shard
  long long gb_lo, gb_hi;             // byte range [lo, hi) of the flat buffer to fetch, multiples of 16
  long long gb_b_off, gb_b_bytes;     // where B lies inside the flat buffer
  long long ldb;                      // row stride of B in elements
  // swiglu_I > 0: B is the fused [2 I, K] gate / up weight.  CTA 0 of a pair loads 128 gate rows and CTA 1 the matching
  // 128 up rows, so the 256 accumulator columns of a row are gate_j | up_j for the same 128 hidden indices j, and the
  // epilogue writes gate and up (kept for the backward pass) and z = silu(gate) * up in one go
  int swiglu_I;
  __nv_bfloat16* Z;
  long long ldz;
  int s_world;          // > 0: scatter mode, rows are stored into the owner rank's receive slot
  int s_rank, s_rows_per_rank;
  void* s_dst[16];
};

struct Smem2 {
  static constexpr int A_BYTES = BMH * BK * 2;
  static constexpr int B_BYTES = BNH * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;  // 32 KB
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void remote_expect_tx(uint32_t cluster_bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void remote_arrive(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// TMA load issued by either CTA of the pair; completion bytes are credited to the barrier at `cluster_bar`
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t cluster_bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::
          "r"(smem_u32(smem_dst)),
      "l"(map), "r"(cluster_bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void mma2_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}
// arrive on the barrier at this shared-memory offset in BOTH CTAs of the pair once the issued MMAs are done:
// one commit per destination (the leader's own barrier, then the peer's through its cluster address)
__device__ __forceinline__ void mma2_commit_both(uint64_t* bar) {
  const uint32_t mine = smem_u32(bar);
  const uint32_t peer = map_to_cta(mine, 1);
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mine) : "memory");
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(peer) : "memory");
}

__device__ __forceinline__ void unit_to_tile(const Gemm2Params& p, int unit, int& tm, int& tn, int& split) {
  int tile = unit / p.splits;
  split = unit - tile * p.splits;
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

__device__ __forceinline__ int ld_acquire_gpu2(const int* addr) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
__device__ __forceinline__ int ld_acquire_sys2(const int* addr) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
// kind::f8f6f4: 8-bit floating-point operands (K = 32 per instruction), fp32 accumulation
__device__ __forceinline__ void mma2_ss_f8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}

template <bool SYS>
__device__ __forceinline__ bool wait_flag2(const int* addr, int value, int* status, unsigned long long limit_ns) {
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while ((SYS ? ld_acquire_sys2(addr) : ld_acquire_gpu2(addr)) < value) {
    if ((++spins & 0xFF) == 0 && globaltimer_ns() - t0 > limit_ns) {
      report(status, ERR_WAIT_PEER);
      return false;
    }
    __nanosleep(32);
  }
  return true;
}

// Copy role of the gather mode: shard chunks are fetched in ring order starting with the local shard and every landed
// chunk is published through its flag.  The data moves with bulk asynchronous copies (no multicast): peer global memory
// -> this CTA's shared memory -> local global memory, in pieces of up to 32 KB through a ring of six slots, all issued by
// one thread.  Five peer loads stay in flight per CTA while one store drains, so the NVLink pipe stays full with a few
// CTAs (a load round trip is microseconds; sixteen CTAs keep about 2.5 MB in flight).
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

__device__ void gather_copy_role2(const Gemm2Params& p, uint8_t* smem, uint64_t* bars, volatile int* abort_flag) {
  constexpr int NSLOT = STAGES;
  constexpr uint32_t SLOT = Smem2::STAGE_BYTES;  // 32 KB
  if (threadIdx.x != 0) return;
  for (int s = 0; s < NSLOT; ++s) mbar_init(&bars[s], 1);
  *abort_flag = 0;
  mbar_fence_init();
  const int cpr = p.g_rows_per_rank / p.g_chunk_rows;
  const int total = cpr * p.g_world;
  const long long row_bytes = (long long)p.K * 2;
  const bool flat = (p.g_ld == p.K);                        // rows are back to back: a chunk is one byte range
  uint32_t issued = 0, consumed = 0;                        // pieces issued / stored so far (ring positions)
  for (int c = blockIdx.x; c < total; c += p.g_ncopy) {
    const int src = (p.g_rank + c / cpr) % p.g_world;
    const int cc = c % cpr;
    const bool ok = (src == p.g_rank) || wait_flag2<true>(p.g_ready + src, p.g_epoch, p.status, p.g_wait_ns);
    const long long src_row0 = (long long)cc * p.g_chunk_rows;
    const long long dst_row0 = (long long)src * p.g_rows_per_rank + src_row0;
    if (ok) {
      const uint8_t* sp = reinterpret_cast<const uint8_t*>(p.g_src[src]) + src_row0 * p.g_ld * 2;
      uint8_t* dp = reinterpret_cast<uint8_t*>(p.g_dst) + dst_row0 * p.g_ld * 2;
      // piece i covers bytes [off(i), off(i) + len(i)) of the chunk (flat) or row i (strided rows)
      const long long chunk_bytes = (long long)p.g_chunk_rows * row_bytes;
      const long long npieces = flat ? (chunk_bytes + SLOT - 1) / SLOT : p.g_chunk_rows;
      auto piece = [&](long long i, long long& off, uint32_t& len) {
        if (flat) {
          off = i * SLOT;
          len = (uint32_t)min((long long)SLOT, chunk_bytes - off);
        } else {
          off = i * p.g_ld * 2;
          len = (uint32_t)row_bytes;
        }
      };
      long long next = 0;  // next piece of this chunk to load
      bool alive = true;
      // prologue: fill the ring
      for (; next < npieces && next < NSLOT; ++next) {
        long long off; uint32_t len;
        piece(next, off, len);
        const uint32_t slot = issued % NSLOT;
        mbar_expect_tx(&bars[slot], len);
        bulk_load(smem + slot * SLOT, sp + off, len, &bars[slot]);
        ++issued;
      }
      for (long long i = 0; i < npieces && alive; ++i) {
        long long off; uint32_t len;
        piece(i, off, len);
        const uint32_t slot = consumed % NSLOT;
        if (!mbar_wait(&bars[slot], (consumed / NSLOT) & 1, p.status, abort_flag, ERR_WAIT_FULL)) { alive = false; break; }
        bulk_store(dp + off, smem + slot * SLOT, len);
        ++consumed;
        if (next < npieces) {
          // the slot may be refilled once the store has finished reading it
          asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          long long off2; uint32_t len2;
          piece(next, off2, len2);
          mbar_expect_tx(&bars[slot], len2);
          bulk_load(smem + slot * SLOT, sp + off2, len2, &bars[slot]);
          ++issued;
          ++next;
        }
      }
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // every store of the chunk has been performed
      asm volatile("fence.proxy.async.global;" ::: "memory");    // async-proxy writes before the generic-proxy flag store
      if (!alive) {
        // a load did not arrive within the limit: loads of this chunk may still be in flight, so stop using the ring
        __threadfence();
        asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p.g_flags + dst_row0 / p.g_chunk_rows), "r"(p.g_epoch) : "memory");
        for (int c2 = c + p.g_ncopy; c2 < total; c2 += p.g_ncopy) {  // publish the rest so that nobody waits for them
          const int src2 = (p.g_rank + c2 / cpr) % p.g_world;
          const long long d2 = (long long)src2 * p.g_rows_per_rank + (long long)(c2 % cpr) * p.g_chunk_rows;
          asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p.g_flags + d2 / p.g_chunk_rows), "r"(p.g_epoch) : "memory");
        }
        return;
      }
    }
    __threadfence();
    asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p.g_flags + dst_row0 / p.g_chunk_rows), "r"(p.g_epoch) : "memory");
  }
}

// Copy role of the flat gather mode (g_mode 1).  One thread per copy CTA moves chunks peer (or local) shard -> shared
// memory ring -> local flat buffer with bulk asynchronous copies (no multicast) and publishes one flag per chunk.  Nothing
// here waits for another GPU: the launch is ordered after a bounded wait for the peers' "parameters written" flags.
__device__ void gather_flat_role2(const Gemm2Params& p, uint8_t* smem, uint64_t* bars, volatile int* abort_flag) {
  constexpr int NSLOT = STAGES;
  constexpr long long SLOT = Smem2::STAGE_BYTES;  // 32 KB
  if (threadIdx.x != 0) return;
  for (int s = 0; s < NSLOT; ++s) mbar_init(&bars[s], 1);
  *abort_flag = 0;
  mbar_fence_init();
  const long long CH = 1ll << p.gb_chunk_shift;
  const int c_lo = (int)(p.gb_lo >> p.gb_chunk_shift);
  const int c_hi = (int)((p.gb_hi + CH - 1) >> p.gb_chunk_shift);
  const int total = c_hi - c_lo;
  uint32_t issued = 0, consumed = 0;
  bool alive = true;
  for (int idx = blockIdx.x; idx < total; idx += p.g_ncopy) {
    const int c = c_lo + (p.gb_first_chunk - c_lo + idx) % total;
    if (alive) {
      const long long b0 = max((long long)c * CH, p.gb_lo), b1 = min((long long)(c + 1) * CH, p.gb_hi);
      const int src = (int)(b0 / p.gb_shard_bytes);
      const uint8_t* sp = reinterpret_cast<const uint8_t*>(p.g_src[src]) + (b0 - (long long)src * p.gb_shard_bytes);
      uint8_t* dp = reinterpret_cast<uint8_t*>(p.g_dst) + b0;
      const long long bytes = b1 - b0;
      const long long npieces = (bytes + SLOT - 1) / SLOT;
      long long next = 0;
      for (; next < npieces && next < NSLOT; ++next) {
        const uint32_t len = (uint32_t)min(SLOT, bytes - next * SLOT);
        const uint32_t slot = issued % NSLOT;
        mbar_expect_tx(&bars[slot], len);
        bulk_load(smem + slot * SLOT, sp + next * SLOT, len, &bars[slot]);
        ++issued;
      }
      for (long long i = 0; i < npieces; ++i) {
        const uint32_t len = (uint32_t)min(SLOT, bytes - i * SLOT);
        const uint32_t slot = consumed % NSLOT;
        if (!mbar_wait(&bars[slot], (consumed / NSLOT) & 1, p.status, abort_flag, ERR_WAIT_FULL)) { alive = false; break; }
        bulk_store(dp + i * SLOT, smem + slot * SLOT, len);
        ++consumed;
        if (next < npieces) {
          asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          const uint32_t len2 = (uint32_t)min(SLOT, bytes - next * SLOT);
          mbar_expect_tx(&bars[slot], len2);
          bulk_load(smem + slot * SLOT, sp + next * SLOT, len2, &bars[slot]);
          ++issued;
          ++next;
        }
      }
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
      asm volatile("fence.proxy.async.global;" ::: "memory");
    }
    // published even after a failed load (the status word is set): no consumer waits for ever
    __threadfence();
    asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p.g_flags + c), "r"(p.g_epoch) : "memory");
  }
}

// FP8: both operands are K-major 8-bit floats; a stage still holds 128-byte rows, i.e. 128 elements of K instead of 64.
template <bool A_MN, bool B_MN, bool FP8>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, Gemm2Params p) {
  using L = Smem2;
  static_assert(!FP8 || (!A_MN && !B_MN), "fp8 operands are K-major");
  constexpr int BKE = FP8 ? 2 * BK : BK;  // elements of K per stage
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = (uint64_t*)(smem + L::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = (uint32_t*)(tempty_bar + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  if (p.g_ncopy > 0 && (int)blockIdx.x < p.g_ncopy) {  // whole CTA pairs take this branch: nobody waits for them
    if (p.g_mode == 1) gather_flat_role2(p, smem, full_bar, abort_flag);
    else gather_copy_role2(p, smem, full_bar, abort_flag);
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = ((int)blockIdx.x - p.g_ncopy) >> 1, npairs = ((int)gridDim.x - p.g_ncopy) >> 1;
  const int total_units = p.tiles_m * p.tiles_n * p.splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 2);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 8);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc2(tmem_slot, 512);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int b_waited_tn = -1;  // flat gather mode: the tile column whose B chunks were already awaited
      for (int unit = pair; unit < total_units && ok; unit += npairs) {
        int tm, tn, split;
        unit_to_tile(p, unit, tm, tn, split);
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(p.num_kb, kb0 + p.kb_per_split);
        if (p.g_ncopy > 0 && p.g_mode == 1) {
          // this CTA's half of the B tile comes out of the gathered flat buffer: K-major B = 128 consecutive rows of the
          // weight (one byte range); MN-major B touches every row, so the whole weight must have landed
          if (B_MN ? (b_waited_tn < 0) : (b_waited_tn != tn)) {
            long long lo_b = p.gb_b_off, hi_b = p.gb_b_off + p.gb_b_bytes;
            if (!B_MN) {
              const long long n0 = (long long)tn * BN + (long long)rank * BNH;
              const long long n1 = min((long long)p.N, n0 + BNH);
              lo_b = p.gb_b_off + n0 * p.ldb * 2;
              hi_b = p.gb_b_off + n1 * p.ldb * 2;
            }
            if (hi_b > lo_b) {
              const int c0 = (int)(lo_b >> p.gb_chunk_shift), c1 = (int)((hi_b - 1) >> p.gb_chunk_shift);
              for (int c = c0; c <= c1; ++c)
                if (!wait_flag2<false>(p.g_flags + c, p.g_epoch, p.status, kWaitLimitNs)) { *abort_flag = 1; break; }
            }
            asm volatile("fence.proxy.async.global;" ::: "memory");
            b_waited_tn = tn;
          }
        } else if (p.g_ncopy > 0) {
          // this CTA's 128 rows of A come from one gathered chunk: wait until the copy CTAs published it, then order
          // their generic-proxy writes before the TMA reads of the async proxy
          if (!wait_flag2<false>(p.g_flags + (tm * BM2 + (int)rank * BMH) / p.g_chunk_rows, p.g_epoch, p.status, p.g_wait_ns + kWaitLimitNs)) *abort_flag = 1;
          asm volatile("fence.proxy.async.global;" ::: "memory");
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, abort_flag, ERR_WAIT_EMPTY)) { ok = false; break; }
          const uint32_t lead_full = map_to_cta(smem_u32(&full_bar[stage]), 0);
          uint8_t* sA = smem + stage * L::STAGE_BYTES;
          uint8_t* sB = sA + L::A_BYTES;
          remote_expect_tx(lead_full, L::STAGE_BYTES);
          const int m0 = tm * BM2 + (int)rank * BMH;
          const int n0 = p.swiglu_I > 0 ? tn * BNH + (int)rank * p.swiglu_I : tn * BN + (int)rank * BNH;
          if (!A_MN) {
            tma_load_2d_pair(sA, &tmA, lead_full, kb * BKE, m0);
          } else {
#pragma unroll
            for (int g = 0; g < BMH / 64; ++g) tma_load_2d_pair(sA + g * (64 * BK * 2), &tmA, lead_full, m0 + g * 64, kb * BK);
          }
          if (!B_MN) {
            tma_load_2d_pair(sB, &tmB, lead_full, kb * BKE, n0);
          } else {
#pragma unroll
            for (int g = 0; g < BNH / 64; ++g) tma_load_2d_pair(sB + g * (64 * BK * 2), &tmB, lead_full, n0 + g * 64, kb * BK);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (leader && lane == 0) {
      const uint32_t idesc = FP8 ? (make_idesc_fp8(BM2, BN) | p.fp8_formats) : make_idesc_bf16(BM2, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      constexpr uint32_t A_LBO = A_MN ? 64 * BK * 2 : 16;
      constexpr uint32_t B_LBO = B_MN ? 64 * BK * 2 : 16;
      constexpr uint32_t A_KSTEP = A_MN ? 16 * 128 : 32;
      constexpr uint32_t B_KSTEP = B_MN ? 16 * 128 : 32;
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int unit = pair; unit < total_units && ok; unit += npairs, ++it) {
        int tm, tn, split;
        unit_to_tile(p, unit, tm, tn, split);
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(p.num_kb, kb0 + p.kb_per_split);
        const int acc = it & 1;
        if (!mbar_wait(&tempty_bar[acc], ((it >> 1) & 1) ^ 1, p.status, abort_flag, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, p.status, abort_flag, ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + stage * L::STAGE_BYTES);
          const uint32_t sB = sA + L::A_BYTES;
          const uint64_t adesc = make_smem_desc(sA, A_LBO, 1024);
          const uint64_t bdesc = make_smem_desc(sB, B_LBO, 1024);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            if (FP8)
              mma2_ss_f8(d_tmem, desc_advance(adesc, k * A_KSTEP), desc_advance(bdesc, k * B_KSTEP), idesc,
                         (kb > kb0 || k > 0) ? 1u : 0u);
            else
              mma2_ss(d_tmem, desc_advance(adesc, k * A_KSTEP), desc_advance(bdesc, k * B_KSTEP), idesc,
                      (kb > kb0 || k > 0) ? 1u : 0u);
          }
          mma2_commit_both(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) mma2_commit_both(&tfull_bar[acc]);
      }
    }
  } else {
    const int quarter = warp & 3;
    int it = 0;
    bool ok = true;
    float alpha = p.alpha;
    if (FP8) {
      if (p.alpha_a) alpha *= __ldg(p.alpha_a);
      if (p.alpha_b) alpha *= __ldg(p.alpha_b);
    }
    for (int unit = pair; unit < total_units && ok; unit += npairs, ++it) {
      int tm, tn, split;
      unit_to_tile(p, unit, tm, tn, split);
      const int acc = it & 1;
      if (!mbar_wait_warp(&tfull_bar[acc], (it >> 1) & 1, p.status, abort_flag, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int row = tm * BM2 + (int)rank * BMH + quarter * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t t_row = tmem_base + acc * BN + ((uint32_t)(quarter * 32) << 16);
      if (p.swiglu_I > 0) {
        __nv_bfloat16* grow = (__nv_bfloat16*)p.C + (long long)row * p.ldc + tn * BNH;
        __nv_bfloat16* urow = grow + p.swiglu_I;
        __nv_bfloat16* zrow = p.Z + (long long)row * p.ldz + tn * BNH;
#pragma unroll 1
        for (int c = 0; c < BNH; c += 32) {
          uint32_t g[32], u[32];
          tmem_ld_32x32(t_row + c, g);
          tmem_ld_32x32(t_row + BNH + c, u);
          tmem_ld_wait();
          if (!row_ok) continue;
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 qg, qu, qz;
            uint32_t* wg = reinterpret_cast<uint32_t*>(&qg);
            uint32_t* wu = reinterpret_cast<uint32_t*>(&qu);
            uint32_t* wz = reinterpret_cast<uint32_t*>(&qz);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              // the activation is taken on the bf16 values that are stored, so a backward pass that re-reads gate and up
              // sees exactly the operands of z
              wg[e] = pack_bf16(__uint_as_float(g[j + 2 * e]), __uint_as_float(g[j + 2 * e + 1]));
              wu[e] = pack_bf16(__uint_as_float(u[j + 2 * e]), __uint_as_float(u[j + 2 * e + 1]));
              const float2 gf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wg[e]));
              const float2 uf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wu[e]));
              wz[e] = pack_bf16(gf.x / (1.f + __expf(-gf.x)) * uf.x, gf.y / (1.f + __expf(-gf.y)) * uf.y);
            }
            *reinterpret_cast<uint4*>(grow + c + j) = qg;
            *reinterpret_cast<uint4*>(urow + c + j) = qu;
            *reinterpret_cast<uint4*>(zrow + c + j) = qz;
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) remote_arrive(map_to_cta(smem_u32(&tempty_bar[acc]), 0));
        continue;
      }
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        const int col0 = tn * BN + c;
        if (col0 >= p.N) break;
        uint32_t r[32];
        tmem_ld_32x32(t_row + c, r);
        tmem_ld_wait();
        if (!row_ok) continue;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * alpha;
        const bool full = (col0 + 32 <= p.N);
        if (p.epi == 0) {
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
          const bool accumulate = (p.epi == 2);
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
      if (lane == 0) remote_arrive(map_to_cta(smem_u32(&tempty_bar[acc]), 0));
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // nobody leaves while the peer may still signal into this CTA
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, 512);
  }
}

template <bool A_MN, bool B_MN, bool FP8 = false>
int launch2(const CUtensorMap& tmA, const CUtensorMap& tmB, const Gemm2Params& p, int sm_count, cudaStream_t stream) {
  auto kern = gemm2_bf16_kernel<A_MN, B_MN, FP8>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem2::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  // CTA pairs that can be resident at once (a GPC with an odd number of free SMs strands one)
  static int max_pairs = 0;
  if (max_pairs == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((sm_count / 2) * 2);
    cfg.blockDim = dim3(192);
    cfg.dynamicSmemBytes = Smem2::TOTAL;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = sm_count / 2;
    }
    max_pairs = n < sm_count / 2 ? n : sm_count / 2;
  }
  int units = p.tiles_m * p.tiles_n * p.splits;
  int avail = max_pairs - p.g_ncopy / 2;  // the copy pairs of the gather mode occupy SMs of their own
  if (avail < 1) avail = 1;
  int pairs = units < avail ? units : avail;
  kern<<<pairs * 2 + p.g_ncopy, 192, Smem2::TOTAL, stream>>>(tmA, tmB, p);
  return fb::launch_ok(FP8 ? "gemm2_fp8_kernel" : "gemm2_bf16_kernel");
}

}  // namespace

extern "C" {

// Same contract as fb_gemm_bf16 without bias; splits > 1 writes fp32 partials [splits, M, N] into `workspace`
// (the caller reduces them with the split-K reduction of gemm.cu).  Returns 0 on success.
int fb_gemm2_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb, long long ldc,
                  int a_mn, int b_mn, int out_mode, float alpha, int splits, void* workspace, int sm_count,
                  cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda & 7) || (ldb & 7) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15)) return -2;
  Gemm2Params p;
  p.M = M; p.N = N; p.K = K;
  p.tiles_m = (M + BM2 - 1) / BM2;
  p.tiles_n = (N + BN - 1) / BN;
  p.num_kb = (K + BK - 1) / BK;
  if (splits < 1) splits = 1;
  if (splits > p.num_kb) splits = p.num_kb;
  p.kb_per_split = (p.num_kb + splits - 1) / splits;
  p.splits = (p.num_kb + p.kb_per_split - 1) / p.kb_per_split;
  p.alpha = alpha;
  p.alpha_a = nullptr; p.alpha_b = nullptr; p.fp8_formats = 0;
  p.group_m = 8;
  p.status = fb::status_ptr();
  p.m_rot = 0; p.g_ncopy = 0; p.g_mode = 0; p.s_world = 0; p.swiglu_I = 0;
  if (p.splits > 1) {
    if (workspace == nullptr) return -3;
    p.C = workspace; p.ldc = N; p.split_stride = (long long)M * N; p.epi = 1;
  } else {
    p.C = C; p.ldc = ldc; p.split_stride = 0; p.epi = out_mode;
  }
  CUtensorMap tmA, tmB;
  int rc;
  if (!a_mn) rc = fb::make_tmap_2d(&tmA, A, 2, M, K, lda, BMH, BK, true);
  else       rc = fb::make_tmap_2d(&tmA, A, 2, K, M, lda, BK, 64, true);
  if (rc) return rc;
  if (!b_mn) rc = fb::make_tmap_2d(&tmB, B, 2, N, K, ldb, BNH, BK, true);
  else       rc = fb::make_tmap_2d(&tmB, B, 2, K, N, ldb, BK, 64, true);
  if (rc) return rc;
  if (!a_mn && !b_mn) return launch2<false, false>(tmA, tmB, p, sm_count, stream);
  if (!a_mn && b_mn)  return launch2<false, true>(tmA, tmB, p, sm_count, stream);
  if (a_mn && !b_mn)  return launch2<true, false>(tmA, tmB, p, sm_count, stream);
  return launch2<true, true>(tmA, tmB, p, sm_count, stream);
}


// C[M, N] = alpha * inv_a * inv_b * A[M, K] @ B[N, K]^T with 8-bit floating-point operands (row strides in bytes =
// elements, multiples of 16).  a_e5m2 / b_e5m2 pick e5m2 over e4m3 per operand; inv_a / inv_b are device scalars (the
// operands' dequantisation factors) or null.  out_mode: 0 bf16, 1 fp32 store, 2 fp32 accumulate.
int fb_gemm2_fp8(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb, long long ldc,
                 int a_e5m2, int b_e5m2, const float* inv_a, const float* inv_b, int out_mode, float alpha, int sm_count,
                 cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda & 15) || (ldb & 15) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15)) return -2;
  Gemm2Params p;
  p.M = M; p.N = N; p.K = K;
  p.tiles_m = (M + BM2 - 1) / BM2;
  p.tiles_n = (N + BN - 1) / BN;
  p.num_kb = (K + 2 * BK - 1) / (2 * BK);
  p.splits = 1;
  p.kb_per_split = p.num_kb;
  p.alpha = alpha;
  p.alpha_a = inv_a; p.alpha_b = inv_b;
  p.fp8_formats = ((uint32_t)(a_e5m2 ? 1 : 0) << 7) | ((uint32_t)(b_e5m2 ? 1 : 0) << 10);
  p.group_m = 8;
  p.status = fb::status_ptr();
  p.m_rot = 0; p.g_ncopy = 0; p.g_mode = 0; p.s_world = 0; p.swiglu_I = 0;
  p.C = C; p.ldc = ldc; p.split_stride = 0; p.epi = out_mode;
  CUtensorMap tmA, tmB;
  int rc = fb::make_tmap_2d(&tmA, A, 1, M, K, lda, BMH, 2 * BK, true);
  if (rc) return rc;
  rc = fb::make_tmap_2d(&tmB, B, 1, N, K, ldb, BNH, 2 * BK, true);
  if (rc) return rc;
  return launch2<false, false, true>(tmA, tmB, p, sm_count, stream);
}

// All-gather -> GEMM on CTA pairs; arguments as fb_gemm_allgather_a (gemm.cu).  M = world * rows_per_rank must be a
// multiple of 256.
int fb_gemm2_allgather_a(const unsigned long long* shard_ptrs, int world, int rank, int rows_per_rank, long long ld,
                         void* a_full, int* chunk_flags, const int* ready, int epoch, const void* B, void* C, int N, int K,
                         long long ldb, long long ldc, int b_mn, int sm_count, cudaStream_t stream) {
  const int M = world * rows_per_rank;
  if (world > 16 || (rows_per_rank % BMH) || (M % BM2) || (ld & 7) || (ldb & 7) || (K & 7)) return -2;
  if (ld != K && (long long)K * 2 > Smem2::STAGE_BYTES) return -2;  // a strided row must fit one 32 KB copy slot
  int chunk_rows = 1024;
  while (rows_per_rank % chunk_rows) chunk_rows >>= 1;
  Gemm2Params p;
  p.M = M; p.N = N; p.K = K;
  p.tiles_m = M / BM2;
  p.tiles_n = (N + BN - 1) / BN;
  p.num_kb = (K + BK - 1) / BK;
  p.splits = 1; p.kb_per_split = p.num_kb;
  p.C = C; p.ldc = ldc; p.split_stride = 0;
  p.alpha = 1.f; p.epi = 0; p.group_m = 8;
  p.status = fb::status_ptr();
  p.m_rot = (rank * rows_per_rank) / BM2;  // start at the tile row that holds the local shard
  p.g_ncopy = 16;
  p.g_mode = 0; p.swiglu_I = 0;
  p.g_world = world; p.g_rank = rank; p.g_rows_per_rank = rows_per_rank; p.g_chunk_rows = chunk_rows; p.g_epoch = epoch;
  p.g_wait_ns = fb::peer_wait_ns();
  p.g_ld = ld;
  for (int r = 0; r < 16; ++r) p.g_src[r] = r < world ? (const void*)shard_ptrs[r] : nullptr;
  p.g_dst = (__nv_bfloat16*)a_full;
  p.g_flags = chunk_flags;
  p.g_ready = ready;
  p.s_world = 0;
  CUtensorMap tmA, tmB;
  int rc = fb::make_tmap_2d(&tmA, a_full, 2, M, K, ld, BMH, BK, true);
  if (rc) return rc;
  if (!b_mn) rc = fb::make_tmap_2d(&tmB, B, 2, N, K, ldb, BNH, BK, true);
  else       rc = fb::make_tmap_2d(&tmB, B, 2, K, N, ldb, BK, 64, true);
  if (rc) return rc;
  if (!b_mn) return launch2<false, false>(tmA, tmB, p, sm_count, stream);
  return launch2<false, true>(tmA, tmB, p, sm_count, stream);
}

// gate | up projection with the SwiGLU activation in the epilogue:
//   GU[M, 2 I] = A[M, K] * W[2 I, K]^T  (gate columns first, then up, as the backward pass wants them)  and
//   Z[M, I]    = silu(GU[:, :I]) * GU[:, I:]
// from one pass over the accumulators; I must be a multiple of 128.  Takes the place of the GEMM plus the stand-alone
// SwiGLU kernel (fla/modules/activations.py:553-628 after fla/modules/mlp.py:58-60).
int fb_gemm2_swiglu(const void* A, const void* W, void* GU, void* Z, int M, int I, int K, long long lda, long long ldw,
                    long long ldgu, long long ldz, int sm_count, cudaStream_t stream) {
  if (M <= 0 || I <= 0 || K <= 0) return 0;
  if ((I % BNH) || (lda & 7) || (ldw & 7) || (ldgu & 7) || (ldz & 7) || ((uintptr_t)A & 15) || ((uintptr_t)W & 15) ||
      ((uintptr_t)GU & 15) || ((uintptr_t)Z & 15))
    return -2;
  Gemm2Params p;
  p.M = M; p.N = 2 * I; p.K = K;
  p.tiles_m = (M + BM2 - 1) / BM2;
  p.tiles_n = I / BNH;
  p.num_kb = (K + BK - 1) / BK;
  p.splits = 1; p.kb_per_split = p.num_kb;
  p.alpha = 1.f; p.alpha_a = nullptr; p.alpha_b = nullptr; p.fp8_formats = 0;
  p.group_m = 8;
  p.status = fb::status_ptr();
  p.m_rot = 0; p.g_ncopy = 0; p.g_mode = 0; p.s_world = 0;
  p.swiglu_I = I; p.Z = (__nv_bfloat16*)Z; p.ldz = ldz;
  p.C = GU; p.ldc = ldgu; p.split_stride = 0; p.epi = 0;
  CUtensorMap tmA, tmB;
  int rc = fb::make_tmap_2d(&tmA, A, 2, M, K, lda, BMH, BK, true);
  if (rc) return rc;
  rc = fb::make_tmap_2d(&tmB, W, 2, 2 * I, K, ldw, BNH, BK, true);
  if (rc) return rc;
  return launch2<false, false>(tmA, tmB, p, sm_count, stream);
}

// Sharded-parameter all-gather fused into the first GEMM that consumes one of the gathered weights.
//   C[M, N] = A[M, K] * B^T   with B = a weight that lies inside a flat parameter buffer `flat_dst` whose contents are
//   sharded evenly over `world` ranks (`shard_ptrs[r]` = rank r's shard, `shard_bytes` each; peer memory).
// Sixteen copy CTAs pull bytes [lo, hi) of the flat buffer from the shards (plain bulk copies, no multicast, through a
// shared-memory ring) and raise one flag per 2^chunk_shift bytes in `chunk_flags` (value `epoch`); the MMA CTA pairs wait
// only for the chunks that hold their B rows, so the product starts as soon as the first rows of the weight have landed
// and the rest of the unit's parameters arrive underneath it.  When the kernel ends the whole range is in place for the
// kernels that follow on the stream.  b_mn: 0 = B is [N, K] (forward), 1 = B is [K, N] (data gradient).  bf16 output.
// Requirements: lo, hi, b_off, shard_bytes multiples of 16; shard_bytes a multiple of the chunk size; the caller has
// ordered this launch after a (bounded) wait for the peers' shards to be final.
int fb_gemm2_gather_b(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb, long long ldc,
                      int b_mn, const unsigned long long* shard_ptrs, int world, int rank, long long shard_bytes,
                      void* flat_dst, long long lo, long long hi, int chunk_shift, int* chunk_flags, int epoch, int sm_count,
                      cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda & 7) || (ldb & 7) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15)) return -2;
  if (world > 16 || world < 1 || (lo & 15) || (hi & 15) || (shard_bytes & 15) || lo < 0 || hi > shard_bytes * world || hi <= lo)
    return -2;
  if (chunk_shift < 12 || (shard_bytes & ((1ll << chunk_shift) - 1))) return -2;
  const long long b_off = (const uint8_t*)B - (const uint8_t*)flat_dst;
  const long long b_rows = b_mn ? K : N;
  const long long b_bytes = ((b_rows - 1) * ldb + (b_mn ? N : K)) * 2;
  if (b_off < lo || b_off + b_bytes > hi) return -3;  // B is not inside the gathered range
  Gemm2Params p;
  p.M = M; p.N = N; p.K = K;
  p.tiles_m = (M + BM2 - 1) / BM2;
  p.tiles_n = (N + BN - 1) / BN;
  p.num_kb = (K + BK - 1) / BK;
  p.splits = 1; p.kb_per_split = p.num_kb;
  p.C = C; p.ldc = ldc; p.split_stride = 0;
  p.alpha = 1.f; p.alpha_a = nullptr; p.alpha_b = nullptr; p.fp8_formats = 0;
  p.epi = 0; p.group_m = 8;
  p.status = fb::status_ptr();
  p.m_rot = 0;
  p.g_ncopy = 16;
  p.g_mode = 1; p.swiglu_I = 0;
  p.g_world = world; p.g_rank = rank; p.g_rows_per_rank = 0; p.g_chunk_rows = 1; p.g_epoch = epoch;
  p.g_wait_ns = fb::peer_wait_ns();
  p.g_ld = 0;
  for (int r = 0; r < 16; ++r) p.g_src[r] = r < world ? (const void*)shard_ptrs[r] : nullptr;
  p.g_dst = (__nv_bfloat16*)flat_dst;
  p.g_flags = chunk_flags;
  p.g_ready = nullptr;
  p.gb_chunk_shift = chunk_shift;
  p.gb_first_chunk = (int)(b_off >> chunk_shift);
  p.gb_shard_bytes = shard_bytes;
  p.gb_lo = lo; p.gb_hi = hi;
  p.gb_b_off = b_off; p.gb_b_bytes = b_bytes;
  p.ldb = ldb;
  p.s_world = 0;
  CUtensorMap tmA, tmB;
  int rc = fb::make_tmap_2d(&tmA, A, 2, M, K, lda, BMH, BK, true);
  if (rc) return rc;
  if (!b_mn) rc = fb::make_tmap_2d(&tmB, B, 2, N, K, ldb, BNH, BK, true);
  else       rc = fb::make_tmap_2d(&tmB, B, 2, K, N, ldb, BK, 64, true);
  if (rc) return rc;
  if (!b_mn) return launch2<false, false>(tmA, tmB, p, sm_count, stream);
  return launch2<false, true>(tmA, tmB, p, sm_count, stream);
}

// GEMM -> scatter of rows into the owners' receive slots on CTA pairs; arguments as fb_gemm_scatter_rows (gemm.cu).
int fb_gemm2_scatter_rows(const void* A, const void* B, const unsigned long long* recv_ptrs, int world, int rank,
                          int rows_per_rank, int N, int K, long long lda, long long ldb, long long ldc, int b_mn, int sm_count,
                          cudaStream_t stream) {
  const int M = world * rows_per_rank;
  if (world > 16 || (rows_per_rank % BMH) || (M % BM2) || (lda & 7) || (ldb & 7) || (ldc & 7)) return -2;
  Gemm2Params p;
  p.M = M; p.N = N; p.K = K;
  p.tiles_m = M / BM2;
  p.tiles_n = (N + BN - 1) / BN;
  p.num_kb = (K + BK - 1) / BK;
  p.splits = 1; p.kb_per_split = p.num_kb;
  p.C = nullptr; p.ldc = ldc; p.split_stride = 0;
  p.alpha = 1.f; p.epi = 0; p.group_m = 8;
  p.status = fb::status_ptr();
  p.m_rot = ((((rank + 1) % world) * rows_per_rank) / BM2) % p.tiles_m;  // remote rows first, own rows last
  p.g_ncopy = 0; p.g_mode = 0; p.swiglu_I = 0;
  p.s_world = world; p.s_rank = rank; p.s_rows_per_rank = rows_per_rank;
  for (int r = 0; r < 16; ++r) p.s_dst[r] = r < world ? (void*)recv_ptrs[r] : nullptr;
  CUtensorMap tmA, tmB;
  int rc = fb::make_tmap_2d(&tmA, A, 2, M, K, lda, BMH, BK, true);
  if (rc) return rc;
  if (!b_mn) rc = fb::make_tmap_2d(&tmB, B, 2, N, K, ldb, BNH, BK, true);
  else       rc = fb::make_tmap_2d(&tmB, B, 2, K, N, ldb, BK, 64, true);
  if (rc) return rc;
  if (!b_mn) return launch2<false, false>(tmA, tmB, p, sm_count, stream);
  return launch2<false, true>(tmA, tmB, p, sm_count, stream);
}

}  // extern "C"
