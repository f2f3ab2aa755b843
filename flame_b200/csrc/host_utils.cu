#include "host_utils.cuh"
#include <mutex>

namespace fb {

static int* g_status_host = nullptr;
static std::once_flag g_status_once;

int* status_ptr() {
  std::call_once(g_status_once, []() {
    void* p = nullptr;
    if (cudaHostAlloc(&p, 256, cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) {
      fprintf(stderr, "[flame_b200] cannot allocate the pinned status word\n");
      p = nullptr;
    } else {
      for (int i = 0; i < 64; ++i) ((int*)p)[i] = 0;
    }
    g_status_host = (int*)p;
  });
  return g_status_host;
}

// Limit of the waits on flags that ANOTHER GPU raises (peer gradients final, peer shard published).  Two seconds by
// default; a trainer raises it for the first step (peers may still be compiling or loading) and lowers it afterwards.
static unsigned long long g_peer_wait_ns = 2000000000ull;
unsigned long long peer_wait_ns() { return g_peer_wait_ns; }

static EncodeTiledFn g_encode = nullptr;
static std::once_flag g_encode_once;

EncodeTiledFn encode_fn() {
  // cuTensorMapEncodeTiled is a driver call and wants a context current on the calling thread; a fresh thread (the
  // autograd worker) has none until its first runtime call, so make one here: cudaFree(nullptr) binds the primary
  // context of the thread's current device and does nothing else.
  static thread_local bool context_bound = false;
  if (!context_bound) {
    cudaFree(nullptr);
    context_bound = true;
  }
  std::call_once(g_encode_once, []() {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess) {
      fprintf(stderr, "[flame_b200] cuTensorMapEncodeTiled is not available from this driver\n");
      fn = nullptr;
    }
    g_encode = (EncodeTiledFn)fn;
  });
  return g_encode;
}

int make_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint64_t cols, uint64_t ld,
                 uint32_t box_rows, uint32_t box_cols, bool swizzle128) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * (uint64_t)elem_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr,
            "[flame_b200] tensor map 2d rejected (%d): base=%p rows=%llu cols=%llu ld=%llu box=%ux%u elem=%d\n", (int)r,
            base, (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)ld, box_rows, box_cols,
            elem_bytes);
    return (int)r;
  }
  return 0;
}

int make_tmap_3d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t d2, uint64_t d1, uint64_t d0,
                 uint64_t stride2, uint64_t stride1, uint32_t b2, uint32_t b1, uint32_t b0, int swizzle) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1 * (uint64_t)elem_bytes, stride2 * (uint64_t)elem_bytes};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = fn(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle == kSwizzle64 ? CU_TENSOR_MAP_SWIZZLE_64B : swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "[flame_b200] tensor map 3d rejected (%d): base=%p dims=%llu,%llu,%llu box=%u,%u,%u\n", (int)r, base,
            (unsigned long long)d2, (unsigned long long)d1, (unsigned long long)d0, b2, b1, b0);
    return (int)r;
  }
  return 0;
}

int make_tmap_4d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t d3, uint64_t d2, uint64_t d1, uint64_t d0,
                 uint64_t stride3, uint64_t stride2, uint64_t stride1, uint32_t b1, uint32_t b0, bool swizzle128) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[4] = {d0, d1, d2, d3};
  cuuint64_t strides[3] = {stride1 * (uint64_t)elem_bytes, stride2 * (uint64_t)elem_bytes, stride3 * (uint64_t)elem_bytes};
  cuuint32_t box[4] = {b0, b1, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = fn(out, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "[flame_b200] tensor map 4d rejected (%d): base=%p dims=%llu,%llu,%llu,%llu strides=%llu,%llu,%llu box=%u,%u\n",
            (int)r, base, (unsigned long long)d3, (unsigned long long)d2, (unsigned long long)d1, (unsigned long long)d0,
            (unsigned long long)stride3, (unsigned long long)stride2, (unsigned long long)stride1, b1, b0);
    return (int)r;
  }
  return 0;
}

}  // namespace fb

extern "C" {
// Returns the library status word (0 = ok; otherwise code << 16 | block index) without synchronising.
int fb_status_read() {
  int* p = fb::status_ptr();
  return p ? *(volatile int*)p : -1;
}
void fb_status_clear() {
  int* p = fb::status_ptr();
  if (p) *(volatile int*)p = 0;
}
// Sets the limit of every later wait on a flag raised by another GPU (seconds; values below 1 ms are raised to 1 ms).
void fb_set_peer_wait_seconds(double seconds) {
  if (seconds < 1e-3) seconds = 1e-3;
  fb::g_peer_wait_ns = (unsigned long long)(seconds * 1e9);
}
double fb_get_peer_wait_seconds() { return (double)fb::g_peer_wait_ns * 1e-9; }
}
