// Tensor-map cache, device status word and library-level C entry points.
#include "host_common.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace sb {

// One status word per device; kernels record the first bounded wait that gave up.
static __device__ int g_status_word;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

struct Key {
  uint64_t v[9];
  bool operator==(const Key& o) const { return std::memcmp(v, o.v, sizeof(v)) == 0; }
};
struct KeyHash {
  size_t operator()(const Key& k) const {
    uint64_t h = 1469598103934665603ull;
    for (uint64_t x : k.v) {
      h ^= x;
      h *= 1099511628211ull;
    }
    return static_cast<size_t>(h);
  }
};

static std::mutex g_mu;
static std::unordered_map<Key, CUtensorMap*, KeyHash> g_cache;

static const CUtensorMap* lookup_or_make(const Key& key, uint32_t rank, void* ptr, const cuuint64_t* dims,
                                         const cuuint64_t* strides, const cuuint32_t* box) {
  std::lock_guard<std::mutex> lock(g_mu);
  auto it = g_cache.find(key);
  if (it != g_cache.end()) return it->second;
  EncodeTiledFn fn = encode_fn();
  if (!fn) return nullptr;
  if (g_cache.size() > 16384) {
    // Entries are leaked on purpose when the cache is reset: launches that are
    // still being enqueued may hold pointers into it.
    g_cache.clear();
  }
  CUtensorMap* m = nullptr;
  if (posix_memalign(reinterpret_cast<void**>(&m), 64, sizeof(CUtensorMap)) != 0) return nullptr;
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, ptr, dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_ERROR_INVALID_CONTEXT) {
    // The driver entry point needs the primary context current on the calling thread; a thread that has made
    // no runtime call yet (an autograd worker thread, say) binds it here and retries.  Never reached while a
    // stream is capturing, because capture starts on a thread that has already launched work.
    cudaFree(nullptr);
    r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  if (r != CUDA_SUCCESS) {
    std::fprintf(stderr, "[skyrl_b200] cuTensorMapEncodeTiled failed: %d (rank %u ptr %p)\n", (int)r, rank, ptr);
    free(m);
    return nullptr;
  }
  g_cache.emplace(key, m);
  return m;
}

const CUtensorMap* get_tmap_bf16_2d(const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                                    uint32_t box_cols) {
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || ((ld * 2) & 15)) return nullptr;
  int dev = 0;
  cudaGetDevice(&dev);
  Key key{{reinterpret_cast<uint64_t>(ptr), rows, cols, ld, box_rows, box_cols, 2, (uint64_t)dev, 0}};
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  return lookup_or_make(key, 2, const_cast<void*>(ptr), dims, strides, box);
}

const CUtensorMap* get_tmap_bf16_3d(const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_bytes,
                                    uint64_t stride2_bytes, uint32_t box0, uint32_t box1, uint32_t box2) {
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (stride1_bytes & 15) || (stride2_bytes & 15)) return nullptr;
  int dev = 0;
  cudaGetDevice(&dev);
  Key key{{reinterpret_cast<uint64_t>(ptr), d0, d1, d2, stride1_bytes, stride2_bytes,
           (uint64_t)box0 | ((uint64_t)box1 << 20) | ((uint64_t)box2 << 40), (uint64_t)dev, 3}};
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {box0, box1, box2};
  return lookup_or_make(key, 3, const_cast<void*>(ptr), dims, strides, box);
}

int* device_status_ptr() {
  static int* ptrs[64] = {nullptr};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return nullptr;
  if (!ptrs[dev]) {
    int* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_status_word) != cudaSuccess) return nullptr;
    ptrs[dev] = p;
  }
  return ptrs[dev];
}

int device_index() {
  int dev = 0;
  cudaGetDevice(&dev);
  return dev < 0 ? 0 : (dev > 63 ? 63 : dev);
}

bool pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("SB_PDL");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

int sm_count() {
  static int counts[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 148;
  if (!counts[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    counts[dev] = n;
  }
  return counts[dev];
}

}  // namespace sb

extern "C" {

// Reads (and clears) the status word of the current device. Synchronises the device.
int sb_status_read_clear() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, sb::g_status_word, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) {
    int z = 0;
    cudaMemcpyToSymbol(sb::g_status_word, &z, sizeof(int));
  }
  return v;
}

int sb_sm_count() { return sb::sm_count(); }

const char* sb_version() { return "skyrl_b200-kernels sm_100a"; }

}  // extern "C"
