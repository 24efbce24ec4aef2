// Host-side support shared by all entry points: error string, TMA descriptor
// construction through the driver entry point (no link-time libcuda dependency),
// device queries.
#include "tt_common.cuh"
#include <stdarg.h>
#include <atomic>
#include <mutex>
#include <unordered_map>

static thread_local char g_err[1024] = "";

void tt_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

TT_API const char* tt_last_error() { return g_err; }

static std::atomic<long long> g_launches{0};
void tt_count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
// Number of kernels this library has launched in this process.
TT_API long long tt_launch_count() { return g_launches.load(std::memory_order_relaxed); }

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
    if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) fn = (EncodeTiledFn)p;
  });
  return fn;
}

// Descriptors are pure functions of their arguments (a descriptor holds an address, not a device), so they are kept
// by (address, element size, rank, extents, strides, box, swizzle): a training step launches the same few hundred
// GEMM / attention shapes on the same buffers again and again, and the driver call costs microseconds of host time.
namespace {
struct TmapKey {
  uint64_t w[16];
  bool operator==(const TmapKey& o) const { return memcmp(w, o.w, sizeof(w)) == 0; }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    uint64_t h = 1469598103934665603ull;
    for (uint64_t x : k.w) {
      h ^= x;
      h *= 1099511628211ull;
    }
    return (size_t)h;
  }
};
std::mutex g_tmap_mu;
std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> g_tmaps;
constexpr size_t TMAP_CACHE_MAX = 1 << 16;   // cleared when full; an entry never goes stale (same arguments, same descriptor)
}  // namespace

TT_API long long tt_tmap_cache_size() {
  std::lock_guard<std::mutex> lk(g_tmap_mu);
  return (long long)g_tmaps.size();
}

int tt_make_tmap(CUtensorMap* out, const void* base, int elem_bytes, int rank, const uint64_t* dims,
                 const uint64_t* strides_bytes, const uint32_t* box, int swizzle128) {
  TT_CHECK(rank >= 1 && rank <= 5, "TMA rank %d out of range", rank);
  TmapKey key;
  memset(&key, 0, sizeof(key));
  key.w[0] = (uint64_t)(uintptr_t)base;
  key.w[1] = (uint64_t)elem_bytes | ((uint64_t)rank << 8) | ((uint64_t)(swizzle128 != 0) << 16);
  for (int i = 0; i < rank; ++i) {
    key.w[2 + i] = dims[i];
    key.w[7 + i] = (i + 1 < rank) ? strides_bytes[i] : 0;
    key.w[12 + i / 2] |= (uint64_t)box[i] << (32 * (i & 1));
  }
  {
    std::lock_guard<std::mutex> lk(g_tmap_mu);
    auto it = g_tmaps.find(key);
    if (it != g_tmaps.end()) {
      *out = it->second;
      return 0;
    }
  }
  EncodeTiledFn enc = get_encode();
  TT_CHECK(enc != nullptr, "cuTensorMapEncodeTiled entry point not available");
  TT_CHECK(((uintptr_t)base & 15) == 0, "TMA base address %p is not 16-byte aligned", base);
  cuuint64_t gdim[5];
  cuuint64_t gstr[5];
  cuuint32_t bx[5];
  cuuint32_t es[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
    if (i + 1 < rank) {
      gstr[i] = strides_bytes[i];
      TT_CHECK((gstr[i] & 15) == 0, "TMA stride %llu of dim %d is not a multiple of 16 bytes",
               (unsigned long long)gstr[i], i + 1);
    }
  }
  TT_CHECK(((uint64_t)box[0] * elem_bytes) % 16 == 0, "TMA inner box extent must cover 16-byte units");
  CUtensorMapDataType dt = elem_bytes == 2   ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                             : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = enc(out, dt, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, bx, es,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TT_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  {
    std::lock_guard<std::mutex> lk(g_tmap_mu);
    if (g_tmaps.size() >= TMAP_CACHE_MAX) g_tmaps.clear();
    g_tmaps.emplace(key, *out);
  }
  return 0;
}

TT_API int tt_num_sms() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
  return n;
}

TT_API int tt_abi_version() { return 1; }
