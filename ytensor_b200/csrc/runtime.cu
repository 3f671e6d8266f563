// Host-side plumbing of libytensor_cuda.so: error text, storage helpers, the device
// status word, the tensor-map encoder and a small per-device workspace.
#include <mutex>
#include <unordered_map>
#include <cstring>
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <mutex>

#include "ytc_common.cuh"

namespace ytk {

static thread_local char g_err[512] = {0};
static std::atomic<uint64_t> g_launches{0};
void count_launch(uint64_t n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

void set_last_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return YTC_OK;
  set_last_error("CUDA error %d (%s) in %s", static_cast<int>(e), cudaGetErrorString(e), what);
  return YTC_CUDA_ERROR;
}

static constexpr int kMaxDev = 16;

int sm_count() {
  static int cached[kMaxDev] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

static std::mutex g_mu;
static int* g_status[kMaxDev] = {nullptr};

int* device_status_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_status[dev]) {
    int* p = nullptr;
    if (cudaMalloc(&p, 256) != cudaSuccess) return nullptr;
    if (cudaMemset(p, 0, 256) != cudaSuccess) return nullptr;
    g_status[dev] = p;
  }
  return g_status[dev];
}

int read_device_status(cudaStream_t st) {
  int* w = device_status_word();
  if (!w) {
    set_last_error("no device status word (no CUDA device?)");
    return YTC_CUDA_ERROR;
  }
  int h = 0;
  YTC_CUDA(cudaMemcpyAsync(&h, w, sizeof(int), cudaMemcpyDeviceToHost, st));
  YTC_CUDA(cudaStreamSynchronize(st));
  if (h != 0) {
    YTC_CUDA(cudaMemsetAsync(w, 0, sizeof(int), st));
    set_last_error("a device-side bounded wait ran out (status %d)", h);
  }
  return h;
}

static void* g_ws[kMaxDev] = {nullptr};
static size_t g_ws_cap[kMaxDev] = {0};

void* device_workspace(size_t bytes) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_ws_cap[dev] < bytes) {
    if (g_ws[dev]) {
      cudaDeviceSynchronize();
      cudaFree(g_ws[dev]);
      g_ws[dev] = nullptr;
      g_ws_cap[dev] = 0;
    }
    size_t cap = bytes < (1u << 20) ? (1u << 20) : bytes;
    if (cudaMalloc(&g_ws[dev], cap) != cudaSuccess) return nullptr;
    g_ws_cap[dev] = cap;
  }
  return g_ws[dev];
}

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

// A tensor map is a pure function of its arguments (address, extents, strides, box, type, swizzle) and encoding one
// costs the host a microsecond or more; launch-bound loops (a decode step issues hundreds of GEMMs over the same
// buffers) get them from this small cache instead.
struct MapKey {
  uint64_t v[16];
  bool operator==(const MapKey& o) const { return std::memcmp(v, o.v, sizeof(v)) == 0; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t h = 1469598103934665603ull;
    for (uint64_t x : k.v) {
      h ^= x;
      h *= 1099511628211ull;
    }
    return static_cast<size_t>(h);
  }
};
static std::mutex g_map_mutex;
static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_map_cache;

int encode_tensor_map(CUtensorMap* map, CUtensorMapDataType dt, uint32_t rank, const void* base,
                      const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                      CUtensorMapSwizzle swz) {
  MapKey key{};
  if (rank <= 4) {
    key.v[0] = reinterpret_cast<uint64_t>(base);
    key.v[1] = (static_cast<uint64_t>(dt) << 32) | (static_cast<uint64_t>(swz) << 8) | rank;
    for (uint32_t i = 0; i < rank; ++i) {
      key.v[2 + i] = dims[i];
      key.v[6 + i] = i + 1 < rank ? strides_bytes[i] : 0;
      key.v[10 + i] = box[i];
    }
    std::lock_guard<std::mutex> lock(g_map_mutex);
    auto it = g_map_cache.find(key);
    if (it != g_map_cache.end()) {
      *map = it->second;
      return YTC_OK;
    }
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    set_last_error("cuTensorMapEncodeTiled is not available from this driver");
    return YTC_CUDA_ERROR;
  }
  cuuint64_t gdim[5];
  cuuint64_t gstr[5];
  cuuint32_t bx[5];
  cuuint32_t es[5];
  for (uint32_t i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
    if (i + 1 < rank) gstr[i] = strides_bytes[i];  // stride of dim i+1
  }
  CUresult r = fn(map, dt, rank, const_cast<void*>(base), gdim, gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("cuTensorMapEncodeTiled failed with %d (rank %u, dims %llu %llu %llu, strides %llu %llu, box %u %u %u)",
                   static_cast<int>(r), rank, (unsigned long long)dims[0], (unsigned long long)(rank > 1 ? dims[1] : 0),
                   (unsigned long long)(rank > 2 ? dims[2] : 0), (unsigned long long)(rank > 1 ? strides_bytes[0] : 0),
                   (unsigned long long)(rank > 2 ? strides_bytes[1] : 0), box[0], rank > 1 ? box[1] : 0,
                   rank > 2 ? box[2] : 0);
    return YTC_INVALID_ARG;
  }
  if (rank <= 4) {
    std::lock_guard<std::mutex> lock(g_map_mutex);
    if (g_map_cache.size() >= 8192) g_map_cache.clear();
    g_map_cache.emplace(key, *map);
  }
  return YTC_OK;
}

}  // namespace ytk

using namespace ytk;

extern "C" {

const char* ytcuda_last_error_string(void) { return g_err; }

int ytcuda_malloc(void** dptr, uint64_t bytes) {
  YTC_REQUIRE(dptr != nullptr, "ytcuda_malloc: null output pointer");
  *dptr = nullptr;
  if (bytes == 0) return YTC_OK;
  YTC_CUDA(cudaMalloc(dptr, bytes));
  return YTC_OK;
}
int ytcuda_free(void* dptr) {
  if (!dptr) return YTC_OK;
  YTC_CUDA(cudaFree(dptr));
  return YTC_OK;
}
int ytcuda_host_alloc(void** hptr, uint64_t bytes) {
  YTC_REQUIRE(hptr != nullptr, "ytcuda_host_alloc: null output pointer");
  *hptr = nullptr;
  if (bytes == 0) return YTC_OK;
  YTC_CUDA(cudaHostAlloc(hptr, bytes, cudaHostAllocDefault));
  return YTC_OK;
}
int ytcuda_host_free(void* hptr) {
  if (!hptr) return YTC_OK;
  YTC_CUDA(cudaFreeHost(hptr));
  return YTC_OK;
}
int ytcuda_memcpy_h2d(void* dst, const void* src, uint64_t bytes, void* stream) {
  if (bytes == 0) return YTC_OK;
  YTC_REQUIRE(dst && src, "ytcuda_memcpy_h2d: null pointer");
  YTC_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)));
  return YTC_OK;
}
int ytcuda_memcpy_d2h(void* dst, const void* src, uint64_t bytes, void* stream) {
  if (bytes == 0) return YTC_OK;
  YTC_REQUIRE(dst && src, "ytcuda_memcpy_d2h: null pointer");
  YTC_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)));
  return YTC_OK;
}
int ytcuda_stream_sync(void* stream) {
  YTC_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  return YTC_OK;
}
int ytcuda_device_status(void* stream) { return read_device_status(static_cast<cudaStream_t>(stream)); }
uint64_t ytcuda_launch_count(void) { return g_launches.load(); }

}  // extern "C"
