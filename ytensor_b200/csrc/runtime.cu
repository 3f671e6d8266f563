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
#include "ptx_sm100.cuh"

namespace ytk {

static thread_local char g_err[512] = {0};
static std::atomic<uint64_t> g_launches{0};
static std::atomic<uint64_t> g_h2d{0}, g_d2h{0};
void count_launch(uint64_t n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
bool& overlap_scope() {
  static thread_local bool on = false;
  return on;
}

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

// Scratch memory of the allocating entry points: one buffer per (device, stream), so that calls on different streams
// never share scratch. Growing is stream-ordered (cudaFreeAsync / cudaMallocAsync on the caller's stream): work
// already queued on the stream keeps the old buffer until it has run, and nothing synchronises the device.
struct WsKey {
  int dev;
  cudaStream_t st;
  bool operator==(const WsKey& o) const { return dev == o.dev && st == o.st; }
};
struct WsKeyHash {
  size_t operator()(const WsKey& k) const {
    return std::hash<uint64_t>()(reinterpret_cast<uint64_t>(k.st) * 31u + static_cast<uint64_t>(k.dev));
  }
};
struct WsBuf {
  void* ptr = nullptr;
  size_t cap = 0;
};
static std::unordered_map<WsKey, WsBuf, WsKeyHash> g_ws;
// Buffers above this size are handed back after the call that asked for them (device_workspace_release).
static constexpr size_t kWsKeep = 256u << 20;

void* device_workspace(size_t bytes, cudaStream_t st) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  WsBuf& b = g_ws[WsKey{dev, st}];
  if (b.cap < bytes) {
    if (b.ptr) {
      cudaFreeAsync(b.ptr, st);
      b.ptr = nullptr;
      b.cap = 0;
    }
    size_t cap = bytes < (1u << 20) ? (1u << 20) : bytes;
    if (cudaMallocAsync(&b.ptr, cap, st) != cudaSuccess) {
      b.ptr = nullptr;
      cudaGetLastError();
      return nullptr;
    }
    b.cap = cap;
  }
  return b.ptr;
}

void device_workspace_release(cudaStream_t st) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return;
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_ws.find(WsKey{dev, st});
  if (it == g_ws.end() || it->second.cap <= kWsKeep) return;
  cudaFreeAsync(it->second.ptr, st);  // stream-ordered: the kernels queued before this keep their scratch
  g_ws.erase(it);
}

// cudaFuncAttributeMaxDynamicSharedMemorySize belongs to (device, kernel): a process that uses several GPUs has to
// raise it on each of them, and a smaller request must never lower what another caller of the same kernel needs.
struct FnKey {
  int dev;
  const void* fn;
  bool operator==(const FnKey& o) const { return dev == o.dev && fn == o.fn; }
};
struct FnKeyHash {
  size_t operator()(const FnKey& k) const {
    return std::hash<uint64_t>()(reinterpret_cast<uint64_t>(k.fn) * 31u + static_cast<uint64_t>(k.dev));
  }
};
static std::unordered_map<FnKey, int, FnKeyHash> g_smem_limit;

int ensure_dynamic_smem(const void* fn, int bytes) {
  int dev = 0;
  YTC_CUDA(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lk(g_mu);
  int& cur = g_smem_limit[FnKey{dev, fn}];
  if (cur < bytes) {
    YTC_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    cur = bytes;
  }
  return YTC_OK;
}

// Cycle budget of the bounded device-side waits (mbarrier, grid and cross-GPU barriers), settable at run time.
static std::atomic<long long> g_wait_cycles{2000000000ll};
long long wait_cycle_limit() { return g_wait_cycles.load(std::memory_order_relaxed); }

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

// One CTA waits on an mbarrier that nothing ever arrives on, with the run-time cycle budget: the wait gives up,
// the kernel raises the device status word and returns. This is the give-up path of every bounded wait of the
// library (TMA / MMA / epilogue roles, grid and cross-GPU barriers) on its own, so that a test can watch it.
__global__ void wait_probe_kernel(int* status, long long limit, long long* waited) {
  __shared__ uint64_t bar;
  __shared__ int abort_word;
  if (threadIdx.x == 0) {
    abort_word = 0;
    mbar_init(&bar, 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const long long t0 = clock64();
    const bool ok = mbar_wait_limit(&bar, 0u, &abort_word, limit);
    if (waited) *waited = clock64() - t0;
    if (!ok) atomicExch(status, YTC_TIMEOUT);
  }
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
  g_h2d.fetch_add(1, std::memory_order_relaxed);
  YTC_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)));
  return YTC_OK;
}
int ytcuda_memcpy_d2h(void* dst, const void* src, uint64_t bytes, void* stream) {
  if (bytes == 0) return YTC_OK;
  YTC_REQUIRE(dst && src, "ytcuda_memcpy_d2h: null pointer");
  g_d2h.fetch_add(1, std::memory_order_relaxed);
  YTC_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)));
  return YTC_OK;
}
int ytcuda_memcpy_d2d(void* dst, const void* src, uint64_t bytes, void* stream) {
  if (bytes == 0) return YTC_OK;
  YTC_REQUIRE(dst && src, "ytcuda_memcpy_d2d: null pointer");
  YTC_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream)));
  return YTC_OK;
}
int ytcuda_pointer_is_device(const void* p) {
  if (!p) return 0;
  cudaPointerAttributes a;
  if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return (a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged) ? 1 : 0;
}
int ytcuda_stream_sync(void* stream) {
  YTC_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  return YTC_OK;
}
int ytcuda_device_status(void* stream) { return read_device_status(static_cast<cudaStream_t>(stream)); }
uint64_t ytcuda_launch_count(void) { return g_launches.load(); }
void ytcuda_copy_counts(uint64_t* h2d, uint64_t* d2h) {
  if (h2d) *h2d = g_h2d.load();
  if (d2h) *d2h = g_d2h.load();
}
int ytcuda_set_wait_limit(int64_t cycles) {
  YTC_REQUIRE(cycles > 0, "ytcuda_set_wait_limit: the limit must be positive");
  g_wait_cycles.store(cycles, std::memory_order_relaxed);
  return YTC_OK;
}
int64_t ytcuda_get_wait_limit(void) { return g_wait_cycles.load(std::memory_order_relaxed); }
int ytcuda_wait_probe(int64_t* waited_cycles_dev, void* stream) {
  int* status = device_status_word();
  YTC_REQUIRE(status != nullptr, "ytcuda_wait_probe: no device status word");
  wait_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status, wait_cycle_limit(),
                                                                    reinterpret_cast<long long*>(waited_cycles_dev));
  count_launch();
  YTC_CUDA(cudaGetLastError());
  return YTC_OK;
}

}  // extern "C"
