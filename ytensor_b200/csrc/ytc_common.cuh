// Shared host/device helpers of the YTensor CUDA backend: status codes, dtype
// tags, the reference's scalar conversion rules and small launch utilities.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "../../include/ytcuda.h"

namespace ytk {

// ---- scalar conversions that follow the reference's own types ---------------
// yt::bfloat16(float) (reference include/types/bfloat16.hpp:78-80): adds half an
// ulp only when the kept LSB is 1, then truncates. No NaN/Inf special case.
__host__ __device__ __forceinline__ uint16_t f32_to_bf16_bits_ref(float x) {
#ifdef __CUDA_ARCH__
  uint32_t u = __float_as_uint(x);
#else
  uint32_t u;
  memcpy(&u, &x, 4);
#endif
  return static_cast<uint16_t>((u + ((u & 0x00010000u) >> 1)) >> 16);
}
__host__ __device__ __forceinline__ float bf16_bits_to_f32(uint16_t b) {
  uint32_t u = static_cast<uint32_t>(b) << 16;
#ifdef __CUDA_ARCH__
  return __uint_as_float(u);
#else
  float f;
  memcpy(&f, &u, 4);
  return f;
#endif
}

// yt::float16 = FloatSpec<1,5,10>, float -> half (reference
// include/types/float_spec.hpp:435-491): fp32 zero/subnormal -> signed zero; Inf -> Inf;
// NaN -> exponent all ones with mantissa 1; a result whose biased half exponent would be
// <= 0 is flushed to signed zero BEFORE rounding; otherwise round-to-nearest-even on the
// 13 dropped bits with carry into the exponent and overflow to infinity.
__host__ __device__ __forceinline__ uint16_t f32_to_f16_bits_ref(float x) {
#ifdef __CUDA_ARCH__
  uint32_t bits = __float_as_uint(x);
#else
  uint32_t bits;
  memcpy(&bits, &x, 4);
#endif
  const uint32_t s = bits >> 31, e = (bits >> 23) & 0xFFu, m = bits & 0x7FFFFFu;
  uint32_t ne = 0, nm = 0;
  if (e == 0) {
  } else if (e == 0xFFu) {
    ne = 31;
    nm = m ? 1u : 0u;
  } else {
    const int re = static_cast<int>(e) - 127 + 15;
    if (re <= 0) {
    } else if (re >= 31) {
      ne = 31;
    } else {
      ne = static_cast<uint32_t>(re);
      nm = m >> 13;
      const uint32_t rem = m & 0x1FFFu;
      if (rem > 0x1000u || (rem == 0x1000u && (nm & 1u))) {
        ++nm;
        if (nm >= 1024u) {
          nm = 0;
          ++ne;
          if (ne >= 31u) ne = 31u;
        }
      }
    }
  }
  return static_cast<uint16_t>((s << 15) | (ne << 10) | nm);
}
// half -> float of the same type (reference include/types/float_spec.hpp:299-371, toFloat32).
// Normal numbers widen exactly; Inf stays Inf; NaN becomes 0x7F800001 with the sign kept.
// A subnormal encoding (exponent 0, mantissa m != 0) is normalised by the reference with the
// exponent set to 1 - shift, where shift is the number of left shifts that bring the leading
// one to mantissa bit 9: the value read is twice m * 2^-24. That is followed here bit for bit.
__host__ __device__ __forceinline__ float f16_bits_to_f32_ref(uint16_t h) {
  const uint32_t s = (h >> 15) & 1u, e = (h >> 10) & 0x1Fu;
  uint32_t m = h & 0x3FFu;
  uint32_t out;
  if (e == 0) {
    if (m == 0) {
      out = s << 31;
    } else {
      uint32_t shift = 0;
      while ((m & 0x200u) == 0 && shift < 10) {
        m <<= 1;
        ++shift;
      }
      m = (m << 1) & 0x3FFu;
      out = (s << 31) | ((113u - shift) << 23) | (m << 13);
    }
  } else if (e == 31u) {
    out = (s << 31) | 0x7F800000u | (m ? 1u : 0u);
  } else {
    out = (s << 31) | ((e + 112u) << 23) | (m << 13);
  }
#ifdef __CUDA_ARCH__
  return __uint_as_float(out);
#else
  float f;
  memcpy(&f, &out, 4);
  return f;
#endif
}

// The reference's generic small float FloatSpec<S, E, M> (include/types/float_spec.hpp): float -> spec (fromFloat32,
// :435-491) and spec -> float (toFloat32, :299-371), the same rules as the float16 functions above for any sign /
// exponent / mantissa widths with M <= 23: zero and fp32 subnormals -> signed zero; Inf / NaN -> exponent all ones,
// mantissa 1 for NaN; biased exponent <= 0 flushes to zero; >= all ones overflows to infinity; otherwise round to
// nearest even with carry into the exponent. An unsigned format (S = 0) drops the sign.
template <int S, int E, int M>
__host__ __device__ __forceinline__ uint32_t f32_to_spec_bits(float x) {
#ifdef __CUDA_ARCH__
  uint32_t bits = __float_as_uint(x);
#else
  uint32_t bits;
  memcpy(&bits, &x, 4);
#endif
  constexpr int bias = (1 << (E - 1)) - 1;
  constexpr uint32_t emax = (1u << E) - 1u;
  const uint32_t s = S ? (bits >> 31) : 0u, e = (bits >> 23) & 0xFFu, m = bits & 0x7FFFFFu;
  uint32_t ne = 0, nm = 0;
  if (e == 0) {
  } else if (e == 0xFFu) {
    ne = emax;
    nm = m ? 1u : 0u;
  } else {
    const int re = static_cast<int>(e) - 127 + bias;
    if (re <= 0) {
    } else if (re >= static_cast<int>(emax)) {
      ne = emax;
    } else {
      ne = static_cast<uint32_t>(re);
      nm = m >> (23 - M);
      const uint32_t rem = m & ((1u << (23 - M)) - 1u), half = 1u << (22 - M);
      if (rem > half || (rem == half && (nm & 1u))) {
        ++nm;
        if (nm >= (1u << M)) {
          nm = 0;
          ++ne;
          if (ne >= emax) ne = emax;
        }
      }
    }
  }
  return (s << (E + M)) | (ne << M) | nm;
}
template <int S, int E, int M>
__host__ __device__ __forceinline__ float spec_bits_to_f32(uint32_t h) {
  constexpr int bias = (1 << (E - 1)) - 1;
  constexpr uint32_t emax = (1u << E) - 1u, mmask = (1u << M) - 1u;
  const uint32_t s = S ? ((h >> (E + M)) & 1u) : 0u;
  const uint32_t e = (h >> M) & emax;
  uint32_t m = h & mmask;
  uint32_t out;
  if (e == 0) {
    if (m == 0 || M == 0) {
      out = s << 31;
    } else {
      // a subnormal encoding: normalised with the exponent set to 1 - shift (twice the IEEE value; followed as is)
      int shift = 0;
      while ((m & (1u << (M > 0 ? M - 1 : 0))) == 0 && shift < M) {
        m <<= 1;
        ++shift;
      }
      m = (m << 1) & mmask;
      const int ne = 1 - shift - bias + 127;
      out = ne <= 0 ? ((s << 31) | (m << (23 - M))) : ((s << 31) | (static_cast<uint32_t>(ne) << 23) | (m << (23 - M)));
    }
  } else if (e == emax) {
    out = (s << 31) | 0x7F800000u | (m ? 1u : 0u);
  } else {
    const int ne = static_cast<int>(e) - bias + 127;
    if (ne <= 0) out = s << 31;
    else if (ne >= 255) out = (s << 31) | 0x7F800000u;
    else out = (s << 31) | (static_cast<uint32_t>(ne) << 23) | (m << (23 - M));
  }
#ifdef __CUDA_ARCH__
  return __uint_as_float(out);
#else
  float f;
  memcpy(&f, &out, 4);
  return f;
#endif
}

template <int DT>
struct DType;
template <>
struct DType<YTC_F32> {
  using storage = float;
  __device__ static __forceinline__ float load(const void* p, int64_t i) { return static_cast<const float*>(p)[i]; }
  __device__ static __forceinline__ void store(void* p, int64_t i, float v) { static_cast<float*>(p)[i] = v; }
};
template <>
struct DType<YTC_BF16> {
  using storage = uint16_t;
  __device__ static __forceinline__ float load(const void* p, int64_t i) {
    return bf16_bits_to_f32(static_cast<const uint16_t*>(p)[i]);
  }
  __device__ static __forceinline__ void store(void* p, int64_t i, float v) {
    static_cast<uint16_t*>(p)[i] = f32_to_bf16_bits_ref(v);
  }
};
template <>
struct DType<YTC_F16> {
  using storage = uint16_t;
  __device__ static __forceinline__ float load(const void* p, int64_t i) {
    return f16_bits_to_f32_ref(static_cast<const uint16_t*>(p)[i]);
  }
  __device__ static __forceinline__ void store(void* p, int64_t i, float v) {
    static_cast<uint16_t*>(p)[i] = f32_to_f16_bits_ref(v);
  }
};

__host__ __device__ __forceinline__ int dtype_size(int dt) { return dt == YTC_F32 ? 4 : (dt >= YTC_F8_E5M2 ? 1 : 2); }

__device__ __forceinline__ float f8_bits_to_f32(uint8_t b, int dt) {
  if (dt == YTC_F8_E5M2) return spec_bits_to_f32<1, 5, 2>(b);
  if (dt == YTC_F8_E4M3) return spec_bits_to_f32<1, 4, 3>(b);
  return spec_bits_to_f32<0, 8, 0>(b);
}
__device__ __forceinline__ uint8_t f32_to_f8_bits(float v, int dt) {
  if (dt == YTC_F8_E5M2) return static_cast<uint8_t>(f32_to_spec_bits<1, 5, 2>(v));
  if (dt == YTC_F8_E4M3) return static_cast<uint8_t>(f32_to_spec_bits<1, 4, 3>(v));
  return static_cast<uint8_t>(f32_to_spec_bits<0, 8, 0>(v));
}

__device__ __forceinline__ float load_as_f32(const void* p, int64_t i, int dt) {
  if (dt == YTC_F32) return DType<YTC_F32>::load(p, i);
  if (dt == YTC_BF16) return DType<YTC_BF16>::load(p, i);
  if (dt == YTC_F16) return DType<YTC_F16>::load(p, i);
  return f8_bits_to_f32(static_cast<const uint8_t*>(p)[i], dt);
}
__device__ __forceinline__ void store_from_f32(void* p, int64_t i, float v, int dt) {
  if (dt == YTC_F32) DType<YTC_F32>::store(p, i, v);
  else if (dt == YTC_BF16) DType<YTC_BF16>::store(p, i, v);
  else if (dt == YTC_F16) DType<YTC_F16>::store(p, i, v);
  else static_cast<uint8_t*>(p)[i] = f32_to_f8_bits(v, dt);
}

// ---- host-side plumbing -------------------------------------------------------
// Counts kernel launches of this library (reported by ytcuda_launch_count).
void count_launch(uint64_t n = 1);
void set_last_error(const char* fmt, ...);
int check_cuda(cudaError_t e, const char* what);
int sm_count();
// Device word that kernels with bounded waits write a status into (0 = fine).
int* device_status_word();
// Reads and clears the device status word (synchronises the stream).
int read_device_status(cudaStream_t st);

// Scratch buffer owned by the library, one per (device, stream), grown on demand with stream-ordered allocation:
// calls on different streams never share scratch, calls on one stream are ordered by the stream itself.
void* device_workspace(size_t bytes, cudaStream_t st);
// Hands a buffer above 256 MiB back (stream-ordered) once the kernels using it have been queued; smaller ones stay.
void device_workspace_release(cudaStream_t st);
// Raises the dynamic shared-memory limit of `fn` on the current device to at least `bytes` (once per device).
int ensure_dynamic_smem(const void* fn, int bytes);
// Cycle budget of bounded device-side waits (ytcuda_set_wait_limit).
long long wait_cycle_limit();

// Programmatic dependent launch. A kernel launched through launch_overlapped while overlap_scope() is on may start
// (be scheduled, run its set-up) while the kernel before it in the stream is still running; it calls
// dependent_wait() before it touches any global memory, which returns once that kernel has finished and its writes are
// visible. A kernel that calls dependent_trigger() lets the next one be scheduled from that point on. Both calls do
// nothing in a kernel launched the ordinary way.
bool& overlap_scope();  // thread-local switch, set by callers that queue a chain of dependent launches
#ifdef __CUDACC__
__device__ __forceinline__ void dependent_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void dependent_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
template <typename... KArgs, typename... Args>
cudaError_t launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = overlap_scope() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

// cuTensorMapEncodeTiled through the runtime's driver entry point lookup, so that
// the library has no link-time dependency on libcuda.
int encode_tensor_map(CUtensorMap* map, CUtensorMapDataType dt, uint32_t rank, const void* base,
                      const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                      CUtensorMapSwizzle swz);

#define YTC_REQUIRE(cond, ...)        \
  do {                                \
    if (!(cond)) {                    \
      ytk::set_last_error(__VA_ARGS__); \
      return YTC_INVALID_ARG;         \
    }                                 \
  } while (0)

#define YTC_CUDA(expr)                               \
  do {                                               \
    int _s = ytk::check_cuda((expr), #expr);         \
    if (_s != YTC_OK) return _s;                     \
  } while (0)

}  // namespace ytk
