/* C ABI of libytensor_cuda.so: the sm_100a device backend for YTensor's dense hot path.
 *
 * Every entry point takes plain pointers and sizes, returns a ytc_status and never
 * falls back to the CPU. Unless stated otherwise pointers are DEVICE pointers,
 * strides are in ELEMENTS, `stream` is a cudaStream_t (NULL = default stream) and the
 * call is asynchronous on that stream. Empty problems (a zero extent) succeed without
 * a launch, as the reference's kernels return silently on empty dims
 * (src/kernel/avx2/sgemm.inl:594, src/kernel/avx2/flash_attention.inl:298-300).
 * Each declaration cites the reference interface it replaces (path within the
 * reference project : line).
 */
#ifndef YTCUDA_H_
#define YTCUDA_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  YTC_OK = 0,
  YTC_INVALID_ARG = 1,     /* maps to std::invalid_argument in the C++ layer */
  YTC_UNSUPPORTED = 2,     /* valid request the device backend has no kernel for: throws, no CPU fallback */
  YTC_CUDA_ERROR = 3,      /* maps to std::runtime_error */
  YTC_TIMEOUT = 4,         /* a bounded device-side wait ran out */
  YTC_NOT_IMPLEMENTED = 5
} ytc_status;

/* Element types, named like the reference's dtype strings (include/ytensor_types.hpp:125-153). */
typedef enum { YTC_F32 = 0, YTC_BF16 = 1, YTC_F16 = 2 } ytc_dtype;

/* ---------------------------------------------------------------- utilities */
/* Text of the last error raised on the calling thread ("" if none). */
const char* ytcuda_last_error_string(void);
/* Device / pinned-host storage for YTensor's shared_ptr<char[]> deleter hook
 * (reference include/ytensor_base.hpp:388-393 owns storage; src/ytensor_base.inl:51-58 custom deleters). */
int ytcuda_malloc(void** dptr, uint64_t bytes);
int ytcuda_free(void* dptr);
int ytcuda_host_alloc(void** hptr, uint64_t bytes);
int ytcuda_host_free(void* hptr);
int ytcuda_memcpy_h2d(void* dst, const void* src, uint64_t bytes, void* stream);
int ytcuda_memcpy_d2h(void* dst, const void* src, uint64_t bytes, void* stream);
int ytcuda_stream_sync(void* stream);
/* Reads and clears the device status word that kernels with bounded waits write
 * (YTC_OK or YTC_TIMEOUT). Synchronises `stream`. */
int ytcuda_device_status(void* stream);
/* Number of kernels this library has launched in the calling process. */
uint64_t ytcuda_launch_count(void);

/* ---------------------------------------------------------------- GEMM
 * C[b] = alpha * A[b] . B[b] + beta * C[b],  A [m,k], B [k,n], C [m,n], b in [0,batch).
 * Replaces yt::kernel::avx2::sgemm / matmul (include/kernel/avx2/sgemm.hpp:51-63) and
 * hgemm / hmatmul (include/kernel/avx2/hgemm.hpp:26-40), plus the per-matrix loop of
 * YTensor::matmul (src/ytensor_math.inl:954-1051) through `batch` and the batch strides
 * (0 = the operand is shared by every batch item, as a 2-D right operand is at :960-1018).
 * dtype_in in {F32, BF16, F16}; accumulation is fp32; C is rounded to dtype_out with the
 * reference's own conversion (yt::bfloat16 / yt::float16 constructors).
 * BF16/F16 inputs run on tcgen05 when each operand has a unit stride along one of its two
 * axes and 16-byte aligned rows; every other layout, and F32, runs on the FFMA kernel. */
int ytcuda_gemm(int dtype_in, int dtype_out, const void* A, const void* B, void* C, int m, int n, int k,
                float alpha, float beta, int64_t rsa, int64_t csa, int64_t rsb, int64_t csb, int64_t rsc,
                int64_t csc, int64_t batch, int64_t bsa, int64_t bsb, int64_t bsc, void* stream);

/* Kernel choice of ytcuda_gemm for 16-bit inputs: 0 = automatic (default), 1 = always the FFMA
 * kernel, 2 = tcgen05 or YTC_UNSUPPORTED. The counterpart of the per-call `backend` argument of
 * YTensor::matmul (include/ytensor_math.hpp:70-73); process-wide, meant for tests. */
int ytcuda_gemm_set_path(int path);

/* Same computation with HOST buffers (pinned or pageable): copies A and B to the device,
 * multiplies, copies C back, and returns when C is complete. Batch items are pipelined so
 * that copies overlap the multiplication. This is what a YTensor that lives in host memory
 * calls (the reference's tensors always do, include/ytensor_base.hpp:388). */
int ytcuda_gemm_host(int dtype_in, int dtype_out, const void* A, const void* B, void* C, int m, int n, int k,
                     float alpha, float beta, int64_t rsa, int64_t csa, int64_t rsb, int64_t csb, int64_t rsc,
                     int64_t csc, int64_t batch, int64_t bsa, int64_t bsb, int64_t bsc);

#ifdef __cplusplus
}
#endif
#endif /* YTCUDA_H_ */
