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
typedef enum {
  YTC_F32 = 0,
  YTC_BF16 = 1,
  YTC_F16 = 2,
  /* 8-bit storage types (yt::float8_e5m2 / float8_e4m3 / float8_e8m0, include/types/float_spec.hpp:534-536): accepted
   * by ytcuda_cast only. They follow the reference's generic FloatSpec rules, not the OCP "fn" variants: the largest
   * exponent is infinity / NaN in every format, results below the smallest normal flush to zero, e8m0 has no sign. */
  YTC_F8_E5M2 = 3,
  YTC_F8_E4M3 = 4,
  YTC_F8_E8M0 = 5
} ytc_dtype;

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
int ytcuda_memcpy_d2d(void* dst, const void* src, uint64_t bytes, void* stream);
int ytcuda_stream_sync(void* stream);
/* 1 when `p` points into device memory (storage from ytcuda_malloc), 0 for host memory, pinned or pageable. The C++
 * layer asks this to tell a device-resident YTensor from a host-resident one: the reference's tensor carries no
 * residency tag (include/ytensor_base.hpp:388-393), only its storage pointer. */
int ytcuda_pointer_is_device(const void* p);
/* Reads and clears the device status word that kernels with bounded waits write
 * (YTC_OK or YTC_TIMEOUT). Synchronises `stream`. */
int ytcuda_device_status(void* stream);
/* Number of kernels this library has launched in the calling process. */
uint64_t ytcuda_launch_count(void);
/* Number of ytcuda_memcpy_h2d / ytcuda_memcpy_d2h calls made by the calling process: lets a caller check that a chain
 * of operators on device-resident tensors crossed PCIe only where it meant to. */
void ytcuda_copy_counts(uint64_t* h2d, uint64_t* d2h);
/* Cycle budget of the bounded device-side waits of the decode step kernel (grid barriers, barriers across
 * tensor-parallel ranks) and of ytcuda_wait_probe; the default, 2e9 cycles, is about a second. A wait that runs out
 * makes its kernel return and ytcuda_device_status report YTC_TIMEOUT. Process-wide. The TMA / MMA pipelines of the
 * GEMM and attention kernels keep their compiled-in budget. No counterpart in the reference (its kernels have no
 * waits). */
int ytcuda_set_wait_limit(int64_t cycles);
int64_t ytcuda_get_wait_limit(void);
/* Launches one small kernel that waits on an mbarrier nothing arrives on, with the current cycle budget: the wait gives
 * up, the kernel returns, ytcuda_device_status reports YTC_TIMEOUT once and the device stays usable. The give-up path
 * of the library's bounded waits in isolation, for tests and health checks. waited_cycles_dev (device pointer, may be
 * NULL) receives the cycles spent. No counterpart in the reference. */
int ytcuda_wait_probe(int64_t* waited_cycles_dev, void* stream);

/* Scratch memory. The entry points that need scratch beyond their inputs and outputs (fp32 GEMM on the tensor cores,
 * long reductions, attention over a KV cache split over keys, the decoder's split-k linears) take it from a buffer the
 * library keeps per (device, stream), grown with stream-ordered allocation on the caller's stream: calls on different
 * streams never share scratch, and growing does not synchronise the device. Such a call may therefore allocate; make
 * the first call of each kind outside any stream capture. ytcuda_reduce_noalloc is the form that never allocates. */

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
/* fp32 products (sgemm, include/kernel/avx2/sgemm.hpp:51-63) on the tensor cores: each operand is split into three
 * bfloat16 planes (24 mantissa bits) and the six partial products that matter at fp32 precision are laid side by
 * side along k and accumulated in fp32 by one bf16 GEMM. Every finite input is represented exactly (values next to
 * the largest float included). One deviation from sgemm: an INFINITE operand gives NaN in the outputs it reaches
 * (its top plane meets zero or opposite-signed lower planes of the other operand) where sgemm gives the infinity;
 * NaN inputs give NaN in both. Callers that rely on infinities select mode 1.
 * 0 = automatic (m, n, k >= 256 with n and k multiples of 8), 1 = never (FFMA kernel), 2 = whenever n and k
 * are multiples of 8. Process-wide, meant for tests; no counterpart in the reference. */
int ytcuda_gemm_set_f32_mode(int mode);

/* Tuning knobs of the tcgen05 kernel. a_prefetch_kblocks: how many 64-wide k-blocks an L2 prefetch of the
 * streamed A operand runs ahead of the shared-memory ring (0 = off, the default: it measured slower).
 * split_loads: fetch K-major operand tiles as 64-row TMA boxes instead of one tall box (default 0).
 * The counterpart of the reference's runtime blocking globals g_gemm_mc/kc/nc and their setters
 * (include/kernel/avx2/gemm_utils.hpp:59-77). */
int ytcuda_gemm_set_tuning(int a_prefetch_kblocks, int split_loads);

/* Use of the CTA-pair (cta_group::2, 256 x 256 tile per two SMs) form of the tcgen05 kernel: 0 = automatic (large
 * problems), 1 = whenever the operands qualify, 2 = never. Process-wide, meant for tests and measurements; the
 * counterpart of the reference's per-call backend choice (include/ytensor_math.hpp:70-73). */
int ytcuda_gemm_set_pair_mode(int mode);

/* Same computation with HOST buffers (pinned or pageable): copies A and B to the device,
 * multiplies, copies C back, and returns when C is complete. Batch items are pipelined so
 * that copies overlap the multiplication. This is what a YTensor that lives in host memory
 * calls (the reference's tensors always do, include/ytensor_base.hpp:388). */
int ytcuda_gemm_host(int dtype_in, int dtype_out, const void* A, const void* B, void* C, int m, int n, int k,
                     float alpha, float beta, int64_t rsa, int64_t csa, int64_t rsb, int64_t csb, int64_t rsc,
                     int64_t csc, int64_t batch, int64_t bsa, int64_t bsb, int64_t bsc);

/* C[b][i][j] = (A[b] . B[b])[i][j] where mask[i][j] != 0, masked_value elsewhere; mask is a bool / uint8 matrix
 * [m, n] (row stride in bytes = elements) shared by every batch item. Replaces YTensor::masked_matmul with a bool
 * mask (src/ytensor_math.inl:318-366, 1053-1090; yt::kernel::avx2::sgemm_masked, src/kernel/avx2/sgemm.inl:342-584).
 * The product runs as ytcuda_gemm does (alpha 1, beta 0) but passes over every output tile in which the mask holds
 * nowhere (the counterpart of the reference's tileAllFalse pruning, src/kernel/avx2/sgemm.inl:449-475); a second pass
 * writes masked_value wherever the mask does not hold. */
int ytcuda_gemm_masked(int dtype_in, int dtype_out, const void* A, const void* B, void* C, int m, int n, int k,
                       int64_t rsa, int64_t csa, int64_t rsb, int64_t csb, int64_t rsc, int64_t csc, int64_t batch,
                       int64_t bsa, int64_t bsb, int64_t bsc, const void* mask, int64_t mask_row_stride,
                       float masked_value, void* stream);

/* The predicate form of YTensor::masked_matmul (src/ytensor_math.inl:368-412, sgemm_masked with a predicate,
 * src/kernel/avx2/sgemm.inl:342-584) for the causal predicate, evaluated on the device: element (i, j) is computed iff
 * j <= i + causal_offset. No mask is read; tiles entirely above the diagonal are skipped. Any other predicate is
 * materialised into a bool matrix by the caller (device code cannot call a host lambda). */
int ytcuda_gemm_masked_causal(int dtype_in, int dtype_out, const void* A, const void* B, void* C, int m, int n, int k,
                              int64_t rsa, int64_t csa, int64_t rsb, int64_t csb, int64_t rsc, int64_t csc,
                              int64_t batch, int64_t bsa, int64_t bsb, int64_t bsc, int causal_offset,
                              float masked_value, void* stream);

/* ---------------------------------------------------------------- reductions over axes
 * All N-d entry points take `ndim` (1..8) extents and ELEMENT strides; `axes` lists the reduced axes
 * (negative values count from the end). The reduced elements of one output position are walked
 * as an odometer over the axes in the order listed, as the reference does. Trailing contiguous
 * axes take the single-pass register kernel; any other axes / strides take the generic kernel. */

/* y = softmax(x) jointly over `axes`. Replaces yt::function::softmax / softmax_
 * (include/function/activation.hpp:30-39, src/function/activation.inl:130-409). */
int ytcuda_softmax(int dt_in, int dt_out, const void* x, void* y, const int64_t* shape, const int64_t* xstrides,
                   const int64_t* ystrides, int ndim, const int* axes, int naxes, void* stream);

/* y = x / sqrt(mean_axes(x*x) + eps) * weight. `weight` (may be NULL) is contiguous over the reduced dims in
 * ascending axis order. Replaces yt::function::rmsNorm / rmsNorm_ (include/function/normalization.hpp:55-88,
 * src/function/normalization.inl:33-54,88-101,234-277). */
int ytcuda_rmsnorm(int dt_in, int dt_out, int dt_w, const void* x, const void* weight, void* y, const int64_t* shape,
                   const int64_t* xstrides, const int64_t* ystrides, int ndim, const int* axes, int naxes, float eps,
                   void* stream);

/* y = x / (sum_axes |x|^p + eps)^(1/p): the Lp normalisation of yt::function::normalize / normalize_
 * (include/function/normalization.hpp, src/function/normalization.inl:56-85, 278-318); p > 0. The affine forms apply
 * gamma and bias afterwards with ytcuda_binary, as the reference's _applyScale_ / _applyBias_ do (:88-116). */
int ytcuda_normalize(int dt_in, int dt_out, const void* x, void* y, const int64_t* shape, const int64_t* xstrides,
                     const int64_t* ystrides, int ndim, const int* axes, int naxes, float p, float eps, void* stream);

/* y = (x - mean) / sqrt(var + eps) * gamma + beta (gamma and beta both NULL for the plain form).
 * Replaces yt::function::layerNorm / layerNorm_ (include/function/normalization.hpp:8-53,
 * src/function/normalization.inl:3-30,159-230). */
int ytcuda_layernorm(int dt_in, int dt_out, int dt_w, const void* x, const void* gamma, const void* beta, void* y,
                     const int64_t* shape, const int64_t* xstrides, const int64_t* ystrides, int ndim, const int* axes,
                     int naxes, float eps, void* stream);

/* op 0 = sum, 1 = mean, 2 = max. y is contiguous with size-1 dims on the reduced axes; for max, `index`
 * (may be NULL) receives the position of the FIRST maximum in the odometer walk. Replaces YTensor::sum / mean /
 * max (include/ytensor_math.hpp:105-121, src/ytensor_math.inl:414-692). */
int ytcuda_reduce(int op, int dt_in, int dt_out, const void* x, void* y, int32_t* index, const int64_t* shape,
                  const int64_t* xstrides, int ndim, const int* axes, int naxes, void* stream);

/* Same result as ytcuda_reduce for callers that must not allocate device memory while they run: a serving or
 * real-time loop that cannot afford the allocator's lock and implicit synchronisation, a process whose device memory
 * budget is fixed at start-up, a plug-in host that forbids cudaMalloc after initialisation. It has no counterpart in the reference (a CPU library, whose temporaries
 * are thread_local host buffers). The long-reduction path keeps its partial results in a fixed 64 KiB array compiled
 * into the library (8192 value/index pairs; each GPU that loads the library holds it until the process ends) instead
 * of the library's grown-on-demand workspace, and the call makes no cudaMalloc / cudaFree of its own.
 * A request whose partials do not fit the array is refused with YTC_INVALID_ARG and a message naming both sizes.
 * The very first call on each device looks up the array's device address (cudaGetSymbolAddress), which may load the
 * library's device code on that device; make that call once, with the device current, before starting any stream
 * capture. All calls share the one array and do not clear
 * it (every slot a call reads it has written first): two calls that overlap on the GPU, on different streams or
 * from different threads, race on it - serialise them. */
int ytcuda_reduce_noalloc(int op, int dt_in, int dt_out, const void* x, void* y, int32_t* index, const int64_t* shape,
                          const int64_t* xstrides, int ndim, const int* axes, int naxes, void* stream);
/* Bytes of the fixed array a ytcuda_reduce_noalloc call may use (0 = all 65536). With the library's own chunking a
 * call needs at most 8 bytes x 6 x the SM count (about 7 KiB on a 148-SM part), so the refusal cannot occur at the
 * default; an embedder that wants the guarantee checked, or a test, lowers the limit. No counterpart in the reference. */
int ytcuda_reduce_noalloc_set_limit(uint64_t bytes);

/* Fused memory-bound chain: out = cast(softmax(rmsNorm(x, weight, -1, eps) + residual, -1)).
 * x [batch, rows, hidden] fp32 contiguous; residual [batch, rows, hidden] (residual_batched != 0) or
 * [1, rows, hidden] broadcast over batch; one read of x and of the residual, one write of out.
 * Replaces the sequence rmsNorm -> operator+= -> softmax_ -> copy_ (src/function/normalization.inl:234-277,
 * src/ytensor_math.inl:35-49, src/function/activation.inl:376-409, src/ytensor_base.inl:257-430). */
int ytcuda_rmsnorm_add_softmax_cast(int dt_out, const float* x, const float* weight, const float* residual, void* out,
                                    int64_t batch, int64_t rows, int hidden, int residual_batched, float eps,
                                    void* stream);

/* ---------------------------------------------------------------- elementwise
 * out = a (op) b with broadcasting expressed as zero strides; op 0 add, 1 sub, 2 mul, 3 div. `out` may alias
 * `a` (the in-place operators). Replaces the operator macros over yt::kernel::broadcast / broadcastInplace
 * (src/ytensor_math.inl:22-124, src/kernel/broadcast.inl:167-469). */
int ytcuda_binary(int op, int dt_a, int dt_b, int dt_out, const void* a, const void* b, void* out, int ndim,
                  const int64_t* shape, const int64_t* astrides, const int64_t* bstrides, const int64_t* ostrides,
                  void* stream);

/* y = f(x): op 0 copy, 1 swish (x * stable sigmoid(x)), 2 x * param, 3 x + param, and the forward forms of the other
 * activations of yt::function (src/function/activation.inl): 4 relu, 5 exp, 6 sigmoid, 7 leakyRelu (param = alpha),
 * 8 elu (param = alpha), 9 selu, 10 gelu (erf form), 11 tanh, 12 softplus, 13 mish, 14 hardSigmoid, 15 hardSwish.
 * op + 32 for an activation (33, 36 .. 47) is its first derivative, the `order = 1` form of the same functions.
 * Replaces yt::function::swish_ (:631-647) and its siblings, and scalar broadcastInplace calls. */
int ytcuda_unary(int op, int dt_in, int dt_out, const void* x, void* y, int ndim, const int64_t* shape,
                 const int64_t* xstrides, const int64_t* ystrides, float param, void* stream);

/* Strided dtype conversion with the reference's own rounding (the 8-bit types YTC_F8_* included, through the same
 * FloatSpec rule as float16, include/types/float_spec.hpp:299-371, 435-491): yt::bfloat16(float) adds half an ulp only when
 * the kept LSB is 1 (include/types/bfloat16.hpp:78-80); yt::float16 rounds to nearest even and flushes results
 * below the smallest normal to zero (include/types/float_spec.hpp:435-491). Bit-exact with the reference.
 * Replaces YTensorBase::copy_ / cast (src/ytensor_base.inl:257-430, include/ytensor_base.hpp:399-404). */
int ytcuda_cast(int dt_in, int dt_out, const void* x, void* y, int ndim, const int64_t* shape, const int64_t* xstrides,
                const int64_t* ystrides, void* stream);

/* out[r, i] = swish(gate_up[r, i]) * gate_up[r, inter + i], i < inter: the gate / up halves of the fused
 * projection (example/qwen3/src/qwen3.cpp:193-200: swish_ on one slice, then *= the other slice). */
int ytcuda_swiglu(int dt_in, int dt_out, const void* gate_up, void* out, int64_t rows, int inter, int64_t gu_row_stride,
                  int64_t out_row_stride, void* stream);

/* ---------------------------------------------------------------- attention
 * O = softmax(scale * Q K^T + bias, masked) V per (batch, query head). Q [batch, kv_heads*groups, q_len, head_dim],
 * K [batch, kv_heads, kv_len, head_dim], V [batch, kv_heads, kv_len, value_dim], O like Q with value_dim; query head
 * h reads K/V head h / groups (the zero-stride repeat_kv view of example/qwen3/src/qwen3.cpp:252-264,583-589).
 * *_strides = {batch, head, row} strides in elements; the innermost dim has unit stride.
 * scale == 0 means 1/sqrt(head_dim) (src/function/ops.inl:378-381).
 * mask_kind 0: none; 1: causal, key c is visible to query r iff c <= r + causal_offset (the reference's
 * make_causal_mask uses causal_offset = kv_len - q_len, qwen3.cpp:46-55); 2: bool mask bytes [q_len, kv_len] with
 * row stride mask_row_stride. bias: optional fp32 [q_len, kv_len] added to the scaled scores. A query row that sees
 * no key yields zeros (src/kernel/avx2/flash_attention.inl:241-244,327-331).
 * BF16 / F16 with head_dim == value_dim in {64, 128} and 16-byte aligned rows run on the tcgen05 kernel; every other
 * case (F32 included) runs on the one-warp-per-row kernel.
 * Replaces yt::function::scaledDotProductAttention (include/function/ops.hpp:26-70, src/function/ops.inl:109-234,
 * 368-503) and yt::kernel::avx2::flash_attention (include/kernel/avx2/flash_attention.hpp:21-69). */
int ytcuda_flash_attn_fwd(int dtype, const void* Q, const void* K, const void* V, void* O, int batch, int kv_heads,
                          int groups, int q_len, int kv_len, int head_dim, int value_dim, float scale,
                          const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                          const int64_t* o_strides, int mask_kind, int causal_offset, const uint8_t* mask,
                          int64_t mask_row_stride, const float* bias, int64_t bias_row_stride, int64_t bias_col_stride,
                          void* stream);

/* Kernel choice of ytcuda_flash_attn_fwd: 0 = automatic, 1 = always the one-warp-per-row kernel, 2 = tcgen05 or
 * YTC_UNSUPPORTED. The counterpart of the per-call sdpaBackend argument (include/function/ops.hpp:21-24). */
int ytcuda_attn_set_path(int path);

/* ---------------------------------------------------------------- decoder (Qwen3 block structure)
 * The reference's example model (example/qwen3/include/qwen3.hpp:46-182, src/qwen3.cpp) on the device. Activations,
 * residual stream, KV cache and logits are fp32 as in the reference; weights stay in bfloat16 storage. */

/* cos / sin tables [max_len, dim] on the HOST, as RoPECache::precompute fills them (qwen3.cpp:161-175). */
int ytcuda_rope_tables(int dim, int max_len, float theta, float* cos_host, float* sin_host);

/* out[t, :] = float(table[ids[t], :]), table bf16 [vocab, hidden] (embedding gather, qwen3.cpp:378-385). */
int ytcuda_embedding(const void* table_bf16, const int32_t* ids, float* out, int64_t n, int hidden, int vocab,
                     void* stream);

/* y[m, n] (+)= x[m, k] . W[n, k]^T with fp32 x, y and bf16 W [n, k] row-major: yt::function::linear
 * (src/function/ops.inl:84-91) with the weight left in its storage type. Up to 4 rows: one pass over W with FFMA
 * (decode). More rows: x is split into two bf16 planes (hi + lo) and multiplied on tcgen05 (up to 128 rows with the
 * k range cut into pieces that run side by side, partial sums added in a fixed order); `hi_lo_scratch` must then
 * hold 4*m*k bytes of device memory. */
int ytcuda_linear_w16(const float* x, int64_t x_row_stride, const void* w_bf16, float* y, int64_t y_row_stride,
                      int64_t m, int n, int k, int accumulate, void* hi_lo_scratch, void* stream);

/* Top-k sampling of qwen3::Qwen3ForCausalLM::generate (example/qwen3/src/qwen3.cpp:465-486): per row of fp32 logits
 * [rows, vocab], probabilities = softmax, the k <= 64 most probable tokens in descending order go to top_probs /
 * top_idx [rows, k] (the first index wins ties), and, when `sampled` is given, the token whose running sum of kept
 * probabilities first reaches uniform[row] * (sum of the kept probabilities) goes to sampled[row]. The uniform numbers
 * in [0, 1] come from the caller (the reference draws them on the host from std::mt19937); null means 0. */
int ytcuda_topk_sample(const float* logits, int64_t row_stride, int rows, int vocab, int k, const float* uniform,
                       float* top_probs, int32_t* top_idx, int32_t* sampled, void* stream);

/* Fused per-head RMSNorm (q, k) + rotate-half RoPE + KV-cache append on the fused projection output
 * qkv [batch, len, (heads + 2 kv_heads) * 128] -> q_out [batch, heads, len, 128], k_cache / v_cache
 * [batch, kv_heads, max_len, 128] at slots slot0 .. slot0 + len - 1, RoPE positions pos0 .. (qwen3.cpp:237-247,
 * 70-88, 522-559). */
int ytcuda_qwen3_qkv_post(const float* qkv, float* q_out, float* k_cache, float* v_cache, const float* q_norm,
                          const float* k_norm, const float* cos_table, const float* sin_table, int batch, int len,
                          int heads, int kv_heads, int head_dim, int max_len, int pos0, int slot0, float eps,
                          void* stream);

/* Model handle: qwen3::Qwen3ForCausalLM (qwen3.hpp:146-168) with its KV caches, for `batch` sequences, as rank
 * tp_rank of tp_world tensor-parallel ranks (heads and FFN columns split; vocabulary rows split for the logits).
 * Returns NULL on an unsupported configuration (see ytcuda_last_error_string). */
void* ytcuda_qwen3_create(int hidden, int layers, int vocab, int inter, int heads, int kv_heads, int head_dim, float eps,
                          float theta, int max_pos, int batch, int tp_rank, int tp_world);
void ytcuda_qwen3_destroy(void* handle);
/* Registers a device weight (borrowed, not copied). "embed" [vocab, hidden], "lm_head" [rank's vocab rows, hidden],
 * per layer "qkv", "o", "gate_up", "down": bf16 [out, in] already sliced for the rank; "norm", "q_norm", "k_norm",
 * "norm1", "norm2": fp32 (members of Qwen3Model / Qwen3DecoderLayer, qwen3.hpp:62-137). */
int ytcuda_qwen3_set_weight(void* handle, const char* name, int layer, const void* dptr);
/* Sum all-reduce over the tensor-parallel group, called between kernels after the attention output projection and
 * after the down projection (the reference has no counterpart: it is single-process). */
int ytcuda_qwen3_set_allreduce(void* handle, int (*fn)(void* buf, int64_t count, void* user), void* user);
/* Qwen3ForCausalLM::reset_kv_cache / get_kv_cache_len (qwen3.cpp:425-435). */
int ytcuda_qwen3_reset(void* handle);
int ytcuda_qwen3_cache_len(void* handle);
/* How a forward of ONE new token per sequence runs: 0 = automatic (one persistent cooperative kernel for the whole
 * step for batch <= 6, or <= 8 under tensor parallelism, where it needs connected exchange buffers, see
 * ytcuda_qwen3_tp_export),
 * 1 = one launch per operator as for longer inputs, 2 = the persistent kernel (batch <= 32) or YTC_UNSUPPORTED.
 * 3 = as 2, with the FFMA form of the kernel's linear phases even where the tensor-core form (five or more
 * sequences, hidden <= 1024) applies. Up to four sequences the kernel streams its weights through a ring of
 * shared-memory slots filled by bulk async copies that run ahead of the phases and, on one GPU, has no grid barriers:
 * the activations that cross between phases are stored as {value, tag} pairs that the consumers poll, and the linear
 * phases run on mma.sync with the activations split into two bf16 planes (paths 0, 2 and 3 alike); 4 = as 3 without
 * the ring (every phase loads its weights after the barrier before it); 5 = the ring with grid barriers;
 * 6 = as 1, and under tensor parallelism every sum over ranks goes through the all-reduce callback (otherwise inputs
 * of 5 to 128 rows exchange the ranks' shares inside the kernel that adds a projection to the residual stream: each
 * rank pushes its row sums as {value, tag} pairs into the peers' buffers and polls its own).
 * Both forms compute the operator sequence of Qwen3ForCausalLM::forward (qwen3.cpp:365-457); the switch itself has
 * no counterpart in the reference. */
int ytcuda_qwen3_set_decode_path(void* handle, int path);
/* Timeline of the single-kernel decode step, for tuning: with a device buffer of 2 * slots_per_cta int64 set, the first
 * and the last CTA of every following step kernel write their SM's cycle counter at slot 4 * b + k of their half of
 * the buffer: k = 0 on arriving at grid barrier number b, 1 on leaving it, 2 once the linear phase after it has staged
 * its activations (streaming form only). NULL / 0 switches it off (the default). No counterpart in the reference. */
int ytcuda_qwen3_set_trace(void* handle, int64_t* dev_buf, int slots_per_cta);
/* Tensor-parallel decode steps without a host-side collective: every rank exports the CUDA IPC handle (64 bytes) of
 * its exchange buffer, the caller distributes the handles (one all-gather at start-up), and every rank imports its
 * peers'. From then on a forward of one token per sequence (batch <= 8) is ONE kernel per rank that all-reduces the
 * partial sums of the o and down projections itself over NVLink: up to four sequences by pushing {value, tag} pairs
 * into the peers' buffers and polling its own, beyond that by loads from the peers' buffers behind a barrier. All
 * ranks must call forward the same number of times. The all-reduce callback is still used for longer inputs. No counterpart in
 * the reference (single process). */
int ytcuda_qwen3_tp_export(void* handle, void* ipc_handle_64);
int ytcuda_qwen3_tp_import(void* handle, int rank, const void* ipc_handle_64);
/* Tear-down order of a tensor-parallel group: every rank calls ytcuda_qwen3_tp_disconnect (waits for its own kernels,
 * closes the peers' buffers), the caller runs a barrier over the group, then every rank calls ytcuda_qwen3_destroy
 * (which frees the buffer it exported). Freeing an exported buffer that a peer still has open is undefined. */
int ytcuda_qwen3_tp_disconnect(void* handle);
/* Recovery after ytcuda_device_status reported YTC_TIMEOUT under tensor parallelism (a peer never arrived): every rank
 * waits for its own stream, the caller runs a barrier, every rank calls this (exchange counters and arrival words
 * start again from zero, KV caches reset), a second barrier, then forward may be called again. */
int ytcuda_qwen3_tp_resync(void* handle);
/* ids [batch, len] int32 (device) -> logits of the last position [batch, rank's vocab rows] fp32 (device); appends
 * len tokens to the KV caches (Qwen3ForCausalLM::forward, qwen3.cpp:449-457). The caches are ring buffers as in the
 * reference (qwen3.cpp:70-126): a token written past the end overwrites the oldest slot. A call with len == 1 into a
 * full cache attends to every slot and uses rotary position 0 (the reference's position rule, :365-375); a call with
 * len > 1 that runs over the end appends all its tokens first and lets every query see the slots that are not younger
 * than itself (KVCache::get_mask), with the rotary positions restarting at the cache length or at 0 as that rule
 * says. len > max_position_embeddings returns YTC_UNSUPPORTED. */
int ytcuda_qwen3_forward(void* handle, const int32_t* ids, int len, float* logits, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* YTCUDA_H_ */
