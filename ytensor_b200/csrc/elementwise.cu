// Broadcast elementwise operators, unary maps and dtype casts with N-d strides.
//
// Contiguous operands move as 128-bit (fp32) / 64-bit (16-bit types) vectors in a grid-stride loop;
// a right operand that repeats over the leading dims (bias, residual shared by the batch) is
// indexed by a modulo; everything else goes through per-element index arithmetic on the device.
//
// Replaces the operator macros and yt::kernel::broadcast / broadcastInplace (reference
// src/ytensor_math.inl:22-124, src/kernel/broadcast.inl:167-469), yt::function::swish_
// (src/function/activation.inl:631-647) and YTensorBase::copy_ / cast (src/ytensor_base.inl:257-430).
#include "ytc_common.cuh"

namespace ytk {

constexpr int EW_MAXD = 8;
enum BinOp { B_ADD = 0, B_SUB = 1, B_MUL = 2, B_DIV = 3 };
enum UnOp {
  U_COPY = 0, U_SWISH = 1, U_SCALE = 2, U_ADD_SCALAR = 3,
  // the other activations of yt::function (src/function/activation.inl), forward form (order 0)
  U_RELU = 4, U_EXP = 5, U_SIGMOID = 6, U_LEAKY_RELU = 7, U_ELU = 8, U_SELU = 9, U_GELU = 10, U_TANH = 11,
  U_SOFTPLUS = 12, U_MISH = 13, U_HARD_SIGMOID = 14, U_HARD_SWISH = 15
};
constexpr int U_LAST = U_HARD_SWISH;
constexpr int U_DERIV = 32;  // op + 32: the first derivative (order 1) of activation `op`

__device__ __forceinline__ float bin_apply(int op, float a, float b) {
  switch (op) {
    case B_ADD: return a + b;
    case B_SUB: return a - b;
    case B_MUL: return a * b;
    default: return a / b;
  }
}
// swish(x) = x * sigmoid(x), sigmoid in the reference's two-branch stable form
// (src/ytensor_function.inl:42-52).
__device__ __forceinline__ float swish_ref(float v) {
  float sig;
  if (v >= 0.f) {
    const float z = expf(-v);
    sig = 1.0f / (1.0f + z);
  } else {
    const float z = expf(v);
    sig = z / (1.0f + z);
  }
  return v * sig;
}
// sigmoid and softplus in the reference's stable forms (src/ytensor_function.inl:42-59)
__device__ __forceinline__ float sigmoid_ref(float v) {
  if (v >= 0.f) return 1.0f / (1.0f + expf(-v));
  const float z = expf(v);
  return z / (1.0f + z);
}
__device__ __forceinline__ float softplus_ref(float v) { return fmaxf(v, 0.f) + log1pf(expf(-fabsf(v))); }

// First derivatives (the order == 1 branches of src/function/activation.inl)
__device__ __forceinline__ float un_deriv(int op, float a, float param) {
  switch (op) {
    case U_SWISH: {                                                                 // :621-629
      const float sig = sigmoid_ref(a);
      return sig * (1.0f + a * (1.0f - sig));
    }
    case U_RELU: return a > 0.f ? 1.f : 0.f;                                        // :11-14
    case U_EXP: return expf(a);                                                     // :67-84
    case U_SIGMOID: {                                                               // :94-99
      const float sig = sigmoid_ref(a);
      return sig * (1.0f - sig);
    }
    case U_LEAKY_RELU: return a > 0.f ? 1.f : param;                                // :421-425
    case U_ELU: return a > 0.f ? 1.f : param * expf(a);                             // :457-461
    case U_SELU: {                                                                  // :495-503
      const float l = 1.0507009873554804934193349852946f, al = 1.6732632423543772848170429916717f;
      return a > 0.f ? l : l * al * expf(a);
    }
    case U_GELU: {                                                                  // :538-547
      const float cdf = 0.5f * (1.0f + erff(a / 1.4142135623730950488016887242097f));
      const float pdf = 0.3989422804014326779399460599343f * expf(-0.5f * a * a);
      return cdf + a * pdf;
    }
    case U_TANH: {                                                                  // :583-588
      const float t = tanhf(a);
      return 1.0f - t * t;
    }
    case U_SOFTPLUS: return sigmoid_ref(a);                                         // :658-660
    case U_MISH: {                                                                  // :689-697
      const float tsp = tanhf(softplus_ref(a));
      return tsp + a * (1.0f - tsp * tsp) * sigmoid_ref(a);
    }
    case U_HARD_SIGMOID: return (a > -3.f && a < 3.f) ? 1.0f / 6.0f : 0.f;          // :733-739
    default:                                                                        // hardSwish, :776-783
      if (a <= -3.f) return 0.f;
      if (a >= 3.f) return 1.f;
      return (2.f * a + 3.f) / 6.0f;
  }
}

__device__ __forceinline__ float un_apply(int op, float a, float param) {
  if (op >= U_DERIV) return un_deriv(op - U_DERIV, a, param);
  switch (op) {
    case U_COPY: return a;
    case U_SWISH: return swish_ref(a);
    case U_SCALE: return a * param;
    case U_ADD_SCALAR: return a + param;
    case U_RELU: return fmaxf(a, 0.f);                                              // activation.inl:3-10
    case U_EXP: return expf(a);                                                     // :67-72
    case U_SIGMOID: return sigmoid_ref(a);                                          // :87-93
    case U_LEAKY_RELU: return a > 0.f ? a : param * a;                              // :413-420
    case U_ELU: return a > 0.f ? a : param * (expf(a) - 1.0f);                      // :449-456
    case U_SELU: {                                                                  // :485-494
      const float l = 1.0507009873554804934193349852946f, al = 1.6732632423543772848170429916717f;
      return a > 0.f ? l * a : l * al * (expf(a) - 1.0f);
    }
    case U_GELU: return 0.5f * a * (1.0f + erff(a / 1.4142135623730950488016887242097f));  // :529-537
    case U_TANH: return tanhf(a);                                                   // :575-582
    case U_SOFTPLUS: return softplus_ref(a);                                        // :651-657
    case U_MISH: return a * tanhf(softplus_ref(a));                                 // :681-688
    case U_HARD_SIGMOID: return fmaxf(0.f, fminf(1.f, a / 6.0f + 0.5f));            // :724-731
    default:                                                                        // hardSwish, :760-775
      if (a <= -3.f) return 0.f;
      if (a >= 3.f) return a;
      return a * (a + 3.f) / 6.0f;
  }
}

struct V4 {
  float v[4];
};
__device__ __forceinline__ V4 ld4(const void* p, int64_t i, int dt) {
  V4 r;
  if (dt == YTC_F32) {
    const float4 t = *reinterpret_cast<const float4*>(static_cast<const float*>(p) + i);
    r.v[0] = t.x; r.v[1] = t.y; r.v[2] = t.z; r.v[3] = t.w;
  } else if (dt >= YTC_F8_E5M2) {
    const uint32_t t = *reinterpret_cast<const uint32_t*>(static_cast<const uint8_t*>(p) + i);
#pragma unroll
    for (int k = 0; k < 4; ++k) r.v[k] = f8_bits_to_f32(static_cast<uint8_t>(t >> (8 * k)), dt);
  } else {
    const uint2 t = *reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(p) + i);
    const uint16_t h[4] = {static_cast<uint16_t>(t.x & 0xFFFF), static_cast<uint16_t>(t.x >> 16),
                           static_cast<uint16_t>(t.y & 0xFFFF), static_cast<uint16_t>(t.y >> 16)};
#pragma unroll
    for (int k = 0; k < 4; ++k) r.v[k] = (dt == YTC_BF16) ? bf16_bits_to_f32(h[k]) : f16_bits_to_f32_ref(h[k]);
  }
  return r;
}
__device__ __forceinline__ void st4(void* p, int64_t i, const V4& r, int dt) {
  if (dt == YTC_F32) {
    *reinterpret_cast<float4*>(static_cast<float*>(p) + i) = make_float4(r.v[0], r.v[1], r.v[2], r.v[3]);
  } else if (dt >= YTC_F8_E5M2) {
    uint32_t t = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) t |= static_cast<uint32_t>(f32_to_f8_bits(r.v[k], dt)) << (8 * k);
    *reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(p) + i) = t;
  } else {
    uint16_t h[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) h[k] = (dt == YTC_BF16) ? f32_to_bf16_bits_ref(r.v[k]) : f32_to_f16_bits_ref(r.v[k]);
    uint2 t;
    t.x = static_cast<uint32_t>(h[0]) | (static_cast<uint32_t>(h[1]) << 16);
    t.y = static_cast<uint32_t>(h[2]) | (static_cast<uint32_t>(h[3]) << 16);
    *reinterpret_cast<uint2*>(static_cast<uint16_t*>(p) + i) = t;
  }
}

// out[i] = a[i] op b[i % bmod] over contiguous memory, 4 elements per thread per trip.
__global__ void __launch_bounds__(256) binary_vec_kernel(int op, const void* a, const void* b, void* out, int64_t n4,
                                                         int64_t bmod, int dt_a, int dt_b, int dt_out) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t e = i * 4;
    const V4 x = ld4(a, e, dt_a);
    const V4 y = ld4(b, e % bmod, dt_b);
    V4 r;
#pragma unroll
    for (int k = 0; k < 4; ++k) r.v[k] = bin_apply(op, x.v[k], y.v[k]);
    st4(out, e, r, dt_out);
  }
}

struct NdIndex {
  int nd;
  int64_t shape[EW_MAXD], s0[EW_MAXD], s1[EW_MAXD], s2[EW_MAXD];
};

__global__ void __launch_bounds__(256) binary_nd_kernel(int op, const void* a, const void* b, void* out, int64_t n,
                                                        const NdIndex ix, int dt_a, int dt_b, int dt_out) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    int64_t rem = i, oa = 0, ob = 0, oo = 0;
    for (int d = ix.nd - 1; d >= 0; --d) {
      const int64_t c = rem % ix.shape[d];
      rem /= ix.shape[d];
      oa += c * ix.s0[d];
      ob += c * ix.s1[d];
      oo += c * ix.s2[d];
    }
    store_from_f32(out, oo, bin_apply(op, load_as_f32(a, oa, dt_a), load_as_f32(b, ob, dt_b)), dt_out);
  }
}

__global__ void __launch_bounds__(256) unary_vec_kernel(int op, const void* x, void* y, int64_t n4, float param,
                                                        int dt_in, int dt_out) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    V4 v = ld4(x, i * 4, dt_in);
#pragma unroll
    for (int k = 0; k < 4; ++k) v.v[k] = un_apply(op, v.v[k], param);
    st4(y, i * 4, v, dt_out);
  }
}

__global__ void __launch_bounds__(256) unary_nd_kernel(int op, const void* x, void* y, int64_t n, const NdIndex ix,
                                                       float param, int dt_in, int dt_out) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    int64_t rem = i, oi = 0, oo = 0;
    for (int d = ix.nd - 1; d >= 0; --d) {
      const int64_t c = rem % ix.shape[d];
      rem /= ix.shape[d];
      oi += c * ix.s0[d];
      oo += c * ix.s2[d];
    }
    store_from_f32(y, oo, un_apply(op, load_as_f32(x, oi, dt_in), param), dt_out);
  }
}

// out[r, i] = swish(gu[r, i]) * gu[r, inter + i]: the gate/up halves of a fused projection
// (reference example/qwen3/src/qwen3.cpp:193-200 does swish_ on one slice, then *= the other).
__global__ void __launch_bounds__(256) swiglu_kernel(const void* gu, void* out, int64_t rows, int inter, int64_t gu_rs,
                                                     int64_t out_rs, int dt_in, int dt_out) {
  dependent_wait();     // (under a programmatic dependent launch: the kernel before this one has finished)
  dependent_trigger();  // the kernel queued behind this one may be scheduled meanwhile
  const int64_t per_row = inter / 4;
  const int64_t n4 = rows * per_row;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / per_row, c = (i - r * per_row) * 4;
    const V4 g = ld4(gu, r * gu_rs + c, dt_in);
    const V4 u = ld4(gu, r * gu_rs + inter + c, dt_in);
    V4 o;
#pragma unroll
    for (int k = 0; k < 4; ++k) o.v[k] = swish_ref(g.v[k]) * u.v[k];
    st4(out, r * out_rs + c, o, dt_out);
  }
}

static int grid_for(int64_t work_items) {
  const int64_t blocks = (work_items + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  return static_cast<int>(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

static bool is_contig(int nd, const int64_t* shape, const int64_t* st) {
  int64_t exp = 1;
  for (int d = nd - 1; d >= 0; --d) {
    if (shape[d] != 1 && st[d] != exp) return false;
    exp *= shape[d];
  }
  return true;
}
static bool aligned(const void* p, int dt) { return (reinterpret_cast<uint64_t>(p) % (4 * dtype_size(dt))) == 0; }

}  // namespace ytk

using namespace ytk;

extern "C" {

static int unary_impl(int op, int dt_in, int dt_out, const void* x, void* y, int ndim, const int64_t* shape,
                      const int64_t* xstrides, const int64_t* ystrides, float param, void* stream);

int ytcuda_binary(int op, int dt_a, int dt_b, int dt_out, const void* a, const void* b, void* out, int ndim,
                  const int64_t* shape, const int64_t* astrides, const int64_t* bstrides, const int64_t* ostrides,
                  void* stream) {
  YTC_REQUIRE(op >= 0 && op <= 3, "ytcuda_binary: op must be 0..3 (add, sub, mul, div)");
  YTC_REQUIRE(ndim >= 1 && ndim <= EW_MAXD, "ytcuda_binary: ndim %d outside [1, %d]", ndim, EW_MAXD);
  YTC_REQUIRE(shape && astrides && bstrides && ostrides, "ytcuda_binary: null shape/strides");
  YTC_REQUIRE(dt_a >= 0 && dt_a <= 2 && dt_b >= 0 && dt_b <= 2 && dt_out >= 0 && dt_out <= 2, "ytcuda_binary: bad dtype");
  int64_t n = 1;
  for (int d = 0; d < ndim; ++d) {
    YTC_REQUIRE(shape[d] >= 0, "ytcuda_binary: negative extent");
    n *= shape[d];
  }
  if (n == 0) return YTC_OK;
  YTC_REQUIRE(a && b && out, "ytcuda_binary: null tensor");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (is_contig(ndim, shape, astrides) && is_contig(ndim, shape, ostrides) && n % 4 == 0 && aligned(a, dt_a) &&
      aligned(b, dt_b) && aligned(out, dt_out)) {
    // b: zero stride on leading dims, contiguous on the trailing ones => index i % bmod
    int split = ndim;
    int64_t exp = 1;
    while (split > 0 && (shape[split - 1] == 1 || bstrides[split - 1] == exp)) {
      exp *= shape[split - 1];
      --split;
    }
    bool lead_zero = true;
    for (int d = 0; d < split; ++d)
      if (shape[d] != 1 && bstrides[d] != 0) lead_zero = false;
    if (lead_zero && exp % 4 == 0) {
      binary_vec_kernel<<<grid_for(n / 4), 256, 0, st>>>(op, a, b, out, n / 4, exp, dt_a, dt_b, dt_out);
      count_launch();
      YTC_CUDA(cudaGetLastError());
      return YTC_OK;
    }
  }
  NdIndex ix;
  ix.nd = ndim;
  for (int d = 0; d < ndim; ++d) {
    ix.shape[d] = shape[d];
    ix.s0[d] = astrides[d];
    ix.s1[d] = bstrides[d];
    ix.s2[d] = ostrides[d];
  }
  binary_nd_kernel<<<grid_for(n), 256, 0, st>>>(op, a, b, out, n, ix, dt_a, dt_b, dt_out);
  count_launch();
  YTC_CUDA(cudaGetLastError());
  return YTC_OK;
}

int ytcuda_unary(int op, int dt_in, int dt_out, const void* x, void* y, int ndim, const int64_t* shape,
                 const int64_t* xstrides, const int64_t* ystrides, float param, void* stream) {
  YTC_REQUIRE(dt_in >= 0 && dt_in <= 2 && dt_out >= 0 && dt_out <= 2, "ytcuda_unary: bad dtype");
  return unary_impl(op, dt_in, dt_out, x, y, ndim, shape, xstrides, ystrides, param, stream);
}

static int unary_impl(int op, int dt_in, int dt_out, const void* x, void* y, int ndim, const int64_t* shape,
                      const int64_t* xstrides, const int64_t* ystrides, float param, void* stream) {
  {
    const int base = op >= U_DERIV ? op - U_DERIV : op;
    YTC_REQUIRE(op >= 0 && base <= U_LAST && (op < U_DERIV || base == U_SWISH || base >= U_RELU),
                "ytcuda_unary: op %d is neither 0..%d nor %d + an activation (1, 4..%d)", op, U_LAST, U_DERIV, U_LAST);
  }
  YTC_REQUIRE(ndim >= 1 && ndim <= EW_MAXD, "ytcuda_unary: ndim %d outside [1, %d]", ndim, EW_MAXD);
  YTC_REQUIRE(shape && xstrides && ystrides, "ytcuda_unary: null shape/strides");
  int64_t n = 1;
  for (int d = 0; d < ndim; ++d) {
    YTC_REQUIRE(shape[d] >= 0, "ytcuda_unary: negative extent");
    n *= shape[d];
  }
  if (n == 0) return YTC_OK;
  YTC_REQUIRE(x && y, "ytcuda_unary: null tensor");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (is_contig(ndim, shape, xstrides) && is_contig(ndim, shape, ystrides) && n % 4 == 0 && aligned(x, dt_in) &&
      aligned(y, dt_out)) {
    unary_vec_kernel<<<grid_for(n / 4), 256, 0, st>>>(op, x, y, n / 4, param, dt_in, dt_out);
  } else {
    NdIndex ix;
    ix.nd = ndim;
    for (int d = 0; d < ndim; ++d) {
      ix.shape[d] = shape[d];
      ix.s0[d] = xstrides[d];
      ix.s1[d] = 0;
      ix.s2[d] = ystrides[d];
    }
    unary_nd_kernel<<<grid_for(n), 256, 0, st>>>(op, x, y, n, ix, param, dt_in, dt_out);
  }
  count_launch();
  YTC_CUDA(cudaGetLastError());
  return YTC_OK;
}

int ytcuda_cast(int dt_in, int dt_out, const void* x, void* y, int ndim, const int64_t* shape, const int64_t* xstrides,
                const int64_t* ystrides, void* stream) {
  YTC_REQUIRE(dt_in >= 0 && dt_in <= YTC_F8_E8M0 && dt_out >= 0 && dt_out <= YTC_F8_E8M0, "ytcuda_cast: bad dtype");
  return unary_impl(U_COPY, dt_in, dt_out, x, y, ndim, shape, xstrides, ystrides, 0.f, stream);
}

int ytcuda_swiglu(int dt_in, int dt_out, const void* gate_up, void* out, int64_t rows, int inter, int64_t gu_row_stride,
                  int64_t out_row_stride, void* stream) {
  YTC_REQUIRE(dt_in >= 0 && dt_in <= 2 && dt_out >= 0 && dt_out <= 2, "ytcuda_swiglu: bad dtype");
  YTC_REQUIRE(rows >= 0 && inter >= 0, "ytcuda_swiglu: negative extent");
  if (rows == 0 || inter == 0) return YTC_OK;
  YTC_REQUIRE(gate_up && out, "ytcuda_swiglu: null tensor");
  if (inter % 4 != 0 || gu_row_stride % 4 != 0 || out_row_stride % 4 != 0 || !aligned(gate_up, dt_in) ||
      !aligned(out, dt_out)) {
    set_last_error("ytcuda_swiglu: the half width and the row strides must be multiples of 4 elements");
    return YTC_UNSUPPORTED;
  }
  YTC_CUDA(launch_overlapped(swiglu_kernel, dim3(grid_for(rows * (inter / 4))), dim3(256), 0,
                             static_cast<cudaStream_t>(stream), gate_up, out, rows, inter, gu_row_stride, out_row_stride,
                             dt_in, dt_out));
  count_launch();
  YTC_CUDA(cudaGetLastError());
  return YTC_OK;
}

}  // extern "C"
