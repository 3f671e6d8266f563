// TEST INFRASTRUCTURE, not product code: a C-callable wrapper around the UNMODIFIED reference
// (header-only YTensor + its Qwen3 example), compiled from the reference sources where they lie
// by oracle/Makefile into oracle/_ref/libyt_ref.so. It exists to (1) generate golden vectors,
// (2) pin the plain-C restatement in yt_oracle.c, (3) time the reference's CPU path.
// Only tests/, the smoke check and the benchmark's CPU-baseline legs may load it.
//
// All tensors are fp32, row-major contiguous unless a function says otherwise.
// The typed YTensor<T,N> path is used throughout (the type-erased YTensorBase::matmul multiplies
// in the wrong order under g++: src/ytensor_base_math.inl:105-117 evaluates a pack expansion
// with a side effect inside function arguments).
#include "ytensor.hpp"
#include "qwen3.hpp"

#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <vector>

using yt::YTensor;

namespace {

template <int N>
YTensor<float, N> make(const float* src, const int* shape) {
  std::vector<int> s(shape, shape + N);
  YTensor<float, N> t(s);
  if (src) std::memcpy(t.data(), src, t.size() * sizeof(float));
  return t;
}
template <int N>
void dump(const YTensor<float, N>& t, float* dst) {
  auto c = t.contiguous();
  std::memcpy(dst, c.data(), c.size() * sizeof(float));
}

struct CausalPred {
  // key index c is visible to query row r when c <= r + offset (offset = kv_len - q_len)
  int offset;
  bool operator()(int r, int c) const { return c <= r + offset; }
  bool tileAllTrue(int r0, int c0, int mr, int nr) const { (void)mr; return c0 + nr - 1 <= r0 + offset; }
  bool tileAllFalse(int r0, int c0, int mr, int nr) const { (void)nr; return c0 > r0 + mr - 1 + offset; }
};

template <int N, typename F>
int with_rank(int ndim, F&& f);

}  // namespace

extern "C" {

void ytref_set_threads(int n) {
  yt::kernel::avx2::set_num_threads(n > 0 ? n : yt::kernel::avx2::default_num_threads());
}
int ytref_get_threads() { return yt::kernel::avx2::get_num_threads(); }
int ytref_default_backend() { return static_cast<int>(yt::infos::defaultMatmulBackend); }

// A [batch,m,k] . B ([k,n] when b_batched == 0, else [batch,k,n]) through YTensor::matmul.
// backend: 0 = Naive, 2 = AVX2 (values of yt::infos::MatmulBackend).
int ytref_matmul_f32(const float* A, const float* B, float* C, int batch, int m, int n, int k, int b_batched,
                     int backend) {
  try {
    const int as[3] = {batch, m, k};
    auto a = make<3>(A, as);
    const auto be = static_cast<yt::infos::MatmulBackend>(backend);
    if (b_batched) {
      const int bs[3] = {batch, k, n};
      auto b = make<3>(B, bs);
      dump(a.matmul(b, be), C);
    } else {
      const int bs[2] = {k, n};
      auto b = make<2>(B, bs);
      dump(a.matmul(b, be), C);
    }
    return 0;
  } catch (const std::exception&) {
    return 1;
  }
}

// YTensor::masked_matmul with a bool mask [m,n] shared by every batch item (src/ytensor_math.inl:318-366).
// backend: 0 = Naive, 2 = AVX2.
int ytref_masked_matmul_f32(const float* A, const float* B, const unsigned char* mask, float masked_value, float* C,
                            int batch, int m, int n, int k, int b_batched, int backend) {
  try {
    const int as[3] = {batch, m, k};
    auto a = make<3>(A, as);
    yt::YTensor<bool, 2> mk(m, n);
    for (int i = 0; i < m; ++i)
      for (int j = 0; j < n; ++j) mk.at(i, j) = mask[static_cast<size_t>(i) * n + j] != 0;
    const auto be = static_cast<yt::infos::MatmulBackend>(backend);
    if (b_batched) {
      const int bs[3] = {batch, k, n};
      auto b = make<3>(B, bs);
      dump(a.masked_matmul(b, mk, masked_value, be), C);
    } else {
      const int bs[2] = {k, n};
      auto b = make<2>(B, bs);
      dump(a.masked_matmul(b, mk, masked_value, be), C);
    }
    return 0;
  } catch (const std::exception&) {
    return 1;
  }
}

// yt::io::YTensorIO (include/ytensor_io.hpp:90-140): appends one 2-D tensor to a .yt file (created when `append`
// is 0). dtype: 0 = float32, 1 = bfloat16 (bit patterns), 3 = int32. compress: "" or "zlib".
int ytref_yt_save(const char* path, int append, const char* name, int dtype, const void* data, int rows, int cols,
                  const char* compress) {
  try {
    yt::io::compressMethod = compress ? compress : "";
    yt::io::YTensorIO io;
    if (!io.open(path, append ? yt::io::Append : yt::io::Write)) return 2;
    bool ok = false;
    const size_t n = static_cast<size_t>(rows) * cols;
    if (dtype == 0) {
      YTensor<float, 2> t(rows, cols);
      std::memcpy(t.data(), data, n * 4);
      ok = io.save(t, name);
    } else if (dtype == 1) {
      YTensor<yt::bfloat16, 2> t(rows, cols);
      std::memcpy(t.data(), data, n * 2);
      ok = io.save(t, name);
    } else if (dtype == 3) {
      YTensor<int32_t, 2> t(rows, cols);
      std::memcpy(t.data(), data, n * 4);
      ok = io.save(t, name);
    }
    io.close();
    yt::io::compressMethod = "";
    return ok ? 0 : 3;
  } catch (const std::exception&) {
    return 1;
  }
}

// Reads a tensor back as float32 (float32 and bfloat16 tensors, as qwen3.cpp:16-44 widens them); returns the
// element count or a negative error.
long long ytref_yt_load_f32(const char* path, const char* name, float* out, long long capacity, int* shape2) {
  try {
    yt::io::YTensorIO io;
    if (!io.open(path, yt::io::Read)) return -2;
    yt::YTensorBase base;
    if (!io.load(base, name)) return -3;
    io.close();
    const long long n = static_cast<long long>(base.size());
    if (n > capacity || base.shape().size() != 2) return -4;
    shape2[0] = base.shape()[0];
    shape2[1] = base.shape()[1];
    if (base.dtype() == "float32") {
      std::memcpy(out, base.data<float>(), static_cast<size_t>(n) * 4);
    } else if (base.dtype() == "bfloat16") {
      const yt::bfloat16* src = base.data<yt::bfloat16>();
      for (long long i = 0; i < n; ++i) out[i] = static_cast<float>(src[i]);
    } else {
      return -5;
    }
    return n;
  } catch (const std::exception&) {
    return -1;
  }
}

// yt::function::linear: x [rows,k] . W[n,k]^T (+ bias[n])
int ytref_linear_f32(const float* X, const float* W, const float* bias, float* Y, int rows, int n, int k) {
  try {
    const int xs[2] = {rows, k}, ws[2] = {n, k}, bs[1] = {n};
    auto x = make<2>(X, xs);
    auto w = make<2>(W, ws);
    if (bias) {
      auto b = make<1>(bias, bs);
      dump(yt::function::linear(x, w, b), Y);
    } else {
      dump(yt::function::linear(x, w), Y);
    }
    return 0;
  } catch (const std::exception&) {
    return 1;
  }
}

// Kernel-level strided GEMM, C = alpha*A.B + beta*C (include/kernel/avx2/sgemm.hpp:51-58).
void ytref_sgemm_strided(const float* A, const float* B, float* C, int m, int n, int k, float alpha, float beta,
                         int64_t rsa, int64_t csa, int64_t rsb, int64_t csb, int64_t rsc, int64_t csc) {
  yt::kernel::avx2::sgemm(A, B, C, m, n, k, alpha, beta, rsa, csa, rsb, csb, rsc, csc);
}

// scaledDotProductAttention on q [b,kvh,g,ql,d], k [b,kvh,kl,d], v [b,kvh,kl,dv]; k and v are repeated
// over g by a zero-stride view as the Qwen3 example does (example/qwen3/src/qwen3.cpp:252-264).
// mask_kind: 0 none, 1 bool mask [ql,kl] (bytes), 2 causal predicate with tile pruning (c <= r + kl - ql).
// backend: 0 MATH, 1 FLASH_AVX2. bias: optional [ql,kl].
int ytref_sdpa_f32(const float* q, const float* k, const float* v, float* out, int b, int kvh, int g, int ql, int kl,
                   int d, int dv, float scale, int mask_kind, const uint8_t* mask, const float* bias, int backend) {
  try {
    const int qs[5] = {b, kvh, g, ql, d}, ks[4] = {b, kvh, kl, d}, vs[4] = {b, kvh, kl, dv};
    auto q5 = make<5>(q, qs);
    auto k4 = make<4>(k, ks);
    auto v4 = make<4>(v, vs);
    auto k5 = qwen3::ops::repeat_kv(k4, g);
    auto v5 = qwen3::ops::repeat_kv(v4, g);
    const auto be = backend ? yt::function::sdpaBackend::FLASH_AVX2 : yt::function::sdpaBackend::MATH;
    YTensor<float, 2> bias_t;
    YTensor<float, 2>* bias_p = nullptr;
    if (bias) {
      const int bs[2] = {ql, kl};
      bias_t = make<2>(bias, bs);
      bias_p = &bias_t;
    }
    YTensor<float, 5> o;
    if (mask_kind == 2) {
      CausalPred pred{kl - ql};
      o = yt::function::scaledDotProductAttention(q5, k5, v5, scale, pred, bias_p, be);
    } else if (mask_kind == 1) {
      YTensor<bool, 2> m(ql, kl);
      for (int r = 0; r < ql; ++r)
        for (int c = 0; c < kl; ++c) m.at(r, c) = mask[static_cast<size_t>(r) * kl + c] != 0;
      o = yt::function::scaledDotProductAttention(q5, k5, v5, scale, &m, bias_p, be);
    } else {
      o = yt::function::scaledDotProductAttention(q5, k5, v5, scale, static_cast<YTensor<bool, 2>*>(nullptr), bias_p,
                                                  be);
    }
    dump(o, out);
    return 0;
  } catch (const std::exception&) {
    return 1;
  }
}

}  // extern "C"

namespace {

template <int N>
int softmax_n(const float* x, float* y, const int* shape, const int* axes, int naxes) {
  auto t = make<N>(x, shape);
  std::vector<int> ax(axes, axes + naxes);
  dump(yt::function::softmax(t, ax), y);
  return 0;
}
template <int N>
int rms_n(const float* x, const float* w, float* y, const int* shape, const int* axes, int naxes, float eps) {
  auto t = make<N>(x, shape);
  std::vector<int> ax(axes, axes + naxes);
  std::vector<int> norm_ax;
  for (int a : ax) norm_ax.push_back((a % N + N) % N);
  if (naxes == 1) {
    const int ws[1] = {shape[norm_ax[0]]};
    auto wt = make<1>(w, ws);
    dump(yt::function::rmsNorm(t, wt, ax, eps), y);
  } else if (naxes == 2) {
    const int ws[2] = {shape[norm_ax[0]], shape[norm_ax[1]]};
    auto wt = make<2>(w, ws);
    dump(yt::function::rmsNorm(t, wt, ax, eps), y);
  } else {
    return 2;
  }
  return 0;
}
template <int N>
int ln_n(const float* x, const float* gamma, const float* beta, float* y, const int* shape, const int* axes,
         int naxes, float eps) {
  auto t = make<N>(x, shape);
  std::vector<int> ax(axes, axes + naxes);
  std::vector<int> norm_ax;
  for (int a : ax) norm_ax.push_back((a % N + N) % N);
  if (!gamma) {
    dump(yt::function::layerNorm(t, ax, eps), y);
  } else if (naxes == 1) {
    const int ws[1] = {shape[norm_ax[0]]};
    auto g = make<1>(gamma, ws);
    auto bt = make<1>(beta, ws);
    dump(yt::function::layerNorm(t, g, bt, ax, eps), y);
  } else if (naxes == 2) {
    const int ws[2] = {shape[norm_ax[0]], shape[norm_ax[1]]};
    auto g = make<2>(gamma, ws);
    auto bt = make<2>(beta, ws);
    dump(yt::function::layerNorm(t, g, bt, ax, eps), y);
  } else {
    return 2;
  }
  return 0;
}
// kind 0 normalize (Lp over `axes`), 1 instanceNorm, 2 batchNorm, 3 groupNorm (channel axis = axes[0] for 1..3);
// gamma / bias: per channel for 1..3, one dim (naxes == 1) for 0; null = the plain form.
template <int N>
int norm_n(int kind, const float* x, const float* gamma, const float* bias, float* y, const int* shape, const int* axes,
           int naxes, int groups, float p, float eps) {
  auto t = make<N>(x, shape);
  std::vector<int> ax(axes, axes + naxes);
  const int c = ((ax[0] % N) + N) % N;
  const int ws[1] = {shape[c]};
  YTensor<float, 1> g, b;
  if (gamma) {
    g = make<1>(gamma, ws);
    b = make<1>(bias, ws);
  }
  switch (kind) {
    case 0:
      if (gamma) {
        if (naxes != 1) return 2;
        dump(yt::function::normalize(t, g, b, ax, p, eps), y);
      } else {
        dump(yt::function::normalize(t, ax, p, eps), y);
      }
      return 0;
    case 1:
      if (gamma) dump(yt::function::instanceNorm(t, g, b, ax[0], eps), y);
      else dump(yt::function::instanceNorm(t, ax[0], eps), y);
      return 0;
    case 2:
      if (gamma) dump(yt::function::batchNorm(t, g, b, ax[0], eps), y);
      else dump(yt::function::batchNorm(t, ax[0], eps), y);
      return 0;
    case 3:
      if (gamma) dump(yt::function::groupNorm(t, g, b, groups, ax[0], eps), y);
      else dump(yt::function::groupNorm(t, groups, ax[0], eps), y);
      return 0;
    default: return 2;
  }
}
template <int N>
int reduce_n(const float* x, float* y, int* idx, const int* shape, const int* axes, int naxes, int op) {
  auto t = make<N>(x, shape);
  std::vector<int> ax(axes, axes + naxes);
  if (op == 0) {
    if (naxes == 1) dump(t.sum(ax[0]), y); else dump(t.sum(ax), y);
  } else if (op == 1) {
    if (naxes == 1) dump(t.mean(ax[0]), y); else dump(t.mean(ax), y);
  } else {
    auto pr = (naxes == 1) ? t.max(ax[0]) : t.max(ax);
    dump(pr.first, y);
    if (idx) {
      auto ic = pr.second.contiguous();
      std::memcpy(idx, ic.data(), ic.size() * sizeof(int));
    }
  }
  return 0;
}
template <int N>
int binary_n(const float* a, const int* ashape, const float* b, const int* bshape, float* out, int op) {
  auto ta = make<N>(a, ashape);
  auto tb = make<N>(b, bshape);
  switch (op) {
    case 0: dump(ta + tb, out); break;
    case 1: dump(ta - tb, out); break;
    case 2: dump(ta * tb, out); break;
    case 3: dump(ta / tb, out); break;
    default: return 2;
  }
  return 0;
}

}  // namespace

#define RANK_SWITCH(ndim, CALL)              \
  try {                                      \
    switch (ndim) {                          \
      case 2: return CALL(2);                \
      case 3: return CALL(3);                \
      case 4: return CALL(4);                \
      case 5: return CALL(5);                \
      default: return 2;                     \
    }                                        \
  } catch (const std::exception&) {          \
    return 1;                                \
  }

extern "C" {

int ytref_softmax_f32(const float* x, float* y, const int* shape, int ndim, const int* axes, int naxes) {
#define CALL(N) softmax_n<N>(x, y, shape, axes, naxes)
  RANK_SWITCH(ndim, CALL)
#undef CALL
}
int ytref_rmsnorm_f32(const float* x, const float* w, float* y, const int* shape, int ndim, const int* axes, int naxes,
                      float eps) {
#define CALL(N) rms_n<N>(x, w, y, shape, axes, naxes, eps)
  RANK_SWITCH(ndim, CALL)
#undef CALL
}
int ytref_layernorm_f32(const float* x, const float* gamma, const float* beta, float* y, const int* shape, int ndim,
                        const int* axes, int naxes, float eps) {
#define CALL(N) ln_n<N>(x, gamma, beta, y, shape, axes, naxes, eps)
  RANK_SWITCH(ndim, CALL)
#undef CALL
}
int ytref_norm_f32(int kind, const float* x, const float* gamma, const float* bias, float* y, const int* shape,
                   int ndim, const int* axes, int naxes, int groups, float p, float eps) {
#define CALL(N) norm_n<N>(kind, x, gamma, bias, y, shape, axes, naxes, groups, p, eps)
  RANK_SWITCH(ndim, CALL)
#undef CALL
}
// The reference's 8-bit float types (include/types/float_spec.hpp:534-536): kind 3 e5m2, 4 e4m3, 5 e8m0.
int ytref_f32_to_fp8(int kind, const float* x, uint8_t* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    if (kind == 3) { yt::float8_e5m2 v(x[i]); std::memcpy(out + i, &v, 1); }
    else if (kind == 4) { yt::float8_e4m3 v(x[i]); std::memcpy(out + i, &v, 1); }
    else if (kind == 5) { yt::float8_e8m0 v(x[i]); std::memcpy(out + i, &v, 1); }
    else return 2;
  }
  return 0;
}
int ytref_fp8_to_f32(int kind, const uint8_t* in, float* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    if (kind == 3) { yt::float8_e5m2 v; std::memcpy(&v, in + i, 1); out[i] = static_cast<float>(v); }
    else if (kind == 4) { yt::float8_e4m3 v; std::memcpy(&v, in + i, 1); out[i] = static_cast<float>(v); }
    else if (kind == 5) { yt::float8_e8m0 v; std::memcpy(&v, in + i, 1); out[i] = static_cast<float>(v); }
    else return 2;
  }
  return 0;
}
// masked_matmul with the causal predicate j <= i + offset (tile-pruning form, src/ytensor_math.inl:368-412)
int ytref_masked_matmul_causal_f32(const float* a, const float* b, int offset, float masked_value, float* c, int batch,
                                   int m, int n, int k) {
  try {
    const int as[3] = {batch, m, k}, bs[2] = {k, n};
    auto ta = make<3>(a, as);
    auto tb = make<2>(b, bs);
    CausalPred pred{offset};
    dump(ta.masked_matmul(tb, pred, masked_value), c);
    return 0;
  } catch (const std::exception&) {
    return 1;
  }
}
// op: 0 sum, 1 mean, 2 max (idx receives the int index tensor, may be null)
int ytref_reduce_f32(const float* x, float* y, int* idx, const int* shape, int ndim, const int* axes, int naxes,
                     int op) {
#define CALL(N) reduce_n<N>(x, y, idx, shape, axes, naxes, op)
  RANK_SWITCH(ndim, CALL)
#undef CALL
}
// op: 0 add, 1 sub, 2 mul, 3 div; shapes have the same rank and broadcast against each other.
int ytref_binary_f32(const float* a, const int* ashape, const float* b, const int* bshape, int ndim, float* out,
                     int op) {
#define CALL(N) binary_n<N>(a, ashape, b, bshape, out, op)
  RANK_SWITCH(ndim, CALL)
#undef CALL
}

int ytref_swish_f32(const float* x, float* y, int64_t n) {
  try {
    const int s[2] = {1, static_cast<int>(n)};
    auto t = make<2>(x, s);
    yt::function::swish_(t);
    dump(t, y);
    return 0;
  } catch (const std::exception&) {
    return 1;
  }
}

// The activations of include/function/activation.hpp:9-109, forward form (order 0), in place on a copy of x.
// op: 4 relu, 5 exp, 6 sigmoid, 7 leakyRelu(alpha), 8 elu(alpha), 9 selu, 10 gelu, 11 tanh, 12 softplus, 13 mish,
// 14 hardSigmoid, 15 hardSwish (1 is swish).
int ytref_activation_f32(int op, const float* x, float* y, int64_t n, float alpha) {
  try {
    const int s[2] = {1, static_cast<int>(n)};
    auto t = make<2>(x, s);
    namespace F = yt::function;
    switch (op) {
      case 1: F::swish_(t); break;
      case 4: F::relu_(t); break;
      case 5: F::exp_(t); break;
      case 6: F::sigmoid_(t); break;
      case 7: F::leakyRelu_(t, alpha); break;
      case 8: F::elu_(t, alpha); break;
      case 9: F::selu_(t); break;
      case 10: F::gelu_(t); break;
      case 11: F::tanh_(t); break;
      case 12: F::softplus_(t); break;
      case 13: F::mish_(t); break;
      case 14: F::hardSigmoid_(t); break;
      case 15: F::hardSwish_(t); break;
      default: return 2;
    }
    dump(t, y);
    return 0;
  } catch (const std::exception&) {
    return 1;
  }
}

// The same activations with their `order` argument (1: first derivative), include/function/activation.hpp:9-109.
int ytref_activation_order_f32(int op, int order, const float* x, float* y, int64_t n, float alpha) {
  try {
    const int s[2] = {1, static_cast<int>(n)};
    auto t = make<2>(x, s);
    namespace F = yt::function;
    switch (op) {
      case 1: F::swish_(t, order); break;
      case 4: F::relu_(t, order); break;
      case 5: F::exp_(t, order); break;
      case 6: F::sigmoid_(t, order); break;
      case 7: F::leakyRelu_(t, alpha, order); break;
      case 8: F::elu_(t, alpha, order); break;
      case 9: F::selu_(t, order); break;
      case 10: F::gelu_(t, order); break;
      case 11: F::tanh_(t, order); break;
      case 12: F::softplus_(t, order); break;
      case 13: F::mish_(t, order); break;
      case 14: F::hardSigmoid_(t, order); break;
      case 15: F::hardSwish_(t, order); break;
      default: return 2;
    }
    dump(t, y);
    return 0;
  } catch (const std::exception&) {
    return 1;
  }
}

void ytref_f32_to_bf16(const float* x, uint16_t* y, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    yt::bfloat16 v(x[i]);
    std::memcpy(&y[i], &v, 2);
  }
}
void ytref_bf16_to_f32(const uint16_t* x, float* y, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    yt::bfloat16 v;
    std::memcpy(&v, &x[i], 2);
    y[i] = static_cast<float>(v);
  }
}
void ytref_f32_to_f16(const float* x, uint16_t* y, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    yt::float16 v(x[i]);
    std::memcpy(&y[i], &v, 2);
  }
}
void ytref_f16_to_f32(const uint16_t* x, float* y, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    yt::float16 v;
    std::memcpy(&v, &x[i], 2);
    y[i] = static_cast<float>(v);
  }
}

// The memory-bound chain: y = softmax(rmsNorm(x, w, -1, eps) + r, -1) cast to bfloat16 with copy_.
// x [B,L,H]; r [B,L,H] when r_batched else [1,L,H].
int ytref_chain_f32(const float* x, const float* w, const float* r, uint16_t* out, int B, int L, int H, int r_batched,
                    float eps) {
  try {
    const int xs[3] = {B, L, H}, ws[1] = {H}, rs[3] = {r_batched ? B : 1, L, H};
    auto xt = make<3>(x, xs);
    auto wt = make<1>(w, ws);
    auto rt = make<3>(r, rs);
    auto y = yt::function::rmsNorm(xt, wt, -1, eps);
    y += rt;
    yt::function::softmax_(y, -1);
    YTensor<yt::bfloat16, 3> o(B, L, H);
    o.copy_(y);
    std::memcpy(out, o.data(), o.size() * 2);
    return 0;
  } catch (const std::exception&) {
    return 1;
  }
}

// ---------------------------------------------------------------- Qwen3 example model
struct RefQwen3 {
  qwen3::Qwen3ForCausalLM lm;
  int batch = 1;
};

void* ytref_qwen3_create(int hidden, int layers, int vocab, int inter, int heads, int kv_heads, int head_dim,
                         float eps, float theta, int max_pos, int batch) {
  try {
    auto* m = new RefQwen3();
    qwen3::Qwen3Config c;
    c.hidden_size = hidden;
    c.num_hidden_layers = layers;
    c.vocab_size = vocab;
    c.intermediate_size = inter;
    c.num_attention_heads = heads;
    c.num_key_value_heads = kv_heads;
    c.head_dim = head_dim;
    c.rms_norm_eps = eps;
    c.rope_theta = theta;
    c.max_position_embeddings = max_pos;
    m->lm.init(c);
    m->batch = batch;
    // The example hard-codes KV-cache batch 1 (qwen3.cpp:415-423): re-init for the asked batch.
    for (auto& cache : m->lm.kv_caches) cache.init(batch, max_pos, kv_heads, head_dim);
    return m;
  } catch (const std::exception&) {
    return nullptr;
  }
}
void ytref_qwen3_destroy(void* h) { delete static_cast<RefQwen3*>(h); }

// name: "embed", "norm", "lm_head", or per layer "qkv", "o", "q_norm", "k_norm", "gate_up", "down", "norm1", "norm2".
int ytref_qwen3_set_weight(void* h, const char* name, int layer, const float* data, int rows, int cols) {
  try {
    auto* m = static_cast<RefQwen3*>(h);
    const std::string n(name);
    auto set2 = [&](YTensor<float, 2>& t) {
      const int s[2] = {rows, cols};
      t = make<2>(data, s);
    };
    auto set1 = [&](YTensor<float, 1>& t) {
      const int s[1] = {rows};
      t = make<1>(data, s);
    };
    if (n == "embed") { set2(m->lm.model.embed); return 0; }
    if (n == "norm") { set1(m->lm.model.norm.weight); return 0; }
    if (n == "lm_head") { set2(m->lm.lm_head); m->lm.use_lm_head = true; return 0; }
    auto& L = m->lm.model.layers.at(layer);
    if (n == "qkv") set2(L.attn.qkv_proj);
    else if (n == "o") set2(L.attn.o_proj);
    else if (n == "q_norm") set1(L.attn.q_norm.weight);
    else if (n == "k_norm") set1(L.attn.k_norm.weight);
    else if (n == "gate_up") set2(L.mlp.gate_up);
    else if (n == "down") set2(L.mlp.down);
    else if (n == "norm1") set1(L.norm1.weight);
    else if (n == "norm2") set1(L.norm2.weight);
    else return 2;
    return 0;
  } catch (const std::exception&) {
    return 1;
  }
}
void ytref_qwen3_reset(void* h) { static_cast<RefQwen3*>(h)->lm.reset_kv_cache(); }

// ids [batch, l] -> logits [batch, vocab] of the last position; updates the KV caches.
int ytref_qwen3_forward(void* h, const int* ids, int l, float* logits) {
  try {
    auto* m = static_cast<RefQwen3*>(h);
    YTensor<int, 2> t(m->batch, l);
    std::memcpy(t.data(), ids, sizeof(int) * static_cast<size_t>(m->batch) * l);
    auto out = m->lm.forward(t, false);
    dump(out, logits);
    return 0;
  } catch (const std::exception&) {
    return 1;
  }
}

}  // extern "C"
