// Host side of the device backend in the reference's own language: yt::cuda::* take and return yt::YTensor<T, N>
// (host-resident, as every YTensor is) and run the work on the GPU through the C ABI of libytensor_cuda.so.
// Include after "ytensor.hpp". Names, argument meaning and exceptions follow the reference entry points they stand
// in for (cited at each function); nothing here computes on the CPU and nothing falls back to it.
//
//   #include "ytensor.hpp"
//   #include "ytensor_cuda.hpp"
//   auto c = yt::cuda::matmul(a, b);                       // YTensor::matmul (masked_matmul likewise)
//   auto o = yt::cuda::scaledDotProductAttention(q, k, v, 0.f, yt::cuda::Causal{kv_len - q_len});
#pragma once
#include <cstdint>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <type_traits>
#include <utility>
#include <vector>

#include "ytcuda.h"

namespace yt::cuda {

// std::invalid_argument for a refused request (as src/ytensor_math.inl:290-292 throws), std::runtime_error otherwise.
inline void check(int status) {
  if (status == YTC_OK) return;
  const std::string msg = ytcuda_last_error_string();
  if (status == YTC_INVALID_ARG || status == YTC_UNSUPPORTED) throw std::invalid_argument(msg);
  throw std::runtime_error(msg);
}

template <typename T>
constexpr int dtype_of() {
  if constexpr (std::is_same_v<T, float>) return YTC_F32;
  else if constexpr (std::is_same_v<T, yt::bfloat16>) return YTC_BF16;
  else if constexpr (std::is_same_v<T, yt::float16>) return YTC_F16;
  else static_assert(sizeof(T) == 0, "the device backend handles float, yt::bfloat16 and yt::float16");
}

// Device memory for the duration of one call.
class DeviceBuffer {
 public:
  explicit DeviceBuffer(size_t bytes) : bytes_(bytes) { check(ytcuda_malloc(&p_, bytes)); }
  ~DeviceBuffer() { ytcuda_free(p_); }
  DeviceBuffer(const DeviceBuffer&) = delete;
  DeviceBuffer& operator=(const DeviceBuffer&) = delete;
  DeviceBuffer(DeviceBuffer&& o) noexcept : p_(o.p_), bytes_(o.bytes_) { o.p_ = nullptr; }
  void* get() const { return p_; }
  void upload(const void* host) { check(ytcuda_memcpy_h2d(p_, host, bytes_, nullptr)); }
  void download(void* host) const {
    check(ytcuda_memcpy_d2h(host, p_, bytes_, nullptr));
    check(ytcuda_stream_sync(nullptr));
  }

 private:
  void* p_ = nullptr;
  size_t bytes_;
};

namespace detail {
template <typename T, int dim>
DeviceBuffer to_device(const yt::YTensor<T, dim>& t) {
  auto c = t.contiguous();
  DeviceBuffer d(c.size() * sizeof(T));
  d.upload(c.data());
  return d;
}
inline std::vector<int64_t> contiguous_strides(const std::vector<int>& shape) {
  std::vector<int64_t> s(shape.size());
  int64_t acc = 1;
  for (int d = static_cast<int>(shape.size()) - 1; d >= 0; --d) {
    s[d] = acc;
    acc *= shape[d];
  }
  return s;
}
inline std::vector<int64_t> widen(const std::vector<int>& v) { return std::vector<int64_t>(v.begin(), v.end()); }
}  // namespace detail

// ------------------------------------------------------------------ matmul / linear
// YTensor<T, dim>::matmul (reference src/ytensor_math.inl:284-316). Supported operand forms, the ones the hot path
// uses: a [..., m, k] with b [k, n] (shared right operand, :960-1018), and a, b of equal rank with equal leading
// dims. The operands stay where they are on the host; their strides go to the device call as they are.
template <typename T, int dim0, int dim1>
auto matmul(const yt::YTensor<T, dim0>& a, const yt::YTensor<T, dim1>& b) {
  static_assert(dim0 >= 2 && dim1 >= 2, "matmul needs rank >= 2 operands");
  constexpr int odim = dim0 > dim1 ? dim0 : dim1;
  if (a.shape(-1) != b.shape(-2)) throw std::invalid_argument("matmul: inner dimensions do not match");
  if constexpr (dim1 != 2) {
    static_assert(dim0 == dim1, "matmul: the right operand is 2-D or has the rank of the left operand");
    for (int d = 0; d < dim0 - 2; ++d)
      if (a.shape(d) != b.shape(d)) throw std::invalid_argument("matmul: batch dimensions do not match");
  }
  const int m = a.shape(-2), k = a.shape(-1), n = b.shape(-1);
  auto ac = a.isContiguous() ? a : a.contiguous();  // leading dims must collapse into one batch stride
  auto bc = (dim1 == 2 || b.isContiguous()) ? b : b.contiguous();
  std::vector<int> oshape = ac.shape();
  oshape[odim - 1] = n;
  yt::YTensor<T, odim> out(oshape);
  int64_t batch = 1;
  for (int d = 0; d < dim0 - 2; ++d) batch *= ac.shape(d);
  const int64_t bsb = (dim1 == 2) ? 0 : static_cast<int64_t>(k) * n;
  check(ytcuda_gemm_host(dtype_of<T>(), dtype_of<T>(), ac.data(), bc.data(), out.data(), m, n, k, 1.0f, 0.0f,
                         ac.stride_(-2), ac.stride_(-1), bc.stride_(-2), bc.stride_(-1), n, 1, batch,
                         static_cast<int64_t>(m) * k, bsb, static_cast<int64_t>(m) * n));
  return out;
}

// YTensor<T, dim>::masked_matmul with a bool mask (reference src/ytensor_math.inl:318-366): products where the mask
// holds, maskedValue elsewhere; a [..., m, k] with b [k, n], mask [m, n] shared by every batch item.
template <typename T, int dim0>
yt::YTensor<T, dim0> masked_matmul(const yt::YTensor<T, dim0>& a, const yt::YTensor<T, 2>& b,
                                   const yt::YTensor<bool, 2>& mask, const T& maskedValue = T{}) {
  static_assert(dim0 >= 2, "masked_matmul needs a rank >= 2 left operand");
  if (a.shape(-1) != b.shape(-2)) throw std::invalid_argument("masked_matmul: inner dimensions do not match");
  const int m = a.shape(-2), k = a.shape(-1), n = b.shape(-1);
  if (mask.shape(0) != m || mask.shape(1) != n) throw std::invalid_argument("masked_matmul: mask shape not match");
  DeviceBuffer da = detail::to_device(a), db = detail::to_device(b), dm = detail::to_device(mask);
  std::vector<int> oshape = a.shape();
  oshape[dim0 - 1] = n;
  yt::YTensor<T, dim0> out(oshape);
  DeviceBuffer dc(out.size() * sizeof(T));
  int64_t batch = 1;
  for (int d = 0; d < dim0 - 2; ++d) batch *= a.shape(d);
  check(ytcuda_gemm_masked(dtype_of<T>(), dtype_of<T>(), da.get(), db.get(), dc.get(), m, n, k, k, 1, n, 1, n, 1, batch,
                           static_cast<int64_t>(m) * k, 0, static_cast<int64_t>(m) * n, dm.get(), n,
                           static_cast<float>(maskedValue), nullptr));
  dc.download(out.data());
  return out;
}

// yt::function::linear: x . weight^T, weight [out_features, in_features] (src/function/ops.inl:84-91). The transpose
// is a view: the device kernel reads the weight with its unit stride along k.
template <typename T, int dim>
yt::YTensor<T, dim> linear(const yt::YTensor<T, dim>& x, const yt::YTensor<T, 2>& weight) {
  return matmul(x, weight.transpose());
}

// ------------------------------------------------------------------ attention
struct Causal {
  int offset;  // key c is visible to query r iff c <= r + offset (the reference's masks use kv_len - q_len)
  // the callable and tile-pruning forms the reference's predicate overloads expect (src/ytensor_math.inl:386,
  // src/kernel/avx2/sgemm.inl:449-475), so that the same object also works with its CPU back-ends
  bool operator()(int r, int c) const { return c <= r + offset; }
  bool tileAllTrue(int r0, int c0, int, int nr) const { return c0 + nr - 1 <= r0 + offset; }
  bool tileAllFalse(int r0, int c0, int mr, int) const { return c0 > r0 + mr - 1 + offset; }
};

// YTensor<T, dim>::masked_matmul with the predicate `c <= r + offset` (reference src/ytensor_math.inl:368-412 with a
// functor that has tileAllTrue / tileAllFalse): the device evaluates the predicate itself and skips the 128 x 128
// output tiles it leaves empty (ytcuda_gemm_masked_causal); no mask tensor is built or uploaded.
template <typename T, int dim0>
yt::YTensor<T, dim0> masked_matmul(const yt::YTensor<T, dim0>& a, const yt::YTensor<T, 2>& b, const Causal& mask,
                                   const T& maskedValue = T{}) {
  static_assert(dim0 >= 2, "masked_matmul needs a rank >= 2 left operand");
  if (a.shape(-1) != b.shape(-2)) throw std::invalid_argument("masked_matmul: inner dimensions do not match");
  const int m = a.shape(-2), k = a.shape(-1), n = b.shape(-1);
  DeviceBuffer da = detail::to_device(a), db = detail::to_device(b);
  std::vector<int> oshape = a.shape();
  oshape[dim0 - 1] = n;
  yt::YTensor<T, dim0> out(oshape);
  DeviceBuffer dc(out.size() * sizeof(T));
  int64_t batch = 1;
  for (int d = 0; d < dim0 - 2; ++d) batch *= a.shape(d);
  check(ytcuda_gemm_masked_causal(dtype_of<T>(), dtype_of<T>(), da.get(), db.get(), dc.get(), m, n, k, k, 1, n, 1, n, 1,
                                  batch, static_cast<int64_t>(m) * k, 0, static_cast<int64_t>(m) * n, mask.offset,
                                  static_cast<float>(maskedValue), nullptr));
  dc.download(out.data());
  return out;
}

namespace detail {
template <typename T>
yt::YTensor<T, 5> sdpa(yt::YTensor<T, 5>& q, yt::YTensor<T, 5>& k, yt::YTensor<T, 5>& v, T scale, int mask_kind,
                       int causal_offset, const yt::YTensor<bool, 2>* mask, const yt::YTensor<T, 2>* bias) {
  if (q.shape(-1) != k.shape(-1)) throw std::invalid_argument("Query and key head dim must match.");
  if (k.shape(-2) != v.shape(-2)) throw std::invalid_argument("Key/value sequence length must match.");
  const int b = q.shape(0), kvh = q.shape(1), g = q.shape(2), lq = q.shape(3), d = q.shape(4);
  const int lk = k.shape(3), dv = v.shape(4);
  if (mask && (mask->shape(0) != lq || mask->shape(1) != lk))
    throw std::invalid_argument("Mask shape must match the last two dimensions of the score tensor.");
  if (bias && (bias->shape(0) != lq || bias->shape(1) != lk))
    throw std::invalid_argument("Bias shape must match the last two dimensions of the score tensor.");
  // K / V arrive repeated over the group dim by a zero stride (example/qwen3/src/qwen3.cpp:252-264): take group 0
  auto k4 = yt::YTensor<T, 4>(k.slice(2, 0, 1).reshape(b, kvh, lk, d)).contiguous();
  auto v4 = yt::YTensor<T, 4>(v.slice(2, 0, 1).reshape(b, kvh, lk, dv)).contiguous();
  DeviceBuffer dq = to_device(q), dk = to_device(k4), dvv = to_device(v4);
  yt::YTensor<T, 5> out(b, kvh, g, lq, dv);
  DeviceBuffer dout(out.size() * sizeof(T));
  const int64_t qs[3] = {static_cast<int64_t>(kvh) * g * lq * d, static_cast<int64_t>(lq) * d, d};
  const int64_t ks[3] = {static_cast<int64_t>(kvh) * lk * d, static_cast<int64_t>(lk) * d, d};
  const int64_t vs[3] = {static_cast<int64_t>(kvh) * lk * dv, static_cast<int64_t>(lk) * dv, dv};
  const int64_t os[3] = {static_cast<int64_t>(kvh) * g * lq * dv, static_cast<int64_t>(lq) * dv, dv};
  std::vector<uint8_t> m8;
  DeviceBuffer dmask(mask ? static_cast<size_t>(lq) * lk : 16);
  if (mask) {
    m8.resize(static_cast<size_t>(lq) * lk);
    for (int r = 0; r < lq; ++r)
      for (int c = 0; c < lk; ++c) m8[static_cast<size_t>(r) * lk + c] = mask->at(r, c) ? 1 : 0;
    dmask.upload(m8.data());
  }
  std::vector<float> bf;
  DeviceBuffer dbias(bias ? static_cast<size_t>(lq) * lk * sizeof(float) : 16);
  if (bias) {
    bf.resize(static_cast<size_t>(lq) * lk);
    for (int r = 0; r < lq; ++r)
      for (int c = 0; c < lk; ++c) bf[static_cast<size_t>(r) * lk + c] = static_cast<float>(bias->at(r, c));
    dbias.upload(bf.data());
  }
  check(ytcuda_flash_attn_fwd(dtype_of<T>(), dq.get(), dk.get(), dvv.get(), dout.get(), b, kvh, g, lq, lk, d, dv,
                              static_cast<float>(scale), qs, ks, vs, os, mask_kind, causal_offset,
                              mask ? static_cast<const uint8_t*>(dmask.get()) : nullptr, lk,
                              bias ? static_cast<const float*>(dbias.get()) : nullptr, lk, 1, nullptr));
  dout.download(out.data());
  return out;
}
}  // namespace detail

// yt::function::scaledDotProductAttention with a bool mask / no mask (src/function/ops.inl:368-425), on the 5-D
// [b, kv_heads, groups, len, dim] form its callers use.
template <typename T>
yt::YTensor<T, 5> scaledDotProductAttention(yt::YTensor<T, 5>& q, yt::YTensor<T, 5>& k, yt::YTensor<T, 5>& v,
                                            T scale = static_cast<T>(0.0), yt::YTensor<bool, 2>* mask = nullptr,
                                            yt::YTensor<T, 2>* bias = nullptr) {
  return detail::sdpa(q, k, v, scale, mask ? 2 : 0, 0, mask, bias);
}
// The predicate form (src/function/ops.inl:427-503) for the one predicate device code can evaluate: causal.
template <typename T>
yt::YTensor<T, 5> scaledDotProductAttention(yt::YTensor<T, 5>& q, yt::YTensor<T, 5>& k, yt::YTensor<T, 5>& v, T scale,
                                            Causal causal, yt::YTensor<T, 2>* bias = nullptr) {
  return detail::sdpa<T>(q, k, v, scale, 1, causal.offset, nullptr, bias);
}

// ------------------------------------------------------------------ softmax / norms / reductions
// yt::function::softmax (src/function/activation.inl:336-375)
template <typename T, int dim>
yt::YTensor<T, dim> softmax(const yt::YTensor<T, dim>& x, const std::vector<int>& axes) {
  DeviceBuffer dx = detail::to_device(x);
  yt::YTensor<T, dim> y(x.shape());
  DeviceBuffer dy(y.size() * sizeof(T));
  const auto shape = detail::widen(x.shape());
  const auto st = detail::contiguous_strides(x.shape());
  check(ytcuda_softmax(dtype_of<T>(), dtype_of<T>(), dx.get(), dy.get(), shape.data(), st.data(), st.data(), dim,
                       axes.data(), static_cast<int>(axes.size()), nullptr));
  dy.download(y.data());
  return y;
}
template <typename T, int dim>
yt::YTensor<T, dim> softmax(const yt::YTensor<T, dim>& x, int axis = -1) {
  return softmax(x, std::vector<int>{axis});
}

// yt::function::rmsNorm (src/function/normalization.inl:234-277); weight has one dim per axis
template <typename T, int dim, int wdim>
yt::YTensor<T, dim> rmsNorm(const yt::YTensor<T, dim>& x, const yt::YTensor<T, wdim>& weight,
                            const std::vector<int>& axes, T eps = static_cast<T>(1e-5)) {
  if (static_cast<int>(axes.size()) != wdim) throw std::invalid_argument("rmsNorm: weight dim must match axes size");
  for (int i = 0; i < wdim; ++i)
    if (weight.shape(i) != x.shape(axes[i])) throw std::invalid_argument("rmsNorm: weight shape must match affine axes");
  DeviceBuffer dx = detail::to_device(x), dw = detail::to_device(weight);
  yt::YTensor<T, dim> y(x.shape());
  DeviceBuffer dy(y.size() * sizeof(T));
  const auto shape = detail::widen(x.shape());
  const auto st = detail::contiguous_strides(x.shape());
  check(ytcuda_rmsnorm(dtype_of<T>(), dtype_of<T>(), dtype_of<T>(), dx.get(), dw.get(), dy.get(), shape.data(),
                       st.data(), st.data(), dim, axes.data(), wdim, static_cast<float>(eps), nullptr));
  dy.download(y.data());
  return y;
}
template <typename T, int dim, int wdim>
yt::YTensor<T, dim> rmsNorm(const yt::YTensor<T, dim>& x, const yt::YTensor<T, wdim>& weight, int axis = -1,
                            T eps = static_cast<T>(1e-5)) {
  return rmsNorm(x, weight, std::vector<int>{axis}, eps);
}

// yt::function::layerNorm with gamma and bias (src/function/normalization.inl:188-230)
template <typename T, int dim, int gdim>
yt::YTensor<T, dim> layerNorm(const yt::YTensor<T, dim>& x, const yt::YTensor<T, gdim>& gamma,
                              const yt::YTensor<T, gdim>& bias, const std::vector<int>& axes,
                              T eps = static_cast<T>(1e-5)) {
  if (static_cast<int>(axes.size()) != gdim) throw std::invalid_argument("layerNorm: gamma dim must match axes size");
  DeviceBuffer dx = detail::to_device(x), dg = detail::to_device(gamma), db = detail::to_device(bias);
  yt::YTensor<T, dim> y(x.shape());
  DeviceBuffer dy(y.size() * sizeof(T));
  const auto shape = detail::widen(x.shape());
  const auto st = detail::contiguous_strides(x.shape());
  check(ytcuda_layernorm(dtype_of<T>(), dtype_of<T>(), dtype_of<T>(), dx.get(), dg.get(), db.get(), dy.get(),
                         shape.data(), st.data(), st.data(), dim, axes.data(), gdim, static_cast<float>(eps), nullptr));
  dy.download(y.data());
  return y;
}

// yt::function::normalize without gamma / bias: x / (sum_axes |x|^p + eps)^(1/p)
// (include/function/normalization.hpp:91-107, src/function/normalization.inl:56-85, 278-318)
template <typename T, int dim>
yt::YTensor<T, dim> normalize(const yt::YTensor<T, dim>& x, const std::vector<int>& axes, T p = static_cast<T>(2),
                              T eps = static_cast<T>(1e-12)) {
  if (!(static_cast<float>(p) > 0.f)) throw std::invalid_argument("yt::function::normalize: p must be positive");
  DeviceBuffer dx = detail::to_device(x);
  yt::YTensor<T, dim> y(x.shape());
  DeviceBuffer dy(y.size() * sizeof(T));
  const auto shape = detail::widen(x.shape());
  const auto st = detail::contiguous_strides(x.shape());
  check(ytcuda_normalize(dtype_of<T>(), dtype_of<T>(), dx.get(), dy.get(), shape.data(), st.data(), st.data(), dim,
                         axes.data(), static_cast<int>(axes.size()), static_cast<float>(p), static_cast<float>(eps),
                         nullptr));
  dy.download(y.data());
  return y;
}
template <typename T, int dim>
yt::YTensor<T, dim> normalize(const yt::YTensor<T, dim>& x, int axis = -1, T p = static_cast<T>(2),
                              T eps = static_cast<T>(1e-12)) {
  return normalize(x, std::vector<int>{axis}, p, eps);
}

namespace detail {
// (x - mean) / sqrt(var + eps) over `axes` of a tensor given by shape and element strides (any view), no affine part
template <typename T>
void standardize(const void* dx, void* dy, const std::vector<int64_t>& shape, const std::vector<int64_t>& strides,
                 const std::vector<int>& axes, float eps) {
  check(ytcuda_layernorm(dtype_of<T>(), dtype_of<T>(), dtype_of<T>(), dx, nullptr, nullptr, dy, shape.data(),
                         strides.data(), strides.data(), static_cast<int>(shape.size()), axes.data(),
                         static_cast<int>(axes.size()), eps, nullptr));
}
template <typename T, int dim>
int channel_axis(const yt::YTensor<T, dim>&, int channelAxis, const char* who) {
  static_assert(dim >= 2, "requires dim >= 2");
  const int c = ((channelAxis % dim) + dim) % dim;
  if (c == 0) throw std::invalid_argument(std::string(who) + ": channelAxis must not be batch axis 0");
  return c;
}
}  // namespace detail

// yt::function::instanceNorm without gamma / bias: every (sample, channel) standardised over the remaining axes
// (include/function/normalization.hpp:166-172, src/function/normalization.inl:378-433)
template <typename T, int dim>
yt::YTensor<T, dim> instanceNorm(const yt::YTensor<T, dim>& x, int channelAxis = 1, T eps = static_cast<T>(1e-5)) {
  const int c = detail::channel_axis(x, channelAxis, "yt::function::instanceNorm_");
  std::vector<int> axes;
  for (int a = 1; a < dim; ++a)
    if (a != c) axes.push_back(a);
  if (axes.empty()) throw std::invalid_argument("yt::function::instanceNorm: requires at least one spatial axis");
  DeviceBuffer dx = detail::to_device(x);
  yt::YTensor<T, dim> y(x.shape());
  DeviceBuffer dy(y.size() * sizeof(T));
  detail::standardize<T>(dx.get(), dy.get(), detail::widen(x.shape()), detail::contiguous_strides(x.shape()), axes,
                         static_cast<float>(eps));
  dy.download(y.data());
  return y;
}

// yt::function::batchNorm without gamma / bias: every channel standardised over all other axes, batch included;
// statistics of the tensor itself (include/function/normalization.hpp:199-205, src/function/normalization.inl:435-489)
template <typename T, int dim>
yt::YTensor<T, dim> batchNorm(const yt::YTensor<T, dim>& x, int channelAxis = 1, T eps = static_cast<T>(1e-5)) {
  const int c = detail::channel_axis(x, channelAxis, "yt::function::batchNorm_");
  std::vector<int> axes;
  for (int a = 0; a < dim; ++a)
    if (a != c) axes.push_back(a);
  DeviceBuffer dx = detail::to_device(x);
  yt::YTensor<T, dim> y(x.shape());
  DeviceBuffer dy(y.size() * sizeof(T));
  detail::standardize<T>(dx.get(), dy.get(), detail::widen(x.shape()), detail::contiguous_strides(x.shape()), axes,
                         static_cast<float>(eps));
  dy.download(y.data());
  return y;
}

// yt::function::groupNorm without gamma / bias (include/function/normalization.hpp:232-239,
// src/function/normalization.inl:491-577): every (sample, group of channels) standardised over the group's channels
// and the remaining axes. The grouped tensor is a strided VIEW [n, groups, channels / groups, rest...] of x and of
// the result: the channel axis is split and moved next to the batch axis in the shape / stride lists only.
template <typename T, int dim>
yt::YTensor<T, dim> groupNorm(const yt::YTensor<T, dim>& x, int groups, int channelAxis = 1,
                              T eps = static_cast<T>(1e-5)) {
  const int c = detail::channel_axis(x, channelAxis, "yt::function::groupNorm_");
  if (groups <= 0) throw std::invalid_argument("yt::function::groupNorm: groups must be positive");
  const int ch = x.shape(c);
  if (ch % groups) throw std::invalid_argument("yt::function::groupNorm: channel count must be divisible by groups");
  static_assert(dim + 1 <= 8, "groupNorm: at most 7 dims");
  const auto st = detail::contiguous_strides(x.shape());
  std::vector<int64_t> gshape = {x.shape(0), groups, ch / groups}, gstride = {st[0], st[c] * (ch / groups), st[c]};
  for (int a = 1; a < dim; ++a)
    if (a != c) {
      gshape.push_back(x.shape(a));
      gstride.push_back(st[a]);
    }
  std::vector<int> axes;
  for (int a = 2; a < static_cast<int>(gshape.size()); ++a) axes.push_back(a);
  DeviceBuffer dx = detail::to_device(x);
  yt::YTensor<T, dim> y(x.shape());
  DeviceBuffer dy(y.size() * sizeof(T));
  detail::standardize<T>(dx.get(), dy.get(), gshape, gstride, axes, static_cast<float>(eps));
  dy.download(y.data());
  return y;
}

namespace detail {
template <typename T, int dim>
std::pair<yt::YTensor<T, dim>, yt::YTensor<int, dim>> reduce(int op, const yt::YTensor<T, dim>& x,
                                                             const std::vector<int>& axes) {
  auto oshape = x.shape();
  for (int a : axes) oshape[((a % dim) + dim) % dim] = 1;
  yt::YTensor<T, dim> y(oshape);
  yt::YTensor<int, dim> idx(oshape);
  DeviceBuffer dx = to_device(x), dy(y.size() * sizeof(T)), di(idx.size() * sizeof(int));
  const auto shape = widen(x.shape());
  const auto st = contiguous_strides(x.shape());
  check(ytcuda_reduce(op, dtype_of<T>(), dtype_of<T>(), dx.get(), dy.get(), static_cast<int32_t*>(di.get()),
                      shape.data(), st.data(), dim, axes.data(), static_cast<int>(axes.size()), nullptr));
  dy.download(y.data());
  if (op == 2) di.download(idx.data());
  return {y, idx};
}
}  // namespace detail

// YTensor::sum / mean / max (src/ytensor_math.inl:414-692), keep-dim
template <typename T, int dim>
yt::YTensor<T, dim> sum(const yt::YTensor<T, dim>& x, const std::vector<int>& axes) {
  return detail::reduce(0, x, axes).first;
}
template <typename T, int dim>
yt::YTensor<T, dim> mean(const yt::YTensor<T, dim>& x, const std::vector<int>& axes) {
  return detail::reduce(1, x, axes).first;
}
template <typename T, int dim>
std::pair<yt::YTensor<T, dim>, yt::YTensor<int, dim>> max(const yt::YTensor<T, dim>& x, const std::vector<int>& axes) {
  return detail::reduce(2, x, axes);
}

// ------------------------------------------------------------------ elementwise
namespace detail {
template <typename T, int dim>
yt::YTensor<T, dim> binary(int op, const yt::YTensor<T, dim>& a, const yt::YTensor<T, dim>& b) {
  std::vector<int> oshape(dim);
  for (int d = 0; d < dim; ++d) {
    if (a.shape(d) != b.shape(d) && a.shape(d) != 1 && b.shape(d) != 1)
      throw std::runtime_error("broadcast: shapes do not match");  // std::runtime_error, src/kernel/broadcast.inl:133
    oshape[d] = a.shape(d) > b.shape(d) ? a.shape(d) : b.shape(d);
  }
  yt::YTensor<T, dim> out(oshape);
  DeviceBuffer da = to_device(a), db = to_device(b), dout(out.size() * sizeof(T));
  auto as = contiguous_strides(a.shape()), bs = contiguous_strides(b.shape());
  for (int d = 0; d < dim; ++d) {
    if (a.shape(d) == 1) as[d] = 0;
    if (b.shape(d) == 1) bs[d] = 0;
  }
  const auto os = contiguous_strides(oshape);
  const auto shape = widen(oshape);
  check(ytcuda_binary(op, dtype_of<T>(), dtype_of<T>(), dtype_of<T>(), da.get(), db.get(), dout.get(), dim,
                      shape.data(), as.data(), bs.data(), os.data(), nullptr));
  dout.download(out.data());
  return out;
}
}  // namespace detail

// the operator macros (src/ytensor_math.inl:22-124) for same-rank operands with size-1 broadcasting
template <typename T, int dim> yt::YTensor<T, dim> add(const yt::YTensor<T, dim>& a, const yt::YTensor<T, dim>& b) { return detail::binary(0, a, b); }
template <typename T, int dim> yt::YTensor<T, dim> sub(const yt::YTensor<T, dim>& a, const yt::YTensor<T, dim>& b) { return detail::binary(1, a, b); }
template <typename T, int dim> yt::YTensor<T, dim> mul(const yt::YTensor<T, dim>& a, const yt::YTensor<T, dim>& b) { return detail::binary(2, a, b); }
template <typename T, int dim> yt::YTensor<T, dim> div(const yt::YTensor<T, dim>& a, const yt::YTensor<T, dim>& b) { return detail::binary(3, a, b); }

namespace detail {
template <typename T, int dim>
yt::YTensor<T, dim> unary(int op, const yt::YTensor<T, dim>& x, float param = 0.f) {
  DeviceBuffer dx = to_device(x);
  yt::YTensor<T, dim> y(x.shape());
  DeviceBuffer dy(y.size() * sizeof(T));
  const auto shape = widen(x.shape());
  const auto st = contiguous_strides(x.shape());
  check(ytcuda_unary(op, dtype_of<T>(), dtype_of<T>(), dx.get(), dy.get(), dim, shape.data(), st.data(), st.data(),
                     param, nullptr));
  dy.download(y.data());
  return y;
}
}  // namespace detail

namespace detail {
inline int act_op(int op, int order) {
  if (order == 0) return op;
  if (order == 1) return op + 32;
  throw std::invalid_argument("yt::cuda activation: only order 0 and 1 run on the device");
}
}  // namespace detail

// the activations of yt::function (include/function/activation.hpp:9-109): order 0 the function, 1 its first derivative
template <typename T, int dim> yt::YTensor<T, dim> swish(const yt::YTensor<T, dim>& x, int order = 0) { return detail::unary(detail::act_op(1, order), x); }
template <typename T, int dim> yt::YTensor<T, dim> relu(const yt::YTensor<T, dim>& x, int order = 0) { return detail::unary(detail::act_op(4, order), x); }
template <typename T, int dim> yt::YTensor<T, dim> exp(const yt::YTensor<T, dim>& x, int order = 0) { return detail::unary(detail::act_op(5, order), x); }
template <typename T, int dim> yt::YTensor<T, dim> sigmoid(const yt::YTensor<T, dim>& x, int order = 0) { return detail::unary(detail::act_op(6, order), x); }
template <typename T, int dim> yt::YTensor<T, dim> leakyRelu(const yt::YTensor<T, dim>& x, float alpha = 0.01f, int order = 0) { return detail::unary(detail::act_op(7, order), x, alpha); }
template <typename T, int dim> yt::YTensor<T, dim> elu(const yt::YTensor<T, dim>& x, float alpha = 1.0f, int order = 0) { return detail::unary(detail::act_op(8, order), x, alpha); }
template <typename T, int dim> yt::YTensor<T, dim> selu(const yt::YTensor<T, dim>& x, int order = 0) { return detail::unary(detail::act_op(9, order), x); }
template <typename T, int dim> yt::YTensor<T, dim> gelu(const yt::YTensor<T, dim>& x, int order = 0) { return detail::unary(detail::act_op(10, order), x); }
template <typename T, int dim> yt::YTensor<T, dim> tanh(const yt::YTensor<T, dim>& x, int order = 0) { return detail::unary(detail::act_op(11, order), x); }
template <typename T, int dim> yt::YTensor<T, dim> softplus(const yt::YTensor<T, dim>& x, int order = 0) { return detail::unary(detail::act_op(12, order), x); }
template <typename T, int dim> yt::YTensor<T, dim> mish(const yt::YTensor<T, dim>& x, int order = 0) { return detail::unary(detail::act_op(13, order), x); }
template <typename T, int dim> yt::YTensor<T, dim> hardSigmoid(const yt::YTensor<T, dim>& x, int order = 0) { return detail::unary(detail::act_op(14, order), x); }
template <typename T, int dim> yt::YTensor<T, dim> hardSwish(const yt::YTensor<T, dim>& x, int order = 0) { return detail::unary(detail::act_op(15, order), x); }

// YTensorBase::cast / copy_ between float, bfloat16 and float16 (src/ytensor_base.inl:257-430), bit-exact with the
// reference's own constructors
template <typename U, typename T, int dim>
yt::YTensor<U, dim> cast(const yt::YTensor<T, dim>& x) {
  DeviceBuffer dx = detail::to_device(x);
  yt::YTensor<U, dim> y(x.shape());
  DeviceBuffer dy(y.size() * sizeof(U));
  const auto shape = detail::widen(x.shape());
  const auto st = detail::contiguous_strides(x.shape());
  check(ytcuda_cast(dtype_of<T>(), dtype_of<U>(), dx.get(), dy.get(), dim, shape.data(), st.data(), st.data(), nullptr));
  dy.download(y.data());
  return y;
}


// ------------------------------------------------------------------ device-resident tensors
// A device-resident tensor IS a yt::YTensor<T, dim>: its storage comes from ytcuda_malloc and is released by
// ytcuda_free through the deleter of the tensor's std::shared_ptr<char[]> (the hook the reference already uses for
// its own storage, include/ytensor_base.hpp:388-393, src/ytensor_base.inl:51-58). Shape, strides, offset, views
// (slice / transpose / reshape) and shallow copies work as on any YTensor; element access (at(), printing, host
// loops) must not be used on it. The functions of yt::cuda::dev below take and return such tensors and copy nothing
// between host and device, so that a chain of operators pays PCIe once on the way in and once on the way out.
namespace detail {
template <typename T, int dim>
class DeviceBacked : public yt::YTensor<T, dim> {
 public:
  explicit DeviceBacked(const std::vector<int>& shape) {
    if (static_cast<int>(shape.size()) != dim) throw std::invalid_argument("device tensor: wrong number of dims");
    size_t n = 1;
    for (int v : shape) {
      if (v < 0) throw std::invalid_argument("device tensor: negative extent");
      n *= static_cast<size_t>(v);
    }
    void* p = nullptr;
    check(ytcuda_malloc(&p, n * sizeof(T) > 0 ? n * sizeof(T) : 1));
    this->_data = std::shared_ptr<char[]>(static_cast<char*>(p), [](char* q) { ytcuda_free(q); });
    this->_shape = shape;
    this->_stride.assign(dim, 1);
    for (int d = dim - 2; d >= 0; --d) this->_stride[d] = this->_stride[d + 1] * shape[d + 1];
    this->_offset = 0;
    this->_element_size = sizeof(T);
    this->_dtype = yt::types::getTypeName<T>();
  }
};
template <typename T, int dim>
std::vector<int64_t> strides_of(const yt::YTensor<T, dim>& t) {
  std::vector<int64_t> s(dim);
  for (int d = 0; d < dim; ++d) s[d] = t.stride_(d);
  return s;
}
}  // namespace detail

// True when the tensor's storage is device memory.
template <typename T, int dim>
bool on_device(const yt::YTensor<T, dim>& t) {
  return t.size() > 0 && ytcuda_pointer_is_device(t.data()) != 0;
}

// A new device-resident tensor (contents undefined).
template <typename T, int dim>
yt::YTensor<T, dim> empty_device(const std::vector<int>& shape) {
  const detail::DeviceBacked<T, dim> backed(shape);
  const yt::YTensor<T, dim>& as_tensor = backed;  // (the copy constructor: shares the storage)
  return yt::YTensor<T, dim>(as_tensor);
}
// One upload: a contiguous device-resident copy of a host tensor.
template <typename T, int dim>
yt::YTensor<T, dim> to_device(const yt::YTensor<T, dim>& host) {
  auto c = host.isContiguous() ? host : host.contiguous();
  auto d = empty_device<T, dim>(c.shape());
  check(ytcuda_memcpy_h2d(d.data(), c.data(), c.size() * sizeof(T), nullptr));
  check(ytcuda_stream_sync(nullptr));
  return d;
}
// One download: a host tensor with the contents of a device-resident one (any strides).
template <typename T, int dim>
yt::YTensor<T, dim> to_host(const yt::YTensor<T, dim>& dev_t);

namespace dev {
// contiguous device copy of a device tensor with any strides (ytcuda_cast with equal types is a strided copy)
template <typename T, int dim>
yt::YTensor<T, dim> contiguous(const yt::YTensor<T, dim>& x) {
  if (x.isContiguous()) return x;
  auto y = empty_device<T, dim>(x.shape());
  const auto shape = detail::widen(x.shape());
  const auto xs = detail::strides_of(x), ys = detail::strides_of(y);
  check(ytcuda_cast(dtype_of<T>(), dtype_of<T>(), x.data(), y.data(), dim, shape.data(), xs.data(), ys.data(), nullptr));
  return y;
}

// YTensor::matmul on device-resident operands (same operand forms as yt::cuda::matmul); the result stays on the device.
template <typename T, int dim0, int dim1>
auto matmul(const yt::YTensor<T, dim0>& a, const yt::YTensor<T, dim1>& b) {
  static_assert(dim0 >= 2 && dim1 >= 2, "matmul needs rank >= 2 operands");
  static_assert(dim1 == 2 || dim0 == dim1, "matmul: the right operand is 2-D or has the rank of the left operand");
  if (a.shape(-1) != b.shape(-2)) throw std::invalid_argument("matmul: inner dimensions do not match");
  if constexpr (dim1 != 2)
    for (int d = 0; d < dim0 - 2; ++d)
      if (a.shape(d) != b.shape(d)) throw std::invalid_argument("matmul: batch dimensions do not match");
  const int m = a.shape(-2), k = a.shape(-1), n = b.shape(-1);
  auto ac = dim0 == 2 ? a : contiguous(a);  // leading dims must collapse into one batch stride
  auto bc = dim1 == 2 ? b : contiguous(b);
  std::vector<int> oshape = ac.shape();
  oshape[dim0 - 1] = n;
  auto out = empty_device<T, dim0>(oshape);
  int64_t batch = 1;
  for (int d = 0; d < dim0 - 2; ++d) batch *= ac.shape(d);
  check(ytcuda_gemm(dtype_of<T>(), dtype_of<T>(), ac.data(), bc.data(), out.data(), m, n, k, 1.0f, 0.0f, ac.stride_(-2),
                    ac.stride_(-1), bc.stride_(-2), bc.stride_(-1), n, 1, batch, static_cast<int64_t>(m) * k,
                    dim1 == 2 ? 0 : static_cast<int64_t>(k) * n, static_cast<int64_t>(m) * n, nullptr));
  return out;
}

// yt::function::softmax_ (src/function/activation.inl:376-409) in place on a device tensor, any strides.
template <typename T, int dim>
yt::YTensor<T, dim>& softmax_(yt::YTensor<T, dim>& x, const std::vector<int>& axes) {
  const auto shape = detail::widen(x.shape());
  const auto st = detail::strides_of(x);
  check(ytcuda_softmax(dtype_of<T>(), dtype_of<T>(), x.data(), x.data(), shape.data(), st.data(), st.data(), dim,
                       axes.data(), static_cast<int>(axes.size()), nullptr));
  return x;
}
template <typename T, int dim>
yt::YTensor<T, dim> softmax(const yt::YTensor<T, dim>& x, const std::vector<int>& axes) {
  auto y = empty_device<T, dim>(x.shape());
  const auto shape = detail::widen(x.shape());
  const auto xs = detail::strides_of(x), ys = detail::strides_of(y);
  check(ytcuda_softmax(dtype_of<T>(), dtype_of<T>(), x.data(), y.data(), shape.data(), xs.data(), ys.data(), dim,
                       axes.data(), static_cast<int>(axes.size()), nullptr));
  return y;
}

// yt::function::rmsNorm_ / rmsNorm (src/function/normalization.inl:234-277) on device tensors; the weight (device
// resident, one dim per axis, contiguous) multiplies after the division.
template <typename T, int dim, int wdim>
void rmsNorm_into(const yt::YTensor<T, dim>& x, const yt::YTensor<T, wdim>& weight, const std::vector<int>& axes, T eps,
                  yt::YTensor<T, dim>& y) {
  if (static_cast<int>(axes.size()) != wdim) throw std::invalid_argument("rmsNorm: weight dim must match axes size");
  for (int i = 0; i < wdim; ++i)
    if (weight.shape(i) != x.shape(axes[i])) throw std::invalid_argument("rmsNorm: weight shape must match affine axes");
  auto w = contiguous(weight);
  const auto shape = detail::widen(x.shape());
  const auto xs = detail::strides_of(x), ys = detail::strides_of(y);
  check(ytcuda_rmsnorm(dtype_of<T>(), dtype_of<T>(), dtype_of<T>(), x.data(), w.data(), y.data(), shape.data(),
                       xs.data(), ys.data(), dim, axes.data(), wdim, static_cast<float>(eps), nullptr));
}
template <typename T, int dim, int wdim>
yt::YTensor<T, dim>& rmsNorm_(yt::YTensor<T, dim>& x, const yt::YTensor<T, wdim>& weight, const std::vector<int>& axes,
                              T eps) {
  rmsNorm_into(x, weight, axes, eps, x);
  return x;
}
template <typename T, int dim, int wdim>
yt::YTensor<T, dim> rmsNorm(const yt::YTensor<T, dim>& x, const yt::YTensor<T, wdim>& weight,
                            const std::vector<int>& axes, T eps) {
  auto y = empty_device<T, dim>(x.shape());
  rmsNorm_into(x, weight, axes, eps, y);
  return y;
}

// The in-place operators += -= *= /= (src/ytensor_math.inl:35-49) with the right operand broadcast over `a` by the
// reference's rule: shapes are aligned at the last dim and a size-1 (or missing) dim of b repeats.
template <typename T, int dim, int dim1>
yt::YTensor<T, dim>& binary_(int op, yt::YTensor<T, dim>& a, const yt::YTensor<T, dim1>& b) {
  static_assert(dim1 <= dim, "in-place operator: the right operand may not have more dims than the left");
  std::vector<int64_t> bs(dim, 0);
  for (int d = 0; d < dim1; ++d) {
    const int ad = dim - dim1 + d;
    if (b.shape(d) != a.shape(ad) && b.shape(d) != 1)
      throw std::runtime_error("broadcast: shapes do not match");  // std::runtime_error, src/kernel/broadcast.inl:133
    bs[ad] = b.shape(d) == 1 ? 0 : b.stride_(d);
  }
  const auto shape = detail::widen(a.shape());
  const auto as = detail::strides_of(a);
  check(ytcuda_binary(op, dtype_of<T>(), dtype_of<T>(), dtype_of<T>(), a.data(), b.data(), a.data(), dim, shape.data(),
                      as.data(), bs.data(), as.data(), nullptr));
  return a;
}

// YTensorBase::copy_ / cast between device tensors (src/ytensor_base.inl:257-430): strided, with the reference's
// own float -> bfloat16 / float16 rounding.
template <typename U, typename T, int dim>
yt::YTensor<U, dim>& copy_(yt::YTensor<U, dim>& dst, const yt::YTensor<T, dim>& src) {
  if (dst.shape() != src.shape()) throw std::invalid_argument("copy_: shapes do not match");
  const auto shape = detail::widen(src.shape());
  const auto xs = detail::strides_of(src), ys = detail::strides_of(dst);
  check(ytcuda_cast(dtype_of<T>(), dtype_of<U>(), src.data(), dst.data(), dim, shape.data(), xs.data(), ys.data(),
                    nullptr));
  return dst;
}
template <typename U, typename T, int dim>
yt::YTensor<U, dim> cast(const yt::YTensor<T, dim>& x) {
  auto y = empty_device<U, dim>(x.shape());
  return copy_(y, x);
}

// scaledDotProductAttention on device tensors: query [b, kv_heads, groups, lq, d] with key / value either
// [b, kv_heads, groups (stride 0), lk, d] as example/qwen3/src/qwen3.cpp:252-264 builds them, or any equal-rank form
// whose leading dims are then all "heads". mask_kind as in ytcuda_flash_attn_fwd; mask / bias device pointers.
template <typename T, int dim>
yt::YTensor<T, dim> sdpa(const yt::YTensor<T, dim>& q, const yt::YTensor<T, dim>& k, const yt::YTensor<T, dim>& v,
                         T scale, int mask_kind, int causal_offset, const uint8_t* mask_dev, const float* bias_dev) {
  static_assert(dim >= 2, "attention needs [..., len, dim] operands");
  const int lq = q.shape(-2), d = q.shape(-1), lk = k.shape(-2), dv = v.shape(-1);
  std::vector<int> oshape = q.shape();
  oshape[dim - 1] = dv;
  auto out = empty_device<T, dim>(oshape);
  int b = 1, kvh = 1, g = 1;
  int64_t qs[3], ks[3], vs[3], os[3];
  bool gqa = false;
  if constexpr (dim == 5) gqa = k.stride_(2) == 0 && v.stride_(2) == 0 && q.isContiguous() && k.stride_(4) == 1 && v.stride_(4) == 1;
  if (gqa) {
    if constexpr (dim == 5) {
      b = q.shape(0); kvh = q.shape(1); g = q.shape(2);
      qs[0] = q.stride_(0); qs[1] = q.stride_(2); qs[2] = q.stride_(3);
      ks[0] = k.stride_(0); ks[1] = k.stride_(1); ks[2] = k.stride_(3);
      vs[0] = v.stride_(0); vs[1] = v.stride_(1); vs[2] = v.stride_(3);
      os[0] = out.stride_(0); os[1] = out.stride_(2); os[2] = out.stride_(3);
      check(ytcuda_flash_attn_fwd(dtype_of<T>(), q.data(), k.data(), v.data(), out.data(), b, kvh, g, lq, lk, d, dv,
                                  static_cast<float>(scale), qs, ks, vs, os, mask_kind, causal_offset, mask_dev, lk,
                                  bias_dev, lk, 1, nullptr));
    }
    return out;
  }
  auto qc = contiguous(q), kc = contiguous(k), vc = contiguous(v);
  for (int i = 0; i < dim - 2; ++i) kvh *= q.shape(i);
  qs[0] = 0; qs[1] = static_cast<int64_t>(lq) * d; qs[2] = d;
  ks[0] = 0; ks[1] = static_cast<int64_t>(lk) * d; ks[2] = d;
  vs[0] = 0; vs[1] = static_cast<int64_t>(lk) * dv; vs[2] = dv;
  os[0] = 0; os[1] = static_cast<int64_t>(lq) * dv; os[2] = dv;
  check(ytcuda_flash_attn_fwd(dtype_of<T>(), qc.data(), kc.data(), vc.data(), out.data(), b, kvh, g, lq, lk, d, dv,
                              static_cast<float>(scale), qs, ks, vs, os, mask_kind, causal_offset, mask_dev, lk,
                              bias_dev, lk, 1, nullptr));
  return out;
}
}  // namespace dev

template <typename T, int dim>
yt::YTensor<T, dim> to_host(const yt::YTensor<T, dim>& dev_t) {
  auto c = dev::contiguous(dev_t);
  yt::YTensor<T, dim> h(c.shape());
  check(ytcuda_memcpy_d2h(h.data(), c.data(), c.size() * sizeof(T), nullptr));
  check(ytcuda_stream_sync(nullptr));
  return h;
}

// ------------------------------------------------------------------ the seam: what YTensor's own entry points call
// With -DYT_USE_CUDA=1 the reference's dispatch sites gain one branch each (matmul's switch on MatmulBackend, the
// sdpaBackend tests of scaledDotProductAttention, the first lines of softmax / softmax_ / rmsNorm / rmsNorm_ /
// copy_ and of the in-place operators); those branches are one-line calls into this namespace. Operators asked for
// explicitly by a backend argument (MatmulBackend::CUDA, sdpaBackend::FLASH_CUDA) take host tensors through the device
// and return host tensors, or stay on the device when the operands live there; the named functions and operators go
// to the device exactly when their tensor is device-resident. Nothing here computes on the CPU.
namespace seam {
template <typename T>
inline constexpr bool device_type_v =
    std::is_same_v<T, float> || std::is_same_v<T, yt::bfloat16> || std::is_same_v<T, yt::float16>;

template <typename T, int dim0, int dim1>
auto matmul(const yt::YTensor<T, dim0>& a, const yt::YTensor<T, dim1>& b) {
  constexpr int odim = dim0 > dim1 ? (dim0 > 2 ? dim0 : 2) : (dim1 > 2 ? dim1 : 2);
  if constexpr (device_type_v<T> && dim0 >= 2 && dim1 >= 2 && (dim1 == 2 || dim0 == dim1)) {
    const bool da = on_device(a), db = on_device(b);
    if (da != db) throw std::invalid_argument("matmul: one operand is device-resident and the other is not");
    if (da) return yt::YTensor<T, odim>(dev::matmul(a, b));
    return yt::YTensor<T, odim>(yt::cuda::matmul(a, b));
  } else {
    throw std::invalid_argument("MatmulBackend::CUDA: float / bfloat16 / float16 operands of rank >= 2, the right one "
                                "2-D or of the left one's rank (no CPU fallback)");
    return yt::YTensor<T, odim>();
  }
}

// bool mask (or none) and optional bias; any rank >= 2
template <typename T, int dim>
yt::YTensor<T, dim> sdpa(yt::YTensor<T, dim>& q, yt::YTensor<T, dim>& k, yt::YTensor<T, dim>& v, T scale, int mask_kind,
                         int causal_offset, const yt::YTensor<bool, 2>* mask, const yt::YTensor<T, 2>* bias) {
  if constexpr (!device_type_v<T> || dim < 2) {
    throw std::invalid_argument("sdpaBackend::FLASH_CUDA: float / bfloat16 / float16 tensors of rank >= 2");
    return yt::YTensor<T, dim>();
  } else {
    const int lq = q.shape(-2), lk = k.shape(-2);
    if (mask && (mask->shape(0) != lq || mask->shape(1) != lk))
      throw std::invalid_argument("Mask shape must match the last two dimensions of the score tensor.");
    if (bias && (bias->shape(0) != lq || bias->shape(1) != lk))
      throw std::invalid_argument("Bias shape must match the last two dimensions of the score tensor.");
    const bool dq = on_device(q);
    if (dq != on_device(k) || dq != on_device(v))
      throw std::invalid_argument("scaledDotProductAttention: operands must all be host- or all device-resident");
    // mask and bias are small [lq, lk] host tensors in the reference's API: upload them for the call
    std::vector<uint8_t> m8;
    DeviceBuffer dmask(mask ? static_cast<size_t>(lq) * lk : 16);
    if (mask) {
      m8.resize(static_cast<size_t>(lq) * lk);
      for (int r = 0; r < lq; ++r)
        for (int c = 0; c < lk; ++c) m8[static_cast<size_t>(r) * lk + c] = mask->at(r, c) ? 1 : 0;
      dmask.upload(m8.data());
    }
    std::vector<float> bf;
    DeviceBuffer dbias(bias ? static_cast<size_t>(lq) * lk * sizeof(float) : 16);
    if (bias) {
      bf.resize(static_cast<size_t>(lq) * lk);
      for (int r = 0; r < lq; ++r)
        for (int c = 0; c < lk; ++c) bf[static_cast<size_t>(r) * lk + c] = static_cast<float>(bias->at(r, c));
      dbias.upload(bf.data());
    }
    const uint8_t* mp = mask ? static_cast<const uint8_t*>(dmask.get()) : nullptr;
    const float* bp = bias ? static_cast<const float*>(dbias.get()) : nullptr;
    if (dq) {
      auto out = dev::sdpa(q, k, v, scale, mask_kind, causal_offset, mp, bp);
      check(ytcuda_stream_sync(nullptr));  // dmask / dbias leave scope
      return out;
    }
    // host operands: one upload each (a zero-stride group repeat of K / V is uploaded once, not g times)
    auto qd = to_device(q);
    yt::YTensor<T, dim> kd, vd;
    bool repeated = false;
    if constexpr (dim == 5) repeated = k.stride_(2) == 0 && v.stride_(2) == 0 && k.shape(2) > 1;
    if (repeated) {
      if constexpr (dim == 5) {
        auto k1 = to_device(yt::YTensor<T, 5>(k.slice(2, 0, 1)));
        auto v1 = to_device(yt::YTensor<T, 5>(v.slice(2, 0, 1)));
        kd = k1.repeat(1, 1, k.shape(2), 1, 1);
        vd = v1.repeat(1, 1, v.shape(2), 1, 1);
      }
    } else {
      kd = to_device(k);
      vd = to_device(v);
    }
    return to_host(dev::sdpa(qd, kd, vd, scale, mask_kind, causal_offset, mp, bp));
  }
}

// a predicate mask: Causal is evaluated on the device; any other callable (r, c) -> bool is materialised once on the
// host into a bool tensor (device code cannot call a host lambda)
template <typename T, int dim, typename MaskFunc>
yt::YTensor<T, dim> sdpa_pred(yt::YTensor<T, dim>& q, yt::YTensor<T, dim>& k, yt::YTensor<T, dim>& v, T scale,
                              MaskFunc&& pred, const yt::YTensor<T, 2>* bias) {
  if constexpr (std::is_same_v<std::decay_t<MaskFunc>, Causal>) {
    return sdpa<T, dim>(q, k, v, scale, 1, pred.offset, nullptr, bias);
  } else {
    const int lq = q.shape(-2), lk = k.shape(-2);
    yt::YTensor<bool, 2> m(lq, lk);
    for (int r = 0; r < lq; ++r)
      for (int c = 0; c < lk; ++c) m.at(r, c) = static_cast<bool>(pred(r, c));
    return sdpa<T, dim>(q, k, v, scale, 2, 0, &m, bias);
  }
}

// in-place operator on a device-resident left operand; false = not ours (host tensor or a type the device has not)
template <typename T, int dim, int dim1>
bool inplace_op(const char* op, yt::YTensor<T, dim>& a, const yt::YTensor<T, dim1>& b) {
  if constexpr (device_type_v<T> && dim1 <= dim) {
    if (!on_device(a)) return false;
    const int code = op[0] == '+' ? 0 : op[0] == '-' ? 1 : op[0] == '*' ? 2 : op[0] == '/' ? 3 : -1;
    if (code < 0 || op[1] != 0) throw std::invalid_argument(std::string("operator ") + op + "= has no device kernel");
    if (!on_device(b)) throw std::invalid_argument("in-place operator: the right operand is not device-resident");
    dev::binary_(code, a, b);
    return true;
  } else {
    return false;
  }
}

// YTensor::copy_(src) when either side is device-resident. dst and src on the device: strided copy with dtype
// conversion (float / bfloat16 / float16). One side on the host: a plain upload or download of equal element type and
// shape (a strided side is staged through a contiguous tensor). Both on the host: false, the reference's own copy_ runs.
template <typename T, int dim>
bool copy_any(yt::YTensor<T, dim>& dst, const yt::YTensorBase& src) {
  const bool dd = on_device(dst);
  const bool sd = src.size() > 0 && ytcuda_pointer_is_device(src.template data<char>()) != 0;
  if (!dd && !sd) return false;
  if (src.ndim() != dim || src.shape() != dst.shape()) throw std::invalid_argument("copy_: shapes do not match");
  const std::string st = src.dtype();
  auto as = [&](auto tag) {
    using S = decltype(tag);
    return yt::YTensor<S, dim>(src);
  };
  if (dd && sd) {
    if (st == yt::types::getTypeName<float>()) dev::copy_(dst, as(float{}));
    else if (st == yt::types::getTypeName<yt::bfloat16>()) dev::copy_(dst, as(yt::bfloat16{}));
    else if (st == yt::types::getTypeName<yt::float16>()) dev::copy_(dst, as(yt::float16{}));
    else throw std::invalid_argument("copy_: the device converts between float32, bfloat16 and float16 only");
    return true;
  }
  if (st != yt::types::getTypeName<T>())
    throw std::invalid_argument("copy_: a copy between host and device keeps the element type (convert on the device)");
  yt::YTensor<T, dim> s(src);
  if (dd) {  // host -> device
    auto staged = to_device(s);
    if (dst.isContiguous()) check(ytcuda_memcpy_d2d(dst.data(), staged.data(), staged.size() * sizeof(T), nullptr));
    else dev::copy_(dst, staged);
    check(ytcuda_stream_sync(nullptr));
  } else {   // device -> host
    auto h = to_host(s);
    if (dst.isContiguous()) std::memcpy(dst.data(), h.data(), h.size() * sizeof(T));
    else dst.copy_(h);
  }
  return true;
}
}  // namespace seam

}  // namespace yt::cuda
