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
};

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

}  // namespace yt::cuda
