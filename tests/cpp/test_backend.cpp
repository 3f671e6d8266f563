// TEST INFRASTRUCTURE. Exercises the device backend through the reference's own tensor type: every case builds
// yt::YTensor operands, calls the reference's CPU implementation and yt::cuda::* (ytensor_b200/cpp/ytensor_cuda.hpp)
// on the same data and compares. Built by tests/cpp/Makefile against the reference sources where they lie; the
// binary (tests/cpp/_build/test_backend) travels to the GPU box and is run by tests/test_cpp_backend_gpu.py.
#include "ytensor.hpp"
#include "ytensor_cuda.hpp"

#include <cmath>
#include <cstdio>
#include <random>

using yt::YTensor;

static std::mt19937 g_rng(123);
template <int N>
YTensor<float, N> randn(std::vector<int> shape, float scale = 1.0f) {
  YTensor<float, N> t(shape);
  std::normal_distribution<float> d(0.f, scale);
  float* p = t.data();
  for (size_t i = 0; i < t.size(); ++i) p[i] = d(g_rng);
  return t;
}
template <typename T, int N>
double normwise(const YTensor<T, N>& got, const YTensor<T, N>& want) {
  auto a = got.contiguous();
  auto b = want.contiguous();
  double num = 0, den = 1e-30;
  for (size_t i = 0; i < a.size(); ++i) {
    const double x = static_cast<float>(a.data()[i]), y = static_cast<float>(b.data()[i]);
    num = std::max(num, std::fabs(x - y));
    den = std::max(den, std::fabs(y));
  }
  return num / den;
}
static int g_fail = 0;
static void report(const char* name, double err, double tol) {
  const bool ok = err < tol;
  std::printf("%-44s err=%.3e tol=%.1e %s\n", name, err, tol, ok ? "PASS" : "FAIL");
  if (!ok) ++g_fail;
}

int main() {
  yt::kernel::avx2::set_num_threads(yt::kernel::avx2::default_num_threads());
  {  // matmul: [3, 70, 96] x [96, 40] and a batched right operand
    auto a = randn<3>({3, 70, 96});
    auto b = randn<2>({96, 40});
    report("matmul [3,70,96]x[96,40]", normwise(yt::cuda::matmul(a, b), a.matmul(b)), 1e-5);
    auto b3 = randn<3>({3, 96, 40});
    report("matmul batched right operand", normwise(yt::cuda::matmul(a, b3), a.matmul(b3)), 1e-5);
    auto w = randn<2>({40, 96});
    report("linear (transposed weight view)", normwise(yt::cuda::linear(a, w), yt::function::linear(a, w)), 1e-5);
    bool threw = false;
    try {
      yt::cuda::matmul(a, randn<2>({95, 40}));
    } catch (const std::invalid_argument&) {
      threw = true;
    }
    report("matmul shape mismatch throws invalid_argument", threw ? 0.0 : 1.0, 0.5);
  }
  {  // masked_matmul with a bool mask: products where it holds, the fill value elsewhere
    auto a = randn<3>({2, 37, 45});
    auto b = randn<2>({45, 26});
    YTensor<bool, 2> mask(37, 26);
    for (int i = 0; i < 37; ++i)
      for (int j = 0; j < 26; ++j) mask.at(i, j) = ((i * 31 + j * 17) % 5) != 0 && i != 4;
    report("masked_matmul (bool mask, fill -1.5)", normwise(yt::cuda::masked_matmul(a, b, mask, -1.5f),
                                                              a.masked_matmul(b, mask, -1.5f)), 1e-5);
    bool threw = false;
    try {
      yt::cuda::masked_matmul(a, b, YTensor<bool, 2>(37, 25), 0.f);
    } catch (const std::invalid_argument&) {
      threw = true;
    }
    report("masked_matmul mask shape mismatch throws", threw ? 0.0 : 1.0, 0.5);
  }
  {  // masked_matmul with the causal predicate: evaluated on the device, empty tiles skipped
    auto a = randn<3>({2, 300, 64});
    auto b = randn<2>({64, 280});
    const yt::cuda::Causal causal{-20};
    report("masked_matmul (causal predicate, fill -inf-like)", normwise(yt::cuda::masked_matmul(a, b, causal, -7.0f),
                                                                         a.masked_matmul(b, causal, -7.0f)), 1e-5);
  }
  {  // Lp normalisation and the instance / batch / group norms without affine part
    auto x = randn<4>({3, 8, 5, 7});
    report("normalize p=2 axis -1", normwise(yt::cuda::normalize(x, -1), yt::function::normalize(x, -1)), 1e-5);
    report("normalize p=1 axes {1,3}", normwise(yt::cuda::normalize(x, std::vector<int>{1, 3}, 1.0f),
                                                 yt::function::normalize(x, std::vector<int>{1, 3}, 1.0f)), 1e-5);
    report("instanceNorm", normwise(yt::cuda::instanceNorm(x), yt::function::instanceNorm(x)), 1e-5);
    report("batchNorm channel axis 2", normwise(yt::cuda::batchNorm(x, 2), yt::function::batchNorm(x, 2)), 1e-5);
    report("groupNorm 4 groups", normwise(yt::cuda::groupNorm(x, 4), yt::function::groupNorm(x, 4)), 1e-5);
    report("groupNorm 2 groups, channel axis 3 (-1)", normwise(yt::cuda::groupNorm(x, 7, -1),
                                                                yt::function::groupNorm(x, 7, -1)), 1e-5);
  }
  {  // bf16 storage: device accumulates in fp32; the CPU recipe is widen -> fp32 matmul -> narrow
    auto af = randn<2>({128, 256});
    auto bf = randn<2>({256, 192}, 0.0625f);
    YTensor<yt::bfloat16, 2> a(128, 256), b(256, 192);
    for (size_t i = 0; i < a.size(); ++i) a.data()[i] = yt::bfloat16(af.data()[i]);
    for (size_t i = 0; i < b.size(); ++i) b.data()[i] = yt::bfloat16(bf.data()[i]);
    YTensor<float, 2> aw(128, 256), bw(256, 192);
    for (size_t i = 0; i < a.size(); ++i) aw.data()[i] = static_cast<float>(a.data()[i]);
    for (size_t i = 0; i < b.size(); ++i) bw.data()[i] = static_cast<float>(b.data()[i]);
    auto cw = aw.matmul(bw);
    YTensor<yt::bfloat16, 2> want(128, 192);
    for (size_t i = 0; i < want.size(); ++i) want.data()[i] = yt::bfloat16(cw.data()[i]);
    report("matmul bfloat16 (tcgen05)", normwise(yt::cuda::matmul(a, b), want), 2e-2);
    report("cast float -> bfloat16 bit-exact", normwise(yt::cuda::cast<yt::bfloat16>(af), a), 1e-30);
  }
  {  // attention on the 5-D GQA form with the zero-stride repeat of K / V
    const int b = 1, kvh = 2, g = 2, l = 70, d = 64;
    auto q = randn<5>({b, kvh, g, l, d});
    auto k4 = randn<4>({b, kvh, l, d});
    auto v4 = randn<4>({b, kvh, l, d});
    auto k = YTensor<float, 5>(k4.unsqueeze(2).repeat(1, 1, g, 1, 1));
    auto v = YTensor<float, 5>(v4.unsqueeze(2).repeat(1, 1, g, 1, 1));
    YTensor<bool, 2> mask(l, l);
    for (int r = 0; r < l; ++r)
      for (int c = 0; c < l; ++c) mask.at(r, c) = c <= r;
    auto want = yt::function::scaledDotProductAttention(q, k, v, 0.0f, &mask, nullptr,
                                                        yt::function::sdpaBackend::FLASH_AVX2);
    report("sdpa causal (predicate form)", normwise(yt::cuda::scaledDotProductAttention(q, k, v, 0.0f, yt::cuda::Causal{0}), want), 1e-5);
    report("sdpa bool mask", normwise(yt::cuda::scaledDotProductAttention(q, k, v, 0.0f, &mask), want), 1e-5);
    auto want_full = yt::function::scaledDotProductAttention(q, k, v, 0.0f, static_cast<YTensor<bool, 2>*>(nullptr),
                                                             nullptr, yt::function::sdpaBackend::MATH);
    report("sdpa no mask vs MATH backend", normwise(yt::cuda::scaledDotProductAttention(q, k, v), want_full), 1e-5);
  }
  {  // softmax / norms / reductions / elementwise
    auto x = randn<3>({4, 9, 256});
    auto w = randn<1>({256}, 0.1f);
    for (size_t i = 0; i < w.size(); ++i) w.data()[i] += 1.0f;
    auto bb = randn<1>({256});
    report("softmax last axis", normwise(yt::cuda::softmax(x, -1), yt::function::softmax(x, -1)), 1e-5);
    report("softmax axis 1", normwise(yt::cuda::softmax(x, 1), yt::function::softmax(x, 1)), 1e-5);
    report("rmsNorm", normwise(yt::cuda::rmsNorm(x, w, -1, 1e-6f), yt::function::rmsNorm(x, w, -1, 1e-6f)), 1e-5);
    report("layerNorm", normwise(yt::cuda::layerNorm(x, w, bb, {-1}, 1e-5f), yt::function::layerNorm(x, w, bb, -1, 1e-5f)), 1e-5);
    report("sum axis 1", normwise(yt::cuda::sum(x, {1}), x.sum(1)), 1e-5);
    report("mean axes {0,2}", normwise(yt::cuda::mean(x, {0, 2}), x.mean(std::vector<int>{0, 2})), 1e-4);
    auto mx = yt::cuda::max(x, {2});
    auto mr = x.max(2);
    report("max values", normwise(mx.first, mr.first), 1e-30);
    bool same = true;
    for (size_t i = 0; i < mx.second.size(); ++i) same = same && mx.second.contiguous().data()[i] == mr.second.contiguous().data()[i];
    report("max indices equal", same ? 0.0 : 1.0, 0.5);
    auto r = randn<3>({1, 9, 256});
    report("operator+ with broadcast", normwise(yt::cuda::add(x, r), x + r), 1e-30);
    report("operator* with broadcast", normwise(yt::cuda::mul(x, r), x * r), 1e-30);
    report("swish", normwise(yt::cuda::swish(x), yt::function::swish(x)), 1e-6);
    {  // (the reference's out-of-place relu does not compile for float: its lambda returns two types)
      auto xr = x.clone();
      report("relu", normwise(yt::cuda::relu(x), yt::function::relu_(xr)), 1e-30);
    }
    report("gelu", normwise(yt::cuda::gelu(x), yt::function::gelu(x)), 1e-6);
    report("elu(0.5)", normwise(yt::cuda::elu(x, 0.5f), yt::function::elu(x, 0.5f)), 1e-6);
    report("mish", normwise(yt::cuda::mish(x), yt::function::mish(x)), 1e-6);
    report("hardSwish", normwise(yt::cuda::hardSwish(x), yt::function::hardSwish(x)), 1e-30);
    report("gelu'", normwise(yt::cuda::gelu(x, 1), yt::function::gelu(x, 1)), 1e-6);
    report("mish'", normwise(yt::cuda::mish(x, 1), yt::function::mish(x, 1)), 1e-6);
    report("elu'(0.5)", normwise(yt::cuda::elu(x, 0.5f, 1), yt::function::elu(x, 0.5f, 1)), 1e-6);
  }
  std::printf("%s (%d failures)\n", g_fail ? "SOME CASES FAILED" : "ALL CASES PASSED", g_fail);
  return g_fail ? 1 : 0;
}
