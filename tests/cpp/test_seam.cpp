// TEST INFRASTRUCTURE. The device backend behind YTensor's OWN entry points. Compiled with -DYT_USE_CUDA=1 against a
// copy of the reference tree that integration/apply_seam.py has added the backend branches to: every case calls the
// reference API exactly as a user would (a.matmul(b, MatmulBackend::CUDA), scaledDotProductAttention(...,
// sdpaBackend::FLASH_CUDA), yt::function::rmsNorm / softmax_, operator+=, copy_) and compares with the reference's CPU
// path on the same data. Built by tests/cpp/Makefile; run on the GPU by tests/test_cpp_backend_gpu.py.
#include "ytensor.hpp"

#include <cmath>
#include <cstdio>
#include <random>

using yt::YTensor;
using yt::function::sdpaBackend;
using yt::infos::MatmulBackend;

static_assert(YT_USE_CUDA == 1, "build with -DYT_USE_CUDA=1");
static_assert(yt::infos::defaultMatmulBackend == MatmulBackend::CUDA, "CUDA comes first in the default's priority");

static std::mt19937 g_rng(321);
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
  std::printf("%-58s err=%.3e tol=%.1e %s\n", name, err, tol, ok ? "PASS" : "FAIL");
  if (!ok) ++g_fail;
}
struct CausalPred {  // the predicate form the reference's flash path prunes tiles with
  int offset;
  bool operator()(int r, int c) const { return c <= r + offset; }
  bool tileAllTrue(int r0, int c0, int, int nr) const { return c0 + nr - 1 <= r0 + offset; }
  bool tileAllFalse(int r0, int c0, int mr, int) const { return c0 > r0 + mr - 1 + offset; }
};

int main() {
  yt::kernel::avx2::set_num_threads(yt::kernel::avx2::default_num_threads());
  {  // YTensor::matmul with the backend argument, and by default
    auto a = randn<3>({3, 70, 96});
    auto b = randn<2>({96, 40});
    auto want = a.matmul(b, MatmulBackend::AVX2);
    const uint64_t n0 = ytcuda_launch_count();
    report("a.matmul(b, MatmulBackend::CUDA)", normwise(a.matmul(b, MatmulBackend::CUDA), want), 1e-5);
    report("  ... launched a device kernel", ytcuda_launch_count() > n0 ? 0.0 : 1.0, 0.5);
    const uint64_t n1 = ytcuda_launch_count();
    report("a.matmul(b) (default backend = CUDA)", normwise(a.matmul(b), want), 1e-5);
    report("  ... launched a device kernel", ytcuda_launch_count() > n1 ? 0.0 : 1.0, 0.5);
    auto b3 = randn<3>({3, 96, 40});
    report("batched right operand", normwise(a.matmul(b3, MatmulBackend::CUDA), a.matmul(b3, MatmulBackend::AVX2)), 1e-5);
    report("yt::function::matmul", normwise(yt::function::matmul(a, b), want), 1e-5);
    bool threw = false;
    try {
      YTensor<double, 2> ad(8, 8), bd(8, 8);
      ad.matmul(bd, MatmulBackend::CUDA);  // an element type the device has no kernel for: refused, not sent to the CPU
    } catch (const std::invalid_argument&) {
      threw = true;
    }
    report("unsupported operand form throws invalid_argument", threw ? 0.0 : 1.0, 0.5);
  }
  {  // bf16 storage through the same switch
    auto af = randn<2>({128, 256});
    auto bf = randn<2>({256, 192}, 0.0625f);
    YTensor<yt::bfloat16, 2> a(128, 256), b(256, 192);
    for (size_t i = 0; i < a.size(); ++i) a.data()[i] = yt::bfloat16(af.data()[i]);
    for (size_t i = 0; i < b.size(); ++i) b.data()[i] = yt::bfloat16(bf.data()[i]);
    YTensor<float, 2> aw(128, 256), bw(256, 192);
    for (size_t i = 0; i < a.size(); ++i) aw.data()[i] = static_cast<float>(a.data()[i]);
    for (size_t i = 0; i < b.size(); ++i) bw.data()[i] = static_cast<float>(b.data()[i]);
    auto want = aw.matmul(bw, MatmulBackend::AVX2);
    auto got = a.matmul(b, MatmulBackend::CUDA);
    YTensor<float, 2> gw(128, 192);
    for (size_t i = 0; i < got.size(); ++i) gw.data()[i] = static_cast<float>(got.data()[i]);
    report("bfloat16 a.matmul(b, MatmulBackend::CUDA)", normwise(gw, want), 2e-2);
  }
  {  // scaledDotProductAttention with the backend argument: the decoder's 5-D form with zero-stride K / V repeats
    const int b = 2, kvh = 2, g = 2, lq = 40, lk = 72, d = 64;
    auto q = randn<5>({b, kvh, g, lq, d});
    auto k4 = randn<4>({b, kvh, lk, d});
    auto v4 = randn<4>({b, kvh, lk, d});
    auto k = YTensor<float, 5>(k4.unsqueeze(2).repeat(1, 1, g, 1, 1));
    auto v = YTensor<float, 5>(v4.unsqueeze(2).repeat(1, 1, g, 1, 1));
    YTensor<bool, 2> mask(lq, lk);
    for (int r = 0; r < lq; ++r)
      for (int c = 0; c < lk; ++c) mask.at(r, c) = r != 3 && ((r * 7 + c * 3) % 4 != 0);
    auto bias = randn<2>({lq, lk}, 0.3f);
    using yt::function::scaledDotProductAttention;
    report("sdpa FLASH_CUDA, no mask",
           normwise(scaledDotProductAttention(q, k, v, 0.f, static_cast<YTensor<bool, 2>*>(nullptr), nullptr, sdpaBackend::FLASH_CUDA),
                    scaledDotProductAttention(q, k, v, 0.f, static_cast<YTensor<bool, 2>*>(nullptr), nullptr, sdpaBackend::FLASH_AVX2)), 1e-5);
    report("sdpa FLASH_CUDA, bool mask (row 3 sees nothing) + bias",
           normwise(scaledDotProductAttention(q, k, v, 0.2f, &mask, &bias, sdpaBackend::FLASH_CUDA),
                    scaledDotProductAttention(q, k, v, 0.2f, &mask, &bias, sdpaBackend::FLASH_AVX2)), 1e-5);
    CausalPred pred{lk - lq};
    report("sdpa FLASH_CUDA, predicate (materialised)",
           normwise(scaledDotProductAttention(q, k, v, 0.f, pred, nullptr, sdpaBackend::FLASH_CUDA),
                    scaledDotProductAttention(q, k, v, 0.f, pred, nullptr, sdpaBackend::FLASH_AVX2)), 1e-5);
    report("sdpa FLASH_CUDA, yt::cuda::Causal (device predicate)",
           normwise(scaledDotProductAttention(q, k, v, 0.f, yt::cuda::Causal{lk - lq}, &bias, sdpaBackend::FLASH_CUDA),
                    scaledDotProductAttention(q, k, v, 0.f, pred, &bias, sdpaBackend::FLASH_AVX2)), 1e-5);
    auto q3 = randn<3>({3, 33, 32});
    auto k3 = randn<3>({3, 50, 32});
    auto v3 = randn<3>({3, 50, 48});
    report("sdpa FLASH_CUDA, 3-D operands, value_dim != head_dim",
           normwise(scaledDotProductAttention(q3, k3, v3, 0.f, static_cast<YTensor<bool, 2>*>(nullptr), nullptr, sdpaBackend::FLASH_CUDA),
                    scaledDotProductAttention(q3, k3, v3, 0.f, static_cast<YTensor<bool, 2>*>(nullptr), nullptr, sdpaBackend::MATH)), 1e-5);
    bool threw = false;
    try {
      YTensor<bool, 2> bad(lq, lk + 1);
      scaledDotProductAttention(q, k, v, 0.f, &bad, nullptr, sdpaBackend::FLASH_CUDA);
    } catch (const std::invalid_argument&) {
      threw = true;
    }
    report("sdpa FLASH_CUDA mask shape mismatch throws", threw ? 0.0 : 1.0, 0.5);
  }
  {  // device-resident tensors: rmsNorm -> += -> softmax_ -> copy_ with one upload per input and one download
    const int B = 3, L = 50, H = 1024;
    auto x = randn<3>({B, L, H});
    YTensor<float, 1> w(H);
    for (int i = 0; i < H; ++i) w.at(i) = 0.9f + 0.2f * static_cast<float>(i % 17) / 17.f;
    auto r = randn<3>({1, L, H});
    // the reference on the host
    auto yh = yt::function::rmsNorm(x, w, -1, 1e-6f);
    yh += r;
    yt::function::softmax_(yh, -1);
    YTensor<yt::bfloat16, 3> outh(B, L, H);
    outh.copy_(yh);
    // the same calls on device-resident tensors
    uint64_t h0, d0, h1, d1;
    ytcuda_copy_counts(&h0, &d0);
    auto xd = yt::cuda::to_device(x);
    auto wd = yt::cuda::to_device(w);
    auto rd = yt::cuda::to_device(r);
    const uint64_t k0 = ytcuda_launch_count();
    auto yd = yt::function::rmsNorm(xd, wd, -1, 1e-6f);
    yd += rd;
    yt::function::softmax_(yd, -1);
    auto outd = yt::cuda::empty_device<yt::bfloat16, 3>({B, L, H});
    outd.copy_(yd);
    const uint64_t k1 = ytcuda_launch_count();
    auto out = yt::cuda::to_host(outd);
    ytcuda_copy_counts(&h1, &d1);
    report("device chain: the tensors are device-resident",
           (yt::cuda::on_device(yd) && yt::cuda::on_device(outd) && !yt::cuda::on_device(out)) ? 0.0 : 1.0, 0.5);
    report("device chain: 3 uploads (x, w, r), 1 download", (h1 - h0 == 3 && d1 - d0 == 1) ? 0.0 : 1.0, 0.5);
    report("device chain: one kernel per operator (4 to 6 launches)", (k1 - k0 >= 4 && k1 - k0 <= 6) ? 0.0 : 1.0, 0.5);
    YTensor<float, 3> gw(B, L, H), ww(B, L, H);
    for (size_t i = 0; i < out.size(); ++i) {
      gw.data()[i] = static_cast<float>(out.data()[i]);
      ww.data()[i] = static_cast<float>(outh.data()[i]);
    }
    report("rmsNorm -> += -> softmax_ -> copy_(bfloat16) on the device", normwise(gw, ww), 1e-2);
    // matmul keeps device operands on the device; a view (transpose) costs nothing
    auto a = randn<2>({64, 96});
    auto bm = randn<2>({80, 96});
    auto ad = yt::cuda::to_device(a), bd = yt::cuda::to_device(bm);
    auto cd = ad.matmul(bd.transpose(), MatmulBackend::CUDA);
    report("device-resident a.matmul(b.transpose())", yt::cuda::on_device(cd) ? normwise(yt::cuda::to_host(cd), a.matmul(bm.transpose(), MatmulBackend::AVX2)) : 1.0, 1e-5);
    // copy_ between host and device
    YTensor<float, 2> back(64, 96);
    back.copy_(ad);
    report("host.copy_(device) downloads", normwise(back, a), 1e-12);
    auto dev2 = yt::cuda::empty_device<float, 2>({64, 96});
    dev2.copy_(a);
    report("device.copy_(host) uploads", normwise(yt::cuda::to_host(dev2), a), 1e-12);
    bool threw = false;
    try {
      yd += r;  // a host operand against a device tensor: refused
    } catch (const std::invalid_argument&) {
      threw = true;
    }
    report("device += host throws invalid_argument", threw ? 0.0 : 1.0, 0.5);
  }
  if (ytcuda_device_status(nullptr) != YTC_OK) {
    std::printf("device status not clean: %s\n", ytcuda_last_error_string());
    ++g_fail;
  }
  std::printf(g_fail ? "%d CASES FAILED\n" : "ALL SEAM CASES PASSED\n", g_fail);
  return g_fail ? 1 : 0;
}
