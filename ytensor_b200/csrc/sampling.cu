// Top-k sampling over the vocabulary for the YTensor device backend.
//
// Device form of the sample_token step of qwen3::Qwen3ForCausalLM::generate (reference
// example/qwen3/src/qwen3.cpp:465-486): probabilities = softmax(logits), the k most probable tokens are kept in
// descending order, a uniform number drawn in [0, sum of the kept probabilities] picks the first token whose running
// sum reaches it. The random number comes from the caller (the reference draws it from a host std::mt19937), so the
// device part is deterministic: one CTA per row finds maximum and sum, then extracts the k largest probabilities one
// after the other (a block-wide arg-max per extraction, the first index winning ties; the logits of a row stay in L2
// between the passes).
#include <math_constants.h>

#include "ytc_common.cuh"

namespace ytk {

constexpr int TK_THREADS = 1024;
constexpr int TK_MAX_K = 64;

struct TkPair {
  float v;
  int i;
};

__device__ __forceinline__ TkPair tk_better(TkPair a, TkPair b) {
  return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;  // larger value, then smaller index
}

__device__ __forceinline__ TkPair tk_block_argmax(TkPair m, TkPair* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    TkPair other;
    other.v = __shfl_xor_sync(0xffffffffu, m.v, o);
    other.i = __shfl_xor_sync(0xffffffffu, m.i, o);
    m = tk_better(m, other);
  }
  __syncthreads();  // `red` may still be read from the previous round
  if (lane == 0) red[warp] = m;
  __syncthreads();
  TkPair r = red[lane < (TK_THREADS / 32) ? lane : 0];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    TkPair other;
    other.v = __shfl_xor_sync(0xffffffffu, r.v, o);
    other.i = __shfl_xor_sync(0xffffffffu, r.i, o);
    r = tk_better(r, other);
  }
  return r;  // the same in every thread
}

__global__ void __launch_bounds__(TK_THREADS) topk_sample_kernel(const float* logits, int64_t row_stride, int vocab,
                                                                 int k, const float* uniform, float* top_probs,
                                                                 int32_t* top_idx, int32_t* sampled) {
  __shared__ TkPair red[32];
  __shared__ float red_f[32];
  __shared__ int taken[TK_MAX_K];
  const int row = blockIdx.x, t = threadIdx.x;
  const float* x = logits + static_cast<int64_t>(row) * row_stride;
  // maximum and sum of exponentials (softmax denominators, src/function/activation.inl:163-177)
  float m = -CUDART_INF_F;
  for (int i = t; i < vocab; i += TK_THREADS) m = fmaxf(m, x[i]);
  {
    TkPair p{m, 0};
    m = tk_block_argmax(p, red).v;
  }
  float s = 0.f;
  for (int i = t; i < vocab; i += TK_THREADS) s += expf(x[i] - m);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((t & 31) == 0) red_f[t >> 5] = s;
  __syncthreads();
  s = red_f[(t & 31) < (TK_THREADS / 32) ? (t & 31) : 0];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  const float inv = 1.0f / s;
  // k extractions; an index already taken is skipped
  float kept = 0.f;
  for (int j = 0; j < k; ++j) {
    TkPair best{-CUDART_INF_F, 0x7fffffff};
    for (int i = t; i < vocab; i += TK_THREADS) {
      bool skip = false;
      for (int u = 0; u < j; ++u) skip = skip || (taken[u] == i);
      if (!skip) best = tk_better(best, TkPair{x[i], i});
    }
    best = tk_block_argmax(best, red);
    // (a product that cannot be contracted into the sum below: the kept sum must be the sum of the stored values)
    const float pr = __fmul_rn(expf(best.v - m), inv);
    if (t == 0) {
      taken[j] = best.i;
      top_probs[static_cast<int64_t>(row) * k + j] = pr;
      top_idx[static_cast<int64_t>(row) * k + j] = best.i;
    }
    kept += pr;
    __syncthreads();
  }
  if (sampled && t == 0) {
    const float r = (uniform ? uniform[row] : 0.f) * kept;
    float cum = 0.f;
    int pick = taken[0];
    bool found = false;
    for (int j = 0; j < k && !found; ++j) {
      cum += top_probs[static_cast<int64_t>(row) * k + j];
      if (r <= cum) {
        pick = taken[j];
        found = true;
      }
    }
    sampled[row] = pick;
  }
}

}  // namespace ytk

using namespace ytk;

extern "C" {

int ytcuda_topk_sample(const float* logits, int64_t row_stride, int rows, int vocab, int k, const float* uniform,
                       float* top_probs, int32_t* top_idx, int32_t* sampled, void* stream) {
  YTC_REQUIRE(rows >= 0 && vocab >= 0, "ytcuda_topk_sample: negative extent");
  if (rows == 0) return YTC_OK;
  YTC_REQUIRE(logits && top_probs && top_idx, "ytcuda_topk_sample: null tensor");
  YTC_REQUIRE(k >= 1 && k <= TK_MAX_K && k <= vocab, "ytcuda_topk_sample: k = %d outside [1, min(%d, vocab = %d)]", k,
              TK_MAX_K, vocab);
  YTC_REQUIRE(row_stride >= vocab, "ytcuda_topk_sample: row stride shorter than the vocabulary");
  topk_sample_kernel<<<rows, TK_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(logits, row_stride, vocab, k, uniform,
                                                                                 top_probs, top_idx, sampled);
  count_launch();
  YTC_CUDA(cudaGetLastError());
  return YTC_OK;
}

}  // extern "C"
