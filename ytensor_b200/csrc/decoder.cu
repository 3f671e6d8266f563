// Decoder-only language model forward (Qwen3 block structure) for the YTensor device backend.
//
// The host loop below is the device counterpart of qwen3::Qwen3ForCausalLM::forward (reference
// example/qwen3/src/qwen3.cpp:271-283,365-457): embedding gather, per layer
//   h1 = rmsNorm(x); qkv = linear(h1, Wqkv); per-head rmsNorm(q), rmsNorm(k); rope; KV-cache append;
//   attention over the cache; x2 = linear(attn, Wo) + x; h2 = rmsNorm(x2); x2 += linear(swish(gate)*up, Wdown)
// then the final rmsNorm of the last position and logits = h . W_vocab^T.
// As in the reference, the residual stream, the activations, the KV cache and the logits are fp32; the weights
// are bfloat16 (the reference widens bf16 checkpoints to fp32 at load, qwen3.cpp:16-44 - the products are the same
// numbers). Tensor parallelism splits heads and FFN columns over ranks; the partial sums after the attention
// output projection and after the down projection are reduced by a callback the caller provides (NCCL all-reduce).
//
// Kernels here: embedding gather; weight-streaming linear for few rows (decode); fp32 -> (hi, lo) bf16 split that
// lets the tcgen05 GEMM multiply fp32 activations by bf16 weights (prefill); fused per-head RMSNorm + RoPE + KV
// append; argmax partials for a vocabulary split over ranks.
#include <math_constants.h>

#include <cmath>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "decode_step.cuh"
#include "decode_stream.cuh"
#include "decode_ll.cuh"
#include "ytc_common.cuh"

namespace ytk {

// ------------------------------------------------------------------ embedding gather
// out[t, :] = float(table[ids[t], :])   (reference qwen3.cpp:378-385)
__global__ void __launch_bounds__(256) embedding_kernel(const uint16_t* table, const int* ids, float* out, int64_t n,
                                                        int hidden, int vocab) {
  const int per_row = hidden / 4;
  const int64_t total = n * per_row;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t t = i / per_row;
    const int c = static_cast<int>(i - t * per_row) * 4;
    int id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    const uint2 w = *reinterpret_cast<const uint2*>(table + static_cast<int64_t>(id) * hidden + c);
    float4 o;
    o.x = bf16_bits_to_f32(static_cast<uint16_t>(w.x & 0xFFFF));
    o.y = bf16_bits_to_f32(static_cast<uint16_t>(w.x >> 16));
    o.z = bf16_bits_to_f32(static_cast<uint16_t>(w.y & 0xFFFF));
    o.w = bf16_bits_to_f32(static_cast<uint16_t>(w.y >> 16));
    *reinterpret_cast<float4*>(out + t * hidden + c) = o;
  }
}

// ------------------------------------------------------------------ few-row linear (decode)
// y[m, n] (+)= sum_k x[m, k] * float(W[n, k]),  m < M <= MT. One warp owns ROWS weight rows and streams them once
// with 128-bit loads (32 lanes x 8 bf16 = 256 consecutive k per trip, fully coalesced); x lives in shared memory
// in K-chunks; every lane keeps M partial sums per weight row and the warp reduces them at the end in a fixed
// order (bit-stable from run to run). Memory-bound on W for small M; FFMA-bound as M grows.
constexpr int SK_WARPS = 4;
constexpr int SK_ROWS = 2;
constexpr int SK_KC = 1024;
constexpr int SK_UNROLL = 4;  // 256-column trips fetched together per lane
// Rows up to which the FFMA kernel is used; above, the activations are split into two bf16 planes and the tensor
// cores do the product (the FFMA kernel's time grows with the rows, the tensor-core GEMM's hardly does).
// Sequences from which the step kernel's linear phases run on the tensor cores. Measured per step on the 0.6B shape
// (FFMA form / tensor-core form): 2 sequences 1.30 / 1.71 ms, 4: 1.83 / 2.08, 8: 3.01 / 2.69, 16: 6.6 / 3.5, 32: 13.4 / 6.1.
#ifndef DS_MMA_MIN_B
#define DS_MMA_MIN_B 5
#endif
#ifndef SK_MAX_ROWS
#define SK_MAX_ROWS 4
#endif

template <int MT>
__global__ void __launch_bounds__(SK_WARPS * 32) skinny_linear_kernel(const float* __restrict__ x, int64_t x_rs,
                                                                      const uint16_t* __restrict__ W, int64_t w_rs,
                                                                      float* __restrict__ y, int64_t y_rs, int M, int N,
                                                                      int K, int accumulate) {
  extern __shared__ float xs[];  // [MT][SK_KC]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = (blockIdx.x * SK_WARPS + warp) * SK_ROWS;
  float acc[SK_ROWS][MT];
#pragma unroll
  for (int r = 0; r < SK_ROWS; ++r)
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[r][m] = 0.f;

  for (int k0 = 0; k0 < K; k0 += SK_KC) {
    const int kc = (K - k0 < SK_KC) ? K - k0 : SK_KC;
    __syncthreads();
    for (int i = threadIdx.x; i < MT * (SK_KC / 4); i += SK_WARPS * 32) {
      const int m = i / (SK_KC / 4), c = (i - m * (SK_KC / 4)) * 4;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (m < M && c < kc) v = *reinterpret_cast<const float4*>(x + m * x_rs + k0 + c);
      *reinterpret_cast<float4*>(&xs[m * SK_KC + c]) = v;
    }
    __syncthreads();
    // SK_UNROLL trips of 256 columns are fetched together: several 128-bit loads per lane are in flight at once,
    // which is what hides the HBM latency when a row is only a few KB long
    for (int kk0 = lane * 8; kk0 < kc; kk0 += 256 * SK_UNROLL) {
      uint4 w[SK_UNROLL][SK_ROWS];
#pragma unroll
      for (int u = 0; u < SK_UNROLL; ++u) {
        const int kk = kk0 + u * 256;
#pragma unroll
        for (int r = 0; r < SK_ROWS; ++r) {
          const int n = n0 + r;
          w[u][r] = (n < N && kk < kc) ? *reinterpret_cast<const uint4*>(W + static_cast<int64_t>(n) * w_rs + k0 + kk)
                                       : make_uint4(0u, 0u, 0u, 0u);
        }
      }
#pragma unroll
      for (int u = 0; u < SK_UNROLL; ++u) {
        const int kk = kk0 + u * 256;
        if (kk >= kc) break;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          const float4 xa = *reinterpret_cast<const float4*>(&xs[m * SK_KC + kk]);
          const float4 xb = *reinterpret_cast<const float4*>(&xs[m * SK_KC + kk + 4]);
#pragma unroll
          for (int r = 0; r < SK_ROWS; ++r) {
            float a = acc[r][m];
            a = fmaf(xa.x, __uint_as_float(w[u][r].x << 16), a);
            a = fmaf(xa.y, __uint_as_float(w[u][r].x & 0xFFFF0000u), a);
            a = fmaf(xa.z, __uint_as_float(w[u][r].y << 16), a);
            a = fmaf(xa.w, __uint_as_float(w[u][r].y & 0xFFFF0000u), a);
            a = fmaf(xb.x, __uint_as_float(w[u][r].z << 16), a);
            a = fmaf(xb.y, __uint_as_float(w[u][r].z & 0xFFFF0000u), a);
            a = fmaf(xb.z, __uint_as_float(w[u][r].w << 16), a);
            a = fmaf(xb.w, __uint_as_float(w[u][r].w & 0xFFFF0000u), a);
            acc[r][m] = a;
          }
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < SK_ROWS; ++r)
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      float v = acc[r][m];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      acc[r][m] = v;
    }
  if (lane == 0) {
#pragma unroll
    for (int r = 0; r < SK_ROWS; ++r) {
      const int n = n0 + r;
      if (n >= N) continue;
#pragma unroll
      for (int m = 0; m < MT; ++m)
        if (m < M) {
          float* dst = y + m * y_rs + n;
          *dst = accumulate ? *dst + acc[r][m] : acc[r][m];
        }
    }
  }
}

// y[r][c] (+)= sum over p of (part[p][0][r][c] + part[p][1][r][c]): partials of two stacked [rows][cols] blocks
// (the hi and lo planes of the activations) per k piece, added in index order.
__global__ void __launch_bounds__(256) sum_partials_kernel(const float* part, int n_part, int64_t mn, float* y,
                                                           int64_t y_rs, int cols, int accumulate) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < mn;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float s = 0.f;
#pragma unroll 8
    for (int p = 0; p < n_part; ++p) s += part[2 * p * mn + i] + part[(2 * p + 1) * mn + i];
    const int64_t r = i / cols, c = i - r * cols;
    float* dst = y + r * y_rs + c;
    *dst = accumulate ? *dst + s : s;
  }
}

// x (fp32) = hi + lo with hi = bf16(x) (round to nearest even) and lo = bf16(x - hi): the two 16-bit operands of
// the tensor-core products that together carry 16 mantissa bits of the activation.
__global__ void __launch_bounds__(256) split_hi_lo_kernel(const float* x, int64_t x_rs, uint16_t* hi, uint16_t* lo,
                                                          int64_t rows, int K) {
  dependent_wait();     // (launched as a programmatic dependent of the kernel before it: that one has finished)
  dependent_trigger();  // the kernel queued behind this one may be scheduled and set itself up meanwhile
  const int per_row = K / 4;
  const int64_t total = rows * per_row;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / per_row;
    const int c = static_cast<int>(i - r * per_row) * 4;
    const float4 v = *reinterpret_cast<const float4*>(x + r * x_rs + c);
    const float f[4] = {v.x, v.y, v.z, v.w};
    uint16_t h[4], l[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const __nv_bfloat16 hb = __float2bfloat16_rn(f[k]);
      const float rest = f[k] - __bfloat162float(hb);
      const __nv_bfloat16 lb = __float2bfloat16_rn(rest);
      h[k] = *reinterpret_cast<const uint16_t*>(&hb);
      l[k] = *reinterpret_cast<const uint16_t*>(&lb);
    }
    uint2 ph, pl;
    ph.x = h[0] | (static_cast<uint32_t>(h[1]) << 16);
    ph.y = h[2] | (static_cast<uint32_t>(h[3]) << 16);
    pl.x = l[0] | (static_cast<uint32_t>(l[1]) << 16);
    pl.y = l[2] | (static_cast<uint32_t>(l[3]) << 16);
    *reinterpret_cast<uint2*>(hi + r * K + c) = ph;
    *reinterpret_cast<uint2*>(lo + r * K + c) = pl;
  }
}

__device__ __forceinline__ void split_store4(const float f[4], uint16_t* hi, uint16_t* lo) {
  uint16_t h[4], l[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const __nv_bfloat16 hb = __float2bfloat16_rn(f[k]);
    const __nv_bfloat16 lb = __float2bfloat16_rn(f[k] - __bfloat162float(hb));
    h[k] = *reinterpret_cast<const uint16_t*>(&hb);
    l[k] = *reinterpret_cast<const uint16_t*>(&lb);
  }
  uint2 ph, pl;
  ph.x = h[0] | (static_cast<uint32_t>(h[1]) << 16);
  ph.y = h[2] | (static_cast<uint32_t>(h[3]) << 16);
  pl.x = l[0] | (static_cast<uint32_t>(l[1]) << 16);
  pl.y = l[2] | (static_cast<uint32_t>(l[3]) << 16);
  *reinterpret_cast<uint2*>(hi) = ph;
  *reinterpret_cast<uint2*>(lo) = pl;
}

// sum over the k pieces p of both planes, in index order (the order of sum_partials_kernel), of 4 adjacent elements
__device__ __forceinline__ float4 sum_pieces4(const float* part, int n_part, int64_t mn, int64_t off) {
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
  for (int p = 0; p < n_part; ++p) {
    const float4 a = *reinterpret_cast<const float4*>(part + 2 * p * mn + off);
    const float4 b = *reinterpret_cast<const float4*>(part + (2 * p + 1) * mn + off);
    s.x += a.x + b.x; s.y += a.y + b.y; s.z += a.z + b.z; s.w += a.w + b.w;
  }
  return s;
}

// The glue between two projections of a decode step with 5 .. 128 rows, one CTA per row of the residual stream:
//   x[r] += sum of the k-split partial products of the projection before (when there are any),
//   y = rmsNorm(x[r]) * w   (reference src/function/normalization.inl:234-277),
//   y -> hi + lo bf16 planes, the left operand of the projection that follows.
// Three launches (sum_partials, the row kernel, split_hi_lo) as one.
// Tensor parallelism: the pieces above are this rank's share of the sum over k. RowExchange describes where the ranks
// meet: area[q] is rank q's pair area (its own memory or the peer's), [source rank][2 slots][TP_PUSH_ROWS][hidden]
// {bits, tag} pairs. A thread pushes its four sums as pairs into slot [its rank] of every peer's area (8-byte
// system-scope stores over NVLink), polls its own area for the peers' pairs (bounded), and adds all ranks' shares in
// rank order, so that every rank holds bitwise the same residual stream. world == 1: no exchange.
constexpr int TP_PUSH_ROWS = 128;
struct RowExchange {
  uint2* area[DS_MAX_TP];
  int rank, world, slot;
  unsigned int tag;
  long long wait_cycles;
  int* status;
};
__device__ __forceinline__ float4 exchange_row_sums(const RowExchange& ex, int row, int hidden, int c, float4 mine) {
  const size_t per_src = static_cast<size_t>(2) * TP_PUSH_ROWS * hidden;
  const size_t at = (static_cast<size_t>(ex.slot) * TP_PUSH_ROWS + row) * hidden + c;
  const float mv[4] = {mine.x, mine.y, mine.z, mine.w};
  for (int q = 0; q < ex.world; ++q) {
    if (q == ex.rank) continue;
    uint2* dst = ex.area[q] + ex.rank * per_src + at;
#pragma unroll
    for (int e = 0; e < 4; ++e)
      asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(dst + e), "r"(__float_as_uint(mv[e])), "r"(ex.tag)
                   : "memory");
  }
  // the peers' pairs are requested together (one trip to the L2 for all of them), then taken in rank order
  uint4 pa[DS_MAX_TP], pb[DS_MAX_TP];  // pairs 0, 1 and 2, 3 of every rank
#pragma unroll
  for (int r = 0; r < DS_MAX_TP; ++r) {
    pa[r] = pb[r] = make_uint4(0u, ex.tag, 0u, ex.tag);
    if (r < ex.world && r != ex.rank) {
      const uint2* src = ex.area[ex.rank] + r * per_src + at;
      asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(pa[r].x), "=r"(pa[r].y), "=r"(pa[r].z), "=r"(pa[r].w) : "l"(src) : "memory");
      asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(pb[r].x), "=r"(pb[r].y), "=r"(pb[r].z), "=r"(pb[r].w) : "l"(src + 2) : "memory");
    }
  }
  float tot[4] = {0.f, 0.f, 0.f, 0.f};
  const long long t0 = clock64();
#pragma unroll
  for (int r = 0; r < DS_MAX_TP; ++r) {
    if (r >= ex.world) break;
    if (r == ex.rank) {
#pragma unroll
      for (int e = 0; e < 4; ++e) tot[e] += mv[e];
      continue;
    }
    const uint2* src = ex.area[ex.rank] + r * per_src + at;
    int spins = 0;
    while (!(pa[r].y == ex.tag && pa[r].w == ex.tag && pb[r].y == ex.tag && pb[r].w == ex.tag)) {
      if ((++spins & 63) == 0 && clock64() - t0 > ex.wait_cycles) {  // a peer never arrived: report, carry on
        atomicExch(ex.status, YTC_TIMEOUT);
        break;
      }
      asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(pa[r].x), "=r"(pa[r].y), "=r"(pa[r].z), "=r"(pa[r].w) : "l"(src) : "memory");
      asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(pb[r].x), "=r"(pb[r].y), "=r"(pb[r].z), "=r"(pb[r].w) : "l"(src + 2) : "memory");
    }
    tot[0] += __uint_as_float(pa[r].x);
    tot[1] += __uint_as_float(pa[r].z);
    tot[2] += __uint_as_float(pb[r].x);
    tot[3] += __uint_as_float(pb[r].z);
  }
  return make_float4(tot[0], tot[1], tot[2], tot[3]);
}

// w == nullptr: only the sum (and the exchange) into x, no norm and no planes (after the last layer).
__global__ void __launch_bounds__(1024) sum_norm_split_kernel(const float* part, int n_part, int64_t mn, float* x,
                                                              const float* w, float eps, uint16_t* hi, uint16_t* lo,
                                                              int hidden, const RowExchange ex) {
  dependent_wait();     // (launched as a programmatic dependent of the kernel before it: that one has finished)
  dependent_trigger();  // the kernel queued behind this one may be scheduled and set itself up meanwhile
  extern __shared__ float row_s[];  // [4][hidden]: the sums of the four thread groups, then (in [0]) the row
  __shared__ float red[32];
  const int64_t base = static_cast<int64_t>(blockIdx.x) * hidden;
  if (n_part > 0) {
    // group q of 256 threads adds the pieces q, q + 4, ... (both planes) with all its loads in flight at once
    const int q = threadIdx.x >> 8, t = threadIdx.x & 255;
    for (int c = t * 4; c < hidden; c += 1024) {
      float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 6
      for (int p = q; p < n_part; p += 4) {
        const float4 a = *reinterpret_cast<const float4*>(part + 2 * p * mn + base + c);
        const float4 b = *reinterpret_cast<const float4*>(part + (2 * p + 1) * mn + base + c);
        s.x += a.x + b.x; s.y += a.y + b.y; s.z += a.z + b.z; s.w += a.w + b.w;
      }
      *reinterpret_cast<float4*>(row_s + q * hidden + c) = s;
    }
    __syncthreads();
  }
  float ss = 0.f;
  for (int c = threadIdx.x * 4; c < hidden; c += 4096) {
    float4 v = *reinterpret_cast<const float4*>(x + base + c);
    if (n_part > 0) {
      const float4 s0 = *reinterpret_cast<const float4*>(row_s + c);
      const float4 s1 = *reinterpret_cast<const float4*>(row_s + hidden + c);
      const float4 s2 = *reinterpret_cast<const float4*>(row_s + 2 * hidden + c);
      const float4 s3 = *reinterpret_cast<const float4*>(row_s + 3 * hidden + c);
      float4 y;  // a fixed order: the result does not depend on timing
      y.x = (s0.x + s1.x) + (s2.x + s3.x);
      y.y = (s0.y + s1.y) + (s2.y + s3.y);
      y.z = (s0.z + s1.z) + (s2.z + s3.z);
      y.w = (s0.w + s1.w) + (s2.w + s3.w);
      if (ex.world > 1) y = exchange_row_sums(ex, static_cast<int>(blockIdx.x), hidden, c, y);
      v.x += y.x;
      v.y += y.y;
      v.z += y.z;
      v.w += y.w;
      *reinterpret_cast<float4*>(x + base + c) = v;
    }
    *reinterpret_cast<float4*>(row_s + c) = v;  // (read back by this thread only)
    ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
  }
  if (!w) return;  // (uniform: the sum was all that was asked for)
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) tot += red[i];
  const float inv = 1.0f / sqrtf(tot * (1.0f / hidden) + eps);
  for (int c = threadIdx.x * 4; c < hidden; c += 4096) {
    const float4 v = *reinterpret_cast<const float4*>(row_s + c);
    const float4 g = *reinterpret_cast<const float4*>(w + c);
    const float f[4] = {v.x * inv * g.x, v.y * inv * g.y, v.z * inv * g.z, v.w * inv * g.w};
    split_store4(f, hi + base + c, lo + base + c);
  }
}

// gate_up partial products [pieces][2][rows][2 * inter] -> swish(gate) * up (reference qwen3.cpp:150-162) -> hi + lo
// planes [rows][inter] for the down projection. Three launches (sum_partials, swiglu, split_hi_lo) as one.
__global__ void __launch_bounds__(256) sum_swiglu_split_kernel(const float* part, int n_part, int64_t mn, uint16_t* hi,
                                                               uint16_t* lo, int64_t rows, int inter) {
  dependent_wait();     // (launched as a programmatic dependent of the kernel before it: that one has finished)
  dependent_trigger();  // the kernel queued behind this one may be scheduled and set itself up meanwhile
  const int per_row = inter / 4;
  const int64_t total = rows * per_row;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / per_row;
    const int c = static_cast<int>(i - r * per_row) * 4;
    const float4 g = sum_pieces4(part, n_part, mn, r * 2 * inter + c);
    const float4 u = sum_pieces4(part, n_part, mn, r * 2 * inter + inter + c);
    const float f[4] = {ds_swish(g.x) * u.x, ds_swish(g.y) * u.y, ds_swish(g.z) * u.z, ds_swish(g.w) * u.w};
    split_store4(f, hi + r * inter + c, lo + r * inter + c);
  }
}

// ------------------------------------------------------------------ per-head RMSNorm + RoPE + KV append
// qkv [B, L, (H + 2*KVH) * D] fp32 (the fused projection output). One warp per (b, t, head) vector, D == 128:
//   q heads: rmsNorm over D with q_norm, rotate-half RoPE at position pos0 + t -> q_out [B, H, L, D]
//   k heads: rmsNorm with k_norm, RoPE -> k_cache [B, KVH, max_len, D] at slot (slot0 + t) % max_len (the cache is a
//            ring buffer: KVCache::append, qwen3.cpp:70-88)
//   v heads: copy -> v_cache at the same slot
// (reference qwen3.cpp:237-247: slice/reshape/permute, HeadRMSNorm, ops::rope, KVCache::append; rope math :522-559).
__global__ void __launch_bounds__(128) qkv_post_kernel(const float* qkv, float* q_out, float* k_cache, float* v_cache,
                                                       const float* q_norm, const float* k_norm, const float* cos_t,
                                                       const float* sin_t, int B, int L, int H, int KVH, int max_len,
                                                       int pos0, int slot0, float eps, int n_part, int64_t mn) {
  dependent_wait();
  dependent_trigger();
  constexpr int D = 128;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads_all = H + 2 * KVH;
  const int64_t vecs = static_cast<int64_t>(B) * L * heads_all;
  for (int64_t v = static_cast<int64_t>(blockIdx.x) * 4 + warp; v < vecs; v += static_cast<int64_t>(gridDim.x) * 4) {
    const int hh = static_cast<int>(v % heads_all);
    const int t = static_cast<int>((v / heads_all) % L);
    const int b = static_cast<int>(v / (static_cast<int64_t>(heads_all) * L));
    const float* src = qkv + (static_cast<int64_t>(b) * L + t) * heads_all * D + static_cast<int64_t>(hh) * D;
    float x[4];
    if (n_part > 0) {  // `qkv` holds the k-split partial products [pieces][2][B * L][heads_all * D]: add them here
#pragma unroll
      for (int i = 0; i < 4; ++i) x[i] = 0.f;
#pragma unroll 8
      for (int p = 0; p < n_part; ++p) {
#pragma unroll
        for (int i = 0; i < 4; ++i) x[i] += src[2 * p * mn + lane + 32 * i] + src[(2 * p + 1) * mn + lane + 32 * i];
      }
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) x[i] = src[lane + 32 * i];
    }
    if (hh >= H + KVH) {  // value head
      float* dst = v_cache + ((static_cast<int64_t>(b) * KVH + (hh - H - KVH)) * max_len + (slot0 + t) % max_len) * D;
#pragma unroll
      for (int i = 0; i < 4; ++i) dst[lane + 32 * i] = x[i];
      continue;
    }
    const bool is_q = hh < H;
    float ss = x[0] * x[0];
    ss = fmaf(x[1], x[1], ss);
    ss = fmaf(x[2], x[2], ss);
    ss = fmaf(x[3], x[3], ss);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float denom = sqrtf(ss * (1.0f / D) + eps);
    const float* wn = is_q ? q_norm : k_norm;
#pragma unroll
    for (int i = 0; i < 4; ++i) x[i] = (x[i] / denom) * wn[lane + 32 * i];
    // rotate-half pairs (i, i + 64): elements {lane, lane+64} and {lane+32, lane+96} sit in this lane
    const float* cr = cos_t + static_cast<int64_t>(pos0 + t) * D;
    const float* sr = sin_t + static_cast<int64_t>(pos0 + t) * D;
    float y[4];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float c = cr[lane + 32 * i], s = sr[lane + 32 * i];
      const float re = x[i], im = x[i + 2];
      y[i] = re * c - im * s;
      y[i + 2] = im * c + re * s;
    }
    float* dst = is_q ? q_out + ((static_cast<int64_t>(b) * H + hh) * L + t) * D
                      : k_cache + ((static_cast<int64_t>(b) * KVH + (hh - H)) * max_len + (slot0 + t) % max_len) * D;
#pragma unroll
    for (int i = 0; i < 4; ++i) dst[lane + 32 * i] = y[i];
  }
}

// ------------------------------------------------------------------ model
struct LayerW {
  const uint16_t *qkv = nullptr, *o = nullptr, *gate_up = nullptr, *down = nullptr;  // bf16 [out, in]
  const float *q_norm = nullptr, *k_norm = nullptr, *norm1 = nullptr, *norm2 = nullptr;
};

typedef int (*AllReduceFn)(void* buf, int64_t count, void* user);

struct Qwen3Model {
  // global shape
  int hidden, layers, vocab, inter, heads, kv_heads, head_dim, max_pos;
  float eps, theta;
  // this rank's share (tensor parallel)
  int tp_rank = 0, tp_world = 1;
  int l_heads, l_kv_heads, l_inter, l_vocab;
  int batch = 0;
  std::vector<LayerW> lw;
  const uint16_t* embed = nullptr;    // [vocab, hidden] (full, replicated: the gather needs every row)
  const uint16_t* lm_head = nullptr;  // [l_vocab, hidden] (this rank's rows)
  const float* final_norm = nullptr;
  // device state owned by the model
  float *cos_t = nullptr, *sin_t = nullptr;
  float *k_cache = nullptr, *v_cache = nullptr;  // [layers][batch, l_kv_heads, max_pos, head_dim]
  int cur_len = 0;           // tokens in the cache (at most max_pos)
  int64_t total_written = 0; // tokens ever appended: the ring buffer writes slot total_written % max_pos
  // activations
  float *x = nullptr, *h = nullptr, *qkv = nullptr, *q = nullptr, *attn = nullptr, *gu = nullptr, *act = nullptr,
        *proj = nullptr, *last = nullptr;
  uint16_t* hi = nullptr;  // bf16 planes of the activations: hi [rows][k], then lo [rows][k]
  int64_t act_rows = 0;
  AllReduceFn allreduce = nullptr;
  void* allreduce_user = nullptr;
  // single-kernel decode step (decode_step.cuh)
  int decode_path = 0;              // 0 automatic, 1 one launch per operator, 2 the persistent step kernel or fail
  uint8_t* ring_mask = nullptr;     // [len, max_pos] visibility of a multi-token forward that wraps the ring buffer
  size_t ring_mask_bytes = 0;
  long long* trace = nullptr;       // optional timeline buffer of the step kernel (ytcuda_qwen3_set_trace)
  char* ll_buf = nullptr;           // pair buffers of the barrier-free step kernel (decode_ll.cuh) + unit counters
  size_t ll_bytes = 0;
  unsigned int ll_base = 1;         // tag base of the next launch
  int trace_cap = 0;
  DsLayer* ds_lw = nullptr;         // device copy of the per-layer weight pointers
  bool ds_lw_stale = true;
  float* ds_part = nullptr;         // attention partials
  unsigned int* ds_sync = nullptr;  // barrier counter + per (sequence, kv head) chunk counters
  // exchange buffers of the tensor-parallel step kernel: this rank's (mailbox, flag words, release word) and the
  // peers' buffers opened through CUDA IPC
  char* tp_comm = nullptr;
  char* tp_peer[DS_MAX_TP] = {};
  bool tp_ready = false;
  unsigned int ar_seq = 0;  // exchanges completed so far (the same on every rank)
  unsigned int push_seq = 0;  // exchanges of the operator path's pushed row sums so far (the same on every rank)
  std::vector<void*> owned;
};

// Layout of a rank's exchange buffer: two mailbox slots of [DS_MAX_B][hidden] floats, then (256-byte aligned) the
// DS_MAX_TP flag words the peers write and, 64 bytes further, the release word of this rank's own CTAs.
static size_t tp_flags_offset(int hidden) {
  return (static_cast<size_t>(2) * DS_MAX_B * hidden * sizeof(float) + 255) / 256 * 256;
}
// Behind the flag words: the pair area of the barrier-free step kernel, [source rank][2][4][hidden] {bits, tag} pairs.
static size_t tp_pairs_offset(int hidden) { return tp_flags_offset(hidden) + 256; }
// ... and behind that the pair area of the operator path (5 .. TP_PUSH_ROWS rows): [source rank][2][TP_PUSH_ROWS][hidden].
static size_t tp_rows_offset(int hidden) {
  return tp_pairs_offset(hidden) + static_cast<size_t>(DS_MAX_TP) * 2 * 4 * hidden * sizeof(uint2);
}
static size_t tp_comm_bytes(int hidden) {
  return tp_rows_offset(hidden) + static_cast<size_t>(DS_MAX_TP) * 2 * TP_PUSH_ROWS * hidden * sizeof(uint2);
}

static int dev_alloc(Qwen3Model* m, void** p, size_t bytes) {
  YTC_CUDA(cudaMalloc(p, bytes));
  m->owned.push_back(*p);
  return YTC_OK;
}

// y[M, N] (+)= x[M, K] . W[N, K]^T with fp32 x / y and bf16 W.
// ---- the projections of a step with 5 .. 128 rows, taken apart so that the glue between them can be fused ----
static bool split_k_ok(int64_t M, int K) { return M <= 128 && K % 128 == 0 && K >= 256; }

static int split_planes(Qwen3Model* m, const float* x, int64_t x_rs, int64_t M, int K, cudaStream_t st) {
  const int64_t blocks = (M * (K / 4) + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  YTC_CUDA(launch_overlapped(split_hi_lo_kernel, dim3(static_cast<unsigned>(blocks < cap ? blocks : cap)), dim3(256), 0, st,
                             x, x_rs, m->hi, m->hi + M * K, M, K));
  count_launch();
  YTC_CUDA(cudaGetLastError());
  return YTC_OK;
}

struct Pieces {  // k-split partial products [n][2][M][N] of one projection
  const float* part = nullptr;
  int n = 0;
  int64_t mn = 0;
};

// planes [2 M][K] at m->hi times W^T as one GEMM launch with the k pieces as batch items (see linear_w16)
static int gemm_pieces(Qwen3Model* m, const uint16_t* W, int64_t M, int N, int K, Pieces* out, cudaStream_t st) {
  // As many k pieces as keep the work items (128 x 128 output tiles x pieces) within one wave of the SMs: more
  // pieces than that only add partial sums to write and read back (measured at 32 rows: 4 pieces for the qkv
  // projection of the 0.6B shape, 2 for gate / up, 16 or 12 for the o and down projections).
  const int blocks = K / 128;
  const int tiles = ((N + 127) / 128) * static_cast<int>((2 * M + 127) / 128);
  int splits = 1;
  for (int d = 1; d <= blocks; ++d)
    if (blocks % d == 0 && tiles * d <= sm_count()) splits = d;
  const int kc = K / splits;
  const size_t part_elems = static_cast<size_t>(2) * splits * M * N;
  float* part = static_cast<float*>(device_workspace(part_elems * sizeof(float), st));
  if (!part) {
    set_last_error("linear: cannot allocate %zu bytes for split-k partial sums", part_elems * sizeof(float));
    return YTC_CUDA_ERROR;
  }
  out->part = part;
  out->n = splits;
  out->mn = M * N;
  return ytcuda_gemm(YTC_BF16, YTC_F32, m->hi, W, part, static_cast<int>(2 * M), N, kc, 1.f, 0.f, K, 1, 1, K, N, 1, splits,
                     kc, kc, 2 * out->mn, st);
}

// exchange: the pieces are this rank's share of a sum over k that is split over the tensor-parallel ranks (the o and
// down projections): the ranks' shares are exchanged inside the kernel.
static int sum_norm_split(Qwen3Model* m, const Pieces& pc, float* x, const float* w, int64_t rows, int hidden,
                          cudaStream_t st, bool exchange = false) {
  RowExchange ex{};
  ex.world = 1;
  if (exchange && m->tp_world > 1 && pc.n > 0) {
    for (int r = 0; r < m->tp_world; ++r)
      ex.area[r] = reinterpret_cast<uint2*>((r == m->tp_rank ? m->tp_comm : m->tp_peer[r]) + tp_rows_offset(m->hidden));
    ex.rank = m->tp_rank;
    ex.world = m->tp_world;
    ex.slot = static_cast<int>(m->push_seq & 1u);
    ex.tag = ++m->push_seq;  // (never 0: the areas start zeroed)
    ex.wait_cycles = wait_cycle_limit();
    ex.status = device_status_word();
  }
  YTC_CUDA(launch_overlapped(sum_norm_split_kernel, dim3(static_cast<unsigned>(rows)), dim3(1024),
                             4 * hidden * sizeof(float), st, pc.part, pc.n, pc.mn, x, w, m->eps, m->hi,
                             m->hi + rows * hidden, hidden, ex));
  count_launch();
  YTC_CUDA(cudaGetLastError());
  return YTC_OK;
}

static int linear_w16(Qwen3Model* m, const float* x, int64_t x_rs, const uint16_t* W, float* y, int64_t y_rs, int64_t M,
                      int N, int K, bool accumulate, cudaStream_t st) {
  if (M <= 0 || N <= 0) return YTC_OK;
  if (M <= SK_MAX_ROWS) {
    const int blocks = (N + SK_WARPS * SK_ROWS - 1) / (SK_WARPS * SK_ROWS);
    const int Mi = static_cast<int>(M);
#define SK_LAUNCH(MT)                                                                                          \
  skinny_linear_kernel<MT><<<blocks, SK_WARPS * 32, MT * SK_KC * sizeof(float), st>>>(x, x_rs, W, K, y, y_rs, Mi, N, K, \
                                                                                      accumulate ? 1 : 0)
    if (Mi == 1) SK_LAUNCH(1);
    else if (Mi <= 2) SK_LAUNCH(2);
    else if (Mi <= 4) SK_LAUNCH(4);
    else if (Mi <= 8) SK_LAUNCH(8);
    else if (Mi <= 16) {
      const int sa = ensure_dynamic_smem(reinterpret_cast<const void*>(skinny_linear_kernel<16>), 16 * SK_KC * 4);
      if (sa != YTC_OK) return sa;
      SK_LAUNCH(16);
    } else {
      const int sa = ensure_dynamic_smem(reinterpret_cast<const void*>(skinny_linear_kernel<32>), 32 * SK_KC * 4);
      if (sa != YTC_OK) return sa;
      SK_LAUNCH(32);
    }
#undef SK_LAUNCH
    count_launch();
    YTC_CUDA(cudaGetLastError());
    return YTC_OK;
  }
  // many rows: split the activation into two bf16 planes and run the tensor-core GEMM on each. The lo plane follows
  // the hi plane: [2 M][K] is then one left operand whose rows M .. 2 M - 1 are the lo plane.
  int s = split_planes(m, x, x_rs, M, K, st);
  if (s != YTC_OK) return s;
  uint16_t* hi = m->hi;
  uint16_t* lo = m->hi + M * K;
  // Few rows (decode with a larger batch): there are only N / 128 output tiles, too few to keep the SMs busy and the
  // weight stream at bandwidth. The k range is cut into pieces that run as "batch" items of one GEMM launch (a k
  // offset is a plain pointer offset for both K-major operands), each writing its own partial result, and a small
  // kernel adds the partials of both planes in a fixed order.
  if (split_k_ok(M, K)) {
    Pieces pc;
    if ((s = gemm_pieces(m, W, M, N, K, &pc, st)) != YTC_OK) return s;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
    const int64_t blocks = (pc.mn + 255) / 256;
    sum_partials_kernel<<<static_cast<unsigned>(blocks < cap ? blocks : cap), 256, 0, st>>>(pc.part, pc.n, pc.mn, y, y_rs,
                                                                                             N, accumulate ? 1 : 0);
    count_launch();
    YTC_CUDA(cudaGetLastError());
    return YTC_OK;
  }
  s = ytcuda_gemm(YTC_BF16, YTC_F32, hi, W, y, static_cast<int>(M), N, K, 1.f, accumulate ? 1.f : 0.f, K, 1, 1,
                      K, y_rs, 1, 1, 0, 0, 0, st);
  if (s != YTC_OK) return s;
  return ytcuda_gemm(YTC_BF16, YTC_F32, lo, W, y, static_cast<int>(M), N, K, 1.f, 1.f, K, 1, 1, K, y_rs, 1, 1, 0, 0,
                     0, st);
}

static int rmsnorm_rows(const float* x, const float* w, float* y, int64_t rows, int hidden, float eps, cudaStream_t st) {
  const int64_t shape[2] = {rows, hidden}, strides[2] = {hidden, 1};
  const int axes[1] = {-1};
  return ytcuda_rmsnorm(YTC_F32, YTC_F32, YTC_F32, x, w, y, shape, strides, strides, 2, axes, 1, eps, st);
}
static int add_inplace(float* a, const float* b, int64_t n, cudaStream_t st) {
  const int64_t shape[1] = {n}, strides[1] = {1};
  return ytcuda_binary(0, YTC_F32, YTC_F32, YTC_F32, a, b, a, 1, shape, strides, strides, strides, st);
}

}  // namespace ytk

using namespace ytk;

extern "C" {

// cos / sin tables as the reference precomputes them on the host (example/qwen3/src/qwen3.cpp:161-175):
// freq = 1 / pow(theta, 2 i / dim), angle = t * freq, both halves of a row hold the same values.
int ytcuda_rope_tables(int dim, int max_len, float theta, float* cos_host, float* sin_host) {
  YTC_REQUIRE(dim > 0 && dim % 2 == 0 && max_len >= 0 && cos_host && sin_host, "ytcuda_rope_tables: bad arguments");
  const int half = dim / 2;
  for (int t = 0; t < max_len; ++t)
    for (int i = 0; i < half; ++i) {
      const float freq = 1.0f / std::pow(theta, 2.0f * i / dim);
      const float angle = t * freq;
      cos_host[static_cast<int64_t>(t) * dim + i] = cos_host[static_cast<int64_t>(t) * dim + i + half] = std::cos(angle);
      sin_host[static_cast<int64_t>(t) * dim + i] = sin_host[static_cast<int64_t>(t) * dim + i + half] = std::sin(angle);
    }
  return YTC_OK;
}

int ytcuda_embedding(const void* table_bf16, const int32_t* ids, float* out, int64_t n, int hidden, int vocab,
                     void* stream) {
  YTC_REQUIRE(n >= 0 && hidden >= 0 && vocab > 0, "ytcuda_embedding: bad extent");
  if (n == 0 || hidden == 0) return YTC_OK;
  YTC_REQUIRE(table_bf16 && ids && out, "ytcuda_embedding: null tensor");
  YTC_REQUIRE(hidden % 4 == 0, "ytcuda_embedding: hidden must be a multiple of 4");
  const int64_t blocks = (n * (hidden / 4) + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  embedding_kernel<<<static_cast<unsigned>(blocks < cap ? blocks : cap), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint16_t*>(table_bf16), ids, out, n, hidden, vocab);
  count_launch();
  YTC_CUDA(cudaGetLastError());
  return YTC_OK;
}

// y[M, N] (+)= x[M, K] . W[N, K]^T, x / y fp32 (row strides in elements), W bf16 row-major [N, K].
// The device form of yt::function::linear on fp32 activations with weights kept in their bf16 storage
// (reference src/function/ops.inl:84-91; weights widened at load in example/qwen3/src/qwen3.cpp:16-44).
int ytcuda_linear_w16(const float* x, int64_t x_row_stride, const void* w_bf16, float* y, int64_t y_row_stride,
                      int64_t m, int n, int k, int accumulate, void* hi_lo_scratch, void* stream) {
  YTC_REQUIRE(m >= 0 && n >= 0 && k >= 0, "ytcuda_linear_w16: negative extent");
  if (m == 0 || n == 0) return YTC_OK;
  YTC_REQUIRE(x && w_bf16 && y, "ytcuda_linear_w16: null tensor");
  YTC_REQUIRE(k % 8 == 0 && x_row_stride % 4 == 0 && (reinterpret_cast<uint64_t>(x) & 15) == 0 &&
                  (reinterpret_cast<uint64_t>(w_bf16) & 15) == 0,
              "ytcuda_linear_w16: k must be a multiple of 8 and x / W 16-byte aligned");
  Qwen3Model tmp{};
  if (m > SK_MAX_ROWS) {
    YTC_REQUIRE(hi_lo_scratch != nullptr, "ytcuda_linear_w16: more than %d rows need a scratch of 4*m*k bytes", SK_MAX_ROWS);
    tmp.hi = static_cast<uint16_t*>(hi_lo_scratch);
  }
  return linear_w16(&tmp, x, x_row_stride, static_cast<const uint16_t*>(w_bf16), y, y_row_stride, m, n, k,
                    accumulate != 0, static_cast<cudaStream_t>(stream));
}

static int qkv_post_launch(const float* qkv, int n_part, int64_t mn, float* q_out, float* k_cache, float* v_cache,
                           const float* q_norm, const float* k_norm, const float* cos_table, const float* sin_table,
                           int batch, int len, int heads, int kv_heads, int head_dim, int max_len, int pos0, int slot0,
                           float eps, void* stream) {
  YTC_REQUIRE(batch >= 0 && len >= 0 && heads >= 0 && kv_heads >= 0, "ytcuda_qwen3_qkv_post: negative extent");
  if (batch == 0 || len == 0) return YTC_OK;
  if (head_dim != 128) {
    set_last_error("ytcuda_qwen3_qkv_post: head_dim %d is not supported (128 only)", head_dim);
    return YTC_UNSUPPORTED;
  }
  YTC_REQUIRE(qkv && q_out && k_cache && v_cache && q_norm && k_norm && cos_table && sin_table,
              "ytcuda_qwen3_qkv_post: null tensor");
  YTC_REQUIRE(slot0 >= 0 && slot0 < max_len && len <= max_len,
              "ytcuda_qwen3_qkv_post: %d new tokens at slot %d do not fit a ring of %d slots", len, slot0, max_len);
  YTC_REQUIRE(pos0 >= 0 && pos0 + len <= max_len, "ytcuda_qwen3_qkv_post: rotary positions %d .. %d outside the table of %d",
              pos0, pos0 + len - 1, max_len);
  const int64_t vecs = static_cast<int64_t>(batch) * len * (heads + 2 * kv_heads);
  const int64_t blocks = (vecs + 3) / 4;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  YTC_CUDA(launch_overlapped(qkv_post_kernel, dim3(static_cast<unsigned>(blocks < cap ? blocks : cap)), dim3(128), 0,
                             static_cast<cudaStream_t>(stream), qkv, q_out, k_cache, v_cache, q_norm, k_norm, cos_table,
                             sin_table, batch, len, heads, kv_heads, max_len, pos0, slot0, eps, n_part, mn));
  count_launch();
  YTC_CUDA(cudaGetLastError());
  return YTC_OK;
}

int ytcuda_qwen3_qkv_post(const float* qkv, float* q_out, float* k_cache, float* v_cache, const float* q_norm,
                          const float* k_norm, const float* cos_table, const float* sin_table, int batch, int len,
                          int heads, int kv_heads, int head_dim, int max_len, int pos0, int slot0, float eps,
                          void* stream) {
  return qkv_post_launch(qkv, 0, 0, q_out, k_cache, v_cache, q_norm, k_norm, cos_table, sin_table, batch, len, heads,
                         kv_heads, head_dim, max_len, pos0, slot0, eps, stream);
}

// mask[qi][ki] of KVCache::get_mask for a full ring (reference qwen3.cpp:100-126): slot ki holds the token of logical
// age (ki - write_pos + max_len) % max_len (0 = oldest), query qi of the len new tokens has logical position
// max_len - len + qi, and sees the slots that are not younger than itself.
__global__ void ring_mask_kernel(uint8_t* mask, int len, int max_len, int write_pos) {
  const int64_t total = static_cast<int64_t>(len) * max_len;
  for (int64_t e = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; e < total;
       e += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int qi = static_cast<int>(e / max_len), ki = static_cast<int>(e - static_cast<int64_t>(qi) * max_len);
    const int k_logical = (ki - write_pos + max_len) % max_len;
    mask[e] = k_logical <= max_len - len + qi ? 1 : 0;
  }
}

// ---------------------------------------------------------------- model handle
void* ytcuda_qwen3_create(int hidden, int layers, int vocab, int inter, int heads, int kv_heads, int head_dim, float eps,
                          float theta, int max_pos, int batch, int tp_rank, int tp_world) {
  if (hidden <= 0 || layers <= 0 || vocab <= 0 || inter <= 0 || heads <= 0 || kv_heads <= 0 || head_dim != 128 ||
      max_pos <= 0 || batch <= 0 || tp_world <= 0 || tp_rank < 0 || tp_rank >= tp_world || heads % kv_heads ||
      kv_heads % tp_world || inter % tp_world || hidden % 8 || inter % 8) {
    set_last_error("ytcuda_qwen3_create: unsupported configuration (head_dim must be 128; kv_heads and the FFN width "
                   "must divide by the tensor-parallel size)");
    return nullptr;
  }
  auto* m = new Qwen3Model();
  m->hidden = hidden; m->layers = layers; m->vocab = vocab; m->inter = inter; m->heads = heads;
  m->kv_heads = kv_heads; m->head_dim = head_dim; m->max_pos = max_pos; m->eps = eps; m->theta = theta;
  m->tp_rank = tp_rank; m->tp_world = tp_world; m->batch = batch;
  m->l_heads = heads / tp_world; m->l_kv_heads = kv_heads / tp_world; m->l_inter = inter / tp_world;
  m->l_vocab = (vocab + tp_world - 1) / tp_world;
  if (tp_rank == tp_world - 1) m->l_vocab = vocab - m->l_vocab * (tp_world - 1);
  m->lw.resize(layers);
  std::vector<float> ch(static_cast<size_t>(max_pos) * head_dim), sh(ch.size());
  ytcuda_rope_tables(head_dim, max_pos, theta, ch.data(), sh.data());
  const size_t cache = static_cast<size_t>(layers) * batch * m->l_kv_heads * max_pos * head_dim * sizeof(float);
  bool ok = dev_alloc(m, reinterpret_cast<void**>(&m->cos_t), ch.size() * 4) == YTC_OK &&
            dev_alloc(m, reinterpret_cast<void**>(&m->sin_t), sh.size() * 4) == YTC_OK &&
            dev_alloc(m, reinterpret_cast<void**>(&m->k_cache), cache) == YTC_OK &&
            dev_alloc(m, reinterpret_cast<void**>(&m->v_cache), cache) == YTC_OK;
  if (ok) {
    ok = cudaMemcpy(m->cos_t, ch.data(), ch.size() * 4, cudaMemcpyHostToDevice) == cudaSuccess &&
         cudaMemcpy(m->sin_t, sh.data(), sh.size() * 4, cudaMemcpyHostToDevice) == cudaSuccess &&
         cudaMemset(m->k_cache, 0, cache) == cudaSuccess && cudaMemset(m->v_cache, 0, cache) == cudaSuccess;
  }
  if (!ok) {
    set_last_error("ytcuda_qwen3_create: device allocation failed (KV cache needs %zu bytes twice)", cache);
    for (void* p : m->owned) cudaFree(p);
    delete m;
    return nullptr;
  }
  return m;
}

// Tear-down of a tensor-parallel model is three steps: (1) every rank waits for its own kernels and closes the
// peers' exchange buffers (ytcuda_qwen3_tp_disconnect), (2) the caller runs a barrier over the group, (3) every rank
// destroys its model, which frees the buffer it exported. Freeing an exported buffer while a peer still has it open,
// or while a slower peer's last step kernel may still read its mailbox, is undefined behaviour.
int ytcuda_qwen3_tp_disconnect(void* handle) {
  auto* m = static_cast<Qwen3Model*>(handle);
  YTC_REQUIRE(m, "ytcuda_qwen3_tp_disconnect: null handle");
  YTC_CUDA(cudaDeviceSynchronize());
  for (char*& peer : m->tp_peer)
    if (peer) {
      cudaIpcCloseMemHandle(peer);
      peer = nullptr;
    }
  m->tp_ready = false;
  return YTC_OK;
}

// After a step kernel gave up on a peer (YTC_TIMEOUT) the ranks' exchange counters disagree. Recovery: every rank
// waits for its own kernels, the caller runs a barrier over the group (no kernel anywhere can write a flag any
// more), every rank calls this, and a second barrier follows before the next forward. The arrival words and the
// exchange counter start again from zero; the KV caches are reset as by ytcuda_qwen3_reset.
int ytcuda_qwen3_tp_resync(void* handle) {
  auto* m = static_cast<Qwen3Model*>(handle);
  YTC_REQUIRE(m, "ytcuda_qwen3_tp_resync: null handle");
  YTC_CUDA(cudaDeviceSynchronize());
  if (m->tp_comm) YTC_CUDA(cudaMemset(m->tp_comm, 0, tp_comm_bytes(m->hidden)));  // flags, mailboxes and pairs
  m->ar_seq = 0;
  m->push_seq = 0;
  m->ll_base = 0xFFFFFFFFu;  // the barrier-free kernel starts again from clean pair buffers and tag 1
  m->cur_len = 0;
  m->total_written = 0;
  return YTC_OK;
}

void ytcuda_qwen3_destroy(void* handle) {
  auto* m = static_cast<Qwen3Model*>(handle);
  if (!m) return;
  cudaDeviceSynchronize();
  for (char* peer : m->tp_peer)
    if (peer) cudaIpcCloseMemHandle(peer);
  for (void* p : m->owned) cudaFree(p);
  delete m;
}

// Registers a device weight (not copied; the caller keeps it alive). Names: "embed" [vocab, hidden] bf16,
// "lm_head" [this rank's vocab rows, hidden] bf16, "norm" [hidden] f32; per layer "qkv" [(l_heads + 2 l_kv_heads)
// * head_dim, hidden], "o" [hidden, l_heads * head_dim], "gate_up" [2 * l_inter, hidden], "down" [hidden, l_inter]
// (bf16, already sliced for this rank) and "q_norm", "k_norm" [head_dim], "norm1", "norm2" [hidden] (f32).
int ytcuda_qwen3_set_weight(void* handle, const char* name, int layer, const void* dptr) {
  auto* m = static_cast<Qwen3Model*>(handle);
  YTC_REQUIRE(m && name && dptr, "ytcuda_qwen3_set_weight: null argument");
  YTC_REQUIRE((reinterpret_cast<uint64_t>(dptr) & 15) == 0, "ytcuda_qwen3_set_weight: weights must be 16-byte aligned");
  const std::string n(name);
  m->ds_lw_stale = true;
  if (n == "embed") { m->embed = static_cast<const uint16_t*>(dptr); return YTC_OK; }
  if (n == "lm_head") { m->lm_head = static_cast<const uint16_t*>(dptr); return YTC_OK; }
  if (n == "norm") { m->final_norm = static_cast<const float*>(dptr); return YTC_OK; }
  YTC_REQUIRE(layer >= 0 && layer < m->layers, "ytcuda_qwen3_set_weight: layer %d out of range", layer);
  LayerW& L = m->lw[layer];
  if (n == "qkv") L.qkv = static_cast<const uint16_t*>(dptr);
  else if (n == "o") L.o = static_cast<const uint16_t*>(dptr);
  else if (n == "gate_up") L.gate_up = static_cast<const uint16_t*>(dptr);
  else if (n == "down") L.down = static_cast<const uint16_t*>(dptr);
  else if (n == "q_norm") L.q_norm = static_cast<const float*>(dptr);
  else if (n == "k_norm") L.k_norm = static_cast<const float*>(dptr);
  else if (n == "norm1") L.norm1 = static_cast<const float*>(dptr);
  else if (n == "norm2") L.norm2 = static_cast<const float*>(dptr);
  else {
    set_last_error("ytcuda_qwen3_set_weight: unknown weight name '%s'", name);
    return YTC_INVALID_ARG;
  }
  return YTC_OK;
}

// Sum-reduction over the tensor-parallel group of `count` floats in place, called on the forward's stream between
// kernels (after the attention output projection and after the down projection). NULL when tp_world == 1.
int ytcuda_qwen3_set_allreduce(void* handle, int (*fn)(void*, int64_t, void*), void* user) {
  auto* m = static_cast<Qwen3Model*>(handle);
  YTC_REQUIRE(m, "ytcuda_qwen3_set_allreduce: null handle");
  m->allreduce = fn;
  m->allreduce_user = user;
  return YTC_OK;
}

int ytcuda_qwen3_reset(void* handle) {
  auto* m = static_cast<Qwen3Model*>(handle);
  YTC_REQUIRE(m, "ytcuda_qwen3_reset: null handle");
  m->cur_len = 0;
  m->total_written = 0;
  return YTC_OK;
}
// Allocates this rank's exchange buffer for the tensor-parallel step kernel and returns its CUDA IPC handle
// (64 bytes) for the other ranks to open.
int ytcuda_qwen3_tp_export(void* handle, void* ipc_handle_64) {
  auto* m = static_cast<Qwen3Model*>(handle);
  YTC_REQUIRE(m && ipc_handle_64, "ytcuda_qwen3_tp_export: null argument");
  YTC_REQUIRE(m->tp_world > 1 && m->tp_world <= DS_MAX_TP, "ytcuda_qwen3_tp_export: needs 2..%d ranks", DS_MAX_TP);
  if (!m->tp_comm) {
    const size_t bytes = tp_comm_bytes(m->hidden);
    int s = dev_alloc(m, reinterpret_cast<void**>(&m->tp_comm), bytes);
    if (s != YTC_OK) return s;
    YTC_CUDA(cudaMemset(m->tp_comm, 0, bytes));
  }
  cudaIpcMemHandle_t h;
  YTC_CUDA(cudaIpcGetMemHandle(&h, m->tp_comm));
  static_assert(sizeof(h) == 64, "CUDA IPC handles are 64 bytes");
  std::memcpy(ipc_handle_64, &h, sizeof(h));
  return YTC_OK;
}

// Opens rank `rank`'s exchange buffer (its own rank is accepted and ignored). Once every peer is open, decode
// steps of batch <= 8 run as the single persistent kernel with the all-reduces inside it.
int ytcuda_qwen3_tp_import(void* handle, int rank, const void* ipc_handle_64) {
  auto* m = static_cast<Qwen3Model*>(handle);
  YTC_REQUIRE(m && ipc_handle_64, "ytcuda_qwen3_tp_import: null argument");
  YTC_REQUIRE(m->tp_comm, "ytcuda_qwen3_tp_import: call ytcuda_qwen3_tp_export first");
  YTC_REQUIRE(rank >= 0 && rank < m->tp_world, "ytcuda_qwen3_tp_import: rank %d out of range", rank);
  if (rank != m->tp_rank && !m->tp_peer[rank]) {
    cudaIpcMemHandle_t h;
    std::memcpy(&h, ipc_handle_64, sizeof(h));
    void* ptr = nullptr;
    YTC_CUDA(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
    m->tp_peer[rank] = static_cast<char*>(ptr);
  }
  bool all = true;
  for (int r = 0; r < m->tp_world; ++r) all = all && (r == m->tp_rank || m->tp_peer[r]);
  m->tp_ready = all;
  return YTC_OK;
}

// 0: automatic (the persistent step kernel where it applies), 1: always one launch per operator, 2: the persistent
// step kernel or YTC_UNSUPPORTED, 3: as 2 with the FFMA form of its linear phases at every batch size.
int ytcuda_qwen3_set_decode_path(void* handle, int path) {
  auto* m = static_cast<Qwen3Model*>(handle);
  YTC_REQUIRE(m, "ytcuda_qwen3_set_decode_path: null handle");
  YTC_REQUIRE(path >= 0 && path <= 6, "ytcuda_qwen3_set_decode_path: path must be 0 .. 6");
  m->decode_path = path;
  return YTC_OK;
}
int ytcuda_qwen3_set_trace(void* handle, int64_t* dev_buf, int slots_per_cta) {
  auto* m = static_cast<Qwen3Model*>(handle);
  YTC_REQUIRE(m, "ytcuda_qwen3_set_trace: null handle");
  YTC_REQUIRE(slots_per_cta >= 0 && (dev_buf || slots_per_cta == 0), "ytcuda_qwen3_set_trace: bad buffer");
  m->trace = slots_per_cta > 0 ? reinterpret_cast<long long*>(dev_buf) : nullptr;
  m->trace_cap = slots_per_cta;
  return YTC_OK;
}
int ytcuda_qwen3_cache_len(void* handle) {
  auto* m = static_cast<Qwen3Model*>(handle);
  return m ? m->cur_len : -1;
}

static int ensure_activations(Qwen3Model* m, int64_t rows) {
  if (rows <= m->act_rows) return YTC_OK;
  // (buffers of earlier, smaller calls stay owned until destroy)
  const int D = m->head_dim;
  const int qkv_w = (m->l_heads + 2 * m->l_kv_heads) * D;
  const int kmax = m->hidden > m->l_inter ? m->hidden : m->l_inter;
  const int kmax2 = kmax > m->l_heads * D ? kmax : m->l_heads * D;
  int s;
  if ((s = dev_alloc(m, reinterpret_cast<void**>(&m->x), rows * m->hidden * 4)) != YTC_OK) return s;
  if ((s = dev_alloc(m, reinterpret_cast<void**>(&m->h), rows * m->hidden * 4)) != YTC_OK) return s;
  if ((s = dev_alloc(m, reinterpret_cast<void**>(&m->proj), rows * m->hidden * 4)) != YTC_OK) return s;
  if ((s = dev_alloc(m, reinterpret_cast<void**>(&m->qkv), rows * qkv_w * 4)) != YTC_OK) return s;
  if ((s = dev_alloc(m, reinterpret_cast<void**>(&m->q), rows * m->l_heads * D * 4)) != YTC_OK) return s;
  if ((s = dev_alloc(m, reinterpret_cast<void**>(&m->attn), rows * m->l_heads * D * 4)) != YTC_OK) return s;
  if ((s = dev_alloc(m, reinterpret_cast<void**>(&m->gu), rows * 2 * m->l_inter * 4)) != YTC_OK) return s;
  if ((s = dev_alloc(m, reinterpret_cast<void**>(&m->act), rows * m->l_inter * 4)) != YTC_OK) return s;
  if ((s = dev_alloc(m, reinterpret_cast<void**>(&m->hi), rows * kmax2 * 4)) != YTC_OK) return s;  // hi and lo planes
  if (!m->last && (s = dev_alloc(m, reinterpret_cast<void**>(&m->last), static_cast<size_t>(m->batch) * m->hidden * 8)) != YTC_OK)
    return s;
  m->act_rows = rows;
  return YTC_OK;
}

constexpr int DS_MAX_CHUNKS = 64;
// Sequences up to which the step kernel is the automatic choice. On one GPU the operator path with tensor-core
// linears wins from 7 on (per step at 6 / 8 sequences: 2.37 / 2.70 ms against 2.51 / 2.54); under tensor parallelism
// the step kernel keeps the sums over ranks inside the kernel, which the operator path pays a collective call for.
constexpr int DS_AUTO_B = 6;
constexpr int DS_AUTO_B_TP = 8;
static int ds_auto_b(const Qwen3Model* m) { return m->tp_world > 1 ? DS_AUTO_B_TP : DS_AUTO_B; }


// Whether the persistent step kernel covers this model (one new token per sequence is checked by the caller).
// Activation rows the step kernel is instantiated for, and the columns of them that fit its shared memory at once.
static int ds_rows(int batch) { return batch <= 1 ? 1 : batch <= 2 ? 2 : batch <= 4 ? 4 : batch <= 8 ? 8 : batch <= 16 ? 16 : 32; }
static int ds_xs_cols(int mt) {
  int cols = (160 * 1024 / (mt * 4)) / 256 * 256;
  return cols > 3072 ? 3072 : cols;
}

// Whether the step kernel's linear phases run on the tensor cores: enough sequences for that to pay, activation rows
// that fit the staging area in one piece, whole blocks of 32 columns. decode_path 3 keeps the FFMA form.
static bool decode_step_mma(const Qwen3Model* m) {
  return m->decode_path != 3 && m->batch >= DS_MMA_MIN_B && m->hidden <= DS_MMA_XC && m->hidden % 32 == 0 &&
         (m->l_heads * 128) % 32 == 0 && m->l_inter % 32 == 0;
}

static bool decode_step_supported(const Qwen3Model* m) {
  const int groups = m->heads / m->kv_heads;
  const int xs_cols = ds_xs_cols(ds_rows(m->batch));
  const int gw = sm_count() * DS_WARPS;
  // whole activation rows must fit shared memory unless the phase has at most one weight row per warp
  auto fits = [&](int n, int k) { return k <= xs_cols || n <= gw; };
  if (m->hidden > xs_cols || !fits(m->hidden, m->l_heads * 128) || !fits(m->hidden, m->l_inter)) return false;
  return (m->tp_world == 1 || m->tp_ready) && m->batch <= DS_MAX_B && m->head_dim == 128 && (groups == 1 || groups == 2 || groups == 4) &&
         m->hidden % 8 == 0 && m->inter % 8 == 0;
}

// One decode step as one cooperative launch; activations must have been allocated for `batch` rows.
static int decode_step_launch(Qwen3Model* m, const int32_t* ids, float* logits, cudaStream_t st) {
  const int B = m->batch, D = m->head_dim;
  const int groups = m->heads / m->kv_heads;
  const size_t sync_words = 1;
  if (!m->ds_part) {
    int s;
    const size_t part = static_cast<size_t>(B) * m->l_kv_heads * DS_MAX_CHUNKS * groups * (4 + D) * sizeof(float);
    if ((s = dev_alloc(m, reinterpret_cast<void**>(&m->ds_part), part)) != YTC_OK) return s;
    if ((s = dev_alloc(m, reinterpret_cast<void**>(&m->ds_sync), sync_words * sizeof(unsigned int))) != YTC_OK) return s;
    if ((s = dev_alloc(m, reinterpret_cast<void**>(&m->ds_lw), m->layers * sizeof(DsLayer))) != YTC_OK) return s;
  }
  if (m->ds_lw_stale) {
    std::vector<DsLayer> h(m->layers);
    for (int l = 0; l < m->layers; ++l) {
      const LayerW& L = m->lw[l];
      h[l] = DsLayer{L.qkv, L.o, L.gate_up, L.down, L.q_norm, L.k_norm, L.norm1, L.norm2};
    }
    YTC_CUDA(cudaMemcpyAsync(m->ds_lw, h.data(), h.size() * sizeof(DsLayer), cudaMemcpyHostToDevice, st));
    YTC_CUDA(cudaStreamSynchronize(st));  // `h` leaves scope
    m->ds_lw_stale = false;
  }
  int kmax = m->hidden > m->l_inter ? m->hidden : m->l_inter;
  if (m->l_heads * D > kmax) kmax = m->l_heads * D;
  // the kernel is instantiated for 1 .. 32 activation rows and reads that many rows of shared memory
  const int mt = ds_rows(B);
  const int xs_cols = ds_xs_cols(mt);
  int smem = mt * (kmax < xs_cols ? kmax : xs_cols) * static_cast<int>(sizeof(float));
  const int att = DS_ATT_FLOATS * static_cast<int>(sizeof(float));  // the attention phase's scratch
  if (smem < att) smem = att;
  const bool mma = decode_step_mma(m);
  if (mma) {
    const int need = ds_mma_smem_floats(mt > 16 ? 32 : 16) * static_cast<int>(sizeof(float));
    if (smem < need) smem = need;
  }
  DecodeStepParams p{};
  p.mma = mma ? 1 : 0;
  p.B = B; p.hidden = m->hidden; p.layers = m->layers; p.heads = m->l_heads; p.kv_heads = m->l_kv_heads;
  p.inter = m->l_inter; p.vocab_rows = m->l_vocab; p.vocab = m->vocab; p.max_pos = m->max_pos;
  const bool wrapped = m->total_written >= m->max_pos;  // (the caller has checked that the cache is then full)
  p.pos = static_cast<int>(m->total_written % m->max_pos);
  p.rope_pos = wrapped ? 0 : p.pos;
  p.n_keys = wrapped ? m->max_pos : p.pos + 1;
  p.eps = m->eps; p.scale = 1.0f / std::sqrt(static_cast<float>(D));
  p.ids = ids; p.embed = m->embed; p.lm_head = m->lm_head; p.final_norm = m->final_norm; p.lw = m->ds_lw;
  p.cos_t = m->cos_t; p.sin_t = m->sin_t; p.k_cache = m->k_cache; p.v_cache = m->v_cache;
  p.cache_layer = static_cast<size_t>(B) * m->l_kv_heads * m->max_pos * D;
  p.tp_rank = m->tp_rank; p.tp_world = m->tp_world; p.ar_base = m->ar_seq;
  p.wait_cycles = wait_cycle_limit();
  p.trace = m->trace;
  p.trace_cap = m->trace_cap;
  if (m->tp_world > 1) {
    const size_t flags_at = tp_flags_offset(m->hidden);
    for (int r = 0; r < m->tp_world; ++r) {
      char* base = r == m->tp_rank ? m->tp_comm : m->tp_peer[r];
      p.mail[r] = reinterpret_cast<float*>(base);
      p.flags[r] = reinterpret_cast<unsigned int*>(base + flags_at);
      p.ll_mail[r] = reinterpret_cast<uint2*>(base + tp_pairs_offset(m->hidden));
    }
    p.go = reinterpret_cast<unsigned int*>(m->tp_comm + flags_at) + 16;
  }
  p.x = m->x; p.qkv = m->qkv; p.attn = m->attn; p.act = m->act; p.logits = logits; p.part = m->ds_part;
  p.sync = m->ds_sync; p.status = device_status_word();
  const int keys = p.n_keys;
  // Key chunks of 128 keys (8 per warp), fewer and longer ones when that would be more units than CTAs or more
  // than DS_MAX_CHUNKS chunks.
  // (The barrier-free form has seven worker warps of 16 keys each: chunks of 112 keys keep every warp at one pass.)
  const bool ll_shape = !mma && mt <= 4 && m->decode_path != 4 && m->decode_path != 5;
  const int unit_keys = ll_shape ? LL_WARPS * DS_KB : 128;
  int n_chunks = (keys + unit_keys - 1) / unit_keys;
  const int fit = sm_count() / (B * m->l_kv_heads);
  if (n_chunks > fit) n_chunks = fit > 0 ? fit : 1;
  if (n_chunks > DS_MAX_CHUNKS) n_chunks = DS_MAX_CHUNKS;
  int per = (keys + n_chunks - 1) / n_chunks;
  per = ll_shape ? (per + 15) / 16 * 16 : (per + 31) / 32 * 32;  // whole blocks of keys
  p.keys_per_chunk = per;
  p.chunks = (keys + per - 1) / per;
  p.xs_cols = xs_cols;
  YTC_CUDA(cudaMemsetAsync(m->ds_sync, 0, sync_words * sizeof(unsigned int), st));
  void* args[] = {&p};
  const void* fn = nullptr;
  // Up to four sequences: the forms of the kernel that stream their weights through a shared-memory ring, unless
  // decode_path 4 asks for the older form or a size does not fit the chunks. One GPU: no grid barriers, activations
  // exchanged as tagged pairs (decode_ll.cuh); tensor parallel, or decode_path 5: barriers kept (decode_stream.cuh).
  if (!mma && mt <= 4 && m->decode_path != 4 && m->layers <= DW_MAX_LAYERS) {
    // (a CTA holds at most one attention unit unless there is a single key chunk: the collecting unit of the
    // barrier-free form never waits for a unit of its own CTA)
    const bool ll = m->decode_path != 5 && (m->hidden + sm_count() - 1) / sm_count() + 1 <= LL_MAX_OWN &&
                    (p.chunks == 1 || B * m->l_kv_heads * p.chunks <= sm_count()) && p.chunks <= DS_MAX_CHUNKS_LL;
    const int head = static_cast<int>((sizeof(DwShared) + 127) / 128 * 128) +
                     (ll ? (DS_WARPS * 4 + 4 * LL_MAX_OWN + ll_part_floats(mt)) * 4 : 0);
    int xs_bytes = mt * ll_row_floats(kmax) * static_cast<int>(sizeof(float));  // (rows padded to whole 256-column blocks)
    // the attention phase's scratch: the barrier-free form has seven warps and this model's group size
    const int att_here = ll ? ll_att_floats(groups) * static_cast<int>(sizeof(float)) : att;
    if (xs_bytes < att_here) xs_bytes = att_here;
    xs_bytes = (xs_bytes + 127) / 128 * 128;
    int nslot = (227 * 1024 - head - xs_bytes) / DW_CHUNK;
    if (nslot > DW_MAX_SLOTS) nslot = DW_MAX_SLOTS;
    const bool fits = nslot >= 2 && kmax * 2 <= DW_CHUNK && m->hidden * 4 <= DW_CHUNK && m->hidden % 8 == 0 &&
                      m->l_inter % 8 == 0 && (!ll || (m->hidden % 64 == 0 && m->l_inter % 64 == 0));
    if (fits && ll) {
      const int qkv_w = (m->l_heads + 2 * m->l_kv_heads) * D;
      const size_t part_pairs = static_cast<size_t>(B) * m->l_kv_heads * DS_MAX_CHUNKS_LL * groups * (2 + D);
      const size_t pairs = static_cast<size_t>(B) * (m->hidden + qkv_w + m->l_heads * D + m->l_inter) + part_pairs;
      const size_t need = pairs * sizeof(uint2);
      if (!m->ll_buf || m->ll_bytes < need) {
        int s = dev_alloc(m, reinterpret_cast<void**>(&m->ll_buf), need);
        if (s != YTC_OK) return s;
        m->ll_bytes = need;
        m->ll_base = 0xFFFFFFFFu;  // forces the clearing below
      }
      const unsigned int per_step = 2u + 5u * static_cast<unsigned int>(m->layers);
      if (m->ll_base > 0xF0000000u) {  // first use, or the tags are about to wrap: start again from clean buffers
        YTC_CUDA(cudaMemsetAsync(m->ll_buf, 0, m->ll_bytes, st));
        m->ll_base = 1;
      }
      uint2* q = reinterpret_cast<uint2*>(m->ll_buf);
      p.ll_x = q;
      p.ll_qkv = p.ll_x + static_cast<size_t>(B) * m->hidden;
      p.ll_att = p.ll_qkv + static_cast<size_t>(B) * qkv_w;
      p.ll_act = p.ll_att + static_cast<size_t>(B) * m->l_heads * D;
      p.ll_part = p.ll_act + static_cast<size_t>(B) * m->l_inter;
      p.ll_base = m->ll_base;
      p.dw_xs_bytes = xs_bytes;
      p.dw_nslot = nslot;
      const int dsmem = head + xs_bytes + nslot * DW_CHUNK;
#define LL_PICK(MT)                                                                         \
  fn = groups == 1   ? reinterpret_cast<const void*>(decode_ll_kernel<MT, 1>)               \
       : groups == 2 ? reinterpret_cast<const void*>(decode_ll_kernel<MT, 2>)               \
                     : reinterpret_cast<const void*>(decode_ll_kernel<MT, 4>)
      if (mt == 1) LL_PICK(1);
      else if (mt == 2) LL_PICK(2);
      else LL_PICK(4);
#undef LL_PICK
      const int sa = ensure_dynamic_smem(fn, dsmem);
      if (sa != YTC_OK) return sa;
      YTC_CUDA(cudaLaunchCooperativeKernel(fn, dim3(sm_count()), dim3(LL_THREADS), args, dsmem, st));
      count_launch();
      m->ll_base += per_step;
      return YTC_OK;
    }
    if (fits && m->decode_path == 5) {  // (on request only: with its barriers kept, the ring alone does not pay)
      p.dw_xs_bytes = xs_bytes;
      p.dw_nslot = nslot;
      const int dsmem = head + xs_bytes + nslot * DW_CHUNK;
#define DW_PICK(MT)                                                                             \
  fn = groups == 1   ? reinterpret_cast<const void*>(decode_stream_kernel<MT, 1>)               \
       : groups == 2 ? reinterpret_cast<const void*>(decode_stream_kernel<MT, 2>)               \
                     : reinterpret_cast<const void*>(decode_stream_kernel<MT, 4>)
      if (mt == 1) DW_PICK(1);
      else if (mt == 2) DW_PICK(2);
      else DW_PICK(4);
#undef DW_PICK
      const int sa = ensure_dynamic_smem(fn, dsmem);
      if (sa != YTC_OK) return sa;
      YTC_CUDA(cudaLaunchCooperativeKernel(fn, dim3(sm_count()), dim3(DS_THREADS), args, dsmem, st));
      count_launch();
      if (m->tp_world > 1) m->ar_seq += 2u * static_cast<unsigned int>(m->layers);
      return YTC_OK;
    }
  }
#define DS_PICK_G(MT, MMA)                                                                    \
  fn = groups == 1   ? reinterpret_cast<const void*>(decode_step_kernel<MT, 1, MMA>)          \
       : groups == 2 ? reinterpret_cast<const void*>(decode_step_kernel<MT, 2, MMA>)          \
                     : reinterpret_cast<const void*>(decode_step_kernel<MT, 4, MMA>)
#define DS_PICK(MT)              \
  do {                           \
    if (mma) DS_PICK_G(MT, true); \
    else DS_PICK_G(MT, false);   \
  } while (0)
  if (mt == 1) DS_PICK_G(1, false);
  else if (mt == 2) DS_PICK(2);
  else if (mt == 4) DS_PICK(4);
  else if (mt == 8) DS_PICK(8);
  else if (mt == 16) DS_PICK(16);
  else DS_PICK(32);
#undef DS_PICK_G
#undef DS_PICK
  // the limit belongs to the (device, kernel) pair, not to the model: several models (other paths, other sizes)
  // share a kernel, and a smaller request must not lower what another model's launches need
  {
    const int sa = ensure_dynamic_smem(fn, smem);
    if (sa != YTC_OK) return sa;
  }
  YTC_CUDA(cudaLaunchCooperativeKernel(fn, dim3(sm_count()), dim3(DS_THREADS), args, smem, st));
  count_launch();
  if (m->tp_world > 1) m->ar_seq += 2u * static_cast<unsigned int>(m->layers);
  return YTC_OK;
}

// ids [batch, len] (device int32) -> logits [batch, this rank's vocab rows] (device fp32) of the LAST position;
// appends `len` tokens to the KV caches (qwen3::Qwen3ForCausalLM::forward, reference qwen3.cpp:449-457).
int ytcuda_qwen3_forward(void* handle, const int32_t* ids, int len, float* logits, void* stream) {
  struct OverlapGuard {
    OverlapGuard() { overlap_scope() = true; }
    ~OverlapGuard() { overlap_scope() = false; }
  } overlap_guard;  // the tile GEMMs of this forward are queued as programmatic dependent launches
  auto* m = static_cast<Qwen3Model*>(handle);
  YTC_REQUIRE(m && ids && logits, "ytcuda_qwen3_forward: null argument");
  YTC_REQUIRE(len > 0, "ytcuda_qwen3_forward: len must be positive");
  // The KV cache is a ring buffer (reference example/qwen3/src/qwen3.cpp:70-126): once it is full, a new token
  // overwrites the oldest slot, sees every slot, and takes rotary position 0 (the position rule of
  // Qwen3Model::forward, :365-375, falls back to 0 when the running position no longer fits the table). The device
  // follows that for one new token per call; a longer input that would run over the end of the cache is refused.
  const bool wrap_step = len == 1 && m->total_written >= m->max_pos;
  // several tokens that run over the end of the ring: every token is appended (the later ones overwrite the oldest
  // slots), then each query sees the slots that are not younger than itself (KVCache::append / get_mask, :70-126)
  const bool ring_multi = !wrap_step && m->total_written + len > m->max_pos;
  if (ring_multi && len > m->max_pos) {
    set_last_error("ytcuda_qwen3_forward: %d new tokens do not fit a cache of %d slots", len, m->max_pos);
    return YTC_UNSUPPORTED;
  }
  YTC_REQUIRE(m->embed && m->lm_head && m->final_norm, "ytcuda_qwen3_forward: embed / lm_head / norm not set");
  for (const LayerW& L : m->lw)
    YTC_REQUIRE(L.qkv && L.o && L.gate_up && L.down && L.q_norm && L.k_norm && L.norm1 && L.norm2,
                "ytcuda_qwen3_forward: a layer weight is not set");
  YTC_REQUIRE(m->tp_world == 1 || m->allreduce ||
                  (len == 1 && m->tp_ready && ((m->decode_path >= 2 && m->decode_path <= 5) || (m->decode_path == 0 && m->batch <= ds_auto_b(m)))),
              "ytcuda_qwen3_forward: tensor parallel needs an all-reduce callback");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int B = m->batch, D = m->head_dim, Hd = m->hidden;
  const int64_t rows = static_cast<int64_t>(B) * len;
  int s = ensure_activations(m, rows);
  if (s != YTC_OK) return s;
  // rotary position of the first new token, the slot it is written to, and the keys visible after the append
  // rotary position of the first new token (Qwen3Model::forward, :365-375): the running position while it fits the
  // table, else the cache length, else 0
  int pos0 = wrap_step ? 0 : static_cast<int>(m->total_written);
  if (ring_multi) pos0 = m->cur_len + len <= m->max_pos ? m->cur_len : 0;
  const int slot0 = static_cast<int>(m->total_written % m->max_pos);
  const int kv_len = (wrap_step || ring_multi) ? m->max_pos : pos0 + len;
  int mask_kind = wrap_step ? 0 : 1;
  const uint8_t* mask_ptr = nullptr;
  if (ring_multi) {
    const size_t need = static_cast<size_t>(len) * m->max_pos;
    if (m->ring_mask_bytes < need) {
      if ((s = dev_alloc(m, reinterpret_cast<void**>(&m->ring_mask), need)) != YTC_OK) return s;
      m->ring_mask_bytes = need;
    }
    const int write_pos = static_cast<int>((m->total_written + len) % m->max_pos);
    ring_mask_kernel<<<static_cast<unsigned>((need + 255) / 256 < 1024 ? (need + 255) / 256 : 1024), 256, 0, st>>>(
        m->ring_mask, len, m->max_pos, write_pos);
    count_launch();
    YTC_CUDA(cudaGetLastError());
    mask_kind = 2;
    mask_ptr = m->ring_mask;
  }
  auto advance = [&]() {
    m->total_written += len;
    m->cur_len = m->total_written < m->max_pos ? static_cast<int>(m->total_written) : m->max_pos;
  };
  // Automatic choice: the step kernel up to ds_auto_b() sequences. Beyond that its linear phases lose against the
  // tensor-core linears of the operator path (measured at 16 and 32 sequences), so it runs only when asked for.
  const bool want_step = m->decode_path >= 2 && m->decode_path <= 5;  // (6: operator path, sums over ranks by callback)
  if (len == 1 && (want_step || (m->decode_path == 0 && m->batch <= ds_auto_b(m))) && decode_step_supported(m)) {
    if ((s = decode_step_launch(m, ids, logits, st)) != YTC_OK) return s;
    advance();
    return YTC_OK;
  }
  if (len == 1 && want_step) {
    set_last_error("ytcuda_qwen3_forward: the single-kernel decode step needs batch <= %d, 1, 2 or %d query heads "
                   "per kv head and, under tensor parallelism, connected exchange buffers", DS_MAX_B, DS_MAX_G);
    return YTC_UNSUPPORTED;
  }
  const int qkv_w = (m->l_heads + 2 * m->l_kv_heads) * D;
  const int groups = m->heads / m->kv_heads;
  const float scale = 1.0f / std::sqrt(static_cast<float>(D));
  const size_t cache_layer = static_cast<size_t>(B) * m->l_kv_heads * m->max_pos * D;

  if ((s = ytcuda_embedding(m->embed, ids, m->x, rows, Hd, m->vocab, st)) != YTC_OK) return s;
  // 5 .. 128 rows on one GPU: every projection runs as k pieces on the tensor cores, and the kernels between two
  // projections (sum of the pieces, residual, rmsNorm or SwiGLU or the per-head norm + RoPE, the split into bf16
  // planes) are one launch each: 11 launches per layer instead of 18.
  // Tensor parallel (exchange buffers connected, up to TP_PUSH_ROWS rows): the same launches; the kernel that adds the
  // pieces of the o or down projection to the residual stream also exchanges the ranks' shares (no collective call).
  const bool fused_glue = (m->tp_world == 1 || (m->tp_ready && rows <= TP_PUSH_ROWS && m->decode_path != 6)) &&
                          rows > SK_MAX_ROWS && split_k_ok(rows, Hd) && split_k_ok(rows, m->l_heads * D) &&
                          split_k_ok(rows, m->l_inter) && Hd <= 3072;
  if (fused_glue) {
    Pieces pc;  // the projection whose pieces still have to be added to the residual stream
    const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
    for (int l = 0; l < m->layers; ++l) {
      const LayerW& W = m->lw[l];
      float* kc = m->k_cache + l * cache_layer;
      float* vc = m->v_cache + l * cache_layer;
      if ((s = sum_norm_split(m, pc, m->x, W.norm1, rows, Hd, st, true)) != YTC_OK) return s;
      if ((s = gemm_pieces(m, W.qkv, rows, qkv_w, Hd, &pc, st)) != YTC_OK) return s;
      if ((s = qkv_post_launch(pc.part, pc.n, pc.mn, m->q, kc, vc, W.q_norm, W.k_norm, m->cos_t, m->sin_t, B, len,
                               m->l_heads, m->l_kv_heads, D, m->max_pos, pos0, slot0, m->eps, st)) != YTC_OK)
        return s;
      const int64_t qs[3] = {static_cast<int64_t>(m->l_heads) * len * D, static_cast<int64_t>(len) * D, D};
      const int64_t ks[3] = {static_cast<int64_t>(m->l_kv_heads) * m->max_pos * D, static_cast<int64_t>(m->max_pos) * D, D};
      const int64_t os[3] = {static_cast<int64_t>(len) * m->l_heads * D, D, static_cast<int64_t>(m->l_heads) * D};
      if ((s = ytcuda_flash_attn_fwd(YTC_F32, m->q, kc, vc, m->attn, B, m->l_kv_heads, groups, len, kv_len, D, D, scale,
                                     qs, ks, ks, os, mask_kind, kv_len - len, mask_ptr, m->max_pos, nullptr, 0, 0, st)) !=
          YTC_OK)
        return s;
      if ((s = split_planes(m, m->attn, m->l_heads * D, rows, m->l_heads * D, st)) != YTC_OK) return s;
      if ((s = gemm_pieces(m, W.o, rows, Hd, m->l_heads * D, &pc, st)) != YTC_OK) return s;
      if ((s = sum_norm_split(m, pc, m->x, W.norm2, rows, Hd, st, true)) != YTC_OK) return s;
      if ((s = gemm_pieces(m, W.gate_up, rows, 2 * m->l_inter, Hd, &pc, st)) != YTC_OK) return s;
      {
        const int64_t blocks = (rows * (m->l_inter / 4) + 127) / 128;
        YTC_CUDA(launch_overlapped(sum_swiglu_split_kernel, dim3(static_cast<unsigned>(blocks < cap ? blocks : cap)),
                                   dim3(128), 0, st, pc.part, pc.n, pc.mn, m->hi, m->hi + rows * m->l_inter, rows,
                                   m->l_inter));
        count_launch();
        YTC_CUDA(cudaGetLastError());
      }
      if ((s = gemm_pieces(m, W.down, rows, Hd, m->l_inter, &pc, st)) != YTC_OK) return s;
    }
    if (m->tp_world > 1) {  // the last down projection joins the residual stream (sum and exchange only)
      if ((s = sum_norm_split(m, pc, m->x, nullptr, rows, Hd, st, true)) != YTC_OK) return s;
    } else {
      const int64_t blocks = (pc.mn + 255) / 256;
      sum_partials_kernel<<<static_cast<unsigned>(blocks < cap ? blocks : cap), 256, 0, st>>>(pc.part, pc.n, pc.mn,
                                                                                               m->x, Hd, Hd, 1);
      count_launch();
      YTC_CUDA(cudaGetLastError());
    }
  }
  for (int l = fused_glue ? m->layers : 0; l < m->layers; ++l) {
    const LayerW& W = m->lw[l];
    float* kc = m->k_cache + l * cache_layer;
    float* vc = m->v_cache + l * cache_layer;
    if ((s = rmsnorm_rows(m->x, W.norm1, m->h, rows, Hd, m->eps, st)) != YTC_OK) return s;
    if ((s = linear_w16(m, m->h, Hd, W.qkv, m->qkv, qkv_w, rows, qkv_w, Hd, false, st)) != YTC_OK) return s;
    if ((s = ytcuda_qwen3_qkv_post(m->qkv, m->q, kc, vc, W.q_norm, W.k_norm, m->cos_t, m->sin_t, B, len, m->l_heads,
                                   m->l_kv_heads, D, m->max_pos, pos0, slot0, m->eps, st)) != YTC_OK)
      return s;
    // attention over the cache; the output lands as [B, len, heads, D] = rows x (heads * D)
    const int64_t qs[3] = {static_cast<int64_t>(m->l_heads) * len * D, static_cast<int64_t>(len) * D, D};
    const int64_t ks[3] = {static_cast<int64_t>(m->l_kv_heads) * m->max_pos * D, static_cast<int64_t>(m->max_pos) * D, D};
    const int64_t os[3] = {static_cast<int64_t>(len) * m->l_heads * D, D, static_cast<int64_t>(m->l_heads) * D};
    if ((s = ytcuda_flash_attn_fwd(YTC_F32, m->q, kc, vc, m->attn, B, m->l_kv_heads, groups, len, kv_len, D, D, scale, qs,
                                   ks, ks, os, mask_kind, kv_len - len, mask_ptr, m->max_pos, nullptr, 0, 0, st)) != YTC_OK)
      return s;
    if (m->tp_world == 1) {  // x2 = attn + x: the projection accumulates into the residual stream
      if ((s = linear_w16(m, m->attn, m->l_heads * D, W.o, m->x, Hd, rows, Hd, m->l_heads * D, true, st)) != YTC_OK)
        return s;
    } else {
      if ((s = linear_w16(m, m->attn, m->l_heads * D, W.o, m->proj, Hd, rows, Hd, m->l_heads * D, false, st)) != YTC_OK)
        return s;
      if ((s = m->allreduce(m->proj, rows * Hd, m->allreduce_user)) != 0) {
        set_last_error("ytcuda_qwen3_forward: all-reduce callback failed with %d", s);
        return YTC_CUDA_ERROR;
      }
      if ((s = add_inplace(m->x, m->proj, rows * Hd, st)) != YTC_OK) return s;
    }
    if ((s = rmsnorm_rows(m->x, W.norm2, m->h, rows, Hd, m->eps, st)) != YTC_OK) return s;
    if ((s = linear_w16(m, m->h, Hd, W.gate_up, m->gu, 2 * m->l_inter, rows, 2 * m->l_inter, Hd, false, st)) != YTC_OK)
      return s;
    if ((s = ytcuda_swiglu(YTC_F32, YTC_F32, m->gu, m->act, rows, m->l_inter, 2 * m->l_inter, m->l_inter, st)) != YTC_OK)
      return s;
    if (m->tp_world == 1) {  // x2 += mlp
      if ((s = linear_w16(m, m->act, m->l_inter, W.down, m->x, Hd, rows, Hd, m->l_inter, true, st)) != YTC_OK) return s;
    } else {
      if ((s = linear_w16(m, m->act, m->l_inter, W.down, m->proj, Hd, rows, Hd, m->l_inter, false, st)) != YTC_OK)
        return s;
      if ((s = m->allreduce(m->proj, rows * Hd, m->allreduce_user)) != 0) {
        set_last_error("ytcuda_qwen3_forward: all-reduce callback failed with %d", s);
        return YTC_CUDA_ERROR;
      }
      if ((s = add_inplace(m->x, m->proj, rows * Hd, st)) != YTC_OK) return s;
    }
  }
  // last position of every sequence -> final norm -> vocabulary projection
  float* last_in = m->last;
  float* last_out = m->last + static_cast<size_t>(B) * Hd;
  YTC_CUDA(cudaMemcpy2DAsync(last_in, Hd * sizeof(float), m->x + static_cast<int64_t>(len - 1) * Hd,
                             static_cast<size_t>(len) * Hd * sizeof(float), Hd * sizeof(float), B,
                             cudaMemcpyDeviceToDevice, st));
  if ((s = rmsnorm_rows(last_in, m->final_norm, last_out, B, Hd, m->eps, st)) != YTC_OK) return s;
  if ((s = linear_w16(m, last_out, Hd, m->lm_head, logits, m->l_vocab, B, m->l_vocab, Hd, false, st)) != YTC_OK) return s;
  advance();
  return YTC_OK;
}

}  // extern "C"
