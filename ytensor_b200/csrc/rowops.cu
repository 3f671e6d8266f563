// Bandwidth-bound reductions over one or several axes: softmax, RMSNorm, LayerNorm, the fused
// RMSNorm + residual + softmax + cast chain, and sum / mean / max(+argmax).
//
// Two kernels:
//  * row_kernel  : the reduced axes are the trailing, contiguous dims. A group of G threads owns a row,
//                  keeps it in registers (4 x 128-bit loads per thread), reduces with warp shuffles
//                  (+ one shared-memory hop above 32 threads) and writes the result once: one read and
//                  one write of HBM per element.
//  * line_kernel : any axes, any strides. A "line" is the set of elements reduced together; its
//                  elements are walked as an odometer over the reduced dims in the order the caller
//                  listed them (the order the reference's argmax index refers to). Either one CTA
//                  per line, or one thread per line when neighbouring lines are contiguous in memory.
//
// Replaces yt::function::softmax / rmsNorm / layerNorm (reference src/function/activation.inl:130-409,
// src/function/normalization.inl:3-54,159-277) and YTensor::sum / mean / max
// (src/ytensor_math.inl:414-692).
#include <math_constants.h>

#include <atomic>
#include <mutex>

#include "ytc_common.cuh"

namespace ytk {

enum RowOp { OP_SOFTMAX = 0, OP_RMSNORM = 1, OP_LAYERNORM = 2, OP_CHAIN = 3, OP_SUM = 4, OP_MEAN = 5, OP_MAX = 6,
             OP_LPNORM = 7 };

struct F4 {
  float v[4];
};

__device__ __forceinline__ F4 load4(const void* p, int64_t i, int dt) {
  F4 r;
  if (dt == YTC_F32) {
    const float4 t = *reinterpret_cast<const float4*>(static_cast<const float*>(p) + i);
    r.v[0] = t.x; r.v[1] = t.y; r.v[2] = t.z; r.v[3] = t.w;
  } else {
    const uint2 t = *reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(p) + i);
    const uint16_t h[4] = {static_cast<uint16_t>(t.x & 0xFFFF), static_cast<uint16_t>(t.x >> 16),
                           static_cast<uint16_t>(t.y & 0xFFFF), static_cast<uint16_t>(t.y >> 16)};
#pragma unroll
    for (int k = 0; k < 4; ++k) r.v[k] = (dt == YTC_BF16) ? bf16_bits_to_f32(h[k]) : f16_bits_to_f32_ref(h[k]);
  }
  return r;
}
__device__ __forceinline__ void store4(void* p, int64_t i, const F4& r, int dt) {
  if (dt == YTC_F32) {
    *reinterpret_cast<float4*>(static_cast<float*>(p) + i) = make_float4(r.v[0], r.v[1], r.v[2], r.v[3]);
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

struct MaxIdx {
  float v;
  int i;
};
// Keeps the first maximum: a later element wins only if it is strictly greater
// (reference src/ytensor_math.inl:591-617 compares with `>` walking upwards).
__device__ __forceinline__ MaxIdx max_combine(MaxIdx a, MaxIdx b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

template <int G>
__device__ __forceinline__ float group_sum(float v, float* red, int group, int t) {
#pragma unroll
  for (int o = (G < 32 ? G : 32) / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if constexpr (G > 32) {
    constexpr int W = G / 32;
    if ((t & 31) == 0) red[group * W + (t >> 5)] = v;
    __syncthreads();
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < W; ++w) s += red[group * W + w];
    __syncthreads();
    v = s;
  }
  return v;
}
template <int G>
__device__ __forceinline__ float group_max(float v, float* red, int group, int t) {
#pragma unroll
  for (int o = (G < 32 ? G : 32) / 2; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if constexpr (G > 32) {
    constexpr int W = G / 32;
    if ((t & 31) == 0) red[group * W + (t >> 5)] = v;
    __syncthreads();
    float s = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < W; ++w) s = fmaxf(s, red[group * W + w]);
    __syncthreads();
    v = s;
  }
  return v;
}
template <int G>
__device__ __forceinline__ MaxIdx group_maxidx(MaxIdx m, float* red, int* redi, int group, int t) {
#pragma unroll
  for (int o = (G < 32 ? G : 32) / 2; o > 0; o >>= 1) {
    MaxIdx b;
    b.v = __shfl_xor_sync(0xffffffffu, m.v, o);
    b.i = __shfl_xor_sync(0xffffffffu, m.i, o);
    m = max_combine(m, b);
  }
  if constexpr (G > 32) {
    constexpr int W = G / 32;
    if ((t & 31) == 0) {
      red[group * W + (t >> 5)] = m.v;
      redi[group * W + (t >> 5)] = m.i;
    }
    __syncthreads();
    MaxIdx s = {red[group * W], redi[group * W]};
#pragma unroll
    for (int w = 1; w < W; ++w) s = max_combine(s, MaxIdx{red[group * W + w], redi[group * W + w]});
    __syncthreads();
    m = s;
  }
  return m;
}

struct RowParams {
  const void* x;
  void* y;
  const void* w;   // weight / gamma (per column), may be null
  const void* b;   // beta (layernorm) or residual r (chain), may be null
  int* idx;        // argmax output (OP_MAX), may be null
  int64_t rows;
  int L;           // row length (multiple of 4)
  int64_t x_rs, y_rs;  // row strides in elements
  int64_t r_rows;  // chain: residual row = row % r_rows
  float eps;
  int dt_in, dt_out, dt_w;
};

template <int OP, int G>
__global__ void __launch_bounds__(G < 256 ? 256 : G) row_kernel(const RowParams p) {
  dependent_wait();     // (under a programmatic dependent launch: the kernel before this one has finished)
  dependent_trigger();  // the kernel queued behind this one may be scheduled meanwhile
  constexpr int THREADS = G < 256 ? 256 : G;
  constexpr int RPC = THREADS / G;  // rows per CTA
  constexpr int VPT = 4;
  __shared__ float red[32];
  __shared__ int redi[32];
  const int group = threadIdx.x / G, t = threadIdx.x % G;
  const int64_t row_blocks = (p.rows + RPC - 1) / RPC;
  const float invL = 1.0f / static_cast<float>(p.L);

  // chain with a residual shared by `copies` batch items: walk the rows so that the `copies` rows that read the same
  // residual row are handled back to back (by neighbouring CTAs) - the residual row then comes from HBM once and
  // from L2 for the other uses, instead of being evicted between uses that lie a whole batch item apart.
  const int64_t copies = (OP == OP_CHAIN && p.r_rows < p.rows) ? p.rows / p.r_rows : 1;
  for (int64_t rb = blockIdx.x; rb < row_blocks; rb += gridDim.x) {
    int64_t row = rb * RPC + group;
    const bool row_ok = row < p.rows;
    if (OP == OP_CHAIN && copies > 1 && row_ok) row = (row % copies) * p.r_rows + row / copies;
    F4 x[VPT];
    bool act[VPT];
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      const int col = (v * G + t) * 4;
      act[v] = row_ok && col < p.L;
      if (act[v]) x[v] = load4(p.x, row * p.x_rs + col, p.dt_in);
      else x[v] = F4{{0.f, 0.f, 0.f, 0.f}};
    }

    if constexpr (OP == OP_SUM || OP == OP_MEAN) {
      float s = 0.f;
#pragma unroll
      for (int v = 0; v < VPT; ++v) s += (x[v].v[0] + x[v].v[1]) + (x[v].v[2] + x[v].v[3]);
      s = group_sum<G>(s, red, group, t);
      if (row_ok && t == 0) store_from_f32(p.y, row, OP == OP_MEAN ? s * invL : s, p.dt_out);
      continue;
    }
    if constexpr (OP == OP_MAX) {
      MaxIdx m = {-CUDART_INF_F, 0x7fffffff};
#pragma unroll
      for (int v = 0; v < VPT; ++v)
        if (act[v]) {
#pragma unroll
          for (int k = 0; k < 4; ++k) m = max_combine(m, MaxIdx{x[v].v[k], (v * G + t) * 4 + k});
        }
      m = group_maxidx<G>(m, red, redi, group, t);
      if (row_ok && t == 0) {
        if (m.i == 0x7fffffff) {  // every element failed `>` (all NaN): the reference keeps element 0
          m.v = load_as_f32(p.x, row * p.x_rs, p.dt_in);
          m.i = 0;
        }
        store_from_f32(p.y, row, m.v, p.dt_out);
        if (p.idx) p.idx[row] = m.i;
      }
      continue;
    }

    if constexpr (OP == OP_RMSNORM || OP == OP_CHAIN) {
      float ss = 0.f;
#pragma unroll
      for (int v = 0; v < VPT; ++v)
#pragma unroll
        for (int k = 0; k < 4; ++k) ss = fmaf(x[v].v[k], x[v].v[k], ss);
      // issue the residual / weight loads before the reduction so that they overlap it
      F4 rr[VPT], ww[VPT];
      if constexpr (OP == OP_CHAIN) {
        const int64_t r_off = (row_ok ? (p.r_rows == p.rows ? row : row % p.r_rows) : 0) * static_cast<int64_t>(p.L);
#pragma unroll
        for (int v = 0; v < VPT; ++v)
          if (act[v]) {
            rr[v] = load4(p.b, r_off + (v * G + t) * 4, YTC_F32);
            ww[v] = load4(p.w, (v * G + t) * 4, YTC_F32);
          }
      }
      ss = group_sum<G>(ss, red, group, t);
      const float inv = 1.0f / sqrtf(ss * invL + p.eps);
#pragma unroll
      for (int v = 0; v < VPT; ++v)
        if (act[v]) {
          const int col = (v * G + t) * 4;
#pragma unroll
          for (int k = 0; k < 4; ++k) x[v].v[k] *= inv;
          if constexpr (OP == OP_CHAIN) {
#pragma unroll
            for (int k = 0; k < 4; ++k) x[v].v[k] = fmaf(x[v].v[k], ww[v].v[k], rr[v].v[k]);
          } else if (p.w) {
            const F4 w = load4(p.w, col, p.dt_w);
#pragma unroll
            for (int k = 0; k < 4; ++k) x[v].v[k] *= w.v[k];
          }
        }
    }
    if constexpr (OP == OP_LAYERNORM) {
      float s = 0.f;
#pragma unroll
      for (int v = 0; v < VPT; ++v) s += (x[v].v[0] + x[v].v[1]) + (x[v].v[2] + x[v].v[3]);
      const float mu = group_sum<G>(s, red, group, t) * invL;
      float ss = 0.f;
#pragma unroll
      for (int v = 0; v < VPT; ++v)
        if (act[v]) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            x[v].v[k] -= mu;
            ss = fmaf(x[v].v[k], x[v].v[k], ss);
          }
        }
      ss = group_sum<G>(ss, red, group, t);
      const float inv = 1.0f / sqrtf(ss * invL + p.eps);
#pragma unroll
      for (int v = 0; v < VPT; ++v)
        if (act[v]) {
          const int col = (v * G + t) * 4;
#pragma unroll
          for (int k = 0; k < 4; ++k) x[v].v[k] *= inv;
          if (p.w) {
            const F4 w = load4(p.w, col, p.dt_w);
            const F4 bb = load4(p.b, col, p.dt_w);
#pragma unroll
            for (int k = 0; k < 4; ++k) x[v].v[k] = x[v].v[k] * w.v[k] + bb.v[k];
          }
        }
    }
    if constexpr (OP == OP_SOFTMAX || OP == OP_CHAIN) {
      float m = -CUDART_INF_F;
#pragma unroll
      for (int v = 0; v < VPT; ++v)
        if (act[v]) m = fmaxf(m, fmaxf(fmaxf(x[v].v[0], x[v].v[1]), fmaxf(x[v].v[2], x[v].v[3])));
      m = group_max<G>(m, red, group, t);
      float s = 0.f;
#pragma unroll
      for (int v = 0; v < VPT; ++v)
        if (act[v]) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            x[v].v[k] = __expf(x[v].v[k] - m);
            s += x[v].v[k];
          }
        }
      s = group_sum<G>(s, red, group, t);
      const float inv = 1.0f / s;
#pragma unroll
      for (int v = 0; v < VPT; ++v)
#pragma unroll
        for (int k = 0; k < 4; ++k) x[v].v[k] *= inv;
    }
#pragma unroll
    for (int v = 0; v < VPT; ++v)
      if (act[v]) store4(p.y, row * p.y_rs + (v * G + t) * 4, x[v], p.dt_out);
  }
}



// ------------------------------------------------------------------ fused chain, specialised
// fp32 in, bf16 out, contiguous rows of exactly 1024 * VPT columns, 256 threads per row: no predicates, no dtype
// switches, exp2 by ex2.approx with the log2(e) factor folded into one FMA, bf16 narrowing (the reference's rule:
// add half an ulp only when the kept LSB is 1, then truncate) in three integer operations plus one byte permute per
// pair. About a dozen instructions per element, 4 CTAs per SM.
__device__ __forceinline__ float ex2_ftz(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t bf16_pair_ref(float lo, float hi) {
  uint32_t a = __float_as_uint(lo), b = __float_as_uint(hi);
  a += (a >> 1) & 0x8000u;
  b += (b >> 1) & 0x8000u;
  return __byte_perm(a, b, 0x7632);  // {a.byte2, a.byte3, b.byte2, b.byte3}: the two upper halves
}

template <int VPT>
__global__ void __launch_bounds__(256, 4) chain_fast_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                            const float* __restrict__ r, uint2* __restrict__ out,
                                                            int64_t rows, int64_t r_rows, float eps) {
  constexpr int L = 1024 * VPT;
  __shared__ float red[32];
  const int t = threadIdx.x;
  const int64_t copies = r_rows < rows ? rows / r_rows : 1;
  const float invL = 1.0f / static_cast<float>(L);
  float4 wv[VPT];
#pragma unroll
  for (int v = 0; v < VPT; ++v) wv[v] = *reinterpret_cast<const float4*>(w + (v * 256 + t) * 4);
  for (int64_t rb = blockIdx.x; rb < rows; rb += gridDim.x) {
    // rows that share a residual row are handled back to back (see row_kernel)
    const int64_t row = copies > 1 ? (rb % copies) * r_rows + rb / copies : rb;
    const int64_t rrow = copies > 1 ? rb / copies : (r_rows == rows ? rb : rb % r_rows);
    const float4* xp = reinterpret_cast<const float4*>(x + row * L);
    const float4* rp = reinterpret_cast<const float4*>(r + rrow * L);
    float4 xv[VPT], rv[VPT];
#pragma unroll
    for (int v = 0; v < VPT; ++v) xv[v] = xp[v * 256 + t];
#pragma unroll
    for (int v = 0; v < VPT; ++v) rv[v] = rp[v * 256 + t];
    float ss = 0.f;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      ss = fmaf(xv[v].x, xv[v].x, ss);
      ss = fmaf(xv[v].y, xv[v].y, ss);
      ss = fmaf(xv[v].z, xv[v].z, ss);
      ss = fmaf(xv[v].w, xv[v].w, ss);
    }
    ss = group_sum<256>(ss, red, 0, t);
    const float inv = 1.0f / sqrtf(ss * invL + eps);
    float m = -CUDART_INF_F;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      xv[v].x = fmaf(xv[v].x * inv, wv[v].x, rv[v].x);
      xv[v].y = fmaf(xv[v].y * inv, wv[v].y, rv[v].y);
      xv[v].z = fmaf(xv[v].z * inv, wv[v].z, rv[v].z);
      xv[v].w = fmaf(xv[v].w * inv, wv[v].w, rv[v].w);
      m = fmaxf(m, fmaxf(fmaxf(xv[v].x, xv[v].y), fmaxf(xv[v].z, xv[v].w)));
    }
    m = group_max<256>(m, red, 0, t);
    const float nm = -m * 1.4426950408889634f;
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      xv[v].x = ex2_ftz(fmaf(xv[v].x, 1.4426950408889634f, nm));
      xv[v].y = ex2_ftz(fmaf(xv[v].y, 1.4426950408889634f, nm));
      xv[v].z = ex2_ftz(fmaf(xv[v].z, 1.4426950408889634f, nm));
      xv[v].w = ex2_ftz(fmaf(xv[v].w, 1.4426950408889634f, nm));
      s0 += xv[v].x + xv[v].y;
      s1 += xv[v].z + xv[v].w;
    }
    const float isum = 1.0f / group_sum<256>(s0 + s1, red, 0, t);
    uint2* op = out + row * (L / 4);
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      uint2 o;
      o.x = bf16_pair_ref(xv[v].x * isum, xv[v].y * isum);
      o.y = bf16_pair_ref(xv[v].z * isum, xv[v].w * isum);
      op[v * 256 + t] = o;
    }
  }
}

// ------------------------------------------------------------------ generic lines
constexpr int MAXD = 8;

struct LineParams {
  const void* x;
  void* y;
  const void* w;
  const void* b;
  int* idx;
  int nk, nr;                       // kept / reduced dim counts
  int64_t kshape[MAXD], kxs[MAXD], kys[MAXD];   // kept dims: extent, x stride, y stride
  int64_t rshape[MAXD], rxs[MAXD], rys[MAXD];   // reduced dims in LISTED order: extent, x stride, y stride
  int64_t rws[MAXD];                // stride of each reduced dim inside the weight (ascending-axis order layout)
  int64_t lines, R;
  float eps;
  float lp;  // exponent of OP_LPNORM
  int dt_in, dt_out, dt_w;
};

struct LineCtx {
  int64_t xbase, ybase;
};

__device__ __forceinline__ void line_offsets(const LineParams& p, int64_t r, int64_t& xo, int64_t& yo, int64_t& wo) {
  xo = 0; yo = 0; wo = 0;
  for (int d = p.nr - 1; d >= 0; --d) {
    const int64_t c = r % p.rshape[d];
    r /= p.rshape[d];
    xo += c * p.rxs[d];
    yo += c * p.rys[d];
    wo += c * p.rws[d];
  }
}

// PER_THREAD: one thread walks a whole line; otherwise the CTA's threads stride over it.
template <int OP, bool PER_THREAD>
__global__ void __launch_bounds__(128) line_kernel(const LineParams p) {
  __shared__ float red[32];
  __shared__ int redi[32];
  const int tid = threadIdx.x;
  int64_t line = PER_THREAD ? (blockIdx.x * static_cast<int64_t>(blockDim.x) + tid) : blockIdx.x;
  const int64_t line_step = PER_THREAD ? static_cast<int64_t>(gridDim.x) * blockDim.x : gridDim.x;
  const int64_t r0 = PER_THREAD ? 0 : tid, rstep = PER_THREAD ? 1 : 128;
  const float invR = 1.0f / static_cast<float>(p.R);
  // PER_THREAD lines finish independently; CTA lines keep every thread in the loop (block reductions inside).
  for (; PER_THREAD ? (line < p.lines) : (line < p.lines); line += line_step) {
    int64_t xb = 0, yb = 0, rem = line;
    for (int d = p.nk - 1; d >= 0; --d) {
      const int64_t c = rem % p.kshape[d];
      rem /= p.kshape[d];
      xb += c * p.kxs[d];
      yb += c * p.kys[d];
    }
    auto bsum = [&](float v) -> float {
      if constexpr (PER_THREAD) return v;
      else return group_sum<128>(v, red, 0, tid);
    };
    auto bmax = [&](float v) -> float {
      if constexpr (PER_THREAD) return v;
      else return group_max<128>(v, red, 0, tid);
    };
    int64_t xo, yo, wo;
    if constexpr (OP == OP_SUM || OP == OP_MEAN) {
      float s = 0.f;
      for (int64_t r = r0; r < p.R; r += rstep) {
        line_offsets(p, r, xo, yo, wo);
        s += load_as_f32(p.x, xb + xo, p.dt_in);
      }
      s = bsum(s);
      if (PER_THREAD || tid == 0) store_from_f32(p.y, yb, OP == OP_MEAN ? s * invR : s, p.dt_out);
    } else if constexpr (OP == OP_MAX) {
      MaxIdx m = {-CUDART_INF_F, 0x7fffffff};
      for (int64_t r = r0; r < p.R; r += rstep) {
        line_offsets(p, r, xo, yo, wo);
        m = max_combine(m, MaxIdx{load_as_f32(p.x, xb + xo, p.dt_in), static_cast<int>(r)});
      }
      if constexpr (!PER_THREAD) m = group_maxidx<128>(m, red, redi, 0, tid);
      if (PER_THREAD || tid == 0) {
        if (m.i == 0x7fffffff) {
          m.v = load_as_f32(p.x, xb, p.dt_in);
          m.i = 0;
        }
        store_from_f32(p.y, yb, m.v, p.dt_out);
        if (p.idx) p.idx[line] = m.i;
      }
    } else if constexpr (OP == OP_SOFTMAX) {
      float m = -CUDART_INF_F;
      for (int64_t r = r0; r < p.R; r += rstep) {
        line_offsets(p, r, xo, yo, wo);
        m = fmaxf(m, load_as_f32(p.x, xb + xo, p.dt_in));
      }
      m = bmax(m);
      float s = 0.f;
      for (int64_t r = r0; r < p.R; r += rstep) {
        line_offsets(p, r, xo, yo, wo);
        s += __expf(load_as_f32(p.x, xb + xo, p.dt_in) - m);
      }
      s = bsum(s);
      const float inv = 1.0f / s;
      for (int64_t r = r0; r < p.R; r += rstep) {
        line_offsets(p, r, xo, yo, wo);
        store_from_f32(p.y, yb + yo, __expf(load_as_f32(p.x, xb + xo, p.dt_in) - m) * inv, p.dt_out);
      }
    } else if constexpr (OP == OP_RMSNORM) {
      float ss = 0.f;
      for (int64_t r = r0; r < p.R; r += rstep) {
        line_offsets(p, r, xo, yo, wo);
        const float v = load_as_f32(p.x, xb + xo, p.dt_in);
        ss = fmaf(v, v, ss);
      }
      ss = bsum(ss);
      const float inv = 1.0f / sqrtf(ss * invR + p.eps);
      for (int64_t r = r0; r < p.R; r += rstep) {
        line_offsets(p, r, xo, yo, wo);
        float v = load_as_f32(p.x, xb + xo, p.dt_in) * inv;
        if (p.w) v *= load_as_f32(p.w, wo, p.dt_w);
        store_from_f32(p.y, yb + yo, v, p.dt_out);
      }
    } else if constexpr (OP == OP_LPNORM) {
      // yt::function::normalize (reference src/function/normalization.inl:56-85): x / (sum |x|^p + eps)^(1/p)
      float s = 0.f;
      for (int64_t r = r0; r < p.R; r += rstep) {
        line_offsets(p, r, xo, yo, wo);
        s += powf(fabsf(load_as_f32(p.x, xb + xo, p.dt_in)), p.lp);
      }
      s = bsum(s);
      const float den = powf(s + p.eps, 1.0f / p.lp);
      for (int64_t r = r0; r < p.R; r += rstep) {
        line_offsets(p, r, xo, yo, wo);
        store_from_f32(p.y, yb + yo, load_as_f32(p.x, xb + xo, p.dt_in) / den, p.dt_out);
      }
    } else if constexpr (OP == OP_LAYERNORM) {
      float s = 0.f;
      for (int64_t r = r0; r < p.R; r += rstep) {
        line_offsets(p, r, xo, yo, wo);
        s += load_as_f32(p.x, xb + xo, p.dt_in);
      }
      const float mu = bsum(s) * invR;
      float ss = 0.f;
      for (int64_t r = r0; r < p.R; r += rstep) {
        line_offsets(p, r, xo, yo, wo);
        const float c = load_as_f32(p.x, xb + xo, p.dt_in) - mu;
        ss = fmaf(c, c, ss);
      }
      ss = bsum(ss);
      const float inv = 1.0f / sqrtf(ss * invR + p.eps);
      for (int64_t r = r0; r < p.R; r += rstep) {
        line_offsets(p, r, xo, yo, wo);
        float v = (load_as_f32(p.x, xb + xo, p.dt_in) - mu) * inv;
        if (p.w) v = v * load_as_f32(p.w, wo, p.dt_w) + load_as_f32(p.b, wo, p.dt_w);
        store_from_f32(p.y, yb + yo, v, p.dt_out);
      }
    }
  }
}

// ------------------------------------------------------------------ few lines, long reductions
// sum / mean / max over very many elements per output (e.g. a whole-tensor sum) would leave all but a
// few SMs idle with one CTA per line. The reduced range of every line is cut into `chunks` pieces, one
// CTA each; the partial results go to a scratch buffer in global memory and a second small kernel
// combines them. The scratch holds chunks * lines (value, index) pairs.
struct SplitParams {
  LineParams lp;
  int chunks;
  int64_t chunk_len;
  int contiguous;  // the reduced elements of a line are one contiguous run in x
  float* part_val;
  int* part_idx;
};

template <int OP>
__global__ void __launch_bounds__(256) split_partial_kernel(const SplitParams sp) {
  __shared__ float red[32];
  __shared__ int redi[32];
  const LineParams& p = sp.lp;
  const int tid = threadIdx.x;
  const int chunk = blockIdx.x;
  const int64_t line = blockIdx.y;
  int64_t xb = 0, rem = line;
  for (int d = p.nk - 1; d >= 0; --d) {
    const int64_t c = rem % p.kshape[d];
    rem /= p.kshape[d];
    xb += c * p.kxs[d];
  }
  const int64_t r_begin = chunk * sp.chunk_len;
  const int64_t r_end = (r_begin + sp.chunk_len < p.R) ? r_begin + sp.chunk_len : p.R;
  int64_t xo, yo, wo;
  if constexpr (OP == OP_MAX) {
    MaxIdx m = {-CUDART_INF_F, 0x7fffffff};
    for (int64_t r = r_begin + tid; r < r_end; r += 256) {
      if (sp.contiguous) xo = r; else line_offsets(p, r, xo, yo, wo);
      m = max_combine(m, MaxIdx{load_as_f32(p.x, xb + xo, p.dt_in), static_cast<int>(r)});
    }
    m = group_maxidx<256>(m, red, redi, 0, tid);
    if (tid == 0) {
      sp.part_val[line * sp.chunks + chunk] = m.v;
      sp.part_idx[line * sp.chunks + chunk] = m.i;
    }
  } else {
    float s = 0.f;
    for (int64_t r = r_begin + tid; r < r_end; r += 256) {
      if (sp.contiguous) xo = r; else line_offsets(p, r, xo, yo, wo);
      s += load_as_f32(p.x, xb + xo, p.dt_in);
    }
    s = group_sum<256>(s, red, 0, tid);
    if (tid == 0) sp.part_val[line * sp.chunks + chunk] = s;
  }
}

template <int OP>
__global__ void __launch_bounds__(32) split_finish_kernel(const SplitParams sp) {
  const LineParams& p = sp.lp;
  const int lane = threadIdx.x;
  const int64_t line = blockIdx.x;
  if constexpr (OP == OP_MAX) {
    MaxIdx m = {-CUDART_INF_F, 0x7fffffff};
    for (int c = lane; c < sp.chunks; c += 32)
      m = max_combine(m, MaxIdx{sp.part_val[line * sp.chunks + c], sp.part_idx[line * sp.chunks + c]});
    m = group_maxidx<32>(m, nullptr, nullptr, 0, lane);
    if (lane == 0) {
      int64_t xb = 0, rem = line;
      for (int d = p.nk - 1; d >= 0; --d) {
        const int64_t c = rem % p.kshape[d];
        rem /= p.kshape[d];
        xb += c * p.kxs[d];
      }
      if (m.i == 0x7fffffff) {
        m.v = load_as_f32(p.x, xb, p.dt_in);
        m.i = 0;
      }
      store_from_f32(p.y, line, m.v, p.dt_out);
      if (p.idx) p.idx[line] = m.i;
    }
  } else {
    float s = 0.f;
    for (int c = lane; c < sp.chunks; c += 32) s += sp.part_val[line * sp.chunks + c];
    s = group_sum<32>(s, nullptr, 0, lane);
    if (lane == 0) store_from_f32(p.y, line, OP == OP_MEAN ? s / static_cast<float>(p.R) : s, p.dt_out);
  }
}

// ------------------------------------------------------------------ host side
struct NdArgs {
  const int64_t* shape;
  const int64_t* xs;
  const int64_t* ys;
  int ndim;
  const int* axes;
  int naxes;
};

static int normalize_axes(const NdArgs& a, int* ax, bool* used, const char* who) {
  if (a.ndim < 1 || a.ndim > MAXD) {
    set_last_error("%s: ndim %d outside [1, %d]", who, a.ndim, MAXD);
    return YTC_INVALID_ARG;
  }
  if (a.naxes < 1 || a.naxes > a.ndim) {
    set_last_error("%s: %d axes for %d dims", who, a.naxes, a.ndim);
    return YTC_INVALID_ARG;
  }
  for (int d = 0; d < a.ndim; ++d) used[d] = false;
  for (int i = 0; i < a.naxes; ++i) {
    const int v = ((a.axes[i] % a.ndim) + a.ndim) % a.ndim;
    if (used[v]) {
      set_last_error("%s: axis %d listed twice", who, v);
      return YTC_INVALID_ARG;
    }
    used[v] = true;
    ax[i] = v;
  }
  for (int d = 0; d < a.ndim; ++d)
    if (a.shape[d] < 0) {
      set_last_error("%s: negative extent", who);
      return YTC_INVALID_ARG;
    }
  return YTC_OK;
}

template <int OP, int G>
static void launch_row(const RowParams& p, cudaStream_t st) {
  constexpr int THREADS = G < 256 ? 256 : G;
  constexpr int RPC = THREADS / G;
  const int64_t row_blocks = (p.rows + RPC - 1) / RPC;
  const int64_t cap = static_cast<int64_t>(sm_count()) * (2048 / THREADS) * 2;
  const int grid = static_cast<int>(row_blocks < cap ? row_blocks : cap);
  (void)launch_overlapped(row_kernel<OP, G>, dim3(grid), dim3(THREADS), 0, st, p);
  count_launch();
}
template <int OP>
static void launch_row_g(const RowParams& p, cudaStream_t st) {
  if (p.L <= 512) launch_row<OP, 32>(p, st);
  else if (p.L <= 2048) launch_row<OP, 128>(p, st);
  else if (p.L <= 4096) launch_row<OP, 256>(p, st);
  else launch_row<OP, 1024>(p, st);
}
static void launch_row_op(int op, const RowParams& p, cudaStream_t st) {
  switch (op) {
    case OP_SOFTMAX: launch_row_g<OP_SOFTMAX>(p, st); break;
    case OP_RMSNORM: launch_row_g<OP_RMSNORM>(p, st); break;
    case OP_LAYERNORM: launch_row_g<OP_LAYERNORM>(p, st); break;
    case OP_CHAIN: launch_row_g<OP_CHAIN>(p, st); break;
    case OP_SUM: launch_row_g<OP_SUM>(p, st); break;
    case OP_MEAN: launch_row_g<OP_MEAN>(p, st); break;
    default: launch_row_g<OP_MAX>(p, st); break;
  }
}
template <int OP>
static void launch_line(const LineParams& p, bool per_thread, cudaStream_t st) {
  if (per_thread) {
    const int64_t blocks = (p.lines + 127) / 128;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 32;
    line_kernel<OP, true><<<static_cast<int>(blocks < cap ? blocks : cap), 128, 0, st>>>(p);
  } else {
    const int64_t cap = static_cast<int64_t>(sm_count()) * 32;
    line_kernel<OP, false><<<static_cast<int>(p.lines < cap ? p.lines : cap), 128, 0, st>>>(p);
  }
  count_launch();
}
static void launch_line_op(int op, const LineParams& p, bool per_thread, cudaStream_t st) {
  switch (op) {
    case OP_SOFTMAX: launch_line<OP_SOFTMAX>(p, per_thread, st); break;
    case OP_RMSNORM: launch_line<OP_RMSNORM>(p, per_thread, st); break;
    case OP_LAYERNORM: launch_line<OP_LAYERNORM>(p, per_thread, st); break;
    case OP_LPNORM: launch_line<OP_LPNORM>(p, per_thread, st); break;
    case OP_SUM: launch_line<OP_SUM>(p, per_thread, st); break;
    case OP_MEAN: launch_line<OP_MEAN>(p, per_thread, st); break;
    default: launch_line<OP_MAX>(p, per_thread, st); break;
  }
}

// Shared driver of all N-d reductions. `reduce_out` = the output keeps size-1 dims on the reduced axes
// (sum / mean / max) instead of the input's shape (softmax / norms).
static int run_nd(int op, int dt_in, int dt_out, int dt_w, const void* x, void* y, const void* w, const void* b,
                  int* idx, const NdArgs& a, float eps, bool reduce_out, cudaStream_t st, const char* who,
                  void* scratch = nullptr, size_t scratch_bytes = 0, float lp = 2.f) {
  int ax[MAXD];
  bool used[MAXD];
  int s = normalize_axes(a, ax, used, who);
  if (s != YTC_OK) return s;
  YTC_REQUIRE(dt_in >= 0 && dt_in <= 2 && dt_out >= 0 && dt_out <= 2 && dt_w >= 0 && dt_w <= 2, "%s: bad dtype", who);
  int64_t total = 1, R = 1;
  for (int d = 0; d < a.ndim; ++d) total *= a.shape[d];
  for (int i = 0; i < a.naxes; ++i) R *= a.shape[ax[i]];
  if (total == 0) return YTC_OK;
  YTC_REQUIRE(x && y, "%s: null tensor", who);
  YTC_REQUIRE(R <= 0x7fffffffll, "%s: more than 2^31 elements per reduction", who);
  const int64_t lines = total / R;

  // Fast path: the reduced axes are the trailing dims in ascending listed order, contiguous in x (and in y
  // for the shape-preserving ops), rows 16-byte aligned.
  bool trailing = true;
  for (int i = 0; i < a.naxes; ++i)
    if (ax[i] != a.ndim - a.naxes + i) trailing = false;
  if (trailing) {
    int64_t exp = 1;
    for (int d = a.ndim - 1; d >= a.ndim - a.naxes; --d) {
      if (a.shape[d] != 1 && (a.xs[d] != exp || (!reduce_out && a.ys[d] != exp))) trailing = false;
      exp *= a.shape[d];
    }
  }
  // kept dims must collapse into one row stride
  int64_t x_rs = R, y_rs = reduce_out ? 1 : R;
  if (trailing) {
    int64_t expx = -1, expy = -1;
    for (int d = a.ndim - a.naxes - 1; d >= 0; --d) {
      if (a.shape[d] == 1) continue;
      if (expx < 0) {
        expx = a.xs[d];
        expy = a.ys[d];
        x_rs = a.xs[d];
        y_rs = a.ys[d];
      } else if (a.xs[d] != expx || a.ys[d] != expy) {
        trailing = false;
        break;
      }
      expx *= a.shape[d];
      expy *= a.shape[d];
    }
    if (reduce_out && lines > 1 && y_rs != 1) trailing = false;
  }
  const int esz_in = dtype_size(dt_in), esz_out = dtype_size(dt_out);
  if (op != OP_LPNORM && trailing && R % 4 == 0 && R <= 16384 && x_rs >= 0 && y_rs >= 0 &&
      (reinterpret_cast<uint64_t>(x) % (4 * esz_in)) == 0 && (x_rs * esz_in) % (4 * esz_in) == 0 &&
      (reduce_out || ((reinterpret_cast<uint64_t>(y) % (4 * esz_out)) == 0 && (y_rs * esz_out) % (4 * esz_out) == 0)) &&
      (!w || reinterpret_cast<uint64_t>(w) % (4 * dtype_size(dt_w)) == 0) &&
      (!b || reinterpret_cast<uint64_t>(b) % (4 * dtype_size(dt_w)) == 0)) {
    RowParams p;
    p.x = x; p.y = y; p.w = w; p.b = b; p.idx = idx;
    p.rows = lines; p.L = static_cast<int>(R);
    p.x_rs = x_rs; p.y_rs = y_rs; p.r_rows = 1; p.eps = eps;
    p.dt_in = dt_in; p.dt_out = dt_out; p.dt_w = dt_w;
    launch_row_op(op, p, st);
    YTC_CUDA(cudaGetLastError());
    return YTC_OK;
  }

  LineParams p;
  p.x = x; p.y = y; p.w = w; p.b = b; p.idx = idx;
  p.nk = 0; p.nr = a.naxes;
  p.eps = eps; p.lp = lp; p.dt_in = dt_in; p.dt_out = dt_out; p.dt_w = dt_w;
  p.lines = lines; p.R = R;
  for (int d = 0; d < a.ndim; ++d)
    if (!used[d]) {
      p.kshape[p.nk] = a.shape[d];
      p.kxs[p.nk] = a.xs[d];
      p.kys[p.nk] = a.ys[d];
      ++p.nk;
    }
  // weight layout: contiguous over the reduced dims in ASCENDING axis order (the reference views the
  // weight's memory with shape [1,..,size(axis),..,1], src/ytensor_function.inl:137-158)
  int64_t wstride[MAXD];
  {
    int64_t acc = 1;
    for (int d = a.ndim - 1; d >= 0; --d)
      if (used[d]) {
        wstride[d] = acc;
        acc *= a.shape[d];
      }
  }
  for (int i = 0; i < a.naxes; ++i) {
    p.rshape[i] = a.shape[ax[i]];
    p.rxs[i] = a.xs[ax[i]];
    p.rys[i] = reduce_out ? 0 : a.ys[ax[i]];
    p.rws[i] = wstride[ax[i]];
  }
  // few outputs, long reductions: split every line over several CTAs through a scratch buffer
  if (reduce_out && lines <= 2 * sm_count() && R >= 32768) {
    SplitParams sp;
    sp.lp = p;
    int64_t chunks = (4ll * sm_count() + lines - 1) / lines;
    const int64_t max_chunks = (R + 2047) / 2048;
    if (chunks > max_chunks) chunks = max_chunks;
    if (chunks > 4096) chunks = 4096;
    sp.chunks = static_cast<int>(chunks);
    sp.chunk_len = (R + chunks - 1) / chunks;
    bool contig = true;
    {
      int64_t exp = 1;
      for (int i = a.naxes - 1; i >= 0; --i) {
        if (p.rshape[i] != 1 && p.rxs[i] != exp) contig = false;
        exp *= p.rshape[i];
      }
    }
    sp.contiguous = contig ? 1 : 0;
    const size_t need = static_cast<size_t>(lines) * chunks;
    void* ws = scratch ? scratch : device_workspace(need * 8, st);
    if (!ws) {
      set_last_error("%s: cannot allocate %zu bytes of scratch", who, need * 8);
      return YTC_CUDA_ERROR;
    }
    if (scratch && need * 8 > scratch_bytes) {
      set_last_error("%s: needs %zu bytes of scratch, the fixed buffer holds %zu", who, need * 8, scratch_bytes);
      return YTC_INVALID_ARG;
    }
    sp.part_val = static_cast<float*>(ws);
    sp.part_idx = reinterpret_cast<int*>(sp.part_val + need);
    dim3 grid(static_cast<unsigned>(chunks), static_cast<unsigned>(lines));
    if (op == OP_SUM) {
      split_partial_kernel<OP_SUM><<<grid, 256, 0, st>>>(sp);
      split_finish_kernel<OP_SUM><<<static_cast<unsigned>(lines), 32, 0, st>>>(sp);
    } else if (op == OP_MEAN) {
      split_partial_kernel<OP_MEAN><<<grid, 256, 0, st>>>(sp);
      split_finish_kernel<OP_MEAN><<<static_cast<unsigned>(lines), 32, 0, st>>>(sp);
    } else {
      split_partial_kernel<OP_MAX><<<grid, 256, 0, st>>>(sp);
      split_finish_kernel<OP_MAX><<<static_cast<unsigned>(lines), 32, 0, st>>>(sp);
    }
    count_launch(2);
    YTC_CUDA(cudaGetLastError());
    return YTC_OK;
  }
  // one thread per line when neighbouring lines sit next to each other in memory
  const bool per_thread = p.nk > 0 && p.kxs[p.nk - 1] == 1 && p.kshape[p.nk - 1] >= 32 && lines >= 4096;
  launch_line_op(op, p, per_thread, st);
  YTC_CUDA(cudaGetLastError());
  return YTC_OK;
}

// ------------------------------------------------------------------ fixed scratch for callers that cannot allocate
// Partial results of the split reduction for ytcuda_reduce_noalloc live here instead of in a cudaMalloc'ed
// workspace: 8192 (value, index) pairs. Every GPU that loads the library carries these 64 KiB until exit.
constexpr size_t NOALLOC_SCRATCH_BYTES = 64 * 1024;
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_SCRATCH_BYTES];
// Bytes of the array a call may use (ytcuda_reduce_noalloc_set_limit); never more than the array holds.
static std::atomic<size_t> g_noalloc_limit{NOALLOC_SCRATCH_BYTES};

// The array's name is only a host-side handle here: the device address has to be asked for, once per device,
// while that device is current.
static void* noalloc_scratch_address() {
  static void* addr[16] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) {
    set_last_error("ytcuda_reduce_noalloc: cannot identify the current device");
    return nullptr;
  }
  std::lock_guard<std::mutex> lk(mu);
  if (!addr[dev]) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || !p) {
      set_last_error("ytcuda_reduce_noalloc: cudaGetSymbolAddress failed with %d (%s)", static_cast<int>(e),
                     cudaGetErrorString(e));
      return nullptr;
    }
    addr[dev] = p;
  }
  return addr[dev];
}

}  // namespace ytk

using namespace ytk;

extern "C" {

int ytcuda_reduce_noalloc(int op, int dt_in, int dt_out, const void* x, void* y, int32_t* index, const int64_t* shape,
                          const int64_t* xstrides, int ndim, const int* axes, int naxes, void* stream) {
  YTC_REQUIRE(op >= 0 && op <= 2, "ytcuda_reduce_noalloc: op must be 0 (sum), 1 (mean) or 2 (max)");
  YTC_REQUIRE(shape && xstrides && axes, "ytcuda_reduce_noalloc: null shape/strides/axes");
  YTC_REQUIRE(ndim >= 1 && ndim <= MAXD, "ytcuda_reduce_noalloc: ndim %d outside [1, %d]", ndim, MAXD);
  void* scratch = noalloc_scratch_address();
  if (!scratch) return YTC_CUDA_ERROR;
  int64_t ys[MAXD];
  {
    bool red[MAXD] = {false};
    for (int i = 0; i < naxes && i < MAXD; ++i) red[((axes[i] % ndim) + ndim) % ndim] = true;
    int64_t acc = 1;
    for (int d = ndim - 1; d >= 0; --d) {
      ys[d] = red[d] ? 0 : acc;
      if (!red[d]) acc *= shape[d];
    }
  }
  NdArgs a{shape, xstrides, ys, ndim, axes, naxes};
  const int rop = op == 0 ? OP_SUM : op == 1 ? OP_MEAN : OP_MAX;
  return run_nd(rop, dt_in, dt_out, YTC_F32, x, y, nullptr, nullptr, index, a, 0.f, true,
                static_cast<cudaStream_t>(stream), "ytcuda_reduce_noalloc", scratch, g_noalloc_limit.load());
}

int ytcuda_reduce_noalloc_set_limit(uint64_t bytes) {
  YTC_REQUIRE(bytes <= NOALLOC_SCRATCH_BYTES, "ytcuda_reduce_noalloc_set_limit: %llu bytes asked for, the array holds %zu",
              static_cast<unsigned long long>(bytes), NOALLOC_SCRATCH_BYTES);
  g_noalloc_limit.store(bytes == 0 ? NOALLOC_SCRATCH_BYTES : static_cast<size_t>(bytes));
  return YTC_OK;
}

int ytcuda_softmax(int dt_in, int dt_out, const void* x, void* y, const int64_t* shape, const int64_t* xstrides,
                   const int64_t* ystrides, int ndim, const int* axes, int naxes, void* stream) {
  YTC_REQUIRE(shape && xstrides && ystrides && axes, "ytcuda_softmax: null shape/strides/axes");
  NdArgs a{shape, xstrides, ystrides, ndim, axes, naxes};
  return run_nd(OP_SOFTMAX, dt_in, dt_out, YTC_F32, x, y, nullptr, nullptr, nullptr, a, 0.f, false,
                static_cast<cudaStream_t>(stream), "ytcuda_softmax");
}

int ytcuda_normalize(int dt_in, int dt_out, const void* x, void* y, const int64_t* shape, const int64_t* xstrides,
                     const int64_t* ystrides, int ndim, const int* axes, int naxes, float p, float eps, void* stream) {
  YTC_REQUIRE(shape && xstrides && ystrides && axes, "ytcuda_normalize: null shape/strides/axes");
  YTC_REQUIRE(p > 0.f, "yt::function::normalize: p must be positive");
  NdArgs a{shape, xstrides, ystrides, ndim, axes, naxes};
  return run_nd(OP_LPNORM, dt_in, dt_out, YTC_F32, x, y, nullptr, nullptr, nullptr, a, eps, false,
                static_cast<cudaStream_t>(stream), "ytcuda_normalize", nullptr, 0, p);
}

int ytcuda_rmsnorm(int dt_in, int dt_out, int dt_w, const void* x, const void* weight, void* y, const int64_t* shape,
                   const int64_t* xstrides, const int64_t* ystrides, int ndim, const int* axes, int naxes, float eps,
                   void* stream) {
  YTC_REQUIRE(shape && xstrides && ystrides && axes, "ytcuda_rmsnorm: null shape/strides/axes");
  NdArgs a{shape, xstrides, ystrides, ndim, axes, naxes};
  return run_nd(OP_RMSNORM, dt_in, dt_out, dt_w, x, y, weight, nullptr, nullptr, a, eps, false,
                static_cast<cudaStream_t>(stream), "ytcuda_rmsnorm");
}

int ytcuda_layernorm(int dt_in, int dt_out, int dt_w, const void* x, const void* gamma, const void* beta, void* y,
                     const int64_t* shape, const int64_t* xstrides, const int64_t* ystrides, int ndim, const int* axes,
                     int naxes, float eps, void* stream) {
  YTC_REQUIRE(shape && xstrides && ystrides && axes, "ytcuda_layernorm: null shape/strides/axes");
  YTC_REQUIRE((gamma == nullptr) == (beta == nullptr), "ytcuda_layernorm: gamma and beta come together");
  NdArgs a{shape, xstrides, ystrides, ndim, axes, naxes};
  return run_nd(OP_LAYERNORM, dt_in, dt_out, dt_w, x, y, gamma, beta, nullptr, a, eps, false,
                static_cast<cudaStream_t>(stream), "ytcuda_layernorm");
}

int ytcuda_reduce(int op, int dt_in, int dt_out, const void* x, void* y, int32_t* index, const int64_t* shape,
                  const int64_t* xstrides, int ndim, const int* axes, int naxes, void* stream) {
  YTC_REQUIRE(op >= 0 && op <= 2, "ytcuda_reduce: op must be 0 (sum), 1 (mean) or 2 (max)");
  YTC_REQUIRE(shape && xstrides && axes, "ytcuda_reduce: null shape/strides/axes");
  YTC_REQUIRE(ndim >= 1 && ndim <= MAXD, "ytcuda_reduce: ndim %d outside [1, %d]", ndim, MAXD);
  // the output is contiguous with size-1 dims on the reduced axes
  int64_t ys[MAXD];
  {
    bool red[MAXD] = {false};
    for (int i = 0; i < naxes && i < MAXD; ++i) red[((axes[i] % ndim) + ndim) % ndim] = true;
    int64_t acc = 1;
    for (int d = ndim - 1; d >= 0; --d) {
      ys[d] = red[d] ? 0 : acc;
      if (!red[d]) acc *= shape[d];
    }
  }
  NdArgs a{shape, xstrides, ys, ndim, axes, naxes};
  const int rop = op == 0 ? OP_SUM : op == 1 ? OP_MEAN : OP_MAX;
  return run_nd(rop, dt_in, dt_out, YTC_F32, x, y, nullptr, nullptr, index, a, 0.f, true,
                static_cast<cudaStream_t>(stream), "ytcuda_reduce");
}

int ytcuda_rmsnorm_add_softmax_cast(int dt_out, const float* x, const float* weight, const float* residual, void* out,
                                    int64_t batch, int64_t rows, int hidden, int residual_batched, float eps,
                                    void* stream) {
  YTC_REQUIRE(dt_out >= 0 && dt_out <= 2, "ytcuda_rmsnorm_add_softmax_cast: bad dt_out");
  YTC_REQUIRE(batch >= 0 && rows >= 0 && hidden >= 0, "ytcuda_rmsnorm_add_softmax_cast: negative extent");
  if (batch == 0 || rows == 0 || hidden == 0) return YTC_OK;
  YTC_REQUIRE(x && weight && residual && out, "ytcuda_rmsnorm_add_softmax_cast: null tensor");
  if (hidden % 4 != 0 || hidden > 16384 || (reinterpret_cast<uint64_t>(x) & 15) || (reinterpret_cast<uint64_t>(weight) & 15) ||
      (reinterpret_cast<uint64_t>(residual) & 15) || (reinterpret_cast<uint64_t>(out) & 7)) {
    set_last_error("ytcuda_rmsnorm_add_softmax_cast: hidden must be a multiple of 4, at most 16384, tensors 16-byte aligned");
    return YTC_UNSUPPORTED;
  }
  RowParams p;
  p.x = x; p.y = out; p.w = weight; p.b = residual; p.idx = nullptr;
  p.rows = batch * rows; p.L = hidden;
  p.x_rs = hidden; p.y_rs = hidden;
  p.r_rows = residual_batched ? batch * rows : rows;
  p.eps = eps; p.dt_in = YTC_F32; p.dt_out = dt_out; p.dt_w = YTC_F32;
  if (dt_out == YTC_BF16 && (hidden == 1024 || hidden == 2048 || hidden == 4096)) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t cap = static_cast<int64_t>(sm_count()) * 4 * 4;
    const unsigned grid = static_cast<unsigned>(p.rows < cap ? p.rows : cap);
    uint2* o2 = static_cast<uint2*>(out);
    if (hidden == 4096) chain_fast_kernel<4><<<grid, 256, 0, st>>>(x, weight, residual, o2, p.rows, p.r_rows, eps);
    else if (hidden == 2048) chain_fast_kernel<2><<<grid, 256, 0, st>>>(x, weight, residual, o2, p.rows, p.r_rows, eps);
    else chain_fast_kernel<1><<<grid, 256, 0, st>>>(x, weight, residual, o2, p.rows, p.r_rows, eps);
    count_launch();
    YTC_CUDA(cudaGetLastError());
    return YTC_OK;
  }
  launch_row_op(OP_CHAIN, p, static_cast<cudaStream_t>(stream));
  YTC_CUDA(cudaGetLastError());
  return YTC_OK;
}

}  // extern "C"
