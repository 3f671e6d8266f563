// One decode step (one new token per sequence) of the Qwen3-shape decoder as ONE persistent cooperative kernel.
//
// The operator-per-launch forward needs about 340 launches of kernels that each move a few MB; at batch 1 the step
// is then bound by launch and ramp latency, not by the 1.2 GB of weights it has to stream. Here one CTA per SM stays
// resident for the whole step and walks the same operator sequence (reference example/qwen3/src/qwen3.cpp:237-283,
// 365-457) as phases separated by a grid-wide barrier:
//
//   embedding | per layer: [rmsNorm -> qkv linear] | [per-head rmsNorm + RoPE + KV append + attention over the
//   cache, split over key chunks, last chunk merges] | [o projection + residual] | [rmsNorm -> gate/up linear ->
//   swish(gate) * up] | [down projection + residual] | final rmsNorm -> vocabulary projection
//
// In a linear phase every warp of the grid owns whole weight rows (bf16, streamed once with 128-bit loads) and the
// few activation rows sit in shared memory as fp32, so the arithmetic (fp32 FMA chains along k, lane partials
// combined by shuffles) is the same as in skinny_linear_kernel. A warp requests its first weights BEFORE the
// activations are staged (the weights do not depend on them), and at the start of every phase it asks the L2 to fetch
// the rows it will own in the next phase, so HBM keeps streaming across the barriers. Activations that cross a
// barrier are read with ld.global.cg: another SM wrote them, so this SM's L1 may not be used.
//
// Attention: a unit is (sequence, kv head, chunk of 128 keys or more) and belongs to one CTA; a warp takes 32 keys at
// a time with coalesced row loads: 8 lanes share a key for the dot products with the query heads of the group, the
// warp takes maximum and sum once per 32 keys, and P.V runs with the value dimension across lanes and the
// probabilities broadcast by shuffles. The 16 warps combine through shared memory and leave one partial (m, l, o)
// per chunk and head in global memory; the o-projection phase combines the chunks while it stages its input. The
// K / V rows of a unit are requested from HBM into the L2 one phase earlier.
//
// Tensor parallelism: every rank runs this kernel on its share of the heads, FFN columns and vocabulary rows. The
// partial sums of the o and down projections are all-reduced inside the kernel: each rank writes its partial vector
// into a mailbox in its own memory, a barrier over the local CTAs and the peers (flag words written with system-scope
// release stores over NVLink) follows, and then every rank adds the mailboxes of all ranks in rank order.
//
// The barrier is a counter in global memory (one arrival per CTA, acquire loads while waiting). The launch is
// cooperative, so all CTAs are resident; the wait is still bounded: when the cycle budget runs out the CTA raises
// the device status word and every CTA leaves at its next barrier.
#pragma once

#include <math_constants.h>

#include "ytc_common.cuh"

namespace ytk {

constexpr int DS_THREADS = 256;
constexpr int DS_WARPS = DS_THREADS / 32;
constexpr int DS_MAX_B = 32;       // sequences per step (activation rows kept in shared memory)
constexpr int DS_MAX_G = 4;        // query heads per kv head
constexpr int DS_MAX_TP = 8;       // tensor-parallel ranks (one GPU each, peers reached by NVLink loads / stores)
// attention scratch of a CTA: q of the group, and per warp (m, l, o[128]) for every head of the group
constexpr int DS_ATT_FLOATS = DS_MAX_G * 128 + 2 * DS_WARPS * DS_MAX_G + DS_WARPS * DS_MAX_G * 128;  // for G = DS_MAX_G

struct DsLayer {
  const uint16_t *qkv, *o, *gate_up, *down;
  const float *q_norm, *k_norm, *norm1, *norm2;
};

struct DecodeStepParams {
  int B, hidden, layers, heads, kv_heads, inter, vocab_rows, vocab, max_pos;
  // pos: cache slot the token of this step is written to; rope_pos: its rotary position; n_keys: keys it attends
  // to, the new one included (pos + 1, or the whole cache once the ring buffer has wrapped: reference
  // example/qwen3/src/qwen3.cpp:70-126, 365-375)
  int pos, rope_pos, n_keys;
  float eps, scale;
  const int32_t* ids;
  const uint16_t* embed;
  const uint16_t* lm_head;
  const float* final_norm;
  const DsLayer* lw;  // device array [layers]
  const float *cos_t, *sin_t;
  float *k_cache, *v_cache;
  size_t cache_layer;  // elements per layer
  float *x, *qkv, *attn, *act, *logits, *part;
  unsigned int* sync;  // grid barrier counter
  int chunks, keys_per_chunk;
  int xs_cols;  // activation columns that fit shared memory at once (a multiple of 256, at most 3072)
  int mma;      // 1: the linear phases run on the tensor cores (ds_linear_mma), 0: FFMA (ds_linear_phase)
  int* status;
  // Tensor parallelism (tp_world > 1): heads, kv_heads, inter and vocab_rows above are this rank's share. The partial
  // sums of the o and down projections are exchanged through "mailboxes" in peer-visible device memory:
  //   mail[r]   rank r's mailbox, two slots of [DS_MAX_B][hidden] floats (slot = exchange number & 1)
  //   flags[r]  rank r's arrival words: flags[r][q] = number of the last exchange rank q has finished writing
  //   go        this rank's release word for its own CTAs
  int tp_rank, tp_world;
  float* mail[DS_MAX_TP];
  unsigned int* flags[DS_MAX_TP];
  unsigned int* go;
  unsigned int ar_base;  // exchanges completed before this launch
  long long wait_cycles;  // budget of every bounded wait (ytcuda_set_wait_limit)
  int dw_xs_bytes, dw_nslot;  // decode_stream_kernel: bytes of its activation area, slots of its weight ring
  // Optional timeline (ytcuda_qwen3_set_trace): the first and the last CTA write their SM's cycle counter into
  // trace[cta ? trace_cap : 0 + 4 * barrier + k], k = 0 on arriving at grid barrier number `barrier`, 1 on leaving it,
  // 2 once the following linear phase has staged its activations.
  long long* trace;
  int trace_cap;
  // decode_ll_kernel: activations and attention partial results exchanged as {bits, tag} pairs, and the tag base of
  // this launch
  uint2 *ll_x, *ll_qkv, *ll_att, *ll_act, *ll_part;
  unsigned int ll_base;
  // decode_ll_kernel under tensor parallelism: ll_mail[q] is rank q's pair area [source rank][2][4][hidden] (own
  // memory or the peer's): a rank PUSHES its partial sums of the o and down projections as pairs into slot
  // [its rank] of every peer's area and polls its own area for the peers' pairs
  uint2* ll_mail[DS_MAX_TP];
};

__device__ __forceinline__ float ds_ldcg(const float* p) { return __ldcg(p); }
__device__ __forceinline__ float4 ds_ldcg4(const float* p) { return __ldcg(reinterpret_cast<const float4*>(p)); }

__device__ __forceinline__ void ds_trace(const DecodeStepParams& p, unsigned int barrier, int k) {
  if (p.trace && threadIdx.x == 0 && (blockIdx.x == 0 || blockIdx.x + 1 == gridDim.x)) {
    const int idx = 4 * static_cast<int>(barrier) + k;
    if (idx < p.trace_cap) p.trace[(blockIdx.x ? p.trace_cap : 0) + idx] = clock64();
  }
}

// Grid-wide barrier; false when the wait gave up (the caller returns).
__device__ __forceinline__ bool ds_grid_sync(const DecodeStepParams& p, unsigned int& epoch) {
  __syncthreads();
  int ok = 1;
  if (threadIdx.x == 0) {
    ds_trace(p, epoch / gridDim.x, 0);
    epoch += gridDim.x;
    // release: the CTA's writes (ordered before this by the barrier above) are visible to whoever reads the count
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.sync) : "memory");
    const long long t0 = clock64();
    unsigned int v;
    while (true) {
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p.sync) : "memory");
      if (v >= epoch) break;  // also true once any CTA has set the give-up bit
      if (clock64() - t0 > p.wait_cycles) {
        atomicExch(p.status, YTC_TIMEOUT);
        atomicOr(p.sync, 0x80000000u);  // releases every waiting CTA at once
        v = 0x80000000u;
        break;
      }
    }
    if (v & 0x80000000u) ok = 0;
    ds_trace(p, epoch / gridDim.x - 1, 1);
  }
  return __syncthreads_and(ok) != 0;
}

// Grid-wide barrier that also waits for every tensor-parallel peer: exchange number `seq` is complete on all ranks
// (their mailbox writes are visible) when it returns true. CTA 0 collects the local arrivals, tells every peer by a
// system-scope release store into the peer's flag words, waits for the peers' words in its own memory, and then
// releases the other CTAs of this GPU through `go`. All waits are bounded.
__device__ __forceinline__ bool ds_cross_sync(const DecodeStepParams& p, unsigned int& epoch, unsigned int seq) {
  __syncthreads();
  int ok = 1;
  if (threadIdx.x == 0) {
    epoch += gridDim.x;
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.sync) : "memory");
    const long long t0 = clock64();
    unsigned int v;
    if (blockIdx.x == 0) {
      while (true) {  // every CTA of this GPU has written its part of the mailbox
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p.sync) : "memory");
        if (v >= epoch) break;
        if (clock64() - t0 > p.wait_cycles) {
          v = 0x80000000u;
          break;
        }
      }
      if (!(v & 0x80000000u)) {
        __threadfence_system();
        for (int q = 0; q < p.tp_world; ++q)
          if (q != p.tp_rank)
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.flags[q] + p.tp_rank), "r"(seq) : "memory");
        for (int q = 0; q < p.tp_world && !(v & 0x80000000u); ++q) {
          if (q == p.tp_rank) continue;
          while (true) {
            unsigned int f;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(f) : "l"(p.flags[p.tp_rank] + q) : "memory");
            if (f >= seq) break;
            if (clock64() - t0 > p.wait_cycles) {
              v = 0x80000000u;
              break;
            }
          }
        }
      }
      if (v & 0x80000000u) {
        atomicExch(p.status, YTC_TIMEOUT);
        atomicOr(p.sync, 0x80000000u);
        ok = 0;
      } else {
        asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.go), "r"(seq) : "memory");
      }
    } else {
      while (true) {
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p.go) : "memory");
        if (v >= seq) break;
        unsigned int c;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(c) : "l"(p.sync) : "memory");
        if ((c & 0x80000000u) || clock64() - t0 > p.wait_cycles) {
          atomicExch(p.status, YTC_TIMEOUT);
          atomicOr(p.sync, 0x80000000u);
          ok = 0;
          break;
        }
      }
    }
  }
  return __syncthreads_and(ok) != 0;
}

// x[b][:] += sum over ranks of the partial sums in slot `slot` of every rank's mailbox, in rank order (every rank
// forms bitwise the same sum); the elements are spread over the threads of the grid.
__device__ __forceinline__ void ds_reduce_mailboxes(const DecodeStepParams& p, int slot) {
  const int n = p.B * p.hidden;
  const int64_t off = static_cast<int64_t>(slot) * DS_MAX_B * p.hidden;
  for (int e = blockIdx.x * DS_THREADS + threadIdx.x; e < n; e += gridDim.x * DS_THREADS) {
    float s = ds_ldcg(p.x + e);
    for (int r = 0; r < p.tp_world; ++r) {
      float v;
      asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p.mail[r] + off + e) : "memory");
      s += v;
    }
    p.x[e] = s;
  }
}

// Asks the L2 for the rows n = gw, gw + GW, ... < N of W (K bf16 each); nothing is held in registers.
__device__ __forceinline__ void ds_prefetch_rows(const uint16_t* W, int N, int K, int gw, int GW, int lane) {
  const int lines = (K * 2 + 127) / 128;
  for (int n = gw; n < N; n += GW) {
    const char* row = reinterpret_cast<const char*>(W + static_cast<int64_t>(n) * K);
    for (int i = lane; i < lines; i += 32) asm volatile("prefetch.global.L2 [%0];" ::"l"(row + i * 128));
  }
}

// 8 bf16 weights (one 128-bit load) times 8 activations, added to s.
__device__ __forceinline__ float ds_dot8(const uint4& w, const float4& xa, const float4& xb, float s) {
  s = fmaf(xa.x, __uint_as_float(w.x << 16), s);
  s = fmaf(xa.y, __uint_as_float(w.x & 0xFFFF0000u), s);
  s = fmaf(xa.z, __uint_as_float(w.y << 16), s);
  s = fmaf(xa.w, __uint_as_float(w.y & 0xFFFF0000u), s);
  s = fmaf(xb.x, __uint_as_float(w.z << 16), s);
  s = fmaf(xb.y, __uint_as_float(w.z & 0xFFFF0000u), s);
  s = fmaf(xb.z, __uint_as_float(w.w << 16), s);
  s = fmaf(xb.w, __uint_as_float(w.w & 0xFFFF0000u), s);
  return s;
}

// xs[b][:] = rmsNorm(src[b][:]) * w for b < B (src in global memory, read around L1). One warp per row takes the
// sum of squares with all its loads in flight at once; meanwhile every thread has requested its piece of w, so the
// whole staging costs about one trip to the L2.
// TWO: a warp takes two rows at a time (worth it with more than 8 sequences, at the cost of 32 more registers).
template <bool TWO = false>
__device__ __forceinline__ void ds_stage_rmsnorm(float* xs, int xs_ld, const float* src, const float* w, int B, int H,
                                                 float eps, int warp, int lane) {
  __shared__ float row_inv[DS_MAX_B];
  const int n4 = H / 4;
  float4 wreg[2];  // this thread's columns of w: float4 index threadIdx.x and threadIdx.x + DS_THREADS (H <= 4096)
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int c4 = threadIdx.x + i * DS_THREADS;
    wreg[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c4 < n4) wreg[i] = __ldg(reinterpret_cast<const float4*>(w) + c4);
  }
  for (int b0 = warp; b0 < B; b0 += (TWO ? 2 : 1) * DS_WARPS) {
    const int b1 = b0 + DS_WARPS;
    const bool two = TWO && b1 < B;
    float ss0 = 0.f, ss1 = 0.f;
    for (int c0 = 0; c0 < H; c0 += 1024) {
      float4 v0[8], v1[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int c = c0 + i * 128 + lane * 4;
        v0[i] = v1[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < H) v0[i] = ds_ldcg4(src + static_cast<int64_t>(b0) * H + c);
        if (two && c < H) v1[i] = ds_ldcg4(src + static_cast<int64_t>(b1) * H + c);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int c = c0 + i * 128 + lane * 4;
        if (c < H) *reinterpret_cast<float4*>(&xs[b0 * xs_ld + c]) = v0[i];
        if (two && c < H) *reinterpret_cast<float4*>(&xs[b1 * xs_ld + c]) = v1[i];
        ss0 = fmaf(v0[i].x, v0[i].x, ss0);
        ss0 = fmaf(v0[i].y, v0[i].y, ss0);
        ss0 = fmaf(v0[i].z, v0[i].z, ss0);
        ss0 = fmaf(v0[i].w, v0[i].w, ss0);
        ss1 = fmaf(v1[i].x, v1[i].x, ss1);
        ss1 = fmaf(v1[i].y, v1[i].y, ss1);
        ss1 = fmaf(v1[i].z, v1[i].z, ss1);
        ss1 = fmaf(v1[i].w, v1[i].w, ss1);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ss0 += __shfl_xor_sync(0xffffffffu, ss0, o);
      ss1 += __shfl_xor_sync(0xffffffffu, ss1, o);
    }
    if (lane == 0) {
      row_inv[b0] = 1.0f / sqrtf(ss0 * (1.0f / static_cast<float>(H)) + eps);
      if (two) row_inv[b1] = 1.0f / sqrtf(ss1 * (1.0f / static_cast<float>(H)) + eps);
    }
  }
  __syncthreads();
  for (int b = 0; b < B; ++b) {
    const float inv = row_inv[b];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int c4 = threadIdx.x + i * DS_THREADS;
      if (c4 < n4) {
        float4 v = *reinterpret_cast<float4*>(&xs[b * xs_ld + c4 * 4]);
        v.x = v.x * inv * wreg[i].x;
        v.y = v.y * inv * wreg[i].y;
        v.z = v.z * inv * wreg[i].z;
        v.w = v.w * inv * wreg[i].w;
        *reinterpret_cast<float4*>(&xs[b * xs_ld + c4 * 4]) = v;
      }
    }
    for (int c4 = threadIdx.x + 2 * DS_THREADS; c4 < n4; c4 += DS_THREADS) {  // hidden sizes above 4096
      float4 v = *reinterpret_cast<float4*>(&xs[b * xs_ld + c4 * 4]);
      const float4 g = __ldg(reinterpret_cast<const float4*>(w) + c4);
      v.x = v.x * inv * g.x;
      v.y = v.y * inv * g.y;
      v.z = v.z * inv * g.z;
      v.w = v.w * inv * g.w;
      *reinterpret_cast<float4*>(&xs[b * xs_ld + c4 * 4]) = v;
    }
  }
  __syncthreads();
}

// xs[b][0 .. kc) = src[b][c0 .. c0 + kc) for b < B (src rows of K floats); U 128-bit loads per thread in flight
template <int U = 4>
__device__ __forceinline__ void ds_stage_copy(float* xs, int xs_ld, const float* src, int B, int K, int c0, int kc) {
  const int per_row = kc / 4;
  const int n4 = B * per_row;
  for (int i0 = threadIdx.x; i0 < n4; i0 += U * DS_THREADS) {
    float4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = i0 + u * DS_THREADS;
      if (i < n4) {
        const int b = i / per_row, c = (i - b * per_row) * 4;
        v[u] = ds_ldcg4(src + static_cast<int64_t>(b) * K + c0 + c);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = i0 + u * DS_THREADS;
      if (i < n4) {
        const int b = i / per_row, c = (i - b * per_row) * 4;
        *reinterpret_cast<float4*>(&xs[b * xs_ld + c]) = v[u];
      }
    }
  }
  __syncthreads();
}

// xs[b][head * 128 + d] = attention output, combined from the per-chunk partials (m, l, o[128]) the attention phase
// left in global memory: o = sum_c e^(m_c - m) o_c / sum_c e^(m_c - m) l_c. Every CTA combines for itself while it
// stages, so the chunks need no finishing step of their own.
// Columns c0 .. c0 + kc (whole heads) of the rows go to xs[b][0 .. kc).
// U outputs (128-bit pieces of a head's output row) per thread at a time, CS chunks of each requested together.
template <int U, int CS>
__device__ __forceinline__ void ds_stage_attention_t(float* xs, int xs_ld, const float* part, int B, int heads,
                                                     int kv_heads, int chunks, int c0, int kc) {
  constexpr int D = 128;
  const int G = heads / kv_heads;
  const int per_row = kc / 4;
  const int total = B * per_row;
  const int64_t cs = static_cast<int64_t>(G) * (4 + D);  // chunk stride
  for (int i0 = threadIdx.x; i0 < total; i0 += U * DS_THREADS) {
    const float* base[U];
    int d4[U];
    float m[U], lsum[U];
    float4 o[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = i0 + u * DS_THREADS;
      const int ii = i < total ? i : 0;
      const int b = ii / per_row, r = ii - b * per_row;
      const int head = c0 / D + r / (D / 4);
      d4[u] = r % (D / 4);
      const int kvh = head / G, g = head - kvh * G;
      base[u] = part + ((static_cast<int64_t>(b) * kv_heads + kvh) * chunks * G + g) * (4 + D);
      m[u] = -CUDART_INF_F;
      lsum[u] = 0.f;
      o[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    // the running combination is an online softmax over the chunks
    for (int cb = 0; cb < chunks; cb += CS) {
      float mc[U][CS], lc[U][CS];
      float4 oc[U][CS];
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int c = 0; c < CS; ++c) {
          mc[u][c] = -CUDART_INF_F;
          lc[u][c] = 0.f;
          oc[u][c] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (cb + c < chunks && i0 + u * DS_THREADS < total) {
            mc[u][c] = ds_ldcg(base[u] + (cb + c) * cs);
            lc[u][c] = ds_ldcg(base[u] + (cb + c) * cs + 1);
            oc[u][c] = ds_ldcg4(base[u] + (cb + c) * cs + 4 + d4[u] * 4);
          }
        }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        float m_new = m[u];
#pragma unroll
        for (int c = 0; c < CS; ++c) m_new = fmaxf(m_new, mc[u][c]);
        const float alpha = (m[u] == -CUDART_INF_F) ? 0.f : __expf(m[u] - m_new);
        lsum[u] *= alpha;
        o[u].x *= alpha;
        o[u].y *= alpha;
        o[u].z *= alpha;
        o[u].w *= alpha;
#pragma unroll
        for (int c = 0; c < CS; ++c) {
          const float f = (mc[u][c] == -CUDART_INF_F) ? 0.f : __expf(mc[u][c] - m_new);
          lsum[u] = fmaf(lc[u][c], f, lsum[u]);
          o[u].x = fmaf(oc[u][c].x, f, o[u].x);
          o[u].y = fmaf(oc[u][c].y, f, o[u].y);
          o[u].z = fmaf(oc[u][c].z, f, o[u].z);
          o[u].w = fmaf(oc[u][c].w, f, o[u].w);
        }
        m[u] = m_new;
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = i0 + u * DS_THREADS;
      if (i >= total) continue;
      const int b = i / per_row, r = i - b * per_row;
      const float inv = lsum[u] > 0.f ? 1.0f / lsum[u] : 0.f;
      float4 v = o[u];
      v.x *= inv;
      v.y *= inv;
      v.z *= inv;
      v.w *= inv;
      *reinterpret_cast<float4*>(&xs[b * xs_ld + r * 4]) = v;
    }
  }
  __syncthreads();
}

// One chunk per sequence and head (many sequences): the output is o / l of that chunk; U outputs per thread in flight.
template <int U>
__device__ __forceinline__ void ds_stage_attention_one(float* xs, int xs_ld, const float* part, int B, int heads, int c0,
                                                       int kc) {
  constexpr int D = 128;
  const int per_row = kc / 4;
  const int total = B * per_row;
  for (int i0 = threadIdx.x; i0 < total; i0 += U * DS_THREADS) {
    float l[U];
    float4 o[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = i0 + u * DS_THREADS;
      if (i < total) {
        const int b = i / per_row, r = i - b * per_row;
        const float* base = part + (static_cast<int64_t>(b) * heads + c0 / D + r / (D / 4)) * (4 + D);
        l[u] = ds_ldcg(base + 1);
        o[u] = ds_ldcg4(base + 4 + (r % (D / 4)) * 4);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = i0 + u * DS_THREADS;
      if (i < total) {
        const int b = i / per_row, r = i - b * per_row;
        const float inv = l[u] > 0.f ? 1.0f / l[u] : 0.f;
        *reinterpret_cast<float4*>(&xs[b * xs_ld + r * 4]) = make_float4(o[u].x * inv, o[u].y * inv, o[u].z * inv, o[u].w * inv);
      }
    }
  }
  __syncthreads();
}

template <bool WIDE = false>
__device__ __forceinline__ void ds_stage_attention(float* xs, int xs_ld, const float* part, int B, int heads,
                                                   int kv_heads, int chunks, int c0, int kc) {
  if constexpr (WIDE) {
    if (chunks == 1) {
      ds_stage_attention_one<4>(xs, xs_ld, part, B, heads, c0, kc);
      return;
    }
  }
  ds_stage_attention_t<1, 8>(xs, xs_ld, part, B, heads, kv_heads, chunks, c0, kc);
}

__device__ __forceinline__ float ds_swish(float v) {  // x * sigmoid(x), two-branch stable sigmoid
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

// Per-head rmsNorm (weight wn) and rotate-half RoPE of the 128 values this warp holds as x[i] = element lane + 32 i.
__device__ __forceinline__ void ds_norm_rope(float (&x)[4], const float* wn, const float* cr, const float* sr,
                                             float eps, int lane) {
  float wv[4], cv[2], sv[2];  // requested before the reduction so that they overlap it
#pragma unroll
  for (int i = 0; i < 4; ++i) wv[i] = __ldg(wn + lane + 32 * i);
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    cv[i] = __ldg(cr + lane + 32 * i);
    sv[i] = __ldg(sr + lane + 32 * i);
  }
  float ss = x[0] * x[0];
  ss = fmaf(x[1], x[1], ss);
  ss = fmaf(x[2], x[2], ss);
  ss = fmaf(x[3], x[3], ss);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float denom = sqrtf(ss * (1.0f / 128.f) + eps);
#pragma unroll
  for (int i = 0; i < 4; ++i) x[i] = (x[i] / denom) * wv[i];
  float y[4];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float c = cv[i], s = sv[i];
    const float re = x[i], im = x[i + 2];
    y[i] = re * c - im * s;
    y[i + 2] = im * c + re * s;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) x[i] = y[i];
}

__device__ __forceinline__ float ds_warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float ds_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

constexpr int DS_KB = 16;  // keys a warp takes per step of the attention phase (four groups of four)
constexpr int DS_UN = 6;  // 256-column trips requested together per weight row slot

// One linear phase, described at run time so that its code exists once in the kernel (the step walks five of them
// per layer; a copy per call site made the kernel larger than the instruction cache).
struct DsLinear {
  const uint16_t* W;    // [N (or 2 N when epi == 2)][K] bf16
  int N, K;
  int stage;            // 0: xs = rmsNorm(src) * norm_w, 1: xs = src, 2: xs = attention output from the partials in src
  int heads, kv_heads, chunks;  // for stage == 2
  int xs_cols;                  // see DecodeStepParams
  const float* src;     // [B][K] fp32 in global memory
  const float* norm_w;
  int epi;              // 0: dst[m][n] = y, 1: dst[m][n] += y, 2: dst[m][n] = swish(y[n]) * y[N + n]
  float* dst;
  int ld;               // row stride of dst
  // requests for later phases, issued behind this phase's own first loads
  const uint16_t* pf_w[2];
  int pf_n[2], pf_k[2];
  const char *pf_k_rows, *pf_v_rows;  // K / V rows of this CTA's next attention unit (or null)
  int pf_lines;
};

__device__ __forceinline__ void ds_prefetch_later(const DsLinear& L, int gw, int GW, int lane) {
  for (int i = 0; i < 2; ++i)
    if (L.pf_w[i]) ds_prefetch_rows(L.pf_w[i], L.pf_n[i], L.pf_k[i], gw, GW, lane);
  if (L.pf_k_rows)
    for (int i = threadIdx.x; i < L.pf_lines; i += DS_THREADS) {
      asm volatile("prefetch.global.L2 [%0];" ::"l"(L.pf_k_rows + i * 128));
      asm volatile("prefetch.global.L2 [%0];" ::"l"(L.pf_v_rows + i * 128));
    }
}

// y[b][n] = sum_k xs[b][k] * W[n][k] for the rows this warp owns (n = gw, gw + GW, ...).
// Two "slots" of DS_UN 128-bit loads per lane are in flight at once: two rows when the warp owns several, the two
// halves of a piece of one row when it owns at most one, rows n and N + n of a fused gate / up weight when
// epi == 2. The activations are staged into shared memory after the first loads have been issued.
template <int MT>
__device__ __noinline__ void ds_linear_phase(const DsLinear& L, float* xs, int B, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gw = blockIdx.x * DS_WARPS + warp;
  const int GW = gridDim.x * DS_WARPS;
  const int K = L.K, N = L.N;
  const bool pair = L.epi == 2;
  const bool split_k = !pair && N <= GW;  // at most one row per warp: the slots take the two halves of the row
  auto prefetch_later_phases = [&]() { ds_prefetch_later(L, gw, GW, lane); };
  if (split_k) {
    // One row per warp at most. The activations are staged in pieces of xs_cols columns (all of them at once when
    // they fit); within a piece slot 0 takes the first half of the columns and slot 1 the second.
    const int n0 = gw;
    const bool have = n0 < N;
    const int XC = K < L.xs_cols ? K : L.xs_cols;
    float acc0[MT], acc1[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc0[m] = acc1[m] = 0.f;
    const uint16_t* wrow = L.W + static_cast<int64_t>(have ? n0 : 0) * K;
    for (int c0 = 0; c0 < K; c0 += XC) {
      const int kc = K - c0 < XC ? K - c0 : XC;
      const int hc = ((kc + 255) / 256 + 1) / 2;  // trips of slot 0 (at most DS_UN: xs_cols <= 3072)
      uint4 a[DS_UN], b[DS_UN];
#pragma unroll
      for (int u = 0; u < DS_UN; ++u) {
        const int k0 = u * 256 + lane * 8, k1 = (hc + u) * 256 + lane * 8;
        a[u] = b[u] = make_uint4(0u, 0u, 0u, 0u);
        if (have && u < hc && k0 < kc) a[u] = __ldg(reinterpret_cast<const uint4*>(wrow + c0 + k0));
        if (have && u < hc && k1 < kc) b[u] = __ldg(reinterpret_cast<const uint4*>(wrow + c0 + k1));
      }
      if (c0 == 0) prefetch_later_phases();
      else __syncthreads();  // every warp has finished with the previous piece
      if (L.stage == 0) ds_stage_rmsnorm(xs, K, L.src, L.norm_w, B, K, eps, warp, lane);  // (K <= xs_cols: one piece)
      else if (L.stage == 1) ds_stage_copy(xs, XC, L.src, B, K, c0, kc);
      else ds_stage_attention(xs, XC, L.src, B, L.heads, L.kv_heads, L.chunks, c0, kc);
      if (!have) continue;
#pragma unroll
      for (int u = 0; u < DS_UN; ++u) {
        const int k0 = u * 256 + lane * 8, k1 = (hc + u) * 256 + lane * 8;
        const bool on0 = u < hc && k0 < kc, on1 = u < hc && k1 < kc;
        if (!on0 && !on1) continue;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          if (on0) {
            const float4 xa = *reinterpret_cast<const float4*>(&xs[m * XC + k0]);
            const float4 xb = *reinterpret_cast<const float4*>(&xs[m * XC + k0 + 4]);
            acc0[m] = ds_dot8(a[u], xa, xb, acc0[m]);
          }
          if (on1) {
            const float4 xa = *reinterpret_cast<const float4*>(&xs[m * XC + k1]);
            const float4 xb = *reinterpret_cast<const float4*>(&xs[m * XC + k1 + 4]);
            acc1[m] = ds_dot8(b[u], xa, xb, acc1[m]);
          }
        }
      }
    }
    if (!have) return;
#pragma unroll
    for (int m = 0; m < MT; ++m) acc0[m] = ds_warp_sum(acc0[m] + acc1[m]);
    if (lane == 0) {
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        if (m >= B) break;
        float* d0 = L.dst + static_cast<int64_t>(m) * L.ld + n0;
        *d0 = L.epi == 1 ? acc0[m] + ds_ldcg(d0) : acc0[m];  // (epi 1: this warp is the only writer of the element)
      }
    }
    return;
  }
  // Several rows per warp: the whole activation rows are in shared memory (K <= xs_cols).
  const int trips = (K + 255) / 256;
  const int step = pair ? GW : 2 * GW;
  bool staged = false;
  for (int n0 = gw; n0 < N || !staged; n0 += step) {
    const bool have = n0 < N;
    const int n1 = n0 + GW;
    const bool two = have && !pair && n1 < N;
    float acc0[MT], acc1[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc0[m] = acc1[m] = 0.f;
    const uint16_t* w0 = L.W + static_cast<int64_t>(have ? n0 : 0) * K;
    const uint16_t* w1 = pair ? L.W + static_cast<int64_t>(N + (have ? n0 : 0)) * K
                              : L.W + static_cast<int64_t>(two ? n1 : 0) * K;
    const int k1_off = 0;
    const int t0_end = trips, t1_end = trips;
    const bool use1 = have && (pair || two);
    for (int t = 0; t < t0_end || !staged; t += DS_UN) {
      uint4 a[DS_UN], b[DS_UN];
#pragma unroll
      for (int u = 0; u < DS_UN; ++u) {
        const int kk = (t + u) * 256 + lane * 8;
        a[u] = b[u] = make_uint4(0u, 0u, 0u, 0u);
        if (have && t + u < t0_end && kk < K) a[u] = __ldg(reinterpret_cast<const uint4*>(w0 + kk));
        if (use1 && t + u < t1_end && k1_off + kk < K) b[u] = __ldg(reinterpret_cast<const uint4*>(w1 + kk));
      }
      if (!staged) {
        prefetch_later_phases();
        if (L.stage == 0) ds_stage_rmsnorm(xs, K, L.src, L.norm_w, B, K, eps, warp, lane);
        else if (L.stage == 1) ds_stage_copy(xs, K, L.src, B, K, 0, K);
        else ds_stage_attention(xs, K, L.src, B, L.heads, L.kv_heads, L.chunks, 0, K);
        staged = true;
      }
      if (!have) break;
#pragma unroll
      for (int u = 0; u < DS_UN; ++u) {
        const int kk = (t + u) * 256 + lane * 8;
        const int kk1 = k1_off + kk;
        const bool on0 = t + u < t0_end && kk < K;
        const bool on1 = use1 && t + u < t1_end && kk1 < K;
        if (!on0 && !on1) continue;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          if (on0) {
            const float4 xa = *reinterpret_cast<const float4*>(&xs[m * K + kk]);
            const float4 xb = *reinterpret_cast<const float4*>(&xs[m * K + kk + 4]);
            acc0[m] = ds_dot8(a[u], xa, xb, acc0[m]);
          }
          if (on1) {
            const float4 xa = *reinterpret_cast<const float4*>(&xs[m * K + kk1]);
            const float4 xb = *reinterpret_cast<const float4*>(&xs[m * K + kk1 + 4]);
            acc1[m] = ds_dot8(b[u], xa, xb, acc1[m]);
          }
        }
      }
    }
    if (!have) break;
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      acc0[m] = ds_warp_sum(acc0[m]);
      acc1[m] = ds_warp_sum(acc1[m]);
    }
    if (lane == 0) {
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        if (m >= B) break;
        float* d0 = L.dst + static_cast<int64_t>(m) * L.ld + n0;
        if (L.epi == 0) {
          *d0 = acc0[m];
          if (two) d0[GW] = acc1[m];
        } else if (L.epi == 1) {  // this warp is the only writer of these elements
          *d0 = acc0[m] + ds_ldcg(d0);
          if (two) d0[GW] = acc1[m] + ds_ldcg(d0 + GW);
        } else {
          *d0 = ds_swish(acc0[m]) * acc1[m];
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------------------------
// The linear phases on the tensor cores (two or more sequences). The FFMA form above spends one FMA per weight and
// sequence and is bound by that and by shared-memory reads from 2 sequences on; here a warp multiplies 8 x 32 pieces
// of W with 16 x 32 pieces of the activations by mma.sync (m16n8k16, bf16 operands, fp32 accumulators):
//   * the activations are the row operand: fp32 in shared memory, split into hi = bf16(x) and lo = bf16(x - hi) in
//     registers, both multiplied and added into the same accumulator (16 mantissa bits of x take part, as in the
//     operator path's tensor-core linears);
//   * 8 weight rows are the column operand, loaded straight from global memory with one 128-bit load per lane: lane
//     (g, t) holds W[n0 + g][k0 + 8 t .. k0 + 8 t + 7]. The k order inside a block of 32 is permuted the same way for
//     both operands (a sum over k does not care), so that no lane needs less than 16 contiguous bytes;
//   * a CTA owns 8 R weight rows (R = 1, 2, 4, chosen per phase so that the units fill the grid), its 8 warps split
//     the k range, their accumulators are added in warp order through shared memory (a fixed order: results do not
//     depend on timing), and the epilogue of ds_linear_phase is applied;
//   * k ranges longer than DS_MMA_XC are staged piece by piece.
constexpr int DS_MMA_XC = 1024;                       // activation columns staged at once
constexpr int DS_MMA_LD = DS_MMA_XC + 4;              // their row stride in shared memory (rows 4 banks apart)
constexpr int DS_MMA_NB = DS_MMA_XC / DS_WARPS / 32;  // blocks of 32 columns per warp and piece
constexpr int DS_MMA_RTS = 40;                        // row stride of the per-warp accumulator tiles (8 R <= 32, + 8)

// floats of dynamic shared memory the tensor-core phases need for `rows` (16 or 32) activation rows
constexpr int ds_mma_smem_floats(int rows) { return rows * DS_MMA_LD + DS_WARPS * rows * DS_MMA_RTS; }

__device__ __forceinline__ void ds_mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                            uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// (x0, x1) -> packed bf16 pairs hi and lo with x = hi + lo up to 16 mantissa bits; x0 in the low half
__device__ __forceinline__ void ds_split2(float x0, float x1, uint32_t& hi, uint32_t& lo) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(x0, x1);
  const __nv_bfloat162 l = __floats2bfloat162_rn(x0 - __low2float(h), x1 - __high2float(h));
  hi = *reinterpret_cast<const uint32_t*>(&h);
  lo = *reinterpret_cast<const uint32_t*>(&l);
}

// R: tiles of 8 weight rows per unit of work (a CTA takes units blockIdx.x, + gridDim.x, ...);
// MTILES: tiles of 16 activation rows (1: up to 16 sequences, 2: up to 32). Rows of `xs` beyond B hold anything:
// they only reach accumulator rows that are never stored.
template <int R, int MTILES>
__device__ __noinline__ void ds_linear_mma(const DsLinear& L, float* xs, int B, float eps) {
  constexpr int ROWS = 16 * MTILES;
  constexpr int NB = DS_MMA_NB;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int gw = blockIdx.x * DS_WARPS + warp, GW = gridDim.x * DS_WARPS;
  const int K = L.K, N = L.N;
  const bool pair = L.epi == 2;         // rows n and N + n of a fused gate / up weight: half of the tiles each
  const int out = pair ? 4 * R : 8 * R;  // output columns of a unit
  const int units = (N + out - 1) / out;
  const int pieces = (K + DS_MMA_XC - 1) / DS_MMA_XC;
  float* red = xs + ROWS * DS_MMA_LD;
  if (static_cast<int>(blockIdx.x) >= units) {  // nothing to multiply here: only the requests for later phases
    ds_prefetch_later(L, gw, GW, lane);
    return;
  }
  bool first = true;
  for (int u = blockIdx.x; u < units; u += gridDim.x) {
    const uint16_t* wrow[R];  // the row of W this lane loads for tile r
    bool wok[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      int local = r * 8 + g, base = 0;
      if constexpr (R >= 2) {
        if (pair) {
          local = (r % (R / 2)) * 8 + g;
          base = r >= R / 2 ? N : 0;
        }
      }
      const int n = u * out + local;
      wok[r] = n < N;
      wrow[r] = L.W + static_cast<int64_t>(base + (wok[r] ? n : 0)) * K;
    }
    float acc[R][MTILES][4];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int mt = 0; mt < MTILES; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[r][mt][i] = 0.f;
    uint4 wc[R][NB];
    auto load = [&](uint4(&w)[R][NB], int piece) {
#pragma unroll
      for (int r = 0; r < R; ++r)
#pragma unroll
        for (int j = 0; j < NB; ++j) {
          const int k = piece * DS_MMA_XC + (warp * NB + j) * 32 + 8 * t;
          w[r][j] = make_uint4(0u, 0u, 0u, 0u);
          if (wok[r] && k < K) w[r][j] = __ldg(reinterpret_cast<const uint4*>(wrow[r] + k));
        }
    };
    load(wc, 0);
    for (int pc = 0; pc < pieces; ++pc) {
      const int c0 = pc * DS_MMA_XC;
      const int kc = K - c0 < DS_MMA_XC ? K - c0 : DS_MMA_XC;
      if (first || pieces > 1) {
        if (first) ds_prefetch_later(L, gw, GW, lane);
        else __syncthreads();  // every warp has finished with what `xs` held
        if (L.stage == 0) ds_stage_rmsnorm(xs, DS_MMA_LD, L.src, L.norm_w, B, K, eps, warp, lane);  // (K <= DS_MMA_XC)
        else if (L.stage == 1) ds_stage_copy(xs, DS_MMA_LD, L.src, B, K, c0, kc);
        else ds_stage_attention<true>(xs, DS_MMA_LD, L.src, B, L.heads, L.kv_heads, L.chunks, c0, kc);
        first = false;
      }
      const bool more = pc + 1 < pieces;
      uint4 wn[1][NB];  // with one tile per unit the next piece's weights are requested ahead
      if constexpr (R == 1) {
        if (more) load(wn, pc + 1);
      }
#pragma unroll
      for (int j = 0; j < NB; ++j) {
        const int kl = (warp * NB + j) * 32;  // first column of the block within the piece (the same for the warp)
        if (kl >= kc) continue;
#pragma unroll
        for (int mt = 0; mt < MTILES; ++mt) {
          const float* r0 = xs + (16 * mt + g) * DS_MMA_LD + kl + 8 * t;
          const float4 x00 = *reinterpret_cast<const float4*>(r0);
          const float4 x01 = *reinterpret_cast<const float4*>(r0 + 4);
          const float4 x10 = *reinterpret_cast<const float4*>(r0 + 8 * DS_MMA_LD);
          const float4 x11 = *reinterpret_cast<const float4*>(r0 + 8 * DS_MMA_LD + 4);
          uint32_t h[8], l[8];
          ds_split2(x00.x, x00.y, h[0], l[0]);  // rows g / g + 8, columns 8 t + {0, 1} and + {2, 3}
          ds_split2(x10.x, x10.y, h[1], l[1]);
          ds_split2(x00.z, x00.w, h[2], l[2]);
          ds_split2(x10.z, x10.w, h[3], l[3]);
          ds_split2(x01.x, x01.y, h[4], l[4]);  // columns 8 t + {4, 5} and + {6, 7}
          ds_split2(x11.x, x11.y, h[5], l[5]);
          ds_split2(x01.z, x01.w, h[6], l[6]);
          ds_split2(x11.z, x11.w, h[7], l[7]);
#pragma unroll
          for (int r = 0; r < R; ++r) {
            const uint4 w = wc[r][j];
            ds_mma_bf16(acc[r][mt], h[0], h[1], h[2], h[3], w.x, w.y);
            ds_mma_bf16(acc[r][mt], l[0], l[1], l[2], l[3], w.x, w.y);
            ds_mma_bf16(acc[r][mt], h[4], h[5], h[6], h[7], w.z, w.w);
            ds_mma_bf16(acc[r][mt], l[4], l[5], l[6], l[7], w.z, w.w);
          }
        }
      }
      if (more) {
        if constexpr (R == 1) {
#pragma unroll
          for (int j = 0; j < NB; ++j) wc[0][j] = wn[0][j];
        } else {
          load(wc, pc + 1);
        }
      }
    }
    // the warps' accumulators, added in warp order
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int mt = 0; mt < MTILES; ++mt) {
        float* d = red + (warp * ROWS + 16 * mt + g) * DS_MMA_RTS + 8 * r + 2 * t;
        *reinterpret_cast<float2*>(d) = make_float2(acc[r][mt][0], acc[r][mt][1]);
        *reinterpret_cast<float2*>(d + 8 * DS_MMA_RTS) = make_float2(acc[r][mt][2], acc[r][mt][3]);
      }
    __syncthreads();
    for (int e = threadIdx.x; e < B * out; e += DS_THREADS) {
      const int b = e / out, c = e - b * out;
      const int n = u * out + c;
      if (n >= N) continue;
      float y = 0.f;
#pragma unroll
      for (int w = 0; w < DS_WARPS; ++w) y += red[(w * ROWS + b) * DS_MMA_RTS + c];
      float* d0 = L.dst + static_cast<int64_t>(b) * L.ld + n;
      if (pair) {
        float up = 0.f;
#pragma unroll
        for (int w = 0; w < DS_WARPS; ++w) up += red[(w * ROWS + b) * DS_MMA_RTS + 4 * R + c];
        *d0 = ds_swish(y) * up;
      } else if (L.epi == 1) {
        *d0 = y + ds_ldcg(d0);  // this thread is the only writer of the element
      } else {
        *d0 = y;
      }
    }
    __syncthreads();
  }
}

// Chooses the tiles per unit so that the busiest CTA streams the fewest weight rows (more tiles per unit when that
// costs at most a few per cent: the activations are then read from shared memory once for more rows).
template <int MTILES>
__device__ __forceinline__ void ds_linear_mma_any(const DsLinear& L, float* xs, int B, float eps) {
  const bool pair = L.epi == 2;
  int best = 0;
  float best_cost = 1e30f;
  for (int R = 4; R >= (pair ? 2 : 1); R >>= 1) {
    const int out = pair ? 4 * R : 8 * R;
    const int units = (L.N + out - 1) / out;
    const int rounds = (units + gridDim.x - 1) / gridDim.x;
    const float cost = static_cast<float>(rounds * R);
    if (cost < 0.94f * best_cost) {
      best = R;
      best_cost = cost;
    }
  }
  if (best == 4) ds_linear_mma<4, MTILES>(L, xs, B, eps);
  else if (best == 2) ds_linear_mma<2, MTILES>(L, xs, B, eps);
  else ds_linear_mma<1, MTILES>(L, xs, B, eps);
}

// (A kernel holds one form only: with both in one kernel the register allocation of every phase function suffered.)
template <int MT, bool MMA>
__device__ __forceinline__ void ds_linear(const DecodeStepParams& p, const DsLinear& L, float* xs, int B) {
  if constexpr (MMA) ds_linear_mma_any<(MT > 16 ? 2 : 1)>(L, xs, B, p.eps);
  else ds_linear_phase<MT>(L, xs, B, p.eps);
}

// The attention phase of one layer (see the file header). G = query heads per kv head.
template <int G>
__device__ __noinline__ void ds_attention_phase(const DecodeStepParams& p, const DsLayer& W, float* kc, float* vc,
                                                float* xs) {
  constexpr int D = 128;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int B = p.B;
  const int qkv_w = (p.heads + 2 * p.kv_heads) * D;
  const int units = B * p.kv_heads * p.chunks;
  const int n_keys = p.n_keys;
  const float* cr = p.cos_t + static_cast<int64_t>(p.rope_pos) * D;
  const float* sr = p.sin_t + static_cast<int64_t>(p.rope_pos) * D;
  float* qs = xs;                 // [G][128] query heads of the group, normalised and rotated
  float* pm = qs + G * D;         // [DS_WARPS][G] running maxima of the warps
  float* pl = pm + DS_WARPS * G;  // sums
  float* po = pl + DS_WARPS * G;  // [DS_WARPS][G][128] unnormalised outputs
  for (int u = blockIdx.x; u < units; u += gridDim.x) {
    const int chunk = u % p.chunks;
    const int bk = u / p.chunks;
    const int b = bk / p.kv_heads, kvh = bk - b * p.kv_heads;
    const float* row = p.qkv + static_cast<int64_t>(b) * qkv_w;
    const int k_begin = chunk * p.keys_per_chunk;
    int k_end = k_begin + p.keys_per_chunk;
    if (k_end > n_keys) k_end = n_keys;
    if (warp < G) {
      float x[4];
      const float* src = row + (kvh * G + warp) * D;
#pragma unroll
      for (int i = 0; i < 4; ++i) x[i] = ds_ldcg(src + lane + 32 * i);
      ds_norm_rope(x, W.q_norm, cr, sr, p.eps, lane);
#pragma unroll
      for (int i = 0; i < 4; ++i) qs[warp * D + lane + 32 * i] = x[i];
    } else if (warp == G && k_begin <= p.pos && p.pos < k_end) {  // this unit holds the token of this step
      float x[4], y[4];
      const float* ksrc = row + (p.heads + kvh) * D;
      const float* vsrc = row + (p.heads + p.kv_heads + kvh) * D;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        x[i] = ds_ldcg(ksrc + lane + 32 * i);
        y[i] = ds_ldcg(vsrc + lane + 32 * i);
      }
      ds_norm_rope(x, W.k_norm, cr, sr, p.eps, lane);
      float* kdst = kc + ((static_cast<int64_t>(b) * p.kv_heads + kvh) * p.max_pos + p.pos) * D;
      float* vdst = vc + ((static_cast<int64_t>(b) * p.kv_heads + kvh) * p.max_pos + p.pos) * D;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        kdst[lane + 32 * i] = x[i];
        vdst[lane + 32 * i] = y[i];
      }
    }
    __syncthreads();
    const float* kb = kc + (static_cast<int64_t>(b) * p.kv_heads + kvh) * p.max_pos * D;
    const float* vb = vc + (static_cast<int64_t>(b) * p.kv_heads + kvh) * p.max_pos * D;
    float m_run[G], l_run[G];
    float4 acc[G];  // value columns 4 lane .. 4 lane + 3
#pragma unroll
    for (int g = 0; g < G; ++g) {
      m_run[g] = -CUDART_INF_F;
      l_run[g] = 0.f;
      acc[g] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    // Scores: 8 lanes share a key (16 of its 128 values each), so one load instruction covers 4 whole K rows
    // (4 x 512 contiguous bytes) and a dot product is finished by 3 shuffles; a warp takes DS_KB keys per step, so
    // that the keys of a chunk spread over all 16 warps.
    const int j8 = lane & 7, kq = lane >> 3;
    float4 qreg[G][4];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int i = 0; i < 4; ++i) qreg[g][i] = *reinterpret_cast<const float4*>(&qs[g * D + (j8 + 8 * i) * 4]);
    for (int key0 = k_begin + warp * DS_KB; key0 < k_end; key0 += DS_WARPS * DS_KB) {
      // (The row of this step's token was stored by a warp of this CTA before the barrier above: plain loads.)
      float sc[G][DS_KB / 4];
      float4 vv[DS_KB];  // V rows of the step, requested before the scores are formed
#pragma unroll
      for (int t = 0; t < DS_KB; ++t) {
        vv[t] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (key0 + t < k_end) vv[t] = *(reinterpret_cast<const float4*>(vb + static_cast<int64_t>(key0 + t) * D) + lane);
      }
      float4 kvr[DS_KB / 4][4];
#pragma unroll
      for (int kg = 0; kg < DS_KB / 4; ++kg) {
        const int key = key0 + kg * 4 + kq;
        const float4* krow =
            reinterpret_cast<const float4*>(kb + static_cast<int64_t>(key < k_end ? key : k_begin) * D);
#pragma unroll
        for (int i = 0; i < 4; ++i) kvr[kg][i] = krow[j8 + 8 * i];
      }
#pragma unroll
      for (int kg = 0; kg < DS_KB / 4; ++kg) {
        const int key = key0 + kg * 4 + kq;
        const bool valid = key < k_end;
#pragma unroll
        for (int g = 0; g < G; ++g) {
          float d = 0.f;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            d = fmaf(qreg[g][i].x, kvr[kg][i].x, d);
            d = fmaf(qreg[g][i].y, kvr[kg][i].y, d);
            d = fmaf(qreg[g][i].z, kvr[kg][i].z, d);
            d = fmaf(qreg[g][i].w, kvr[kg][i].w, d);
          }
          d += __shfl_xor_sync(0xffffffffu, d, 1);
          d += __shfl_xor_sync(0xffffffffu, d, 2);
          d += __shfl_xor_sync(0xffffffffu, d, 4);
          sc[g][kg] = valid ? d * p.scale : -CUDART_INF_F;
        }
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float mx = sc[g][0];
#pragma unroll
        for (int kg = 1; kg < DS_KB / 4; ++kg) mx = fmaxf(mx, sc[g][kg]);
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
        const float m_new = fmaxf(m_run[g], mx);       // finite: every step has a valid key
        const float alpha = __expf(m_run[g] - m_new);  // 0 on the first step (m_run = -inf)
        float sum = 0.f;
#pragma unroll
        for (int kg = 0; kg < DS_KB / 4; ++kg) {
          sc[g][kg] = __expf(sc[g][kg] - m_new);  // probabilities from here on; 0 for keys past the end
          sum += sc[g][kg];
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 8);  // over the 4 key slots; the 8 lanes of a key hold copies
        sum += __shfl_xor_sync(0xffffffffu, sum, 16);
        l_run[g] = l_run[g] * alpha + sum;
        m_run[g] = m_new;
        acc[g].x *= alpha;
        acc[g].y *= alpha;
        acc[g].z *= alpha;
        acc[g].w *= alpha;
      }
      // P.V: value columns across lanes (one coalesced row per key), probabilities broadcast key by key
#pragma unroll
      for (int kg = 0; kg < DS_KB / 4; ++kg) {
#pragma unroll
        for (int t = 0; t < 4; ++t) {
#pragma unroll
          for (int g = 0; g < G; ++g) {
            const float pt = __shfl_sync(0xffffffffu, sc[g][kg], t * 8);
            acc[g].x = fmaf(pt, vv[kg * 4 + t].x, acc[g].x);
            acc[g].y = fmaf(pt, vv[kg * 4 + t].y, acc[g].y);
            acc[g].z = fmaf(pt, vv[kg * 4 + t].z, acc[g].z);
            acc[g].w = fmaf(pt, vv[kg * 4 + t].w, acc[g].w);
          }
        }
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      if (lane == 0) {
        pm[warp * G + g] = m_run[g];
        pl[warp * G + g] = l_run[g];
      }
      *reinterpret_cast<float4*>(&po[(warp * G + g) * D + lane * 4]) = acc[g];
    }
    __syncthreads();
    if (warp < G) {
      // warp g combines the 16 warps' results of query head g
      const int g = warp;
      const float mw = lane < DS_WARPS ? pm[lane * G + g] : -CUDART_INF_F;
      const float lw = lane < DS_WARPS ? pl[lane * G + g] : 0.f;
      const float m = ds_warp_max(mw);
      const float fw = (mw == -CUDART_INF_F) ? 0.f : __expf(mw - m);
      const float lsum = ds_warp_sum(lw * fw);
      float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
      for (int w = 0; w < DS_WARPS; ++w) {
        const float f = __shfl_sync(0xffffffffu, fw, w);
        const float4 ow = *reinterpret_cast<const float4*>(&po[(w * G + g) * D + lane * 4]);
        o.x = fmaf(ow.x, f, o.x);
        o.y = fmaf(ow.y, f, o.y);
        o.z = fmaf(ow.z, f, o.z);
        o.w = fmaf(ow.w, f, o.w);
      }
      // partial of this chunk: m, l, unnormalised o; the o-projection phase combines the chunks while it stages
      float* dst = p.part + ((static_cast<int64_t>(bk) * p.chunks + chunk) * G + g) * (4 + D);
      if (lane == 0) {
        dst[0] = m;
        dst[1] = lsum;
      }
      *reinterpret_cast<float4*>(dst + 4 + lane * 4) = o;
    }
    __syncthreads();  // the scratch is reused by this CTA's next unit
  }
}

template <int MT, int G, bool MMA>
__global__ void __launch_bounds__(DS_THREADS, 1) decode_step_kernel(const DecodeStepParams p) {
  extern __shared__ __align__(16) float xs[];  // [MT][max K]; the attention phase uses it as scratch
  constexpr int D = 128;
  const int B = p.B, H = p.hidden;
  const int qkv_w = (p.heads + 2 * p.kv_heads) * D;
  const int attn_w = p.heads * D;
  unsigned int epoch = 0;
  unsigned int ar = 0;  // exchanges between the tensor-parallel ranks done in this launch

  // ---- embedding gather: x[b, :] = float(embed[ids[b], :])
  {
    const int per_row = H / 4;
    for (int i = blockIdx.x * DS_THREADS + threadIdx.x; i < B * per_row; i += gridDim.x * DS_THREADS) {
      const int b = i / per_row, c = (i - b * per_row) * 4;
      int id = p.ids[b];
      id = id < 0 ? 0 : (id >= p.vocab ? p.vocab - 1 : id);
      const uint2 w = __ldg(reinterpret_cast<const uint2*>(p.embed + static_cast<int64_t>(id) * H + c));
      float4 o;
      o.x = __uint_as_float(w.x << 16);
      o.y = __uint_as_float(w.x & 0xFFFF0000u);
      o.z = __uint_as_float(w.y << 16);
      o.w = __uint_as_float(w.y & 0xFFFF0000u);
      *reinterpret_cast<float4*>(p.x + static_cast<int64_t>(b) * H + c) = o;
    }
  }
  if (!ds_grid_sync(p, epoch)) return;

  // K / V rows of this CTA's first attention unit (a CTA has more than one only with very many sequences or
  // very long contexts; the others are then fetched on demand)
  const char *kv_k = nullptr, *kv_v = nullptr;
  int kv_lines = 0;
  int64_t kv_off = 0;
  if (static_cast<int>(blockIdx.x) < B * p.kv_heads * p.chunks) {
    const int chunk = blockIdx.x % p.chunks, bk = blockIdx.x / p.chunks;
    const int k_begin = chunk * p.keys_per_chunk;
    int k_end = k_begin + p.keys_per_chunk;
    if (k_end > p.n_keys) k_end = p.n_keys;
    kv_off = (static_cast<int64_t>(bk) * p.max_pos + k_begin) * D;
    kv_lines = k_end > k_begin ? (k_end - k_begin) * 4 : 0;
  }

  for (int l = 0; l < p.layers; ++l) {
    const DsLayer W = p.lw[l];
    float* kc = p.k_cache + static_cast<size_t>(l) * p.cache_layer;
    float* vc = p.v_cache + static_cast<size_t>(l) * p.cache_layer;
    if (kv_lines > 0) {
      kv_k = reinterpret_cast<const char*>(kc + kv_off);
      kv_v = reinterpret_cast<const char*>(vc + kv_off);
    }
    DsLinear L;

    // ---- qkv = rmsNorm(x) . Wqkv^T
    L = DsLinear{W.qkv, qkv_w, H, 0, 0, 0, 0, p.xs_cols, p.x, W.norm1, 0, p.qkv, qkv_w, {W.o, nullptr}, {H, 0}, {attn_w, 0},
                 kv_k, kv_v, kv_lines};
    ds_linear<MT, MMA>(p, L, xs, B);
    if (!ds_grid_sync(p, epoch)) return;

    // ---- attention over the cache (+ per-head rmsNorm, RoPE, KV append); the gate / up rows are requested here
    {
      const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
      const int gw = blockIdx.x * DS_WARPS + warp, GW = gridDim.x * DS_WARPS;
      ds_prefetch_rows(W.gate_up, p.inter, H, gw, GW, lane);
      ds_prefetch_rows(W.gate_up + static_cast<int64_t>(p.inter) * H, p.inter, H, gw, GW, lane);
    }
    ds_attention_phase<G>(p, W, kc, vc, xs);
    if (!ds_grid_sync(p, epoch)) return;

    // ---- x += attn . Wo^T
    L = DsLinear{W.o, H, attn_w, 2, p.heads, p.kv_heads, p.chunks, p.xs_cols, p.part, nullptr, 1, p.x, H, {W.down, nullptr},
                 {H, 0}, {p.inter, 0}, nullptr, nullptr, 0};
    if (p.tp_world > 1) {  // partial sums over this rank's heads go to the mailbox, the ranks' sums to x
      L.epi = 0;
      L.dst = p.mail[p.tp_rank] + static_cast<int64_t>((p.ar_base + ar) & 1) * DS_MAX_B * H;
    }
    ds_linear<MT, MMA>(p, L, xs, B);
    if (p.tp_world > 1) {
      if (!ds_cross_sync(p, epoch, p.ar_base + ar + 1)) return;
      ds_reduce_mailboxes(p, (p.ar_base + ar) & 1);
      ++ar;
    }
    if (!ds_grid_sync(p, epoch)) return;

    // ---- act = swish(gate) * up, gate / up = rmsNorm(x) . Wgu^T (rows i and inter + i of the fused weight)
    {
      const bool last = l + 1 == p.layers;
      const int4 nxt = last ? make_int4(p.vocab_rows < 4 * static_cast<int>(gridDim.x) * DS_WARPS
                                            ? p.vocab_rows
                                            : 4 * static_cast<int>(gridDim.x) * DS_WARPS, H, 0, 0)
                            : make_int4(qkv_w, H, 0, 0);
      L = DsLinear{W.gate_up, p.inter, H, 0, 0, 0, 0, p.xs_cols, p.x, W.norm2, 2, p.act, p.inter,
                   {last ? p.lm_head : p.lw[l + 1].qkv, nullptr}, {nxt.x, 0}, {nxt.y, 0}, nullptr, nullptr, 0};
    }
    ds_linear<MT, MMA>(p, L, xs, B);
    if (!ds_grid_sync(p, epoch)) return;

    // ---- x += act . Wdown^T
    L = DsLinear{W.down, H, p.inter, 1, 0, 0, 0, p.xs_cols, p.act, nullptr, 1, p.x, H, {nullptr, nullptr}, {0, 0}, {0, 0},
                 nullptr, nullptr, 0};
    if (p.tp_world > 1) {
      L.epi = 0;
      L.dst = p.mail[p.tp_rank] + static_cast<int64_t>((p.ar_base + ar) & 1) * DS_MAX_B * H;
    }
    ds_linear<MT, MMA>(p, L, xs, B);
    if (p.tp_world > 1) {
      if (!ds_cross_sync(p, epoch, p.ar_base + ar + 1)) return;
      ds_reduce_mailboxes(p, (p.ar_base + ar) & 1);
      ++ar;
    }
    if (!ds_grid_sync(p, epoch)) return;
  }

  // ---- logits = rmsNorm(x) . Wvocab^T
  DsLinear L{p.lm_head, p.vocab_rows, H, 0, 0, 0, 0, p.xs_cols, p.x, p.final_norm, 0, p.logits, p.vocab_rows, {nullptr, nullptr},
             {0, 0}, {0, 0}, nullptr, nullptr, 0};
  ds_linear<MT, MMA>(p, L, xs, B);
}

}  // namespace ytk
