// One decode step (up to four sequences; one GPU, or one rank of a tensor-parallel group) as ONE kernel WITHOUT grid
// barriers.
//
// A decode step of the 0.6B shape is 141 dependent phases of a few microseconds; with a grid barrier between them
// every phase pays three trips through the L2 (arrive, poll, then load what the others wrote) on top of its work. Here
// the activations that cross from one phase to the next carry their own synchronisation: every value is stored as an
// 8-byte pair {bits, tag} with one store instruction (8-byte stores are single-copy atomic), where the tag names the
// phase that produced it. A consumer simply loads the pairs it needs and repeats the load of any pair whose tag is not
// yet the one it expects; when the tag is there, so is the value. A phase therefore starts one L2 trip after its
// producers have stored, with no arrive / poll round in between.
//
//   tags      base + 0 the step's embedding (not exchanged: every CTA gathers the rows itself); per layer l,
//             base + 1 + 5 l + {0 qkv, 1 attention output, 2 residual after the o projection, 3 swish(gate) * up,
//             4 residual after the down projection}. `base` advances by 2 + 5 layers per launch, so a tag never
//             repeats and leftovers of earlier steps can not be mistaken for this step's values.
//   buffers   x [B][hidden], qkv [B][qkv_w], att [B][heads * 128], act [B][inter], all as pairs. A buffer is
//             rewritten one layer later; every phase's output depends on ALL CTAs having staged the previous
//             contents (the dependencies between phases are all-to-all), so no value is overwritten while someone
//             still needs it.
//   residual  the o and down projections have the same row split, so a CTA is the only writer of its rows of x and
//             keeps them in shared memory for the whole step: x += y never reads x back from global memory.
//   weights   stream through the shared-memory ring of decode_stream.cuh (bulk async copies that run ahead of the
//             phases by the depth of the ring).
//   ranks     tensor parallel (heads and FFN columns split): the thread that finishes a row of the o or down projection
//             pushes its rank's share as a pair into slot [its rank] of every peer's pair area (NVLink stores), polls
//             its own area for the peers' shares and adds all of them in rank order: every rank holds bitwise the same
//             residual. A slot is rewritten one layer later, by when its reader has long passed (it has produced the
//             next exchange's share, which needs every CTA of its GPU to have finished this one).
//   rmsNorm   x * weight is staged while the sum of squares is reduced; 1 / sqrt(mean + eps) multiplies the finished
//             dot products (one pass over the row, one block-wide synchronisation).
//   attention (sequence, kv head, key chunk) units as in decode_step.cuh; the units of chunks 1, 2, ... store their
//             partial results (maximum, sum, unnormalised output) as pairs too, and the unit of chunk 0 collects
//             them, combines the chunks and stores the attention output as pairs. A CTA holds at most one unit (the
//             host sizes the chunks that way), so a collecting unit never waits for a unit of its own CTA.
//
// All CTAs must be resident at once (they wait for each other's stores): the launch is cooperative. Every wait is
// bounded by the run-time cycle budget; a CTA that gives up raises the device status word and a global abort flag
// that makes every other wait give up at once, drains the bulk copies in flight into its shared memory and returns.
#pragma once

#include "decode_stream.cuh"

namespace ytk {

constexpr int LL_WARPS = 7;                  // worker warps
constexpr int LL_WORKERS = LL_WARPS * 32;
constexpr int LL_THREADS = LL_WORKERS + 32;  // the eighth warp only issues the weight copies (eight warps of 224
                                             // registers would not fit a ninth: registers are per scheduler)
constexpr int LL_MAX_OWN = 64;  // rows of x one CTA may own (hidden / CTAs, rounded up)
constexpr int DS_MAX_CHUNKS_LL = 64;  // key chunks per (sequence, kv head) the partial-result buffer holds
constexpr int LL_GROUP = 4;     // chunks of the weight ring a linear phase takes at a time
// partial sums of the warps [LL_WARPS][LL_GROUP][16][sequences], and the attention phase's scratch (query heads,
// the warps' maxima, sums and outputs): sized for the kernel instance at hand, every KB not spent here is ring depth
__host__ __device__ constexpr int ll_part_floats(int mt) { return LL_WARPS * LL_GROUP * 16 * mt; }
__host__ __device__ constexpr int ll_att_floats(int g) { return g * 128 + 2 * LL_WARPS * g + LL_WARPS * g * 128; }

// Synchronises the worker threads (named barrier 1); the issuing warp never takes part.
__device__ __forceinline__ void ll_sync() { asm volatile("bar.sync 1, %0;" ::"n"(LL_WORKERS) : "memory"); }

__device__ __forceinline__ uint4 ll_ld2(const uint2* p) {  // two pairs; L1 is bypassed (another SM wrote them)
  uint4 v;
  asm volatile("ld.relaxed.gpu.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ uint2 ll_ld1(const uint2* p) {
  uint2 v;
  asm volatile("ld.relaxed.gpu.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void ll_st(uint2* p, float v, unsigned int tag) {
  asm volatile("st.relaxed.gpu.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(tag) : "memory");
}

// Bounded polling: true when the caller should give up - the cycle budget since t0 is spent, or another CTA has
// already given up (checked every 64th spin).
__device__ __forceinline__ bool ll_expired(const DecodeStepParams& p, int* abort_word, long long t0, int spins) {
  if ((spins & 63) == 63) {
    if (*reinterpret_cast<volatile int*>(abort_word)) return true;
    unsigned int g;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(g) : "l"(p.sync) : "memory");
    if ((g & 0x80000000u) || clock64() - t0 > p.wait_cycles) {
      *reinterpret_cast<volatile int*>(abort_word) = 1;
      return true;
    }
  }
  return false;
}

// Shared-memory layout of a staged activation row: the 8 values of 16-byte weight piece q = lane + 32 i (lane < 32)
// are kept as two float4 at float4 indices (2 i) * 32 + lane and (2 i + 1) * 32 + lane, so that the 32 lanes of a
// warp, each reading "its" piece, touch 512 contiguous bytes per load: no bank conflicts. A row takes
// ll_row_floats(K) floats.
__device__ __forceinline__ int ll_perm(int k) {
  const int q = k >> 3, e8 = k & 7;
  return ((((q >> 5) * 2 + (e8 >> 2)) * 32 + (q & 31)) << 2) + (e8 & 3);
}
__host__ __device__ __forceinline__ int ll_row_floats(int K) { return (K + 255) / 256 * 256; }

// Optional timeline (ytcuda_qwen3_set_trace): the first and the last CTA stamp their SM's cycle counter, slot after slot.
__device__ __forceinline__ void ll_trace(const DecodeStepParams& p, int& idx) {
  if (p.trace && threadIdx.x == 0 && (blockIdx.x == 0 || blockIdx.x + 1 == gridDim.x)) {
    if (idx < p.trace_cap) p.trace[(blockIdx.x ? p.trace_cap : 0) + idx] = clock64();
    ++idx;
  }
}

// xs[b][0 .. n) = value of pair src[b][i] (times scale[i] when given) once every tag equals `tag`; ss[b] += sum of
// squares of the unscaled values. All loads of a pass are in flight together; the worker threads, n even.
template <int MT, bool NORM>
__device__ __forceinline__ void ll_stage(const DecodeStepParams& p, int* abort_word, float* xs, int ld,
                                         const uint2* src, int n, unsigned int tag, const float* scale, float* red) {
  constexpr int U = 4;
  const int tid = threadIdx.x;
  float ss[MT];
#pragma unroll
  for (int b = 0; b < MT; ++b) ss[b] = 0.f;
  const long long t0 = clock64();
  for (int base = 0; base < n; base += U * 2 * LL_WORKERS) {
    float2 g[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = base + (u * LL_WORKERS + tid) * 2;
      g[u] = make_float2(1.f, 1.f);
      if (NORM && i < n) g[u] = __ldg(reinterpret_cast<const float2*>(scale + i));
    }
#pragma unroll
    for (int b = 0; b < MT; ++b) {
      if (b >= p.B) break;
      const uint2* row = src + static_cast<int64_t>(b) * n;
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = base + (u * LL_WORKERS + tid) * 2;
        v[u] = make_uint4(0u, tag, 0u, tag);
        if (i < n) v[u] = ll_ld2(row + i);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = base + (u * LL_WORKERS + tid) * 2;
        if (i >= n) continue;
        int spins = 0;
        while (v[u].y != tag || v[u].w != tag) {
          if (ll_expired(p, abort_word, t0, spins++)) break;
          v[u] = ll_ld2(row + i);
        }
        const float a = __uint_as_float(v[u].x), c = __uint_as_float(v[u].z);
        if (NORM) {
          ss[b] = fmaf(a, a, ss[b]);
          ss[b] = fmaf(c, c, ss[b]);
        }
        uint32_t hi, lo;
        ds_split2(a * g[u].x, c * g[u].y, hi, lo);
        uint32_t* pl = reinterpret_cast<uint32_t*>(xs) + ((2 * b) * ld + i) / 2;  // bf16 planes of ld elements
        pl[0] = hi;
        pl[ld / 2] = lo;
      }
    }
  }
  if (NORM) {
    const int warp = tid >> 5, lane = tid & 31;
#pragma unroll
    for (int b = 0; b < MT; ++b) {
      const float s = ds_warp_sum(ss[b]);
      if (lane == 0) red[b * 8 + warp] = s;
    }
  }
  ll_sync();
}

// One linear phase without barriers, on the tensor cores. stage 0: the staged activations are x * norm_w with the row
// factors 1 / sqrt(mean(x^2) + eps) applied to the dot products; 1: the pairs of src; 3: already staged (first layer:
// the embedding).
// epi 0: dst pairs = y; 1: x_own += y, dst pairs = x_own; 2: dst pairs = swish(y_gate) * y_up; 3: plain floats to out.
//
// Sixteen weight rows from the ring are the row operand of mma.sync m16n8k16;
// the column operand holds the activations as bf16 planes, column 2 b = hi and 2 b + 1 = lo of sequence b
// (x = hi + lo to 16 mantissa bits, as in the other tensor-core linears of this library), so one instruction does the
// work of 16 warp-wide FMAs per sequence and no weight is unpacked. The k order inside a block of 32 is permuted the
// same way for both operands: lane (g, q) takes the 16 contiguous bytes k = 32 kb + 8 q .. + 7 of weight rows g and
// g + 8 and of plane g. The seven warps split the k range; their accumulators are added through shared memory in
// warp order (fixed order: results do not depend on timing).
template <int MT>
__device__ __forceinline__ bool ll_linear(const DecodeStepParams& p, DwShared& S, char* ring, float* xs, float* red,
                                       float* x_own, float* part, int kind, int stage, const uint2* src,
                                       unsigned int src_tag, const float* norm_w, int epi, uint2* dst,
                                       unsigned int dst_tag, float* out, int ld, int& c, int& slot, unsigned int& parity,
                                       int& tr) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gq = lane >> 2, q4 = lane & 3;
  const DwPhase ph = S.ph[kind];
  const int K = ph.K, B = p.B;
  ll_trace(p, tr);
  if (stage == 0) ll_stage<MT, true>(p, &S.abort_word, xs, ll_row_floats(K), src, K, src_tag, norm_w, red);
  else if (stage == 1) ll_stage<MT, false>(p, &S.abort_word, xs, ll_row_floats(K), src, K, src_tag, nullptr, red);
  if (*reinterpret_cast<volatile int*>(&S.abort_word)) return false;
  ll_trace(p, tr);
  const bool pair = kind == 2;
  const int row_bytes = K * 2;
  const int KP = ll_row_floats(K);
  const int nkp = K >> 6;  // pairs of 32-wide blocks along k
  const bool b_on = gq < 2 * B;  // this lane's column of the activation operand is a plane (else zero)
  const char* bsrc = reinterpret_cast<const char*>(xs) + static_cast<size_t>(b_on ? gq : 0) * KP * 2 + q4 * 16;
  for (int j0 = 0; j0 < ph.nchunks; j0 += LL_GROUP) {
    const int gc = ph.nchunks - j0 < LL_GROUP ? ph.nchunks - j0 : LL_GROUP;
    int slots[LL_GROUP];
    unsigned int pars[LL_GROUP];
    {
      int sl = slot;
      unsigned int par = parity;
#pragma unroll
      for (int j = 0; j < LL_GROUP; ++j) {
        slots[j] = sl;
        pars[j] = par;
        if (j < gc && ++sl == S.nslot) {
          sl = 0;
          par ^= 1u;
        }
      }
      slot = sl;
      parity = par;
      // the chunks have normally landed long ago: test all barriers at once, wait only where that fails
      bool ready = true;
#pragma unroll
      for (int j = 0; j < LL_GROUP; ++j)
        if (j < gc) ready &= mbar_test_wait(&S.full[slots[j]], pars[j]);
      if (!ready) {
#pragma unroll
        for (int j = 0; j < LL_GROUP; ++j)
          if (j < gc && !mbar_wait_limit(&S.full[slots[j]], pars[j], &S.abort_word, p.wait_cycles)) return false;
      }
    }
#ifdef LL_TRACE_FINE
    ll_trace(p, tr);
#endif
    // The rows of the group's chunks (pairs: all gate rows, then all up rows) are packed into tiles of 16 whatever
    // chunk they lie in: a lane's two row pointers per tile are free to point into different slots of the ring.
    int P = ph.rows - j0 * ph.rpc;  // rows (gate / up pairs) of the group
    if (P > gc * ph.rpc) P = gc * ph.rpc;
    const int R = pair ? 2 * P : P;
    const int T = (R + 15) >> 4;
    auto row_ptr = [&](int rr) -> const char* {
      rr = rr < R ? rr : R - 1;  // rows past the end repeat the last one (their results are not used)
      const bool up = pair && rr >= P;
      const int pr = up ? rr - P : rr;
      const int jc = (pr >= ph.rpc ? 1 : 0) + (pr >= 2 * ph.rpc ? 1 : 0) + (pr >= 3 * ph.rpc ? 1 : 0);
      const int off = pr - jc * ph.rpc;
      int nrj = P - jc * ph.rpc;
      nrj = nrj < ph.rpc ? nrj : ph.rpc;
      const int sl = jc == 0 ? slots[0] : jc == 1 ? slots[1] : jc == 2 ? slots[2] : slots[3];
      return ring + static_cast<size_t>(sl) * DW_CHUNK + (off + (up ? nrj : 0)) * row_bytes + q4 * 16;
    };
    // Tile after tile (a real loop: straight-line code runs at the speed of instruction fetch here, a loop body is
    // fetched once); a trip takes two neighbouring k blocks (128 bytes of every row) with accumulators of their own
    // and issues all its loads before the first MMA. Weight rows lie a multiple of 128 bytes apart, so eight rows
    // reading the same 64 bytes would meet in the same banks: rows with odd g read the two blocks in the opposite
    // order (each quarter warp then covers all 32 banks) and swap the registers afterwards.
    const bool odd = (gq & 1) != 0;
    const int h1 = odd ? 64 : 0, h2 = 64 - h1;
#pragma unroll 1
    for (int t = 0; t < T; ++t) {
      const char* wa = row_ptr(16 * t + gq);      // this lane's 16 bytes of row g of the tile
      const char* wb = row_ptr(16 * t + gq + 8);  // ... of row g + 8
      float a1[4] = {0.f, 0.f, 0.f, 0.f}, a2[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
      for (int kp = warp; kp < nkp; kp += LL_WARPS) {
        const int o = kp * 128;
        uint4 bx = make_uint4(0u, 0u, 0u, 0u), bx2 = bx;
        if (b_on) {
          bx = *reinterpret_cast<const uint4*>(bsrc + o);
          bx2 = *reinterpret_cast<const uint4*>(bsrc + o + 64);
        }
        const uint4 r1 = *reinterpret_cast<const uint4*>(wa + o + h1);
        const uint4 r2 = *reinterpret_cast<const uint4*>(wa + o + h2);
        const uint4 s1 = *reinterpret_cast<const uint4*>(wb + o + h1);
        const uint4 s2 = *reinterpret_cast<const uint4*>(wb + o + h2);
        const uint4 a_lo = odd ? r2 : r1, c_lo = odd ? r1 : r2;  // first / second block of rows g
        const uint4 a_hi = odd ? s2 : s1, c_hi = odd ? s1 : s2;  // ... of rows g + 8
        ds_mma_bf16(a1, a_lo.x, a_hi.x, a_lo.y, a_hi.y, bx.x, bx.y);
        ds_mma_bf16(a2, c_lo.x, c_hi.x, c_lo.y, c_hi.y, bx2.x, bx2.y);
        ds_mma_bf16(a1, a_lo.z, a_hi.z, a_lo.w, a_hi.w, bx.z, bx.w);
        ds_mma_bf16(a2, c_lo.z, c_hi.z, c_lo.w, c_hi.w, bx2.z, bx2.w);
      }
      // accumulator columns 2 q and 2 q + 1 are the hi and lo products of sequence q: rows g and g + 8
      if (q4 < B) {
        float* pj = part + ((warp * LL_GROUP + t) * 16) * MT;
        pj[gq * MT + q4] = (a1[0] + a2[0]) + (a1[1] + a2[1]);
        pj[(gq + 8) * MT + q4] = (a1[2] + a2[2]) + (a1[3] + a2[3]);
      }
    }
#ifdef LL_TRACE_FINE
    ll_trace(p, tr);
#endif
    float inv[MT];
#pragma unroll
    for (int b = 0; b < MT; ++b) {
      inv[b] = 1.f;
      if (stage == 0 || stage == 3) {
        // red is [MT][8] (the eighth entry of a row is zero): two 128-bit loads per sequence
        const float4 r0 = *reinterpret_cast<const float4*>(&red[b * 8]);
        const float4 r1 = *reinterpret_cast<const float4*>(&red[b * 8 + 4]);
        const float s = ((r0.x + r0.y) + (r0.z + r0.w)) + ((r1.x + r1.y) + (r1.z + r1.w));
        inv[b] = rsqrtf(s * (1.0f / static_cast<float>(K)) + p.eps);
      }
    }
    ll_sync();  // the partial sums are complete; nobody reads the ring slots, xs or red of this group any more
    c += gc;
    if (threadIdx.x == 0) *reinterpret_cast<volatile int*>(&S.consumed) = c;  // the issuing warp refills the slots
    // one thread per (row or pair, sequence): sum over the warps, epilogue, publish
    for (int task = threadIdx.x; task < LL_GROUP * 16 * MT; task += LL_WORKERS) {
      const int r = task / MT, m = task % MT;
      if (r >= P || m >= B) continue;
      const int r2 = P + r;  // the up row of a pair
      float y = 0.f, y2 = 0.f;
#pragma unroll
      for (int w = 0; w < LL_WARPS; ++w) {
        y += part[((w * LL_GROUP + (r >> 4)) * 16 + (r & 15)) * MT + m];
        if (pair) y2 += part[((w * LL_GROUP + (r2 >> 4)) * 16 + (r2 & 15)) * MT + m];
      }
      y *= inv[m];
      const int n = ph.r0 + j0 * ph.rpc + r;
      if (epi == 2) {
        ll_st(dst + static_cast<int64_t>(m) * ld + n, ds_swish(y) * (y2 * inv[m]), dst_tag);
      } else if (epi == 1) {
        if (p.tp_world > 1) {
          // y is this rank's share of the sum over k: push it into every peer's pair area, then add the shares of
          // all ranks in rank order (the same order everywhere: every rank holds bitwise the same x)
          const size_t per_src = static_cast<size_t>(2) * 4 * p.hidden;
          const size_t at = (static_cast<size_t>(kind == 3 ? 1 : 0) * 4 + m) * p.hidden + n;
          for (int q = 0; q < p.tp_world; ++q) {
            if (q == p.tp_rank) continue;
            asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(p.ll_mail[q] + p.tp_rank * per_src + at),
                         "r"(__float_as_uint(y)), "r"(dst_tag)
                         : "memory");
          }
          // the peers' pairs are requested together (one trip to the L2 for all of them), then taken in rank order
          uint2 pr[DS_MAX_TP];
#pragma unroll
          for (int r = 0; r < DS_MAX_TP; ++r) {
            pr[r] = make_uint2(0u, dst_tag);
            if (r < p.tp_world && r != p.tp_rank) {
              const uint2* src_pair = p.ll_mail[p.tp_rank] + r * per_src + at;
              asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(pr[r].x), "=r"(pr[r].y) : "l"(src_pair) : "memory");
            }
          }
          float tot = 0.f;
          const long long t0 = clock64();
#pragma unroll
          for (int r = 0; r < DS_MAX_TP; ++r) {
            if (r >= p.tp_world) break;
            float v = y;
            if (r != p.tp_rank) {
              const uint2* src_pair = p.ll_mail[p.tp_rank] + r * per_src + at;
              int spins = 0;
              while (pr[r].y != dst_tag) {
                if (ll_expired(p, &S.abort_word, t0, spins++)) break;
                asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(pr[r].x), "=r"(pr[r].y) : "l"(src_pair) : "memory");
              }
              v = __uint_as_float(pr[r].x);
            }
            tot += v;
          }
          y = tot;
        }
        float* xo = x_own + m * LL_MAX_OWN + (n - ph.r0);
        const float y0 = xo[0] + y;
        xo[0] = y0;
        ll_st(dst + static_cast<int64_t>(m) * ld + n, y0, dst_tag);
      } else if (epi == 0) {
        ll_st(dst + static_cast<int64_t>(m) * ld + n, y, dst_tag);
      } else {
        out[static_cast<int64_t>(m) * ld + n] = y;
      }
    }
    // The partial sums have been read (another group overwrites them). The synchronisation also keeps the threads
    // without an epilogue task from polling for the next phase's inputs while this CTA's own results are still being
    // stored: without it the polling loads delay those stores, and with them every CTA that waits for them (measured:
    // 8 % more time per layer).
    ll_sync();
  }
  ll_trace(p, tr);
  return true;
}

// The attention phase of one layer without barriers: q, k, v of this step arrive as pairs; the last unit of a
// (sequence, kv head) combines the key chunks and stores the attention output as pairs. xs is scratch (DS_ATT_FLOATS).
template <int G>
__device__ __forceinline__ bool ll_attention(const DecodeStepParams& p, DwShared& S, const DsLayer& W, float* kc, float* vc,
                                          float* xs, unsigned int qkv_tag, unsigned int att_tag, int& tr) {
  constexpr int D = 128;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int B = p.B;
  const int qkv_w = (p.heads + 2 * p.kv_heads) * D;
  const int attn_w = p.heads * D;
  const int units = B * p.kv_heads * p.chunks;
  const int n_keys = p.n_keys;
  const float* cr = p.cos_t + static_cast<int64_t>(p.rope_pos) * D;
  const float* sr = p.sin_t + static_cast<int64_t>(p.rope_pos) * D;
  float* qs = xs;                 // [G][128] query heads of the group, normalised and rotated
  float* pm = qs + G * D;         // [LL_WARPS][G] running maxima of the warps
  float* pl = pm + LL_WARPS * G;  // sums
  float* po = pl + LL_WARPS * G;  // [LL_WARPS][G][128] unnormalised outputs
  ll_trace(p, tr);
  for (int u = blockIdx.x; u < units; u += gridDim.x) {
    const int chunk = u % p.chunks;
    const int bk = u / p.chunks;
    const int b = bk / p.kv_heads, kvh = bk - b * p.kv_heads;
    const uint2* row = p.ll_qkv + static_cast<int64_t>(b) * qkv_w;
    const int k_begin = chunk * p.keys_per_chunk;
    int k_end = k_begin + p.keys_per_chunk;
    if (k_end > n_keys) k_end = n_keys;
    const bool holds_new = k_begin <= p.pos && p.pos < k_end;
    if (warp < G || (warp == G && holds_new)) {
      // warp < G: query head kvh * G + warp; warp == G: the key and the value of this step's token
      const uint2* src = warp < G ? row + (kvh * G + warp) * D : row + (p.heads + kvh) * D;
      const uint2* src2 = row + (p.heads + p.kv_heads + kvh) * D;  // (value: only warp G)
      uint2 a[4], v2[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        a[i] = ll_ld1(src + lane + 32 * i);
        v2[i] = warp == G ? ll_ld1(src2 + lane + 32 * i) : make_uint2(0u, qkv_tag);
      }
      const long long t0 = clock64();
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        int spins = 0;
        while (a[i].y != qkv_tag) {
          if (ll_expired(p, &S.abort_word, t0, spins++)) break;
          a[i] = ll_ld1(src + lane + 32 * i);
        }
        spins = 0;
        while (v2[i].y != qkv_tag) {
          if (ll_expired(p, &S.abort_word, t0, spins++)) break;
          v2[i] = ll_ld1(src2 + lane + 32 * i);
        }
      }
      float x[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) x[i] = __uint_as_float(a[i].x);
      ds_norm_rope(x, warp < G ? W.q_norm : W.k_norm, cr, sr, p.eps, lane);
      if (warp < G) {
#pragma unroll
        for (int i = 0; i < 4; ++i) qs[warp * D + lane + 32 * i] = x[i];
      } else {
        float* kdst = kc + ((static_cast<int64_t>(b) * p.kv_heads + kvh) * p.max_pos + p.pos) * D;
        float* vdst = vc + ((static_cast<int64_t>(b) * p.kv_heads + kvh) * p.max_pos + p.pos) * D;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          kdst[lane + 32 * i] = x[i];
          vdst[lane + 32 * i] = __uint_as_float(v2[i].x);
        }
      }
    }
    ll_sync();
    if (*reinterpret_cast<volatile int*>(&S.abort_word)) return false;
    ll_trace(p, tr);
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
    // scores: 8 lanes share a key (16 of its 128 values each); a warp takes DS_KB keys per step (see decode_step.cuh)
    const int j8 = lane & 7, kq = lane >> 3;
    float4 qreg[G][4];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int i = 0; i < 4; ++i) qreg[g][i] = *reinterpret_cast<const float4*>(&qs[g * D + (j8 + 8 * i) * 4]);
    for (int key0 = k_begin + warp * DS_KB; key0 < k_end; key0 += LL_WARPS * DS_KB) {
      float sc[G][DS_KB / 4];
      float4 vv[DS_KB];
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
        const float m_new = fmaxf(m_run[g], mx);
        const float alpha = __expf(m_run[g] - m_new);
        float sum = 0.f;
#pragma unroll
        for (int kg = 0; kg < DS_KB / 4; ++kg) {
          sc[g][kg] = __expf(sc[g][kg] - m_new);
          sum += sc[g][kg];
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 8);
        sum += __shfl_xor_sync(0xffffffffu, sum, 16);
        l_run[g] = l_run[g] * alpha + sum;
        m_run[g] = m_new;
        acc[g].x *= alpha;
        acc[g].y *= alpha;
        acc[g].z *= alpha;
        acc[g].w *= alpha;
      }
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
    ll_sync();
    ll_trace(p, tr);
    uint2* att_row = p.ll_att + static_cast<int64_t>(b) * attn_w;
    if (warp < G) {
      // warp g combines the 8 warps' results of query head g
      const int g = warp;
      const float mw = lane < LL_WARPS ? pm[lane * G + g] : -CUDART_INF_F;
      const float lw = lane < LL_WARPS ? pl[lane * G + g] : 0.f;
      float m = ds_warp_max(mw);
      const float fw = (mw == -CUDART_INF_F) ? 0.f : __expf(mw - m);
      float lsum = ds_warp_sum(lw * fw);
      float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
      for (int w = 0; w < LL_WARPS; ++w) {
        const float f = __shfl_sync(0xffffffffu, fw, w);
        const float4 ow = *reinterpret_cast<const float4*>(&po[(w * G + g) * D + lane * 4]);
        o.x = fmaf(ow.x, f, o.x);
        o.y = fmaf(ow.y, f, o.y);
        o.z = fmaf(ow.z, f, o.z);
        o.w = fmaf(ow.w, f, o.w);
      }
      // partial results of the other chunks travel as pairs: [m, l, o[128]] per (chunk, head)
      constexpr int PW = 2 + D;
      uint2* pbase = p.ll_part + (static_cast<int64_t>(bk) * DS_MAX_CHUNKS_LL * G + g) * PW;
      const int64_t cs = static_cast<int64_t>(G) * PW;
      if (chunk != 0) {
        uint2* dst = pbase + chunk * cs;
        if (lane == 0) {
          ll_st(dst, m, att_tag);
          ll_st(dst + 1, lsum, att_tag);
        }
        ll_st(dst + 2 + lane * 4, o.x, att_tag);
        ll_st(dst + 2 + lane * 4 + 1, o.y, att_tag);
        ll_st(dst + 2 + lane * 4 + 2, o.z, att_tag);
        ll_st(dst + 2 + lane * 4 + 3, o.w, att_tag);
      } else {
        // chunk 0 of a (sequence, kv head) collects the other chunks (an online softmax over the chunks) and stores the
        // attention output; CB chunks are requested together
        constexpr int CB = 4;
        const long long t0 = clock64();
        for (int cb = 1; cb < p.chunks; cb += CB) {
          uint2 hm[CB], hl[CB];
          uint4 oa[CB], ob[CB];
#pragma unroll
          for (int c2 = 0; c2 < CB; ++c2) {
            if (cb + c2 < p.chunks) {
              const uint2* src = pbase + (cb + c2) * cs;
              hm[c2] = ll_ld1(src);
              hl[c2] = ll_ld1(src + 1);
              oa[c2] = ll_ld2(src + 2 + lane * 4);
              ob[c2] = ll_ld2(src + 2 + lane * 4 + 2);
            }
          }
#pragma unroll
          for (int c2 = 0; c2 < CB; ++c2) {
            if (cb + c2 < p.chunks) {
              const uint2* src = pbase + (cb + c2) * cs;
              int spins = 0;
              while (hm[c2].y != att_tag || hl[c2].y != att_tag || oa[c2].y != att_tag || oa[c2].w != att_tag ||
                     ob[c2].y != att_tag || ob[c2].w != att_tag) {
                if (ll_expired(p, &S.abort_word, t0, spins++)) break;
                hm[c2] = ll_ld1(src);
                hl[c2] = ll_ld1(src + 1);
                oa[c2] = ll_ld2(src + 2 + lane * 4);
                ob[c2] = ll_ld2(src + 2 + lane * 4 + 2);
              }
              const float mc = __uint_as_float(hm[c2].x), lc = __uint_as_float(hl[c2].x);
              const float m_new = fmaxf(m, mc);
              const float fa = (m == -CUDART_INF_F) ? 0.f : __expf(m - m_new);
              const float fb = (mc == -CUDART_INF_F) ? 0.f : __expf(mc - m_new);
              lsum = lsum * fa + lc * fb;
              o.x = o.x * fa + __uint_as_float(oa[c2].x) * fb;
              o.y = o.y * fa + __uint_as_float(oa[c2].z) * fb;
              o.z = o.z * fa + __uint_as_float(ob[c2].x) * fb;
              o.w = o.w * fa + __uint_as_float(ob[c2].z) * fb;
              m = m_new;
            }
          }
        }
        const float inv = lsum > 0.f ? 1.0f / lsum : 0.f;
        uint2* d = att_row + (kvh * G + g) * D + lane * 4;
        ll_st(d, o.x * inv, att_tag);
        ll_st(d + 1, o.y * inv, att_tag);
        ll_st(d + 2, o.z * inv, att_tag);
        ll_st(d + 3, o.w * inv, att_tag);
      }
    }
    ll_sync();  // the scratch is reused by this CTA's next unit
    ll_trace(p, tr);
  }
  return true;
}

template <int MT, int G>
__global__ void __launch_bounds__(LL_THREADS, 1) decode_ll_kernel(const DecodeStepParams p) {
  extern __shared__ __align__(128) char dw_smem[];
  // layout: DwShared | red [4][8] | x_own [4][LL_MAX_OWN] | part | xs | ring
  DwShared& S = *reinterpret_cast<DwShared*>(dw_smem);
  float* red = reinterpret_cast<float*>(dw_smem + ((sizeof(DwShared) + 127) / 128) * 128);
  float* x_own = red + 32;  // (red holds up to 8 warps x 4 sequences)
  float* part = x_own + 4 * LL_MAX_OWN;  // partial sums of the warps [LL_WARPS][LL_GROUP][16][MT]
  float* xs = part + ll_part_floats(MT);
  char* ring = reinterpret_cast<char*>(xs) + p.dw_xs_bytes;
  constexpr int D = 128;
  const int B = p.B, H = p.hidden;
  const int qkv_w = (p.heads + 2 * p.kv_heads) * D;
  const int attn_w = p.heads * D;

  if (threadIdx.x == 0) {
    S.abort_word = 0;
    S.issued = 0;
    S.consumed = 0;
    S.issuer_done = 0;
    S.nslot = p.dw_nslot;
    for (int s = 0; s < DW_MAX_SLOTS; ++s) {
      mbar_init(&S.full[s], 1);
      S.done[s] = 0;
    }
    fence_mbar_init();
    const int rows_of[DW_KINDS] = {qkv_w, H, p.inter, H, p.vocab_rows};
    const int k_of[DW_KINDS] = {H, attn_w, H, p.inter, H};
    const int G_ = static_cast<int>(gridDim.x), b = static_cast<int>(blockIdx.x);
    int per_layer = 0;
    for (int kd = 0; kd < DW_KINDS; ++kd) {
      DwPhase ph;
      ph.K = k_of[kd];
      ph.r0 = static_cast<int>(static_cast<int64_t>(rows_of[kd]) * b / G_);
      ph.rows = static_cast<int>(static_cast<int64_t>(rows_of[kd]) * (b + 1) / G_) - ph.r0;
      ph.rpc = DW_CHUNK / (ph.K * (kd == 2 ? 4 : 2));
      const int cap = kd == 2 ? 8 : 16;  // a chunk is one 16-row operand of the tensor-core linear phase
      if (ph.rpc > cap) ph.rpc = cap;
      ph.nchunks = (ph.rows + ph.rpc - 1) / ph.rpc;
      S.ph[kd] = ph;
      if (kd < 4) per_layer += ph.nchunks;
    }
    S.per_layer = per_layer;
    S.total = per_layer * p.layers + S.ph[4].nchunks;
    dw_fill_desc(S, p);
  }
  if (threadIdx.x < 32) red[threadIdx.x] = 0.f;  // [4 sequences][8]: the entries of warps that do not exist stay zero
  for (int i = threadIdx.x; i < p.layers; i += LL_THREADS) {
    const DsLayer W = p.lw[i];
    S.w[i][0] = W.qkv;
    S.w[i][1] = W.o;
    S.w[i][2] = W.gate_up;
    S.w[i][3] = W.down;
    S.nw[i][0] = W.q_norm;
    S.nw[i][1] = W.k_norm;
    S.nw[i][2] = W.norm1;
    S.nw[i][3] = W.norm2;
  }
  __syncthreads();  // (the only synchronisation of all nine warps)
  // K / V rows of this CTA's first attention unit: the issuing lane asks for them into the L2 (one bulk prefetch each
  // per layer) when it starts on the layer's weights, most of a layer ahead of the attention phase
  uint32_t kv_bytes = 0;
  int64_t kv_off = 0;
  if (static_cast<int>(blockIdx.x) < B * p.kv_heads * p.chunks) {
    const int chunk = blockIdx.x % p.chunks, bk = blockIdx.x / p.chunks;
    const int k_begin = chunk * p.keys_per_chunk;
    int k_end = k_begin + p.keys_per_chunk;
    if (k_end > p.n_keys) k_end = p.n_keys;
    kv_off = (static_cast<int64_t>(bk) * p.max_pos + k_begin) * D;
    kv_bytes = k_end > k_begin ? static_cast<uint32_t>(k_end - k_begin) * D * 4u : 0u;
  }
  if (threadIdx.x >= LL_WORKERS) {
    // The issuing warp: one lane keeps the ring full. Chunk number n may be issued once chunk n - nslot has been
    // consumed (the workers publish the count after the synchronisation that ends a group of chunks), so the copies
    // run ahead of the phases by the depth of the ring and never sit on a worker's critical path.
    if (threadIdx.x == LL_WORKERS) {
      DwIssuer iss{0, 0, 0, 0};
      const long long t0 = clock64();
      long long last = t0;
      int pf_layer = 0;  // next layer whose K / V rows have not been asked for
      while (iss.next < S.total) {
        if (*reinterpret_cast<volatile int*>(&S.abort_word)) break;
        if (kv_bytes && pf_layer < p.layers && iss.next >= pf_layer * S.per_layer) {
          const float* kr = p.k_cache + static_cast<size_t>(pf_layer) * p.cache_layer + kv_off;
          const float* vr = p.v_cache + static_cast<size_t>(pf_layer) * p.cache_layer + kv_off;
          asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(kr), "r"(kv_bytes) : "memory");
          asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(vr), "r"(kv_bytes) : "memory");
          ++pf_layer;
        }
        const int consumed = *reinterpret_cast<volatile int*>(&S.consumed);
        if (iss.next < consumed + S.nslot) {
          dw_issue_next(S, p, ring, iss);
          last = clock64();
        } else if (clock64() - last > p.wait_cycles) {  // the workers are stuck: they will have raised the status
          break;
        }
      }
      *reinterpret_cast<volatile int*>(&S.issuer_done) = 1;
    }
    return;
  }
  int c = 0, slot = 0, tr = 0;
  unsigned int parity = 0;

  // ---- embedding: every CTA gathers the rows itself (nothing to wait for): xs = x * norm1 of layer 0, the sums of
  // squares go to `red`, and the CTA's own rows of x go to x_own
  {
    const DwPhase own = S.ph[1];
    const float* g0 = p.lw[0].norm1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int b = 0; b < MT; ++b) {
      float ss = 0.f;
      if (b < B) {
        int id = p.ids[b];
        id = id < 0 ? 0 : (id >= p.vocab ? p.vocab - 1 : id);
        const uint16_t* erow = p.embed + static_cast<int64_t>(id) * H;
        for (int i = threadIdx.x * 2; i < H; i += 2 * LL_WORKERS) {
          const uint32_t w = __ldg(reinterpret_cast<const uint32_t*>(erow + i));
          const float2 g = __ldg(reinterpret_cast<const float2*>(g0 + i));
          const float a = __uint_as_float(w << 16), c2 = __uint_as_float(w & 0xFFFF0000u);
          ss = fmaf(a, a, ss);
          ss = fmaf(c2, c2, ss);
          uint32_t hi, lo;
          ds_split2(a * g.x, c2 * g.y, hi, lo);
          uint32_t* pl = reinterpret_cast<uint32_t*>(xs) + ((2 * b) * ll_row_floats(H) + i) / 2;
          pl[0] = hi;
          pl[ll_row_floats(H) / 2] = lo;
          if (i >= own.r0 && i < own.r0 + own.rows) x_own[b * LL_MAX_OWN + i - own.r0] = a;
          if (i + 1 >= own.r0 && i + 1 < own.r0 + own.rows) x_own[b * LL_MAX_OWN + i + 1 - own.r0] = c2;
        }
      }
      ss = ds_warp_sum(ss);
      if (lane == 0) red[b * 8 + warp] = ss;
    }
    ll_sync();
  }

  // One loop body serves every phase (the functions are inlined exactly once: a call through the ABI with this
  // many live registers costs more than the phase's arithmetic).
  const int n_phases = 5 * p.layers + 1;
  unsigned int t = p.ll_base + 1;  // tag of the qkv phase of layer 0
  int l = 0, sub = 0;
  for (int phase = 0; phase < n_phases; ++phase) {
    bool ok;
    if (sub == 1) {
      DsLayer W;  // (the pointers come from the table in shared memory: no trip to global memory)
      W.q_norm = S.nw[l][0];
      W.k_norm = S.nw[l][1];
      float* kc = p.k_cache + static_cast<size_t>(l) * p.cache_layer;
      float* vc = p.v_cache + static_cast<size_t>(l) * p.cache_layer;
      ok = ll_attention<G>(p, S, W, kc, vc, xs, t, t + 1, tr);
    } else {
      int kind, stage, epi, ld;
      const uint2* src;
      uint2* dst;
      const float* nw = nullptr;
      unsigned int st, dt;
      if (phase == n_phases - 1) {  // logits = rmsNorm(x) . Wvocab^T
        kind = 4; stage = 0; src = p.ll_x; st = t - 1; nw = p.final_norm; epi = 3; dst = nullptr; dt = 0u; ld = p.vocab_rows;
      } else if (sub == 0) {        // qkv = rmsNorm(x) . Wqkv^T (layer 0: x is the embedding staged above)
        kind = 0; stage = l == 0 ? 3 : 0; src = p.ll_x; st = t - 1; nw = S.nw[l][2]; epi = 0; dst = p.ll_qkv; dt = t; ld = qkv_w;
      } else if (sub == 2) {        // x += attn . Wo^T
        kind = 1; stage = 1; src = p.ll_att; st = t + 1; epi = 1; dst = p.ll_x; dt = t + 2; ld = H;
      } else if (sub == 3) {        // act = swish(gate) * up
        kind = 2; stage = 0; src = p.ll_x; st = t + 2; nw = S.nw[l][3]; epi = 2; dst = p.ll_act; dt = t + 3; ld = p.inter;
      } else {                      // x += act . Wdown^T
        kind = 3; stage = 1; src = p.ll_act; st = t + 3; epi = 1; dst = p.ll_x; dt = t + 4; ld = H;
      }
      ok = ll_linear<MT>(p, S, ring, xs, red, x_own, part, kind, stage, src, st, nw, epi, dst, dt, p.logits, ld, c, slot, parity,
                         tr);
    }
    if (!ok) {
      // give up: raise the status, stop everyone, and wait (bounded) for the copies still on their way into this CTA's
      // shared memory once the issuing warp has stopped
      *reinterpret_cast<volatile int*>(&S.abort_word) = 1;
      ll_sync();
      if (threadIdx.x == 0) {
        atomicExch(p.status, YTC_TIMEOUT);
        atomicOr(p.sync, 0x80000000u);
        const long long t0 = clock64();
        while (!*reinterpret_cast<volatile int*>(&S.issuer_done) && clock64() - t0 < p.wait_cycles) {
        }
        const int issued = *reinterpret_cast<volatile int*>(&S.issued);
        int dummy = 0;
        for (int x = c; x < issued; ++x)
          mbar_wait_limit(&S.full[x % S.nslot], static_cast<uint32_t>((x / S.nslot) & 1), &dummy, p.wait_cycles);
      }
      ll_sync();
      return;
    }
    if (++sub == 5) {
      sub = 0;
      ++l;
      t += 5;
    }
  }
}

}  // namespace ytk
