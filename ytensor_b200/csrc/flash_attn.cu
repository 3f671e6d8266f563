// Scaled dot-product attention forward for the YTensor device backend.
//
//  * flash_tc_kernel  : bf16 / fp16, head_dim == value_dim in {64, 128}. One CTA works on TWO 128-row query
//                       tiles that share the same K/V stream (two query heads of one GQA group, or two
//                       neighbouring row blocks of one head). Warp 0 feeds shared memory with TMA, warp 1
//                       issues tcgen05.mma: S_t = Q_t K^T into tensor memory, and O_t += P_t V with P_t read
//                       straight from tensor memory. Two softmax warpgroups (one per tile, one thread per
//                       query row) turn S into P with an online softmax kept in registers: running maximum
//                       and sum in the log2 domain, exp2 with the scale folded in, and O rescaled only when
//                       the maximum has grown by more than 2^8. While one warpgroup does softmax, the tensor
//                       core works on the other tile.
//  * attn_simt_kernel : any dtype (fp32 included), any head / value dim, one warp per query row. The
//                       catch-all for shapes the tensor-core kernel does not take.
//
// Both honour: no mask / causal window anchored at the end of the keys / a bool mask [q_len, kv_len];
// an optional additive fp32 bias [q_len, kv_len]; rows that see no key produce zeros.
// Replaces yt::function::scaledDotProductAttention and yt::kernel::avx2::flash_attention
// (reference src/function/ops.inl:109-234,368-425, src/kernel/avx2/flash_attention.inl:202-443).
#include <math_constants.h>

#include <atomic>
#include <type_traits>

#include "ptx_sm100.cuh"
#include "ytc_common.cuh"

namespace ytk {

constexpr int FA_BM = 128;      // query rows per tile
constexpr int FA_BN = 128;      // keys per K/V tile
constexpr int FA_STAGES = 2;    // K/V ring depth
constexpr int FA_THREADS = 384; // 4 service warps + 2 softmax warpgroups
constexpr float FA_LOG2E = 1.4426950408889634f;
constexpr float FA_RESCALE_THRESHOLD = 8.0f;  // log2 units

struct FlashParams {
  void* O;
  int64_t o_sb, o_sh, o_sr;  // output strides (elements): batch, head, row; unit stride on the value dim
  const uint8_t* mask;       // bool mask [q_len, kv_len] or null
  int64_t mask_rs;
  const float* bias;         // additive bias [q_len, kv_len] or null
  int64_t bias_rs, bias_cs;
  int batch, kv_heads, groups, q_len, kv_len;
  int causal;                // 1: key c visible to row r iff c <= r + causal_off
  int causal_off;
  float scale_log2;          // scale * log2(e)
  int is_bf16;
  int pair_heads;            // 1: the two tiles are two heads of one group; 0: two neighbouring row blocks
  int row_blocks;            // query row blocks (of one tile with head pairs, of two tiles otherwise)
  int head_slots;            // head pairs (pair_heads) or heads
  int items_per_row_block;   // head_slots * batch
  int n_items;               // row_blocks * items_per_row_block
  uint32_t idesc_s, idesc_pv;
  int* status;
};

// 2^x by the special-function unit (ex2.approx.ftz): -inf gives 0, relative error about 2^-22.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Packed pairs of fp32 (sm_100 f32x2 arithmetic) and the three-input maximum: they halve the instruction count of
// the softmax inner loops, which share their issue slots with the MMA and TMA warps.
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// 2^x for a packed pair on the FMA pipe instead of the special-function unit. That unit retires one ex2 warp
// instruction per 8 cycles and scheduler (16 results per clock and SM), so the 2 x 128 x 128 exponentials of one
// iteration keep it busy for as long as the tensor pipe needs for the four MMAs of the same iteration; the 16-bit
// pack runs there as well. A quarter of the pairs is the measured optimum: the FMA and ALU pipes are nearly as full.
// The method: round x to the nearest integer n with the 1.5 * 2^23
// trick, evaluate a cubic minimax polynomial of 2^f on f = x - n in [-0.5, 0.5] (relative error 7.5e-5, well under
// the rounding of the 16-bit P), and add n to the exponent field. x is clamped at -126 (the result is then ~1e-38
// instead of 0).
#ifndef FA_EMU_EVERY
#define FA_EMU_EVERY 4  // every FA_EMU_EVERY-th pair of a full tile takes this path; 0 switches it off
#endif
__device__ __forceinline__ void exp2_emu2(uint64_t x2, float& p0, float& p1) {
  constexpr float MAGIC = 12582912.f;  // 1.5 * 2^23
  float x0, x1;
  f2_unpack(x2, x0, x1);
  x0 = fmaxf(x0, -126.f);
  x1 = fmaxf(x1, -126.f);
  const uint64_t xc = f2_pack(x0, x1);
  const uint64_t t2 = f2_add(xc, f2_pack(MAGIC, MAGIC));
  const uint64_t j2 = f2_add(t2, f2_pack(-MAGIC, -MAGIC));
  const uint64_t f2 = f2_fma(j2, f2_pack(-1.f, -1.f), xc);
  uint64_t q2 = f2_fma(f2_pack(0.0551716685f, 0.0551716685f), f2, f2_pack(0.242611125f, 0.242611125f));
  q2 = f2_fma(q2, f2, f2_pack(0.693260968f, 0.693260968f));
  q2 = f2_fma(q2, f2, f2_pack(0.999928057f, 0.999928057f));
  float t0, t1, q0, q1;
  f2_unpack(t2, t0, t1);
  f2_unpack(q2, q0, q1);
  p0 = __int_as_float(__float_as_int(q0) + (__float_as_int(t0) << 23));
  p1 = __int_as_float(__float_as_int(q1) + (__float_as_int(t1) << 23));
}

template <int D>
struct FaSmem {
  static constexpr int TILE_BYTES = FA_BM * D * 2;  // one Q / K / V tile
  static constexpr int Q_OFF = 0;
  static constexpr int KV_OFF = 2 * TILE_BYTES;
  static constexpr int BAR_OFF = KV_OFF + FA_STAGES * 2 * TILE_BYTES;
  // q_full, k_full[2], v_full[2], kv_empty[2], s_full[2], p_full[2], o_ready[2], q_free, o_free[2], p_half[2],
  // tmem slot, abort
  static constexpr int NBAR = 1 + 3 * FA_STAGES + 6 + 3 + 2;
  static constexpr int TOTAL = BAR_OFF + NBAR * 8 + 16;
  static constexpr int DYN_BYTES = TOTAL + 1024;
};

// Loads one [128 x D] tile as D/64 boxes of [128 rows x 128 bytes] (128-byte swizzle).
template <int D>
__device__ __forceinline__ void fa_load_tile(uint8_t* dst, const CUtensorMap* m, uint64_t* bar, int row, int head,
                                             int batch) {
#pragma unroll
  for (int c = 0; c < D / 64; ++c) tma_load_4d(dst + c * (FA_BM * 128), m, bar, c * 64, row, head, batch);
}

// Work item = one pair of query tiles (see the file header). The CTAs are persistent: CTA c handles items c,
// c + gridDim.x, ... of a list sorted by decreasing length (long causal row blocks first), so that the Q load and the
// first K/V loads of the next item, and the S MMAs of its first tiles, overlap the last softmax, P.V and the epilogue
// of the current one.
struct FaItem {
  int q_head[2], q_row0[2], kv_head, b;
  bool tile_on[2];
  int n_tiles[2], n_max;
};

__device__ __forceinline__ FaItem fa_decode_item(const FlashParams& p, int w) {
  FaItem it;
  const int per_rb = p.items_per_row_block;
  const int rb = p.row_blocks - 1 - w / per_rb;  // last row block first
  const int rest = w - (w / per_rb) * per_rb;
  const int hsel = rest % p.head_slots;
  it.b = rest / p.head_slots;
  if (p.pair_heads) {
    const int heads = p.kv_heads * p.groups;
    it.q_head[0] = hsel * 2;
    it.q_head[1] = hsel * 2 + 1;
    if (it.q_head[1] >= heads) it.q_head[1] = it.q_head[0];
    it.q_row0[0] = it.q_row0[1] = rb * FA_BM;
    it.kv_head = it.q_head[0] / p.groups;
  } else {
    it.q_head[0] = it.q_head[1] = hsel;
    it.q_row0[0] = rb * 2 * FA_BM;
    it.q_row0[1] = rb * 2 * FA_BM + FA_BM;
    it.kv_head = hsel / p.groups;
  }
  it.tile_on[0] = it.q_row0[0] < p.q_len;
  it.tile_on[1] = it.q_row0[1] < p.q_len && !(p.pair_heads && it.q_head[1] == it.q_head[0]);
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    int last_key = p.kv_len - 1;
    if (p.causal) {
      const int lim = it.q_row0[t] + FA_BM - 1 + p.causal_off;
      if (lim < last_key) last_key = lim;
    }
    it.n_tiles[t] = (!it.tile_on[t] || last_key < 0) ? 0 : last_key / FA_BN + 1;
  }
  it.n_max = it.n_tiles[0] > it.n_tiles[1] ? it.n_tiles[0] : it.n_tiles[1];
  return it;
}

template <int D>
__global__ void __launch_bounds__(FA_THREADS, 1)
    flash_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const FlashParams p) {
  using S = FaSmem<D>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::BAR_OFF);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* v_full = k_full + FA_STAGES;
  uint64_t* kv_empty = v_full + FA_STAGES;
  uint64_t* s_full = kv_empty + FA_STAGES;
  uint64_t* p_full = s_full + 2;
  uint64_t* o_ready = p_full + 2;
  uint64_t* q_free = o_ready + 2;   // the MMAs no longer read the Q tiles of the current item
  uint64_t* o_free = q_free + 1;    // [2] the epilogue has read O_t
  uint64_t* p_half = o_free + 2;    // [2] the first 64 keys' columns of P_t are in tensor memory
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(p_half + 2);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_free, 1);
    for (int s = 0; s < FA_STAGES; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&s_full[t], 1);
      mbar_init(&p_full[t], 4);  // one arrival per softmax warp
      mbar_init(&p_half[t], 4);
      mbar_init(&o_ready[t], 1);
      mbar_init(&o_free[t], 4);
    }
    *abort_word = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // tensor-memory columns: S0/P0 at 0, S1/P1 at 128, O0 at 256, O1 at 384
  const uint32_t t_s[2] = {tmem_base, tmem_base + 128u};
  const uint32_t t_o[2] = {tmem_base + 256u, tmem_base + 384u};

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int kv_cnt = 0;  // K/V tiles loaded so far: stage kv_cnt % 2, fill number kv_cnt / 2
      bool ok = true;
      int n_item = 0;
      for (int w = blockIdx.x; ok && w < p.n_items; w += gridDim.x) {
        const FaItem it = fa_decode_item(p, w);
        if (it.n_max == 0) continue;  // nothing visible: the softmax warpgroups write zeros on their own
        // (n_item counts only items with work; items without work touch no barrier in any role)
        if (n_item > 0 && !mbar_wait(q_free, static_cast<uint32_t>((n_item - 1) & 1), abort_word)) break;
        int n_q = 0;
        for (int t = 0; t < 2; ++t) n_q += it.tile_on[t] ? 1 : 0;
        mbar_expect_tx(q_full, static_cast<uint32_t>(n_q) * S::TILE_BYTES);
        for (int t = 0; t < 2; ++t)
          if (it.tile_on[t])
            fa_load_tile<D>(smem + S::Q_OFF + t * S::TILE_BYTES, &tmQ, q_full, it.q_row0[t], it.q_head[t], it.b);
        for (int j = 0; j < it.n_max; ++j, ++kv_cnt) {
          const int s = kv_cnt % FA_STAGES;
          if (!mbar_wait(&kv_empty[s], static_cast<uint32_t>(((kv_cnt / FA_STAGES) & 1) ^ 1), abort_word)) {
            ok = false;
            break;
          }
          uint8_t* ks = smem + S::KV_OFF + s * 2 * S::TILE_BYTES;
          uint8_t* vs = ks + S::TILE_BYTES;
          mbar_expect_tx(&k_full[s], S::TILE_BYTES);
          fa_load_tile<D>(ks, &tmK, &k_full[s], j * FA_BN, it.kv_head, it.b);
          mbar_expect_tx(&v_full[s], S::TILE_BYTES);
          fa_load_tile<D>(vs, &tmV, &v_full[s], j * FA_BN, it.kv_head, it.b);
        }
        ++n_item;
      }
      if (!ok) {
        // bounded drain of the copies still in flight
        const long long t0 = clock64();
        for (int s = 0; s < FA_STAGES && s < kv_cnt; ++s)
          while (!mbar_try_wait(&v_full[s], 0) && !mbar_try_wait(&v_full[s], 1) && clock64() - t0 < 20000000ll) {
          }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t q_base = smem_u32(smem + S::Q_OFF);
      int kv_cnt = 0;
      int p_cnt[2] = {0, 0};    // P tiles consumed so far per query tile (phase of p_full)
      int e_cnt[2] = {0, 0};    // items finished per query tile (phase of o_free)
      // S_t = Q_t . K^T : both operands K-major, D/16 steps; 64-element chunks are FA_BM*128 bytes apart
      auto issue_s = [&](int t, int stage) {
        const uint32_t qa = q_base + t * S::TILE_BYTES;
        const uint32_t ka = smem_u32(smem + S::KV_OFF + stage * 2 * S::TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * (FA_BM * 128) + (kk & 3) * 32;
          tc_mma_f16(t_s[t], umma_smem_desc_sw128(qa + off, 16, 1024), umma_smem_desc_sw128(ka + off, 16, 1024),
                     p.idesc_s, kk != 0 ? 1u : 0u);
        }
        tc_commit(&s_full[t]);
      };
      // O_t (+)= P_t . V : A = P from tensor memory (16-bit pairs, 8 columns per 16 keys),
      // B = V, unit stride along the value dim (MN-major): 16 keys = 2048 bytes, 64-wide chunks 16 KiB apart
      // O_t (+)= P_t V in two halves of 64 keys: the first is issued as soon as the softmax warps have published the
      // first half of P, while they still compute the second.
      auto issue_pv = [&](int t, int stage, bool accumulate, int half) {
        const uint32_t va = smem_u32(smem + S::KV_OFF + stage * 2 * S::TILE_BYTES + S::TILE_BYTES);
#pragma unroll
        for (int kk = half * (FA_BN / 32); kk < (half + 1) * (FA_BN / 32); ++kk)
          tc_mma_f16_ts(t_o[t], t_s[t] + kk * 8, umma_smem_desc_sw128(va + kk * 2048, FA_BM * 128, 1024), p.idesc_pv,
                        (accumulate || kk != 0) ? 1u : 0u);
        if (half == 1) tc_commit(&o_ready[t]);
      };
      bool ok = true;
      int n_item = 0;
      for (int w = blockIdx.x; ok && w < p.n_items; w += gridDim.x) {
        const FaItem it = fa_decode_item(p, w);
        if (it.n_max == 0) continue;
        if (!mbar_wait(q_full, static_cast<uint32_t>(n_item & 1), abort_word)) break;
        if (!mbar_wait(&k_full[kv_cnt % FA_STAGES], static_cast<uint32_t>((kv_cnt / FA_STAGES) & 1), abort_word)) break;
        tc_fence_after();
        if (it.n_tiles[0] > 0) issue_s(0, kv_cnt % FA_STAGES);
        if (it.n_tiles[1] > 0) issue_s(1, kv_cnt % FA_STAGES);
        if (it.n_max == 1) tc_commit(q_free);
        for (int j = 0; j < it.n_max && ok; ++j, ++kv_cnt) {
          const int s = kv_cnt % FA_STAGES;
          const int sn = (kv_cnt + 1) % FA_STAGES;
          const uint32_t ph = static_cast<uint32_t>((kv_cnt / FA_STAGES) & 1);
          const uint32_t ph_next = static_cast<uint32_t>(((kv_cnt + 1) / FA_STAGES) & 1);
          if (!mbar_wait(&v_full[s], ph, abort_word)) {
            ok = false;
            break;
          }
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            if (j < it.n_tiles[t]) {
              if (!mbar_wait(&p_half[t], static_cast<uint32_t>(p_cnt[t] & 1), abort_word)) {
                ok = false;
                break;
              }
              if (j == 0 && e_cnt[t] > 0 &&
                  !mbar_wait(&o_free[t], static_cast<uint32_t>((e_cnt[t] - 1) & 1), abort_word)) {
                ok = false;  // the first P.V of an item overwrites O_t: the previous epilogue must have read it
                break;
              }
              tc_fence_after();
              issue_pv(t, s, j > 0, 0);
              if (!mbar_wait(&p_full[t], static_cast<uint32_t>(p_cnt[t] & 1), abort_word)) {
                ok = false;
                break;
              }
              ++p_cnt[t];
              tc_fence_after();
              issue_pv(t, s, j > 0, 1);
            }
            if (j + 1 < it.n_tiles[t]) {
              if (!mbar_wait(&k_full[sn], ph_next, abort_word)) {
                ok = false;
                break;
              }
              tc_fence_after();
              issue_s(t, sn);
            }
          }
          if (!ok) break;
          if (j + 2 == it.n_max) tc_commit(q_free);  // the last S MMAs of this item have been issued
          tc_commit(&kv_empty[s]);  // every MMA that read stage s has been issued before this point
        }
        for (int t = 0; t < 2; ++t)
          if (it.n_tiles[t] > 0) ++e_cnt[t];
        ++n_item;
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------ softmax warpgroups (one per query tile)
    const int t = (warp - 4) >> 2;
    const int q = warp & 3;
    const int row_in_tile = q * 32 + lane;
    const uint32_t lane_sel = static_cast<uint32_t>(q * 32) << 16;
    const uint32_t ts = t_s[t] + lane_sel, to = t_o[t] + lane_sel;
    const bool elementwise_mask = (p.mask != nullptr) || (p.bias != nullptr);
    int s_base = 0;  // S tiles (= P tiles = P.V products) of this query tile in earlier items
    bool ok = true;
    for (int w = blockIdx.x; ok && w < p.n_items; w += gridDim.x) {
      const FaItem it = fa_decode_item(p, w);
      const int* q_row0 = it.q_row0;
      const int* q_head = it.q_head;
      const bool* tile_on = it.tile_on;
      const int b = it.b;
      const int row = q_row0[t] + row_in_tile;  // global query row
      const int nt = (it.n_max == 0) ? 0 : it.n_tiles[t];
      const int o_base = s_base;
      float m_run = -CUDART_INF_F;  // running maximum, log2 domain
      float l_run = 0.f;

      for (int j = 0; j < nt; ++j) {
        if (!mbar_wait(&s_full[t], static_cast<uint32_t>((s_base + j) & 1), abort_word)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const int key0 = j * FA_BN;
        // Three kinds of tile: `full` (every key visible to every row), limited (visibility is "key <= per-row
        // limit": causal diagonal, end of the keys, rows past q_len), general (bool mask or bias present).
        int row_limit = (row < p.q_len) ? p.kv_len - 1 : -1;
        if (p.causal && row + p.causal_off < row_limit) row_limit = row + p.causal_off;
        const int cl = row_limit - key0;  // columns 0..cl of this tile are visible to this thread's row
        const bool full = !elementwise_mask && (key0 + FA_BN <= p.kv_len) && (q_row0[t] + FA_BM <= p.q_len) &&
                          (!p.causal || key0 + FA_BN - 1 <= q_row0[t] + p.causal_off);
        auto score = [&](uint32_t raw, int c) -> float {  // general tiles only
          float v = __uint_as_float(raw) * p.scale_log2;
          const int key = key0 + c;
          bool vis = c <= cl;
          if (vis && p.mask) vis = p.mask[static_cast<int64_t>(row) * p.mask_rs + key] != 0;
          if (vis && p.bias) v += p.bias[static_cast<int64_t>(row) * p.bias_rs + key * p.bias_cs] * FA_LOG2E;
          return vis ? v : -CUDART_INF_F;
        };
        // pass 1: row maximum. Without mask / bias the maximum is taken over the raw scores (one instruction per
        // element, two with the per-row limit) and scaled afterwards; a negative scale flips max into min.
        float mx = -CUDART_INF_F;
        if (!elementwise_mask) {
          const bool pos = p.scale_log2 >= 0.f;
          const float ident = pos ? -CUDART_INF_F : CUDART_INF_F;
          float a0 = ident, a1 = ident, a2 = ident, a3 = ident;
#pragma unroll 1
          for (int c0 = 0; c0 < FA_BN; c0 += 64) {
            if (!full && __all_sync(0xffffffffu, cl < c0)) continue;  // no row of this warp sees these columns
            uint32_t r[64];
            tmem_ld_32x32b_x64(ts + c0, r);
            tmem_ld_wait();
            if (full && pos) {  // the common tile: one three-input max per two elements, eight independent chains
              float b0 = ident, b1 = ident, b2 = ident, b3 = ident;
#pragma unroll
              for (int e = 0; e < 64; e += 16) {
                a0 = fmax3(a0, __uint_as_float(r[e]), __uint_as_float(r[e + 1]));
                a1 = fmax3(a1, __uint_as_float(r[e + 2]), __uint_as_float(r[e + 3]));
                a2 = fmax3(a2, __uint_as_float(r[e + 4]), __uint_as_float(r[e + 5]));
                a3 = fmax3(a3, __uint_as_float(r[e + 6]), __uint_as_float(r[e + 7]));
                b0 = fmax3(b0, __uint_as_float(r[e + 8]), __uint_as_float(r[e + 9]));
                b1 = fmax3(b1, __uint_as_float(r[e + 10]), __uint_as_float(r[e + 11]));
                b2 = fmax3(b2, __uint_as_float(r[e + 12]), __uint_as_float(r[e + 13]));
                b3 = fmax3(b3, __uint_as_float(r[e + 14]), __uint_as_float(r[e + 15]));
              }
              a0 = fmaxf(a0, b0);
              a1 = fmaxf(a1, b1);
              a2 = fmaxf(a2, b2);
              a3 = fmaxf(a3, b3);
            } else {
              const int cc = full ? 64 : cl - c0;
#pragma unroll
              for (int e = 0; e < 64; e += 4) {
                const float v0 = (e <= cc) ? __uint_as_float(r[e]) : ident;
                const float v1 = (e + 1 <= cc) ? __uint_as_float(r[e + 1]) : ident;
                const float v2 = (e + 2 <= cc) ? __uint_as_float(r[e + 2]) : ident;
                const float v3 = (e + 3 <= cc) ? __uint_as_float(r[e + 3]) : ident;
                if (pos) {
                  a0 = fmaxf(a0, v0); a1 = fmaxf(a1, v1); a2 = fmaxf(a2, v2); a3 = fmaxf(a3, v3);
                } else {
                  a0 = fminf(a0, v0); a1 = fminf(a1, v1); a2 = fminf(a2, v2); a3 = fminf(a3, v3);
                }
              }
            }
          }
          const float ext = pos ? fmaxf(fmaxf(a0, a1), fmaxf(a2, a3)) : fminf(fminf(a0, a1), fminf(a2, a3));
          mx = (ext == ident) ? -CUDART_INF_F : ext * p.scale_log2;
        } else {
#pragma unroll 1
          for (int c0 = 0; c0 < FA_BN; c0 += 32) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(ts + c0, r);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) mx = fmaxf(mx, score(r[e], c0 + e));
          }
        }
        const float m_new = fmaxf(m_run, mx);
        if (j == 0) {
          m_run = m_new;
        } else {
          const bool grow = (m_new - m_run) > FA_RESCALE_THRESHOLD;  // also true when m_run is -inf and m_new finite
          if (__any_sync(0xffffffffu, grow)) {
            // O_t *= 2^(m_run - m_new) for this warp's 32 rows; needs the previous P.V to have landed
            if (!mbar_wait(&o_ready[t], static_cast<uint32_t>((o_base + j - 1) & 1), abort_word)) {
              ok = false;
              break;
            }
            tc_fence_after();
            const float alpha = (m_new == -CUDART_INF_F) ? 1.f : fast_exp2(m_run - m_new);  // m_run == -inf gives 0
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 16) {
              uint32_t r[16];
              tmem_ld_32x32b_x16(to + c0, r);
              tmem_ld_wait();
#pragma unroll
              for (int e = 0; e < 16; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * alpha);
              tmem_st_32x32b_x16(to + c0, r);
            }
            l_run *= alpha;
            m_run = m_new;
          }
        }
        const float m_use = (m_run == -CUDART_INF_F) ? 0.f : m_run;
        // pass 2: P = 2^(s - m), packed to 16 bits, written over the S columns already consumed.
        // Without mask / bias: one FMA and one ex2.approx per element (plus a select on limited tiles).
        float l0 = 0.f, l1 = 0.f;
        const float neg_m = -m_use;
        auto pack2 = [&](float p0, float p1) -> uint32_t {
          if (p.is_bf16) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
            return *reinterpret_cast<const uint32_t*>(&h);
          }
          const __half2 h = __floats2half2_rn(p0, p1);
          return *reinterpret_cast<const uint32_t*>(&h);
        };
        auto publish_half = [&]() {  // columns of P for keys 0..63 are stored: the MMA warp may start P.V on them
          tmem_st_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&p_half[t]);
        };
        if (!elementwise_mask) {
#pragma unroll 1
          for (int c0 = 0; c0 < FA_BN; c0 += 64) {
            uint32_t pk[32];
            // limited tiles: a 64-column half that no row of this warp sees (right of the causal diagonal, past
            // the last key) is written as zeros without reading S or computing exponentials
            const bool dead = !full && __all_sync(0xffffffffu, cl < c0);
            if (dead) {
#pragma unroll
              for (int e = 0; e < 32; ++e) pk[e] = 0u;
            } else {
              uint32_t r[64];
              tmem_ld_32x32b_x64(ts + c0, r);
              tmem_ld_wait();
              const int cc = cl - c0;  // limited tiles: columns 0..cc of this half are visible
              const uint64_t sc2 = f2_pack(p.scale_log2, p.scale_log2), nm2 = f2_pack(neg_m, neg_m);
              uint64_t lacc = f2_pack(0.f, 0.f), lacc2 = f2_pack(0.f, 0.f);
              auto body = [&](auto is_bf, auto is_limited) {
#pragma unroll
                for (int e = 0; e < 64; e += 2) {
                  const uint64_t x2 =
                      f2_fma(f2_pack(__uint_as_float(r[e]), __uint_as_float(r[e + 1])), sc2, nm2);
                  float p0, p1;
                  const bool emu =
                      FA_EMU_EVERY > 0 && ((e >> 1) % (FA_EMU_EVERY > 0 ? FA_EMU_EVERY : 1)) == FA_EMU_EVERY - 1;
                  if (emu) {
                    exp2_emu2(x2, p0, p1);
                  } else {
                    float t0, t1;
                    f2_unpack(x2, t0, t1);
                    p0 = fast_exp2(t0);
                    p1 = fast_exp2(t1);
                  }
                  if (decltype(is_limited)::value) {  // a hidden score may be anything, its P is exactly zero
                    p0 = (e <= cc) ? p0 : 0.f;
                    p1 = (e + 1 <= cc) ? p1 : 0.f;
                  }
                  if (emu) lacc2 = f2_add(lacc2, f2_pack(p0, p1));
                  else lacc = f2_add(lacc, f2_pack(p0, p1));
                  if (decltype(is_bf)::value) {
                    const __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                    pk[e >> 1] = *reinterpret_cast<const uint32_t*>(&h);
                  } else {
                    const __half2 h = __floats2half2_rn(p0, p1);
                    pk[e >> 1] = *reinterpret_cast<const uint32_t*>(&h);
                  }
                }
              };
              if (full) {
                if (p.is_bf16) body(std::true_type{}, std::false_type{});
                else body(std::false_type{}, std::false_type{});
              } else {
                if (p.is_bf16) body(std::true_type{}, std::true_type{});
                else body(std::false_type{}, std::true_type{});
              }
              float la, lb;
              f2_unpack(f2_add(lacc, lacc2), la, lb);
              l0 += la;
              l1 += lb;
            }
            tmem_st_32x32b_x32(ts + (c0 >> 1), pk);
            if (c0 == 0) publish_half();
          }
        } else {
#pragma unroll 1
          for (int c0 = 0; c0 < FA_BN; c0 += 32) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(ts + c0, r);
            tmem_ld_wait();
            uint32_t pk[16];
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
              const float p0 = fast_exp2(score(r[e], c0 + e) + neg_m);
              const float p1 = fast_exp2(score(r[e + 1], c0 + e + 1) + neg_m);
              l0 += p0;
              l1 += p1;
              pk[e >> 1] = pack2(p0, p1);
            }
            tmem_st_32x32b_x16(ts + (c0 >> 1), pk);
            if (c0 == 32) publish_half();
          }
        }
        l_run += l0 + l1;
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[t]);
      }
      if (!ok) break;

      // ---- epilogue: O / l -> global -----------------------------------------------------------
      if (tile_on[t]) {
        bool have = false;
        if (ok && nt > 0) {
          have = mbar_wait(&o_ready[t], static_cast<uint32_t>((o_base + nt - 1) & 1), abort_word);
          tc_fence_after();
        }
        const float inv = (have && l_run > 0.f) ? 1.0f / l_run : 0.f;
        const bool row_ok = row < p.q_len;
        char* orow = static_cast<char*>(p.O) +
                     (static_cast<int64_t>(b) * p.o_sb + static_cast<int64_t>(q_head[t]) * p.o_sh +
                      static_cast<int64_t>(row) * p.o_sr) * 2;
        const bool vec = ((reinterpret_cast<uint64_t>(orow) & 15u) == 0);
#pragma unroll 1
        for (int c0 = 0; c0 < D; c0 += 32) {
          uint32_t r[32];
          if (have) {
            tmem_ld_32x32b_x32(to + c0, r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) r[e] = 0u;
          }
          if (row_ok) {
            uint32_t w[16];
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
              const float a0 = __uint_as_float(r[e]) * inv, a1 = __uint_as_float(r[e + 1]) * inv;
              const uint16_t lo = p.is_bf16 ? f32_to_bf16_bits_ref(a0) : f32_to_f16_bits_ref(a0);
              const uint16_t hi = p.is_bf16 ? f32_to_bf16_bits_ref(a1) : f32_to_f16_bits_ref(a1);
              w[e >> 1] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
            }
            if (vec) {
              uint4* dst = reinterpret_cast<uint4*>(orow + c0 * 2);
#pragma unroll
              for (int v4 = 0; v4 < 4; ++v4) dst[v4] = make_uint4(w[4 * v4], w[4 * v4 + 1], w[4 * v4 + 2], w[4 * v4 + 3]);
            } else {
              uint32_t* dst = reinterpret_cast<uint32_t*>(orow + c0 * 2);
#pragma unroll
              for (int e = 0; e < 16; ++e) dst[e] = w[e];
            }
          }
        }
      }

      if (nt > 0) {
        // O_t has been read: the MMA warp may overwrite it with the first P.V of the next item
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&o_free[t]);
      }
      s_base += nt;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_word) atomicExch(p.status, YTC_TIMEOUT);
}

// ------------------------------------------------------------------ catch-all: one warp per query row
struct AttnSimtParams {
  const void* Q;
  const void* K;
  const void* V;
  void* O;
  int64_t q_sb, q_sh, q_sr, k_sb, k_sh, k_sr, v_sb, v_sh, v_sr, o_sb, o_sh, o_sr;
  const uint8_t* mask;
  int64_t mask_rs;
  const float* bias;
  int64_t bias_rs, bias_cs;
  int batch, kv_heads, groups, q_len, kv_len, d, dv;
  int causal, causal_off;
  float scale;
  int dt;
};

constexpr int SIMT_MAX_D = 256;

__global__ void __launch_bounds__(128) attn_simt_kernel(const AttnSimtParams p) {
  __shared__ float q_s[4][SIMT_MAX_D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = p.kv_heads * p.groups;
  const int64_t total_rows = static_cast<int64_t>(p.batch) * heads * p.q_len;
  for (int64_t gr = static_cast<int64_t>(blockIdx.x) * 4 + warp; gr < total_rows;
       gr += static_cast<int64_t>(gridDim.x) * 4) {
    const int row = static_cast<int>(gr % p.q_len);
    const int h = static_cast<int>((gr / p.q_len) % heads);
    const int b = static_cast<int>(gr / (static_cast<int64_t>(p.q_len) * heads));
    const int kvh = h / p.groups;
    const int64_t qo = b * p.q_sb + h * p.q_sh + row * p.q_sr;
    const int64_t ko = b * p.k_sb + kvh * p.k_sh;
    const int64_t vo = b * p.v_sb + kvh * p.v_sh;
    __syncwarp();
    for (int i = lane; i < p.d; i += 32) q_s[warp][i] = load_as_f32(p.Q, qo + i, p.dt);
    __syncwarp();
    float acc[SIMT_MAX_D / 32];
#pragma unroll
    for (int i = 0; i < SIMT_MAX_D / 32; ++i) acc[i] = 0.f;
    float m_run = -CUDART_INF_F, l_run = 0.f;
    int last = p.kv_len - 1;
    if (p.causal && row + p.causal_off < last) last = row + p.causal_off;
    for (int k0 = 0; k0 <= last; k0 += 32) {
      const int key = k0 + lane;
      bool vis = key <= last;
      if (vis && p.mask) vis = p.mask[static_cast<int64_t>(row) * p.mask_rs + key] != 0;
      float s = -CUDART_INF_F;
      if (vis) {
        float dot = 0.f;
        const int64_t kb = ko + static_cast<int64_t>(key) * p.k_sr;
        for (int i = 0; i < p.d; ++i) dot = fmaf(q_s[warp][i], load_as_f32(p.K, kb + i, p.dt), dot);
        s = dot * p.scale;
        if (p.bias) s += p.bias[static_cast<int64_t>(row) * p.bias_rs + key * p.bias_cs];
      }
      float mx = s;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float m_new = fmaxf(m_run, mx);
      if (m_new == -CUDART_INF_F) continue;  // nothing visible in this chunk yet
      const float alpha = (m_run == -CUDART_INF_F) ? 0.f : expf(m_run - m_new);
      const float pr = vis ? expf(s - m_new) : 0.f;
      float ps = pr;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
      l_run = l_run * alpha + ps;
      m_run = m_new;
#pragma unroll
      for (int i = 0; i < SIMT_MAX_D / 32; ++i) acc[i] *= alpha;
      const int nk = (last - k0 + 1 < 32) ? last - k0 + 1 : 32;
      for (int kk = 0; kk < nk; ++kk) {
        const float pk = __shfl_sync(0xffffffffu, pr, kk);
        if (pk == 0.f) continue;
        const int64_t vb = vo + static_cast<int64_t>(k0 + kk) * p.v_sr;
#pragma unroll
        for (int i = 0; i < SIMT_MAX_D / 32; ++i) {
          const int c = i * 32 + lane;
          if (c < p.dv) acc[i] = fmaf(pk, load_as_f32(p.V, vb + c, p.dt), acc[i]);
        }
      }
    }
    const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
    const int64_t oo = b * p.o_sb + h * p.o_sh + row * p.o_sr;
#pragma unroll
    for (int i = 0; i < SIMT_MAX_D / 32; ++i) {
      const int c = i * 32 + lane;
      if (c < p.dv) store_from_f32(p.O, oo + c, acc[i] * inv, p.dt);
    }
  }
}


// ------------------------------------------------------------------ few query rows (decode): split over the keys
// One CTA = one (batch, kv head) and one slice of the keys; all R = groups * q_len query rows that share this K/V
// head are handled together, so every K / V row is read once (128-bit, coalesced: a warp reads one whole row).
// Each warp walks its keys with an online softmax per query row (running max, sum, and its 4 value columns per
// lane and 128 columns), warps are merged through shared memory, and the per-slice partials (max, sum, O) go to a
// scratch buffer that attn_decode_merge_kernel combines. Memory-bound on the KV cache.
constexpr int DEC_MAX_ROWS = 8;   // groups * q_len handled per CTA
constexpr int DEC_WARPS = 4;
constexpr int DEC_MAX_VEC = 2;    // float4 per lane per row: head / value dim up to 256
constexpr int DEC_KU = 4;         // keys fetched together per warp trip

struct AttnDecodeParams {
  AttnSimtParams a;
  int splits;
  int keys_per_split;
  float* part;  // [batch*kv_heads][splits][R][2 + dv]
};

__global__ void __launch_bounds__(DEC_WARPS * 32) attn_decode_kernel(const AttnDecodeParams dp) {
  const AttnSimtParams& p = dp.a;
  __shared__ float sm_m[DEC_WARPS][DEC_MAX_ROWS], sm_l[DEC_WARPS][DEC_MAX_ROWS];
  __shared__ float sm_o[DEC_WARPS][DEC_MAX_ROWS][DEC_MAX_VEC * 128];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x;
  const int bk = blockIdx.y;  // batch * kv_heads + kv head
  const int b = bk / p.kv_heads, kvh = bk - b * p.kv_heads;
  const int R = p.groups * p.q_len;
  const int nvq = (p.d + 127) / 128, nvv = (p.dv + 127) / 128;  // float4 slots per lane
  const int64_t ko = b * p.k_sb + kvh * p.k_sh, vo = b * p.v_sb + kvh * p.v_sh;

  // query rows in registers: row r = (group g, query index qi), head = kvh * groups + g
  float4 q[DEC_MAX_ROWS][DEC_MAX_VEC];
  float m_run[DEC_MAX_ROWS], l_run[DEC_MAX_ROWS];
  float4 acc[DEC_MAX_ROWS][DEC_MAX_VEC];
#pragma unroll
  for (int r = 0; r < DEC_MAX_ROWS; ++r) {
    m_run[r] = -CUDART_INF_F;
    l_run[r] = 0.f;
#pragma unroll
    for (int j = 0; j < DEC_MAX_VEC; ++j) {
      acc[r][j] = make_float4(0.f, 0.f, 0.f, 0.f);
      q[r][j] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (r < R && j < nvq) {
        const int g = r / p.q_len, qi = r - g * p.q_len;
        const int c = j * 128 + lane * 4;
        if (c < p.d) {
          const int64_t qo = b * p.q_sb + (kvh * p.groups + g) * p.q_sh + qi * p.q_sr + c;
          q[r][j] = make_float4(load_as_f32(p.Q, qo, p.dt), load_as_f32(p.Q, qo + 1, p.dt),
                                load_as_f32(p.Q, qo + 2, p.dt), load_as_f32(p.Q, qo + 3, p.dt));
        }
      }
    }
  }
  const int k_begin = split * dp.keys_per_split;
  int k_end = k_begin + dp.keys_per_split;
  if (k_end > p.kv_len) k_end = p.kv_len;
  // DEC_KU keys per trip: all their K / V rows are requested before the first one is used
  for (int key0 = k_begin + warp; key0 < k_end; key0 += DEC_WARPS * DEC_KU) {
    float4 kv[DEC_KU][DEC_MAX_VEC], vv[DEC_KU][DEC_MAX_VEC];
#pragma unroll
    for (int u = 0; u < DEC_KU; ++u) {
      const int key = key0 + u * DEC_WARPS;
#pragma unroll
      for (int j = 0; j < DEC_MAX_VEC; ++j) {
        kv[u][j] = make_float4(0.f, 0.f, 0.f, 0.f);
        vv[u][j] = make_float4(0.f, 0.f, 0.f, 0.f);
        const int c = j * 128 + lane * 4;
        if (key < k_end && j < nvq && c < p.d) {
          const int64_t o = ko + static_cast<int64_t>(key) * p.k_sr + c;
          if (p.dt == YTC_F32) kv[u][j] = *reinterpret_cast<const float4*>(static_cast<const float*>(p.K) + o);
          else kv[u][j] = make_float4(load_as_f32(p.K, o, p.dt), load_as_f32(p.K, o + 1, p.dt),
                                      load_as_f32(p.K, o + 2, p.dt), load_as_f32(p.K, o + 3, p.dt));
        }
        if (key < k_end && j < nvv && c < p.dv) {
          const int64_t o = vo + static_cast<int64_t>(key) * p.v_sr + c;
          if (p.dt == YTC_F32) vv[u][j] = *reinterpret_cast<const float4*>(static_cast<const float*>(p.V) + o);
          else vv[u][j] = make_float4(load_as_f32(p.V, o, p.dt), load_as_f32(p.V, o + 1, p.dt),
                                      load_as_f32(p.V, o + 2, p.dt), load_as_f32(p.V, o + 3, p.dt));
        }
      }
    }
#pragma unroll
    for (int u = 0; u < DEC_KU; ++u) {
      const int key = key0 + u * DEC_WARPS;
      if (key >= k_end) break;
#pragma unroll
      for (int r = 0; r < DEC_MAX_ROWS; ++r) {
        if (r >= R) break;
        const int qi = r % p.q_len;
        bool vis = !p.causal || key <= qi + p.causal_off;
        if (vis && p.mask) vis = p.mask[static_cast<int64_t>(qi) * p.mask_rs + key] != 0;
        if (!vis) continue;  // uniform over the warp
        float dot = 0.f;
#pragma unroll
        for (int j = 0; j < DEC_MAX_VEC; ++j) {
          dot = fmaf(q[r][j].x, kv[u][j].x, dot);
          dot = fmaf(q[r][j].y, kv[u][j].y, dot);
          dot = fmaf(q[r][j].z, kv[u][j].z, dot);
          dot = fmaf(q[r][j].w, kv[u][j].w, dot);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        float sc = dot * p.scale;
        if (p.bias) sc += p.bias[static_cast<int64_t>(qi) * p.bias_rs + key * p.bias_cs];
        const float m_new = fmaxf(m_run[r], sc);
        const float alpha = __expf(m_run[r] - m_new);  // 0 on the first visible key (m_run = -inf)
        const float pr = __expf(sc - m_new);
        l_run[r] = l_run[r] * alpha + pr;
        m_run[r] = m_new;
#pragma unroll
        for (int j = 0; j < DEC_MAX_VEC; ++j) {
          acc[r][j].x = fmaf(pr, vv[u][j].x, acc[r][j].x * alpha);
          acc[r][j].y = fmaf(pr, vv[u][j].y, acc[r][j].y * alpha);
          acc[r][j].z = fmaf(pr, vv[u][j].z, acc[r][j].z * alpha);
          acc[r][j].w = fmaf(pr, vv[u][j].w, acc[r][j].w * alpha);
        }
      }
    }
  }
  // merge the warps of this CTA
#pragma unroll
  for (int r = 0; r < DEC_MAX_ROWS; ++r) {
    if (r >= R) break;
    if (lane == 0) {
      sm_m[warp][r] = m_run[r];
      sm_l[warp][r] = l_run[r];
    }
#pragma unroll
    for (int j = 0; j < DEC_MAX_VEC; ++j)
      if (j < nvv) *reinterpret_cast<float4*>(&sm_o[warp][r][j * 128 + lane * 4]) = acc[r][j];
  }
  __syncthreads();
  const int stride = 2 + p.dv;
  float* out = dp.part + (static_cast<int64_t>(bk) * dp.splits + split) * R * stride;
  for (int idx = threadIdx.x; idx < R * p.dv; idx += DEC_WARPS * 32) {
    const int r = idx / p.dv, c = idx - r * p.dv;
    float m = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) m = fmaxf(m, sm_m[w][r]);
    float l = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float f = (sm_m[w][r] == -CUDART_INF_F) ? 0.f : __expf(sm_m[w][r] - m);
      l += sm_l[w][r] * f;
      o += sm_o[w][r][c] * f;
    }
    out[r * stride + 2 + c] = o;
    if (c == 0) {
      out[r * stride] = m;
      out[r * stride + 1] = l;
    }
  }
}

// Decode attention for the common case (fp32, one query row per head, head / value dim 128, no mask or bias, rows
// of K and V contiguous): one CTA of 8 warps per (sequence, kv head, key split). A warp takes 16 keys per step with
// coalesced row loads: 8 lanes share a key for the dot products with the G query heads of the group (3 shuffles
// finish one), maximum and sum are taken once per 16 keys, and P.V runs with the value dim across lanes and the
// probabilities broadcast by shuffles. The V rows of a step are requested together with its K rows. The warps
// combine through shared memory and leave (m, l, o) per split for attn_decode_merge_kernel.
constexpr int DF_WARPS = 8;
constexpr int DF_KB = 16;

template <int G>
__global__ void __launch_bounds__(DF_WARPS * 32) attn_decode_fast_kernel(const AttnDecodeParams dp) {
  dependent_wait();     // (under a programmatic dependent launch: the kernel before this one has finished)
  dependent_trigger();  // the kernel queued behind this one may be scheduled meanwhile
  const AttnSimtParams& p = dp.a;
  constexpr int D = 128;
  __shared__ __align__(16) float qs[G * D];
  __shared__ float pm[DF_WARPS * G], pl[DF_WARPS * G];
  __shared__ __align__(16) float po[DF_WARPS * G * D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x;
  const int bk = blockIdx.y;
  const int b = bk / p.kv_heads, kvh = bk - b * p.kv_heads;
  const float* Q = static_cast<const float*>(p.Q);
  const float* kb = static_cast<const float*>(p.K) + b * p.k_sb + kvh * p.k_sh;
  const float* vb = static_cast<const float*>(p.V) + b * p.v_sb + kvh * p.v_sh;
  int n_keys = p.kv_len;
  if (p.causal && p.causal_off + 1 < n_keys) n_keys = p.causal_off + 1;  // the single query row sees keys <= offset
  const int k_begin = split * dp.keys_per_split;
  int k_end = k_begin + dp.keys_per_split;
  if (k_end > n_keys) k_end = n_keys;
  for (int i = threadIdx.x; i < G * D; i += DF_WARPS * 32) {
    const int g = i / D, c = i - g * D;
    qs[i] = Q[b * p.q_sb + (kvh * G + g) * p.q_sh + c];
  }
  __syncthreads();
  const int j8 = lane & 7, kq = lane >> 3;
  float4 qreg[G][4];
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int i = 0; i < 4; ++i) qreg[g][i] = *reinterpret_cast<const float4*>(&qs[g * D + (j8 + 8 * i) * 4]);
  float m_run[G], l_run[G];
  float4 acc[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m_run[g] = -CUDART_INF_F;
    l_run[g] = 0.f;
    acc[g] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  for (int key0 = k_begin + warp * DF_KB; key0 < k_end; key0 += DF_WARPS * DF_KB) {
    float sc[G][DF_KB / 4];
    float4 vv[DF_KB];
#pragma unroll
    for (int t = 0; t < DF_KB; ++t) {
      vv[t] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (key0 + t < k_end) vv[t] = *(reinterpret_cast<const float4*>(vb + static_cast<int64_t>(key0 + t) * p.v_sr) + lane);
    }
    float4 kvr[DF_KB / 4][4];
#pragma unroll
    for (int kg = 0; kg < DF_KB / 4; ++kg) {
      const int key = key0 + kg * 4 + kq;
      const float4* krow = reinterpret_cast<const float4*>(kb + static_cast<int64_t>(key < k_end ? key : k_begin) * p.k_sr);
#pragma unroll
      for (int i = 0; i < 4; ++i) kvr[kg][i] = krow[j8 + 8 * i];
    }
#pragma unroll
    for (int kg = 0; kg < DF_KB / 4; ++kg) {
      const bool valid = key0 + kg * 4 + kq < k_end;
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
      for (int kg = 1; kg < DF_KB / 4; ++kg) mx = fmaxf(mx, sc[g][kg]);
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
      const float m_new = fmaxf(m_run[g], mx);       // finite: every step has a valid key
      const float alpha = __expf(m_run[g] - m_new);  // 0 on the first step (m_run = -inf)
      float sum = 0.f;
#pragma unroll
      for (int kg = 0; kg < DF_KB / 4; ++kg) {
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
    for (int kg = 0; kg < DF_KB / 4; ++kg)
#pragma unroll
      for (int t = 0; t < 4; ++t)
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float pt = __shfl_sync(0xffffffffu, sc[g][kg], t * 8);
          acc[g].x = fmaf(pt, vv[kg * 4 + t].x, acc[g].x);
          acc[g].y = fmaf(pt, vv[kg * 4 + t].y, acc[g].y);
          acc[g].z = fmaf(pt, vv[kg * 4 + t].z, acc[g].z);
          acc[g].w = fmaf(pt, vv[kg * 4 + t].w, acc[g].w);
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
    const int g = warp;
    const float mw = lane < DF_WARPS ? pm[lane * G + g] : -CUDART_INF_F;
    const float lw = lane < DF_WARPS ? pl[lane * G + g] : 0.f;
    float m = mw;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float fw = (mw == -CUDART_INF_F) ? 0.f : __expf(mw - m);
    float lsum = lw * fw;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, o);
    float4 o4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < DF_WARPS; ++w) {
      const float f = __shfl_sync(0xffffffffu, fw, w);
      const float4 ow = *reinterpret_cast<const float4*>(&po[(w * G + g) * D + lane * 4]);
      o4.x = fmaf(ow.x, f, o4.x);
      o4.y = fmaf(ow.y, f, o4.y);
      o4.z = fmaf(ow.z, f, o4.z);
      o4.w = fmaf(ow.w, f, o4.w);
    }
    // the layout attn_decode_merge_kernel reads: [m, l, o[dv]] per (kv head, split, row); row = g (q_len == 1)
    float* dst = dp.part + ((static_cast<int64_t>(bk) * dp.splits + split) * G + g) * (2 + D);
    if (lane == 0) {
      dst[0] = m;
      dst[1] = lsum;
    }
    float2* d2 = reinterpret_cast<float2*>(dst + 2 + lane * 4);
    d2[0] = make_float2(o4.x, o4.y);
    d2[1] = make_float2(o4.z, o4.w);
  }
}


// Combines the per-slice partials: O = sum_s O_s * 2^(m_s - m) / sum_s l_s * 2^(m_s - m); rows that saw no key -> 0.
__global__ void __launch_bounds__(128) attn_decode_merge_kernel(const AttnDecodeParams dp) {
  dependent_wait();     // (under a programmatic dependent launch: the kernel before this one has finished)
  dependent_trigger();  // the kernel queued behind this one may be scheduled meanwhile
  const AttnSimtParams& p = dp.a;
  const int bk = blockIdx.x;
  const int b = bk / p.kv_heads, kvh = bk - b * p.kv_heads;
  const int R = p.groups * p.q_len;
  const int stride = 2 + p.dv;
  const float* base = dp.part + static_cast<int64_t>(bk) * dp.splits * R * stride;
  for (int idx = threadIdx.x; idx < R * p.dv; idx += blockDim.x) {
    const int r = idx / p.dv, c = idx - r * p.dv;
    float m = -CUDART_INF_F;
    for (int s = 0; s < dp.splits; ++s) m = fmaxf(m, base[(s * R + r) * stride]);
    float l = 0.f, o = 0.f;
    for (int s = 0; s < dp.splits; ++s) {
      const float ms = base[(s * R + r) * stride];
      const float f = (ms == -CUDART_INF_F) ? 0.f : __expf(ms - m);
      l += base[(s * R + r) * stride + 1] * f;
      o += base[(s * R + r) * stride + 2 + c] * f;
    }
    const int g = r / p.q_len, qi = r - g * p.q_len;
    const int64_t oo = b * p.o_sb + (kvh * p.groups + g) * p.o_sh + qi * p.o_sr + c;
    store_from_f32(p.O, oo, l > 0.f ? o / l : 0.f, p.dt);
  }
}

// ------------------------------------------------------------------ fp32-accumulating tiled kernel (any dtype)
// 32 query rows x 32 keys per step, 128 threads: thread (i, g) = (row, quarter). S = Q K^T from shared memory with
// 8 scores per thread in registers, online softmax across the 4 threads of a row by shuffles, then
// O[i, 32 g .. 32 g + 31] += P[i, :] V with P passed through shared memory. The prefill path of the fp32 decoder.
constexpr int TL_BM = 32, TL_BN = 32, TL_D = 128, TL_PAD = 4;

__global__ void __launch_bounds__(128) attn_tile_kernel(const AttnSimtParams p) {
  extern __shared__ __align__(16) float tl_smem[];
  float(*Qs)[TL_D + TL_PAD] = reinterpret_cast<float(*)[TL_D + TL_PAD]>(tl_smem);
  float(*Ks)[TL_D + TL_PAD] = Qs + TL_BM;
  float(*Vs)[TL_D + TL_PAD] = Ks + TL_BN;
  float(*Ps)[TL_BN + 1] = reinterpret_cast<float(*)[TL_BN + 1]>(Vs + TL_BN);
  const int tid = threadIdx.x;
  const int ri = tid >> 2, g = tid & 3;
  const int heads = p.kv_heads * p.groups;
  const int row_blocks = (p.q_len + TL_BM - 1) / TL_BM;
  const int rbk = row_blocks - 1 - static_cast<int>(blockIdx.x);  // long causal rows first
  const int h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / p.groups;
  const int row0 = rbk * TL_BM;
  const int row = row0 + ri;
  const int64_t qo = b * p.q_sb + h * p.q_sh;
  const int64_t ko = b * p.k_sb + kvh * p.k_sh, vo = b * p.v_sb + kvh * p.v_sh;
  (void)heads;
  // stage Q (zero-padded to TL_D columns and TL_BM rows)
  // fp32 operands with 16-byte aligned rows are staged with 128-bit loads; anything else element by element
  const bool vec = p.dt == YTC_F32 && p.d % 4 == 0 && p.dv % 4 == 0 && p.q_sr % 4 == 0 && p.k_sr % 4 == 0 &&
                   p.v_sr % 4 == 0 && p.q_sh % 4 == 0 && p.k_sh % 4 == 0 && p.v_sh % 4 == 0 && p.q_sb % 4 == 0 &&
                   p.k_sb % 4 == 0 && p.v_sb % 4 == 0 && (reinterpret_cast<uint64_t>(p.Q) & 15) == 0 &&
                   (reinterpret_cast<uint64_t>(p.K) & 15) == 0 && (reinterpret_cast<uint64_t>(p.V) & 15) == 0;
  if (vec) {
    const float* Qf = static_cast<const float*>(p.Q);
    for (int i = tid; i < TL_BM * (TL_D / 4); i += 128) {
      const int r = i >> 5, c = (i & 31) * 4;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (row0 + r < p.q_len && c < p.d) v = *reinterpret_cast<const float4*>(Qf + qo + static_cast<int64_t>(row0 + r) * p.q_sr + c);
      *reinterpret_cast<float4*>(&Qs[r][c]) = v;
    }
  } else {
    for (int i = tid; i < TL_BM * TL_D; i += 128) {
      const int r = i / TL_D, c = i - r * TL_D;
      Qs[r][c] = (row0 + r < p.q_len && c < p.d)
                     ? load_as_f32(p.Q, qo + static_cast<int64_t>(row0 + r) * p.q_sr + c, p.dt) : 0.f;
    }
  }
  float acc[32];
#pragma unroll
  for (int c = 0; c < 32; ++c) acc[c] = 0.f;
  float m_run = -CUDART_INF_F, l_run = 0.f;
  int last = p.kv_len - 1;
  if (p.causal) {
    const int lim = row0 + TL_BM - 1 + p.causal_off;
    if (lim < last) last = lim;
  }
  const int my_limit = (row < p.q_len) ? ((p.causal && row + p.causal_off < p.kv_len - 1) ? row + p.causal_off : p.kv_len - 1)
                                       : -1;
  for (int k0 = 0; k0 <= last; k0 += TL_BN) {
    __syncthreads();
    if (vec) {
      const float* Kf = static_cast<const float*>(p.K);
      const float* Vf = static_cast<const float*>(p.V);
      float4 kq[8], vq[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = tid + u * 128;
        const int r = i >> 5, c = (i & 31) * 4;
        const bool in = k0 + r < p.kv_len;
        kq[u] = (in && c < p.d) ? *reinterpret_cast<const float4*>(Kf + ko + static_cast<int64_t>(k0 + r) * p.k_sr + c)
                                : make_float4(0.f, 0.f, 0.f, 0.f);
        vq[u] = (in && c < p.dv) ? *reinterpret_cast<const float4*>(Vf + vo + static_cast<int64_t>(k0 + r) * p.v_sr + c)
                                 : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = tid + u * 128;
        const int r = i >> 5, c = (i & 31) * 4;
        *reinterpret_cast<float4*>(&Ks[r][c]) = kq[u];
        *reinterpret_cast<float4*>(&Vs[r][c]) = vq[u];
      }
    } else {
      for (int i = tid; i < TL_BN * TL_D; i += 128) {
        const int r = i / TL_D, c = i - r * TL_D;
        const bool in = k0 + r < p.kv_len;
        Ks[r][c] = (in && c < p.d) ? load_as_f32(p.K, ko + static_cast<int64_t>(k0 + r) * p.k_sr + c, p.dt) : 0.f;
        Vs[r][c] = (in && c < p.dv) ? load_as_f32(p.V, vo + static_cast<int64_t>(k0 + r) * p.v_sr + c, p.dt) : 0.f;
      }
    }
    __syncthreads();
    float sc[8];
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) sc[jj] = 0.f;
#pragma unroll 4
    for (int k4 = 0; k4 < TL_D; k4 += 4) {
      const float4 qv = *reinterpret_cast<const float4*>(&Qs[ri][k4]);
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) {
        const float4 kv = *reinterpret_cast<const float4*>(&Ks[g * 8 + jj][k4]);
        sc[jj] = fmaf(qv.x, kv.x, sc[jj]);
        sc[jj] = fmaf(qv.y, kv.y, sc[jj]);
        sc[jj] = fmaf(qv.z, kv.z, sc[jj]);
        sc[jj] = fmaf(qv.w, kv.w, sc[jj]);
      }
    }
    float mx = -CUDART_INF_F;
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) {
      const int key = k0 + g * 8 + jj;
      bool vis = key <= my_limit;
      if (vis && p.mask) vis = p.mask[static_cast<int64_t>(row) * p.mask_rs + key] != 0;
      float v = sc[jj] * p.scale;
      if (vis && p.bias) v += p.bias[static_cast<int64_t>(row) * p.bias_rs + key * p.bias_cs];
      sc[jj] = vis ? v : -CUDART_INF_F;
      mx = fmaxf(mx, sc[jj]);
    }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m_run, mx);
    const float m_use = (m_new == -CUDART_INF_F) ? 0.f : m_new;
    const float alpha = (m_run == -CUDART_INF_F) ? 0.f : __expf(m_run - m_use);
    float ps = 0.f;
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) {
      const float pr = __expf(sc[jj] - m_use);  // exp(-inf) = 0 for hidden keys
      Ps[ri][g * 8 + jj] = pr;
      ps += pr;
    }
    ps += __shfl_xor_sync(0xffffffffu, ps, 1);
    ps += __shfl_xor_sync(0xffffffffu, ps, 2);
    l_run = l_run * alpha + ps;
    m_run = m_new;
    __syncwarp();  // the 4 threads of a row sit in one warp: Ps[ri][*] is complete for them
#pragma unroll
    for (int c = 0; c < 32; ++c) acc[c] *= alpha;
#pragma unroll 4
    for (int j = 0; j < TL_BN; ++j) {
      const float pr = Ps[ri][j];
#pragma unroll
      for (int c4 = 0; c4 < 32; c4 += 4) {
        const float4 vv = *reinterpret_cast<const float4*>(&Vs[j][g * 32 + c4]);
        acc[c4] = fmaf(pr, vv.x, acc[c4]);
        acc[c4 + 1] = fmaf(pr, vv.y, acc[c4 + 1]);
        acc[c4 + 2] = fmaf(pr, vv.z, acc[c4 + 2]);
        acc[c4 + 3] = fmaf(pr, vv.w, acc[c4 + 3]);
      }
    }
  }
  if (row < p.q_len) {
    const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
    const int64_t oo = b * p.o_sb + h * p.o_sh + static_cast<int64_t>(row) * p.o_sr;
#pragma unroll
    for (int c = 0; c < 32; ++c) {
      const int col = g * 32 + c;
      if (col < p.dv) store_from_f32(p.O, oo + col, acc[c] * inv, p.dt);
    }
  }
}

// ------------------------------------------------------------------ host side

// ------------------------------------------------------------------ fp32 attention with register tiles (prefill)
// 64 query rows x 64 keys per step and CTA, 256 threads. S = Q K^T is formed in 4 x 4 register tiles (rows
// 4 ry .. 4 ry + 3, keys kx, kx + 16, kx + 32, kx + 48: the strided keys keep the 128-bit shared-memory reads of K free
// of bank conflicts), the row maximum and sum are taken over the 16 lanes that share a row group, P goes to shared
// memory transposed ([key][row]) and O += P V runs in 4 x 8 register tiles (value columns 4 cx .. 4 cx + 3 and
// 64 + 4 cx .. 64 + 4 cx + 3). 8 FMAs per 128-bit shared-memory read in the first product, about 11 in the second,
// against 3.5 in attn_tile_kernel. fp32 operands with 16-byte aligned rows, head / value dim up to 128.
constexpr int T64_BM = 64, T64_BN = 64, T64_LD = 128 + 4, T64_PLD = 64 + 4;
constexpr int T64_SMEM = (3 * 64 * T64_LD + T64_BN * T64_PLD) * 4;

__global__ void __launch_bounds__(256, 1) attn_tile64_kernel(const AttnSimtParams p) {
  dependent_wait();     // (under a programmatic dependent launch: the kernel before this one has finished)
  dependent_trigger();  // the kernel queued behind this one may be scheduled meanwhile
  extern __shared__ __align__(16) float t64_smem[];
  float(*Qs)[T64_LD] = reinterpret_cast<float(*)[T64_LD]>(t64_smem);
  float(*Ks)[T64_LD] = Qs + T64_BM;
  float(*Vs)[T64_LD] = Ks + T64_BN;
  float(*PsT)[T64_PLD] = reinterpret_cast<float(*)[T64_PLD]>(Vs + T64_BN);  // [key][row]
  const int tid = threadIdx.x;
  const int ry = tid >> 4, kx = tid & 15, cx = kx;
  const int row_blocks = (p.q_len + T64_BM - 1) / T64_BM;
  const int rbk = row_blocks - 1 - static_cast<int>(blockIdx.x);  // long causal rows first
  const int h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / p.groups;
  const int row0 = rbk * T64_BM;
  const float* Qf = static_cast<const float*>(p.Q) + b * p.q_sb + h * p.q_sh;
  const float* Kf = static_cast<const float*>(p.K) + b * p.k_sb + kvh * p.k_sh;
  const float* Vf = static_cast<const float*>(p.V) + b * p.v_sb + kvh * p.v_sh;
  for (int i = tid; i < T64_BM * 32; i += 256) {
    const int r = i >> 5, c = (i & 31) * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (row0 + r < p.q_len && c < p.d) v = *reinterpret_cast<const float4*>(Qf + static_cast<int64_t>(row0 + r) * p.q_sr + c);
    *reinterpret_cast<float4*>(&Qs[r][c]) = v;
  }
  float acc[4][8];
  float m_run[4], l_run[4];
  int limit[4];  // last visible key of each of this thread's rows (-1: the row does not exist)
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    m_run[i] = -CUDART_INF_F;
    l_run[i] = 0.f;
    const int row = row0 + ry * 4 + i;
    limit[i] = (row < p.q_len) ? ((p.causal && row + p.causal_off < p.kv_len - 1) ? row + p.causal_off : p.kv_len - 1) : -1;
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[i][c] = 0.f;
  }
  int last = p.kv_len - 1;
  if (p.causal) {
    const int lim = row0 + T64_BM - 1 + p.causal_off;
    if (lim < last) last = lim;
  }
  for (int k0 = 0; k0 <= last; k0 += T64_BN) {
    __syncthreads();  // the previous step has finished with Ks, Vs and PsT
    {
      float4 kq[8], vq[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = tid + u * 256;
        const int r = i >> 5, c = (i & 31) * 4;
        const bool in = k0 + r < p.kv_len;
        kq[u] = (in && c < p.d) ? *reinterpret_cast<const float4*>(Kf + static_cast<int64_t>(k0 + r) * p.k_sr + c)
                                : make_float4(0.f, 0.f, 0.f, 0.f);
        vq[u] = (in && c < p.dv) ? *reinterpret_cast<const float4*>(Vf + static_cast<int64_t>(k0 + r) * p.v_sr + c)
                                 : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = tid + u * 256;
        const int r = i >> 5, c = (i & 31) * 4;
        *reinterpret_cast<float4*>(&Ks[r][c]) = kq[u];
        *reinterpret_cast<float4*>(&Vs[r][c]) = vq[u];
      }
    }
    __syncthreads();
    float sc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) sc[i][j] = 0.f;
#pragma unroll 2
    for (int k4 = 0; k4 < 128; k4 += 4) {
      float4 qv[4], kv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) qv[i] = *reinterpret_cast<const float4*>(&Qs[ry * 4 + i][k4]);
#pragma unroll
      for (int j = 0; j < 4; ++j) kv[j] = *reinterpret_cast<const float4*>(&Ks[kx + 16 * j][k4]);
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          sc[i][j] = fmaf(qv[i].x, kv[j].x, sc[i][j]);
          sc[i][j] = fmaf(qv[i].y, kv[j].y, sc[i][j]);
          sc[i][j] = fmaf(qv[i].z, kv[j].z, sc[i][j]);
          sc[i][j] = fmaf(qv[i].w, kv[j].w, sc[i][j]);
        }
    }
    float alpha[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = row0 + ry * 4 + i;
      float mx = -CUDART_INF_F;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int key = k0 + kx + 16 * j;
        bool vis = key <= limit[i];
        if (vis && p.mask) vis = p.mask[static_cast<int64_t>(row) * p.mask_rs + key] != 0;
        float v = sc[i][j] * p.scale;
        if (vis && p.bias) v += p.bias[static_cast<int64_t>(row) * p.bias_rs + key * p.bias_cs];
        sc[i][j] = vis ? v : -CUDART_INF_F;
        mx = fmaxf(mx, sc[i][j]);
      }
#pragma unroll
      for (int o = 1; o < 16; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float m_new = fmaxf(m_run[i], mx);
      const float m_use = (m_new == -CUDART_INF_F) ? 0.f : m_new;
      alpha[i] = (m_run[i] == -CUDART_INF_F) ? 0.f : __expf(m_run[i] - m_use);
      float ps = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float pr = __expf(sc[i][j] - m_use);  // exp(-inf) = 0 for hidden keys
        PsT[kx + 16 * j][ry * 4 + i] = pr;
        ps += pr;
      }
#pragma unroll
      for (int o = 1; o < 16; o <<= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
      l_run[i] = l_run[i] * alpha[i] + ps;
      m_run[i] = m_new;
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[i][c] *= alpha[i];
    }
    __syncthreads();  // P of all 64 rows x 64 keys is in shared memory
#pragma unroll 4
    for (int j = 0; j < T64_BN; ++j) {
      const float4 pr = *reinterpret_cast<const float4*>(&PsT[j][ry * 4]);
      const float4 v0 = *reinterpret_cast<const float4*>(&Vs[j][cx * 4]);
      const float4 v1 = *reinterpret_cast<const float4*>(&Vs[j][64 + cx * 4]);
      const float pv[4] = {pr.x, pr.y, pr.z, pr.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[i][0] = fmaf(pv[i], v0.x, acc[i][0]);
        acc[i][1] = fmaf(pv[i], v0.y, acc[i][1]);
        acc[i][2] = fmaf(pv[i], v0.z, acc[i][2]);
        acc[i][3] = fmaf(pv[i], v0.w, acc[i][3]);
        acc[i][4] = fmaf(pv[i], v1.x, acc[i][4]);
        acc[i][5] = fmaf(pv[i], v1.y, acc[i][5]);
        acc[i][6] = fmaf(pv[i], v1.z, acc[i][6]);
        acc[i][7] = fmaf(pv[i], v1.w, acc[i][7]);
      }
    }
  }
  float* Of = static_cast<float*>(p.O) + b * p.o_sb + h * p.o_sh;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = row0 + ry * 4 + i;
    if (row >= p.q_len) continue;
    const float inv = l_run[i] > 0.f ? 1.0f / l_run[i] : 0.f;
    float* orow = Of + static_cast<int64_t>(row) * p.o_sr;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      if (cx * 4 + c < p.dv) orow[cx * 4 + c] = acc[i][c] * inv;
      if (64 + cx * 4 + c < p.dv) orow[64 + cx * 4 + c] = acc[i][4 + c] * inv;
    }
  }
}

static std::atomic<int> g_attn_path{0};  // 0 automatic, 1 always the one-warp-per-row kernel, 2 tensor-core kernel or fail

static int make_qkv_map(CUtensorMap* map, const void* base, int d, int64_t len, int64_t heads, int64_t batch,
                        int64_t s_row, int64_t s_head, int64_t s_batch) {
  // dims {d, len, heads, batch}; a dim of extent 1 may carry any stride: give it a harmless one
  uint64_t dims[4] = {static_cast<uint64_t>(d), static_cast<uint64_t>(len), static_cast<uint64_t>(heads),
                      static_cast<uint64_t>(batch)};
  uint64_t strides[3] = {static_cast<uint64_t>(s_row) * 2, static_cast<uint64_t>(s_head) * 2,
                         static_cast<uint64_t>(s_batch) * 2};
  if (len == 1) strides[0] = static_cast<uint64_t>(d) * 2;
  if (heads == 1) strides[1] = strides[0] * dims[1];
  if (batch == 1) strides[2] = strides[1] * dims[2];
  uint32_t box[4] = {64, FA_BM, 1, 1};
  return encode_tensor_map(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 4, base, dims, strides, box,
                           CU_TENSOR_MAP_SWIZZLE_128B);
}

static bool tc_strides_ok(const void* ptr, int64_t s_row, int64_t s_head, int64_t s_batch, int64_t len, int64_t heads,
                          int64_t batch) {
  if (reinterpret_cast<uint64_t>(ptr) & 15u) return false;
  if (len > 1 && (s_row <= 0 || (s_row * 2) % 16)) return false;
  if (heads > 1 && (s_head <= 0 || (s_head * 2) % 16)) return false;
  if (batch > 1 && (s_batch <= 0 || (s_batch * 2) % 16)) return false;
  return true;
}

}  // namespace ytk

using namespace ytk;

extern "C" {

int ytcuda_attn_set_path(int path) {
  YTC_REQUIRE(path >= 0 && path <= 2, "ytcuda_attn_set_path: path must be 0, 1 or 2");
  g_attn_path = path;
  return YTC_OK;
}

int ytcuda_flash_attn_fwd(int dtype, const void* Q, const void* K, const void* V, void* O, int batch, int kv_heads,
                          int groups, int q_len, int kv_len, int head_dim, int value_dim, float scale,
                          const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                          const int64_t* o_strides, int mask_kind, int causal_offset, const uint8_t* mask,
                          int64_t mask_row_stride, const float* bias, int64_t bias_row_stride, int64_t bias_col_stride,
                          void* stream) {
  YTC_REQUIRE(dtype >= YTC_F32 && dtype <= YTC_F16, "ytcuda_flash_attn_fwd: bad dtype %d", dtype);
  YTC_REQUIRE(batch >= 0 && kv_heads >= 0 && groups >= 0 && q_len >= 0 && kv_len >= 0 && head_dim >= 0 &&
                  value_dim >= 0,
              "ytcuda_flash_attn_fwd: negative extent");
  YTC_REQUIRE(mask_kind >= 0 && mask_kind <= 2, "ytcuda_flash_attn_fwd: mask_kind must be 0 (none), 1 (causal), 2 (bool)");
  YTC_REQUIRE(mask_kind != 2 || mask != nullptr, "ytcuda_flash_attn_fwd: bool mask requested but the pointer is null");
  if (batch == 0 || kv_heads == 0 || groups == 0 || q_len == 0 || value_dim == 0) return YTC_OK;
  YTC_REQUIRE(Q && K && V && O, "ytcuda_flash_attn_fwd: null tensor");
  YTC_REQUIRE(q_strides && k_strides && v_strides && o_strides, "ytcuda_flash_attn_fwd: null strides");
  if (scale == 0.f) scale = 1.0f / sqrtf(static_cast<float>(head_dim));  // reference src/function/ops.inl:378-381
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int heads = kv_heads * groups;
  const int causal = mask_kind == 1 ? 1 : 0;
  const uint8_t* mptr = mask_kind == 2 ? mask : nullptr;

  bool tc = dtype != YTC_F32 && g_attn_path != 1 && head_dim == value_dim && (head_dim == 64 || head_dim == 128) &&
            kv_len > 0 && tc_strides_ok(Q, q_strides[2], q_strides[1], q_strides[0], q_len, heads, batch) &&
            tc_strides_ok(K, k_strides[2], k_strides[1], k_strides[0], kv_len, kv_heads, batch) &&
            tc_strides_ok(V, v_strides[2], v_strides[1], v_strides[0], kv_len, kv_heads, batch) &&
            (reinterpret_cast<uint64_t>(O) & 3u) == 0 && o_strides[2] % 2 == 0 && o_strides[1] % 2 == 0 &&
            o_strides[0] % 2 == 0;
  if (!tc && g_attn_path == 2) {
    set_last_error("ytcuda_flash_attn_fwd: tensor-core path required but the operands do not qualify");
    return YTC_UNSUPPORTED;
  }
  if (tc) {
    CUtensorMap tmQ, tmK, tmV;
    int s = make_qkv_map(&tmQ, Q, head_dim, q_len, heads, batch, q_strides[2], q_strides[1], q_strides[0]);
    if (s != YTC_OK) return s;
    s = make_qkv_map(&tmK, K, head_dim, kv_len, kv_heads, batch, k_strides[2], k_strides[1], k_strides[0]);
    if (s != YTC_OK) return s;
    s = make_qkv_map(&tmV, V, value_dim, kv_len, kv_heads, batch, v_strides[2], v_strides[1], v_strides[0]);
    if (s != YTC_OK) return s;
    FlashParams p;
    p.O = O;
    p.o_sb = o_strides[0]; p.o_sh = o_strides[1]; p.o_sr = o_strides[2];
    p.mask = mptr; p.mask_rs = mask_row_stride;
    p.bias = bias; p.bias_rs = bias_row_stride; p.bias_cs = bias_col_stride;
    p.batch = batch; p.kv_heads = kv_heads; p.groups = groups; p.q_len = q_len; p.kv_len = kv_len;
    p.causal = causal; p.causal_off = causal_offset;
    p.scale_log2 = scale * FA_LOG2E;
    p.is_bf16 = dtype == YTC_BF16;
    p.pair_heads = (groups % 2 == 0) ? 1 : 0;
    const uint32_t fmt = dtype == YTC_BF16 ? 1u : 0u;
    p.idesc_s = umma_idesc(fmt, 0, 0, FA_BM, FA_BN);
    p.idesc_pv = umma_idesc(fmt, 0, 1, FA_BM, static_cast<uint32_t>(value_dim));
    p.status = device_status_word();
    if (!p.status) {
      set_last_error("ytcuda_flash_attn_fwd: no device status word");
      return YTC_CUDA_ERROR;
    }
    if (p.pair_heads) {
      p.row_blocks = (q_len + FA_BM - 1) / FA_BM;
      p.head_slots = heads / 2;
    } else {
      p.row_blocks = (q_len + 2 * FA_BM - 1) / (2 * FA_BM);
      p.head_slots = heads;
    }
    const int64_t items = static_cast<int64_t>(p.row_blocks) * p.head_slots * batch;
    if (items > 0x7fffffffll) {
      set_last_error("ytcuda_flash_attn_fwd: too many work items");
      return YTC_UNSUPPORTED;
    }
    p.items_per_row_block = p.head_slots * batch;
    p.n_items = static_cast<int>(items);
    const dim3 grid(static_cast<unsigned>(p.n_items < sm_count() ? p.n_items : sm_count()));
    if (head_dim == 128) {
      const int sa = ensure_dynamic_smem(reinterpret_cast<const void*>(flash_tc_kernel<128>), FaSmem<128>::DYN_BYTES);
      if (sa != YTC_OK) return sa;
      flash_tc_kernel<128><<<grid, FA_THREADS, FaSmem<128>::DYN_BYTES, st>>>(tmQ, tmK, tmV, p);
    } else {
      const int sa = ensure_dynamic_smem(reinterpret_cast<const void*>(flash_tc_kernel<64>), FaSmem<64>::DYN_BYTES);
      if (sa != YTC_OK) return sa;
      flash_tc_kernel<64><<<grid, FA_THREADS, FaSmem<64>::DYN_BYTES, st>>>(tmQ, tmK, tmV, p);
    }
    count_launch();
    YTC_CUDA(cudaGetLastError());
    return YTC_OK;
  }

  if (head_dim > SIMT_MAX_D || value_dim > SIMT_MAX_D) {
    set_last_error("ytcuda_flash_attn_fwd: head_dim / value_dim above %d are not supported", SIMT_MAX_D);
    return YTC_UNSUPPORTED;
  }
  AttnSimtParams p;
  p.Q = Q; p.K = K; p.V = V; p.O = O;
  p.q_sb = q_strides[0]; p.q_sh = q_strides[1]; p.q_sr = q_strides[2];
  p.k_sb = k_strides[0]; p.k_sh = k_strides[1]; p.k_sr = k_strides[2];
  p.v_sb = v_strides[0]; p.v_sh = v_strides[1]; p.v_sr = v_strides[2];
  p.o_sb = o_strides[0]; p.o_sh = o_strides[1]; p.o_sr = o_strides[2];
  p.mask = mptr; p.mask_rs = mask_row_stride;
  p.bias = bias; p.bias_rs = bias_row_stride; p.bias_cs = bias_col_stride;
  p.batch = batch; p.kv_heads = kv_heads; p.groups = groups; p.q_len = q_len; p.kv_len = kv_len;
  p.d = head_dim; p.dv = value_dim;
  p.causal = causal; p.causal_off = causal_offset;
  p.scale = scale; p.dt = dtype;
  // few query rows per K/V head (decode): split the keys over CTAs, merge through a scratch buffer
  const bool vec_ok = dtype != YTC_F32 ||
                      (k_strides[2] % 4 == 0 && k_strides[1] % 4 == 0 && k_strides[0] % 4 == 0 && v_strides[2] % 4 == 0 &&
                       v_strides[1] % 4 == 0 && v_strides[0] % 4 == 0 && (reinterpret_cast<uint64_t>(K) & 15) == 0 &&
                       (reinterpret_cast<uint64_t>(V) & 15) == 0);
  if (groups * q_len <= DEC_MAX_ROWS && head_dim % 4 == 0 && value_dim % 4 == 0 && head_dim <= 128 * DEC_MAX_VEC &&
      value_dim <= 128 * DEC_MAX_VEC && kv_len > 0 && vec_ok && static_cast<int64_t>(batch) * kv_heads <= 65535) {
    AttnDecodeParams dp;
    dp.a = p;
    const int bk = batch * kv_heads;
    int splits = (2 * sm_count() + bk - 1) / bk;
    const int max_splits = (kv_len + 31) / 32;
    if (splits > max_splits) splits = max_splits;
    if (splits < 1) splits = 1;
    dp.keys_per_split = (kv_len + splits - 1) / splits;
    dp.splits = (kv_len + dp.keys_per_split - 1) / dp.keys_per_split;
    const size_t need = static_cast<size_t>(bk) * dp.splits * groups * q_len * (2 + value_dim) * sizeof(float);
    dp.part = static_cast<float*>(device_workspace(need, st));
    if (!dp.part) {
      set_last_error("ytcuda_flash_attn_fwd: cannot allocate %zu bytes of scratch", need);
      return YTC_CUDA_ERROR;
    }
    const bool fast = dtype == YTC_F32 && q_len == 1 && head_dim == 128 && value_dim == 128 && !mptr && !bias &&
                      (groups == 1 || groups == 2 || groups == 4) && q_strides[1] % 4 == 0 && q_strides[0] % 4 == 0 &&
                      (reinterpret_cast<uint64_t>(Q) & 15) == 0 && g_attn_path != 1;
    if (fast) {
      if (groups == 1) YTC_CUDA(launch_overlapped(attn_decode_fast_kernel<1>, dim3(dp.splits, bk), dim3(DF_WARPS * 32), 0, st, dp));
      else if (groups == 2) YTC_CUDA(launch_overlapped(attn_decode_fast_kernel<2>, dim3(dp.splits, bk), dim3(DF_WARPS * 32), 0, st, dp));
      else YTC_CUDA(launch_overlapped(attn_decode_fast_kernel<4>, dim3(dp.splits, bk), dim3(DF_WARPS * 32), 0, st, dp));
    } else {
      attn_decode_kernel<<<dim3(dp.splits, bk), DEC_WARPS * 32, 0, st>>>(dp);
    }
    YTC_CUDA(launch_overlapped(attn_decode_merge_kernel, dim3(bk), dim3(128), 0, st, dp));
    count_launch(2);
    YTC_CUDA(cudaGetLastError());
    return YTC_OK;
  }
  if (dtype == YTC_F32 && q_len >= 64 && head_dim <= 128 && value_dim <= 128 && heads <= 65535 && batch <= 65535 &&
      vec_ok && head_dim % 4 == 0 && value_dim % 4 == 0 && q_strides[0] % 4 == 0 && q_strides[1] % 4 == 0 &&
      q_strides[2] % 4 == 0 && (reinterpret_cast<uint64_t>(Q) & 15) == 0) {
    dim3 grid((q_len + T64_BM - 1) / T64_BM, heads, batch);
    const int sa = ensure_dynamic_smem(reinterpret_cast<const void*>(attn_tile64_kernel), T64_SMEM);
    if (sa != YTC_OK) return sa;
    YTC_CUDA(launch_overlapped(attn_tile64_kernel, dim3(grid), dim3(256), T64_SMEM, st, p));
    count_launch();
    YTC_CUDA(cudaGetLastError());
    return YTC_OK;
  }
  if (head_dim <= TL_D && value_dim <= TL_D && heads <= 65535 && batch <= 65535) {
    dim3 grid((q_len + TL_BM - 1) / TL_BM, heads, batch);
    constexpr int TL_SMEM = ((TL_BM + 2 * TL_BN) * (TL_D + TL_PAD) + TL_BM * (TL_BN + 1)) * 4;
    const int sa = ensure_dynamic_smem(reinterpret_cast<const void*>(attn_tile_kernel), TL_SMEM);
    if (sa != YTC_OK) return sa;
    attn_tile_kernel<<<grid, 128, TL_SMEM, st>>>(p);
    count_launch();
    YTC_CUDA(cudaGetLastError());
    return YTC_OK;
  }
  const int64_t rows = static_cast<int64_t>(batch) * heads * q_len;
  const int64_t blocks = (rows + 3) / 4;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  attn_simt_kernel<<<static_cast<unsigned>(blocks < cap ? blocks : cap), 128, 0, st>>>(p);
  count_launch();
  YTC_CUDA(cudaGetLastError());
  return YTC_OK;
}

}  // extern "C"
