// The decode step kernel with its weights streamed through shared memory (up to four sequences).
//
// decode_step_kernel (decode_step.cuh) starts every phase with its weight rows still in L2 or HBM: the loads of a
// phase are issued after the barrier before it, so each of the 141 phases of a step pays a trip to memory on top of
// the barrier. The weights never depend on the activations, so here they do not wait for anything: every CTA owns a
// FIXED, contiguous block of rows of every weight matrix, which makes the bytes it will read during the whole step
// one known sequence of "chunks" (whole rows, at most 24 KB). The chunks flow through a ring of shared-memory slots
// filled by bulk async copies (cp.async.bulk, completion on an mbarrier) that run ahead of the computation by the
// depth of the ring (about 190 KB per SM, most of one layer's share): by the time a barrier releases a phase, its
// weights are already in shared memory, and HBM keeps streaming across the barriers.
//
//   * chunk c lives in slot c % NSLOT; a warp that has finished its rows of a chunk counts itself off on the slot,
//     and the LAST warp to do so issues the copy of chunk c + NSLOT into the slot it has just freed. Nobody ever
//     waits for a free slot, so there is no producer warp and no producer / consumer deadlock to think about.
//   * within a chunk, row i belongs to warp i % 8; lanes split k (128-bit shared-memory loads of 8 bf16 weights,
//     fp32 FMA chains, shuffles at the end of the row), two rows per warp at a time; gate / up rows of the fused
//     FFN weight travel in the same chunk (two copies) so that swish(gate) * up forms in the warp that owns the pair.
//   * the phases, their barriers, the attention phase, the embedding and the tensor-parallel exchange are those of
//     decode_step_kernel (same functions); only the linear phases differ. Arithmetic per output is the same chain of
//     FMAs along k as there, so results agree with it to rounding.
//
// Bounded waits: the wait for a chunk's mbarrier gives up after the run-time cycle budget like every other wait; a
// CTA that gives up raises the status word, releases the grid barrier for everyone, and before it returns waits
// (bounded again) for the copies still in flight into its shared memory.
#pragma once

#include "decode_step.cuh"
#include "ptx_sm100.cuh"

namespace ytk {

constexpr int DW_CHUNK = 24576;   // bytes per ring slot
constexpr int DW_MAX_SLOTS = 8;
constexpr int DW_MAX_LAYERS = 128;
constexpr int DW_KINDS = 5;       // 0 qkv, 1 o, 2 gate / up (pairs of rows), 3 down, 4 vocabulary projection

struct DwPhase {
  int r0, rows;   // this CTA's rows of the matrix (pairs for kind 2)
  int rpc;        // rows (pairs) per chunk
  int nchunks;
  int K;
};

struct DwDesc {  // one chunk of a layer, the same for every layer up to the weight's base address
  int64_t off;    // element offset of its first row in the weight
  int64_t off2;   // element offset of the up rows of a gate / up chunk
  uint32_t bytes; // bytes of one copy
  int kind;
};
constexpr int DW_MAX_DESC = 24;

struct DwShared {
  uint64_t full[DW_MAX_SLOTS];
  int done[DW_MAX_SLOTS];
  int abort_word;
  int issued;       // chunks whose copies have been issued (index of the last one + 1)
  int per_layer;    // chunks of this CTA per layer
  int total;        // chunks of this CTA per step
  int nslot;
  int consumed;     // barrier-free kernel: chunks the workers have finished with
  int issuer_done;  // barrier-free kernel: the issuing warp has stopped
  int pad[1];
  DwPhase ph[DW_KINDS];
  DwDesc desc[DW_MAX_DESC];             // the chunks of one layer in order (when they fit the table)
  const uint16_t* w[DW_MAX_LAYERS][4];  // qkv, o, gate_up, down of every layer
  const float* nw[DW_MAX_LAYERS][4];    // q_norm, k_norm, norm1, norm2 of every layer
};

__device__ __forceinline__ void dw_bulk_copy(void* dst_smem, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst_smem)),
               "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

struct DwChunk {
  int kind, n0, nrows, K;
  const uint16_t* W;
};

__device__ __forceinline__ DwChunk dw_chunk_info(const DwShared& S, const DecodeStepParams& p, int c) {
  DwChunk ci;
  int r;
  if (c < p.layers * S.per_layer) {
    const int l = c / S.per_layer;
    r = c - l * S.per_layer;
    int kind = 0;
    while (r >= S.ph[kind].nchunks) {
      r -= S.ph[kind].nchunks;
      ++kind;
    }
    ci.kind = kind;
    ci.W = S.w[l][kind];
  } else {
    r = c - p.layers * S.per_layer;
    ci.kind = 4;
    ci.W = p.lm_head;
  }
  const DwPhase& ph = S.ph[ci.kind];
  ci.K = ph.K;
  ci.n0 = ph.r0 + r * ph.rpc;
  const int left = ph.r0 + ph.rows - ci.n0;
  ci.nrows = left < ph.rpc ? left : ph.rpc;
  return ci;
}

// Issues the copies of chunk c into its slot (one thread).
__device__ __forceinline__ void dw_issue(DwShared& S, const DecodeStepParams& p, char* ring, int c) {
  const DwChunk ci = dw_chunk_info(S, p, c);
  const int slot = c % S.nslot;
  char* dst = ring + static_cast<size_t>(slot) * DW_CHUNK;
  const uint32_t bytes = static_cast<uint32_t>(ci.nrows) * static_cast<uint32_t>(ci.K) * 2u;
  const bool pair = ci.kind == 2;
  // (the warps' reads of the slot precede this call through a block-wide or warp-level synchronisation; a copy that
  // overwrites data which has only been READ needs no proxy fence)
  mbar_expect_tx(&S.full[slot], pair ? 2u * bytes : bytes);
  dw_bulk_copy(dst, ci.W + static_cast<int64_t>(ci.n0) * ci.K, bytes, &S.full[slot]);
  if (pair) dw_bulk_copy(dst + bytes, ci.W + static_cast<int64_t>(p.inter + ci.n0) * ci.K, bytes, &S.full[slot]);
  atomicMax(&S.issued, c + 1);
}

// The issuing side of the ring when ONE thread issues every chunk in order: it keeps the position of the next chunk
// (layer, index within the layer, slot) in registers and reads the layer-independent part from the table in shared
// memory, so that issuing a chunk costs a few dozen instructions.
struct DwIssuer {
  int layer, idx, slot, next;  // next = number of the next chunk to issue
};
__device__ __forceinline__ void dw_fill_desc(DwShared& S, const DecodeStepParams& p) {
  int n = 0;
  for (int kind = 0; kind < 4; ++kind) {
    const DwPhase& ph = S.ph[kind];
    for (int j = 0; j < ph.nchunks; ++j, ++n) {
      if (n >= DW_MAX_DESC) continue;
      const int n0 = ph.r0 + j * ph.rpc;
      const int left = ph.r0 + ph.rows - n0;
      const int nrows = left < ph.rpc ? left : ph.rpc;
      DwDesc d;
      d.off = static_cast<int64_t>(n0) * ph.K;
      d.off2 = static_cast<int64_t>(p.inter + n0) * ph.K;
      d.bytes = static_cast<uint32_t>(nrows) * static_cast<uint32_t>(ph.K) * 2u;
      d.kind = kind;
      S.desc[n] = d;
    }
  }
}
__device__ __forceinline__ void dw_issue_next(DwShared& S, const DecodeStepParams& p, char* ring, DwIssuer& it) {
  if (it.next >= S.total) return;
  if (S.per_layer > DW_MAX_DESC) {  // (a shape with more chunks per layer than the table holds: the general form)
    dw_issue(S, p, ring, it.next);
  } else {
    char* dst = ring + static_cast<size_t>(it.slot) * DW_CHUNK;
    uint64_t* bar = &S.full[it.slot];
    if (it.layer < p.layers) {
      const DwDesc d = S.desc[it.idx];
      const uint16_t* W = S.w[it.layer][d.kind];
      const bool pair = d.kind == 2;
      mbar_expect_tx(bar, pair ? 2u * d.bytes : d.bytes);
      dw_bulk_copy(dst, W + d.off, d.bytes, bar);
      if (pair) dw_bulk_copy(dst + d.bytes, W + d.off2, d.bytes, bar);
      if (++it.idx == S.per_layer) {
        it.idx = 0;
        ++it.layer;
      }
    } else {
      const DwPhase& ph = S.ph[4];
      const int n0 = ph.r0 + it.idx * ph.rpc;
      const int left = ph.r0 + ph.rows - n0;
      const uint32_t bytes = static_cast<uint32_t>(left < ph.rpc ? left : ph.rpc) * static_cast<uint32_t>(ph.K) * 2u;
      mbar_expect_tx(bar, bytes);
      dw_bulk_copy(dst, p.lm_head + static_cast<int64_t>(n0) * ph.K, bytes, bar);
      ++it.idx;
    }
    S.issued = it.next + 1;
  }
  ++it.next;
  if (++it.slot == S.nslot) it.slot = 0;
}

// One linear phase: stage the activations (they depend on the barrier just passed), then walk this CTA's chunks of
// the phase. `c` is the running chunk number (the same in every thread). Returns false when a wait gave up.
// stage: 0 xs = rmsNorm(src) * norm_w, 1 xs = src, 2 xs = attention output combined from the partials in src.
// epi: 0 dst = y, 1 dst += y, 2 dst = swish(y_gate) * y_up.
template <int MT>
__device__ __noinline__ bool dw_linear(const DecodeStepParams& p, DwShared& S, char* ring, float* xs, int kind, int stage,
                                       const float* src, const float* norm_w, int epi, float* dst, int ld,
                                       unsigned int barrier_no, int& c) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const DwPhase ph = S.ph[kind];
  const int K = ph.K, B = p.B;
  if (stage == 0) ds_stage_rmsnorm(xs, K, src, norm_w, B, K, p.eps, warp, lane);
  else if (stage == 1) ds_stage_copy(xs, K, src, B, K, 0, K);
  else ds_stage_attention(xs, K, src, B, p.heads, p.kv_heads, p.chunks, 0, K);
  ds_trace(p, barrier_no, 2);
  const bool pair = kind == 2;
  for (int j = 0; j < ph.nchunks; ++j, ++c) {
    const int slot = c % S.nslot;
    if (!mbar_wait_limit(&S.full[slot], static_cast<uint32_t>((c / S.nslot) & 1), &S.abort_word, p.wait_cycles))
      return false;
    const int n0 = ph.r0 + j * ph.rpc;
    const int left = ph.r0 + ph.rows - n0;
    const int nrows = left < ph.rpc ? left : ph.rpc;
    const char* base = ring + static_cast<size_t>(slot) * DW_CHUNK;
    const int64_t row_bytes = static_cast<int64_t>(K) * 2;
    // rows i0 and i1 of the chunk at a time: a gate / up pair, or two rows of this warp
    for (int i0 = warp; i0 < nrows; i0 += pair ? DS_WARPS : 2 * DS_WARPS) {
      const int i1 = i0 + DS_WARPS;
      const bool two = pair || i1 < nrows;
      const char* w0 = base + i0 * row_bytes;
      const char* w1 = pair ? base + (nrows + i0) * row_bytes : base + (two ? i1 : i0) * row_bytes;
      float acc0[MT], acc1[MT];
#pragma unroll
      for (int m = 0; m < MT; ++m) acc0[m] = acc1[m] = 0.f;
      for (int k = lane * 8; k < K; k += 256) {
        const uint4 a = *reinterpret_cast<const uint4*>(w0 + k * 2);
        const uint4 b = *reinterpret_cast<const uint4*>(w1 + k * 2);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          const float4 xa = *reinterpret_cast<const float4*>(&xs[m * K + k]);
          const float4 xb = *reinterpret_cast<const float4*>(&xs[m * K + k + 4]);
          acc0[m] = ds_dot8(a, xa, xb, acc0[m]);
          acc1[m] = ds_dot8(b, xa, xb, acc1[m]);
        }
      }
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        acc0[m] = ds_warp_sum(acc0[m]);
        acc1[m] = ds_warp_sum(acc1[m]);
      }
      if (lane == 0) {
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          if (m >= B) break;
          float* d0 = dst + static_cast<int64_t>(m) * ld + n0 + i0;
          if (epi == 2) {
            *d0 = ds_swish(acc0[m]) * acc1[m];
          } else if (epi == 1) {  // this warp is the only writer of these elements
            *d0 = acc0[m] + ds_ldcg(d0);
            if (two) d0[DS_WARPS] = acc1[m] + ds_ldcg(d0 + DS_WARPS);
          } else {
            *d0 = acc0[m];
            if (two) d0[DS_WARPS] = acc1[m];
          }
        }
      }
    }
    // count this warp off the slot; the last one refills it
    __syncwarp();
    if (lane == 0) {
      __threadfence_block();
      const int old = atomicAdd(&S.done[slot], 1);
      if (old == DS_WARPS - 1) {
        S.done[slot] = 0;
        __threadfence_block();
        if (c + S.nslot < S.total) dw_issue(S, p, ring, c + S.nslot);
      }
    }
  }
  return true;
}

// After a give-up: raise the status, release everyone at the grid barrier, and wait (bounded) for the copies that are
// still on their way into this CTA's shared memory.
__device__ __noinline__ void dw_abort(const DecodeStepParams& p, DwShared& S, int c) {
  __syncthreads();
  if (threadIdx.x == 0) {
    atomicExch(p.status, YTC_TIMEOUT);
    atomicOr(p.sync, 0x80000000u);
    const int issued = S.issued;
    int dummy = 0;
    for (int x = c; x < issued; ++x)
      mbar_wait_limit(&S.full[x % S.nslot], static_cast<uint32_t>((x / S.nslot) & 1), &dummy, p.wait_cycles);
  }
  __syncthreads();
}

__device__ __noinline__ bool dw_grid_sync(const DecodeStepParams& p, unsigned int& epoch) { return ds_grid_sync(p, epoch); }

template <int MT, int G>
__global__ void __launch_bounds__(DS_THREADS, 1) decode_stream_kernel(const DecodeStepParams p) {
  extern __shared__ __align__(128) char dw_smem[];
  // layout: DwShared | xs (p.xs_cols floats per row x MT rows, or the attention scratch) | ring (128-byte aligned)
  DwShared& S = *reinterpret_cast<DwShared*>(dw_smem);
  float* xs = reinterpret_cast<float*>(dw_smem + ((sizeof(DwShared) + 127) / 128) * 128);
  char* ring = reinterpret_cast<char*>(xs) + p.dw_xs_bytes;
  constexpr int D = 128;
  const int B = p.B, H = p.hidden;
  const int qkv_w = (p.heads + 2 * p.kv_heads) * D;
  const int attn_w = p.heads * D;
  unsigned int epoch = 0;
  unsigned int ar = 0;

  if (threadIdx.x == 0) {
    S.abort_word = 0;
    S.issued = 0;
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
      ph.nchunks = (ph.rows + ph.rpc - 1) / ph.rpc;
      S.ph[kd] = ph;
      if (kd < 4) per_layer += ph.nchunks;
    }
    S.per_layer = per_layer;
    S.total = per_layer * p.layers + S.ph[4].nchunks;
  }
  for (int i = threadIdx.x; i < p.layers; i += DS_THREADS) {
    const DsLayer W = p.lw[i];
    S.w[i][0] = W.qkv;
    S.w[i][1] = W.o;
    S.w[i][2] = W.gate_up;
    S.w[i][3] = W.down;
  }
  __syncthreads();
  if (threadIdx.x == 0) {  // the ring fills while the embedding is gathered
    const int first = S.total < S.nslot ? S.total : S.nslot;
    for (int c0 = 0; c0 < first; ++c0) dw_issue(S, p, ring, c0);
  }
  int c = 0;  // chunks consumed so far

  // ---- embedding gather: x[b, :] = float(embed[ids[b], :])
  {
    const int per_row = H / 4;
    for (int i = blockIdx.x * DS_THREADS + threadIdx.x; i < B * per_row; i += gridDim.x * DS_THREADS) {
      const int b = i / per_row, col = (i - b * per_row) * 4;
      int id = p.ids[b];
      id = id < 0 ? 0 : (id >= p.vocab ? p.vocab - 1 : id);
      const uint2 w = __ldg(reinterpret_cast<const uint2*>(p.embed + static_cast<int64_t>(id) * H + col));
      float4 o;
      o.x = __uint_as_float(w.x << 16);
      o.y = __uint_as_float(w.x & 0xFFFF0000u);
      o.z = __uint_as_float(w.y << 16);
      o.w = __uint_as_float(w.y & 0xFFFF0000u);
      *reinterpret_cast<float4*>(p.x + static_cast<int64_t>(b) * H + col) = o;
    }
  }
#define DW_SYNC()                     \
  do {                                \
    if (!dw_grid_sync(p, epoch)) {    \
      dw_abort(p, S, c);              \
      return;                         \
    }                                 \
  } while (0)
#define DW_LINEAR(...)                          \
  do {                                          \
    if (!dw_linear<MT>(p, S, ring, xs, __VA_ARGS__, epoch / gridDim.x - 1, c)) { \
      dw_abort(p, S, c);                        \
      return;                                   \
    }                                           \
  } while (0)
  DW_SYNC();

  // K / V rows of this CTA's first attention unit, requested into the L2 one phase ahead
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
      const char* kr = reinterpret_cast<const char*>(kc + kv_off);
      const char* vr = reinterpret_cast<const char*>(vc + kv_off);
      for (int i = threadIdx.x; i < kv_lines; i += DS_THREADS) {
        asm volatile("prefetch.global.L2 [%0];" ::"l"(kr + i * 128));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(vr + i * 128));
      }
    }
    // ---- qkv = rmsNorm(x) . Wqkv^T
    DW_LINEAR(0, 0, p.x, W.norm1, 0, p.qkv, qkv_w);
    DW_SYNC();
    // ---- attention over the cache (+ per-head rmsNorm, RoPE, KV append)
    ds_attention_phase<G>(p, W, kc, vc, xs);
    DW_SYNC();
    // ---- x += attn . Wo^T
    if (p.tp_world > 1) {
      DW_LINEAR(1, 2, p.part, nullptr, 0, p.mail[p.tp_rank] + static_cast<int64_t>((p.ar_base + ar) & 1) * DS_MAX_B * H, H);
      if (!ds_cross_sync(p, epoch, p.ar_base + ar + 1)) {
        dw_abort(p, S, c);
        return;
      }
      ds_reduce_mailboxes(p, (p.ar_base + ar) & 1);
      ++ar;
    } else {
      DW_LINEAR(1, 2, p.part, nullptr, 1, p.x, H);
    }
    DW_SYNC();
    // ---- act = swish(gate) * up, gate / up = rmsNorm(x) . Wgu^T
    DW_LINEAR(2, 0, p.x, W.norm2, 2, p.act, p.inter);
    DW_SYNC();
    // ---- x += act . Wdown^T
    if (p.tp_world > 1) {
      DW_LINEAR(3, 1, p.act, nullptr, 0, p.mail[p.tp_rank] + static_cast<int64_t>((p.ar_base + ar) & 1) * DS_MAX_B * H, H);
      if (!ds_cross_sync(p, epoch, p.ar_base + ar + 1)) {
        dw_abort(p, S, c);
        return;
      }
      ds_reduce_mailboxes(p, (p.ar_base + ar) & 1);
      ++ar;
    } else {
      DW_LINEAR(3, 1, p.act, nullptr, 1, p.x, H);
    }
    DW_SYNC();
  }
  // ---- logits = rmsNorm(x) . Wvocab^T
  DW_LINEAR(4, 0, p.x, p.final_norm, 0, p.logits, p.vocab_rows);
#undef DW_SYNC
#undef DW_LINEAR
}

}  // namespace ytk
