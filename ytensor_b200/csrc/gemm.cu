// GEMM for the YTensor device backend.
//
//  * gemm_tc_kernel   : bf16 / fp16 inputs, fp32 accumulation in tensor memory. Persistent,
//                       one CTA per SM, warp-specialised: warp 0 feeds a 4-stage shared-memory
//                       ring with TMA, warp 1 issues tcgen05.mma (128 x BN x 16 per instruction),
//                       warps 4-7 drain the accumulator (tcgen05.ld) and write C while the next
//                       tile's MMAs run into the second accumulator stage.
//  * gemm_simt_kernel : any strides, any of {f32, bf16, f16}, FFMA with fp32 accumulation.
//                       It is the fp32 path and the layout catch-all of the tensor-core path.
//
// Replaces yt::kernel::avx2::sgemm / matmul / hgemm (reference src/kernel/avx2/sgemm.inl:586-806,
// src/kernel/avx2/hgemm.inl:139-288) behind ytcuda_gemm.
#include <atomic>

#include "ptx_sm100.cuh"
#include "ytc_common.cuh"

namespace ytk {

// ------------------------------------------------------------------ tcgen05 path
constexpr int TC_BM = 128;
constexpr int TC_BK = 64;  // 64 x 16-bit = one 128-byte swizzle row
constexpr int TC_STAGES = 4;
constexpr int TC_THREADS = 256;

struct GemmTcParams {
  int M, N, K;
  int batch;
  int a_mn, b_mn;        // 1 = the operand's unit stride runs along M (A) / N (B), 0 = along K
  int a_bcast, b_bcast;  // 1 = operand shared by all batch items
  uint32_t idesc;
  float alpha, beta;
  void* C;
  int64_t rsc, csc, bsc;
  int out_dtype;
  int tiles_m, tiles_n, total_tiles, k_blocks;
  int a_prefetch;  // k-blocks by which an L2 prefetch of A runs ahead of the shared-memory loads (0 = off)
  int split_loads; // K-major tiles fetched as 64-row boxes
  int* status;
  // masked product: tile_live[mb * tiles_n + nb] == 0 marks an output tile no element of which is asked for; every
  // role of the kernel passes over it (no loads, no MMAs, no stores). NULL = every tile is computed.
  const uint8_t* tile_live;
};

template <int BN>
struct TcSmem {
  static constexpr int A_BYTES = TC_BM * TC_BK * 2;
  static constexpr int B_BYTES = BN * TC_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = TC_STAGES * STAGE_BYTES;
  // full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], tmem base word, abort word
  static constexpr int TOTAL = BAR_OFFSET + (2 * TC_STAGES + 4) * 8 + 16;
  static constexpr int DYN_BYTES = TOTAL + 1024;  // slack to align the ring to 1024 B
};

template <int BN, int OUT_DT>
__device__ __forceinline__ void tc_store_chunk(const GemmTcParams& p, const uint32_t (&r)[32], int64_t row_off,
                                               int gn0, bool row_ok, bool vec_ok) {
  // One thread holds 32 consecutive columns of one row.
  if (!row_ok) return;
  char* cbase = static_cast<char*>(p.C);
  const float alpha = p.alpha, beta = p.beta;
  if (vec_ok && gn0 + 32 <= p.N) {
    if constexpr (OUT_DT == YTC_F32) {
      float4* dst = reinterpret_cast<float4*>(cbase + (row_off + gn0) * 4);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float4 v;
        v.x = alpha * __uint_as_float(r[4 * j + 0]);
        v.y = alpha * __uint_as_float(r[4 * j + 1]);
        v.z = alpha * __uint_as_float(r[4 * j + 2]);
        v.w = alpha * __uint_as_float(r[4 * j + 3]);
        if (beta != 0.f) {
          float4 o = dst[j];
          v.x += beta * o.x; v.y += beta * o.y; v.z += beta * o.z; v.w += beta * o.w;
        }
        dst[j] = v;
      }
    } else {
      uint4* dst = reinterpret_cast<uint4*>(cbase + (row_off + gn0) * 2);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float v[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) v[t] = alpha * __uint_as_float(r[8 * j + t]);
        if (beta != 0.f) {
          uint4 o = dst[j];
          const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const uint16_t lo = static_cast<uint16_t>(ow[t] & 0xFFFFu), hi = static_cast<uint16_t>(ow[t] >> 16);
            if constexpr (OUT_DT == YTC_BF16) {
              v[2 * t] += beta * bf16_bits_to_f32(lo);
              v[2 * t + 1] += beta * bf16_bits_to_f32(hi);
            } else {
              v[2 * t] += beta * f16_bits_to_f32_ref(lo);
              v[2 * t + 1] += beta * f16_bits_to_f32_ref(hi);
            }
          }
        }
        uint32_t w[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          uint16_t lo, hi;
          if constexpr (OUT_DT == YTC_BF16) {
            lo = f32_to_bf16_bits_ref(v[2 * t]);
            hi = f32_to_bf16_bits_ref(v[2 * t + 1]);
          } else {
            lo = f32_to_f16_bits_ref(v[2 * t]);
            hi = f32_to_f16_bits_ref(v[2 * t + 1]);
          }
          w[t] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
        }
        dst[j] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
  } else {
#pragma unroll 4
    for (int j = 0; j < 32; ++j) {
      const int gn = gn0 + j;
      if (gn < p.N) {
        const int64_t idx = row_off + static_cast<int64_t>(gn) * p.csc;
        float v = alpha * __uint_as_float(r[j]);
        if (beta != 0.f) v += beta * DType<OUT_DT>::load(p.C, idx);
        DType<OUT_DT>::store(p.C, idx, v);
      }
    }
  }
}

template <int BN>
__global__ void __launch_bounds__(TC_THREADS, 1)
    gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   const GemmTcParams p) {
  using S = TcSmem<BN>;
  extern __shared__ uint8_t smem_raw[];
  // The 128-byte swizzle pattern is a function of the shared address: keep the ring 1024-byte aligned.
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);

  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + TC_STAGES;
  uint64_t* tfull_bar = empty_bar + TC_STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < TC_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&tfull_bar[s], 1);
      mbar_init(&tempty_bar[s], 4);
    }
    *abort_word = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Everything above touched shared and tensor memory only: under a programmatic dependent launch it ran while the
  // kernel before this one was finishing. From here on global memory is read and written.
  dependent_wait();
  dependent_trigger();

  const int tiles_per_batch = p.tiles_m * p.tiles_n;

  if (warp == 0) {
    // ------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int issued = 0;
      bool ok = true;
      // A is streamed from HBM once; an L2 prefetch a few k-blocks ahead of the shared-memory ring
      // takes the DRAM latency off the ring (B is small and stays L2-resident by reuse).
      auto prefetch_a = [&](int tile, int kb) {
        if (tile >= p.total_tiles) return;
        const int b = tile / tiles_per_batch;
        const int rem = tile - b * tiles_per_batch;
        const int mb = rem / p.tiles_n;
        const int ba = p.a_bcast ? 0 : b;
        if (!p.a_mn) {
          tma_prefetch_l2_3d(&tmA, kb * TC_BK, mb * TC_BM, ba);
        } else {
#pragma unroll
          for (int c = 0; c < TC_BM / 64; ++c) tma_prefetch_l2_3d(&tmA, mb * TC_BM + c * 64, kb * TC_BK, ba);
        }
      };
      int pf_tile = blockIdx.x, pf_kb = 0;
      if (p.a_prefetch > 0) {
        for (int i = 0; i < p.a_prefetch; ++i) {
          prefetch_a(pf_tile, pf_kb);
          if (++pf_kb == p.k_blocks) {
            pf_kb = 0;
            pf_tile += gridDim.x;
          }
        }
      }
      for (int tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x) {
        const int b = tile / tiles_per_batch;
        const int rem = tile - b * tiles_per_batch;
        if (p.tile_live && !p.tile_live[rem]) continue;
        const int mb = rem / p.tiles_n;
        const int nb = rem - mb * p.tiles_n;
        const int ba = p.a_bcast ? 0 : b;
        const int bb = p.b_bcast ? 0 : b;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_word)) {
            ok = false;
            break;
          }
          if (p.a_prefetch > 0) {
            prefetch_a(pf_tile, pf_kb);
            if (++pf_kb == p.k_blocks) {
              pf_kb = 0;
              pf_tile += gridDim.x;
            }
          }
          mbar_expect_tx(&full_bar[stage], S::STAGE_BYTES);
          uint8_t* sa = smem + stage * S::STAGE_BYTES;
          uint8_t* sb = sa + S::A_BYTES;
          if (!p.a_mn) {
            if (p.split_loads) {
#pragma unroll
              for (int c = 0; c < TC_BM / 64; ++c)
                tma_load_3d(sa + c * 8192, &tmA, &full_bar[stage], kb * TC_BK, mb * TC_BM + c * 64, ba);
            } else {
              tma_load_3d(sa, &tmA, &full_bar[stage], kb * TC_BK, mb * TC_BM, ba);
            }
          } else {
#pragma unroll
            for (int c = 0; c < TC_BM / 64; ++c)
              tma_load_3d(sa + c * 8192, &tmA, &full_bar[stage], mb * TC_BM + c * 64, kb * TC_BK, ba);
          }
          if (!p.b_mn) {
            if (p.split_loads) {
#pragma unroll
              for (int c = 0; c < BN / 64; ++c)
                tma_load_3d(sb + c * 8192, &tmB, &full_bar[stage], kb * TC_BK, nb * BN + c * 64, bb);
            } else {
              tma_load_3d(sb, &tmB, &full_bar[stage], kb * TC_BK, nb * BN, bb);
            }
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_3d(sb + c * 8192, &tmB, &full_bar[stage], nb * BN + c * 64, kb * TC_BK, bb);
          }
          ++issued;
          if (++stage == TC_STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        // Give the copies already in flight a bounded time to land before the CTA goes away.
        const int pending = issued < TC_STAGES ? issued : TC_STAGES;
        int s = stage;
        uint32_t ph = phase;
        for (int i = 0; i < pending; ++i) {
          if (--s < 0) {
            s = TC_STAGES - 1;
            ph ^= 1u;
          }
          const long long t0 = clock64();
          while (!mbar_try_wait(&full_bar[s], ph) && clock64() - t0 < 20000000ll) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x) {
        if (p.tile_live && !p.tile_live[tile % tiles_per_batch]) continue;
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1u, abort_word)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_word)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_base = smem_u32(smem + stage * S::STAGE_BYTES);
          const uint32_t b_base = a_base + S::A_BYTES;
#pragma unroll
          for (int k = 0; k < TC_BK / 16; ++k) {
            const uint64_t adesc = p.a_mn ? umma_smem_desc_sw128(a_base + k * 2048, 8192, 1024)
                                          : umma_smem_desc_sw128(a_base + k * 32, 16, 1024);
            const uint64_t bdesc = p.b_mn ? umma_smem_desc_sw128(b_base + k * 2048, 8192, 1024)
                                          : umma_smem_desc_sw128(b_base + k * 32, 16, 1024);
            tc_mma_f16(d_tmem, adesc, bdesc, p.idesc, (kb | k) != 0 ? 1u : 0u);
          }
          tc_commit(&empty_bar[stage]);  // frees the stage once these MMAs have read it
          if (++stage == TC_STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        tc_commit(&tfull_bar[acc]);  // accumulator complete
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------ epilogue (TMEM -> registers -> global)
    const int q = warp & 3;  // a warp may only touch TMEM lanes 32q .. 32q+31
    const int row = q * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    const bool c_unit = (p.csc == 1);
    const int esz = (p.out_dtype == YTC_F32) ? 4 : 2;
    for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x) {
      const int b = tile / tiles_per_batch;
      const int rem = tile - b * tiles_per_batch;
      if (p.tile_live && !p.tile_live[rem]) continue;
      const int mb = rem / p.tiles_n;
      const int nb = rem - mb * p.tiles_n;
      if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_word)) break;
      tc_fence_after();
      const int gm = mb * TC_BM + row;
      const bool row_ok = gm < p.M;
      const int64_t row_off = static_cast<int64_t>(b) * p.bsc + static_cast<int64_t>(gm) * p.rsc;
      const bool vec_ok =
          c_unit && (((reinterpret_cast<uint64_t>(p.C) + static_cast<uint64_t>(row_off) * esz) & 15u) == 0) &&
          ((static_cast<int64_t>(nb) * BN * esz & 15) == 0);
      const uint32_t t_row = tmem_base + static_cast<uint32_t>(acc * BN) + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + c0, r);
        tmem_ld_wait();
        const int gn0 = nb * BN + c0;
        if (gn0 < p.N) {
          if (p.out_dtype == YTC_BF16) tc_store_chunk<BN, YTC_BF16>(p, r, row_off, gn0, row_ok, vec_ok);
          else if (p.out_dtype == YTC_F32) tc_store_chunk<BN, YTC_F32>(p, r, row_off, gn0, row_ok, vec_ok);
          else tc_store_chunk<BN, YTC_F16>(p, r, row_off, gn0, row_ok, vec_ok);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
  if (threadIdx.x == 0 && *abort_word) atomicExch(p.status, YTC_TIMEOUT);
}


// ------------------------------------------------------------------ tcgen05 path, CTA pairs
// Two CTAs (a cluster of 2 on neighbouring SMs) share one 256 x 256 output tile: each loads its own 128 rows of A
// and HALF of the B tile (128 columns), the leader CTA issues 256 x 256 x 16 MMAs (cta_group::2) that read both
// halves, and each CTA drains its own 128 x 256 accumulator. Per SM this halves the B bytes moved through shared
// memory and leaves room for a 6-stage ring. Barriers: TMA completion of both CTAs is counted on the leader's
// `full` barrier; the leader's commits free the stage in both CTAs and publish the accumulator to both.
constexpr int TC2_STAGES = 6;
constexpr int TC2_BN = 256;

struct Tc2Smem {
  static constexpr int A_BYTES = TC_BM * TC_BK * 2;         // 128 rows of A
  static constexpr int B_BYTES = (TC2_BN / 2) * TC_BK * 2;  // 128 columns of B
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = TC2_STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + (2 * TC2_STAGES + 4) * 8 + 16;
  static constexpr int DYN_BYTES = TOTAL + 1024;
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TC_THREADS, 1)
    gemm_tc2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const GemmTcParams p) {
  using S = Tc2Smem;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + TC2_STAGES;
  uint64_t* tfull_bar = empty_bar + TC2_STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();  // 0 = leader
  const bool leader = cta == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < TC2_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&tfull_bar[s], 1);
      mbar_init(&tempty_bar[s], 8);  // 4 epilogue warps of each CTA
    }
    *abort_word = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 2) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // (set-up done in shared and tensor memory only; under a programmatic dependent launch global memory may be touched
  // from here on)
  dependent_wait();
  dependent_trigger();

  const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
  const int tiles_per_batch = p.tiles_m * p.tiles_n;

  if (warp == 0) {
    // ------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = cluster_id; ok && tile < p.total_tiles; tile += n_clusters) {
        const int b = tile / tiles_per_batch;
        const int rem = tile - b * tiles_per_batch;
        const int mb = rem / p.tiles_n;
        const int nb = rem - mb * p.tiles_n;
        const int ba = p.a_bcast ? 0 : b;
        const int bb = p.b_bcast ? 0 : b;
        const int m0 = mb * 256 + static_cast<int>(cta) * TC_BM;
        const int n0 = nb * TC2_BN + static_cast<int>(cta) * (TC2_BN / 2);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_word)) {
            ok = false;
            break;
          }
          const uint32_t full_leader = map_to_cta(smem_u32(&full_bar[stage]), 0);
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * S::STAGE_BYTES);
          uint8_t* sa = smem + stage * S::STAGE_BYTES;
          uint8_t* sb = sa + S::A_BYTES;
          if (!p.a_mn) {
            tma_load_3d_pair(sa, &tmA, full_leader, kb * TC_BK, m0, ba);
          } else {
#pragma unroll
            for (int c = 0; c < TC_BM / 64; ++c) tma_load_3d_pair(sa + c * 8192, &tmA, full_leader, m0 + c * 64, kb * TC_BK, ba);
          }
          if (!p.b_mn) {
            tma_load_3d_pair(sb, &tmB, full_leader, kb * TC_BK, n0, bb);
          } else {
#pragma unroll
            for (int c = 0; c < TC2_BN / 128; ++c) tma_load_3d_pair(sb + c * 8192, &tmB, full_leader, n0 + c * 64, kb * TC_BK, bb);
          }
          if (++stage == TC2_STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && leader) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = cluster_id; ok && tile < p.total_tiles; tile += n_clusters) {
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1u, abort_word)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * TC2_BN);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_word)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_base = smem_u32(smem + stage * S::STAGE_BYTES);
          const uint32_t b_base = a_base + S::A_BYTES;
#pragma unroll
          for (int k = 0; k < TC_BK / 16; ++k) {
            const uint64_t adesc = p.a_mn ? umma_smem_desc_sw128(a_base + k * 2048, 8192, 1024)
                                          : umma_smem_desc_sw128(a_base + k * 32, 16, 1024);
            const uint64_t bdesc = p.b_mn ? umma_smem_desc_sw128(b_base + k * 2048, 8192, 1024)
                                          : umma_smem_desc_sw128(b_base + k * 32, 16, 1024);
            tc_mma_f16_pair(d_tmem, adesc, bdesc, p.idesc, (kb | k) != 0 ? 1u : 0u);
          }
          // the stage is free in both CTAs once these MMAs have read it
          tc_commit_pair(smem_u32(&empty_bar[stage]));
          tc_commit_pair(map_to_cta(smem_u32(&empty_bar[stage]), 1));
          if (++stage == TC2_STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        tc_commit_pair(smem_u32(&tfull_bar[acc]));
        tc_commit_pair(map_to_cta(smem_u32(&tfull_bar[acc]), 1));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------ epilogue (both CTAs, own 128 rows x 256 columns)
    const int q = warp & 3;
    const int row = q * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    const bool c_unit = (p.csc == 1);
    const int esz = (p.out_dtype == YTC_F32) ? 4 : 2;
    for (int tile = cluster_id; tile < p.total_tiles; tile += n_clusters) {
      const int b = tile / tiles_per_batch;
      const int rem = tile - b * tiles_per_batch;
      const int mb = rem / p.tiles_n;
      const int nb = rem - mb * p.tiles_n;
      if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_word)) break;
      tc_fence_after();
      const int gm = mb * 256 + static_cast<int>(cta) * TC_BM + row;
      const bool row_ok = gm < p.M;
      const int64_t row_off = static_cast<int64_t>(b) * p.bsc + static_cast<int64_t>(gm) * p.rsc;
      const bool vec_ok =
          c_unit && (((reinterpret_cast<uint64_t>(p.C) + static_cast<uint64_t>(row_off) * esz) & 15u) == 0);
      const uint32_t t_row = tmem_base + static_cast<uint32_t>(acc * TC2_BN) + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c0 = 0; c0 < TC2_BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + c0, r);
        tmem_ld_wait();
        const int gn0 = nb * TC2_BN + c0;
        if (gn0 < p.N) {
          if (p.out_dtype == YTC_BF16) tc_store_chunk<TC2_BN, YTC_BF16>(p, r, row_off, gn0, row_ok, vec_ok);
          else if (p.out_dtype == YTC_F32) tc_store_chunk<TC2_BN, YTC_F32>(p, r, row_off, gn0, row_ok, vec_ok);
          else tc_store_chunk<TC2_BN, YTC_F16>(p, r, row_off, gn0, row_ok, vec_ok);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty_bar[acc]), 0));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves while the other may still read its shared or tensor memory
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_word) atomicExch(p.status, YTC_TIMEOUT);
}

// ------------------------------------------------------------------ FFMA path
constexpr int SM_BM = 128, SM_BN = 128, SM_BK = 16, SM_THREADS = 256, SM_PAD = 4;

struct GemmSimtParams {
  const void* A;
  const void* B;
  void* C;
  int M, N, K;
  int64_t rsa, csa, rsb, csb, rsc, csc, bsa, bsb, bsc;
  float alpha, beta;
  int in_dtype, out_dtype;
  int tiles_m, tiles_n;
  const uint8_t* tile_live;  // masked product: 0 marks a 128 x 128 output tile nobody asks for (NULL: all computed)
};

template <int IN_DT>
__global__ void __launch_bounds__(SM_THREADS) gemm_simt_kernel(const GemmSimtParams p) {
  __shared__ __align__(16) float As[2][SM_BK][SM_BM + SM_PAD];
  __shared__ __align__(16) float Bs[2][SM_BK][SM_BN + SM_PAD];

  const int tid = threadIdx.x;
  const int tile = blockIdx.x;
  if (p.tile_live && !p.tile_live[tile]) return;
  const int b = blockIdx.y;
  const int mb = tile / p.tiles_n, nb = tile - mb * p.tiles_n;
  const int m0 = mb * SM_BM, n0 = nb * SM_BN;
  const int64_t a_off = static_cast<int64_t>(b) * p.bsa;
  const int64_t b_off = static_cast<int64_t>(b) * p.bsb;

  // Loader mapping: consecutive threads walk the operand's unit-stride axis.
  const bool a_kfast = (p.csa == 1) || (p.rsa != 1);
  const bool b_nfast = (p.csb == 1) || (p.rsb != 1);

  float ra[8], rb[8];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int idx = tid + i * SM_THREADS;
      int m, kk;
      if (a_kfast) { kk = idx & (SM_BK - 1); m = idx >> 4; } else { m = idx & (SM_BM - 1); kk = idx >> 7; }
      const int gm = m0 + m, gk = k0 + kk;
      ra[i] = (gm < p.M && gk < p.K)
                  ? DType<IN_DT>::load(p.A, a_off + static_cast<int64_t>(gm) * p.rsa + static_cast<int64_t>(gk) * p.csa)
                  : 0.f;
      int n, kb;
      if (b_nfast) { n = idx & (SM_BN - 1); kb = idx >> 7; } else { kb = idx & (SM_BK - 1); n = idx >> 4; }
      const int gn = n0 + n, gk2 = k0 + kb;
      rb[i] = (gn < p.N && gk2 < p.K)
                  ? DType<IN_DT>::load(p.B, b_off + static_cast<int64_t>(gk2) * p.rsb + static_cast<int64_t>(gn) * p.csb)
                  : 0.f;
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int idx = tid + i * SM_THREADS;
      int m, kk;
      if (a_kfast) { kk = idx & (SM_BK - 1); m = idx >> 4; } else { m = idx & (SM_BM - 1); kk = idx >> 7; }
      As[buf][kk][m] = ra[i];
      int n, kb;
      if (b_nfast) { n = idx & (SM_BN - 1); kb = idx >> 7; } else { kb = idx & (SM_BK - 1); n = idx >> 4; }
      Bs[buf][kb][n] = rb[i];
    }
  };

  const int ty = tid >> 4, tx = tid & 15;
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  const int kt = (p.K + SM_BK - 1) / SM_BK;
  fetch(0);
  stash(0);
  __syncthreads();
  for (int t = 0; t < kt; ++t) {
    const int buf = t & 1;
    if (t + 1 < kt) fetch((t + 1) * SM_BK);
#pragma unroll
    for (int kk = 0; kk < SM_BK; ++kk) {
      const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][kk][ty * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][kk][64 + ty * 4]);
      const float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][kk][tx * 4]);
      const float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][kk][64 + tx * 4]);
      const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    if (t + 1 < kt) {
      stash(buf ^ 1);
      __syncthreads();
    }
  }

  const int64_t c_off = static_cast<int64_t>(b) * p.bsc;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int gm = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
    if (gm >= p.M) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int gn = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
      if (gn >= p.N) continue;
      const int64_t idx = c_off + static_cast<int64_t>(gm) * p.rsc + static_cast<int64_t>(gn) * p.csc;
      float v = p.alpha * acc[i][j];
      if (p.beta != 0.f) v += p.beta * load_as_f32(p.C, idx, p.out_dtype);
      store_from_f32(p.C, idx, v, p.out_dtype);
    }
  }
}

// beta-only update for k == 0 (C = beta * C), any strides.
__global__ void gemm_scale_c_kernel(void* C, int M, int N, int64_t rsc, int64_t csc, int64_t bsc, float beta,
                                    int out_dtype) {
  const int64_t total = static_cast<int64_t>(M) * N;
  const int64_t c_off = static_cast<int64_t>(blockIdx.y) * bsc;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t m = i / N, n = i - m * N;
    const int64_t idx = c_off + m * rsc + n * csc;
    const float v = (beta == 0.f) ? 0.f : beta * load_as_f32(C, idx, out_dtype);
    store_from_f32(C, idx, v, out_dtype);
  }
}

// ------------------------------------------------------------------ host dispatch
static bool tc_operand_ok(const void* ptr, int64_t rs, int64_t cs, int64_t bs, int64_t batch, int rows, int cols,
                          int* mn_major) {
  // rows x cols operand with the reduction axis K as `cols` for A (A[m,k]) and as `rows` for B (B[k,n]):
  // the caller passes (unit-stride axis along K ?) through which stride is 1.
  (void)rows;
  (void)cols;
  if ((reinterpret_cast<uint64_t>(ptr) & 15u) != 0) return false;
  int64_t lead;
  if (cs == 1) {
    *mn_major = 0;
    lead = rs;
  } else if (rs == 1) {
    *mn_major = 1;
    lead = cs;
  } else {
    return false;
  }
  if (lead <= 0 || (lead * 2) % 16 != 0) return false;
  if (batch > 1 && bs != 0 && (bs < 0 || (bs * 2) % 16 != 0)) return false;
  return true;
}

// L2 prefetch distance of the A operand in k-blocks (see GemmTcParams::a_prefetch).
static std::atomic<int> g_tc_a_prefetch{0};
// 1 = fetch K-major operand tiles as 64-row boxes instead of one tall box.
static std::atomic<int> g_tc_split_loads{0};
// CTA-pair kernel: 0 = automatic, 1 = whenever the layout allows, 2 = never.
static std::atomic<int> g_tc_pair{0};

// Masked products (YTensor::masked_matmul): what the entry point asked for, seen by the launchers below.
// kind 0: no mask; 1: bool matrix [m, n]; 2: the causal predicate j <= i + offset, evaluated on the device.
struct MaskCtx {
  int kind = 0;
  const uint8_t* mask = nullptr;
  int64_t row_stride = 0;
  int offset = 0;
};
static thread_local MaskCtx g_mask;

__device__ __forceinline__ bool mask_at(int kind, const uint8_t* mask, int64_t mrs, int offset, int i, int j) {
  return kind == 2 ? (j <= i + offset) : (mask[static_cast<int64_t>(i) * mrs + j] != 0);
}

// live[mb * tiles_n + nb] = 1 when some element of output tile (mb, nb) is asked for. The counterpart of the
// tileAllFalse test that lets the reference's sgemm_masked skip whole tiles (src/kernel/avx2/sgemm.inl:449-475).
__global__ void __launch_bounds__(256) gemm_tile_live_kernel(uint8_t* live, int kind, const uint8_t* mask, int64_t mrs,
                                                             int offset, int m, int n, int bm, int bn, int tiles_n) {
  const int mb = blockIdx.x / tiles_n, nb = blockIdx.x - mb * tiles_n;
  const int i0 = mb * bm, j0 = nb * bn;
  const int i1 = i0 + bm < m ? i0 + bm : m, j1 = j0 + bn < n ? j0 + bn : n;
  int any = 0;
  if (kind == 2) {
    any = j0 <= (i1 - 1) + offset;  // the tile's smallest column against its largest row
  } else {
    const int w = j1 - j0;
    for (int e = threadIdx.x; e < (i1 - i0) * w && !any; e += 256) {
      const int i = i0 + e / w, j = j0 + e % w;
      any = mask[static_cast<int64_t>(i) * mrs + j] != 0;
    }
  }
  any = __syncthreads_or(any);
  if (threadIdx.x == 0) live[blockIdx.x] = any ? 1 : 0;
}

// Tile liveness for the current mask and a bm x bn tiling, in stream-ordered scratch (freed by the caller's launcher
// after its kernel has been queued). NULL without a mask.
static int make_tile_live(int m, int n, int bm, int bn, cudaStream_t st, uint8_t** out) {
  *out = nullptr;
  if (g_mask.kind == 0) return YTC_OK;
  const int tiles_m = (m + bm - 1) / bm, tiles_n = (n + bn - 1) / bn;
  uint8_t* live = nullptr;
  YTC_CUDA(cudaMallocAsync(reinterpret_cast<void**>(&live), static_cast<size_t>(tiles_m) * tiles_n, st));
  gemm_tile_live_kernel<<<tiles_m * tiles_n, 256, 0, st>>>(live, g_mask.kind, g_mask.mask, g_mask.row_stride,
                                                          g_mask.offset, m, n, bm, bn, tiles_n);
  count_launch();
  *out = live;
  return YTC_OK;
}

static int launch_tc(int dtype_in, int dtype_out, const void* A, const void* B, void* C, int m, int n, int k,
                     float alpha, float beta, int a_mn, int64_t lda, int b_mn, int64_t ldb, int64_t rsc, int64_t csc,
                     int64_t batch, int64_t bsa, int64_t bsb, int64_t bsc, cudaStream_t st) {
  // A: unit axis = K (a_mn 0, dims {K, M}) or M (a_mn 1, dims {M, K}). B likewise with N.
  CUtensorMap tmA, tmB;
  const int a_bcast = (batch > 1 && bsa == 0) ? 1 : 0;
  const int b_bcast = (batch > 1 && bsb == 0) ? 1 : 0;
  // 256-wide tiles unless the problem is narrow or would leave most SMs without a tile
  const int BN = (n <= 128 || static_cast<int64_t>((m + 127) / 128) * ((n + 255) / 256) * batch < sm_count() / 2) ? 128 : 256;
  // CTA pairs pay off on large problems; small ones keep one CTA per tile (more tiles to spread over the SMs)
  // (a masked product keeps one CTA per tile: the tile-skipping form of the kernel)
  const bool pair = g_mask.kind == 0 && g_tc_pair != 2 &&
                    (g_tc_pair == 1 || (m >= 512 && n >= 256 && k >= 256 &&
                                        static_cast<int64_t>((m + 255) / 256) * ((n + 255) / 256) * batch >= 74));
  {
    const uint64_t nb = (a_bcast || batch == 1) ? 1 : static_cast<uint64_t>(batch);
    uint64_t dims[3], strides[2];
    uint32_t box[3];
    if (!a_mn) { dims[0] = k; dims[1] = m; box[0] = TC_BK; box[1] = g_tc_split_loads ? 64 : TC_BM; }
    else       { dims[0] = m; dims[1] = k; box[0] = 64;    box[1] = TC_BK; }
    dims[2] = nb;
    box[2] = 1;
    strides[0] = static_cast<uint64_t>(lda) * 2;
    strides[1] = (nb > 1) ? static_cast<uint64_t>(bsa) * 2 : strides[0] * dims[1];
    int s = encode_tensor_map(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, A, dims, strides, box,
                              CU_TENSOR_MAP_SWIZZLE_128B);
    if (s != YTC_OK) return s;
  }
  {
    const uint64_t nb = (b_bcast || batch == 1) ? 1 : static_cast<uint64_t>(batch);
    uint64_t dims[3], strides[2];
    uint32_t box[3];
    if (!b_mn) { dims[0] = k; dims[1] = n; box[0] = TC_BK; box[1] = pair ? 128u : (g_tc_split_loads ? 64u : static_cast<uint32_t>(BN)); }
    else       { dims[0] = n; dims[1] = k; box[0] = 64;    box[1] = TC_BK; }
    dims[2] = nb;
    box[2] = 1;
    strides[0] = static_cast<uint64_t>(ldb) * 2;
    strides[1] = (nb > 1) ? static_cast<uint64_t>(bsb) * 2 : strides[0] * dims[1];
    int s = encode_tensor_map(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, B, dims, strides, box,
                              CU_TENSOR_MAP_SWIZZLE_128B);
    if (s != YTC_OK) return s;
  }
  GemmTcParams p;
  p.M = m; p.N = n; p.K = k;
  p.batch = static_cast<int>(batch);
  p.a_mn = a_mn; p.b_mn = b_mn;
  p.a_bcast = a_bcast || batch == 1; p.b_bcast = b_bcast || batch == 1;
  p.idesc = umma_idesc(dtype_in == YTC_BF16 ? 1u : 0u, a_mn, b_mn, TC_BM, BN);
  p.alpha = alpha; p.beta = beta;
  p.C = C; p.rsc = rsc; p.csc = csc; p.bsc = bsc;
  p.out_dtype = dtype_out;
  p.tiles_m = (m + TC_BM - 1) / TC_BM;
  p.tiles_n = (n + BN - 1) / BN;
  const int64_t total = static_cast<int64_t>(p.tiles_m) * p.tiles_n * batch;
  if (total > 0x7FFFFFFFll) {
    set_last_error("ytcuda_gemm: too many tiles (%lld)", (long long)total);
    return YTC_UNSUPPORTED;
  }
  p.total_tiles = static_cast<int>(total);
  p.k_blocks = (k + TC_BK - 1) / TC_BK;
  p.a_prefetch = g_tc_a_prefetch;
  p.split_loads = g_tc_split_loads;
  p.status = device_status_word();
  if (!p.status) {
    set_last_error("ytcuda_gemm: no device status word");
    return YTC_CUDA_ERROR;
  }
  if (pair) {
    p.idesc = umma_idesc(dtype_in == YTC_BF16 ? 1u : 0u, a_mn, b_mn, 256, TC2_BN);
    p.tiles_m = (m + 255) / 256;
    p.tiles_n = (n + TC2_BN - 1) / TC2_BN;
    p.total_tiles = static_cast<int>(static_cast<int64_t>(p.tiles_m) * p.tiles_n * batch);
    int clusters = sm_count() / 2;
    if (clusters > p.total_tiles) clusters = p.total_tiles;
    {
      const int s = ensure_dynamic_smem(reinterpret_cast<const void*>(gemm_tc2_kernel), Tc2Smem::DYN_BYTES);
      if (s != YTC_OK) return s;
    }
    YTC_CUDA(launch_overlapped(gemm_tc2_kernel, dim3(clusters * 2), dim3(TC_THREADS), Tc2Smem::DYN_BYTES, st, tmA, tmB, p));
    count_launch();
    YTC_CUDA(cudaGetLastError());
    return YTC_OK;
  }
  const int grid = p.total_tiles < sm_count() ? p.total_tiles : sm_count();
  uint8_t* live = nullptr;
  {
    const int s = make_tile_live(m, n, TC_BM, BN, st, &live);
    if (s != YTC_OK) return s;
    p.tile_live = live;
  }
  if (BN == 256) {
    const int s = ensure_dynamic_smem(reinterpret_cast<const void*>(gemm_tc_kernel<256>), TcSmem<256>::DYN_BYTES);
    if (s != YTC_OK) return s;
    YTC_CUDA(launch_overlapped(gemm_tc_kernel<256>, dim3(grid), dim3(TC_THREADS), TcSmem<256>::DYN_BYTES, st, tmA, tmB, p));
  } else {
    const int s = ensure_dynamic_smem(reinterpret_cast<const void*>(gemm_tc_kernel<128>), TcSmem<128>::DYN_BYTES);
    if (s != YTC_OK) return s;
    YTC_CUDA(launch_overlapped(gemm_tc_kernel<128>, dim3(grid), dim3(TC_THREADS), TcSmem<128>::DYN_BYTES, st, tmA, tmB, p));
  }
  count_launch();
  if (live) cudaFreeAsync(live, st);
  YTC_CUDA(cudaGetLastError());
  return YTC_OK;
}

static int launch_simt(int dtype_in, int dtype_out, const void* A, const void* B, void* C, int m, int n, int k,
                       float alpha, float beta, int64_t rsa, int64_t csa, int64_t rsb, int64_t csb, int64_t rsc,
                       int64_t csc, int64_t batch, int64_t bsa, int64_t bsb, int64_t bsc, cudaStream_t st) {
  GemmSimtParams p;
  p.A = A; p.B = B; p.C = C;
  p.M = m; p.N = n; p.K = k;
  p.rsa = rsa; p.csa = csa; p.rsb = rsb; p.csb = csb; p.rsc = rsc; p.csc = csc;
  p.bsa = bsa; p.bsb = bsb; p.bsc = bsc;
  p.alpha = alpha; p.beta = beta;
  p.in_dtype = dtype_in; p.out_dtype = dtype_out;
  p.tiles_m = (m + SM_BM - 1) / SM_BM;
  p.tiles_n = (n + SM_BN - 1) / SM_BN;
  uint8_t* live = nullptr;
  {
    const int s = make_tile_live(m, n, SM_BM, SM_BN, st, &live);
    if (s != YTC_OK) return s;
    p.tile_live = live;
  }
  const int64_t tiles = static_cast<int64_t>(p.tiles_m) * p.tiles_n;
  if (tiles > 0x7FFFFFFFll || batch > 65535) {
    // gridDim.y is limited to 65535: split the batch.
    if (tiles > 0x7FFFFFFFll) {
      set_last_error("ytcuda_gemm: too many tiles");
      return YTC_UNSUPPORTED;
    }
  }
  for (int64_t b0 = 0; b0 < batch; b0 += 65535) {
    const int64_t nb = (batch - b0 < 65535) ? batch - b0 : 65535;
    GemmSimtParams q = p;
    q.A = static_cast<const char*>(A) + b0 * bsa * dtype_size(dtype_in);
    q.B = static_cast<const char*>(B) + b0 * bsb * dtype_size(dtype_in);
    q.C = static_cast<char*>(C) + b0 * bsc * dtype_size(dtype_out);
    dim3 grid(static_cast<unsigned>(tiles), static_cast<unsigned>(nb));
    if (dtype_in == YTC_F32) gemm_simt_kernel<YTC_F32><<<grid, SM_THREADS, 0, st>>>(q);
    else if (dtype_in == YTC_BF16) gemm_simt_kernel<YTC_BF16><<<grid, SM_THREADS, 0, st>>>(q);
    else gemm_simt_kernel<YTC_F16><<<grid, SM_THREADS, 0, st>>>(q);
    count_launch();
  }
  if (live) cudaFreeAsync(live, st);
  YTC_CUDA(cudaGetLastError());
  return YTC_OK;
}

// x (fp32) = h + m + l with h = bf16(x), m = bf16(x - h), l = bf16(x - h - m): three 16-bit values that together
// carry the 24 mantissa bits of x (the differences are exact in fp32). The six partial products of an fp32 GEMM
// that matter, (l,h) (m,m) (h,l) (m,h) (h,m) (h,h) smallest first, are laid side by side along k so that ONE
// bf16 GEMM with k' = 6 k forms their sum in its fp32 accumulator:
//   left operand  (is_b == 0, x is [rows = m][cols = k]): out[b][i][c k + j] = plane_a(c) of x[b][i][j]
//   right operand (is_b == 1, x is [rows = k][cols = n]): out[b][c k + i][j] = plane_b(c) of x[b][i][j]
// with plane_a = l m h m h h and plane_b = h m l h m h. Non-finite values keep m = l = 0 (an infinite operand then
// meets zero planes of the other operand and the sum becomes NaN where the FFMA kernel gives the infinity).
// One operand of the split; `blocks` CTAs of the launch work on it.
struct SplitOp {
  const float* x;
  int64_t rs, cs, bs;
  int rows, cols;
  int64_t batch;
  int is_b;
  __nv_bfloat16* out;
  int blocks;
};
// One launch splits both operands (or one: b.blocks == 0): CTAs [0, a.blocks) take a, the rest b.
__global__ void __launch_bounds__(256) gemm_split3_kernel(const SplitOp oa, const SplitOp ob) {
  dependent_wait();     // (under a programmatic dependent launch: the kernel before this one has finished)
  dependent_trigger();  // the kernel queued behind this one may be scheduled and set itself up meanwhile
  const bool second = static_cast<int>(blockIdx.x) >= oa.blocks;
  const SplitOp& op = second ? ob : oa;
  const float* x = op.x;
  const int64_t rs = op.rs, cs = op.cs, bs = op.bs, batch = op.batch;
  const int rows = op.rows, cols = op.cols, is_b = op.is_b;
  __nv_bfloat16* out = op.out;
  const int64_t block = static_cast<int64_t>(blockIdx.x) - (second ? oa.blocks : 0);
  const int64_t per = static_cast<int64_t>(rows) * cols;
  const int64_t total = per * batch;
  for (int64_t t = block * static_cast<int64_t>(blockDim.x) + threadIdx.x; t < total;
       t += static_cast<int64_t>(op.blocks) * blockDim.x) {
    const int64_t b = t / per, r = t - b * per;
    const int i = static_cast<int>(r / cols), j = static_cast<int>(r - static_cast<int64_t>(i) * cols);
    const float v = x[b * bs + i * rs + j * cs];
    __nv_bfloat16 p[3];  // h, m, l
    p[0] = __float2bfloat16_rn(v);
    p[1] = p[2] = __float2bfloat16_rn(0.f);
    float fh = __bfloat162float(p[0]);
    if (!isfinite(fh) && isfinite(v)) {
      // a finite value so close to the largest float that rounding its top plane overflows: truncate instead, the
      // two lower planes still hold the remaining 16 mantissa bits exactly
      fh = __uint_as_float(__float_as_uint(v) & 0xffff0000u);
      p[0] = __float2bfloat16_rn(fh);
    }
    if (isfinite(fh)) {
      const float r1 = v - fh;
      p[1] = __float2bfloat16_rn(r1);
      p[2] = __float2bfloat16_rn(r1 - __bfloat162float(p[1]));
    }
    __nv_bfloat16* o = out + b * per * 6;
    if (is_b) {
      // chunks h m l h m h
      const int64_t at = static_cast<int64_t>(i) * cols + j;
      o[at] = p[0];
      o[per + at] = p[1];
      o[2 * per + at] = p[2];
      o[3 * per + at] = p[0];
      o[4 * per + at] = p[1];
      o[5 * per + at] = p[0];
    } else {
      // chunks l m h m h h
      __nv_bfloat16* row = o + static_cast<int64_t>(i) * cols * 6 + j;
      row[0] = p[2];
      row[cols] = p[1];
      row[2 * cols] = p[0];
      row[3 * cols] = p[1];
      row[4 * cols] = p[0];
      row[5 * cols] = p[0];
    }
  }
}

// C[b][i][j] = masked_value wherever mask[i][j] == 0 (the mask is shared by every batch item); the second half of
// YTensor::masked_matmul (reference src/ytensor_math.inl:1053-1090 fills the output with maskedValue and lets
// sgemm_masked write the masked-in products only).
__global__ void __launch_bounds__(256) gemm_apply_mask_kernel(void* C, int dt, int m, int n, int64_t rsc, int64_t csc,
                                                              int64_t batch, int64_t bsc, const uint8_t* mask,
                                                              int64_t mask_rs, float masked_value, int causal,
                                                              int offset) {
  const int64_t per = static_cast<int64_t>(m) * n;
  const int64_t total = per * batch;
  for (int64_t t = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; t < total;
       t += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t b = t / per, r = t - b * per;
    const int i = static_cast<int>(r / n), j = static_cast<int>(r - static_cast<int64_t>(i) * n);
    const bool keep = causal ? (j <= i + offset) : (mask[static_cast<int64_t>(i) * mask_rs + j] != 0);
    if (!keep) store_from_f32(C, b * bsc + i * rsc + j * csc, masked_value, dt);
  }
}

// Which kernel ytcuda_gemm picks: 0 = automatic, 1 = force FFMA, 2 = require tcgen05.
static std::atomic<int> g_gemm_path{0};

// fp32 GEMM on the tensor cores (see gemm_split3_kernel): 0 = automatic (large problems), 1 = never,
// 2 = whenever the shapes allow.
static std::atomic<int> g_f32_split{0};

static bool f32_split_ok(int m, int n, int k, int64_t rsc, int64_t csc, int64_t bsc) {
  if (g_f32_split == 1) return false;
  if (k % 8 || n % 8 || rsc < 0 || csc < 0 || bsc < 0) return false;
  if (g_f32_split == 2) return m >= 1 && n >= 8 && k >= 8;
  return m >= 256 && n >= 256 && k >= 256;
}

static int launch_f32_split(const float* A, const float* B, float* C, int m, int n, int k, float alpha, float beta,
                            int64_t rsa, int64_t csa, int64_t rsb, int64_t csb, int64_t rsc, int64_t csc, int64_t batch,
                            int64_t bsa, int64_t bsb, int64_t bsc, cudaStream_t st) {
  // the split launches and the product are one chain of dependent kernels: each is scheduled while the one before it
  // still runs (programmatic dependent launches)
  struct Scope {
    bool was = overlap_scope();
    Scope() { overlap_scope() = true; }
    ~Scope() { overlap_scope() = was; }
  } scope;
  const bool b_shared = batch > 1 && bsb == 0;
  const int64_t a_per = static_cast<int64_t>(m) * k * 6, b_per = static_cast<int64_t>(k) * n * 6;  // bf16 elements
  // batch items per pass so that the expanded operands stay below about 2 GiB
  int64_t chunk = batch;
  const int64_t per_item = 2 * (a_per + (b_shared ? 0 : b_per));
  const int64_t budget = (int64_t{2} << 30) - (b_shared ? 2 * b_per : 0);
  if (per_item * chunk > budget) chunk = budget / per_item > 0 ? budget / per_item : 1;
  const size_t a_bytes = (static_cast<size_t>(2) * a_per * chunk + 255) / 256 * 256;
  const size_t b_bytes = static_cast<size_t>(2) * b_per * (b_shared ? 1 : chunk);
  char* ws = static_cast<char*>(device_workspace(a_bytes + b_bytes, st));
  if (!ws) {
    set_last_error("ytcuda_gemm: could not allocate %zu bytes for the bf16 form of an fp32 product", a_bytes + b_bytes);
    return YTC_CUDA_ERROR;
  }
  __nv_bfloat16* a6 = reinterpret_cast<__nv_bfloat16*>(ws);
  __nv_bfloat16* b6 = reinterpret_cast<__nv_bfloat16*>(ws + a_bytes);
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  auto op_of = [&](const float* x, int64_t rs, int64_t cs, int64_t bs, int rows, int cols, int64_t nb, int is_b,
                   __nv_bfloat16* out) {
    const int64_t blocks = (static_cast<int64_t>(rows) * cols * nb + 255) / 256;
    return SplitOp{x, rs, cs, bs, rows, cols, nb, is_b, out, static_cast<int>(blocks < cap ? blocks : cap)};
  };
  auto split = [&](const SplitOp& a, const SplitOp& b) {  // b.blocks == 0: one operand only
    (void)launch_overlapped(gemm_split3_kernel, dim3(static_cast<unsigned>(a.blocks + b.blocks)), dim3(256), 0, st, a, b);
    count_launch();
  };
  const SplitOp none{nullptr, 0, 0, 0, 0, 0, 0, 0, nullptr, 0};
  if (b_shared) split(op_of(B, rsb, csb, 0, k, n, 1, 1, b6), none);
  for (int64_t b0 = 0; b0 < batch; b0 += chunk) {
    const int64_t nb = batch - b0 < chunk ? batch - b0 : chunk;
    split(op_of(A + b0 * bsa, rsa, csa, bsa, m, k, nb, 0, a6),
          b_shared ? none : op_of(B + b0 * bsb, rsb, csb, bsb, k, n, nb, 1, b6));
    YTC_CUDA(cudaGetLastError());
    const int s = launch_tc(YTC_BF16, YTC_F32, a6, b6, C + b0 * bsc, m, n, 6 * k, alpha, beta, /*a_mn=*/0, 6 * k,
                            /*b_mn=*/1, n, rsc, csc, nb, a_per, b_shared ? 0 : b_per, bsc, st);
    if (s != YTC_OK) return s;
  }
  device_workspace_release(st);  // large expanded operands do not stay resident
  return YTC_OK;
}

}  // namespace ytk

using namespace ytk;

extern "C" {

int ytcuda_gemm_set_pair_mode(int mode) {
  YTC_REQUIRE(mode >= 0 && mode <= 2, "ytcuda_gemm_set_pair_mode: mode must be 0 (auto), 1 (always) or 2 (never)");
  g_tc_pair = mode;
  return YTC_OK;
}

int ytcuda_gemm_set_tuning(int a_prefetch_kblocks, int split_loads) {
  YTC_REQUIRE(a_prefetch_kblocks >= 0 && a_prefetch_kblocks <= 64, "ytcuda_gemm_set_tuning: prefetch distance outside [0, 64]");
  g_tc_a_prefetch = a_prefetch_kblocks;
  g_tc_split_loads = split_loads ? 1 : 0;
  return YTC_OK;
}

int ytcuda_gemm_set_f32_mode(int mode) {
  YTC_REQUIRE(mode >= 0 && mode <= 2, "ytcuda_gemm_set_f32_mode: mode must be 0, 1 or 2");
  g_f32_split = mode;
  return YTC_OK;
}

int ytcuda_gemm_set_path(int path) {
  YTC_REQUIRE(path >= 0 && path <= 2, "ytcuda_gemm_set_path: path must be 0, 1 or 2");
  g_gemm_path = path;
  return YTC_OK;
}

int ytcuda_gemm(int dtype_in, int dtype_out, const void* A, const void* B, void* C, int m, int n, int k, float alpha,
                float beta, int64_t rsa, int64_t csa, int64_t rsb, int64_t csb, int64_t rsc, int64_t csc,
                int64_t batch, int64_t bsa, int64_t bsb, int64_t bsc, void* stream) {
  YTC_REQUIRE(dtype_in >= YTC_F32 && dtype_in <= YTC_F16, "ytcuda_gemm: bad dtype_in %d", dtype_in);
  YTC_REQUIRE(dtype_out >= YTC_F32 && dtype_out <= YTC_F16, "ytcuda_gemm: bad dtype_out %d", dtype_out);
  YTC_REQUIRE(m >= 0 && n >= 0 && k >= 0 && batch >= 0, "ytcuda_gemm: negative extent (m=%d n=%d k=%d batch=%lld)", m,
              n, k, (long long)batch);
  if (m == 0 || n == 0 || batch == 0) return YTC_OK;
  YTC_REQUIRE(C != nullptr, "ytcuda_gemm: C is null");
  YTC_REQUIRE(k == 0 || (A != nullptr && B != nullptr), "ytcuda_gemm: A or B is null");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (k == 0) {
    if (beta == 1.f) return YTC_OK;
    for (int64_t b0 = 0; b0 < batch; b0 += 65535) {
      const int64_t nb = (batch - b0 < 65535) ? batch - b0 : 65535;
      dim3 grid(static_cast<unsigned>(sm_count() * 4), static_cast<unsigned>(nb));
      gemm_scale_c_kernel<<<grid, 256, 0, st>>>(static_cast<char*>(C) + b0 * bsc * dtype_size(dtype_out), m, n, rsc,
                                                csc, bsc, beta, dtype_out);
      count_launch();
    }
    YTC_CUDA(cudaGetLastError());
    return YTC_OK;
  }
  if (dtype_in == YTC_F32 && dtype_out == YTC_F32 && g_gemm_path != 1 && f32_split_ok(m, n, k, rsc, csc, bsc))
    return launch_f32_split(static_cast<const float*>(A), static_cast<const float*>(B), static_cast<float*>(C), m, n, k,
                            alpha, beta, rsa, csa, rsb, csb, rsc, csc, batch, bsa, bsb, bsc, st);
  int a_mn = 0, b_mn = 0;
  bool tc = (dtype_in != YTC_F32) && g_gemm_path != 1;
  if (tc) {
    // A[m,k]: unit stride along k (csa == 1) or along m (rsa == 1).
    tc = tc_operand_ok(A, rsa, csa, bsa, batch, m, k, &a_mn);
    // B[k,n]: unit stride along n (csb == 1) means N-major; along k (rsb == 1) means K-major.
    int b_k_unit = 0;
    if (tc) {
      tc = tc_operand_ok(B, csb, rsb, bsb, batch, n, k, &b_k_unit);  // view B as [n,k]
      b_mn = b_k_unit;  // viewed as [n,k]: "cs == 1" is rsb == 1 (K-major, 0); "rs == 1" is csb == 1 (N-major, 1)
    }
    if (tc && (rsc < 0 || csc < 0 || bsc < 0)) tc = false;
  }
  if (!tc && g_gemm_path == 2) {
    set_last_error("ytcuda_gemm: tcgen05 path required but the operands do not qualify");
    return YTC_UNSUPPORTED;
  }
  if (tc) {
    const int64_t lda = a_mn ? csa : rsa;
    const int64_t ldb = b_mn ? rsb : csb;
    // A single k extent of 1 makes both strides of an axis "unit"; the leading stride must still be sane.
    return launch_tc(dtype_in, dtype_out, A, B, C, m, n, k, alpha, beta, a_mn, lda, b_mn, ldb, rsc, csc, batch, bsa,
                     bsb, bsc, st);
  }
  return launch_simt(dtype_in, dtype_out, A, B, C, m, n, k, alpha, beta, rsa, csa, rsb, csb, rsc, csc, batch, bsa,
                     bsb, bsc, st);
}

}  // extern "C"

// ------------------------------------------------------------------ host-buffer variant
namespace ytk {

struct HostGemmCtx {
  cudaStream_t s_in = nullptr, s_run = nullptr, s_out = nullptr;
  static constexpr int NBUF = 3;
  cudaEvent_t in_done[NBUF] = {}, run_done[NBUF] = {}, out_done[NBUF] = {}, b_done = nullptr;
  void* a_buf[NBUF] = {};
  void* c_buf[NBUF] = {};
  void* b_buf = nullptr;
  size_t b_cap = 0;
  bool ready = false;
};

static HostGemmCtx* host_ctx() {
  static HostGemmCtx ctx[16];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return nullptr;
  HostGemmCtx& c = ctx[dev];
  if (!c.ready) {
    if (cudaStreamCreateWithFlags(&c.s_in, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
    if (cudaStreamCreateWithFlags(&c.s_run, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
    if (cudaStreamCreateWithFlags(&c.s_out, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
    for (int i = 0; i < HostGemmCtx::NBUF; ++i) {
      if (cudaEventCreateWithFlags(&c.in_done[i], cudaEventDisableTiming) != cudaSuccess) return nullptr;
      if (cudaEventCreateWithFlags(&c.run_done[i], cudaEventDisableTiming) != cudaSuccess) return nullptr;
      if (cudaEventCreateWithFlags(&c.out_done[i], cudaEventDisableTiming) != cudaSuccess) return nullptr;
    }
    if (cudaEventCreateWithFlags(&c.b_done, cudaEventDisableTiming) != cudaSuccess) return nullptr;
    c.ready = true;
  }
  return &c;
}

static int grow(void** buf, size_t* cap, size_t need) {
  if (*cap >= need) return YTC_OK;
  if (*buf) YTC_CUDA(cudaFree(*buf));
  *buf = nullptr;
  *cap = 0;
  YTC_CUDA(cudaMalloc(buf, need));
  *cap = need;
  return YTC_OK;
}

// Elements spanned by an r x c view with non-negative strides.
static int64_t span_of(int64_t r, int64_t c, int64_t rs, int64_t cs) { return (r - 1) * rs + (c - 1) * cs + 1; }

}  // namespace ytk

// The product skips the output tiles the mask leaves nothing in (the launchers read g_mask), then one pass writes
// masked_value wherever the mask does not hold (dead tiles included).
static int gemm_masked_impl(int kind, int dtype_in, int dtype_out, const void* A, const void* B, void* C, int m, int n,
                            int k, int64_t rsa, int64_t csa, int64_t rsb, int64_t csb, int64_t rsc, int64_t csc,
                            int64_t batch, int64_t bsa, int64_t bsb, int64_t bsc, const void* mask,
                            int64_t mask_row_stride, int offset, float masked_value, void* stream) {
  ytk::g_mask.kind = kind;
  ytk::g_mask.mask = static_cast<const uint8_t*>(mask);
  ytk::g_mask.row_stride = mask_row_stride;
  ytk::g_mask.offset = offset;
  const int s = ytcuda_gemm(dtype_in, dtype_out, A, B, C, m, n, k, 1.0f, 0.0f, rsa, csa, rsb, csb, rsc, csc, batch, bsa,
                            bsb, bsc, stream);
  ytk::g_mask = ytk::MaskCtx{};
  if (s != YTC_OK) return s;
  const int64_t total = static_cast<int64_t>(m) * n * batch;
  const int64_t blocks = (total + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  gemm_apply_mask_kernel<<<static_cast<unsigned>(blocks < cap ? blocks : cap), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      C, dtype_out, m, n, rsc, csc, batch, bsc, static_cast<const uint8_t*>(mask), mask_row_stride, masked_value,
      kind == 2 ? 1 : 0, offset);
  count_launch();
  YTC_CUDA(cudaGetLastError());
  return YTC_OK;
}

int ytcuda_gemm_masked_causal(int dtype_in, int dtype_out, const void* A, const void* B, void* C, int m, int n, int k,
                              int64_t rsa, int64_t csa, int64_t rsb, int64_t csb, int64_t rsc, int64_t csc,
                              int64_t batch, int64_t bsa, int64_t bsb, int64_t bsc, int causal_offset,
                              float masked_value, void* stream) {
  YTC_REQUIRE(m >= 0 && n >= 0 && k >= 0 && batch >= 0, "ytcuda_gemm_masked_causal: negative extent");
  if (m == 0 || n == 0 || batch == 0) return YTC_OK;
  return gemm_masked_impl(2, dtype_in, dtype_out, A, B, C, m, n, k, rsa, csa, rsb, csb, rsc, csc, batch, bsa, bsb, bsc,
                          nullptr, 0, causal_offset, masked_value, stream);
}

int ytcuda_gemm_masked(int dtype_in, int dtype_out, const void* A, const void* B, void* C, int m, int n, int k,
                       int64_t rsa, int64_t csa, int64_t rsb, int64_t csb, int64_t rsc, int64_t csc, int64_t batch,
                       int64_t bsa, int64_t bsb, int64_t bsc, const void* mask, int64_t mask_row_stride,
                       float masked_value, void* stream) {
  YTC_REQUIRE(m >= 0 && n >= 0 && k >= 0 && batch >= 0, "ytcuda_gemm_masked: negative extent");
  if (m == 0 || n == 0 || batch == 0) return YTC_OK;
  YTC_REQUIRE(mask != nullptr, "ytcuda_gemm_masked: mask is null");
  YTC_REQUIRE(mask_row_stride >= n, "ytcuda_gemm_masked: mask row stride %lld shorter than n = %d",
              (long long)mask_row_stride, n);
  return gemm_masked_impl(1, dtype_in, dtype_out, A, B, C, m, n, k, rsa, csa, rsb, csb, rsc, csc, batch, bsa, bsb, bsc,
                          mask, mask_row_stride, 0, masked_value, stream);
}


extern "C" int ytcuda_gemm_host(int dtype_in, int dtype_out, const void* A, const void* B, void* C, int m, int n, int k,
                                float alpha, float beta, int64_t rsa, int64_t csa, int64_t rsb, int64_t csb,
                                int64_t rsc, int64_t csc, int64_t batch, int64_t bsa, int64_t bsb, int64_t bsc) {
  YTC_REQUIRE(dtype_in >= YTC_F32 && dtype_in <= YTC_F16, "ytcuda_gemm_host: bad dtype_in %d", dtype_in);
  YTC_REQUIRE(dtype_out >= YTC_F32 && dtype_out <= YTC_F16, "ytcuda_gemm_host: bad dtype_out %d", dtype_out);
  YTC_REQUIRE(m >= 0 && n >= 0 && k >= 0 && batch >= 0, "ytcuda_gemm_host: negative extent");
  if (m == 0 || n == 0 || batch == 0) return YTC_OK;
  YTC_REQUIRE(A && B && C, "ytcuda_gemm_host: null operand");
  YTC_REQUIRE(k > 0, "ytcuda_gemm_host: k must be positive");
  YTC_REQUIRE(rsa >= 0 && csa >= 0 && rsb >= 0 && csb >= 0 && bsa >= 0 && bsb >= 0,
              "ytcuda_gemm_host: negative input strides are not supported");
  const bool c_rows = (csc == 1 && rsc >= n), c_cols = (rsc == 1 && csc >= m);
  if (!(c_rows || c_cols) || bsc < 0) {
    set_last_error("ytcuda_gemm_host: C must have a unit stride along one axis and no overlap");
    return YTC_UNSUPPORTED;
  }
  HostGemmCtx* cx = host_ctx();
  if (!cx) {
    set_last_error("ytcuda_gemm_host: cannot create streams");
    return YTC_CUDA_ERROR;
  }
  const int64_t ein = dtype_size(dtype_in), eout = dtype_size(dtype_out);
  const int64_t a_span = span_of(m, k, rsa, csa), b_span = span_of(k, n, rsb, csb), c_span = span_of(m, n, rsc, csc);
  const bool b_shared = (batch == 1 || bsb == 0);
  const bool a_shared = (batch > 1 && bsa == 0);
  // Batch items per chunk: about 64 MiB of A + C traffic per chunk, at least one item.
  const int64_t per_item = a_span * ein + c_span * eout;
  int64_t g = (64ll << 20) / (per_item > 0 ? per_item : 1);
  if (g < 1) g = 1;
  if (g > batch) g = batch;
  const int64_t a_chunk = a_shared ? a_span : ((g - 1) * bsa + a_span);
  const int64_t c_chunk = (g - 1) * bsc + c_span;
  const int64_t b_all = b_shared ? b_span : ((batch - 1) * bsb + b_span);
  static size_t a_caps[16][HostGemmCtx::NBUF], c_caps[16][HostGemmCtx::NBUF];
  int dev = 0;
  YTC_CUDA(cudaGetDevice(&dev));
  for (int i = 0; i < HostGemmCtx::NBUF; ++i) {
    int s = grow(&cx->a_buf[i], &a_caps[dev][i], static_cast<size_t>(a_chunk * ein));
    if (s != YTC_OK) return s;
    s = grow(&cx->c_buf[i], &c_caps[dev][i], static_cast<size_t>(c_chunk * eout));
    if (s != YTC_OK) return s;
  }
  {
    int s = grow(&cx->b_buf, &cx->b_cap, static_cast<size_t>(b_all * ein));
    if (s != YTC_OK) return s;
  }
  YTC_CUDA(cudaMemcpyAsync(cx->b_buf, B, static_cast<size_t>(b_all * ein), cudaMemcpyHostToDevice, cx->s_in));
  YTC_CUDA(cudaEventRecord(cx->b_done, cx->s_in));
  YTC_CUDA(cudaStreamWaitEvent(cx->s_run, cx->b_done, 0));
  if (a_shared) {
    YTC_CUDA(cudaMemcpyAsync(cx->a_buf[0], A, static_cast<size_t>(a_span * ein), cudaMemcpyHostToDevice, cx->s_in));
    YTC_CUDA(cudaEventRecord(cx->b_done, cx->s_in));
    YTC_CUDA(cudaStreamWaitEvent(cx->s_run, cx->b_done, 0));
  }
  const bool c_dense = (c_span == static_cast<int64_t>(m) * n) && (batch == 1 || bsc == c_span);
  int64_t chunk_idx = 0;
  for (int64_t b0 = 0; b0 < batch; b0 += g, ++chunk_idx) {
    const int64_t nb = (batch - b0 < g) ? batch - b0 : g;
    const int buf = static_cast<int>(chunk_idx % HostGemmCtx::NBUF);
    const char* a_src = static_cast<const char*>(A) + b0 * bsa * ein;
    char* c_host = static_cast<char*>(C) + b0 * bsc * eout;
    void* a_dev = a_shared ? cx->a_buf[0] : cx->a_buf[buf];
    if (chunk_idx >= HostGemmCtx::NBUF) YTC_CUDA(cudaStreamWaitEvent(cx->s_in, cx->out_done[buf], 0));
    if (!a_shared)
      YTC_CUDA(cudaMemcpyAsync(a_dev, a_src, static_cast<size_t>(((nb - 1) * bsa + a_span) * ein),
                               cudaMemcpyHostToDevice, cx->s_in));
    if (beta != 0.f)
      YTC_CUDA(cudaMemcpyAsync(cx->c_buf[buf], c_host, static_cast<size_t>(((nb - 1) * bsc + c_span) * eout),
                               cudaMemcpyHostToDevice, cx->s_in));
    YTC_CUDA(cudaEventRecord(cx->in_done[buf], cx->s_in));
    YTC_CUDA(cudaStreamWaitEvent(cx->s_run, cx->in_done[buf], 0));
    const char* b_dev = static_cast<const char*>(cx->b_buf) + (b_shared ? 0 : b0 * bsb * ein);
    int s = ytcuda_gemm(dtype_in, dtype_out, a_dev, b_dev, cx->c_buf[buf], m, n, k, alpha, beta, rsa, csa, rsb, csb,
                        rsc, csc, nb, a_shared ? 0 : bsa, b_shared ? 0 : bsb, bsc, cx->s_run);
    if (s != YTC_OK) {
      cudaDeviceSynchronize();
      return s;
    }
    YTC_CUDA(cudaEventRecord(cx->run_done[buf], cx->s_run));
    YTC_CUDA(cudaStreamWaitEvent(cx->s_out, cx->run_done[buf], 0));
    if (c_dense) {
      YTC_CUDA(cudaMemcpyAsync(c_host, cx->c_buf[buf], static_cast<size_t>(nb * c_span * eout),
                               cudaMemcpyDeviceToHost, cx->s_out));
    } else {
      for (int64_t i = 0; i < nb; ++i) {
        const size_t off = static_cast<size_t>(i * bsc * eout);
        const size_t pitch = static_cast<size_t>((c_rows ? rsc : csc) * eout);
        const size_t width = static_cast<size_t>((c_rows ? n : m) * eout);
        const size_t height = static_cast<size_t>(c_rows ? m : n);
        YTC_CUDA(cudaMemcpy2DAsync(c_host + off, pitch, static_cast<char*>(cx->c_buf[buf]) + off, pitch, width, height,
                                   cudaMemcpyDeviceToHost, cx->s_out));
      }
    }
    YTC_CUDA(cudaEventRecord(cx->out_done[buf], cx->s_out));
  }
  YTC_CUDA(cudaStreamSynchronize(cx->s_out));
  YTC_CUDA(cudaStreamSynchronize(cx->s_run));
  YTC_CUDA(cudaStreamSynchronize(cx->s_in));
  return read_device_status(cx->s_run) == 0 ? YTC_OK : YTC_TIMEOUT;
}
