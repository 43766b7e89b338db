// CTA-pair variant of the tcgen05 GEMM: dense / batched, ragged grouped, and grouped SwiGLU.
//
// Two CTAs of a cluster share one 256 x 256 output tile: CTA r of the pair owns rows
// [m0 + 128 r, m0 + 128 r + 128), loads its own A tile (128 x 64) and ITS HALF of the B tile
// (64 x 128 of the 64 x 256), and the even CTA issues tcgen05.mma.cta_group::2 (M 256, N 256,
// K 16), which reads A from each CTA's shared memory and the two B halves from both. Per CTA and
// k-block that is 32 KB from L2 instead of 48 KB, and 8 KB of shared-memory operand reads per
// MMA instead of 12 KB — less data moved per FLOP, which is what a power-capped GEMM needs — and
// the freed shared memory deepens the ring from 4 to 6 stages.
//
// Synchronisation (all waits bounded, as in the single-CTA kernel):
//   full[s]    even CTA only. Armed by its producer with the bytes of BOTH CTAs' loads; both
//              producers' TMA loads count on it (cta_group::2 loads, peer bit cleared).
//   empty[s]   one per CTA, released by the even CTA's tcgen05.commit to both (an mbarrier
//              arrival multicast; no data is multicast anywhere).
//   tfull[a]   one per CTA, same commit form after the last k-block of a tile.
//   tempty[a]  even CTA only, 8 arrivals: the four epilogue warps of each CTA.
// Grouped modes: a pair tile is 256 rows of ONE group; a CTA whose 128 rows reach past the end of
// the group computes on whatever rows follow (the next group's, or zeros past the end) and stores
// only its valid rows, as the single-CTA kernel does for partial tiles. In the SwiGLU mode the B
// halves are the two weight matrices: the even CTA loads the 128 gate columns, the odd CTA the
// matching 128 up columns, and every CTA's accumulator holds gate | up for its own rows.
// Both CTAs allocate TMEM with cta_group::2 from the same warp index, and free it only after
// a cluster barrier; a second cluster barrier after barrier initialisation keeps either CTA
// from signalling a barrier the other has not initialised yet.
#pragma once
#include "gemm_sm100.cuh"

namespace tsb {
namespace gemm2 {

using gemm::BK;
using gemm::BM;
using gemm::BN;
using gemm::EPI_BUF_BYTES;
using gemm::Params;
using gemm::kGrouped;
using gemm::kGroupedSwiGLU;
using gemm::kPlain;

#ifndef TESSERA_GEMM2_STAGES
#define TESSERA_GEMM2_STAGES 6
#endif
constexpr int STAGES = TESSERA_GEMM2_STAGES;
constexpr int A_STAGE_BYTES = BM * BK * 2;        // 128 x 64
constexpr int B_BLOCK_BYTES = BK * 64 * 2;        // one [64 k][64 n] block
constexpr int B_STAGE_BYTES = 2 * B_BLOCK_BYTES;  // this CTA's 128 columns
constexpr int PAIR_TX_BYTES = 2 * (A_STAGE_BYTES + B_STAGE_BYTES);
constexpr int SMEM_A_OFF = 0;
constexpr int SMEM_B_OFF = SMEM_A_OFF + STAGES * A_STAGE_BYTES;
constexpr int SMEM_EPI_OFF = SMEM_B_OFF + STAGES * B_STAGE_BYTES;
constexpr int SMEM_BAR_OFF = SMEM_EPI_OFF + 4 * 2 * EPI_BUF_BYTES;
constexpr int SMEM_BYTES = SMEM_BAR_OFF + 256;
constexpr int SMEM_ALLOC = SMEM_BYTES + 1024;
constexpr int NUM_THREADS = 192;
constexpr uint32_t TMEM_COLS = 512;
#ifndef TESSERA_GEMM2_GROUP
#define TESSERA_GEMM2_GROUP 8
#endif
constexpr int GROUP_PAIRS = TESSERA_GEMM2_GROUP;  // 256-row tile pairs per raster group (L2 reuse)

struct PairTile {
  int m0, n0, b;  // m0 = first row of the PAIR
  int rows;       // valid rows of the pair from m0 (grouped modes; 2 * BM when plain)
};

// Static tile list shared by both CTAs of a pair. Plain: pair tiles of 256 x 256, rastered in
// groups of GROUP_PAIRS row blocks so consecutive clusters reuse the same B columns out of L2.
// Grouped: per group, ceil(rows / 256) pair tiles per output column block, m fastest.
template <int kMode>
struct PairWalker {
  int t, step;
  int e = 0, base = 0;  // grouped cursor
  __device__ PairWalker(int first, int stride) : t(first), step(stride) {}
  __device__ bool next(const Params& p, PairTile& out) {
    if constexpr (kMode == kPlain) {
      const int m_pairs = (p.m_tiles + 1) / 2;
      const int per_b = m_pairs * p.n_tiles;
      if (t >= per_b * p.batch) return false;
      const int b = t / per_b;
      const int r = t - b * per_b;
      const int gspan = GROUP_PAIRS * p.n_tiles;
      const int g = r / gspan;
      const int first_m = g * GROUP_PAIRS;
      const int gsz = min(m_pairs - first_m, GROUP_PAIRS);
      const int rr = r - g * gspan;
      out.m0 = (first_m + rr % gsz) * 2 * BM;
      out.n0 = (rr / gsz) * BN;
      out.b = b;
      out.rows = 2 * BM;
    } else {
      constexpr int kOutW = (kMode == kGroupedSwiGLU) ? BN / 2 : BN;
      int rows_e = 0, mp = 0;
      while (e < p.batch) {
        rows_e = p.group_offsets[e + 1] - p.group_offsets[e];
        mp = (rows_e + 2 * BM - 1) / (2 * BM);
        const int cnt = mp * p.n_tiles;
        if (t < base + cnt) break;
        base += cnt;
        ++e;
      }
      if (e >= p.batch) return false;
      const int local = t - base;
      const int n_idx = local / mp;
      const int m_idx = local - n_idx * mp;
      out.m0 = p.group_offsets[e] + m_idx * 2 * BM;
      out.n0 = n_idx * kOutW;
      out.b = e;
      out.rows = min(2 * BM, rows_e - m_idx * 2 * BM);
    }
    t += step;
    return true;
  }
};

template <typename OutT, int kMode, bool kFp8 = false>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
             const __grid_constant__ CUtensorMap tmB2, const __grid_constant__ CUtensorMap tmD,
             const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const uint32_t sA = smem_base + SMEM_A_OFF;
  const uint32_t sB = smem_base + SMEM_B_OFF;
  const uint32_t sEpi = smem_base + SMEM_EPI_OFF;
  const uint32_t bars = smem_base + SMEM_BAR_OFF;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };
  volatile uint32_t* tmem_slot =
      reinterpret_cast<volatile uint32_t*>(smem_gen + SMEM_BAR_OFF + 8 * (2 * STAGES + 4));
  volatile int* abort_flag =
      reinterpret_cast<volatile int*>(smem_gen + SMEM_BAR_OFF + 8 * (2 * STAGES + 4) + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = even CTA (issues the MMAs), 1 = its peer
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;
  constexpr int kBKe = kFp8 ? 2 * BK : BK;  // K elements per stage
  const int num_kb = (p.K + kBKe - 1) / kBKe;
  constexpr int kOutW = (kMode == kGroupedSwiGLU) ? BN / 2 : BN;  // output columns per tile
  constexpr int kChunk = (sizeof(OutT) == 4) ? 32 : 64;            // output columns per store

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 8);
    }
    fence_mbar_init();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if constexpr (kMode == kGroupedSwiGLU) tma_prefetch_desc(&tmB2);
    tma_prefetch_desc(&tmD);
  }
  if (warp == 5) {
    tmem_alloc_2cta(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
    tmem_relinquish_2cta();
  }
  tc_fence_before();
  __syncthreads();
  // Both CTAs' barriers exist before either side signals across the pair.
  cluster_arrive();
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      PairWalker<kMode> walk(cluster_id, num_clusters);
      PairTile tile;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      // SwiGLU: the even CTA fetches gate columns, the odd CTA the same columns of the up matrix.
      const CUtensorMap* my_b = (kMode == kGroupedSwiGLU && rank == 1) ? &tmB2 : &tmB;
      while (ok && walk.next(p, tile)) {
        const int my_m0 = tile.m0 + static_cast<int>(rank) * BM;
        const int my_n0 =
            (kMode == kGroupedSwiGLU) ? tile.n0 : tile.n0 + static_cast<int>(rank) * (BN / 2);
        const int a_b = (kMode == kPlain) ? tile.b : 0;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.err, kErrWaitEmpty, kb)) {
            ok = false;
            break;
          }
          if (rank == 0) mbar_arrive_expect_tx(full_bar(stage), PAIR_TX_BYTES);
          const int k0 = kb * kBKe;
          tma_load_3d_2cta(sA + stage * A_STAGE_BYTES, &tmA, full_bar(stage), k0, my_m0, a_b);
          const uint32_t b_dst = sB + stage * B_STAGE_BYTES;
          if constexpr (kFp8) {
            // this CTA's 128 rows of Bt[N,K]: one box of 128 rows x 128 B
            tma_load_3d_2cta(b_dst, my_b, full_bar(stage), k0, my_n0, tile.b);
          } else {
#pragma unroll
            for (int j = 0; j < 2; ++j)
              tma_load_3d_2cta(b_dst + j * B_BLOCK_BYTES, my_b, full_bar(stage), my_n0 + 64 * j, k0,
                               tile.b);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------ MMA issuer (even CTA only)
    if (lane == 0 && rank == 0) {
      PairWalker<kMode> walk(cluster_id, num_clusters);
      PairTile tile;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      const uint32_t desc_hi = smem_desc_hi(1024);
      const uint32_t a_lo0 = smem_desc_lo(sA, 16);
      const uint32_t b_lo0 = smem_desc_lo(sB, kFp8 ? 16 : B_BLOCK_BYTES);
      while (ok && walk.next(p, tile)) {
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p.err, kErrWaitTmemEmpty)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.err, kErrWaitFull, kb)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + stage * (A_STAGE_BYTES >> 4);
          const uint32_t b_lo = b_lo0 + stage * (B_STAGE_BYTES >> 4);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if constexpr (kFp8)
              umma_f8_ss_parts_2cta(d_tmem, a_lo + k * 2, desc_hi, b_lo + k * 2, desc_hi, p.idesc,
                                    (kb > 0 || k > 0) ? 1u : 0u);
            else
              umma_f16_ss_parts_2cta(d_tmem, a_lo + k * 2, desc_hi, b_lo + k * 128, desc_hi, p.idesc,
                                     (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit_2cta(empty_bar(stage), 3);  // this stage is free again in both CTAs
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit_2cta(tfull_bar(acc), 3);  // both CTAs' epilogues may read their lanes
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps 0..3 (both CTAs)
    PairWalker<kMode> walk(cluster_id, num_clusters);
    PairTile tile;
    int acc = 0;
    uint32_t acc_phase = 0;
    int sbuf = 0;
    bool ok = true;
    const uint32_t lane_base = static_cast<uint32_t>(32 * warp) << 16;
    while (ok && walk.next(p, tile)) {
      if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.err, kErrWaitTmemFull)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int cta_m0 = tile.m0 + static_cast<int>(rank) * BM;  // first row of this CTA's half
      const int row0 = cta_m0 + 32 * warp;                        // first output row of this warp
      // valid rows of this warp: all 32 in plain mode (TMA clips at M), the group's tail otherwise
      const int rows_w = max(0, min(32, tile.rows - static_cast<int>(rank) * BM - 32 * warp));
      const bool warp_has_rows = (kMode == kPlain) ? (row0 < p.M) : (rows_w > 0);
      const uint32_t t_acc = tmem_base + static_cast<uint32_t>(acc * BN) + lane_base;
      constexpr int kChunks = kOutW / kChunk;
      float sc = 1.f, sc2 = 1.f, amax = 0.f;  // dequantisation scales of this tile (fp8 operands)
      if constexpr (kFp8) {
        const float sa = __ldg(p.scale_a);
        sc = sa * __ldg(p.scale_b + tile.b);
        if constexpr (kMode == kGroupedSwiGLU) sc2 = sa * __ldg(p.scale_b2 + tile.b);
      } else if (p.scale_a) {
        // 16-bit operands that stand for quantised values with one scale for A (e.g. e4m3 values
        // held as bf16 against dequantised 4-bit weights): applied to the fp32 accumulators
        sc = sc2 = __ldg(p.scale_a);
      }
      (void)sc2;
      bool released = false;
#pragma unroll 1
      for (int c = 0; c < kChunks; ++c) {
        const int col0 = tile.n0 + c * kChunk;
        if (col0 >= p.N || !warp_has_rows) break;
        const uint32_t buf = sEpi + static_cast<uint32_t>((warp * 2 + sbuf) * EPI_BUF_BYTES);
        if (lane == 0) tma_store_wait_read<1>();
        __syncwarp();
        if constexpr (kMode == kGroupedSwiGLU) {
          // kChunk output columns (64 for 16-bit, 32 for fp32) in halves of 32.
#pragma unroll
          for (int h = 0; h < kChunk / 32; ++h) {
            uint32_t g[32], u[32];
            tmem_ld_32x32b_x32(t_acc + c * kChunk + h * 32, g);
            tmem_ld_32x32b_x32(t_acc + (BN / 2) + c * kChunk + h * 32, u);
            tmem_ld_wait();
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j)
              v[j] = gemm::silu_mul(__uint_as_float(g[j]) * sc, __uint_as_float(u[j]) * sc2);
            if constexpr (kFp8) amax = fmaxf(amax, gemm::stored_amax32<OutT>(v));
            gemm::stage_row32<OutT>(buf, lane, h * 32 * sizeof(OutT), v);
          }
        } else {
#pragma unroll
          for (int h = 0; h < kChunk / 32; ++h) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(t_acc + c * kChunk + h * 32, r);
            tmem_ld_wait();
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * sc;
            if constexpr (kMode == kPlain) {
              if (p.bias || p.residual || p.activation)
                gemm::apply_epilogue<OutT>(v, p, row0 + lane, col0 + h * 32);
            }
            if constexpr (kFp8) amax = fmaxf(amax, gemm::stored_amax32<OutT>(v));
            gemm::stage_row32<OutT>(buf, lane, h * 32 * sizeof(OutT), v);
          }
        }
        if (c == kChunks - 1 || col0 + kChunk >= p.N) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_even_cta(tempty_bar(acc));
          released = true;
        }
        const bool full_rows = (kMode == kPlain) || (rows_w == 32);
        if (full_rows) {
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            const int d_b = (kMode == kPlain) ? tile.b : 0;
            tma_store_3d(&tmD, buf, col0, row0, d_b);
            tma_store_commit();
          }
        } else {
          // Tail of a ragged group: copy the valid rows out with predicated 16-byte stores.
          __syncwarp();
          constexpr int kElemsPer16 = 16 / sizeof(OutT);
          OutT* Dp = reinterpret_cast<OutT*>(p.D);
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int r = it * 4 + (lane >> 3);
            const int ch = lane & 7;
            const int col = col0 + ch * kElemsPer16;
            if (r < rows_w && col < p.N) {
              uint4 val;
              const uint32_t addr = buf + swz128(r, ch);
              asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                           : "=r"(val.x), "=r"(val.y), "=r"(val.z), "=r"(val.w)
                           : "r"(addr));
              *reinterpret_cast<uint4*>(Dp + static_cast<long long>(row0 + r) * p.ldd + col) = val;
            }
          }
          __syncwarp();
        }
        sbuf ^= 1;
      }
      if (!released) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_even_cta(tempty_bar(acc));
      }
      if constexpr (kFp8) {
        const bool lane_valid = (kMode == kPlain) ? (row0 + lane < p.M) : (lane < rows_w);
        float a = lane_valid ? amax : 0.f;
#pragma unroll
        for (int sh = 16; sh; sh >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, sh));
        if (p.amax_out && lane == 0 && a > 0.f) atomicMax(p.amax_out, __float_as_uint(a));
      }
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
    if (lane == 0) tma_store_wait<0>();
  }

  // ------------------------------------------------------------ tear-down
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(10000);
    __syncthreads();
  }
  // Neither CTA may leave (or free TMEM) while the other can still read its shared memory or
  // signal its barriers.
  cluster_arrive();
  cluster_wait();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc_2cta(tmem_base, TMEM_COLS);
  }
}

}  // namespace gemm2
}  // namespace tsb
