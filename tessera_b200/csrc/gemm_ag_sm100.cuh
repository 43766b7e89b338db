// Column-parallel GEMM whose epilogue is the all-gather: every finished output piece is stored into
// ALL ranks' copies of Y (this rank's own and the peers', mapped into this address space) with plain
// TMA stores, so the exchange over NVLink overlaps the main loop.
//
// The main loop is the CTA-pair form (tcgen05.mma.cta_group::2, 256 x 256 x 64 per pair and stage,
// six TMA stages, two accumulators in TMEM): it is the tile shape that needs the fewest bytes from
// L2 per FLOP, and narrower tiles measured slower (a 256 x 128 pair tile needs 1.5x the L2 traffic
// and ran the same product in 155 us instead of 104 us).
//
// What is specific to the fused exchange:
//   * Split K in the FIRST wave. With `ksplit` = 2 the first unit of every cluster is one half of
//     the K loop of a tile: clusters 2t and 2t+1 work on tile t at the same time, the odd one (the
//     helper) writes its fp32 partial sums to a workspace and raises one flag per epilogue warp, the
//     even one (the finisher) adds them to its own accumulator, converts, and issues the stores to
//     every copy. All later units are whole tiles. The first stores therefore leave after half a tile
//     time instead of a whole one, and the NVLink exchange, which bounds the step from four ranks on,
//     starts that much earlier. A finisher only waits for the unit its neighbour runs at the same
//     time and helpers wait for nobody, so there is no cycle; the wait is bounded like every other.
//     Measured on four GPUs (8192^3): 248 us against 273 us unsplit. The host only asks for the
//     split with at most four copies: with eight, a CTA has more bytes to store per tile than the
//     tile takes to compute, what counts is that all CTAs store evenly all the time, and every split
//     form measured slower there (first wave 465 us, every tile with alternating roles 281 us, every
//     tile with each cluster finishing half of the columns 296 us, unsplit 250 us).
//   * The copies are issued in an order that starts at a different rank for every rank, CTA, warp and
//     piece, so the ranks do not all write to the same peer at the same moment.
// Barriers as in the general pair kernel: full[s] in the even CTA counts both CTAs' TMA bytes,
// empty[s] / tfull[a] are released in both CTAs by one tcgen05.commit (an mbarrier arrival, no data
// is multicast), tempty[a] in the even CTA collects the eight epilogue warps. No load ever reads
// peer memory.
#pragma once
#include "gemm_sm100.cuh"

namespace tsb {
namespace gemm_ag {

using gemm::BK;
using gemm::BM;
using gemm::BN;
using gemm::EPI_BUF_BYTES;
using gemm::Params;
using gemm::PeerMaps;

constexpr int STAGES = 6;
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
constexpr int GROUP_PAIRS = 8;  // 256-row blocks per raster group (L2 reuse of A and B)
// fp32 partial sums of one epilogue warp for one tile: 64 groups of 4 columns x 32 lanes x 16 bytes
constexpr int PARTIAL_FLOATS_PER_WARP = BN * 32;
constexpr size_t PARTIAL_BYTES_PER_TILE = size_t(8) * PARTIAL_FLOATS_PER_WARP * 4;  // 2 CTAs x 4 warps
constexpr int FLAGS_PER_TILE = 8;

struct Unit {
  int m0, n0;  // first row of the PAIR, first column
  int tile;    // tile index (workspace slot of a split tile)
  int split;   // 1: this unit is half of the K loop of its tile
  int half;    // which half (split units)
  int helper;  // split units: 1 = hands its partial sums to the neighbour, 0 = finishes the tile
};

// Static unit list shared by both CTAs of a pair. Tiles are rastered in groups of GROUP_PAIRS row
// blocks, rows fastest. With ksplit = 2 (an even number of clusters C) the first unit of cluster c is
// half (c & 1) of tile c / 2, and its later units are the whole tiles C / 2 + c, C / 2 + c + C, ...
struct Walker {
  int cluster, step;
  int iter = 0;
  __device__ Walker(int first, int stride) : cluster(first), step(stride) {}
  __device__ bool next(const Params& p, Unit& out) {
    const int m_pairs = (p.m_tiles + 1) / 2;
    const int tiles = m_pairs * p.n_tiles;
    int t;
    if (p.ksplit == 2) {
      out.split = (iter == 0);
      t = (iter == 0) ? (cluster >> 1) : (step >> 1) + cluster + (iter - 1) * step;
    } else {
      out.split = 0;
      t = cluster + iter * step;
    }
    if (t >= tiles) return false;
    const int gspan = GROUP_PAIRS * p.n_tiles;
    const int g = t / gspan;
    const int first_m = g * GROUP_PAIRS;
    const int gsz = min(m_pairs - first_m, GROUP_PAIRS);
    const int rr = t - g * gspan;
    out.m0 = (first_m + rr % gsz) * 2 * BM;
    out.n0 = (rr / gsz) * BN;
    out.tile = t;
    out.half = out.split ? (cluster & 1) : 0;
    out.helper = out.half;
    ++iter;
    return true;
  }
};

__device__ __forceinline__ void st_release_gpu(int* p, int v) {
  asm volatile("st.release.gpu.global.b32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.b32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_cg_f4(const float* p) {
  float4 v;
  asm volatile("ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

template <typename OutT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_ag_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ PeerMaps peers, const Params p) {
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
  const int num_kb = (p.K + BK - 1) / BK;
  const int kb_mid = num_kb / 2;  // split units: half 0 is [0, kb_mid), half 1 the rest
  constexpr int kChunk = (sizeof(OutT) == 4) ? 32 : 64;      // output columns per stored piece

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
      Walker walk(cluster_id, num_clusters);
      Unit unit;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      while (ok && walk.next(p, unit)) {
        const int my_m0 = unit.m0 + static_cast<int>(rank) * BM;
        const int my_n0 = unit.n0 + static_cast<int>(rank) * (BN / 2);
        const int kb0 = (unit.split && unit.half) ? kb_mid : 0;
        const int kb1 = (unit.split && !unit.half) ? kb_mid : num_kb;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.err, kErrWaitEmpty, kb)) {
            ok = false;
            break;
          }
          if (rank == 0) mbar_arrive_expect_tx(full_bar(stage), PAIR_TX_BYTES);
          const int k0 = kb * BK;
          tma_load_3d_2cta(sA + stage * A_STAGE_BYTES, &tmA, full_bar(stage), k0, my_m0, 0);
          const uint32_t b_dst = sB + stage * B_STAGE_BYTES;
#pragma unroll
          for (int j = 0; j < 2; ++j)
            tma_load_3d_2cta(b_dst + j * B_BLOCK_BYTES, &tmB, full_bar(stage), my_n0 + 64 * j, k0, 0);
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
      Walker walk(cluster_id, num_clusters);
      Unit unit;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      const uint32_t desc_hi = smem_desc_hi(1024);
      const uint32_t a_lo0 = smem_desc_lo(sA, 16);
      const uint32_t b_lo0 = smem_desc_lo(sB, B_BLOCK_BYTES);
      while (ok && walk.next(p, unit)) {
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p.err, kErrWaitTmemEmpty)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        const int kb0 = (unit.split && unit.half) ? kb_mid : 0;
        const int kb1 = (unit.split && !unit.half) ? kb_mid : num_kb;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.err, kErrWaitFull, kb)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + stage * (A_STAGE_BYTES >> 4);
          const uint32_t b_lo = b_lo0 + stage * (B_STAGE_BYTES >> 4);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16_ss_parts_2cta(d_tmem, a_lo + k * 2, desc_hi, b_lo + k * 128, desc_hi, p.idesc,
                                   (kb > kb0 || k > 0) ? 1u : 0u);
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
    Walker walk(cluster_id, num_clusters);
    Unit unit;
    int acc = 0;
    uint32_t acc_phase = 0;
    int sbuf = 0;
    int rot = p.peer_first + warp + static_cast<int>(blockIdx.x);  // first copy of the next piece
    bool ok = true;
    const uint32_t lane_base = static_cast<uint32_t>(32 * warp) << 16;
    while (ok && walk.next(p, unit)) {
      if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.err, kErrWaitTmemFull)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int row0 = unit.m0 + static_cast<int>(rank) * BM + 32 * warp;
      const uint32_t t_acc = tmem_base + static_cast<uint32_t>(acc * BN) + lane_base;
      const int slot = unit.tile * FLAGS_PER_TILE + static_cast<int>(rank) * 4 + warp;
      float* part = p.partial + static_cast<size_t>(slot) * PARTIAL_FLOATS_PER_WARP + lane * 4;
      if (unit.split && unit.helper) {
        // Helper: this warp's 32 x 256 fp32 partial sums go to the workspace (each store instruction
        // writes 512 contiguous bytes), then its flag goes up.
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_acc + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 8; ++q)
            *reinterpret_cast<uint4*>(part + (c * 8 + q) * 128) =
                make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
        }
        tc_fence_before();
        __threadfence();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive_even_cta(tempty_bar(acc));
          st_release_gpu(p.flags + slot, 1);
        }
      } else {
        const bool has_rows = row0 < p.M;
        if (unit.split) {
          // Finisher: the neighbour cluster's partial sums of these rows must have landed.
          int seen = 1;
          if (lane == 0) {
            seen = ld_acquire_gpu(p.flags + slot);
            if (!seen) {
              const long long t0 = clock64();
              while (!(seen = ld_acquire_gpu(p.flags + slot))) {
                if (*abort_flag) break;
                if (clock64() - t0 > kWaitLimitCycles) {
                  *abort_flag = 1;
                  if (atomicCAS(p.err, 0, kErrWaitOther) == 0) {
                    p.err[1] = static_cast<int>(blockIdx.x);
                    p.err[2] = unit.tile;
                  }
                  __threadfence();
                  break;
                }
                __nanosleep(64);
              }
            }
          }
          seen = __shfl_sync(0xffffffffu, seen, 0);
          if (!seen) ok = false;
        }
        // 32 accumulator columns per step; the neighbour's partial sums of the next step are
        // fetched while this one is converted.
        constexpr int kSteps = BN / 32;
        constexpr int kStepsPerChunk = kChunk / 32;
        const bool add_partial = unit.split && ok;
        float4 nxt[8];
        if (add_partial) {
#pragma unroll
          for (int q = 0; q < 8; ++q) nxt[q] = ld_cg_f4(part + q * 128);
        }
#pragma unroll 1
        for (int st = 0; st < kSteps; ++st) {
          const int c = st / kStepsPerChunk, h = st % kStepsPerChunk;
          const int col0 = unit.n0 + c * kChunk;
          const bool store = ok && has_rows && col0 < p.N;
          const uint32_t buf = sEpi + static_cast<uint32_t>((warp * 2 + sbuf) * EPI_BUF_BYTES);
          float4 add[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) add[q] = nxt[q];
          if (add_partial && st + 1 < kSteps) {
#pragma unroll
            for (int q = 0; q < 8; ++q) nxt[q] = ld_cg_f4(part + ((st + 1) * 8 + q) * 128);
          }
          if (store) {
            if (h == 0) {
              if (lane == 0) tma_store_wait_read<1>();
              __syncwarp();
            }
            uint32_t r[32];
            tmem_ld_32x32b_x32(t_acc + st * 32, r);
            tmem_ld_wait();
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
            if (add_partial) {
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                v[4 * q] += add[q].x;
                v[4 * q + 1] += add[q].y;
                v[4 * q + 2] += add[q].z;
                v[4 * q + 3] += add[q].w;
              }
            }
            gemm::stage_row32<OutT>(buf, lane, h * 32 * sizeof(OutT), v);
          }
          if (st == kSteps - 1) {
            // last read of this accumulator: hand it back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_even_cta(tempty_bar(acc));
          }
          if (store && h == kStepsPerChunk - 1) {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              const int n = p.num_peers;
              int idx = rot % n;
              for (int i = 0; i < n; ++i) {
                tma_store_3d(&peers.m[idx], buf, col0, row0, 0);
                if (++idx == n) idx = 0;
              }
              tma_store_commit();
            }
            ++rot;
            sbuf ^= 1;
          }
        }
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

}  // namespace gemm_ag
}  // namespace tsb
