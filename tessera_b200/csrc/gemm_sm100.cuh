// Persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
//   D[b][M,N] = A[b][M,K] * B[b][K,N]       A, B row-major 16-bit (bf16 or f16), f32 accumulate
//
// CTA = 6 warps: warps 0-3 epilogue (TMEM -> registers -> swizzled smem -> TMA store),
// warp 4 TMA producer, warp 5 MMA issuer + TMEM owner. One CTA per SM walks a static list of
// 128 x 256 output tiles; the accumulator is double-buffered in TMEM (2 x 256 columns) so the
// epilogue of tile i overlaps the main loop of tile i+1.
//
// Shared memory per stage: A tile 128 x 64 (K-major, 128-byte swizzle, 16 KB) and B tile
// 64 x 256 (N-major: four [64 k][64 n] 128-byte-swizzled blocks of 8 KB). Each 64-deep stage
// feeds four tcgen05.mma (M128 N256 K16).
//
// With kFp8 the operands are e4m3 bytes, both K-major: A[M,K] as before and B given TRANSPOSED as
// Bt[N,K] (per batch / expert), a stage covers 128 elements of K (same bytes: A 16 KB, B 32 KB as
// 256 rows of 128 B), the MMA is kind::f8f6f4 (K 32 per instruction) and the epilogue applies the
// dequantisation scales. Everything else — ring, barriers, tile walk, epilogue paths — is shared.
//
// Three tile sources share the kernel:
//   kPlain          batched dense GEMM (TMA clips ragged edges)
//   kGrouped        ragged grouped GEMM: rows of group e (contiguous, from `group_offsets`)
//                   times B[e]; tiles never straddle a group, partial tiles use masked stores
//   kGroupedSwiGLU  as kGrouped, but the 256 accumulator columns hold 128 gate columns and
//                   the matching 128 up columns and the epilogue writes silu(gate) * up
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "sm100_ptx.cuh"

namespace tsb {
namespace gemm {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int GROUP_M = 16;  // m-tiles per raster group (L2 reuse)
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int B_BLOCK_BYTES = BK * 64 * 2;  // one [64 k][64 n] block
constexpr int B_STAGE_BYTES = BK * BN * 2;
constexpr int STAGE_TX_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int EPI_BUF_BYTES = 32 * 128;  // 32 rows x 128 B per epilogue warp buffer
constexpr int SMEM_A_OFF = 0;
constexpr int SMEM_B_OFF = SMEM_A_OFF + STAGES * A_STAGE_BYTES;
constexpr int SMEM_EPI_OFF = SMEM_B_OFF + STAGES * B_STAGE_BYTES;
constexpr int SMEM_BAR_OFF = SMEM_EPI_OFF + 4 * 2 * EPI_BUF_BYTES;
constexpr int SMEM_BYTES = SMEM_BAR_OFF + 128;
constexpr int SMEM_ALLOC = SMEM_BYTES + 1024;  // slack for 1024-byte alignment of the base
constexpr int NUM_THREADS = 192;
constexpr uint32_t TMEM_COLS = 512;

enum Mode : int { kPlain = 0, kGrouped = 1, kGroupedSwiGLU = 2 };

struct Params {
  int M, N, K, batch;   // plain: per-batch sizes. grouped: M = total rows, batch = #groups
  int m_tiles, n_tiles; // n_tiles is per output tile width (256, or 128 for SwiGLU)
  uint32_t idesc;
  const int* group_offsets;  // grouped modes: batch + 1 row offsets (device memory)
  void* D;                   // grouped modes: output base for masked stores
  long long ldd;             // grouped modes: output leading dimension (elements)
  // all-gather kernel only (gemm_ag_sm100.cuh): number of output copies, where this rank's
  // rotation over them starts, and the split of the K loop in two (fp32 partial sums and one flag
  // per epilogue warp and tile in a device workspace, flags zeroed before the launch)
  int num_peers;
  int peer_first;
  int ksplit;
  float* partial;
  int* flags;
  // plain mode, optional fused epilogue: D = act(A*B + bias[col] + residual[row, col])
  const float* bias;         // [N] fp32 or null
  const void* residual;      // [M, N] in the output dtype, leading dimension ldr, or null
  long long ldr;
  int activation;            // 0 none, 1 relu, 2 gelu (tanh form), 3 silu
  // fp8 operands (kFp8): D = (A_q * B_q) * scale_a[0] * scale_b[group or batch index]; the SwiGLU
  // mode scales the up half with scale_b2. amax_out (optional) receives max |D| of the values as
  // stored (bit pattern of a non-negative float, combined with atomicMax).
  const float* scale_a;
  const float* scale_b;
  const float* scale_b2;
  unsigned int* amax_out;
  int* err;
};

// Output tensor maps of every rank's copy of Y, for the column-parallel GEMM whose epilogue is the
// all-gather (gemm_ag_sm100.cuh).
constexpr int MAX_PEERS = 8;
struct PeerMaps {
  CUtensorMap m[MAX_PEERS];
};

struct Tile {
  int m0, n0, b, rows;
};

template <int kMode>
struct TileWalker {
  int t, step;
  int e = 0, base = 0;  // grouped cursor
  __device__ TileWalker(int first, int stride) : t(first), step(stride) {}

  __device__ bool next(const Params& p, Tile& out) {
    if constexpr (kMode == kPlain) {
      const int per_b = p.m_tiles * p.n_tiles;
      if (t >= per_b * p.batch) return false;
      const int b = t / per_b;
      const int r = t - b * per_b;
      const int gspan = GROUP_M * p.n_tiles;
      const int g = r / gspan;
      const int first_m = g * GROUP_M;
      const int gsz = min(p.m_tiles - first_m, GROUP_M);
      const int rr = r - g * gspan;
      out.m0 = (first_m + rr % gsz) * BM;
      out.n0 = (rr / gsz) * BN;
      out.b = b;
      out.rows = BM;
    } else {
      constexpr int kOutW = (kMode == kGroupedSwiGLU) ? BN / 2 : BN;
      int rows_e = 0, mt = 0;
      while (e < p.batch) {
        rows_e = p.group_offsets[e + 1] - p.group_offsets[e];
        mt = (rows_e + BM - 1) / BM;
        const int cnt = mt * p.n_tiles;
        if (t < base + cnt) break;
        base += cnt;
        ++e;
      }
      if (e >= p.batch) return false;
      const int local = t - base;
      const int n_idx = local / mt;
      const int m_idx = local - n_idx * mt;
      out.m0 = p.group_offsets[e] + m_idx * BM;
      out.n0 = n_idx * kOutW;
      out.b = e;
      out.rows = min(BM, rows_e - m_idx * BM);
    }
    t += step;
    return true;
  }
};

// Converts 32 consecutive f32 values of one row to OutT and writes them, 16 bytes at a time,
// to the swizzled staging row. `col_bytes0` is the byte offset of v[0] inside the 128-byte row.
template <typename OutT>
__device__ __forceinline__ void stage_row32(uint32_t buf, uint32_t row, uint32_t col_bytes0,
                                            const float (&v)[32]) {
  if constexpr (sizeof(OutT) == 4) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t addr = buf + swz128(row, (col_bytes0 >> 4) + j);
      asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v[4 * j]),
                   "f"(v[4 * j + 1]), "f"(v[4 * j + 2]), "f"(v[4 * j + 3])
                   : "memory");
    }
  } else {
    uint32_t w[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      if constexpr (std::is_same<OutT, __nv_bfloat16>::value) {
        __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
        w[j] = *reinterpret_cast<uint32_t*>(&h);
      } else {
        __half2 h = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
        w[j] = *reinterpret_cast<uint32_t*>(&h);
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t addr = buf + swz128(row, (col_bytes0 >> 4) + j);
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[4 * j]),
                   "r"(w[4 * j + 1]), "r"(w[4 * j + 2]), "r"(w[4 * j + 3])
                   : "memory");
    }
  }
}

// bias + residual + activation on 32 consecutive columns of one output row, in the order of the
// reference's fused_epilogue (python/tessera/__init__.py:2658-2675): bias, residual, activation.
template <typename OutT>
__device__ __forceinline__ void apply_epilogue(float (&v)[32], const Params& p, int row, int col0) {
  if (row >= p.M) return;
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    const int col = col0 + j;
    if (col < p.N) {
      float x = v[j];
      if (p.bias) x += __ldg(p.bias + col);
      if (p.residual) {
        const OutT* r = static_cast<const OutT*>(p.residual) + static_cast<long long>(row) * p.ldr + col;
        x += static_cast<float>(*r);
      }
      if (p.activation == 1) {
        x = fmaxf(x, 0.f);
      } else if (p.activation == 2) {
        x = 0.5f * x * (1.0f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
      } else if (p.activation == 3) {
        x = x / (1.0f + __expf(-x));
      }
      v[j] = x;
    }
  }
}

// max |x| over 32 values after rounding to the stored type (what a later quantisation will see).
template <typename OutT>
__device__ __forceinline__ float stored_amax32(const float (&v)[32]) {
  float a = 0.f;
#pragma unroll
  for (int j = 0; j < 32; ++j) a = fmaxf(a, fabsf(static_cast<float>(static_cast<OutT>(v[j]))));
  return a;
}

__device__ __forceinline__ float silu_mul(float g, float u) {
  return __fdividef(g, 1.0f + __expf(-g)) * u;
}

template <typename OutT, int kMode, bool kFp8 = false>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ CUtensorMap tmB2, const __grid_constant__ CUtensorMap tmD,
            const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const uint32_t sA = smem_base + SMEM_A_OFF;
  const uint32_t sB = smem_base + SMEM_B_OFF;
  const uint32_t sEpi = smem_base + SMEM_EPI_OFF;
  const uint32_t bars = smem_base + SMEM_BAR_OFF;
  // barrier layout: full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2]
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
  constexpr int kBKe = kFp8 ? 2 * BK : BK;  // K elements per stage (128 bytes of K either way)
  const int num_kb = (p.K + kBKe - 1) / kBKe;
  constexpr int kOutW = (kMode == kGroupedSwiGLU) ? BN / 2 : BN;   // output columns per tile
  constexpr int kChunk = (sizeof(OutT) == 4) ? 32 : 64;            // output columns per store

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);
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
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      TileWalker<kMode> walk(blockIdx.x, gridDim.x);
      Tile tile;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      while (ok && walk.next(p, tile)) {
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.err, kErrWaitEmpty, kb)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(full_bar(stage), STAGE_TX_BYTES);
          const int k0 = kb * kBKe;
          const int a_b = (kMode == kPlain) ? tile.b : 0;
          tma_load_3d(sA + stage * A_STAGE_BYTES, &tmA, full_bar(stage), k0, tile.m0, a_b);
          const uint32_t b_dst = sB + stage * B_STAGE_BYTES;
          if constexpr (kFp8) {
            // Bt[N,K]: two boxes of 128 rows x 128 B. SwiGLU: gate rows, then the same rows of up.
            const CUtensorMap* second = (kMode == kGroupedSwiGLU) ? &tmB2 : &tmB;
            const int n1 = (kMode == kGroupedSwiGLU) ? tile.n0 : tile.n0 + 128;
            tma_load_3d(b_dst, &tmB, full_bar(stage), k0, tile.n0, tile.b);
            tma_load_3d(b_dst + B_STAGE_BYTES / 2, second, full_bar(stage), k0, n1, tile.b);
          } else if constexpr (kMode == kGroupedSwiGLU) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              tma_load_3d(b_dst + j * B_BLOCK_BYTES, &tmB, full_bar(stage), tile.n0 + 64 * j, k0,
                          tile.b);
              tma_load_3d(b_dst + (j + 2) * B_BLOCK_BYTES, &tmB2, full_bar(stage),
                          tile.n0 + 64 * j, k0, tile.b);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              tma_load_3d(b_dst + j * B_BLOCK_BYTES, &tmB, full_bar(stage), tile.n0 + 64 * j, k0,
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
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      TileWalker<kMode> walk(blockIdx.x, gridDim.x);
      Tile tile;
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
          // Descriptor low words of this stage; per MMA only a constant is added to the start
          // address field (16-byte units). A: K-major, 16 elements = 32 B inside the 128-byte
          // swizzle row. B: N-major, 16 k-rows = 2048 B; 64-column blocks are 8 KB apart (LBO).
          const uint32_t a_lo = a_lo0 + stage * (A_STAGE_BYTES >> 4);
          const uint32_t b_lo = b_lo0 + stage * (B_STAGE_BYTES >> 4);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            // 32 bytes of K per step in a K-major operand; 16 k-rows = 2048 B in the N-major B.
            if constexpr (kFp8)
              umma_f8_ss_parts(d_tmem, a_lo + k * 2, desc_hi, b_lo + k * 2, desc_hi, p.idesc,
                               (kb > 0 || k > 0) ? 1u : 0u);
            else
              umma_f16_ss_parts(d_tmem, a_lo + k * 2, desc_hi, b_lo + k * 128, desc_hi, p.idesc,
                                (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit(tfull_bar(acc));
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps 0..3
    TileWalker<kMode> walk(blockIdx.x, gridDim.x);
    Tile tile;
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
      const int row0 = tile.m0 + 32 * warp;          // first output row of this warp
      const int rows_w = max(0, min(32, tile.rows - 32 * warp));  // valid rows (grouped)
      const int m_limit = (kMode == kPlain) ? p.M : (tile.m0 + tile.rows);
      const bool warp_has_rows = (kMode == kPlain) ? (row0 < p.M) : (rows_w > 0);
      const uint32_t t_acc = tmem_base + static_cast<uint32_t>(acc * BN) + lane_base;
      constexpr int kChunks = kOutW / kChunk;
      // dequantisation scales of this tile (1 when the operands are 16-bit)
      float sc = 1.f, sc2 = 1.f, amax = 0.f;
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
#pragma unroll 1
      for (int c = 0; c < kChunks; ++c) {
        const int col0 = tile.n0 + c * kChunk;
        if (col0 >= p.N || !warp_has_rows) break;
        const uint32_t buf = sEpi + static_cast<uint32_t>((warp * 2 + sbuf) * EPI_BUF_BYTES);
        // The TMA store that last read this buffer must be done reading it.
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
              v[j] = silu_mul(__uint_as_float(g[j]) * sc, __uint_as_float(u[j]) * sc2);
            if constexpr (kFp8) amax = fmaxf(amax, stored_amax32<OutT>(v));
            stage_row32<OutT>(buf, lane, h * 32 * sizeof(OutT), v);
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
                apply_epilogue<OutT>(v, p, row0 + lane, col0 + h * 32);
            }
            if constexpr (kFp8) amax = fmaxf(amax, stored_amax32<OutT>(v));
            stage_row32<OutT>(buf, lane, h * 32 * sizeof(OutT), v);
          }
        }
        if (c == kChunks - 1 || col0 + kChunk >= p.N) {
          // Last read of this accumulator: hand it back to the MMA warp.
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(tempty_bar(acc));
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
          // Partial tile of a ragged group: copy valid rows out with predicated 16-byte stores.
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
      if (!warp_has_rows || tile.n0 >= p.N) {
        // Nothing to store for this warp, still release the accumulator.
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(acc));
      }
      (void)m_limit;
      if constexpr (kFp8) {
        // rows beyond the valid range hold products of foreign rows: only lanes with a valid row count
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
    // A wait expired: give copies still in flight time to land before shared memory goes away.
    for (int i = 0; i < 64; ++i) __nanosleep(10000);
    __syncthreads();
  }
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace gemm
}  // namespace tsb
