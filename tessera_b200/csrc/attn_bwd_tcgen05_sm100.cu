// Attention backward with tcgen05 MMA and TMEM accumulators: bf16, D = Dv = 128, no bias / window /
// soft-cap, bottom-right causal mask, grouped-query heads. Same mathematics and the same ownership
// (one CTA per block of gradient rows, fixed summation order, no atomics) as the mma.sync kernels
// in attn_bwd_tc_sm100.cu; inputs are the forward's row log-sum-exps (base 2) and delta = dO . O.
//
// dkv5_kernel: one CTA per 128 keys of one KV head. K and V stay in shared memory; the Q and dO
// tiles (128 query rows) of every query head of the group stream through a two-deep TMA ring.
// Per tile the MMA warp forms the TRANSPOSED products S^T = K Q^T and dP^T = V dO^T into TMEM
// (keys on the 128 lanes, query rows along the columns), the four softmax warps (thread = key)
// turn them in place into bf16 P^T and dS^T, and the MMA warp accumulates dV += P^T dO and
// dK += dS^T Q with the A operand read straight from TMEM. The tile's 128 query rows are handled as
// two halves of 64 with their own score buffers, so the softmax warps convert one half while the
// tensor core finishes the other and starts the next tile. TMEM: (S^T_h | dP^T_h) x 2 halves of
// 64 fp32 columns, then dV and dK, 128 columns each.
// dq5_kernel: one CTA per 128 query rows of one head. Q and dO stay, K and V stream; S = Q K^T and
// dP = dO V^T, dS in place (thread = query row, so lse and delta are per-thread scalars), and
// dQ += dS K, with the same two-half schedule over the 128 keys of a tile. TMEM: (S_h | dP_h) x 2, dQ.
// Warps 0-3 softmax + epilogue (TMEM lane = 32 * warp + lane), warp 4 MMA issuer and TMEM owner,
// warp 5 TMA producer. Every wait is bounded (error word + abort flag), as in the forward kernel.
#include <cuda_bf16.h>

#include <cmath>

#include "../../include/tessera_sm100.h"
#include "device_ctx.h"
#include "sm100_ptx.cuh"

namespace tsb {
namespace attn_bwd5 {

constexpr int D = 128;
constexpr int BLK = 128;
constexpr int TILE_BYTES = 128 * 128 * 2;
constexpr int HALF_BYTES = TILE_BYTES / 2;
constexpr int SMEM_BAR_OFF = 6 * TILE_BYTES;               // six 32 KB tiles
constexpr int SMEM_STAT_OFF = SMEM_BAR_OFF + 256;           // lse[2][128], delta[2][128] (dkv only)
constexpr int SMEM_BYTES = SMEM_STAT_OFF + 4 * BLK * 4;
constexpr int SMEM_ALLOC = SMEM_BYTES + 1024;
constexpr int THREADS = 192;

struct Params {
  int B, Hq, Hkv, Sq, Sk;
  int causal, shift;
  float scale, scale_log2;
  const float* lse2;
  const float* delta;
  int* err;
};

// Optional timeline of one dK/dV CTA (compile with -DTESSERA_BWD_TRACE): clock64 stamps of the hand-offs
// between the softmax warps and the MMA warp, read back with tessera_sm100_bwd_trace_read. Not part
// of the normal build.
#ifdef TESSERA_BWD_TRACE
__device__ long long g_bwd_trace[2 * 4096];
#define BW_TRACE(role, idx)                                                              \
  do {                                                                                   \
    if (trace_on && (idx) < 4096) g_bwd_trace[(role) * 4096 + (idx)] = clock64();        \
  } while (0)
#else
#define BW_TRACE(role, idx) \
  do {                      \
  } while (0)
#endif

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
// The same pack on the integer pipe (compile with -DTESSERA_BWD_ALU_PACK): add half an ulp of bf16 to
// the bit pattern and keep the upper halves (round half away from zero). It takes the convert off
// the special-function pipe it shares with ex2; measured, the step time does not change (5.65 ms
// either way), so the conversion loop is not bound by that pipe and the exact convert stays.
__device__ __forceinline__ uint32_t pack_bf16_alu(float lo, float hi) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, 0x7632;" : "=r"(d) : "r"(__float_as_uint(lo) + 0x8000u), "r"(__float_as_uint(hi) + 0x8000u));
  return d;
}
#ifdef TESSERA_BWD_ALU_PACK
#define PACK_PROB pack_bf16_alu
#else
#define PACK_PROB pack_bf16
#endif

// Half-tile forms for the two-buffer schedule: 64 rows of B per product.
// d_tmem[128 x 64] = A(128 rows) . B(rows 64h .. 64h+63)^T over d
__device__ __forceinline__ void issue_rows_x_half(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, int h,
                                                  uint32_t desc_hi, uint32_t idesc) {
  const uint32_t brow = static_cast<uint32_t>(h * 64 * 128) >> 4;   // 64 rows of 128 B inside each half-tile
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    const uint32_t off = ((ks >> 2) * HALF_BYTES + (ks & 3) * 32) >> 4;
    umma_f16_ss_parts(d_tmem, a_lo + off, desc_hi, b_lo + brow + off, desc_hi, idesc, ks > 0 ? 1u : 0u);
  }
}
// d_tmem[128 x 128 d] (+)= A (bf16 in TMEM, 128 lanes x 64) . B rows 64h .. 64h+63 of an MN-major tile
__device__ __forceinline__ void issue_tmem_x_half(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, int h,
                                                  uint32_t desc_hi, uint32_t idesc, bool accumulate) {
#pragma unroll
  for (int ks = 0; ks < 4; ++ks)
    umma_f16_ts_parts(d_tmem, a_tmem + 8u * ks, b_lo + (((4 * h + ks) * 2048) >> 4), desc_hi, idesc,
                      (accumulate || ks > 0) ? 1u : 0u);
}

// accumulator (128 lanes x 128 fp32 columns at t_acc) * mul -> bf16 -> swizzled tile at obuf
__device__ __forceinline__ void acc_to_smem(uint32_t t_acc, uint32_t obuf, int r, float mul) {
#pragma unroll 1
  for (int c = 0; c < 4; ++c) {
    uint32_t v[32];
    tmem_ld_32x32b_x32(t_acc + c * 32, v);
    tmem_ld_wait();
    const uint32_t blk = obuf + (c >> 1) * HALF_BYTES;
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) {
      uint32_t w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e)
        w[e] = pack_bf16(__uint_as_float(v[ch * 8 + 2 * e]) * mul, __uint_as_float(v[ch * 8 + 2 * e + 1]) * mul);
      const uint32_t addr = blk + swz128(r, (c & 1) * 4 + ch);
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                   : "memory");
    }
  }
}
__device__ __forceinline__ void zeros_to_smem(uint32_t obuf, int r) {
#pragma unroll
  for (int ch = 0; ch < 16; ++ch)
    asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(obuf + (ch >> 3) * HALF_BYTES + swz128(r, ch & 7)), "r"(0)
                 : "memory");
}

__global__ void __launch_bounds__(THREADS, 1)
dkv5_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
            const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
            const __grid_constant__ CUtensorMap tmdK, const __grid_constant__ CUtensorMap tmdV, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sK = smem_base, sV = smem_base + TILE_BYTES;
  const uint32_t sQ = smem_base + 2 * TILE_BYTES, sdO = smem_base + 4 * TILE_BYTES;
  const uint32_t bars = smem_base + SMEM_BAR_OFF;
  const uint32_t kv_full = bars;
  auto q_full = [&](int s) { return bars + 8u * (1 + s); };
  auto q_empty = [&](int s) { return bars + 8u * (3 + s); };
  auto s_full = [&](int h) { return bars + 8u * (5 + h); };   // scores of half h (64 query rows) ready
  auto p_full = [&](int h) { return bars + 8u * (7 + h); };   // P^T / dS^T of half h written
  const uint32_t o_full = bars + 8u * 9;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + SMEM_BAR_OFF + 128);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + SMEM_BAR_OFF + 132);
  float* s_lse = reinterpret_cast<float*>(smem_gen + SMEM_STAT_OFF);   // [2][128]
  float* s_del = s_lse + 2 * BLK;                                      // [2][128]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BLK, hk = blockIdx.y, b = blockIdx.z;
#ifdef TESSERA_BWD_TRACE
  const bool trace_on = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && lane == 0 && (warp == 0 || warp == 4);
#endif
  const int ratio = p.Hq / p.Hkv;
  const int nqb = (p.Sq + BLK - 1) / BLK;
  const int i_start = p.causal ? max(0, n0 - p.shift) / BLK : 0;   // first block with a legal row
  const int per_head = max(0, nqb - i_start);
  const int iters = per_head * ratio;
  auto head_of = [&](int it) { return hk * ratio + it / per_head; };
  auto m0_of = [&](int it) { return (i_start + it % per_head) * BLK; };

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(q_full(s), 1);
      mbar_init(q_empty(s), 1);
    }
    for (int h = 0; h < 2; ++h) {
      mbar_init(s_full(h), 1);
      mbar_init(p_full(h), 4);   // one arrival per softmax warp
    }
    mbar_init(o_full, 1);
    fence_mbar_init();
  }
  if (warp == 4) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // TMEM: per half h of the query tile S^T_h (64 columns) | dP^T_h (64), then dV and dK
  auto tS = [&](int h) { return tmem_base + static_cast<uint32_t>(128 * h); };
  auto tdP = [&](int h) { return tmem_base + static_cast<uint32_t>(128 * h + 64); };
  const uint32_t tdV = tmem_base + 256, tdK = tmem_base + 384;

  if (warp == 5) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && iters > 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmdO);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      mbar_arrive_expect_tx(kv_full, 2 * TILE_BYTES);
      tma_load_4d(sK, &tmK, kv_full, 0, n0, hk, b);
      tma_load_4d(sK + HALF_BYTES, &tmK, kv_full, 64, n0, hk, b);
      tma_load_4d(sV, &tmV, kv_full, 0, n0, hk, b);
      tma_load_4d(sV + HALF_BYTES, &tmV, kv_full, 64, n0, hk, b);
      for (int it = 0; it < iters; ++it) {
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait(q_empty(st), ph ^ 1u, abort_flag, p.err, kErrWaitEmpty, it)) break;
        const int hq = head_of(it), m0 = m0_of(it);
        mbar_arrive_expect_tx(q_full(st), 2 * TILE_BYTES);
        tma_load_4d(sQ + st * TILE_BYTES, &tmQ, q_full(st), 0, m0, hq, b);
        tma_load_4d(sQ + st * TILE_BYTES + HALF_BYTES, &tmQ, q_full(st), 64, m0, hq, b);
        tma_load_4d(sdO + st * TILE_BYTES, &tmdO, q_full(st), 0, m0, hq, b);
        tma_load_4d(sdO + st * TILE_BYTES + HALF_BYTES, &tmdO, q_full(st), 64, m0, hq, b);
      }
    }
  } else if (warp == 4) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && iters > 0) {
      const uint32_t idesc_ss = make_idesc_f16(true, false, false, BLK, 64);    // 128 keys x 64 query rows
      const uint32_t idesc_ts = make_idesc_f16(true, false, true, BLK, D);      // TMEM A, N-major B
      const uint32_t desc_hi = smem_desc_hi(1024);
      const uint32_t k_lo = smem_desc_lo(sK, 16), v_lo = smem_desc_lo(sV, 16);
      const uint32_t q_lo[2] = {smem_desc_lo(sQ, 16), smem_desc_lo(sQ + TILE_BYTES, 16)};
      const uint32_t g_lo[2] = {smem_desc_lo(sdO, 16), smem_desc_lo(sdO + TILE_BYTES, 16)};
      const uint32_t qn_lo[2] = {smem_desc_lo(sQ, HALF_BYTES), smem_desc_lo(sQ + TILE_BYTES, HALF_BYTES)};
      const uint32_t gn_lo[2] = {smem_desc_lo(sdO, HALF_BYTES), smem_desc_lo(sdO + TILE_BYTES, HALF_BYTES)};
      bool ok = mbar_wait(kv_full, 0, abort_flag, p.err, kErrWaitFull, 1000);
      // The tile's 128 query rows are handled as two halves with their own TMEM buffers, so the
      // softmax warps work on one half while the tensor core finishes the other and starts the
      // next tile's scores.
      auto issue_scores = [&](int it, int h) {
        const int st = it & 1;
        if (h == 0) {
          if (!(ok = mbar_wait(q_full(st), (it >> 1) & 1, abort_flag, p.err, kErrWaitFull, it))) return;
          tc_fence_after();
        }
        issue_rows_x_half(tS(h), k_lo, q_lo[st], h, desc_hi, idesc_ss);     // S^T_h  = K Q_h^T
        issue_rows_x_half(tdP(h), v_lo, g_lo[st], h, desc_hi, idesc_ss);    // dP^T_h = V dO_h^T
        umma_commit(s_full(h));
      };
      if (ok) issue_scores(0, 0);
      if (ok) issue_scores(0, 1);
      for (int it = 0; it < iters && ok; ++it) {
        const int st = it & 1;
        for (int h = 0; h < 2 && ok; ++h) {
          BW_TRACE(1, (it * 2 + h) * 4 + 0);
          if (!(ok = mbar_wait(p_full(h), it & 1, abort_flag, p.err, kErrWaitOther, 2000 + it))) break;
          BW_TRACE(1, (it * 2 + h) * 4 + 1);
          tc_fence_after();
          issue_tmem_x_half(tdV, tS(h), gn_lo[st], h, desc_hi, idesc_ts, it > 0 || h > 0);    // dV += P^T_h dO_h
          issue_tmem_x_half(tdK, tdP(h), qn_lo[st], h, desc_hi, idesc_ts, it > 0 || h > 0);   // dK += dS^T_h Q_h
          if (h == 1) umma_commit(q_empty(st));
          BW_TRACE(1, (it * 2 + h) * 4 + 2);
          if (it + 1 < iters) issue_scores(it + 1, h);
          else if (h == 1) umma_commit(o_full);
          BW_TRACE(1, (it * 2 + h) * 4 + 3);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax warps: thread = key
    const int r = warp * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const int key = n0 + r;
    const bool key_ok = key < p.Sk;
    bool ok = true;
    float lse_n = INFINITY, del_n = 0.f;
    auto fetch_stats = [&](int it) {   // this thread's COLUMN (query row m0 + r) of tile `it`
      const int m = m0_of(it) + r;
      const long long row = (static_cast<long long>(b) * p.Hq + head_of(it)) * p.Sq + m;
      lse_n = m < p.Sq ? p.lse2[row] : INFINITY;   // a row that does not exist: p = 0
      del_n = m < p.Sq ? p.delta[row] : 0.f;
    };
    if (iters > 0) fetch_stats(0);
    // Every thread runs every iteration and meets the named barrier even after a wait has given up
    // (`ok` only gates the work): a thread that left early would leave the others at the barrier.
    for (int it = 0; it < iters; ++it) {
      const int sl = (it & 1) * BLK;
      s_lse[sl + r] = lse_n;
      s_del[sl + r] = del_n;
      if (it + 1 < iters) fetch_stats(it + 1);
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const int m0 = m0_of(it);
      // query rows of this tile the key is legal for: m >= key - shift (causal)
      const int m_first = p.causal ? key - p.shift : -0x40000000;
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {            // 64 query columns per half
        BW_TRACE(0, (it * 2 + h) * 4 + 0);
        if (ok) ok = mbar_wait(s_full(h), it & 1, abort_flag, p.err, kErrWaitTmemFull, it);
        if (!ok) continue;
        BW_TRACE(0, (it * 2 + h) * 4 + 1);
        tc_fence_after();
        uint32_t pk[32], dk[32];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int c0 = half * 32;
          uint32_t s[32], g[32];
          tmem_ld_32x32b_x32(tS(h) + lane_base + c0, s);
          tmem_ld_32x32b_x32(tdP(h) + lane_base + c0, g);
          tmem_ld_wait();
#pragma unroll
          for (int k = 0; k < 32; k += 2) {
            float pe[2], ds[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int col = 64 * h + c0 + k + e;
              const bool legal = key_ok && (m0 + col >= m_first);
              const float x = __uint_as_float(s[k + e]) * p.scale_log2 - s_lse[sl + col];
              pe[e] = legal ? ex2(x) : 0.f;
              ds[e] = pe[e] * (__uint_as_float(g[k + e]) - s_del[sl + col]);
            }
            pk[half * 16 + (k >> 1)] = PACK_PROB(pe[0], pe[1]);
            dk[half * 16 + (k >> 1)] = PACK_PROB(ds[0], ds[1]);
          }
        }
        // bf16 P^T_h / dS^T_h over the columns just consumed: 64 fp32 columns -> 32 packed columns
        BW_TRACE(0, (it * 2 + h) * 4 + 2);
        tmem_st_32x32b_x32(tS(h) + lane_base, pk);
        tmem_st_32x32b_x32(tdP(h) + lane_base, dk);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full(h));
        BW_TRACE(0, (it * 2 + h) * 4 + 3);
      }
    }
    // ---- epilogue: dV, scale * dK -> bf16 -> swizzled smem (the Q ring) -> TMA store
    if (iters > 0) {
      if (ok) ok = mbar_wait(o_full, 0, abort_flag, p.err, kErrWaitTmemFull, 9000);
      tc_fence_after();
      acc_to_smem(tdV + lane_base, sQ, r, 1.0f);
      acc_to_smem(tdK + lane_base, sQ + TILE_BYTES, r, p.scale);
    } else {
      zeros_to_smem(sQ, r);
      zeros_to_smem(sQ + TILE_BYTES, r);
    }
    fence_proxy_async_smem();
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (r == 0 && ok) {
      tma_store_4d(&tmdV, sQ, 0, n0, hk, b);
      tma_store_4d(&tmdV, sQ + HALF_BYTES, 64, n0, hk, b);
      tma_store_4d(&tmdK, sQ + TILE_BYTES, 0, n0, hk, b);
      tma_store_4d(&tmdK, sQ + TILE_BYTES + HALF_BYTES, 64, n0, hk, b);
      tma_store_commit();
      tma_store_wait<0>();
    }
  }
  // -------------------------------------------------------------------- tear-down
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int k = 0; k < 64; ++k) __nanosleep(10000);
    __syncthreads();
  }
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

__global__ void __launch_bounds__(THREADS, 1)
dq5_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
           const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
           const __grid_constant__ CUtensorMap tmdQ, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sQ = smem_base, sdO = smem_base + TILE_BYTES;
  const uint32_t sK = smem_base + 2 * TILE_BYTES, sV = smem_base + 4 * TILE_BYTES;
  const uint32_t bars = smem_base + SMEM_BAR_OFF;
  const uint32_t q_full = bars;
  auto kv_full = [&](int s) { return bars + 8u * (1 + s); };
  auto kv_empty = [&](int s) { return bars + 8u * (3 + s); };
  auto s_full = [&](int h) { return bars + 8u * (5 + h); };
  auto p_full = [&](int h) { return bars + 8u * (7 + h); };
  const uint32_t o_full = bars + 8u * 9;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + SMEM_BAR_OFF + 128);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + SMEM_BAR_OFF + 132);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = (gridDim.x - 1 - blockIdx.x) * BLK;   // the longest rows first
  const int hq = blockIdx.y, b = blockIdx.z;
  const int hk = hq / (p.Hq / p.Hkv);
  int n_end = p.Sk;
  if (p.causal) n_end = min(n_end, min(m0 + BLK - 1, p.Sq - 1) + p.shift + 1);
  const int iters = n_end > 0 ? (n_end + BLK - 1) / BLK : 0;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(kv_full(s), 1);
      mbar_init(kv_empty(s), 1);
    }
    for (int h = 0; h < 2; ++h) {
      mbar_init(s_full(h), 1);
      mbar_init(p_full(h), 4);
    }
    mbar_init(o_full, 1);
    fence_mbar_init();
  }
  if (warp == 4) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // TMEM: per half h of the key tile S_h (64 columns) | dP_h (64), then dQ
  auto tS = [&](int h) { return tmem_base + static_cast<uint32_t>(128 * h); };
  auto tdP = [&](int h) { return tmem_base + static_cast<uint32_t>(128 * h + 64); };
  const uint32_t tdQ = tmem_base + 256;

  if (warp == 5) {
    if (lane == 0 && iters > 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmdO);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      mbar_arrive_expect_tx(q_full, 2 * TILE_BYTES);
      tma_load_4d(sQ, &tmQ, q_full, 0, m0, hq, b);
      tma_load_4d(sQ + HALF_BYTES, &tmQ, q_full, 64, m0, hq, b);
      tma_load_4d(sdO, &tmdO, q_full, 0, m0, hq, b);
      tma_load_4d(sdO + HALF_BYTES, &tmdO, q_full, 64, m0, hq, b);
      for (int it = 0; it < iters; ++it) {
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait(kv_empty(st), ph ^ 1u, abort_flag, p.err, kErrWaitEmpty, it)) break;
        mbar_arrive_expect_tx(kv_full(st), 2 * TILE_BYTES);
        tma_load_4d(sK + st * TILE_BYTES, &tmK, kv_full(st), 0, it * BLK, hk, b);
        tma_load_4d(sK + st * TILE_BYTES + HALF_BYTES, &tmK, kv_full(st), 64, it * BLK, hk, b);
        tma_load_4d(sV + st * TILE_BYTES, &tmV, kv_full(st), 0, it * BLK, hk, b);
        tma_load_4d(sV + st * TILE_BYTES + HALF_BYTES, &tmV, kv_full(st), 64, it * BLK, hk, b);
      }
    }
  } else if (warp == 4) {
    if (lane == 0 && iters > 0) {
      const uint32_t idesc_ss = make_idesc_f16(true, false, false, BLK, 64);
      const uint32_t idesc_ts = make_idesc_f16(true, false, true, BLK, D);
      const uint32_t desc_hi = smem_desc_hi(1024);
      const uint32_t q_lo = smem_desc_lo(sQ, 16), g_lo = smem_desc_lo(sdO, 16);
      const uint32_t k_lo[2] = {smem_desc_lo(sK, 16), smem_desc_lo(sK + TILE_BYTES, 16)};
      const uint32_t v_lo[2] = {smem_desc_lo(sV, 16), smem_desc_lo(sV + TILE_BYTES, 16)};
      const uint32_t kn_lo[2] = {smem_desc_lo(sK, HALF_BYTES), smem_desc_lo(sK + TILE_BYTES, HALF_BYTES)};
      bool ok = mbar_wait(q_full, 0, abort_flag, p.err, kErrWaitFull, 1000);
      auto issue_scores = [&](int it, int h) {
        const int st = it & 1;
        if (h == 0) {
          if (!(ok = mbar_wait(kv_full(st), (it >> 1) & 1, abort_flag, p.err, kErrWaitFull, it))) return;
          tc_fence_after();
        }
        issue_rows_x_half(tS(h), q_lo, k_lo[st], h, desc_hi, idesc_ss);     // S_h  = Q K_h^T
        issue_rows_x_half(tdP(h), g_lo, v_lo[st], h, desc_hi, idesc_ss);    // dP_h = dO V_h^T
        umma_commit(s_full(h));
      };
      if (ok) issue_scores(0, 0);
      if (ok) issue_scores(0, 1);
      for (int it = 0; it < iters && ok; ++it) {
        const int st = it & 1;
        for (int h = 0; h < 2 && ok; ++h) {
          if (!(ok = mbar_wait(p_full(h), it & 1, abort_flag, p.err, kErrWaitOther, 2000 + it))) break;
          tc_fence_after();
          issue_tmem_x_half(tdQ, tdP(h), kn_lo[st], h, desc_hi, idesc_ts, it > 0 || h > 0);   // dQ += dS_h K_h
          if (h == 1) umma_commit(kv_empty(st));
          if (it + 1 < iters) issue_scores(it + 1, h);
          else if (h == 1) umma_commit(o_full);
        }
      }
    }
  } else {
    // softmax warps: thread = query row
    const int r = warp * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const int m = m0 + r;
    const long long row = (static_cast<long long>(b) * p.Hq + hq) * p.Sq + m;
    const float lse = m < p.Sq ? p.lse2[row] : INFINITY;
    const float del = m < p.Sq ? p.delta[row] : 0.f;
    const int n_last = p.causal ? min(m + p.shift, p.Sk - 1) : p.Sk - 1;   // last legal key
    bool ok = true;
    for (int it = 0; it < iters && ok; ++it) {
#pragma unroll 1
      for (int h = 0; h < 2 && ok; ++h) {
        if (!(ok = mbar_wait(s_full(h), it & 1, abort_flag, p.err, kErrWaitTmemFull, it))) break;
        tc_fence_after();
        const int nb = it * BLK + 64 * h;
        uint32_t dk[32];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int c0 = half * 32;
          uint32_t s[32], g[32];
          tmem_ld_32x32b_x32(tS(h) + lane_base + c0, s);
          tmem_ld_32x32b_x32(tdP(h) + lane_base + c0, g);
          tmem_ld_wait();
#pragma unroll
          for (int k = 0; k < 32; k += 2) {
            float ds[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const bool legal = nb + c0 + k + e <= n_last;
              const float pe = legal ? ex2(__uint_as_float(s[k + e]) * p.scale_log2 - lse) : 0.f;
              ds[e] = pe * (__uint_as_float(g[k + e]) - del);
            }
            dk[half * 16 + (k >> 1)] = PACK_PROB(ds[0], ds[1]);
          }
        }
        tmem_st_32x32b_x32(tdP(h) + lane_base, dk);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full(h));
      }
    }
    if (iters > 0) {
      if (ok) ok = mbar_wait(o_full, 0, abort_flag, p.err, kErrWaitTmemFull, 9000);
      tc_fence_after();
      acc_to_smem(tdQ + lane_base, sK, r, p.scale);
    } else {
      zeros_to_smem(sK, r);
    }
    fence_proxy_async_smem();
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (r == 0 && ok) {
      tma_store_4d(&tmdQ, sK, 0, m0, hq, b);
      tma_store_4d(&tmdQ, sK + HALF_BYTES, 64, m0, hq, b);
      tma_store_commit();
      tma_store_wait<0>();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int k = 0; k < 64; ++k) __nanosleep(10000);
    __syncthreads();
  }
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// dO, Q, dQ [B,Hq,Sq,128]; K, V, dK, dV [B,Hkv,Sk,128] bf16 dense; lse2, delta [B,Hq,Sq] fp32.
int launch(const void* dO, const void* Q, const void* K, const void* V, void* dQ, void* dK, void* dV,
           const float* lse2, const float* delta, int B, int Hq, int Hkv, int Sq, int Sk, float scale,
           int causal, cudaStream_t st) {
  for (const void* ptr : {dO, Q, K, V, (const void*)dQ, (const void*)dK, (const void*)dV})
    if (reinterpret_cast<uintptr_t>(ptr) & 15) {
      set_last_error("flash_attn_bwd: pointers must be 16-byte aligned");
      return kBadArg;
    }
  CUtensorMap tQ, tdO, tK, tV, tdQ, tdK, tdV;
  uint32_t box[4] = {64, 128, 1, 1};
  auto encode = [&](CUtensorMap* m, const void* base, int S, int heads) {
    uint64_t dims[4] = {(uint64_t)D, (uint64_t)S, (uint64_t)heads, (uint64_t)B};
    uint64_t str[3] = {(uint64_t)D * 2, (uint64_t)S * D * 2, (uint64_t)heads * S * D * 2};
    return encode_tmap(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, base, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
  };
  if (!encode(&tQ, Q, Sq, Hq) || !encode(&tdO, dO, Sq, Hq) || !encode(&tdQ, dQ, Sq, Hq) ||
      !encode(&tK, K, Sk, Hkv) || !encode(&tV, V, Sk, Hkv) || !encode(&tdK, dK, Sk, Hkv) ||
      !encode(&tdV, dV, Sk, Hkv))
    return kBadArg;
  Params p{};
  p.B = B;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.Sq = Sq;
  p.Sk = Sk;
  p.causal = causal ? 1 : 0;
  p.shift = (causal && Sk > Sq) ? Sk - Sq : 0;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.lse2 = lse2;
  p.delta = delta;
  p.err = device_err_word();
  if (!p.err) return kDeviceFailed;
  TSB_CUDA_OK(cudaFuncSetAttribute(dq5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_ALLOC));
  TSB_CUDA_OK(cudaFuncSetAttribute(dkv5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_ALLOC));
  dim3 g1((Sq + BLK - 1) / BLK, Hq, B);
  dq5_kernel<<<g1, THREADS, SMEM_ALLOC, st>>>(tQ, tdO, tK, tV, tdQ, p);
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  dim3 g2((Sk + BLK - 1) / BLK, Hkv, B);
  dkv5_kernel<<<g2, THREADS, SMEM_ALLOC, st>>>(tQ, tdO, tK, tV, tdK, tdV, p);
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  return kOk;
}

}  // namespace attn_bwd5
}  // namespace tsb

#ifdef TESSERA_BWD_TRACE
extern "C" int tessera_sm100_bwd_trace_read(long long* out, int n) {
  return cudaMemcpyFromSymbol(out, tsb::attn_bwd5::g_bwd_trace, sizeof(long long) * n) == cudaSuccess ? 0 : 3;
}
#endif
