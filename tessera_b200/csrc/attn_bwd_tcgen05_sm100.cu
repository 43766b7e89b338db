// Attention backward with tcgen05 MMA and TMEM accumulators: bf16, D = Dv = 128, no bias / window /
// soft-cap, bottom-right causal mask, grouped-query heads. Same mathematics and the same ownership
// (one CTA per block of gradient rows, fixed summation order, no atomics) as the general CUDA-core
// kernels in attn_bwd_sm100.cu; inputs are the forward's row log-sum-exps (base 2) and
// delta = dO . O (delta_kernel below). The entry points at the end of the file run the forward
// recompute (or take a kept forward state), delta, then the two kernels.
//
// dkv5_kernel: one CTA per 128 keys of one KV head. K and V stay in shared memory; the Q and dO
// tiles (128 query rows) of every query head of the group stream through a two-deep TMA ring.
// Per tile the MMA warp forms the TRANSPOSED products S^T = K Q^T and dP^T = V dO^T into TMEM
// (keys on the 128 lanes, query rows along the columns), two groups of four softmax warps
// (thread = key; group g owns query columns 64 g .. 64 g + 63 and packs them in place, so neither
// group writes a column the other still reads) turn them into bf16 P^T and dS^T, and the MMA warp
// accumulates dV += P^T dO and dK += dS^T Q with the A operand read straight from TMEM. TMEM: S^T | dP^T | dV | dK, 128 fp32
// columns each, all four products at full width (a 128 x 64 shared-shared MMA is bound by operand
// delivery, measured). The overlap comes from handing the two score buffers over separately:
//   softmax:  P^T(t) from S^T(t) (kept packed in registers too) | dS^T(t) from dP^T(t) and P^T(t) | P^T(t+1) ...
//   tensor :  dV += P^T(t) dO(t), then S^T(t+1) over the freed buffer | dK += dS^T(t) Q(t), then dP^T(t+1)
// so the conversion of one buffer runs while the tensor core works on the other.
// dq5_kernel: one CTA per 128 query rows of one head. Q and dO stay, K and V stream; S = Q K^T and
// dP = dO V^T; thread = query row, so lse and delta are per-thread scalars. P is only needed in
// registers, so the S buffer is handed back as soon as it has been read (S(t+1) is formed while
// dS(t) = P(t) (dP(t) - delta) is computed), and dQ += dS K. TMEM: S | dP (even tiles) | dQ | dP (odd tiles).
// Its two conversion groups take alternate tiles; K has three shared-memory stages (K(t) is read by
// S(t) and, a tile later, by dQ(t)), V two, released straight after dP.
// Both kernels: warps 0-7 conversion + epilogue (TMEM lane = 32 * (warp & 3) + lane), warp 8 MMA
// issuer and TMEM owner, warp 9 TMA producer. Every wait is bounded (error word + abort flag), as in
// the forward kernel.
#include <cuda_bf16.h>

#include <cmath>

#include "../../include/tessera_sm100.h"
#include "device_ctx.h"
#include "sm100_ptx.cuh"

namespace tsb {
namespace attn_prefill {
int launch_with_lse(const void* Q, const void* K, const void* V, void* O, float* lse2, int B, int H,
                    int Hkv, int Sq, int Sk, int Dh, float scale, int causal, cudaStream_t st);
}
namespace attn_bwd5 {

constexpr int D = 128;
constexpr int BLK = 128;
constexpr int TILE_BYTES = 128 * 128 * 2;
constexpr int HALF_BYTES = TILE_BYTES / 2;
constexpr int SMEM_BAR_OFF = 6 * TILE_BYTES;               // six 32 KB tiles
constexpr int SMEM_STAT_OFF = SMEM_BAR_OFF + 256;           // lse[2][128], delta[2][128] (dkv only)
constexpr int SMEM_BYTES = SMEM_STAT_OFF + 4 * BLK * 4;
constexpr int SMEM_ALLOC = SMEM_BYTES + 1024;
// dq5_kernel: Q, dO, three K stages, two V stages (seven 32 KB tiles), then barriers
constexpr int DQ_K_STAGES = 3;
constexpr int DQ_BAR_OFF = 7 * TILE_BYTES;
constexpr int DQ_SMEM_ALLOC = DQ_BAR_OFF + 256 + 1024;
static_assert(DQ_SMEM_ALLOC <= 227 * 1024, "dq5_kernel shared memory");
constexpr int THREADS = 320;       // dkv5_kernel: two conversion groups (query columns 0-63 / 64-127), the MMA warp, the TMA warp
constexpr int THREADS_DQ = 320;    // dq5_kernel: two conversion groups (even / odd tiles), the MMA warp, the TMA warp

struct Params {
  int B, Hq, Hkv, Sq, Sk;
  int causal, shift;
  float scale, scale_log2;
  const float* lse2;
  const float* delta;
  int* err;
};


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

// [128 rows of A] x [128 rows of B]^T over d = 128, both tiles K-major (two swizzled 64-wide halves)
__device__ __forceinline__ void issue_rows_x_rows(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo,
                                                  uint32_t desc_hi, uint32_t idesc) {
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    const uint32_t off = ((ks >> 2) * HALF_BYTES + (ks & 3) * 32) >> 4;
    umma_f16_ss_parts(d_tmem, a_lo + off, desc_hi, b_lo + off, desc_hi, idesc, ks > 0 ? 1u : 0u);
  }
}
// d_tmem[128 x 128 d] (+)= A (bf16 in TMEM, 128 lanes x 128 contraction) . B (smem tile whose 128
// rows are the contraction and whose 128 d are contiguous: MN-major, halves HALF_BYTES apart)
// kSplitA: the packed A operand lies in two 32-column pieces, k 0-63 at a_tmem and k 64-127 at
// a_tmem + 64 (each conversion group packs its 64 fp32 columns in place).
template <bool kSplitA = false>
__device__ __forceinline__ void issue_tmem_x_tile(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo,
                                                  uint32_t desc_hi, uint32_t idesc, bool accumulate) {
#pragma unroll
  for (int ks = 0; ks < BLK / 16; ++ks)
    umma_f16_ts_parts(d_tmem, a_tmem + 8u * ks + ((kSplitA && ks >= BLK / 32) ? 32u : 0u), b_lo + ((ks * 2048) >> 4),
                      desc_hi, idesc, (accumulate || ks > 0) ? 1u : 0u);
}
__device__ __forceinline__ uint64_t pack2f(float lo, float hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(__float_as_uint(lo)), "r"(__float_as_uint(hi)));
  return d;
}
__device__ __forceinline__ void unpack2f(uint64_t v, float& lo, float& hi) {
  uint32_t a, b2;
  asm("mov.b64 {%0, %1}, %2;" : "=r"(a), "=r"(b2) : "l"(v));
  lo = __uint_as_float(a);
  hi = __uint_as_float(b2);
}
// 2^x for a pair on the FMA pipe (the special-function pipe, 4 lanes per cycle and scheduler, bounds the
// P^T conversion of the dK/dV kernel): round x to an integer n with the 1.5 * 2^23 trick, a cubic for
// 2^f on f = x - n in [-0.5, 0.5] (relative error 7.5e-5, a thirtieth of the bf16 rounding that follows),
// then n added into the exponent field. x is clamped at -125 (2^-125 instead of 0 below that) and is
// expected <= 0 up to rounding, as it is for a log-sum-exp that belongs to the scores.
__device__ __forceinline__ uint64_t ffma2(uint64_t a, uint64_t b2, uint64_t c);
__device__ __forceinline__ void ex2_poly2(float x0, float x1, float& y0, float& y1) {
  const uint64_t one2 = pack2f(1.f, 1.f), mone2 = pack2f(-1.f, -1.f);
  const uint64_t magic2 = pack2f(12582912.f, 12582912.f), nmagic2 = pack2f(-12582912.f, -12582912.f);
  const uint64_t xx = pack2f(fmaxf(x0, -125.f), fmaxf(x1, -125.f));
  const uint64_t t = ffma2(xx, one2, magic2);     // low mantissa bits = n
  const uint64_t n = ffma2(t, one2, nmagic2);
  const uint64_t f = ffma2(n, mone2, xx);
  uint64_t q = ffma2(pack2f(0.0551716648f, 0.0551716648f), f, pack2f(0.2426111251f, 0.2426111251f));
  q = ffma2(q, f, pack2f(0.6932609677f, 0.6932609677f));
  q = ffma2(q, f, pack2f(0.9999280572f, 0.9999280572f));
  float t0, t1, q0, q1;
  unpack2f(t, t0, t1);
  unpack2f(q, q0, q1);
  y0 = __uint_as_float(__float_as_uint(t0) * 0x800000u + __float_as_uint(q0));
  y1 = __uint_as_float(__float_as_uint(t1) * 0x800000u + __float_as_uint(q1));
}
__device__ __forceinline__ uint64_t ffma2(uint64_t a, uint64_t b2, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b2), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t fmul2(uint64_t a, uint64_t b2) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b2));
  return d;
}
__device__ __forceinline__ float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// accumulator columns [32 c_begin, 32 c_end) of 128 (128 lanes at t_acc) * mul -> bf16 -> swizzled tile at obuf
__device__ __forceinline__ void acc_to_smem(uint32_t t_acc, uint32_t obuf, int r, float mul, int c_begin = 0,
                                            int c_end = 4) {
#pragma unroll 1
  for (int c = c_begin; c < c_end; ++c) {
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
  const uint32_t s_full = bars + 8u * 5;     // S^T formed
  const uint32_t dp_full = bars + 8u * 6;    // dP^T formed
  const uint32_t p_full = bars + 8u * 7;     // P^T written over S^T
  const uint32_t ds_full = bars + 8u * 8;    // dS^T written over dP^T
  const uint32_t o_full = bars + 8u * 9;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + SMEM_BAR_OFF + 128);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + SMEM_BAR_OFF + 132);
  float* s_lse = reinterpret_cast<float*>(smem_gen + SMEM_STAT_OFF);   // [2][128]
  float* s_del = s_lse + 2 * BLK;                                      // [2][128]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BLK, hk = blockIdx.y, b = blockIdx.z;
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
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(p_full, 8);    // one arrival per softmax warp
    mbar_init(ds_full, 8);
    mbar_init(o_full, 1);
    fence_mbar_init();
  }
  if (warp == 8) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tdP = tmem_base + 128, tdV = tmem_base + 256, tdK = tmem_base + 384;

  if (warp == 9) {
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
  } else if (warp == 8) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && iters > 0) {
      const uint32_t idesc_ss = make_idesc_f16(true, false, false, BLK, BLK);   // rows x rows over d
      const uint32_t idesc_ts = make_idesc_f16(true, false, true, BLK, D);      // TMEM A, N-major B
      const uint32_t desc_hi = smem_desc_hi(1024);
      const uint32_t k_lo = smem_desc_lo(sK, 16), v_lo = smem_desc_lo(sV, 16);
      const uint32_t q_lo[2] = {smem_desc_lo(sQ, 16), smem_desc_lo(sQ + TILE_BYTES, 16)};
      const uint32_t g_lo[2] = {smem_desc_lo(sdO, 16), smem_desc_lo(sdO + TILE_BYTES, 16)};
      const uint32_t qn_lo[2] = {smem_desc_lo(sQ, HALF_BYTES), smem_desc_lo(sQ + TILE_BYTES, HALF_BYTES)};
      const uint32_t gn_lo[2] = {smem_desc_lo(sdO, HALF_BYTES), smem_desc_lo(sdO + TILE_BYTES, HALF_BYTES)};
      bool ok = mbar_wait(kv_full, 0, abort_flag, p.err, kErrWaitFull, 1000);
      if (ok) ok = mbar_wait(q_full(0), 0, abort_flag, p.err, kErrWaitFull, 0);
      if (ok) {
        tc_fence_after();
        issue_rows_x_rows(tS, k_lo, q_lo[0], desc_hi, idesc_ss);      // S^T(0)  = K Q^T
        umma_commit(s_full);
        issue_rows_x_rows(tdP, v_lo, g_lo[0], desc_hi, idesc_ss);     // dP^T(0) = V dO^T
        umma_commit(dp_full);
      }
      for (int it = 0; it < iters && ok; ++it) {
        const int st = it & 1, nst = st ^ 1;
        const bool more = it + 1 < iters;
        if (!(ok = mbar_wait(p_full, it & 1, abort_flag, p.err, kErrWaitOther, 2000 + it))) break;
        tc_fence_after();
        issue_tmem_x_tile<true>(tdV, tS, gn_lo[st], desc_hi, idesc_ts, it > 0);       // dV += P^T dO
        if (more) {
          // the S^T buffer is free once dV's MMAs (issued just above, executed in order) have read P^T
          if (!(ok = mbar_wait(q_full(nst), ((it + 1) >> 1) & 1, abort_flag, p.err, kErrWaitFull, it + 1))) break;
          tc_fence_after();
          issue_rows_x_rows(tS, k_lo, q_lo[nst], desc_hi, idesc_ss);            // S^T(t+1)
          umma_commit(s_full);
        }
        if (!(ok = mbar_wait(ds_full, it & 1, abort_flag, p.err, kErrWaitOther, 3000 + it))) break;
        tc_fence_after();
        issue_tmem_x_tile<true>(tdK, tdP, qn_lo[st], desc_hi, idesc_ts, it > 0);      // dK += dS^T Q
        umma_commit(q_empty(st));
        if (more) {
          issue_rows_x_rows(tdP, v_lo, g_lo[nst], desc_hi, idesc_ss);           // dP^T(t+1)
          umma_commit(dp_full);
        } else {
          umma_commit(o_full);
        }
      }
    }
  } else {
    // ------- softmax groups: thread = key; group g (warps 4g .. 4g+3) converts query columns [64 g, 64 g + 64)
    // and packs them in place (P^T at columns 64 g .. 64 g + 31 of S^T, dS^T likewise over dP^T), so
    // neither group ever writes a column the other still has to read
    const int g = warp >> 2;
    const int r = (warp & 3) * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int key = n0 + r;
    const bool key_ok = key < p.Sk;
    bool ok = true;
    float lse_n = INFINITY, del_n = 0.f;
    auto fetch_stats = [&](int it) {   // group 0: this thread's COLUMN (query row m0 + r) of tile `it`
      if (g != 0) return;
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
      if (g == 0) {
        s_lse[sl + r] = -lse_n;   // negated: x = s * scale - lse and dp - delta become packed fmas
        s_del[sl + r] = -del_n;
      }
      if (it + 1 < iters) fetch_stats(it + 1);
      asm volatile("bar.sync 1, 256;" ::: "memory");
      const int m0 = m0_of(it);
      // query rows of this tile the key is legal for: m >= key - shift (causal)
      const int m_first = p.causal ? key - p.shift : -0x40000000;
      const bool tile_legal = n0 + BLK <= p.Sk && (!p.causal || m0 >= n0 + BLK - 1 - p.shift);
      const uint64_t scale2 = pack2f(p.scale_log2, p.scale_log2);
      uint32_t pk[32];   // bf16 P^T of this key row and this group's columns, kept for the dS^T phase
      // ---- phase 1: P^T = exp2(scale * S^T - lse), written over S^T; dV's MMAs may start
      if (ok) ok = mbar_wait(s_full, it & 1, abort_flag, p.err, kErrWaitTmemFull, it);
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int c = 2 * g + half;   // 32-column chunk of S^T
          uint32_t sv[32];
          tmem_ld_32x32b_x32(tS + lane_base + 32 * c, sv);
          tmem_ld_wait();
          if (tile_legal) {   // no mask anywhere in this tile (uniform over the CTA)
#pragma unroll
            for (int k = 0; k < 32; k += 2) {
              const uint64_t nl = *reinterpret_cast<const uint64_t*>(s_lse + sl + 32 * c + k);
              float x0, x1;
              unpack2f(ffma2(pack2f(__uint_as_float(sv[k]), __uint_as_float(sv[k + 1])), scale2, nl), x0, x1);
              if (k & 2) {   // every second pair on the FMA pipe
                float y0, y1;
                ex2_poly2(x0, x1, y0, y1);
                pk[16 * half + (k >> 1)] = PACK_PROB(y0, y1);
              } else {
                pk[16 * half + (k >> 1)] = PACK_PROB(ex2(x0), ex2(x1));
              }
            }
          } else {
#pragma unroll
            for (int k = 0; k < 32; k += 2) {
              float pe[2];
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                const int col = 32 * c + k + e;
                const bool legal = key_ok && (m0 + col >= m_first);
                pe[e] = legal ? ex2(__uint_as_float(sv[k + e]) * p.scale_log2 + s_lse[sl + col]) : 0.f;
              }
              pk[16 * half + (k >> 1)] = PACK_PROB(pe[0], pe[1]);
            }
          }
        }
        tmem_st_32x32b_x32(tS + lane_base + 64 * g, pk);   // 64 fp32 columns consumed -> their 32 packed columns
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full);
      }
      // ---- phase 2: dS^T = P^T (dP^T - delta), written over dP^T; dK's MMAs may start
      if (ok) ok = mbar_wait(dp_full, it & 1, abort_flag, p.err, kErrWaitTmemFull, 500 + it);
      if (ok) {
        tc_fence_after();
        {
          uint32_t dk[32];
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int c = 2 * g + half;
            uint32_t dpv[32];
            tmem_ld_32x32b_x32(tdP + lane_base + 32 * c, dpv);
            tmem_ld_wait();
#pragma unroll
            for (int k = 0; k < 32; k += 2) {
              const uint32_t pw = pk[16 * half + (k >> 1)];
              const uint64_t nd = *reinterpret_cast<const uint64_t*>(s_del + sl + 32 * c + k);
              const uint64_t pp = pack2f(bf16lo(pw), bf16hi(pw));
              // p * dp + p * (-delta)
              float d0, d1;
              unpack2f(ffma2(pp, pack2f(__uint_as_float(dpv[k]), __uint_as_float(dpv[k + 1])), fmul2(pp, nd)), d0, d1);
              dk[16 * half + (k >> 1)] = PACK_PROB(d0, d1);
            }
          }
          tmem_st_32x32b_x32(tdP + lane_base + 64 * g, dk);
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(ds_full);
      }
    }
    // ---- epilogue: dV, scale * dK -> bf16 -> swizzled smem (the Q ring) -> TMA store
    if (iters > 0) {
      if (ok) ok = mbar_wait(o_full, 0, abort_flag, p.err, kErrWaitTmemFull, 9000);
      tc_fence_after();
      if (g == 0) acc_to_smem(tdV + lane_base, sQ, r, 1.0f);                  // group 0 stores dV,
      else acc_to_smem(tdK + lane_base, sQ + TILE_BYTES, r, p.scale);         // group 1 dK
    } else {
      zeros_to_smem(sQ + g * TILE_BYTES, r);
    }
    fence_proxy_async_smem();
    asm volatile("bar.sync %0, 128;" ::"r"(2 + g) : "memory");
    if (r == 0 && ok) {
      const CUtensorMap* tmo = g == 0 ? &tmdV : &tmdK;
      tma_store_4d(tmo, sQ + g * TILE_BYTES, 0, n0, hk, b);
      tma_store_4d(tmo, sQ + g * TILE_BYTES + HALF_BYTES, 64, n0, hk, b);
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
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

__global__ void __launch_bounds__(THREADS_DQ, 1)
dq5_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
           const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
           const __grid_constant__ CUtensorMap tmdQ, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sQ = smem_base, sdO = smem_base + TILE_BYTES;
  const uint32_t sK = smem_base + 2 * TILE_BYTES, sV = smem_base + (2 + DQ_K_STAGES) * TILE_BYTES;
  const uint32_t bars = smem_base + DQ_BAR_OFF;
  const uint32_t q_full = bars;
  // K(t) is read by S(t) and, a whole tile later, by dQ(t); its buffer comes back only when dQ(t) has
  // run, and K(t+2) is wanted right then: three K stages keep that load off the critical path.
  // V(t) is read by dP(t) alone and released straight after it, so two stages are enough.
  auto k_full = [&](int s) { return bars + 8u * (1 + s); };
  auto k_empty = [&](int s) { return bars + 8u * (4 + s); };
  auto v_full = [&](int s) { return bars + 8u * (7 + s); };
  auto v_empty = [&](int s) { return bars + 8u * (9 + s); };
  // Tiles alternate between two conversion groups, so every hand-off barrier exists once per tile
  // parity: each completes every second tile and a commit for tile t+1 can never run a phase ahead
  // of a warp still waiting for tile t.
  auto s_full = [&](int st) { return bars + 8u * (11 + st); };     // S formed
  // dP formed, one barrier per dP buffer (each completes every second tile, so a commit for tile t+1
  // can never run a phase ahead of a warp still waiting for tile t)
  auto dp_full = [&](int st) { return bars + 8u * (13 + st); };
  auto s_free = [&](int st) { return bars + 8u * (15 + st); };     // S read into registers: may be overwritten
  auto ds_full = [&](int st) { return bars + 8u * (17 + st); };    // dS written over dP
  const uint32_t o_full = bars + 8u * 19;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + DQ_BAR_OFF + 192);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + DQ_BAR_OFF + 196);

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
    for (int s = 0; s < DQ_K_STAGES; ++s) {
      mbar_init(k_full(s), 1);
      mbar_init(k_empty(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(v_full(s), 1);
      mbar_init(v_empty(s), 1);
    }
    for (int st = 0; st < 2; ++st) {
      mbar_init(s_full(st), 1);
      mbar_init(dp_full(st), 1);
      mbar_init(s_free(st), 4);    // one arrival per warp of the group that owns the tile
      mbar_init(ds_full(st), 4);
    }
    mbar_init(o_full, 1);
    fence_mbar_init();
  }
  if (warp == 8) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // TMEM: S | dP (even tiles) | dQ | dP (odd tiles): dP has two buffers, so dP(t+1) never waits for dS(t)
  const uint32_t tS = tmem_base, tdQ = tmem_base + 256;
  auto tdP = [&](int st) { return tmem_base + static_cast<uint32_t>(st ? 384 : 128); };

  if (warp == 9) {
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
        const int ks = it % DQ_K_STAGES, vs = it & 1;
        const uint32_t kph = (it / DQ_K_STAGES) & 1, vph = (it >> 1) & 1;
        if (!mbar_wait(k_empty(ks), kph ^ 1u, abort_flag, p.err, kErrWaitEmpty, it)) break;
        mbar_arrive_expect_tx(k_full(ks), TILE_BYTES);
        tma_load_4d(sK + ks * TILE_BYTES, &tmK, k_full(ks), 0, it * BLK, hk, b);
        tma_load_4d(sK + ks * TILE_BYTES + HALF_BYTES, &tmK, k_full(ks), 64, it * BLK, hk, b);
        if (!mbar_wait(v_empty(vs), vph ^ 1u, abort_flag, p.err, kErrWaitEmpty, 100000 + it)) break;
        mbar_arrive_expect_tx(v_full(vs), TILE_BYTES);
        tma_load_4d(sV + vs * TILE_BYTES, &tmV, v_full(vs), 0, it * BLK, hk, b);
        tma_load_4d(sV + vs * TILE_BYTES + HALF_BYTES, &tmV, v_full(vs), 64, it * BLK, hk, b);
      }
    }
  } else if (warp == 8) {
    if (lane == 0 && iters > 0) {
      const uint32_t idesc_ss = make_idesc_f16(true, false, false, BLK, BLK);
      const uint32_t idesc_ts = make_idesc_f16(true, false, true, BLK, D);
      const uint32_t desc_hi = smem_desc_hi(1024);
      const uint32_t q_lo = smem_desc_lo(sQ, 16), g_lo = smem_desc_lo(sdO, 16);
      const uint32_t v_lo[2] = {smem_desc_lo(sV, 16), smem_desc_lo(sV + TILE_BYTES, 16)};
      bool ok = mbar_wait(q_full, 0, abort_flag, p.err, kErrWaitFull, 1000);
      if (ok) ok = mbar_wait(k_full(0), 0, abort_flag, p.err, kErrWaitFull, 0);
      if (ok) {
        tc_fence_after();
        issue_rows_x_rows(tS, q_lo, smem_desc_lo(sK, 16), desc_hi, idesc_ss);   // S(0)  = Q K^T
        umma_commit(s_full(0));
      }
      if (ok) ok = mbar_wait(v_full(0), 0, abort_flag, p.err, kErrWaitFull, 100000);
      if (ok) {
        tc_fence_after();
        issue_rows_x_rows(tdP(0), g_lo, v_lo[0], desc_hi, idesc_ss);    // dP(0) = dO V^T
        umma_commit(v_empty(0));
        umma_commit(dp_full(0));
      }
      for (int it = 0; it < iters && ok; ++it) {
        const int st = it & 1, nst = st ^ 1;
        if (it + 1 < iters) {
          // the softmax warps hold P(t) in registers: S(t+1) and dP(t+1) are formed while they work on dS(t)
          if (!(ok = mbar_wait(s_free(st), (it >> 1) & 1, abort_flag, p.err, kErrWaitOther, 2000 + it))) break;
          const int ksn = (it + 1) % DQ_K_STAGES;
          if (!(ok = mbar_wait(k_full(ksn), ((it + 1) / DQ_K_STAGES) & 1, abort_flag, p.err, kErrWaitFull, it + 1))) break;
          tc_fence_after();
          issue_rows_x_rows(tS, q_lo, smem_desc_lo(sK + ksn * TILE_BYTES, 16), desc_hi, idesc_ss);
          umma_commit(s_full(nst));
          if (!(ok = mbar_wait(v_full(nst), ((it + 1) >> 1) & 1, abort_flag, p.err, kErrWaitFull, 100001 + it))) break;
          tc_fence_after();
          issue_rows_x_rows(tdP(nst), g_lo, v_lo[nst], desc_hi, idesc_ss);
          umma_commit(v_empty(nst));
          umma_commit(dp_full(nst));
        }
        if (!(ok = mbar_wait(ds_full(st), (it >> 1) & 1, abort_flag, p.err, kErrWaitOther, 3000 + it))) break;
        tc_fence_after();
        const int ks = it % DQ_K_STAGES;
        issue_tmem_x_tile(tdQ, tdP(st), smem_desc_lo(sK + ks * TILE_BYTES, HALF_BYTES), desc_hi, idesc_ts,
                          it > 0);   // dQ += dS K
        umma_commit(k_empty(ks));
        if (it + 1 == iters) umma_commit(o_full);
      }
    }
  } else {
    // conversion groups: thread = query row; group g (warps 4g .. 4g+3) converts the tiles of parity g
    const int g = warp >> 2;
    const int r = (warp & 3) * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int m = m0 + r;
    const long long row = (static_cast<long long>(b) * p.Hq + hq) * p.Sq + m;
    const float lse = m < p.Sq ? p.lse2[row] : INFINITY;
    const float del = m < p.Sq ? p.delta[row] : 0.f;
    const int n_last = p.causal ? min(m + p.shift, p.Sk - 1) : p.Sk - 1;   // last legal key
    const uint64_t scale2 = pack2f(p.scale_log2, p.scale_log2);
    const uint64_t nlse2 = pack2f(-lse, -lse), ndel2 = pack2f(-del, -del);
    bool ok = true;
    for (int it = g; it < iters && ok; it += 2) {
      const int nb = it * BLK;
      const bool tile_legal = nb + BLK - 1 <= (p.causal ? min(m0 + p.shift, p.Sk - 1) : p.Sk - 1);
      uint32_t pk[64];   // bf16 P of this query row
      // ---- phase 1: P = exp2(scale * S - lse) into registers, then the S buffer is handed back
      if (!(ok = mbar_wait(s_full(g), (it >> 1) & 1, abort_flag, p.err, kErrWaitTmemFull, it))) break;
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t sv[32];
        tmem_ld_32x32b_x32(tS + lane_base + 32 * c, sv);
        tmem_ld_wait();
        if (c == 3) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(s_free(g));
        }
        if (tile_legal) {   // no mask anywhere in this tile (uniform over the CTA)
#pragma unroll
          for (int k = 0; k < 32; k += 2) {
            float x0, x1;
            unpack2f(ffma2(pack2f(__uint_as_float(sv[k]), __uint_as_float(sv[k + 1])), scale2, nlse2), x0, x1);
            pk[16 * c + (k >> 1)] = PACK_PROB(ex2(x0), ex2(x1));
          }
        } else {
#pragma unroll
          for (int k = 0; k < 32; k += 2) {
            float pe[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const bool legal = nb + 32 * c + k + e <= n_last;
              pe[e] = legal ? ex2(__uint_as_float(sv[k + e]) * p.scale_log2 - lse) : 0.f;
            }
            pk[16 * c + (k >> 1)] = PACK_PROB(pe[0], pe[1]);
          }
        }
      }
      // ---- phase 2: dS = P (dP - delta), written over dP; dQ's MMAs may start
      if (!(ok = mbar_wait(dp_full(g), (it >> 1) & 1, abort_flag, p.err, kErrWaitTmemFull, 500 + it))) break;
      tc_fence_after();
      const uint32_t t_dp = tdP(g) + lane_base;
#pragma unroll
      for (int cp = 0; cp < 2; ++cp) {
        uint32_t dk[32];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int c = 2 * cp + half;
          uint32_t dpv[32];
          tmem_ld_32x32b_x32(t_dp + 32 * c, dpv);
          tmem_ld_wait();
#pragma unroll
          for (int k = 0; k < 32; k += 2) {
            const uint32_t pw = pk[16 * c + (k >> 1)];
            const uint64_t pp = pack2f(bf16lo(pw), bf16hi(pw));
            float d0, d1;   // p * dp + p * (-delta)
            unpack2f(ffma2(pp, pack2f(__uint_as_float(dpv[k]), __uint_as_float(dpv[k + 1])), fmul2(pp, ndel2)), d0, d1);
            dk[16 * half + (k >> 1)] = PACK_PROB(d0, d1);
          }
        }
        tmem_st_32x32b_x32(t_dp + 32 * cp, dk);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full(g));
    }
    if (iters > 0) {
      if (ok) ok = mbar_wait(o_full, 0, abort_flag, p.err, kErrWaitTmemFull, 9000);
      tc_fence_after();
      acc_to_smem(tdQ + lane_base, sK, r, p.scale, 2 * g, 2 * g + 2);   // d columns [64 g, 64 g + 64)
    } else {
      for (int ch = 0; ch < 8; ++ch)
        asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(sK + g * HALF_BYTES + swz128(r, ch)), "r"(0) : "memory");
    }
    fence_proxy_async_smem();
    asm volatile("bar.sync %0, 128;" ::"r"(1 + g) : "memory");
    if (r == 0 && ok) {
      tma_store_4d(&tmdQ, sK + g * HALF_BYTES, 64 * g, m0, hq, b);
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
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// dO, Q, dQ [B,Hq,Sq,128]; K, V, dK, dV [B,Hkv,Sk,128] bf16 dense; lse2, delta [B,Hq,Sq] fp32.
// delta[row] = sum_d dO[row, d] O[row, d], one warp per row.
__global__ void delta_kernel(const __nv_bfloat16* __restrict__ dO, const __nv_bfloat16* __restrict__ O,
                             float* __restrict__ delta, long long rows) {
  const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const uint2 a = *reinterpret_cast<const uint2*>(dO + row * D + lane * 4);
  const uint2 b = *reinterpret_cast<const uint2*>(O + row * D + lane * 4);
  const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float2 x = __bfloat1622float2(pa[i]), y = __bfloat1622float2(pb[i]);
    s += x.x * y.x + x.y * y.y;
  }
#pragma unroll
  for (int sh = 16; sh; sh >>= 1) s += __shfl_xor_sync(0xffffffffu, s, sh);
  if (lane == 0) delta[row] = s;
}

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
  TSB_CUDA_OK(cudaFuncSetAttribute(dq5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DQ_SMEM_ALLOC));
  TSB_CUDA_OK(cudaFuncSetAttribute(dkv5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_ALLOC));
  dim3 g1((Sq + BLK - 1) / BLK, Hq, B);
  dq5_kernel<<<g1, THREADS_DQ, DQ_SMEM_ALLOC, st>>>(tQ, tdO, tK, tV, tdQ, p);
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

using namespace tsb;

extern "C" {

// Workspace of the tensor-core backward: O (bf16), log-sum-exp and delta (fp32) per query row.
size_t tessera_sm100_flash_attn_bwd_bf16_workspace_bytes(int B, int Hq, int Sq) {
  if (B <= 0 || Hq <= 0 || Sq <= 0) return 0;
  const size_t rows = static_cast<size_t>(B) * Hq * Sq;
  return ((rows * attn_bwd5::D * 2 + 255) & ~size_t(255)) + 2 * ((rows * 4 + 255) & ~size_t(255));
}

// dO, Q, dQ [B,Hq,Sq,128]; K, V, dK, dV [B,Hkv,Sk,128], bf16, dense. causal uses the bottom-right
// alignment of tessera.ops.flash_attn (identical to the lane's mask when Sq >= Sk).
static int bwd_bf16_from_state(const void* dO, const void* Q, const void* K, const void* V, const void* O,
                               const float* lse2, float* delta, void* dQ, void* dK, void* dV, int B, int Hq,
                               int Hkv, int Sq, int Sk, float scale, int causal, cudaStream_t st);

int tessera_sm100_flash_attn_bwd_bf16_device(const void* dO, const void* Q, const void* K, const void* V,
                                             void* dQ, void* dK, void* dV, int B, int Hq, int Hkv, int Sq,
                                             int Sk, float scale, int causal, void* workspace,
                                             void* stream) {
  if (!dO || !Q || !K || !V || !dQ || !dK || !dV || !workspace || B <= 0 || Hq <= 0 || Hkv <= 0 ||
      Hq % Hkv || Sq <= 0 || Sk <= 0 || !(scale > 0.f)) {
    set_last_error("flash_attn_bwd_bf16: null pointer, non-positive size or scale, or Hq not divisible by Hkv");
    return kBadArg;
  }
  if (int rc = ensure_device()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t rows = static_cast<size_t>(B) * Hq * Sq;
  char* ws = static_cast<char*>(workspace);
  void* O = ws;
  float* lse2 = reinterpret_cast<float*>(ws + ((rows * attn_bwd5::D * 2 + 255) & ~size_t(255)));
  float* delta = reinterpret_cast<float*>(reinterpret_cast<char*>(lse2) + ((rows * 4 + 255) & ~size_t(255)));
  if (int rc = attn_prefill::launch_with_lse(Q, K, V, O, lse2, B, Hq, Hkv, Sq, Sk, attn_bwd5::D, scale,
                                             causal, st))
    return rc;
  return bwd_bf16_from_state(dO, Q, K, V, O, lse2, delta, dQ, dK, dV, B, Hq, Hkv, Sq, Sk, scale, causal, st);
}

// The backward of a training step that kept the forward's output and row log-sum-exps
// (tessera_sm100_flash_attn_fwd_lse_device): no forward recompute. delta_scratch: B*Hq*Sq floats.
int tessera_sm100_flash_attn_bwd_bf16_saved_device(const void* dO, const void* Q, const void* K,
                                                   const void* V, const void* O, const float* lse2,
                                                   void* dQ, void* dK, void* dV, int B, int Hq, int Hkv,
                                                   int Sq, int Sk, float scale, int causal,
                                                   float* delta_scratch, void* stream) {
  if (!dO || !Q || !K || !V || !O || !lse2 || !dQ || !dK || !dV || !delta_scratch || B <= 0 || Hq <= 0 ||
      Hkv <= 0 || Hq % Hkv || Sq <= 0 || Sk <= 0 || !(scale > 0.f)) {
    set_last_error("flash_attn_bwd_bf16_saved: null pointer, non-positive size or scale, or Hq not divisible by Hkv");
    return kBadArg;
  }
  if (int rc = ensure_device()) return rc;
  return bwd_bf16_from_state(dO, Q, K, V, O, lse2, delta_scratch, dQ, dK, dV, B, Hq, Hkv, Sq, Sk, scale, causal,
                             static_cast<cudaStream_t>(stream));
}

static int bwd_bf16_from_state(const void* dO, const void* Q, const void* K, const void* V, const void* O,
                               const float* lse2, float* delta, void* dQ, void* dK, void* dV, int B, int Hq,
                               int Hkv, int Sq, int Sk, float scale, int causal, cudaStream_t st) {
  const size_t rows = static_cast<size_t>(B) * Hq * Sq;
  attn_bwd5::delta_kernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(dO), static_cast<const __nv_bfloat16*>(O), delta,
      static_cast<long long>(rows));
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  return attn_bwd5::launch(dO, Q, K, V, dQ, dK, dV, lse2, delta, B, Hq, Hkv, Sq, Sk, scale, causal, st);
}

int tessera_sm100_flash_attn_fwd_lse_device(const void* Q, const void* K, const void* V, void* O,
                                            float* lse2, int B, int Hq, int Hkv, int Sq, int Sk, int D,
                                            float scale, int causal, void* stream) {
  if (!lse2) {
    set_last_error("flash_attn_fwd_lse: lse2 is null");
    return kBadArg;
  }
  if (int rc = ensure_device()) return rc;
  return attn_prefill::launch_with_lse(Q, K, V, O, lse2, B, Hq, Hkv, Sq, Sk, D, scale, causal,
                                       static_cast<cudaStream_t>(stream));
}

}  // extern "C"
