// Flash-attention forward (prefill) for sm_100a with tcgen05 MMA and TMEM accumulators.
//
//   O[b,h] = softmax(scale * Q[b,h] K[b,hk]^T + causal mask) V[b,hk],   hk = h / (H/Hkv)
//
// Semantics of tessera.ops.flash_attn (python/tessera/__init__.py:1304-1356): the causal mask is
// bottom-right aligned (key j is visible to query i when j <= i + max(Sk - Sq, 0)); softmax
// statistics are fp32. Head dimension 128, bf16 in / bf16 out.
//
// One CTA owns 256 query rows of one (b, h) as two 128-row tiles and walks the KV sequence in
// blocks of 64. Eleven warps:
//   warps 0-3  softmax group for tile 0   (thread r owns row r: TMEM lane r)
//   warps 4-7  softmax group for tile 1
//   warp  8    MMA issuer for tile 0 (one lane) + TMEM owner
//   warp  9    TMA producer (one lane)
//   warp  10   MMA issuer for tile 1 (one lane)
// TMEM (512 columns): S0a S0b | S1a S1b | O0 | O1. Every tile has TWO 64-column score buffers, so
// the MMA warp forms S(j+1) while the tile's softmax group works on S(j): per tile the issue order
// is S(0) S(1), then PV(j) S(j+2) for j = 0, 1, ..., and a softmax group goes from one block
// straight to the next without waiting for a P.V -> Q.K^T round trip. P (bf16) overwrites the first
// 32 columns of its S buffer and is the A operand of the P.V MMA straight from TMEM. The running
// maximum is only raised (and O rescaled in TMEM) when it grows by more than 2^8, which keeps exp2
// arguments bounded while making the rescale rare; the final O / l normalisation is exact
// regardless.
#include <cuda_bf16.h>

#include <algorithm>
#include <cmath>

#include "../../include/tessera_sm100.h"
#include "device_ctx.h"
#include "sm100_ptx.cuh"

namespace tsb {
namespace attn_prefill {

constexpr int D = 128;
constexpr int BQ = 128;    // rows per Q tile
constexpr int BKV = 64;    // KV positions per block
constexpr int TILE_BYTES = 128 * 128 * 2;  // a 128 x 128 bf16 Q (or O) tile = two 16 KB swizzled blocks
constexpr int HALF_BYTES = TILE_BYTES / 2;
constexpr int KV_BYTES = BKV * 128 * 2;    // a 64 x 128 bf16 K or V block = two 8 KB swizzled blocks
constexpr int KV_HALF = KV_BYTES / 2;
constexpr int STAGES = 4;   // ring slots; slot j % 4 holds V(j) and K(j + 2)
constexpr int SMEM_Q_OFF = 0;                       // Q0, Q1 (reused for the O store)
constexpr int SMEM_K_OFF = 2 * TILE_BYTES;
constexpr int SMEM_V_OFF = SMEM_K_OFF + STAGES * KV_BYTES;
constexpr int SMEM_BAR_OFF = SMEM_V_OFF + STAGES * KV_BYTES;
constexpr int SMEM_BYTES = SMEM_BAR_OFF + 256;
constexpr int SMEM_ALLOC = SMEM_BYTES + 1024;
constexpr int THREADS = 352;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

struct Params {
  int B, H, Hkv, Sq, Sk;
  int causal;
  float scale_log2;
  int* err;
  float* lse2;   // optional [B, H, Sq]: log2-sum-exp2 of scale_log2 * s per row (the backward's input)
};


__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Packed two-wide fp32 arithmetic and the three-input maximum of sm_100.
__device__ __forceinline__ uint64_t pack_u32x2(uint32_t lo, uint32_t hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
  return d;
}
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  return pack_u32x2(__float_as_uint(lo), __float_as_uint(hi));
}
__device__ __forceinline__ float lo_f32(uint64_t v) { return __uint_as_float(static_cast<uint32_t>(v)); }
__device__ __forceinline__ float hi_f32(uint64_t v) { return __uint_as_float(static_cast<uint32_t>(v >> 32)); }
__device__ __forceinline__ uint64_t fadd2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// Volatile forms: the compiler keeps volatile asm statements in program order, which is how the
// softmax loop pins its interleaving.
__device__ __forceinline__ uint64_t ffma2_v(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm volatile("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t fadd2_v(uint64_t a, uint64_t b) {
  uint64_t d;
  asm volatile("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float ex2_v(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// {hi, lo} -> packed bf16x2 (hi in the upper half). cvt.rn.bf16x2.f32 shares the special-function
// unit with ex2 (measured: about half an ex2 per convert), so the conversion is a fifth of the
// exponent phase's time on that unit; packing with integer adds and a byte permute instead takes the
// unit's load down but lengthens the in-order loop, and measured 4 % slower in this kernel.
__device__ __forceinline__ uint32_t cvt_bf16x2_v(float hi, float lo) {
  uint32_t d;
  asm volatile("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// mbarrier.arrive that cannot be scheduled before `dep` has been produced: the barrier address is
// computed from the value's sign bit (dep is a probability, so the bit is 0 -- which the assembler
// cannot know).
__device__ __forceinline__ void mbar_arrive_after(uint32_t bar, float dep) {
  mbar_arrive(bar + ((__float_as_uint(dep) >> 31) << 3));
}

__global__ void __launch_bounds__(THREADS, 1)
prefill_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
               const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
               const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sQ = smem_base + SMEM_Q_OFF;
  const uint32_t sK = smem_base + SMEM_K_OFF;
  const uint32_t sV = smem_base + SMEM_V_OFF;
  const uint32_t bars = smem_base + SMEM_BAR_OFF;
  // barriers: q_full[2] k01_full[2] kv_full[4] kv_empty[4] s_full[2][2] p_full[2][2] x_done[2][2] o_full[2]
  // Ring slot j % 4 holds V(j) and K(j + 2): they are loaded by one producer step, consumed by one
  // MMA iteration and freed by one commit. K(0) and K(1) have barriers of their own.
  auto q_full = [&](int i) { return bars + 8u * (0 + i); };
  auto k01_full = [&](int s) { return bars + 8u * (2 + s); };
  auto kv_full = [&](int s) { return bars + 8u * (4 + s); };
  auto kv_empty = [&](int s) { return bars + 8u * (4 + STAGES + s); };
  constexpr int kBarS = 4 + 2 * STAGES;
  auto s_full = [&](int i, int buf) { return bars + 8u * (kBarS + i * 2 + buf); };
  auto p_full = [&](int i, int buf) { return bars + 8u * (kBarS + 4 + i * 2 + buf); };
  auto x_done = [&](int i, int buf) { return bars + 8u * (kBarS + 8 + i * 2 + buf); };
  auto o_full = [&](int i) { return bars + 8u * (kBarS + 12 + i); };
  static_assert((kBarS + 14) * 8 <= 240, "barrier block overruns its slot");
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + SMEM_BAR_OFF + 240);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + SMEM_BAR_OFF + 244);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int qpair = gridDim.x - 1 - blockIdx.x;  // heaviest (latest) query rows first
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int hk = h / (p.H / p.Hkv);
  const int q_base = qpair * 2 * BQ;
  const int shift = p.causal ? max(p.Sk - p.Sq, 0) : 0;
  const int nblk_total = (p.Sk + BKV - 1) / BKV;
  int nblk[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int qi0 = q_base + i * BQ;
    if (qi0 >= p.Sq) {
      nblk[i] = 0;
    } else if (p.causal) {
      const int last_row = min(qi0 + BQ - 1, p.Sq - 1);
      nblk[i] = min(nblk_total, (last_row + shift) / BKV + 1);
    } else {
      nblk[i] = nblk_total;
    }
  }
  const int n_iter = max(nblk[0], nblk[1]);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < 2; ++i) {
      mbar_init(q_full(i), 1);
      mbar_init(o_full(i), 1);
      mbar_init(k01_full(i), 1);
      for (int buf = 0; buf < 2; ++buf) {
        mbar_init(s_full(i, buf), 1);
        mbar_init(p_full(i, buf), 4);  // one arrival per softmax warp
        mbar_init(x_done(i, buf), 4);
      }
    }
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(kv_full(s), 1);
      mbar_init(kv_empty(s), 2);  // one arrival per MMA issuer
    }
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
  // TMEM columns
  auto tS = [&](int i, int buf) { return tmem_base + static_cast<uint32_t>(i * 128 + buf * 64); };
  auto tO = [&](int i) { return tmem_base + static_cast<uint32_t>(256 + i * 128); };

  if (warp == 9) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      for (int i = 0; i < 2; ++i) {
        if (nblk[i] == 0) continue;
        mbar_arrive_expect_tx(q_full(i), TILE_BYTES);
        tma_load_4d(sQ + i * TILE_BYTES, &tmQ, q_full(i), 0, q_base + i * BQ, h, b);
        tma_load_4d(sQ + i * TILE_BYTES + HALF_BYTES, &tmQ, q_full(i), 64, q_base + i * BQ, h, b);
      }
      // K runs two blocks ahead of V: S(j+2) is formed in the iteration that consumes V(j).
      for (int jj = 0; jj < 2 && jj < n_iter; ++jj) {
        mbar_arrive_expect_tx(k01_full(jj), KV_BYTES);
        tma_load_4d(sK + jj * KV_BYTES, &tmK, k01_full(jj), 0, jj * BKV, hk, b);
        tma_load_4d(sK + jj * KV_BYTES + KV_HALF, &tmK, k01_full(jj), 64, jj * BKV, hk, b);
      }
      for (int j = 0; j < n_iter; ++j) {
        const int st = j % STAGES;
        // Slot st was last freed by iteration j - 4; for slots 2 and 3 the first freeing is the
        // prologue's (K(0), K(1) sit in the K buffers of those slots' successors).
        const int idx = st >= 2 ? j / STAGES : j / STAGES - 1;
        if (j >= 2 && idx >= 0 &&
            !mbar_wait(kv_empty(st), static_cast<uint32_t>(idx & 1), abort_flag, p.err, kErrWaitEmpty, j))
          break;
        const bool with_k = j + 2 < n_iter;
        mbar_arrive_expect_tx(kv_full(st), with_k ? 2 * KV_BYTES : KV_BYTES);
        tma_load_4d(sV + st * KV_BYTES, &tmV, kv_full(st), 0, j * BKV, hk, b);
        tma_load_4d(sV + st * KV_BYTES + KV_HALF, &tmV, kv_full(st), 64, j * BKV, hk, b);
        if (with_k) {
          const int kst = (j + 2) % STAGES;
          tma_load_4d(sK + kst * KV_BYTES, &tmK, kv_full(st), 0, (j + 2) * BKV, hk, b);
          tma_load_4d(sK + kst * KV_BYTES + KV_HALF, &tmK, kv_full(st), 64, (j + 2) * BKV, hk, b);
        }
      }
    }
  } else if (warp == 8 || warp == 10) {
    // ------------------------------------------------------------------ MMA issuers
    // One issuing thread per tile. The tensor pipe takes MMAs only a few ahead of what it is
    // executing, so whatever an issuer spends between two batches (barrier polls, commits) would
    // be a bubble in the pipe; with two issuers one tile's batch runs while the other tile's
    // thread waits for its P. Both walk every KV block and arrive on the stage barriers (count 2)
    // whether or not their tile still needs the block, which keeps them within a ring of each other.
    if (lane == 0) {
      const int i = warp == 8 ? 0 : 1;
      const uint32_t idesc_s = make_idesc_f16(true, false, false, BQ, BKV);  // Q K^T, both K-major
      const uint32_t idesc_pv = make_idesc_f16(true, false, true, BQ, D);    // P (TMEM) V (N-major)
      // Descriptor words kept in registers: one low word per operand buffer, one shared high
      // word (SBO 1024, 128-byte swizzle). Per MMA only a constant is added to a low word.
      const uint32_t desc_hi = smem_desc_hi(1024);
      const uint32_t q_lo = smem_desc_lo(sQ + i * TILE_BYTES, 16);
      const uint32_t k_lo0 = smem_desc_lo(sK, 16);
      const uint32_t v_lo0 = smem_desc_lo(sV, KV_HALF);
      const uint32_t t_o = tO(i);
      const int nb = nblk[i];
      auto issue_s = [&](int kst, int buf) {
        const uint32_t b_lo = k_lo0 + ((kst * KV_BYTES) >> 4), d = tS(i, buf);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          // 16 elements of d per step: 32 B inside a 128-byte row, next 64-wide block after 4.
          const uint32_t a_off = ((ks >> 2) * HALF_BYTES + (ks & 3) * 32) >> 4;
          const uint32_t b_off = ((ks >> 2) * KV_HALF + (ks & 3) * 32) >> 4;
          umma_f16_ss_parts(d, q_lo + a_off, desc_hi, b_lo + b_off, desc_hi, idesc_s, ks > 0 ? 1u : 0u);
        }
      };
      auto issue_pv = [&](int vst, bool accumulate, int buf) {
        const uint32_t b_lo = v_lo0 + ((vst * KV_BYTES) >> 4), a = tS(i, buf);
#pragma unroll
        for (int ks = 0; ks < BKV / 16; ++ks) {
          // A: P rows in TMEM lanes, 16 bf16 of K per 8 columns. B: V[kv][d], 16 kv rows = 2048 B;
          // the two 64-wide d blocks are KV_HALF apart (the LBO field).
          umma_f16_ts_parts(t_o, a + 8u * ks, b_lo + ((ks * 2048) >> 4), desc_hi, idesc_pv,
                            (accumulate || ks > 0) ? 1u : 0u);
        }
      };
      bool ok = true;
      if (nb > 0) ok = mbar_wait(q_full(i), 0, abort_flag, p.err, kErrWaitFull, 2000 + i);
      for (int jj = 0; jj < 2 && jj < n_iter && ok; ++jj) {
        if (!(ok = mbar_wait(k01_full(jj), 0, abort_flag, p.err, kErrWaitFull, jj))) break;
        tc_fence_after();
        if (jj < nb) {
          issue_s(jj, jj);
          umma_commit(s_full(i, jj));
        }
        umma_commit(kv_empty(2 + jj));
      }
      for (int j = 0; j < n_iter && ok; ++j) {
        const int vst = j % STAGES;
        const uint32_t vph = (j / STAGES) & 1;
        const int j2 = j + 2;
        const int kst = j2 % STAGES;
        const int buf = j & 1;
        if (!(ok = mbar_wait(kv_full(vst), vph, abort_flag, p.err, kErrWaitFull, 3000 + j))) break;
        if (j < nb) {
          if (!(ok = mbar_wait(p_full(i, buf), (j >> 1) & 1, abort_flag, p.err, kErrWaitOther, 4000 + j))) break;
          tc_fence_after();
          issue_pv(vst, j > 0, buf);
          if (j2 < nb) issue_s(kst, buf);
          // Completes when S(j+2) is in the buffer -- and, with or without a next block, when
          // PV(j) has finished, which is what a later rescale of O waits for.
          umma_commit(s_full(i, buf));
          if (j == nb - 1) umma_commit(o_full(i));
        }
        umma_commit(kv_empty(vst));
      }
    }
  } else if (warp < 8) {
    // ------------------------------------------------------------------ softmax groups
    const int i = warp >> 2;                    // tile
    const int r = (warp & 3) * 32 + lane;       // row inside the tile == TMEM lane
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int qi0 = q_base + i * BQ;
    const int row_q = qi0 + r;
    const int kv_limit = p.causal ? min(row_q + shift, p.Sk - 1) : (p.Sk - 1);  // last visible key
    float m_used = -INFINITY;
    float l = 0.f;
    bool ok = true;
    // Every lane waits on the barrier itself: one polling lane per warp followed by a shuffle
    // measured a third slower in this kernel (717 against 1045 TFLOP/s).
    auto warp_wait = [&](uint32_t bar, uint32_t parity, int code, int detail) -> bool {
      return mbar_wait(bar, parity, abort_flag, p.err, code, detail);
    };
    for (int j = 0; j < nblk[i] && ok; ++j) {
      const int buf = j & 1;
      if (!(ok = warp_wait(s_full(i, buf), (j >> 1) & 1, kErrWaitTmemFull, j))) break;
      tc_fence_after();
      const int kv0 = j * BKV;
      const bool need_mask = (kv0 + BKV - 1 > qi0 + shift && p.causal) || (kv0 + BKV > p.Sk);
      const uint32_t t_s = tS(i, buf) + lane_base;
      // One pass over TMEM: the 64-column row of S goes to registers (two loads in flight, one
      // wait); maxima and sums run as independent chains.
      uint32_t s0[32], s1[32];
      tmem_ld_32x32b_x32(t_s, s0);
      tmem_ld_32x32b_x32(t_s + 32, s1);
      tmem_ld_wait();
      if (need_mask) {
        constexpr uint32_t kNegInf = 0xff800000u;
#pragma unroll
        for (int k = 0; k < 32; ++k) {
          if (kv0 + k > kv_limit) s0[k] = kNegInf;
          if (kv0 + 32 + k > kv_limit) s1[k] = kNegInf;
        }
      }
      // Row maximum: 3-input max, eight independent chains.
      float mxa[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) mxa[c] = -INFINITY;
#pragma unroll
      for (int k = 0; k < 32; k += 8) {
        mxa[0] = fmax3(mxa[0], __uint_as_float(s0[k]), __uint_as_float(s0[k + 1]));
        mxa[1] = fmax3(mxa[1], __uint_as_float(s0[k + 2]), __uint_as_float(s0[k + 3]));
        mxa[2] = fmax3(mxa[2], __uint_as_float(s0[k + 4]), __uint_as_float(s0[k + 5]));
        mxa[3] = fmax3(mxa[3], __uint_as_float(s0[k + 6]), __uint_as_float(s0[k + 7]));
        mxa[4] = fmax3(mxa[4], __uint_as_float(s1[k]), __uint_as_float(s1[k + 1]));
        mxa[5] = fmax3(mxa[5], __uint_as_float(s1[k + 2]), __uint_as_float(s1[k + 3]));
        mxa[6] = fmax3(mxa[6], __uint_as_float(s1[k + 4]), __uint_as_float(s1[k + 5]));
        mxa[7] = fmax3(mxa[7], __uint_as_float(s1[k + 6]), __uint_as_float(s1[k + 7]));
      }
      const float mx = fmaxf(fmax3(mxa[0], mxa[1], mxa[2]), fmax3(fmax3(mxa[3], mxa[4], mxa[5]), mxa[6], mxa[7]));
      const float m_new = fmaxf(m_used, mx * p.scale_log2);
      const bool need = m_new > m_used + kRescaleThreshold;
      if (j == 0) {
        m_used = m_new;
      } else if (__any_sync(0xffffffffu, need)) {
        // O may still be the target of PV(j-1). The other score buffer's barrier completes for
        // block j+1 only after PV(j-1) has (its commit follows that MMA), block j+1 or not.
        if (!(ok = warp_wait(s_full(i, buf ^ 1), ((j + 1) >> 1) & 1, kErrWaitTmemFull, 7000 + j))) break;
        tc_fence_after();
        const float alpha = need ? ex2(m_used - m_new) : 1.0f;
        if (need) {
          m_used = m_new;
          l *= alpha;
        }
        const uint32_t t_o = tO(i) + lane_base;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(t_o + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int k = 0; k < 32; ++k) v[k] = __float_as_uint(__uint_as_float(v[k]) * alpha);
          tmem_st_32x32b_x32(t_o + c * 32, v);
        }
        tmem_st_wait();
      }
      // P = exp2(S * scale - m) from registers (masked entries are -inf and give exactly 0), row
      // sum, bf16 P into the first 32 columns of the S buffer. The scale-and-shift and the sums use
      // the packed two-wide fp32 instructions. The 64 columns are handled as 32 pairs in a software
      // pipeline whose instruction order is pinned (volatile asm): a warp issues in order, and a run
      // of back-to-back exponentials would hold it for 8 cycles each with nothing else going out.
      // Per step the scale-and-shift of pair t+2, the two exponentials of pair t and the sum and
      // bf16 pack of pair t-3 are interleaved, so the packed FMA / add / convert work sits in the
      // shadow of the MUFU pipe.
      // The two groups share each scheduler's special-function unit, and a group's exponent phase
      // keeps it busy on its own. Taking turns (tile 1 starts block j's exponentials when tile 0
      // has delivered P(j), tile 0 starts block j+1's when tile 1 has delivered P(j)) puts one
      // group's TMEM load and row maximum in the shadow of the other's exponentials instead of
      // letting both phases coincide. The turn passes (x_done) as soon as the last exponential
      // has been issued.
      if (i == 1) {
        if (j < nblk[0] &&
            !(ok = warp_wait(x_done(0, buf), (j >> 1) & 1, kErrWaitOther, 8000 + j)))
          break;
      } else if (j >= 1 && j - 1 < nblk[1]) {
        if (!(ok = warp_wait(x_done(1, buf ^ 1), ((j - 1) >> 1) & 1, kErrWaitOther, 8500 + j)))
          break;
      }
      const uint64_t scale2 = pack_f32x2(p.scale_log2, p.scale_log2);
      const uint64_t negm2 = pack_f32x2(-m_used, -m_used);
      uint64_t sum2[4] = {0ull, 0ull, 0ull, 0ull};
      auto S = [&](int k) -> uint32_t { return k < 32 ? s0[k & 31] : s1[k & 31]; };
      constexpr int kPairs = BKV / 2;
      constexpr int kAhead = 2, kLag = 3;
      uint64_t xs[kPairs];
      float ev[BKV];
      uint32_t pk[kPairs];
#pragma unroll
      for (int t = -kAhead; t < kPairs + kLag; ++t) {
        const int ta = t + kAhead, tc = t - kLag;
        if (ta >= 0 && ta < kPairs) xs[ta] = ffma2_v(pack_u32x2(S(2 * ta), S(2 * ta + 1)), scale2, negm2);
        if (t >= 0 && t < kPairs) ev[2 * t] = ex2_v(lo_f32(xs[t]));
        if (tc >= 0 && tc < kPairs)
          sum2[tc & 3] = fadd2_v(sum2[tc & 3], pack_f32x2(ev[2 * tc], ev[2 * tc + 1]));
        if (t >= 0 && t < kPairs) ev[2 * t + 1] = ex2_v(hi_f32(xs[t]));
        if (tc >= 0 && tc < kPairs) pk[tc] = cvt_bf16x2_v(ev[2 * tc + 1], ev[2 * tc]);
        if (t == kPairs - 1) {
          __syncwarp();
          if (lane == 0) mbar_arrive_after(x_done(i, buf), ev[2 * t + 1]);
        }
      }
      tmem_st_32x32b_x32(t_s, pk);
      {
        const uint64_t t2 = fadd2(fadd2(sum2[0], sum2[1]), fadd2(sum2[2], sum2[3]));
        l += lo_f32(t2) + hi_f32(t2);
      }
      tmem_st_wait();
      tc_fence_before();
      // One arrival per warp: 128 arrivals on a single shared-memory word would serialise.
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full(i, buf));
    }
    // ---- epilogue: O / l -> bf16 -> swizzled smem (the Q tile's buffer) -> TMA store
    if (ok && nblk[i] > 0) ok = warp_wait(o_full(i), 0, kErrWaitTmemFull, 9000);
    if (nblk[i] > 0) {
      tc_fence_after();
      const float inv = 1.0f / l;
      if (p.lse2 && row_q < p.Sq)
        p.lse2[(static_cast<long long>(b) * p.H + h) * p.Sq + row_q] = l > 0.f ? m_used + log2f(l) : INFINITY;
      const uint32_t t_o = tO(i) + lane_base;
      const uint32_t obuf = sQ + i * TILE_BYTES;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(t_o + c * 32, v);
        tmem_ld_wait();
        const uint32_t blk = obuf + (c >> 1) * HALF_BYTES;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e)
            w[e] = pack_bf16(__uint_as_float(v[ch * 8 + 2 * e]) * inv,
                             __uint_as_float(v[ch * 8 + 2 * e + 1]) * inv);
          const uint32_t addr = blk + swz128(r, (c & 1) * 4 + ch);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[0]), "r"(w[1]),
                       "r"(w[2]), "r"(w[3])
                       : "memory");
        }
      }
      fence_proxy_async_smem();
      asm volatile("bar.sync %0, 128;" ::"r"(1 + i) : "memory");
      if (r == 0 && ok) {
        tma_store_4d(&tmO, obuf, 0, qi0, h, b);
        tma_store_4d(&tmO, obuf + HALF_BYTES, 64, qi0, h, b);
        tma_store_commit();
        tma_store_wait<0>();
      }
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

// Strides are in elements, one triple (batch, head, position) per tensor; the head dimension is
// contiguous. Any layout TMA can describe works: [B,H,S,D], [B,S,H,D], or column slices of a fused
// QKV projection output. Every stride must be a multiple of 8 elements (16 bytes).
int launch_strided(const void* Q, const void* K, const void* V, void* O, int B, int H, int Hkv,
                   int Sq, int Sk, int Dh, const long long* qs, const long long* ks,
                   const long long* vs, const long long* os, float scale, int causal,
                   cudaStream_t st, float* lse2 = nullptr) {
  if (!Q || !K || !V || !O || B <= 0 || H <= 0 || Hkv <= 0 || Sq <= 0 || Sk <= 0) {
    set_last_error("attn_prefill: null pointer or non-positive size");
    return kBadArg;
  }
  if (Dh != D) {
    set_last_error("attn_prefill: head dimension must be %d (got %d)", D, Dh);
    return kBadArg;
  }
  if (H % Hkv) {
    set_last_error("attn_prefill: H (%d) must be divisible by Hkv (%d)", H, Hkv);
    return kBadArg;
  }
  if (!(scale > 0.f)) {
    set_last_error("attn_prefill: scale must be positive");
    return kBadArg;
  }
  for (const void* ptr : {Q, K, V, (const void*)O})
    if (reinterpret_cast<uintptr_t>(ptr) & 15) {
      set_last_error("attn_prefill: pointers must be 16-byte aligned");
      return kBadArg;
    }
  for (const long long* t : {qs, ks, vs, os})
    for (int i = 0; i < 3; ++i)
      if (t[i] <= 0 || (t[i] & 7)) {
        set_last_error("attn_prefill: strides must be positive multiples of 8 elements (got %lld)",
                       t[i]);
        return kBadArg;
      }
  CUtensorMap tQ, tK, tV, tO;
  auto encode = [&](CUtensorMap* m, const void* base, int S, int heads, const long long* t, uint32_t rows) {
    uint32_t box[4] = {64, rows, 1, 1};
    uint64_t dims[4] = {(uint64_t)D, (uint64_t)S, (uint64_t)heads, (uint64_t)B};
    uint64_t str[3] = {(uint64_t)t[2] * 2, (uint64_t)t[1] * 2, (uint64_t)t[0] * 2};
    return encode_tmap(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, base, dims, str, box,
                       CU_TENSOR_MAP_SWIZZLE_128B);
  };
  if (!encode(&tQ, Q, Sq, H, qs, BQ) || !encode(&tO, O, Sq, H, os, BQ) || !encode(&tK, K, Sk, Hkv, ks, BKV) ||
      !encode(&tV, V, Sk, Hkv, vs, BKV))
    return kBadArg;
  Params p{};
  p.B = B;
  p.H = H;
  p.Hkv = Hkv;
  p.Sq = Sq;
  p.Sk = Sk;
  p.causal = causal ? 1 : 0;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.err = device_err_word();
  if (!p.err) return kDeviceFailed;
  p.lse2 = lse2;
  TSB_CUDA_OK(cudaFuncSetAttribute(prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   SMEM_ALLOC));
  dim3 grid((Sq + 2 * BQ - 1) / (2 * BQ), H, B);
  prefill_kernel<<<grid, THREADS, SMEM_ALLOC, st>>>(tQ, tK, tV, tO, p);
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  return kOk;
}

int launch(const void* Q, const void* K, const void* V, void* O, int B, int H, int Hkv, int Sq,
           int Sk, int Dh, float scale, int causal, cudaStream_t st) {
  const long long qs[3] = {(long long)H * Sq * D, (long long)Sq * D, D};
  const long long ks[3] = {(long long)Hkv * Sk * D, (long long)Sk * D, D};
  return launch_strided(Q, K, V, O, B, H, Hkv, Sq, Sk, Dh, qs, ks, ks, qs, scale, causal, st);
}

// The forward pass that also records each row's log-sum-exp (base 2, of scale * log2(e) * s):
// what the backward kernels recompute P from.
int launch_with_lse(const void* Q, const void* K, const void* V, void* O, float* lse2, int B, int H,
                    int Hkv, int Sq, int Sk, int Dh, float scale, int causal, cudaStream_t st) {
  const long long qs[3] = {(long long)H * Sq * D, (long long)Sq * D, D};
  const long long ks[3] = {(long long)Hkv * Sk * D, (long long)Sk * D, D};
  return launch_strided(Q, K, V, O, B, H, Hkv, Sq, Sk, Dh, qs, ks, ks, qs, scale, causal, st, lse2);
}

}  // namespace attn_prefill
}  // namespace tsb

using namespace tsb;


extern "C" int tessera_sm100_flash_attn_fwd_strided_device(
    const void* Q, const void* K, const void* V, void* O, int B, int Hq, int Hkv, int Sq, int Sk,
    int D, const long long* q_strides, const long long* k_strides, const long long* v_strides,
    const long long* o_strides, float scale, int causal, void* stream) {
  if (!q_strides || !k_strides || !v_strides || !o_strides) {
    tsb::set_last_error("flash_attn_strided: null stride array");
    return tsb::kBadArg;
  }
  if (int rc = tsb::ensure_device()) return rc;
  return tsb::attn_prefill::launch_strided(Q, K, V, O, B, Hq, Hkv, Sq, Sk, D, q_strides, k_strides,
                                           v_strides, o_strides, scale, causal,
                                           static_cast<cudaStream_t>(stream));
}

extern "C" {

int tessera_sm100_flash_attn_fwd_device(const void* Q, const void* K, const void* V, void* O, int B,
                                        int Hq, int Hkv, int Sq, int Sk, int D, float scale,
                                        int causal, void* stream) {
  return attn_prefill::launch(Q, K, V, O, B, Hq, Hkv, Sq, Sk, D, scale, causal,
                              static_cast<cudaStream_t>(stream));
}

}  // extern "C"
