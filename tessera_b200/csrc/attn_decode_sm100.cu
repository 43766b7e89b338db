// GQA decode attention (one query token per sequence) for sm_100a: a bandwidth-bound
// split-KV flash-decode kernel.
//
//   O[b,hq,:] = softmax(scale * Q[b,hq,:] . K[b,hk,:,:]^T) V[b,hk,:,:],   hk = hq / (Hq/Hkv)
//
// (python/tessera/nn/functional.py:349-356 on top of python/tessera/__init__.py:1304-1356; for a
// single query token the causal mask removes nothing, python/tessera/__init__.py:1344-1349.)
//
// Grid = (kv splits, Hkv * head-groups, B). A CTA streams its KV range through a 3-stage
// TMA + mbarrier ring (64 positions of K and V per stage, 128-byte swizzle) fed by one producer
// warp. Four consumer warps each own 16 of the 64 positions. The up-to-8 query heads that share
// a KV head ride in the N dimension of mma.sync.m16n8k16 (tcgen05 needs M >= 64, which would be
// >= 87% padding here; the kernel is HBM-bound, not tensor-bound):
//     S^T[16 pos x 8 heads]  = K[16 x 128] . Q^T[128 x 8]
//     O^T[128 d  x 8 heads] += V^T[128 x 16 pos] . P^T[16 x 8]     (V via ldmatrix.trans,
//                                                                   P^T via movmatrix)
// Online softmax keeps fp32 running max / sum per head; the max over positions is a
// warp-shuffle reduction. Warps are merged through shared memory, splits through a small
// fp32 partial buffer and a second kernel (the merge of
// python/tessera/_block_attnres_ops.py:104-146).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cmath>
#include <mutex>

#include "../../include/tessera_sm100.h"
#include "device_ctx.h"
#include "sm100_ptx.cuh"

namespace tsb {
namespace attn_decode {

constexpr int D = 128;
constexpr int TILE = 64;      // KV positions per stage
constexpr int STAGES = 3;
constexpr int CONSUMERS = 4;  // warps; each owns TILE / 4 = 16 positions
constexpr int THREADS = (CONSUMERS + 1) * 32;
constexpr int HALF_BYTES = TILE * 64 * 2;        // one [64 pos][64 d] swizzled block
constexpr int KV_BYTES = 2 * HALF_BYTES;         // K or V tile
constexpr int STAGE_BYTES = 2 * KV_BYTES;        // K + V
constexpr int SMEM_BAR_OFF = STAGES * STAGE_BYTES;
constexpr int SMEM_BYTES = SMEM_BAR_OFF + 64;
constexpr int SMEM_ALLOC = SMEM_BYTES + 1024;
constexpr int MAX_SPLITS = 64;
// 8-bit KV (per-token scales): a stage is 8 KB of K bytes + 8 KB of V bytes, each 64 rows of
// 128 bytes under the 128-byte swizzle, plus the tile's 64 + 64 scales. The consumer warps take
// their MMA fragments straight from the byte tiles with ldmatrix (which moves 16-bit units, i.e.
// byte pairs) and widen them in registers with byte permutes; nothing is staged as f16.
constexpr int Q8_KV_BYTES = TILE * D;                 // 8 KB
constexpr int Q8_STAGE_BYTES = 2 * Q8_KV_BYTES;       // 16 KB
constexpr int Q8_SC_STAGE = 2 * TILE * 4;             // per stage: 64 K scales, then 64 V scales
constexpr int Q8_SC_OFF = STAGES * Q8_STAGE_BYTES;     // 48 KB
constexpr int Q8_BAR_OFF = Q8_SC_OFF + STAGES * Q8_SC_STAGE;
constexpr int Q8_SMEM_ALLOC = Q8_BAR_OFF + 64 + 1024;

struct Params {
  const __nv_bfloat16* Q;  // [B, Hq, D]
  __nv_bfloat16* O;        // [B, Hq, D]
  float* part_o;           // [B, Hq, splits, D]   (unnormalised)
  float* part_ml;          // [B, Hq, splits, 2]   (max in log2 units, sum)
  int B, Hq, Hkv, Sk, G;   // G = Hq / Hkv
  int groups_per_kv;       // ceil(G / 8)
  int splits, tiles_total, tiles_per_split;
  float scale_log2;        // scale * log2(e)
  int* err;
  // Paged mode only: K/V live in pages [P, page_size, Hkv, D]; sequence b reads logical page lp
  // from physical page page_table[b * max_pages + lp] and holds seq_lens[b] positions.
  long long q_sb, q_sh, o_sb, o_sh;  // element strides of Q and O over (batch, head)
  // int8 KV: one fp32 scale per token for K and for V, shared by all heads
  // (python/tessera/__init__.py:3228-3236). Dense: [B, Sk]; paged: [num_pages, page_size].
  const float* k_scale;
  const float* v_scale;
  int force_partial;                 // write split partials even when there is one split
  const int* page_table;
  const int* seq_lens;
  int max_pages, num_pages, page_size, page_shift;
};


__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_f16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                              uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_f16(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}
// bf16x2 word -> f16x2 word (exact for values inside the f16 range; larger ones saturate)
__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t w) {
  return pack_f16(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
// The cache stores each quantised value q in [-127, 127] as the byte q + 128. Four such bytes ->
// two f16x2 words with two byte permutes and nothing else: a byte spliced under the f16 exponent
// of 1024 (0x64) IS the f16 number 1024 + byte = q + 1152. The constant 1152 is taken out of the
// dot products afterwards (it multiplies a per-head sum that costs next to nothing), which is
// what makes reading an 8-bit cache cheaper than reading a 16-bit one.
constexpr float kQ8Bias = 1152.0f;
__device__ __forceinline__ void u8x4_to_f16x4(uint32_t w, uint32_t& lo, uint32_t& hi) {
  asm("prmt.b32 %0, %1, %2, 0x5140;" : "=r"(lo) : "r"(w), "r"(0x64646464u));
  asm("prmt.b32 %0, %1, %2, 0x7362;" : "=r"(hi) : "r"(w), "r"(0x64646464u));
}
// The same for a word that ldmatrix.trans made of two rows' byte pairs: bytes (0, 2) are one
// column in two consecutive rows, bytes (1, 3) the next column.
__device__ __forceinline__ void u8x4_to_f16x4_cols(uint32_t w, uint32_t& even, uint32_t& odd) {
  asm("prmt.b32 %0, %1, %2, 0x5240;" : "=r"(even) : "r"(w), "r"(0x64646464u));
  asm("prmt.b32 %0, %1, %2, 0x5341;" : "=r"(odd) : "r"(w), "r"(0x64646464u));
}
__device__ __forceinline__ float f16x2_lo(uint32_t v) { return __low2float(*reinterpret_cast<__half2*>(&v)); }
__device__ __forceinline__ float f16x2_hi(uint32_t v) { return __high2float(*reinterpret_cast<__half2*>(&v)); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void consumer_bar() {
  asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS * 32) : "memory");
}

// kPaged = false: K, V are dense [B, Hkv, Sk, D] (tensor maps over (d, pos, head, batch)).
// kPaged = true : K, V are pages [P, page_size, Hkv, D] (tensor maps over (d, head, offset, page));
//                 the producer walks the sequence's page table and the length comes from
//                 seq_lens[b]. Everything after the TMA loads is shared.
template <bool kPaged, bool kInt8 = false>
__global__ void __launch_bounds__(THREADS, kInt8 ? 3 : 2)
decode_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
              const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  constexpr int kBarOff = kInt8 ? Q8_BAR_OFF : SMEM_BAR_OFF;
  constexpr int kStageBytes = kInt8 ? Q8_STAGE_BYTES : STAGE_BYTES;
  constexpr int kKvBytes = kInt8 ? Q8_KV_BYTES : KV_BYTES;
  const uint32_t bars = smem_base + kBarOff;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + kBarOff + 8 * 2 * STAGES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int split = blockIdx.x;
  const int kvh = blockIdx.y / p.groups_per_kv;
  const int hgroup = blockIdx.y - kvh * p.groups_per_kv;
  const int b = blockIdx.z;
  const int head0 = kvh * p.G + hgroup * 8;             // first query head of this CTA
  const int nheads = min(8, p.G - hgroup * 8);          // valid heads in the N dimension
  int Sk = p.Sk;
  int tiles_total = p.tiles_total;
  if constexpr (kPaged) {
    Sk = max(0, min(p.seq_lens[b], p.Sk));
    tiles_total = (Sk + TILE - 1) / TILE;
  }
  const int tile_begin = split * p.tiles_per_split;
  const int tile_end = min(tiles_total, tile_begin + p.tiles_per_split);
  const int ntiles = max(0, tile_end - tile_begin);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      // int8: the 32 producer lanes each add one arrival, fired when their scale copies land
      mbar_init(full_bar(s), kInt8 ? 33 : 1);
      mbar_init(empty_bar(s), CONSUMERS);
    }
    fence_mbar_init();
  }
  __syncthreads();

  if (warp == CONSUMERS) {
    // ------------------------------------------------------------ TMA producer
    if (kInt8 || lane == 0) {
      if (lane == 0) {
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
      }
      int stage = 0;
      uint32_t phase = 0;
      for (int i = 0; i < ntiles; ++i) {
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.err, kErrWaitEmpty, i)) break;
        const int pos0 = (tile_begin + i) * TILE;
        const uint32_t dst = smem_base + stage * kStageBytes;
        if constexpr (kInt8) {
          // Every lane brings the K and V scales of two of the tile's 64 positions with 4-byte
          // asynchronous copies (any alignment, dense or paged) and hangs an arrival on the
          // stage's full barrier that fires when they have landed. Positions that do not exist
          // get scale 0 (a copy of source size 0).
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int r = lane + 32 * h, pos = pos0 + r;
            long long idx = -1;
            if (pos < Sk) {
              if constexpr (kPaged) {
                const int lp = pos >> p.page_shift;
                if (lp < p.max_pages) {
                  const int phys = p.page_table[static_cast<long long>(b) * p.max_pages + lp];
                  if (phys >= 0 && phys < p.num_pages)
                    idx = static_cast<long long>(phys) * p.page_size + (pos & (p.page_size - 1));
                }
              } else {
                idx = static_cast<long long>(b) * p.Sk + pos;
              }
            }
            const uint32_t dk = smem_base + Q8_SC_OFF + stage * Q8_SC_STAGE + r * 4, dv = dk + TILE * 4;
            // source size 0 = write zeros without touching the source
            const int nbytes = idx >= 0 ? 4 : 0;
            const long long at = idx >= 0 ? idx : 0;
            asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dk), "l"(p.k_scale + at), "r"(nbytes) : "memory");
            asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dv), "l"(p.v_scale + at), "r"(nbytes) : "memory");
          }
          asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(full_bar(stage)) : "memory");
          if (lane != 0) {
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1u;
            }
            continue;
          }
        }
        mbar_arrive_expect_tx(full_bar(stage), kStageBytes);
        if constexpr (kInt8 && !kPaged) {
          // one box per tensor: 64 positions x 128 bytes
          tma_load_4d(dst, &tmK, full_bar(stage), 0, pos0, kvh, b);
          tma_load_4d(dst + kKvBytes, &tmV, full_bar(stage), 0, pos0, kvh, b);
        } else if constexpr (!kPaged) {
          tma_load_4d(dst, &tmK, full_bar(stage), 0, pos0, kvh, b);
          tma_load_4d(dst + HALF_BYTES, &tmK, full_bar(stage), 64, pos0, kvh, b);
          tma_load_4d(dst + KV_BYTES, &tmV, full_bar(stage), 0, pos0, kvh, b);
          tma_load_4d(dst + KV_BYTES + HALF_BYTES, &tmV, full_bar(stage), 64, pos0, kvh, b);
        } else {
          // One box per page piece: min(page_size, 64) positions. Pieces past the end of the
          // sequence (or with a bad table entry) are fetched at page index num_pages, which is
          // outside the tensor and therefore arrives as zeros with the full byte count.
          const int rows = min(p.page_size, TILE);
          const int pieces = TILE / rows;
          const int* table = p.page_table + static_cast<long long>(b) * p.max_pages;
          for (int s = 0; s < pieces; ++s) {
            const int pos = pos0 + s * rows;
            const int lp = pos >> p.page_shift;
            int phys = p.num_pages;
            if (pos < Sk && lp < p.max_pages) {
              phys = table[lp];
              if (phys < 0 || phys >= p.num_pages) {
                if (atomicCAS(p.err, 0, kErrBadPage) == 0) {
                  p.err[1] = b;
                  p.err[2] = lp;
                  p.err[3] = phys;
                }
                phys = p.num_pages;
              }
            }
            const int off = pos & (p.page_size - 1);
            const uint32_t d2 = dst + s * rows * 128;
            if constexpr (kInt8) {
              tma_load_4d(d2, &tmK, full_bar(stage), 0, kvh, off, phys);
              tma_load_4d(d2 + kKvBytes, &tmV, full_bar(stage), 0, kvh, off, phys);
            } else {
              tma_load_4d(d2, &tmK, full_bar(stage), 0, kvh, off, phys);
              tma_load_4d(d2 + HALF_BYTES, &tmK, full_bar(stage), 64, kvh, off, phys);
              tma_load_4d(d2 + KV_BYTES, &tmV, full_bar(stage), 0, kvh, off, phys);
              tma_load_4d(d2 + KV_BYTES + HALF_BYTES, &tmV, full_bar(stage), 64, kvh, off, phys);
            }
          }
        }
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
    if constexpr (kInt8) asm volatile("cp.async.wait_all;" ::: "memory");
    return;  // the producer warp takes no part in the consumer barriers below
  }

  // -------------------------------------------------------------- consumers
  const int g = lane >> 2;  // fragment row group
  const int t = lane & 3;   // fragment column pair
  // Q^T B-fragments for the 8 k-steps over d: head = g (zero beyond nheads).
  uint32_t qb[8][2];
  {
    const bool live = g < nheads;
    const uint32_t* qrow = reinterpret_cast<const uint32_t*>(
        p.Q + static_cast<long long>(b) * p.q_sb + (head0 + (live ? g : 0)) * p.q_sh);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      if constexpr (kInt8) {
        // The K fragments come straight from the byte tile: a lane's word holds d = 4t .. 4t+3
        // of a 16-wide block, which widens into the MMA's k slots (2t, 2t+1) and (2t+8, 2t+9).
        // The contraction only needs both operands to agree on the order, so Q follows it.
        qb[ks][0] = bf16x2_to_f16x2(live ? qrow[(16 * ks + 4 * t) >> 1] : 0u);
        qb[ks][1] = bf16x2_to_f16x2(live ? qrow[((16 * ks + 4 * t) >> 1) + 1] : 0u);
      } else {
        qb[ks][0] = live ? qrow[(16 * ks + 2 * t) >> 1] : 0u;
        qb[ks][1] = live ? qrow[(16 * ks + 8 + 2 * t) >> 1] : 0u;
      }
    }
  }
  // int8 KV: sum over d of the f16 query values of heads 2t and 2t+1 (the score columns this lane
  // holds), times the byte bias: what the biased K adds to every score of that head.
  float qbias0 = 0.f, qbias1 = 0.f;
  if constexpr (kInt8) {
    float part = 0.f;  // this lane's share of head g
#pragma unroll
    for (int ks = 0; ks < 8; ++ks)
      part += f16x2_lo(qb[ks][0]) + f16x2_hi(qb[ks][0]) + f16x2_lo(qb[ks][1]) + f16x2_hi(qb[ks][1]);
    part += __shfl_xor_sync(0xffffffffu, part, 1);
    part += __shfl_xor_sync(0xffffffffu, part, 2);   // lanes 4g .. 4g+3 now hold the sum of head g
    qbias0 = kQ8Bias * __shfl_sync(0xffffffffu, part, (2 * t) * 4);
    qbias1 = kQ8Bias * __shfl_sync(0xffffffffu, part, (2 * t + 1) * 4);
  }
  float lsv0 = 0.f, lsv1 = 0.f;  // int8 KV: running sums of the (scaled, f16) P fed to P.V
  float o[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY;  // running max (log2 units) for heads 2t, 2t+1
  float l0 = 0.f, l1 = 0.f;              // per-lane partial sums

  int stage = 0;
  uint32_t phase = 0;
  bool ok = true;
  for (int i = 0; i < ntiles; ++i) {
    if (!mbar_wait(full_bar(stage), phase, abort_flag, p.err, kErrWaitFull, i)) {
      ok = false;
      break;
    }
    // where this warp's 16 rows of K and V are read from, and how they are laid out
    uint32_t kbase = smem_base + stage * STAGE_BYTES;
    uint32_t vbase = kbase + KV_BYTES;
    uint32_t half_bytes = HALF_BYTES;
    uint32_t row_off = 16 * warp;
    float c[4] = {0.f, 0.f, 0.f, 0.f};
    if constexpr (kInt8) {
      // S^T = K . Q^T with the K fragments taken from the byte tile as they are: one ldmatrix.x4
      // brings 16 rows x 32 bytes, which widen (in registers) into the A fragments of two
      // k-steps. Two accumulators halve the depth of the dependent MMA chain.
      const uint32_t ksrc = smem_base + stage * Q8_STAGE_BYTES;
      float c_odd[4] = {0.f, 0.f, 0.f, 0.f};
      const uint32_t mat = lane >> 3;
      const uint32_t row = 16 * warp + (lane & 7) + ((mat & 1) ? 8 : 0);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t r[4], a[4];
        ldmatrix_x4(ksrc + swz128(row, 2 * j + (mat >> 1)), r);
        u8x4_to_f16x4(r[0], a[0], a[2]);
        u8x4_to_f16x4(r[1], a[1], a[3]);
        mma_f16_16816(c, a, qb[2 * j][0], qb[2 * j][1]);
        u8x4_to_f16x4(r[2], a[0], a[2]);
        u8x4_to_f16x4(r[3], a[1], a[3]);
        mma_f16_16816(c_odd, a, qb[2 * j + 1][0], qb[2 * j + 1][1]);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) c[e] += c_odd[e];
    }
    if constexpr (kPaged && !kInt8) {
      // The tail of the last page may hold anything (stale tokens, never-written memory); a
      // probability of zero times a NaN would still poison O, so this warp clears the V rows it
      // owns beyond the sequence end. K needs nothing: those scores are replaced by -inf below.
      const int first_dead = Sk - ((tile_begin + i) * TILE + 16 * warp);  // rows >= this are dead
      if (first_dead < 16) {
        uint8_t* vgen = smem_gen + stage * STAGE_BYTES + KV_BYTES;
        for (int c2 = lane; c2 < 16 * 16; c2 += 32) {
          const int r = c2 >> 4, chunk = c2 & 15;
          if (r >= first_dead)
            *reinterpret_cast<uint4*>(vgen + (chunk >> 3) * HALF_BYTES + (16 * warp + r) * 128 +
                                      (chunk & 7) * 16) = make_uint4(0, 0, 0, 0);
        }
        __syncwarp();
      }
    }
    if constexpr (!kInt8) {
      // S^T = K . Q^T for this warp's 16 positions
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        uint32_t a[4];
        const uint32_t row = row_off + (lane & 15);
        const uint32_t chunk = (ks & 3) * 2 + (lane >> 4);
        ldmatrix_x4(kbase + (ks >> 2) * half_bytes + swz128(row, chunk), a);
        mma_bf16_16816(c, a, qb[ks][0], qb[ks][1]);
      }
    }
    if constexpr (kInt8) {  // take the byte bias back out: columns are heads 2t, 2t+1
      c[0] -= qbias0;
      c[1] -= qbias1;
      c[2] -= qbias0;
      c[3] -= qbias1;
    }
    const int pos_a = (tile_begin + i) * TILE + 16 * warp + g;  // rows g and g + 8
    const bool va = pos_a < Sk, vb = (pos_a + 8) < Sk;
    // int8 KV: the per-token scales fold into the scores (K) and into P before P.V (V)
    float ka_s = p.scale_log2, kb_s = p.scale_log2, va_s = 1.f, vb_s = 1.f;
    if constexpr (kInt8) {
      const float* sc = reinterpret_cast<const float*>(smem_gen + Q8_SC_OFF + stage * Q8_SC_STAGE);
      ka_s *= sc[16 * warp + g];
      kb_s *= sc[16 * warp + g + 8];
      va_s = sc[TILE + 16 * warp + g];
      vb_s = sc[TILE + 16 * warp + g + 8];
    }
    float s0 = va ? c[0] * ka_s : -INFINITY;
    float s1 = va ? c[1] * ka_s : -INFINITY;
    float s2 = vb ? c[2] * kb_s : -INFINITY;
    float s3 = vb ? c[3] * kb_s : -INFINITY;
    float mx0 = fmaxf(s0, s2), mx1 = fmaxf(s1, s3);
#pragma unroll
    for (int sh = 4; sh <= 16; sh <<= 1) {
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, sh));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, sh));
    }
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float mu0 = (mn0 == -INFINITY) ? 0.f : mn0;
    const float mu1 = (mn1 == -INFINITY) ? 0.f : mn1;
    const float al0 = exp2f(m0 - mu0), al1 = exp2f(m1 - mu1);
    const float p0 = exp2f(s0 - mu0), p1 = exp2f(s1 - mu1);
    const float p2 = exp2f(s2 - mu0), p3 = exp2f(s3 - mu1);
    m0 = mn0;
    m1 = mn1;
    l0 = l0 * al0 + p0 + p2;
    l1 = l1 * al1 + p1 + p3;
    uint32_t pk0, pk1;
    if constexpr (kInt8) {
      pk0 = pack_f16(p0 * va_s, p1 * va_s);
      pk1 = pack_f16(p2 * vb_s, p3 * vb_s);
      // exactly what P.V multiplies the biased V with: needed to take the bias out of O
      lsv0 = lsv0 * al0 + f16x2_lo(pk0) + f16x2_lo(pk1);
      lsv1 = lsv1 * al1 + f16x2_hi(pk0) + f16x2_hi(pk1);
    } else {
      pk0 = pack_bf16(p0, p1);
      pk1 = pack_bf16(p2, p3);
    }
    const uint32_t pb0 = movmatrix_trans(pk0);
    const uint32_t pb1 = movmatrix_trans(pk1);
    if constexpr (kInt8) {
      // O^T += V^T . P^T, again from the byte tile: ldmatrix.trans (on byte PAIRS) hands a lane
      // the bytes (d, d+1) of positions (2t, 2t+1); the even bytes widen into the A fragment row
      // of d = 16 dt + 2g, the odd ones into that of d + 1. So accumulator rows g and g + 8 of
      // chunk dt stand for d = 16 dt + 2g and 16 dt + 2g + 1: the final write undoes that.
      const uint32_t vsrc = smem_base + stage * Q8_STAGE_BYTES + Q8_KV_BYTES;
      const uint32_t mat = lane >> 3;
      const uint32_t row = 16 * warp + (lane & 7) + ((mat & 1) ? 8 : 0);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t r[4], a[4];
        ldmatrix_x4_trans(vsrc + swz128(row, 2 * j + (mat >> 1)), r);
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int dt = 2 * j + e;
          o[dt][0] *= al0;
          o[dt][1] *= al1;
          o[dt][2] *= al0;
          o[dt][3] *= al1;
          u8x4_to_f16x4_cols(r[2 * e], a[0], a[1]);       // positions 0-7 of the warp's 16
          u8x4_to_f16x4_cols(r[2 * e + 1], a[2], a[3]);   // positions 8-15
          mma_f16_16816(o[dt], a, pb0, pb1);
        }
      }
    } else {
#pragma unroll
      for (int dt = 0; dt < 8; ++dt) {
        o[dt][0] *= al0;
        o[dt][1] *= al1;
        o[dt][2] *= al0;
        o[dt][3] *= al1;
        uint32_t a[4];
        const uint32_t mat = lane >> 3;
        const uint32_t row = row_off + (lane & 7) + ((mat & 2) ? 8 : 0);
        const uint32_t chunk = (dt & 3) * 2 + (mat & 1);
        ldmatrix_x4_trans(vbase + (dt >> 2) * half_bytes + swz128(row, chunk), a);
        mma_bf16_16816(o[dt], a, pb0, pb1);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty_bar(stage));
    if (++stage == STAGES) {
      stage = 0;
      phase ^= 1u;
    }
  }
  (void)ok;
  // finish the per-warp row sums (lanes with equal t hold partial sums of the same heads)
#pragma unroll
  for (int sh = 4; sh <= 16; sh <<= 1) {
    l0 += __shfl_xor_sync(0xffffffffu, l0, sh);
    l1 += __shfl_xor_sync(0xffffffffu, l1, sh);
  }
  if constexpr (kInt8) {
    // O' = sum p' (v + 1152): subtract 1152 * sum p' (columns are heads 2t, 2t+1)
#pragma unroll
    for (int sh = 4; sh <= 16; sh <<= 1) {
      lsv0 += __shfl_xor_sync(0xffffffffu, lsv0, sh);
      lsv1 += __shfl_xor_sync(0xffffffffu, lsv1, sh);
    }
#pragma unroll
    for (int dt = 0; dt < 8; ++dt) {
      o[dt][0] -= kQ8Bias * lsv0;
      o[dt][1] -= kQ8Bias * lsv1;
      o[dt][2] -= kQ8Bias * lsv0;
      o[dt][3] -= kQ8Bias * lsv1;
    }
  }
  // ---- merge the four warps through shared memory (the stage buffers are free now)
  consumer_bar();
  float* s_o = reinterpret_cast<float*>(smem_gen);                 // [4][8][128]
  float* s_m = s_o + CONSUMERS * 8 * D;                            // [4][8]
  float* s_l = s_m + CONSUMERS * 8;                                // [4][8]
  if (g == 0) {
    s_m[warp * 8 + 2 * t] = m0;
    s_m[warp * 8 + 2 * t + 1] = m1;
    s_l[warp * 8 + 2 * t] = l0;
    s_l[warp * 8 + 2 * t + 1] = l1;
  }
#pragma unroll
  for (int dt = 0; dt < 8; ++dt) {
    float* base = s_o + (warp * 8) * D;
    const int da = kInt8 ? 16 * dt + 2 * g : 16 * dt + g;        // accumulator row g
    const int db = kInt8 ? 16 * dt + 2 * g + 1 : 16 * dt + g + 8;  // accumulator row g + 8
    base[(2 * t) * D + da] = o[dt][0];
    base[(2 * t + 1) * D + da] = o[dt][1];
    base[(2 * t) * D + db] = o[dt][2];
    base[(2 * t + 1) * D + db] = o[dt][3];
  }
  consumer_bar();
  const int d = threadIdx.x;  // 0..127
  for (int h = 0; h < nheads; ++h) {
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < CONSUMERS; ++w) m = fmaxf(m, s_m[w * 8 + h]);
    const float mu = (m == -INFINITY) ? 0.f : m;
    float acc = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < CONSUMERS; ++w) {
      const float f = exp2f(s_m[w * 8 + h] - mu);
      acc += f * s_o[(w * 8 + h) * D + d];
      l += f * s_l[w * 8 + h];
    }
    const long long row = static_cast<long long>(b) * p.Hq + head0 + h;
    if (p.splits == 1 && !p.force_partial) {
      p.O[static_cast<long long>(b) * p.o_sb + (head0 + h) * p.o_sh + d] = __float2bfloat16_rn(acc / l);
    } else {
      p.part_o[(row * p.splits + split) * D + d] = acc;
      if (d == 0) {
        p.part_ml[(row * p.splits + split) * 2] = m;
        p.part_ml[(row * p.splits + split) * 2 + 1] = l;
      }
    }
  }
}

// One CTA per (b, hq): merges the split partials and writes bf16.
__global__ void merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                             __nv_bfloat16* __restrict__ O, int splits, int Hq, long long o_sb,
                             long long o_sh) {
  const long long row = blockIdx.x;
  const int d = threadIdx.x;
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, part_ml[(row * splits + s) * 2]);
  const float mu = (m == -INFINITY) ? 0.f : m;
  float acc = 0.f, l = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float f = exp2f(part_ml[(row * splits + s) * 2] - mu);
    acc += f * part_o[(row * splits + s) * D + d];
    l += f * part_ml[(row * splits + s) * 2 + 1];
  }
  O[(row / Hq) * o_sb + (row % Hq) * o_sh + d] = __float2bfloat16_rn(acc / l);
}

// One CTA per (b, hq): merges the split partials into one max-shifted state (o, m, l) with m in
// natural-log units, the state of python/tessera/_block_attnres_ops.py:104-131 — what a caller
// needs to merge attention over KV that is sharded further (other GPUs, other cache tiers).
__global__ void merge_state_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                   float* __restrict__ o_state, float* __restrict__ m_state,
                                   float* __restrict__ l_state, int splits) {
  const long long row = blockIdx.x;
  const int d = threadIdx.x;
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, part_ml[(row * splits + s) * 2]);
  const float mu = (m == -INFINITY) ? 0.f : m;
  float acc = 0.f, l = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float f = exp2f(part_ml[(row * splits + s) * 2] - mu);
    acc += f * part_o[(row * splits + s) * D + d];
    l += f * part_ml[(row * splits + s) * 2 + 1];
  }
  o_state[row * D + d] = acc;
  if (d == 0) {
    m_state[row] = m * 0.6931471805599453f;  // log2 units -> natural log
    l_state[row] = l;
  }
}

int choose_splits(int B, int Hkv, int groups_per_kv, int tiles_total) {
  // Measured on B200 (KV 8192, 8 KV heads): once the (batch, KV head) pairs alone fill a third of
  // the 2-CTAs-per-SM slots, one split is fastest (batch 64: 315 us against 327 us with three
  // splits; batch 16: 98 against 105); below that, splitting up to one full wave of CTAs helps
  // (batch 8: 62 us with 4 splits against 74 us with one and 69 us with 19). At least 8 tiles
  // (512 positions) per split keeps the ring's fill and the merge from dominating.
  const long long base = (long long)B * Hkv * groups_per_kv;
  const long long slots = (long long)sm_count() * 2;
  if (base * 3 > slots) return 1;
  long long s = slots / base;
  s = std::min<long long>(s, std::max(1, tiles_total / 8));
  s = std::max<long long>(1, std::min<long long>(s, MAX_SPLITS));
  return (int)s;
}

// The 8-bit cache kernel does more arithmetic per byte and runs three CTAs per SM, so it wants
// more, shorter CTAs. Measured on B200 (KV 8192, 8 KV heads): batch 4 is fastest with 7-13 splits
// (one wave: 28-30 us against 78 us with one), batch 16 with 3 (66 us against 84 us), and batch
// 64, whose (batch, KV head) pairs alone exceed the slots, with 3-5 (207 us against 259 us): a
// partial second wave costs a whole CTA's time, four waves of shorter CTAs even it out.
int choose_splits_int8(int B, int Hkv, int groups_per_kv, int tiles_total) {
  const long long base = (long long)B * Hkv * groups_per_kv;
  const long long slots = (long long)sm_count() * 3;
  long long s = slots / base;
  if (s < 2) s = (4 * slots + base - 1) / base;
  s = std::min<long long>(s, std::max(1, tiles_total / 8));
  s = std::max<long long>(1, std::min<long long>(s, MAX_SPLITS));
  return (int)s;
}

size_t scratch_bytes(int B, int Hq, int splits) {
  return (size_t)B * Hq * splits * (D + 2) * sizeof(float);
}

// K, V: [B, Hkv, Sk, D] bf16 device pointers; Q, O: [B, Hq, 1, D]. `scratch` must hold
// scratch_bytes(B, Hq, splits) bytes when splits > 1.
// Optional strides (elements, triples over (batch, head, position); the position stride of Q and O
// is unused): any layout with a contiguous head dimension, e.g. [B, S, H, D] or slices of a fused
// QKV buffer. Null means the dense layouts above.
int launch(const void* Q, const void* K, const void* V, void* O, int B, int Hq, int Hkv, int Sk,
           int Dh, float scale, int splits, void* scratch, cudaStream_t st,
           const long long* qs = nullptr, const long long* ks = nullptr,
           const long long* vs = nullptr, const long long* os = nullptr, float* o_state = nullptr,
           float* m_state = nullptr, float* l_state = nullptr, const float* k_scale = nullptr,
           const float* v_scale = nullptr) {
  // k_scale / v_scale given: K and V hold int8 with one fp32 scale per token ([B, Sk]).
  const bool int8 = k_scale != nullptr;
  if (int8 && (!v_scale || ks || vs)) {
    set_last_error("attn_decode: int8 K/V need both scale arrays and the dense layout");
    return kBadArg;
  }
  const bool want_state = o_state != nullptr;
  if (!Q || !K || !V || (!O && !want_state) || B <= 0 || Hq <= 0 || Hkv <= 0 || Sk <= 0 ||
      (want_state && (!m_state || !l_state))) {
    set_last_error("attn_decode: null pointer or non-positive size");
    return kBadArg;
  }
  if (Dh != D) {
    set_last_error("attn_decode: head dimension must be %d (got %d)", D, Dh);
    return kBadArg;
  }
  if (Hq % Hkv) {
    set_last_error("attn_decode: Hq (%d) must be divisible by Hkv (%d)", Hq, Hkv);
    return kBadArg;
  }
  if ((reinterpret_cast<uintptr_t>(K) & 15) || (reinterpret_cast<uintptr_t>(V) & 15) ||
      (reinterpret_cast<uintptr_t>(Q) & 3)) {
    set_last_error("attn_decode: K and V must be 16-byte aligned");
    return kBadArg;
  }
  Params p{};
  p.Q = static_cast<const __nv_bfloat16*>(Q);
  p.O = static_cast<__nv_bfloat16*>(O);
  p.B = B;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.Sk = Sk;
  p.G = Hq / Hkv;
  p.q_sb = p.o_sb = (long long)Hq * D;
  p.q_sh = p.o_sh = D;
  p.groups_per_kv = (p.G + 7) / 8;
  p.tiles_total = (Sk + TILE - 1) / TILE;
  if (splits <= 0)
    splits = int8 ? choose_splits_int8(B, Hkv, p.groups_per_kv, p.tiles_total)
                  : choose_splits(B, Hkv, p.groups_per_kv, p.tiles_total);
  splits = std::min(splits, std::min(p.tiles_total, MAX_SPLITS));
  p.tiles_per_split = (p.tiles_total + splits - 1) / splits;
  splits = (p.tiles_total + p.tiles_per_split - 1) / p.tiles_per_split;  // no empty splits
  p.splits = splits;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.err = device_err_word();
  if (!p.err) return kDeviceFailed;
  p.force_partial = want_state ? 1 : 0;
  if (splits > 1 || want_state) {
    if (!scratch) {
      set_last_error("attn_decode: %d splits need a scratch buffer", splits);
      return kBadArg;
    }
    p.part_o = static_cast<float*>(scratch);
    p.part_ml = p.part_o + (size_t)B * Hq * splits * D;
  }
  for (const long long* t : {qs, ks, vs, os})
    if (t)
      for (int i = 0; i < 3; ++i)
        if (t[i] <= 0 || (t[i] & 7)) {
          set_last_error("attn_decode: strides must be positive multiples of 8 elements (got %lld)",
                         t[i]);
          return kBadArg;
        }
  if (qs) {
    p.q_sb = qs[0];
    p.q_sh = qs[1];
  }
  if (os) {
    p.o_sb = os[0];
    p.o_sh = os[1];
  }
  CUtensorMap tK, tV;
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)Sk, (uint64_t)Hkv, (uint64_t)B};
  dim3 grid(splits, Hkv * p.groups_per_kv, B);
  if (int8) {
    p.k_scale = k_scale;
    p.v_scale = v_scale;
    uint64_t str8[3] = {(uint64_t)D, (uint64_t)Sk * D, (uint64_t)Hkv * Sk * D};
    uint32_t box8[4] = {(uint32_t)D, TILE, 1, 1};
    if (!encode_tmap(&tK, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, K, dims, str8, box8,
                     CU_TENSOR_MAP_SWIZZLE_128B) ||
        !encode_tmap(&tV, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, V, dims, str8, box8,
                     CU_TENSOR_MAP_SWIZZLE_128B))
      return kBadArg;
    TSB_CUDA_OK(cudaFuncSetAttribute(decode_kernel<false, true>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, Q8_SMEM_ALLOC));
    decode_kernel<false, true><<<grid, THREADS, Q8_SMEM_ALLOC, st>>>(tK, tV, p);
  } else {
    uint64_t str[3] = {(uint64_t)D * 2, (uint64_t)Sk * D * 2, (uint64_t)Hkv * Sk * D * 2};
    uint64_t strk[3], strv[3];
    for (int i = 0; i < 3; ++i) {
      strk[i] = ks ? (uint64_t)ks[2 - i] * 2 : str[i];
      strv[i] = vs ? (uint64_t)vs[2 - i] * 2 : str[i];
    }
    uint32_t box[4] = {64, TILE, 1, 1};
    if (!encode_tmap(&tK, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, K, dims, strk, box,
                     CU_TENSOR_MAP_SWIZZLE_128B) ||
        !encode_tmap(&tV, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, V, dims, strv, box,
                     CU_TENSOR_MAP_SWIZZLE_128B))
      return kBadArg;
    TSB_CUDA_OK(cudaFuncSetAttribute(decode_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     SMEM_ALLOC));
    decode_kernel<false><<<grid, THREADS, SMEM_ALLOC, st>>>(tK, tV, p);
  }
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  if (want_state) {
    merge_state_kernel<<<B * Hq, D, 0, st>>>(p.part_o, p.part_ml, o_state, m_state, l_state, splits);
    TSB_CUDA_OK(cudaGetLastError());
    note_launch();
  } else if (splits > 1) {
    merge_kernel<<<B * Hq, D, 0, st>>>(p.part_o, p.part_ml, p.O, splits, Hq, p.o_sb, p.o_sh);
    TSB_CUDA_OK(cudaGetLastError());
    note_launch();
  }
  return kOk;
}

// Elementwise merge of two states and the final division (python/tessera/_block_attnres_ops.py:
// 104-146): rows x Dv outputs, rows maxima and normalisers, all fp32.
__global__ void softmax_merge_kernel(const float* __restrict__ oa, const float* __restrict__ ma,
                                     const float* __restrict__ la, const float* __restrict__ ob,
                                     const float* __restrict__ mb, const float* __restrict__ lb,
                                     float* __restrict__ o, float* __restrict__ m,
                                     float* __restrict__ l, long long rows, int Dv) {
  const long long row = blockIdx.x;
  if (row >= rows) return;
  const float xa = ma[row], xb = mb[row];
  const float mx = fmaxf(xa, xb);
  const float sa = expf(xa - mx), sb = expf(xb - mx);
  for (int d = threadIdx.x; d < Dv; d += blockDim.x)
    o[row * Dv + d] = sa * oa[row * Dv + d] + sb * ob[row * Dv + d];
  if (threadIdx.x == 0) {
    m[row] = mx;
    l[row] = sa * la[row] + sb * lb[row];
  }
}

template <typename T>
__global__ void softmax_finalize_kernel(const float* __restrict__ o, const float* __restrict__ l,
                                        T* __restrict__ out, long long rows, int Dv) {
  const long long row = blockIdx.x;
  if (row >= rows) return;
  const float inv = 1.0f / l[row];
  for (int d = threadIdx.x; d < Dv; d += blockDim.x)
    out[row * Dv + d] = static_cast<T>(o[row * Dv + d] * inv);
}

// ---------------------------------------------------------------------------------------------
// Paged KV (python/tessera/cache/paged_kv.py:91-140: pages are [physical_page, page_offset, head,
// dim] and page_table[logical_page] names the physical page). Storage here is bf16 and the table
// is per sequence: page_table[B, max_pages], seq_lens[B].
int launch_paged(const void* Q, const void* k_pages, const void* v_pages, const int* page_table,
                 const int* seq_lens, void* O, int B, int Hq, int Hkv, int Dh, int page_size,
                 int num_pages, int max_pages, int max_seq_len, float scale, int splits,
                 void* scratch, cudaStream_t st, const float* k_scale = nullptr,
                 const float* v_scale = nullptr) {
  // k_scale / v_scale given: int8 pages with one fp32 scale per token, [num_pages, page_size].
  const bool int8 = k_scale != nullptr;
  if (int8 && !v_scale) {
    set_last_error("paged_attn_decode: int8 pages need both scale arrays");
    return kBadArg;
  }
  if (!Q || !k_pages || !v_pages || !page_table || !seq_lens || !O || B <= 0 || Hq <= 0 ||
      Hkv <= 0 || num_pages <= 0 || max_pages <= 0 || max_seq_len <= 0) {
    set_last_error("paged_attn_decode: null pointer or non-positive size");
    return kBadArg;
  }
  if (Dh != D) {
    set_last_error("paged_attn_decode: head dimension must be %d (got %d)", D, Dh);
    return kBadArg;
  }
  if (Hq % Hkv) {
    set_last_error("paged_attn_decode: Hq (%d) must be divisible by Hkv (%d)", Hq, Hkv);
    return kBadArg;
  }
  if (page_size < 8 || page_size > 1024 || (page_size & (page_size - 1))) {
    set_last_error("paged_attn_decode: page_size must be a power of two in [8, 1024] (got %d)",
                   page_size);
    return kBadArg;
  }
  if ((long long)max_pages * page_size < max_seq_len) {
    set_last_error("paged_attn_decode: max_seq_len %d exceeds the table capacity %d x %d",
                   max_seq_len, max_pages, page_size);
    return kBadArg;
  }
  if ((reinterpret_cast<uintptr_t>(k_pages) & 15) || (reinterpret_cast<uintptr_t>(v_pages) & 15) ||
      (reinterpret_cast<uintptr_t>(Q) & 3)) {
    set_last_error("paged_attn_decode: pages must be 16-byte aligned");
    return kBadArg;
  }
  Params p{};
  p.Q = static_cast<const __nv_bfloat16*>(Q);
  p.O = static_cast<__nv_bfloat16*>(O);
  p.B = B;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.Sk = max_seq_len;
  p.G = Hq / Hkv;
  p.q_sb = p.o_sb = (long long)Hq * D;
  p.q_sh = p.o_sh = D;
  p.groups_per_kv = (p.G + 7) / 8;
  p.tiles_total = (max_seq_len + TILE - 1) / TILE;
  p.page_table = page_table;
  p.seq_lens = seq_lens;
  p.max_pages = max_pages;
  p.num_pages = num_pages;
  p.page_size = page_size;
  p.page_shift = 0;
  while ((1 << p.page_shift) < page_size) ++p.page_shift;
  if (splits <= 0)
    splits = int8 ? choose_splits_int8(B, Hkv, p.groups_per_kv, p.tiles_total)
                  : choose_splits(B, Hkv, p.groups_per_kv, p.tiles_total);
  splits = std::min(splits, std::min(p.tiles_total, MAX_SPLITS));
  p.tiles_per_split = (p.tiles_total + splits - 1) / splits;
  splits = (p.tiles_total + p.tiles_per_split - 1) / p.tiles_per_split;
  p.splits = splits;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.err = device_err_word();
  if (!p.err) return kDeviceFailed;
  if (splits > 1) {
    if (!scratch) {
      set_last_error("paged_attn_decode: %d splits need a scratch buffer", splits);
      return kBadArg;
    }
    p.part_o = static_cast<float*>(scratch);
    p.part_ml = p.part_o + (size_t)B * Hq * splits * D;
  }
  CUtensorMap tK, tV;
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)Hkv, (uint64_t)page_size, (uint64_t)num_pages};
  dim3 grid(splits, Hkv * p.groups_per_kv, B);
  if (int8) {
    p.k_scale = k_scale;
    p.v_scale = v_scale;
    uint64_t str8[3] = {(uint64_t)D, (uint64_t)Hkv * D, (uint64_t)page_size * Hkv * D};
    uint32_t box8[4] = {(uint32_t)D, 1, (uint32_t)std::min(page_size, TILE), 1};
    if (!encode_tmap(&tK, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, k_pages, dims, str8, box8,
                     CU_TENSOR_MAP_SWIZZLE_128B) ||
        !encode_tmap(&tV, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, v_pages, dims, str8, box8,
                     CU_TENSOR_MAP_SWIZZLE_128B))
      return kBadArg;
    TSB_CUDA_OK(cudaFuncSetAttribute(decode_kernel<true, true>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, Q8_SMEM_ALLOC));
    decode_kernel<true, true><<<grid, THREADS, Q8_SMEM_ALLOC, st>>>(tK, tV, p);
  } else {
    uint64_t str[3] = {(uint64_t)D * 2, (uint64_t)Hkv * D * 2, (uint64_t)page_size * Hkv * D * 2};
    uint32_t box[4] = {64, 1, (uint32_t)std::min(page_size, TILE), 1};
    if (!encode_tmap(&tK, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, k_pages, dims, str, box,
                     CU_TENSOR_MAP_SWIZZLE_128B) ||
        !encode_tmap(&tV, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, v_pages, dims, str, box,
                     CU_TENSOR_MAP_SWIZZLE_128B))
      return kBadArg;
    TSB_CUDA_OK(cudaFuncSetAttribute(decode_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     SMEM_ALLOC));
    decode_kernel<true><<<grid, THREADS, SMEM_ALLOC, st>>>(tK, tV, p);
  }
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  if (splits > 1) {
    merge_kernel<<<B * Hq, D, 0, st>>>(p.part_o, p.part_ml, p.O, splits, Hq, p.o_sb, p.o_sh);
    TSB_CUDA_OK(cudaGetLastError());
    note_launch();
  }
  return kOk;
}

// Appends one token per sequence: K/V rows [B, Hkv, D] go to position seq_lens[b] of sequence b
// (page page_table[b, pos / page_size], offset pos % page_size) and seq_lens[b] grows by one.
// One CTA per sequence; 16-byte stores. A sequence whose table is full, or whose table entry is
// outside [0, num_pages), is left unchanged and reported through the error word.
__global__ void paged_append_kernel(const uint4* __restrict__ k_new, const uint4* __restrict__ v_new,
                                    uint4* __restrict__ k_pages, uint4* __restrict__ v_pages,
                                    const int* __restrict__ page_table, int* __restrict__ seq_lens,
                                    int row_vecs, int page_size, int num_pages, int max_pages,
                                    int* err) {
  const int b = blockIdx.x;
  const int pos = seq_lens[b];
  const int lp = pos / page_size;
  int phys = -1;
  if (pos >= 0 && lp < max_pages) phys = page_table[static_cast<long long>(b) * max_pages + lp];
  __syncthreads();  // every thread has read seq_lens[b] before thread 0 bumps it
  if (phys < 0 || phys >= num_pages) {
    if (threadIdx.x == 0 && atomicCAS(err, 0, kErrBadPage) == 0) {
      err[1] = b;
      err[2] = lp;
      err[3] = phys;
    }
    return;
  }
  const long long dst = (static_cast<long long>(phys) * page_size + (pos - lp * page_size)) * row_vecs;
  const long long src = static_cast<long long>(b) * row_vecs;
  for (int i = threadIdx.x; i < row_vecs; i += blockDim.x) {
    k_pages[dst + i] = k_new[src + i];
    v_pages[dst + i] = v_new[src + i];
  }
  if (threadIdx.x == 0) seq_lens[b] = pos + 1;
}

// Gathers tokens of one sequence out of the pages, in caller order (the staged read of
// python/tessera/compiler/emit/nvidia_cuda.py:2521, 2532): out[x, h, :] = pages[table[idx[x] /
// L], idx[x] % L, h, :]. One 16-byte vector per thread. Indices outside [0, table capacity) or
// bad table entries produce zeros and set the error word.
__global__ void paged_gather_kernel(const uint4* __restrict__ pages, const int* __restrict__ table,
                                    const long long* __restrict__ idx, uint4* __restrict__ out,
                                    long long T, int row_vecs, int page_size, int num_pages,
                                    int max_pages, int* err) {
  const long long z = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (z >= T * row_vecs) return;
  const long long x = z / row_vecs;
  const int i = static_cast<int>(z - x * row_vecs);
  const long long tok = idx[x];
  const long long lp = tok / page_size;
  int phys = -1;
  if (tok >= 0 && lp < max_pages) phys = table[lp];
  if (phys < 0 || phys >= num_pages) {
    if (atomicCAS(err, 0, kErrBadPage) == 0) {
      err[1] = static_cast<int>(x);
      err[2] = static_cast<int>(lp);
      err[3] = phys;
    }
    out[z] = make_uint4(0, 0, 0, 0);
    return;
  }
  out[z] = pages[(static_cast<long long>(phys) * page_size + (tok - lp * page_size)) * row_vecs + i];
}

// Per-token symmetric int8 quantisation of K and V rows (python/tessera/__init__.py:3224-3236):
// for token t, scale = max(amax over (heads, dim) / 127, 1e-12) and q = clip(rint(x / scale),
// -127, 127), in fp32, K and V each with their own scale. The byte written is q + 128 (the
// cache's storage form, see u8x4_to_f16x4). One CTA per token; `row` elements per
// token (heads * dim) in and out, dense. dst rows may live anywhere (a page slot): q_row(t) gives
// the destination row index.
template <typename T>
__global__ void quantize_kv_kernel(const T* __restrict__ k, const T* __restrict__ v,
                                   uint8_t* __restrict__ kq, uint8_t* __restrict__ vq,
                                   float* __restrict__ k_scale, float* __restrict__ v_scale,
                                   const long long* __restrict__ dst_rows, int row) {
  __shared__ float red[2][8];
  const long long t = blockIdx.x;
  const long long dst = dst_rows ? dst_rows[t] : t;
  if (dst < 0) return;  // nothing to write for this token
  const T* ks = k + t * row;
  const T* vs = v + t * row;
  float ak = 0.f, av = 0.f;
  for (int i = threadIdx.x; i < row; i += blockDim.x) {
    ak = fmaxf(ak, fabsf(static_cast<float>(ks[i])));
    av = fmaxf(av, fabsf(static_cast<float>(vs[i])));
  }
#pragma unroll
  for (int sh = 16; sh; sh >>= 1) {
    ak = fmaxf(ak, __shfl_xor_sync(0xffffffffu, ak, sh));
    av = fmaxf(av, __shfl_xor_sync(0xffffffffu, av, sh));
  }
  if ((threadIdx.x & 31) == 0) {
    red[0][threadIdx.x >> 5] = ak;
    red[1][threadIdx.x >> 5] = av;
  }
  __syncthreads();
  ak = av = 0.f;
  for (int w = 0; w < (blockDim.x >> 5); ++w) {
    ak = fmaxf(ak, red[0][w]);
    av = fmaxf(av, red[1][w]);
  }
  const float sk = fmaxf(__fdiv_rn(ak, 127.0f), 1e-12f), sv = fmaxf(__fdiv_rn(av, 127.0f), 1e-12f);
  if (threadIdx.x == 0) {
    k_scale[dst] = sk;
    v_scale[dst] = sv;
  }
  for (int i = threadIdx.x; i < row; i += blockDim.x) {
    const float qk = fminf(fmaxf(rintf(__fdiv_rn(static_cast<float>(ks[i]), sk)), -127.f), 127.f);
    const float qv = fminf(fmaxf(rintf(__fdiv_rn(static_cast<float>(vs[i]), sv)), -127.f), 127.f);
    kq[dst * row + i] = static_cast<uint8_t>(static_cast<int>(qk) + 128);
    vq[dst * row + i] = static_cast<uint8_t>(static_cast<int>(qv) + 128);
  }
}

// ---------------------------------------------------------------------------------------------
// Decode attention without any allocation.
//
// Some callers must not allocate device memory while they run: a serving loop whose memory
// budget was fixed at start-up (another component owns every remaining byte, so a cudaMalloc from
// inside this library could fail or evict it), or a latency-critical decode step where the
// implicit device-wide synchronisation of cudaMalloc/cudaFree would stall the other streams. For
// them the split-KV partials and the error word live in the two file-scope arrays below, which
// every GPU that loads the library holds until the process exits (8 MiB + 16 bytes per GPU).
constexpr size_t kStaticScratchBytes = 8u << 20;
static __device__ __align__(256) float g_static_partials[kStaticScratchBytes / sizeof(float)];
static __device__ __align__(256) int g_static_err[4];

constexpr int kMaxDevices = 64;
struct StaticSlots {
  float* partials = nullptr;  // DEVICE address of g_static_partials on that device
  int* err = nullptr;         // DEVICE address of g_static_err on that device
};
StaticSlots g_static_slots[kMaxDevices];
std::mutex g_static_mu;

// In host code the array names above are host-side stand-ins, not device addresses. The device
// address is looked up once per device, with that device current, and cached.
int static_slots_for_current_device(StaticSlots* out) {
  const int dev = current_device();
  if (dev < 0 || dev >= kMaxDevices) {
    set_last_error("attn_decode_static: device ordinal %d is outside [0, %d)", dev, kMaxDevices);
    return kBadArg;
  }
  std::lock_guard<std::mutex> lk(g_static_mu);
  StaticSlots& s = g_static_slots[dev];
  if (!s.partials) {
    // First call on this device only: make sure a context exists (this is the one place where the
    // entry point may touch the allocator; it does so with a null free), then resolve the symbols.
    if (int rc = ensure_device()) return rc;
    float* pp = nullptr;
    int* pe = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&pp), g_static_partials);
    if (e == cudaSuccess) e = cudaGetSymbolAddress(reinterpret_cast<void**>(&pe), g_static_err);
    if (e != cudaSuccess || !pp || !pe) {
      cudaGetLastError();
      set_last_error("attn_decode_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return kDeviceFailed;
    }
    s.partials = pp;
    s.err = pe;
  }
  *out = s;
  return kOk;
}

int launch_static(const void* Q, const void* K, const void* V, void* O, int B, int Hq, int Hkv,
                  int Sk, int Dh, float scale, int splits, int check_previous, cudaStream_t st) {
  if (!Q || !K || !V || !O || B <= 0 || Hq <= 0 || Hkv <= 0 || Sk <= 0) {
    set_last_error("attn_decode_static: null pointer or non-positive size");
    return kBadArg;
  }
  if (Dh != D) {
    set_last_error("attn_decode_static: head dimension must be %d (got %d)", D, Dh);
    return kBadArg;
  }
  if (Hq % Hkv) {
    set_last_error("attn_decode_static: Hq (%d) must be divisible by Hkv (%d)", Hq, Hkv);
    return kBadArg;
  }
  if ((reinterpret_cast<uintptr_t>(K) & 15) || (reinterpret_cast<uintptr_t>(V) & 15) ||
      (reinterpret_cast<uintptr_t>(Q) & 3)) {
    set_last_error("attn_decode_static: K and V must be 16-byte aligned and Q 4-byte aligned");
    return kBadArg;
  }
  StaticSlots slots;
  if (int rc = static_slots_for_current_device(&slots)) return rc;
  if (check_previous) {
    // Report (and clear) a bounded-wait expiry of an earlier launch of this entry point.
    int w[4] = {0, 0, 0, 0};
    TSB_CUDA_OK(cudaStreamSynchronize(st));
    TSB_CUDA_OK(cudaMemcpy(w, slots.err, sizeof(w), cudaMemcpyDeviceToHost));
    if (w[0] != 0) {
      TSB_CUDA_OK(cudaMemset(slots.err, 0, sizeof(w)));
      set_last_error("attn_decode_static: an earlier launch gave up a wait (code %d, block %d, "
                     "detail %d)", w[0], w[1], w[2]);
      return kDeviceFailed;
    }
  }
  Params p{};
  p.Q = static_cast<const __nv_bfloat16*>(Q);
  p.O = static_cast<__nv_bfloat16*>(O);
  p.B = B;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.Sk = Sk;
  p.G = Hq / Hkv;
  p.q_sb = p.o_sb = (long long)Hq * D;
  p.q_sh = p.o_sh = D;
  p.groups_per_kv = (p.G + 7) / 8;
  p.tiles_total = (Sk + TILE - 1) / TILE;
  const bool automatic = splits <= 0;
  if (automatic) splits = choose_splits(B, Hkv, p.groups_per_kv, p.tiles_total);
  splits = std::min(splits, std::min(p.tiles_total, MAX_SPLITS));
  if (automatic)  // take the largest split count whose partials fit the static array
    while (splits > 1 && scratch_bytes(B, Hq, splits) > kStaticScratchBytes) --splits;
  p.tiles_per_split = (p.tiles_total + splits - 1) / splits;
  splits = (p.tiles_total + p.tiles_per_split - 1) / p.tiles_per_split;
  if (splits > 1 && scratch_bytes(B, Hq, splits) > kStaticScratchBytes) {
    set_last_error("attn_decode_static: B=%d Hq=%d splits=%d needs %zu bytes of partials; the static "
                   "scratch holds %zu (use fewer splits, or tessera_sm100_attn_decode_device with "
                   "caller scratch)", B, Hq, splits, scratch_bytes(B, Hq, splits), kStaticScratchBytes);
    return kBadArg;
  }
  p.splits = splits;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.err = slots.err;
  if (splits > 1) {
    p.part_o = slots.partials;
    p.part_ml = p.part_o + (size_t)B * Hq * splits * D;
  }
  CUtensorMap tK, tV;
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)Sk, (uint64_t)Hkv, (uint64_t)B};
  uint64_t str[3] = {(uint64_t)D * 2, (uint64_t)Sk * D * 2, (uint64_t)Hkv * Sk * D * 2};
  uint32_t box[4] = {64, TILE, 1, 1};
  if (!encode_tmap(&tK, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, K, dims, str, box,
                   CU_TENSOR_MAP_SWIZZLE_128B) ||
      !encode_tmap(&tV, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, V, dims, str, box,
                   CU_TENSOR_MAP_SWIZZLE_128B))
    return kBadArg;
  TSB_CUDA_OK(cudaFuncSetAttribute(decode_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   SMEM_ALLOC));
  dim3 grid(splits, Hkv * p.groups_per_kv, B);
  decode_kernel<false><<<grid, THREADS, SMEM_ALLOC, st>>>(tK, tV, p);
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  if (splits > 1) {
    merge_kernel<<<B * Hq, D, 0, st>>>(p.part_o, p.part_ml, p.O, splits, Hq, p.o_sb, p.o_sh);
    TSB_CUDA_OK(cudaGetLastError());
    note_launch();
  }
  return kOk;
}

}  // namespace attn_decode
}  // namespace tsb

using namespace tsb;

extern "C" {

static int decode_splits_for(int B, int Hq, int Hkv, int Sk, bool int8) {
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || Sk <= 0 || Hq % Hkv) return 1;
  if (ensure_device()) return 1;
  const int G = Hq / Hkv;
  const int tiles = (Sk + attn_decode::TILE - 1) / attn_decode::TILE;
  int s = int8 ? attn_decode::choose_splits_int8(B, Hkv, (G + 7) / 8, tiles)
               : attn_decode::choose_splits(B, Hkv, (G + 7) / 8, tiles);
  s = std::min(s, std::min(tiles, attn_decode::MAX_SPLITS));
  const int tps = (tiles + s - 1) / s;
  return (tiles + tps - 1) / tps;
}

int tessera_sm100_attn_decode_splits(int B, int Hq, int Hkv, int Sk) {
  return decode_splits_for(B, Hq, Hkv, Sk, false);
}
int tessera_sm100_attn_decode_int8_splits(int B, int Hq, int Hkv, int Sk) {
  return decode_splits_for(B, Hq, Hkv, Sk, true);
}

size_t tessera_sm100_attn_decode_scratch_bytes(int B, int Hq, int splits) {
  return attn_decode::scratch_bytes(B, Hq, splits);
}

int tessera_sm100_attn_decode_device(const void* Q, const void* K, const void* V, void* O, int B,
                                     int Hq, int Hkv, int Sk, int D, float scale, int splits,
                                     void* scratch, void* stream) {
  return attn_decode::launch(Q, K, V, O, B, Hq, Hkv, Sk, D, scale, splits, scratch,
                             static_cast<cudaStream_t>(stream));
}

// Decode attention that stops before the division: the max-shifted state (o [B,Hq,D], m [B,Hq] in
// natural-log units, l [B,Hq], fp32) over this call's K/V. States over disjoint key sets merge
// with tessera_sm100_softmax_merge_device in any order. `scratch` is always needed
// (tessera_sm100_attn_decode_scratch_bytes with max(splits, 1)).
int tessera_sm100_attn_decode_state_device(const void* Q, const void* K, const void* V,
                                           float* o_state, float* m_state, float* l_state, int B,
                                           int Hq, int Hkv, int Sk, int D, float scale, int splits,
                                           void* scratch, void* stream) {
  return attn_decode::launch(Q, K, V, nullptr, B, Hq, Hkv, Sk, D, scale, splits, scratch,
                             static_cast<cudaStream_t>(stream), nullptr, nullptr, nullptr, nullptr,
                             o_state, m_state, l_state);
}

int tessera_sm100_softmax_merge_device(const float* oa, const float* ma, const float* la,
                                       const float* ob, const float* mb, const float* lb, float* o,
                                       float* m, float* l, long long rows, int Dv, void* stream) {
  if (!oa || !ma || !la || !ob || !mb || !lb || !o || !m || !l || rows < 0 || Dv <= 0) {
    set_last_error("softmax_merge: null pointer or bad size");
    return kBadArg;
  }
  if (rows == 0) return kOk;
  if (int rc = ensure_device()) return rc;
  attn_decode::softmax_merge_kernel<<<(unsigned)rows, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      oa, ma, la, ob, mb, lb, o, m, l, rows, Dv);
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  return kOk;
}

int tessera_sm100_softmax_finalize_device(const float* o, const float* l, void* out, long long rows,
                                          int Dv, int out_dtype, void* stream) {
  if (!o || !l || !out || rows < 0 || Dv <= 0) {
    set_last_error("softmax_finalize: null pointer or bad size");
    return kBadArg;
  }
  if (rows == 0) return kOk;
  if (int rc = ensure_device()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (out_dtype == TESSERA_SM100_F32)
    attn_decode::softmax_finalize_kernel<float><<<(unsigned)rows, 128, 0, st>>>(
        o, l, static_cast<float*>(out), rows, Dv);
  else if (out_dtype == TESSERA_SM100_BF16)
    attn_decode::softmax_finalize_kernel<__nv_bfloat16><<<(unsigned)rows, 128, 0, st>>>(
        o, l, static_cast<__nv_bfloat16*>(out), rows, Dv);
  else {
    set_last_error("softmax_finalize: output dtype must be f32 or bf16");
    return kBadArg;
  }
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  return kOk;
}

// Attention forward over strided operands (contiguous head dimension; element strides as triples
// over (batch, head, position) per tensor): one query position goes to the decode kernel, anything
// else to the prefill kernel. Nothing is copied or transposed.
int tessera_sm100_flash_attn_strided_device(const void* Q, const void* K, const void* V, void* O,
                                            int B, int Hq, int Hkv, int Sq, int Sk, int D,
                                            const long long* q_strides, const long long* k_strides,
                                            const long long* v_strides, const long long* o_strides,
                                            float scale, int causal, void* stream) {
  if (!q_strides || !k_strides || !v_strides || !o_strides) {
    set_last_error("flash_attn_strided: null stride array");
    return kBadArg;
  }
  if (Sq != 1)
    return tessera_sm100_flash_attn_fwd_strided_device(Q, K, V, O, B, Hq, Hkv, Sq, Sk, D, q_strides,
                                                       k_strides, v_strides, o_strides, scale,
                                                       causal, stream);
  if (int rc = ensure_device()) return rc;
  const int splits = tessera_sm100_attn_decode_splits(B, Hq, Hkv, Sk);
  void* scratch = nullptr;
  if (splits > 1) {
    scratch = pool_alloc(attn_decode::scratch_bytes(B, Hq, splits));
    if (!scratch) return kDeviceFailed;
  }
  const int rc = attn_decode::launch(Q, K, V, O, B, Hq, Hkv, Sk, D, scale, std::max(splits, 1),
                                     scratch, static_cast<cudaStream_t>(stream), q_strides,
                                     k_strides, v_strides, o_strides);
  if (scratch) pool_free_after(scratch, static_cast<cudaStream_t>(stream));  // reusable once this launch is done
  return rc;
}

// Decode over an int8 KV cache with per-token scales (KVCacheHandle(quantize_bits=8),
// python/tessera/cache/handle.py:72-215; quantize_kv / dequantize_kv,
// python/tessera/__init__.py:3196-3260): Kq, Vq [B, Hkv, Sk, 128] int8, k_scale, v_scale [B, Sk]
// fp32 (one scale per token, shared by the heads). The bytes are widened to f16 inside the kernel
// (exact) and the scales fold into the scores and into P, so the result equals attention over
// the dequantised cache.
int tessera_sm100_attn_decode_int8_device(const void* Q, const void* Kq, const void* Vq,
                                          const float* k_scale, const float* v_scale, void* O,
                                          int B, int Hq, int Hkv, int Sk, int D, float scale,
                                          int splits, void* scratch, void* stream) {
  if (!k_scale || !v_scale) {
    set_last_error("attn_decode_int8: null scale array");
    return kBadArg;
  }
  return attn_decode::launch(Q, Kq, Vq, O, B, Hq, Hkv, Sk, D, scale, splits, scratch,
                             static_cast<cudaStream_t>(stream), nullptr, nullptr, nullptr, nullptr,
                             nullptr, nullptr, nullptr, k_scale, v_scale);
}

// The paged form: pages [num_pages, page_size, Hkv, 128] int8, scale pages [num_pages, page_size].
int tessera_sm100_paged_attn_decode_int8_device(const void* Q, const void* k_pages,
                                                const void* v_pages, const float* k_scale,
                                                const float* v_scale, const int* page_table,
                                                const int* seq_lens, void* O, int B, int Hq, int Hkv,
                                                int D, int page_size, int num_pages, int max_pages,
                                                int max_seq_len, float scale, int splits,
                                                void* scratch, void* stream) {
  if (!k_scale || !v_scale) {
    set_last_error("paged_attn_decode_int8: null scale array");
    return kBadArg;
  }
  return attn_decode::launch_paged(Q, k_pages, v_pages, page_table, seq_lens, O, B, Hq, Hkv, D,
                                   page_size, num_pages, max_pages, max_seq_len, scale, splits,
                                   scratch, static_cast<cudaStream_t>(stream), k_scale, v_scale);
}

// k, v [T, row] (row = heads * dim; dtype code f32 / f16 / bf16) -> kq, vq int8 rows and their
// per-token scales. dst_rows (optional, device int64[T]) redirects token t to row dst_rows[t] of
// the outputs (a slot of a page pool); a negative entry skips the token.
int tessera_sm100_quantize_kv_int8_device(const void* k, const void* v, void* kq, void* vq,
                                          float* k_scale, float* v_scale, const long long* dst_rows,
                                          long long T, int row, int dtype, void* stream) {
  if (!k || !v || !kq || !vq || !k_scale || !v_scale || T < 0 || row <= 0) {
    set_last_error("quantize_kv_int8: null pointer or bad size");
    return kBadArg;
  }
  if (T == 0) return kOk;
  if (int rc = ensure_device()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>(T);
  auto kq8 = static_cast<uint8_t*>(kq);
  auto vq8 = static_cast<uint8_t*>(vq);
  switch (dtype) {
    case TESSERA_SM100_F32:
      attn_decode::quantize_kv_kernel<float><<<grid, 256, 0, st>>>(
          static_cast<const float*>(k), static_cast<const float*>(v), kq8, vq8, k_scale, v_scale, dst_rows, row);
      break;
    case TESSERA_SM100_BF16:
      attn_decode::quantize_kv_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
          static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), kq8, vq8, k_scale, v_scale,
          dst_rows, row);
      break;
    case TESSERA_SM100_F16:
      attn_decode::quantize_kv_kernel<__half><<<grid, 256, 0, st>>>(
          static_cast<const __half*>(k), static_cast<const __half*>(v), kq8, vq8, k_scale, v_scale, dst_rows, row);
      break;
    default:
      set_last_error("quantize_kv_int8: unsupported dtype %d", dtype);
      return kBadArg;
  }
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  return kOk;
}

// Paged decode: Q, O [B, Hq, D] bf16; pages [num_pages, page_size, Hkv, D] bf16; page_table
// [B, max_pages] int32; seq_lens [B] int32 (each in [1, max_seq_len]). `scratch` as for
// tessera_sm100_attn_decode_device, sized with the split count of (B, Hq, Hkv, max_seq_len).
int tessera_sm100_paged_attn_decode_device(const void* Q, const void* k_pages, const void* v_pages,
                                           const int* page_table, const int* seq_lens, void* O,
                                           int B, int Hq, int Hkv, int D, int page_size,
                                           int num_pages, int max_pages, int max_seq_len,
                                           float scale, int splits, void* scratch, void* stream) {
  return attn_decode::launch_paged(Q, k_pages, v_pages, page_table, seq_lens, O, B, Hq, Hkv, D,
                                   page_size, num_pages, max_pages, max_seq_len, scale, splits,
                                   scratch, static_cast<cudaStream_t>(stream));
}

int tessera_sm100_paged_kv_append_device(const void* k_new, const void* v_new, void* k_pages,
                                         void* v_pages, const int* page_table, int* seq_lens, int B,
                                         int Hkv, int D, int page_size, int num_pages,
                                         int max_pages, void* stream) {
  if (!k_new || !v_new || !k_pages || !v_pages || !page_table || !seq_lens || B <= 0 || Hkv <= 0 ||
      D <= 0 || page_size <= 0 || num_pages <= 0 || max_pages <= 0) {
    set_last_error("paged_kv_append: null pointer or non-positive size");
    return kBadArg;
  }
  if ((Hkv * D) % 8) {
    set_last_error("paged_kv_append: Hkv * D must be a multiple of 8 (16-byte rows)");
    return kBadArg;
  }
  if (int rc = ensure_device()) return rc;
  int* err = device_err_word();
  if (!err) return kDeviceFailed;
  const int row_vecs = Hkv * D / 8;
  attn_decode::paged_append_kernel<<<B, std::min(256, std::max(32, row_vecs)), 0,
                                     static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(k_new), static_cast<const uint4*>(v_new),
      static_cast<uint4*>(k_pages), static_cast<uint4*>(v_pages), page_table, seq_lens, row_vecs,
      page_size, num_pages, max_pages, err);
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  return kOk;
}

// pages [num_pages, page_size, H, D] bf16 -> out [T, H, D] bf16 for the logical token indices
// idx[T] (int64) of the sequence whose table is page_table[max_pages].
int tessera_sm100_paged_kv_gather_device(const void* pages, const int* page_table,
                                         const long long* idx, void* out, long long T, int H, int D,
                                         int page_size, int num_pages, int max_pages,
                                         void* stream) {
  if (!pages || !page_table || !idx || !out || T < 0 || H <= 0 || D <= 0 || page_size <= 0 ||
      num_pages <= 0 || max_pages <= 0) {
    set_last_error("paged_kv_gather: null pointer or non-positive size");
    return kBadArg;
  }
  if ((H * D) % 8) {
    set_last_error("paged_kv_gather: H * D must be a multiple of 8 (16-byte rows)");
    return kBadArg;
  }
  if (T == 0) return kOk;
  if (int rc = ensure_device()) return rc;
  int* err = device_err_word();
  if (!err) return kDeviceFailed;
  const int row_vecs = H * D / 8;
  const long long n = T * row_vecs;
  attn_decode::paged_gather_kernel<<<(unsigned)((n + 255) / 256), 256, 0,
                                     static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(pages), page_table, idx, static_cast<uint4*>(out), T, row_vecs,
      page_size, num_pages, max_pages, err);
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  return kOk;
}

// Decode attention that allocates nothing (no cudaMalloc, cudaFree or allocating library call, on
// the first call or any later one): the split-KV partials go to a static device array of 8 MiB.
// The first call on each device looks up that array's device address (cudaGetSymbolAddress, with
// the device current); make that first call before any stream capture.
int tessera_sm100_attn_decode_static_device(const void* Q, const void* K, const void* V, void* O,
                                            int B, int Hq, int Hkv, int Sk, int D, float scale,
                                            int splits, int check_previous, void* stream) {
  return attn_decode::launch_static(Q, K, V, O, B, Hq, Hkv, Sk, D, scale, splits, check_previous,
                                    static_cast<cudaStream_t>(stream));
}

}  // extern "C"
