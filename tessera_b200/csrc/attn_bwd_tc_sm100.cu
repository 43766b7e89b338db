// Attention backward on the tensor cores for the training shape of the benchmark configurations:
// bf16 storage, D = Dv = 128, no bias / window / soft-cap, optional causal mask with the
// bottom-right alignment of tessera.ops.flash_attn (key n is legal for query m when
// n <= m + shift, shift = max(Sk - Sq, 0)), grouped-query heads. Same mathematics as the general
// kernels in attn_bwd_sm100.cu (the reference lane, python/tessera/compiler/emit/nvidia_cuda.py:590-635):
//     p = exp(scale s - lse),  delta = dO . o,  ds = p (dO . v - delta),
//     dQ = scale ds K,  dK = scale ds^T Q,  dV = p^T dO   (dK, dV summed over the group's heads).
//
// Three launches after the forward pass (which also records the log-sum-exp of every row):
//   * delta_kernel: delta[row] = sum_d dO[row, d] O[row, d].
//   * dq_kernel: one CTA per 64 query rows of one head walks the legal 64-key blocks; per block
//     S = Q K^T and dP = dO V^T (mma.sync m16n8k16, fp32 accumulate), P and dS in registers, and
//     dQ += dS K with the dS accumulator fragments reused as the A operand.
//   * dkv_kernel: one CTA per 64 keys of one KV head walks the query heads of its group and their
//     legal 64-row blocks; it forms the TRANSPOSED tiles S^T = K Q^T and dP^T = V dO^T so that P^T
//     and dS^T are already the A operands of dV += P^T dO and dK += dS^T Q.
// Every gradient row is owned by one warp and accumulated in a fixed order (no atomics): reruns
// are bit-identical. The price is that S and dP are formed twice (7 tile products instead of 5).
// K/V (resp. Q/dO) tiles arrive through a two-deep cp.async ring in the 128-byte-swizzled layout
// that ldmatrix reads without bank conflicts.
#include <cuda_bf16.h>

#include <cmath>
#include <cstdlib>

#include "../../include/tessera_sm100.h"
#include "device_ctx.h"
#include "sm100_ptx.cuh"

namespace tsb {
namespace attn_prefill {
int launch_with_lse(const void* Q, const void* K, const void* V, void* O, float* lse2, int B, int H,
                    int Hkv, int Sq, int Sk, int Dh, float scale, int causal, cudaStream_t st);
}
namespace attn_bwd5 {
int launch(const void* dO, const void* Q, const void* K, const void* V, void* dQ, void* dK, void* dV,
           const float* lse2, const float* delta, int B, int Hq, int Hkv, int Sq, int Sk, float scale,
           int causal, cudaStream_t st);
}
namespace attn_bwd_tc {

constexpr int D = 128;
constexpr int BLK = 64;                  // query rows / keys per tile
constexpr int THREADS = 128;             // 4 warps, 16 tile rows each
constexpr int HALF = BLK * 128;          // bytes: 64 rows x 64 bf16, swizzled
constexpr int TILE = 2 * HALF;           // 64 rows x 128 bf16
constexpr int SMEM_DQ = 6 * TILE;                    // Q, dO, K[2], V[2]
constexpr int SMEM_DKV = 6 * TILE + 4 * BLK * 4;     // K, V, Q[2], dO[2], lse[2], delta[2]

struct Params {
  const __nv_bfloat16 *Q, *K, *V, *dO;
  __nv_bfloat16 *dQ, *dK, *dV;
  const float *lse2, *delta;
  int B, Hq, Hkv, Sq, Sk;
  int causal, shift;
  float scale, scale_log2;
};

__device__ __forceinline__ void ldsm(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_t(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
               "{%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// 16 bytes global -> shared, asynchronously; nbytes = 0 writes zeros without reading the source
__device__ __forceinline__ void cp16(uint32_t dst, const void* src, int nbytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(nbytes) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// One 64 x 128 bf16 tile (rows row0 .. row0+63 of a [rows_total, 128] matrix) into the swizzled
// layout: two halves of 64 rows x 128 B. Rows beyond rows_total arrive as zeros.
__device__ __forceinline__ void load_tile(uint32_t dst, const __nv_bfloat16* base, int row0, int rows_total) {
#pragma unroll
  for (int i = 0; i < (BLK * 16) / THREADS; ++i) {
    const int idx = threadIdx.x + THREADS * i;
    const int r = idx >> 4, ch = idx & 15;
    const bool live = row0 + r < rows_total;
    const __nv_bfloat16* src = base + static_cast<long long>(live ? row0 + r : 0) * D + ch * 8;
    cp16(dst + (ch >> 3) * HALF + swz128(r, ch & 7), src, live ? 16 : 0);
  }
}

// acc[8 n-tiles][4] (16 rows x 64 columns) = A(16 rows of a_tile from a_row0, all 128 d) . B^T where
// B^T's columns are the 64 rows of b_tile (both operands contracted over d).
__device__ __forceinline__ void mma_rows_x_rows(float (&acc)[8][4], uint32_t a_tile, int a_row0, uint32_t b_tile,
                                                int lane) {
  const int mat = lane >> 3;
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    uint32_t a[4];
    ldsm(a_tile + (ks >> 2) * HALF + swz128(a_row0 + (lane & 15), (ks & 3) * 2 + (lane >> 4)), a);
#pragma unroll
    for (int np = 0; np < 4; ++np) {
      uint32_t b[4];
      ldsm(b_tile + (ks >> 2) * HALF + swz128(16 * np + (lane & 7) + ((mat & 2) ? 8 : 0), (ks & 3) * 2 + (mat & 1)), b);
      mma(acc[2 * np], a, b[0], b[1]);
      mma(acc[2 * np + 1], a, b[2], b[3]);
    }
  }
}

// out[16 n-tiles][4] (16 rows x 128 d) += A(16 x 64, given as bf16 A fragments a[4 k-steps][4]) . B
// where B's rows (the contraction) are the 64 rows of b_tile and its columns the 128 d.
__device__ __forceinline__ void mma_frag_x_tile(float (&out)[16][4], const uint32_t (&a)[4][4], uint32_t b_tile,
                                                int lane) {
  const int mat = lane >> 3;
#pragma unroll
  for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
    for (int dp = 0; dp < 8; ++dp) {
      uint32_t b[4];
      ldsm_t(b_tile + (dp >> 2) * HALF + swz128(16 * kk + (lane & 7) + ((mat & 1) ? 8 : 0), (dp & 3) * 2 + (mat >> 1)), b);
      mma(out[2 * dp], a[kk], b[0], b[1]);
      mma(out[2 * dp + 1], a[kk], b[2], b[3]);
    }
  }
}

// C fragments of a 16 x 64 tile -> A fragments (bf16) of the same tile for the next product
__device__ __forceinline__ void frag_c_to_a(const float (&c)[8][4], uint32_t (&a)[4][4]) {
#pragma unroll
  for (int kk = 0; kk < 4; ++kk) {
    a[kk][0] = pack2(c[2 * kk][0], c[2 * kk][1]);
    a[kk][1] = pack2(c[2 * kk][2], c[2 * kk][3]);
    a[kk][2] = pack2(c[2 * kk + 1][0], c[2 * kk + 1][1]);
    a[kk][3] = pack2(c[2 * kk + 1][2], c[2 * kk + 1][3]);
  }
}

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

__global__ void __launch_bounds__(THREADS, 2) dq_kernel(const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ = base, sdO = base + TILE, sK = base + 2 * TILE, sV = base + 4 * TILE;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int m0 = blockIdx.x * BLK, hq = blockIdx.y, b = blockIdx.z;
  const int hk = hq / (p.Hq / p.Hkv);
  const long long qoff = (static_cast<long long>(b) * p.Hq + hq) * p.Sq;
  const long long koff = (static_cast<long long>(b) * p.Hkv + hk) * p.Sk;
  const __nv_bfloat16* Kb = p.K + koff * D;
  const __nv_bfloat16* Vb = p.V + koff * D;
  int n_end = p.Sk;
  if (p.causal) n_end = min(n_end, m0 + BLK - 1 + p.shift + 1);
  const int nblocks = n_end > 0 ? (n_end + BLK - 1) / BLK : 0;

  load_tile(sQ, p.Q + qoff * D, m0, p.Sq);
  load_tile(sdO, p.dO + qoff * D, m0, p.Sq);
  if (nblocks > 0) {
    load_tile(sK, Kb, 0, p.Sk);
    load_tile(sV, Vb, 0, p.Sk);
  }
  cp_commit();
  const int ra = m0 + 16 * warp + g, rb = ra + 8;
  const float lse_a = ra < p.Sq ? p.lse2[qoff + ra] : INFINITY;
  const float lse_b = rb < p.Sq ? p.lse2[qoff + rb] : INFINITY;
  const float del_a = ra < p.Sq ? p.delta[qoff + ra] : 0.f;
  const float del_b = rb < p.Sq ? p.delta[qoff + rb] : 0.f;

  float dq[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) dq[i][e] = 0.f;

  for (int j = 0; j < nblocks; ++j) {
    const uint32_t bK = sK + (j & 1) * TILE, bV = sV + (j & 1) * TILE;
    if (j + 1 < nblocks) {
      load_tile(sK + ((j + 1) & 1) * TILE, Kb, (j + 1) * BLK, p.Sk);
      load_tile(sV + ((j + 1) & 1) * TILE, Vb, (j + 1) * BLK, p.Sk);
      cp_commit();
      cp_wait<1>();
    } else {
      cp_wait<0>();
    }
    __syncthreads();
    float s[8][4], dp[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[i][e] = dp[i][e] = 0.f;
    mma_rows_x_rows(dp, sdO, 16 * warp, bV, lane);
    mma_rows_x_rows(s, sQ, 16 * warp, bK, lane);
    const int n0 = j * BLK;
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int col = n0 + 8 * i + 2 * t + (e & 1);
        const int row = (e < 2) ? ra : rb;
        const bool legal = col < p.Sk && (!p.causal || col <= row + p.shift);
        const float pe = legal ? ex2f(s[i][e] * p.scale_log2 - ((e < 2) ? lse_a : lse_b)) : 0.f;
        dp[i][e] = pe * (dp[i][e] - ((e < 2) ? del_a : del_b));   // dS (without the scale)
      }
    uint32_t a[4][4];
    frag_c_to_a(dp, a);
    mma_frag_x_tile(dq, a, bK, lane);
    __syncthreads();   // every warp is done with this ring slot before it is refilled
  }
  __nv_bfloat16* out = p.dQ + qoff * D;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int d = 8 * i + 2 * t;
    if (ra < p.Sq)
      *reinterpret_cast<uint32_t*>(out + static_cast<long long>(ra) * D + d) = pack2(dq[i][0] * p.scale, dq[i][1] * p.scale);
    if (rb < p.Sq)
      *reinterpret_cast<uint32_t*>(out + static_cast<long long>(rb) * D + d) = pack2(dq[i][2] * p.scale, dq[i][3] * p.scale);
  }
}

__global__ void __launch_bounds__(THREADS, 2) dkv_kernel(const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t sK = base, sV = base + TILE, sQ = base + 2 * TILE, sdO = base + 4 * TILE;
  float* s_lse = reinterpret_cast<float*>(gen + 6 * TILE);   // [2][64]
  float* s_del = s_lse + 2 * BLK;                            // [2][64]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * BLK, hk = blockIdx.y, b = blockIdx.z;
  const int ratio = p.Hq / p.Hkv;
  const long long koff = (static_cast<long long>(b) * p.Hkv + hk) * p.Sk;
  // query blocks that hold a legal row for some key of this tile: rows m >= n0 - shift
  const int nqb = (p.Sq + BLK - 1) / BLK;
  int i_start = 0;
  if (p.causal) i_start = max(0, n0 - p.shift) / BLK;
  const int per_head = max(0, nqb - i_start);
  const int iters = per_head * ratio;

  auto issue = [&](int it) {
    const int hq = hk * ratio + it / per_head;
    const int m0 = (i_start + it % per_head) * BLK;
    const long long qoff = (static_cast<long long>(b) * p.Hq + hq) * p.Sq;
    const int slot = it & 1;
    load_tile(sQ + slot * TILE, p.Q + qoff * D, m0, p.Sq);
    load_tile(sdO + slot * TILE, p.dO + qoff * D, m0, p.Sq);
    if (threadIdx.x < BLK) {
      const int m = m0 + threadIdx.x;
      // rows that do not exist get lse = +inf, i.e. p = 0
      s_lse[slot * BLK + threadIdx.x] = m < p.Sq ? p.lse2[qoff + m] : INFINITY;
      s_del[slot * BLK + threadIdx.x] = m < p.Sq ? p.delta[qoff + m] : 0.f;
    }
  };

  load_tile(sK, p.K + koff * D, n0, p.Sk);
  load_tile(sV, p.V + koff * D, n0, p.Sk);
  if (iters > 0) issue(0);
  cp_commit();

  float dk[16][4], dv[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) dk[i][e] = dv[i][e] = 0.f;
  const int ka = n0 + 16 * warp + g, kb = ka + 8;   // this lane's key rows

  for (int it = 0; it < iters; ++it) {
    const int slot = it & 1;
    if (it + 1 < iters) {
      issue(it + 1);
      cp_commit();
      cp_wait<1>();
    } else {
      cp_wait<0>();
    }
    __syncthreads();
    const int m0 = (i_start + it % per_head) * BLK;
    const uint32_t bQ = sQ + slot * TILE, bdO = sdO + slot * TILE;
    float st[8][4], dpt[8][4];   // S^T and dP^T: rows = keys, columns = query rows
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) st[i][e] = dpt[i][e] = 0.f;
    mma_rows_x_rows(dpt, sV, 16 * warp, bdO, lane);
    mma_rows_x_rows(st, sK, 16 * warp, bQ, lane);
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int mc = 8 * i + 2 * t + (e & 1);          // query row inside the block
        const int m = m0 + mc;
        const int key = (e < 2) ? ka : kb;
        const bool legal = key < p.Sk && (!p.causal || key <= m + p.shift);
        const float pe = legal ? ex2f(st[i][e] * p.scale_log2 - s_lse[slot * BLK + mc]) : 0.f;
        st[i][e] = pe;
        dpt[i][e] = pe * (dpt[i][e] - s_del[slot * BLK + mc]);
      }
    uint32_t a[4][4];
    frag_c_to_a(st, a);
    mma_frag_x_tile(dv, a, bdO, lane);
    frag_c_to_a(dpt, a);
    mma_frag_x_tile(dk, a, bQ, lane);
    __syncthreads();
  }
  __nv_bfloat16* ok = p.dK + koff * D;
  __nv_bfloat16* ov = p.dV + koff * D;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int d = 8 * i + 2 * t;
    if (ka < p.Sk) {
      *reinterpret_cast<uint32_t*>(ok + static_cast<long long>(ka) * D + d) = pack2(dk[i][0] * p.scale, dk[i][1] * p.scale);
      *reinterpret_cast<uint32_t*>(ov + static_cast<long long>(ka) * D + d) = pack2(dv[i][0], dv[i][1]);
    }
    if (kb < p.Sk) {
      *reinterpret_cast<uint32_t*>(ok + static_cast<long long>(kb) * D + d) = pack2(dk[i][2] * p.scale, dk[i][3] * p.scale);
      *reinterpret_cast<uint32_t*>(ov + static_cast<long long>(kb) * D + d) = pack2(dv[i][2], dv[i][3]);
    }
  }
}

}  // namespace attn_bwd_tc
}  // namespace tsb

using namespace tsb;

extern "C" {

// Workspace of the tensor-core backward: O (bf16), log-sum-exp and delta (fp32) per query row.
size_t tessera_sm100_flash_attn_bwd_bf16_workspace_bytes(int B, int Hq, int Sq) {
  if (B <= 0 || Hq <= 0 || Sq <= 0) return 0;
  const size_t rows = static_cast<size_t>(B) * Hq * Sq;
  return ((rows * attn_bwd_tc::D * 2 + 255) & ~size_t(255)) + 2 * ((rows * 4 + 255) & ~size_t(255));
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
  float* lse2 = reinterpret_cast<float*>(ws + ((rows * attn_bwd_tc::D * 2 + 255) & ~size_t(255)));
  float* delta = reinterpret_cast<float*>(reinterpret_cast<char*>(lse2) + ((rows * 4 + 255) & ~size_t(255)));
  if (int rc = attn_prefill::launch_with_lse(Q, K, V, O, lse2, B, Hq, Hkv, Sq, Sk, attn_bwd_tc::D, scale,
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
  attn_bwd_tc::delta_kernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(dO), static_cast<const __nv_bfloat16*>(O), delta,
      static_cast<long long>(rows));
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  // The tcgen05 kernels are the default; TESSERA_SM100_ATTN_BWD=mma selects the mma.sync ones
  // (same inputs, same ownership of the gradient rows), kept for comparison.
  static const bool use_mma = [] {
    const char* e = getenv("TESSERA_SM100_ATTN_BWD");
    return e && e[0] == 'm';
  }();
  if (!use_mma)
    return attn_bwd5::launch(dO, Q, K, V, dQ, dK, dV, lse2, delta, B, Hq, Hkv, Sq, Sk, scale, causal, st);
  attn_bwd_tc::Params p{};
  p.Q = static_cast<const __nv_bfloat16*>(Q);
  p.K = static_cast<const __nv_bfloat16*>(K);
  p.V = static_cast<const __nv_bfloat16*>(V);
  p.dO = static_cast<const __nv_bfloat16*>(dO);
  p.dQ = static_cast<__nv_bfloat16*>(dQ);
  p.dK = static_cast<__nv_bfloat16*>(dK);
  p.dV = static_cast<__nv_bfloat16*>(dV);
  p.lse2 = lse2;
  p.delta = delta;
  p.B = B;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.Sq = Sq;
  p.Sk = Sk;
  p.causal = causal ? 1 : 0;
  p.shift = Sk > Sq ? Sk - Sq : 0;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  const int smem_dq = attn_bwd_tc::SMEM_DQ + 1024, smem_dkv = attn_bwd_tc::SMEM_DKV + 1024;
  TSB_CUDA_OK(cudaFuncSetAttribute(attn_bwd_tc::dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_dq));
  TSB_CUDA_OK(cudaFuncSetAttribute(attn_bwd_tc::dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_dkv));
  dim3 g1((Sq + attn_bwd_tc::BLK - 1) / attn_bwd_tc::BLK, Hq, B);
  attn_bwd_tc::dq_kernel<<<g1, attn_bwd_tc::THREADS, smem_dq, st>>>(p);
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  dim3 g2((Sk + attn_bwd_tc::BLK - 1) / attn_bwd_tc::BLK, Hkv, B);
  attn_bwd_tc::dkv_kernel<<<g2, attn_bwd_tc::THREADS, smem_dkv, st>>>(p);
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  return kOk;
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
