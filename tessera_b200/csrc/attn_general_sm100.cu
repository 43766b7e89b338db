// General flash-attention forward: any head dimension (D, Dv <= 512), f32 / f16 / bf16 storage,
// optional additive bias, causal mask, sliding window and logit soft-cap.
//
// This is the contract of the reference's CUDA attention lane
// (python/tessera/compiler/emit/nvidia_cuda.py:251-276; checked by
// tests/device/nvidia/test_flash_attention.py:23-58):
//     s = scale * q . k  (+ bias[b, hq, m, n])
//     s = softcap * tanh(s / softcap)                       when softcap > 0
//     key n is masked for query m when  (causal && n > m + causal_shift)
//                                     || (wl >= 0 && n < m - wl) || (wr >= 0 && n > m + wr)
//     O = softmax(s) V, fp32 math, a fully masked row gives zeros; hk = hq / (Hq / Hkv)
// causal_shift = 0 is the lane's top-left mask; tessera.ops.flash_attn's bottom-right alignment
// (python/tessera/__init__.py:1344-1349) is causal_shift = max(Sk - Sq, 0).
//
// The D = 128 bf16 shapes of the benchmark configurations run on the tcgen05 prefill kernel and
// the split-KV decode kernel; this kernel serves everything else, so no shape falls back to
// the host. One warp per query row: the query sits in shared memory, each lane scores one key
// of a 32-key chunk, the online-softmax state is per warp, and lanes own output columns
// (lane, lane + 32, ...) so V rows are read coalesced.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cmath>

#include "../../include/tessera_sm100.h"
#include "device_ctx.h"

namespace tsb {
namespace attn_general {

constexpr int WARPS = 4;
constexpr int MAX_D = 512;

struct Params {
  long long B, Sq, Sk;
  int Hq, Hkv, D, Dv;
  float scale, softcap;
  int causal;
  long long causal_shift, wl, wr;
};

template <typename T>
__device__ __forceinline__ float ld(const T* p) { return static_cast<float>(*p); }

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attn_general_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                    const float* __restrict__ bias, T* __restrict__ o, const Params p) {
  extern __shared__ float smem[];  // [WARPS][D] query rows
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * WARPS + warp;
  const long long total = p.B * p.Hq * p.Sq;
  if (row >= total) return;  // whole warp leaves together; no block-wide barrier below
  const long long m = row % p.Sq;
  const long long t = row / p.Sq;
  const int qh = static_cast<int>(t % p.Hq);
  const long long b = t / p.Hq;
  const int hk = qh / (p.Hq / p.Hkv);
  float* qs = smem + warp * p.D;
  const T* qrow = q + ((b * p.Hq + qh) * p.Sq + m) * p.D;
  for (int d = lane; d < p.D; d += 32) qs[d] = ld(qrow + d);
  __syncwarp();
  const T* kbase = k + (b * p.Hkv + hk) * p.Sk * p.D;
  const T* vbase = v + (b * p.Hkv + hk) * p.Sk * p.Dv;
  const float* brow = bias ? bias + ((b * p.Hq + qh) * p.Sq + m) * p.Sk : nullptr;

  constexpr int NACC = MAX_D / 32;
  float acc[NACC];
#pragma unroll
  for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
  float mi = -INFINITY, li = 0.f;
  // keys outside [lo, hi] are masked for this row
  long long lo = 0, hi = p.Sk - 1;
  if (p.causal) hi = min(hi, m + p.causal_shift);
  if (p.wl >= 0) lo = max(lo, m - p.wl);
  if (p.wr >= 0) hi = min(hi, m + p.wr);

  for (long long n0 = (lo / 32) * 32; n0 <= hi; n0 += 32) {
    const long long n = n0 + lane;
    const bool live = n >= lo && n <= hi;
    float s = -INFINITY;
    if (live) {
      const T* kr = kbase + n * p.D;
      float dot = 0.f;
      for (int d = 0; d < p.D; ++d) dot += qs[d] * ld(kr + d);
      s = dot * p.scale;
      if (brow) s += brow[n];
      if (p.softcap > 0.f) s = p.softcap * tanhf(s / p.softcap);
    }
    float cmax = s;
#pragma unroll
    for (int sh = 16; sh; sh >>= 1) cmax = fmaxf(cmax, __shfl_xor_sync(0xffffffffu, cmax, sh));
    if (cmax == -INFINITY) continue;  // nothing live in this chunk (uniform across the warp)
    const float mn = fmaxf(mi, cmax);
    const float corr = expf(mi - mn);  // exp(-inf) = 0 on the first live chunk
    const float pj = live ? expf(s - mn) : 0.f;
    float psum = pj;
#pragma unroll
    for (int sh = 16; sh; sh >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, sh);
    li = li * corr + psum;
    mi = mn;
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] *= corr;
    const int jmax = static_cast<int>(min(32ll, p.Sk - n0));
    for (int j = 0; j < jmax; ++j) {
      const float w = __shfl_sync(0xffffffffu, pj, j);
      if (w == 0.f) continue;  // uniform: every lane sees the same w
      const T* vr = vbase + (n0 + j) * p.Dv;
#pragma unroll
      for (int i = 0; i < NACC; ++i) {
        const int d = lane + 32 * i;
        if (d < p.Dv) acc[i] += w * ld(vr + d);
      }
    }
  }
  const float inv = li > 0.f ? 1.f / li : 0.f;
  T* orow = o + ((b * p.Hq + qh) * p.Sq + m) * p.Dv;
#pragma unroll
  for (int i = 0; i < NACC; ++i) {
    const int d = lane + 32 * i;
    if (d < p.Dv) orow[d] = static_cast<T>(acc[i] * inv);
  }
}

template <typename T>
int launch_t(const void* q, const void* k, const void* v, const float* bias, void* o,
             const Params& p, cudaStream_t st) {
  const long long rows = p.B * p.Hq * p.Sq;
  const long long blocks = (rows + WARPS - 1) / WARPS;
  if (blocks > 0x7fffffffLL) {
    set_last_error("flash_attn_general: too many query rows for one launch");
    return kBadArg;
  }
  attn_general_kernel<T><<<static_cast<unsigned>(blocks), WARPS * 32, WARPS * p.D * sizeof(float), st>>>(
      static_cast<const T*>(q), static_cast<const T*>(k), static_cast<const T*>(v), bias,
      static_cast<T*>(o), p);
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  return kOk;
}

}  // namespace attn_general
}  // namespace tsb

using namespace tsb;

extern "C" int tessera_sm100_flash_attn_general_device(
    const void* q, const void* k, const void* v, const float* bias, void* o, long long B, int Hq,
    int Hkv, long long Sq, long long Sk, int D, int Dv, float scale, int causal,
    long long causal_shift, long long window_left, long long window_right, float softcap, int dtype,
    void* stream) {
  if (!q || !k || !v || !o || B <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv || Sq <= 0 || Sk <= 0 ||
      D <= 0 || Dv <= 0) {
    set_last_error("flash_attn_general: null pointer, non-positive size or Hq not divisible by Hkv");
    return kBadArg;
  }
  if (D > attn_general::MAX_D || Dv > attn_general::MAX_D) {
    set_last_error("flash_attn_general: head dimensions up to %d are served (got D=%d Dv=%d)",
                   attn_general::MAX_D, D, Dv);
    return kBadArg;
  }
  if (int rc = ensure_device()) return rc;
  attn_general::Params p{};
  p.B = B;
  p.Sq = Sq;
  p.Sk = Sk;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.D = D;
  p.Dv = Dv;
  p.scale = scale;
  p.softcap = softcap;
  p.causal = causal ? 1 : 0;
  p.causal_shift = causal_shift;
  p.wl = window_left;
  p.wr = window_right;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case TESSERA_SM100_F32: return attn_general::launch_t<float>(q, k, v, bias, o, p, st);
    case TESSERA_SM100_F16: return attn_general::launch_t<__half>(q, k, v, bias, o, p, st);
    case TESSERA_SM100_BF16: return attn_general::launch_t<__nv_bfloat16>(q, k, v, bias, o, p, st);
    default: break;
  }
  set_last_error("flash_attn_general: unsupported dtype %d", dtype);
  return kBadArg;
}
