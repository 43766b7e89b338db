// Flash-attention backward (the VJP of attention): (dO, Q, K, V [, bias]) -> (dQ, dK, dV).
//
// Contract of the reference's CUDA lane (python/tessera/compiler/emit/nvidia_cuda.py:590-635,
// entry tessera_nvidia_flash_attn_bwd; checked by
// tests/device/nvidia/test_flash_attention_backward.py:23-50): with
//     raw = scale * q.k + bias[b, hq, m, n];   s = softcap * tanh(raw / softcap) when softcap > 0
//     key n is legal for query m unless (causal && n > m + causal_shift)
//                                    || (wl >= 0 && n < m - wl) || (wr >= 0 && n > m + wr)
//     p = softmax over the legal keys of s;   delta = sum_n p_n (dO . v_n);   hk = hq / (Hq / Hkv)
//     ds_n = p_n (dO . v_n - delta) (1 - tanh^2(raw / softcap));
//     dQ[m] = sum_n ds_n scale k_n;   dK[n] = sum_{hq in group, m} ds_n scale q_m;
//     dV[n] = sum_{hq in group, m} p_n dO_m;   a row with no legal key contributes nothing.
// fp32 math on f32 / f16 / bf16 storage, gradients returned in the storage type. The reference
// accumulates dK and dV with atomics (or a two-way split and reduce); here every output row is
// owned by one warp and summed in a fixed order, so the result is deterministic and needs no
// zero-fill:
//   * bwd_dq_kernel, one warp per query row: pass 1 over the keys builds the softmax statistics
//     (max, sum) and delta online and saves them (3 floats per row, the workspace); pass 2 forms ds
//     and accumulates dQ with lanes owning output columns, so K rows are read coalesced.
//   * bwd_dkv_kernel, one warp per key row: walks the legal query rows of every query head of its
//     group, recomputes p and ds from the saved statistics and accumulates dK and dV the same way.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cmath>

#include "../../include/tessera_sm100.h"
#include "device_ctx.h"

namespace tsb {
namespace attn_bwd {

constexpr int WARPS = 4;
constexpr int MAX_D = 256;         // the reference's TSR_FA_CAP
constexpr int NACC = MAX_D / 32;

struct Params {
  long long B, Sq, Sk;
  int Hq, Hkv, D, Dv;
  float scale, softcap;
  int causal;
  long long causal_shift, wl, wr;
};

template <typename T>
__device__ __forceinline__ float ld(const T* p) { return static_cast<float>(*p); }

// s (after bias and soft-cap) and d s / d raw for one (query row, key) pair
__device__ __forceinline__ void cap_score(float raw, float cap, float& s, float& deriv) {
  s = raw;
  deriv = 1.f;
  if (cap > 0.f) {
    const float t = tanhf(raw / cap);
    s = cap * t;
    deriv = 1.f - t * t;
  }
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
bwd_dq_kernel(const T* __restrict__ go, const T* __restrict__ q, const T* __restrict__ k,
              const T* __restrict__ v, const float* __restrict__ bias, T* __restrict__ dq,
              float* __restrict__ stats, const Params p) {
  extern __shared__ float smem[];  // per warp: the query row (D) and the dO row (Dv)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * WARPS + warp;
  const long long total = p.B * p.Hq * p.Sq;
  if (row >= total) return;  // whole warp leaves together; no block-wide barrier below
  const long long m = row % p.Sq;
  const long long t = row / p.Sq;
  const int qh = static_cast<int>(t % p.Hq);
  const long long b = t / p.Hq;
  const int hk = qh / (p.Hq / p.Hkv);
  float* qs = smem + warp * (p.D + p.Dv);
  float* gs = qs + p.D;
  for (int d = lane; d < p.D; d += 32) qs[d] = ld(q + row * p.D + d);
  for (int d = lane; d < p.Dv; d += 32) gs[d] = ld(go + row * p.Dv + d);
  __syncwarp();
  const T* kbase = k + (b * p.Hkv + hk) * p.Sk * p.D;
  const T* vbase = v + (b * p.Hkv + hk) * p.Sk * p.Dv;
  const float* brow = bias ? bias + row * p.Sk : nullptr;
  long long lo = 0, hi = p.Sk - 1;  // keys outside [lo, hi] are illegal for this row
  if (p.causal) hi = min(hi, m + p.causal_shift);
  if (p.wl >= 0) lo = max(lo, m - p.wl);
  if (p.wr >= 0) hi = min(hi, m + p.wr);

  auto score = [&](long long n, float& s, float& deriv, float& dp) {
    const T* kr = kbase + n * p.D;
    float dot = 0.f;
    for (int d = 0; d < p.D; ++d) dot += qs[d] * ld(kr + d);
    float raw = dot * p.scale;
    if (brow) raw += brow[n];
    cap_score(raw, p.softcap, s, deriv);
    const T* vr = vbase + n * p.Dv;
    dp = 0.f;
    for (int d = 0; d < p.Dv; ++d) dp += gs[d] * ld(vr + d);
  };

  // pass 1: max, sum of exponentials, sum of exponentials times (dO . v)
  float mx = -INFINITY, z = 0.f, num = 0.f;
  for (long long n0 = (lo / 32) * 32; n0 <= hi; n0 += 32) {
    const long long n = n0 + lane;
    const bool live = n >= lo && n <= hi;
    float s = -INFINITY, deriv = 1.f, dp = 0.f;
    if (live) score(n, s, deriv, dp);
    float cmax = s;
#pragma unroll
    for (int sh = 16; sh; sh >>= 1) cmax = fmaxf(cmax, __shfl_xor_sync(0xffffffffu, cmax, sh));
    if (cmax == -INFINITY) continue;  // uniform across the warp
    const float mn = fmaxf(mx, cmax);
    const float corr = expf(mx - mn);  // exp(-inf) = 0 on the first live chunk
    const float e = live ? expf(s - mn) : 0.f;
    float es = e, en = e * dp;
#pragma unroll
    for (int sh = 16; sh; sh >>= 1) {
      es += __shfl_xor_sync(0xffffffffu, es, sh);
      en += __shfl_xor_sync(0xffffffffu, en, sh);
    }
    z = z * corr + es;
    num = num * corr + en;
    mx = mn;
  }
  const float inv_z = z > 0.f ? 1.f / z : 0.f;
  const float delta = num * inv_z;
  if (lane == 0) {
    stats[row * 3] = mx;
    stats[row * 3 + 1] = inv_z;
    stats[row * 3 + 2] = delta;
  }

  // pass 2: dQ[m] = sum_n ds_n scale k_n, lanes own columns (lane, lane + 32, ...)
  float acc[NACC];
#pragma unroll
  for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
  if (z > 0.f) {
    for (long long n0 = (lo / 32) * 32; n0 <= hi; n0 += 32) {
      const long long n = n0 + lane;
      const bool live = n >= lo && n <= hi;
      float w = 0.f;
      if (live) {
        float s, deriv, dp;
        score(n, s, deriv, dp);
        const float pn = expf(s - mx) * inv_z;
        w = pn * (dp - delta) * deriv * p.scale;
      }
      const int jmax = static_cast<int>(min(32ll, p.Sk - n0));
      for (int j = 0; j < jmax; ++j) {
        const float wj = __shfl_sync(0xffffffffu, w, j);
        if (wj == 0.f) continue;  // uniform
        const T* kr = kbase + (n0 + j) * p.D;
#pragma unroll
        for (int i = 0; i < NACC; ++i) {
          const int d = lane + 32 * i;
          if (d < p.D) acc[i] += wj * ld(kr + d);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NACC; ++i) {
    const int d = lane + 32 * i;
    if (d < p.D) dq[row * p.D + d] = static_cast<T>(acc[i]);
  }
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
bwd_dkv_kernel(const T* __restrict__ go, const T* __restrict__ q, const T* __restrict__ k,
               const T* __restrict__ v, const float* __restrict__ bias, T* __restrict__ dk,
               T* __restrict__ dv, const float* __restrict__ stats, const Params p) {
  extern __shared__ float smem[];  // per warp: the key row (D) and the value row (Dv)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = static_cast<long long>(blockIdx.x) * WARPS + warp;
  const long long total = p.B * p.Hkv * p.Sk;
  if (item >= total) return;
  const long long n = item % p.Sk;
  const long long t = item / p.Sk;
  const int hk = static_cast<int>(t % p.Hkv);
  const long long b = t / p.Hkv;
  const int ratio = p.Hq / p.Hkv;
  float* ks = smem + warp * (p.D + p.Dv);
  float* vs = ks + p.D;
  for (int d = lane; d < p.D; d += 32) ks[d] = ld(k + item * p.D + d);
  for (int d = lane; d < p.Dv; d += 32) vs[d] = ld(v + item * p.Dv + d);
  __syncwarp();
  // query rows for which key n is legal: [mlo, mhi]
  long long mlo = 0, mhi = p.Sq - 1;
  if (p.causal) mlo = max(mlo, n - p.causal_shift);
  if (p.wr >= 0) mlo = max(mlo, n - p.wr);
  if (p.wl >= 0) mhi = min(mhi, n + p.wl);

  float ak[NACC], av[NACC];
#pragma unroll
  for (int i = 0; i < NACC; ++i) ak[i] = av[i] = 0.f;
  for (int qh = hk * ratio; qh < (hk + 1) * ratio; ++qh) {
    const long long rbase = (b * p.Hq + qh) * p.Sq;
    for (long long m0 = (mlo / 32) * 32; m0 <= mhi; m0 += 32) {
      const long long m = m0 + lane;
      const bool live = m >= mlo && m <= mhi;
      float pn = 0.f, w = 0.f;
      if (live) {
        const long long row = rbase + m;
        const float inv_z = stats[row * 3 + 1];
        if (inv_z > 0.f) {
          const T* qr = q + row * p.D;
          float dot = 0.f;
          for (int d = 0; d < p.D; ++d) dot += ks[d] * ld(qr + d);
          float raw = dot * p.scale;
          if (bias) raw += bias[row * p.Sk + n];
          float s, deriv;
          cap_score(raw, p.softcap, s, deriv);
          const T* gr = go + row * p.Dv;
          float dp = 0.f;
          for (int d = 0; d < p.Dv; ++d) dp += vs[d] * ld(gr + d);
          pn = expf(s - stats[row * 3]) * inv_z;
          w = pn * (dp - stats[row * 3 + 2]) * deriv * p.scale;
        }
      }
      const int jmax = static_cast<int>(min(32ll, p.Sq - m0));
      for (int j = 0; j < jmax; ++j) {
        const float pj = __shfl_sync(0xffffffffu, pn, j);
        const float wj = __shfl_sync(0xffffffffu, w, j);
        if (pj == 0.f && wj == 0.f) continue;  // uniform
        const T* qr = q + (rbase + m0 + j) * p.D;
        const T* gr = go + (rbase + m0 + j) * p.Dv;
#pragma unroll
        for (int i = 0; i < NACC; ++i) {
          const int d = lane + 32 * i;
          if (d < p.D) ak[i] += wj * ld(qr + d);
          if (d < p.Dv) av[i] += pj * ld(gr + d);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NACC; ++i) {
    const int d = lane + 32 * i;
    if (d < p.D) dk[item * p.D + d] = static_cast<T>(ak[i]);
    if (d < p.Dv) dv[item * p.Dv + d] = static_cast<T>(av[i]);
  }
}

template <typename T>
int launch_t(const void* go, const void* q, const void* k, const void* v, const float* bias,
             void* dq, void* dk, void* dv, float* stats, const Params& p, cudaStream_t st) {
  const long long rows = p.B * p.Hq * p.Sq, items = p.B * p.Hkv * p.Sk;
  const long long b1 = (rows + WARPS - 1) / WARPS, b2 = (items + WARPS - 1) / WARPS;
  if (b1 > 0x7fffffffLL || b2 > 0x7fffffffLL) {
    set_last_error("flash_attn_bwd: too many rows for one launch");
    return kBadArg;
  }
  const size_t smem = WARPS * (p.D + p.Dv) * sizeof(float);
  bwd_dq_kernel<T><<<static_cast<unsigned>(b1), WARPS * 32, smem, st>>>(
      static_cast<const T*>(go), static_cast<const T*>(q), static_cast<const T*>(k),
      static_cast<const T*>(v), bias, static_cast<T*>(dq), stats, p);
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  bwd_dkv_kernel<T><<<static_cast<unsigned>(b2), WARPS * 32, smem, st>>>(
      static_cast<const T*>(go), static_cast<const T*>(q), static_cast<const T*>(k),
      static_cast<const T*>(v), bias, static_cast<T*>(dk), static_cast<T*>(dv), stats, p);
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  return kOk;
}

int check(const void* go, const void* q, const void* k, const void* v, const void* dq,
          const void* dk, const void* dv, long long B, int Hq, int Hkv, long long Sq, long long Sk,
          int D, int Dv, long long wl, long long wr, float softcap) {
  if (!go || !q || !k || !v || !dq || !dk || !dv || B <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv ||
      Sq <= 0 || Sk <= 0 || D <= 0 || Dv <= 0) {
    set_last_error("flash_attn_bwd: null pointer, non-positive size or Hq not divisible by Hkv");
    return kBadArg;
  }
  if (D > MAX_D || Dv > MAX_D) {
    set_last_error("flash_attn_bwd: head dimensions up to %d are served (got D=%d Dv=%d)", MAX_D, D, Dv);
    return kBadArg;
  }
  if (wl < -1 || wr < -1 || softcap < 0.f) {
    set_last_error("flash_attn_bwd: window bounds must be >= 0 (or -1 for none) and softcap >= 0");
    return kBadArg;
  }
  return kOk;
}

}  // namespace attn_bwd
}  // namespace tsb

using namespace tsb;

extern "C" {

size_t tessera_sm100_flash_attn_bwd_workspace_bytes(long long B, int Hq, long long Sq) {
  if (B <= 0 || Hq <= 0 || Sq <= 0) return 0;
  return static_cast<size_t>(B) * Hq * Sq * 3 * sizeof(float);
}

int tessera_sm100_flash_attn_bwd_device(const void* dO, const void* Q, const void* K, const void* V,
                                        const float* bias, void* dQ, void* dK, void* dV, long long B,
                                        int Hq, int Hkv, long long Sq, long long Sk, int D, int Dv,
                                        float scale, int causal, long long causal_shift,
                                        long long window_left, long long window_right, float softcap,
                                        int dtype, void* workspace, void* stream) {
  if (int rc = attn_bwd::check(dO, Q, K, V, dQ, dK, dV, B, Hq, Hkv, Sq, Sk, D, Dv, window_left,
                               window_right, softcap))
    return rc;
  if (!workspace) {
    set_last_error("flash_attn_bwd: workspace of tessera_sm100_flash_attn_bwd_workspace_bytes is required");
    return kBadArg;
  }
  if (int rc = ensure_device()) return rc;
  attn_bwd::Params p{};
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
  float* stats = static_cast<float*>(workspace);
  switch (dtype) {
    case TESSERA_SM100_F32:
      return attn_bwd::launch_t<float>(dO, Q, K, V, bias, dQ, dK, dV, stats, p, st);
    case TESSERA_SM100_F16:
      return attn_bwd::launch_t<__half>(dO, Q, K, V, bias, dQ, dK, dV, stats, p, st);
    case TESSERA_SM100_BF16:
      return attn_bwd::launch_t<__nv_bfloat16>(dO, Q, K, V, bias, dQ, dK, dV, stats, p, st);
    default: break;
  }
  set_last_error("flash_attn_bwd: unsupported dtype %d", dtype);
  return kBadArg;
}

// Host-pointer form with the argument order of the reference's entry
// (tessera_nvidia_flash_attn_bwd, python/tessera/compiler/emit/nvidia_cuda.py:611): uploads,
// runs, downloads. causal is the lane's top-left mask (key n > query m).
int tessera_sm100_flash_attn_bwd(const void* dO, const void* Q, const void* K, const void* V,
                                 const float* bias, void* dQ, void* dK, void* dV, long long B, int Hq,
                                 int Hkv, long long Sq, long long Sk, int D, int Dv, float scale,
                                 int causal, long long window_left, long long window_right,
                                 float softcap, int dtype) {
  if (int rc = attn_bwd::check(dO, Q, K, V, dQ, dK, dV, B, Hq, Hkv, Sq, Sk, D, Dv, window_left,
                               window_right, softcap))
    return rc;
  if (dtype != TESSERA_SM100_F32 && dtype != TESSERA_SM100_F16 && dtype != TESSERA_SM100_BF16) {
    set_last_error("flash_attn_bwd: unsupported dtype %d", dtype);
    return kBadArg;
  }
  if (int rc = ensure_device()) return rc;
  const size_t es = dtype == TESSERA_SM100_F32 ? 4 : 2;
  const size_t nq = (size_t)B * Hq * Sq * D * es, nk = (size_t)B * Hkv * Sk * D * es;
  const size_t no = (size_t)B * Hq * Sq * Dv * es, nv = (size_t)B * Hkv * Sk * Dv * es;
  const size_t nb = bias ? (size_t)B * Hq * Sq * Sk * 4 : 0;
  const size_t nw = tessera_sm100_flash_attn_bwd_workspace_bytes(B, Hq, Sq);
  auto up = [](size_t n) { return (n + 255) & ~size_t(255); };
  const size_t total = up(no) + 2 * up(nq) + 2 * up(nk) + 2 * up(nv) + up(nb) + up(nw);
  char* base = nullptr;
  TSB_CUDA_OK(cudaMalloc(&base, total));
  char* cur = base;
  auto take = [&](size_t n) { char* r = cur; cur += up(n); return r; };
  char *d_go = take(no), *d_q = take(nq), *d_k = take(nk), *d_v = take(nv), *d_dq = take(nq),
       *d_dk = take(nk), *d_dv = take(nv), *d_b = take(nb), *d_w = take(nw);
  int rc = kOk;
  cudaError_t ce = cudaMemcpy(d_go, dO, no, cudaMemcpyHostToDevice);
  if (ce == cudaSuccess) ce = cudaMemcpy(d_q, Q, nq, cudaMemcpyHostToDevice);
  if (ce == cudaSuccess) ce = cudaMemcpy(d_k, K, nk, cudaMemcpyHostToDevice);
  if (ce == cudaSuccess) ce = cudaMemcpy(d_v, V, nv, cudaMemcpyHostToDevice);
  if (ce == cudaSuccess && bias) ce = cudaMemcpy(d_b, bias, nb, cudaMemcpyHostToDevice);
  if (ce == cudaSuccess) {
    rc = tessera_sm100_flash_attn_bwd_device(d_go, d_q, d_k, d_v, bias ? reinterpret_cast<float*>(d_b) : nullptr,
                                             d_dq, d_dk, d_dv, B, Hq, Hkv, Sq, Sk, D, Dv, scale, causal, 0,
                                             window_left, window_right, softcap, dtype, d_w, nullptr);
    if (rc == kOk) ce = cudaDeviceSynchronize();
  }
  if (rc == kOk && ce == cudaSuccess) ce = cudaMemcpy(dQ, d_dq, nq, cudaMemcpyDeviceToHost);
  if (rc == kOk && ce == cudaSuccess) ce = cudaMemcpy(dK, d_dk, nk, cudaMemcpyDeviceToHost);
  if (rc == kOk && ce == cudaSuccess) ce = cudaMemcpy(dV, d_dv, nv, cudaMemcpyDeviceToHost);
  cudaFree(base);
  if (rc != kOk) return rc;
  if (ce != cudaSuccess) {
    set_last_error("flash_attn_bwd: CUDA error %s", cudaGetErrorString(ce));
    return kDeviceFailed;
  }
  return kOk;
}

}  // extern "C"
