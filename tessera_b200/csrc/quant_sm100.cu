// Per-tensor symmetric fp8 (e4m3) quantisation on the device, with the arithmetic of the
// reference's quantize_fp8 (python/tessera/__init__.py:3340-3374), all in fp32:
//     scale = max(amax(|x|) / 448, 1e-12);   q = e4m3(clip(x / scale, -448, 448))   (round to
//     nearest even);   dequantised value = q * scale.
// The grouped fp8 GEMMs take q and apply the scales in their epilogue.
//
// Weights [E, K, N] are quantised per expert (python/tessera/compiler/grouped_layout.py:371-392) and
// written TRANSPOSED as [E, N, K] so that both GEMM operands are K-major.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <algorithm>

#include "../../include/tessera_sm100.h"
#include "device_ctx.h"

namespace tsb {
namespace quant {

template <typename T>
__device__ __forceinline__ float to_f32(T v) { return static_cast<float>(v); }

__device__ __forceinline__ float scale_from_amax(float amax) {
  return fmaxf(__fdiv_rn(amax, 448.0f), 1e-12f);
}
__device__ __forceinline__ uint8_t to_e4m3(float x, float scale) {
  return __nv_cvt_float_to_fp8(__fdiv_rn(x, scale), __NV_SATFINITE, __NV_E4M3);
}

// amax over n elements of segment blockIdx.y (segments of `seg` elements): non-negative float
// bits combine with an integer max.
template <typename T>
__global__ void amax_kernel(const T* __restrict__ x, long long seg, unsigned int* __restrict__ out) {
  const T* xs = x + static_cast<long long>(blockIdx.y) * seg;
  float a = 0.f;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < seg;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    a = fmaxf(a, fabsf(to_f32(xs[i])));
#pragma unroll
  for (int sh = 16; sh; sh >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, sh));
  if ((threadIdx.x & 31) == 0 && a > 0.f) atomicMax(out + blockIdx.y, __float_as_uint(a));
}

// q[i] = e4m3(x[i] / scale); thread 0 also publishes scale_out[0] = scale, scale_out[1] = amax.
template <typename T>
__global__ void quantize_kernel(const T* __restrict__ x, long long n,
                                const unsigned int* __restrict__ amax_bits,
                                uint8_t* __restrict__ q, float* __restrict__ scale_out) {
  const float amax = __uint_as_float(*amax_bits);
  const float scale = scale_from_amax(amax);
  if (blockIdx.x == 0 && threadIdx.x == 0 && scale_out) {
    scale_out[0] = scale;
    scale_out[1] = amax;
  }
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    q[i] = to_e4m3(to_f32(x[i]), scale);
}

// w[e][k][n] -> q_t[e][n][k] through a 32 x 32 shared-memory tile (both sides coalesced);
// scales[e] = scale, scales[E + e] = amax.
template <typename T>
__global__ void quantize_transpose_kernel(const T* __restrict__ w, int K, int N, int E,
                                          const unsigned int* __restrict__ amax_bits,
                                          uint8_t* __restrict__ q_t, float* __restrict__ scales) {
  __shared__ float tile[32][33];
  const int e = blockIdx.z;
  const float amax = __uint_as_float(amax_bits[e]);
  const float scale = scale_from_amax(amax);
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0 && threadIdx.y == 0) {
    scales[e] = scale;
    scales[E + e] = amax;
  }
  const T* we = w + static_cast<long long>(e) * K * N;
  uint8_t* qe = q_t + static_cast<long long>(e) * K * N;
  const int n0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int k = k0 + r, n = n0 + threadIdx.x;
    tile[r][threadIdx.x] = (k < K && n < N) ? to_f32(we[static_cast<long long>(k) * N + n]) : 0.f;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int n = n0 + r, k = k0 + threadIdx.x;
    if (n < N && k < K) qe[static_cast<long long>(n) * K + k] = to_e4m3(tile[threadIdx.x][r], scale);
  }
}

template <typename T>
int quantize_t(const void* x, long long n, void* q, float* scale_out, unsigned int* amax_bits,
               bool have_amax, cudaStream_t st) {
  const int blocks = (int)std::min<long long>((n + 255) / 256, 148 * 8);
  if (!have_amax) {
    TSB_CUDA_OK(cudaMemsetAsync(amax_bits, 0, sizeof(unsigned int), st));
    amax_kernel<T><<<dim3(blocks, 1), 256, 0, st>>>(static_cast<const T*>(x), n, amax_bits);
    TSB_CUDA_OK(cudaGetLastError());
    note_launch();
  }
  quantize_kernel<T><<<blocks, 256, 0, st>>>(static_cast<const T*>(x), n, amax_bits,
                                            static_cast<uint8_t*>(q), scale_out);
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  return kOk;
}

template <typename T>
int quantize_weights_t(const void* w, int E, int K, int N, void* q_t, float* scales,
                       cudaStream_t st) {
  // the amax words live in the caller's scales buffer: [2E, 3E) as uint32
  unsigned int* amax_bits = reinterpret_cast<unsigned int*>(scales + 2 * E);
  TSB_CUDA_OK(cudaMemsetAsync(amax_bits, 0, sizeof(unsigned int) * E, st));
  const long long seg = static_cast<long long>(K) * N;
  const int blocks = (int)std::min<long long>((seg + 255) / 256, 148 * 4);
  amax_kernel<T><<<dim3(blocks, E), 256, 0, st>>>(static_cast<const T*>(w), seg, amax_bits);
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  dim3 grid((N + 31) / 32, (K + 31) / 32, E);
  quantize_transpose_kernel<T><<<grid, dim3(32, 8), 0, st>>>(static_cast<const T*>(w), K, N, E, amax_bits,
                                                            static_cast<uint8_t*>(q_t), scales);
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  return kOk;
}

}  // namespace quant
}  // namespace tsb

using namespace tsb;

extern "C" {

// x (n elements, dtype code) -> q (n bytes, e4m3). scale_out: 3 device floats — [0] scale,
// [1] amax, [2] scratch. With amax_in != NULL (a device uint32 holding the bits of a non-negative
// float, e.g. the amax the fused SwiGLU GEMM recorded) the amax pass is skipped.
int tessera_sm100_quantize_fp8_device(const void* x, long long n, int dtype, void* q,
                                      float* scale_out, const unsigned int* amax_in, void* stream) {
  if (!x || !q || !scale_out || n < 0) {
    set_last_error("quantize_fp8: null pointer or negative size");
    return kBadArg;
  }
  if (n == 0) return kOk;
  if (int rc = ensure_device()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned int* bits = amax_in ? const_cast<unsigned int*>(amax_in)
                               : reinterpret_cast<unsigned int*>(scale_out + 2);
  const bool have = amax_in != nullptr;
  switch (dtype) {
    case TESSERA_SM100_F32: return quant::quantize_t<float>(x, n, q, scale_out, bits, have, st);
    case TESSERA_SM100_BF16: return quant::quantize_t<__nv_bfloat16>(x, n, q, scale_out, bits, have, st);
    case TESSERA_SM100_F16: return quant::quantize_t<__half>(x, n, q, scale_out, bits, have, st);
    default: break;
  }
  set_last_error("quantize_fp8: unsupported dtype %d", dtype);
  return kBadArg;
}

// w [E, K, N] -> q_t [E, N, K] e4m3 with one scale per expert. scales: 3E device floats — [0, E)
// scales, [E, 2E) amax, [2E, 3E) scratch.
int tessera_sm100_quantize_fp8_weights_device(const void* w, int E, int K, int N, int dtype,
                                              void* q_t, float* scales, void* stream) {
  if (!w || !q_t || !scales || E <= 0 || K <= 0 || N <= 0) {
    set_last_error("quantize_fp8_weights: null pointer or non-positive size");
    return kBadArg;
  }
  if (int rc = ensure_device()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case TESSERA_SM100_F32: return quant::quantize_weights_t<float>(w, E, K, N, q_t, scales, st);
    case TESSERA_SM100_BF16: return quant::quantize_weights_t<__nv_bfloat16>(w, E, K, N, q_t, scales, st);
    case TESSERA_SM100_F16: return quant::quantize_weights_t<__half>(w, E, K, N, q_t, scales, st);
    default: break;
  }
  set_last_error("quantize_fp8_weights: unsupported dtype %d", dtype);
  return kBadArg;
}

}  // extern "C"
