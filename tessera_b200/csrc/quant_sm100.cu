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

// fmt: 0 = e4m3 (largest finite value 448), 1 = e5m2 (57344); the same arithmetic otherwise
__device__ __forceinline__ float scale_from_amax(float amax, int fmt) {
  return fmaxf(__fdiv_rn(amax, fmt ? 57344.0f : 448.0f), 1e-12f);
}
__device__ __forceinline__ uint8_t to_e4m3(float x, float scale, int fmt) {
  const float v = __fdiv_rn(x, scale);
  return fmt ? __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E5M2) : __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}

// amax over n elements of segment blockIdx.y (segments of `seg` elements): non-negative float
// bits combine with an integer max.
template <typename T>
__global__ void amax_kernel(const T* __restrict__ x, long long seg, unsigned int* __restrict__ out) {
  const T* xs = x + static_cast<long long>(blockIdx.y) * seg;
  float a = 0.f;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  constexpr int kVec = 16 / sizeof(T);   // elements per 16-byte load
  const long long nv = (reinterpret_cast<uintptr_t>(xs) & 15) ? 0 : seg / kVec;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nv; i += stride) {
    const uint4 w = reinterpret_cast<const uint4*>(xs)[i];
    const T* h = reinterpret_cast<const T*>(&w);
#pragma unroll
    for (int j = 0; j < kVec; ++j) a = fmaxf(a, fabsf(to_f32(h[j])));
  }
  for (long long i = nv * kVec + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < seg; i += stride)
    a = fmaxf(a, fabsf(to_f32(xs[i])));
#pragma unroll
  for (int sh = 16; sh; sh >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, sh));
  if ((threadIdx.x & 31) == 0 && a > 0.f) atomicMax(out + blockIdx.y, __float_as_uint(a));
}

// q[i] = e4m3(x[i] / scale); thread 0 also publishes scale_out[0] = scale, scale_out[1] = amax.
template <typename T>
__global__ void quantize_kernel(const T* __restrict__ x, long long n,
                                const unsigned int* __restrict__ amax_bits,
                                uint8_t* __restrict__ q, float* __restrict__ scale_out, int fmt) {
  const float amax = __uint_as_float(*amax_bits);
  const float scale = scale_from_amax(amax, fmt);
  if (blockIdx.x == 0 && threadIdx.x == 0 && scale_out) {
    scale_out[0] = scale;
    scale_out[1] = amax;
  }
  // four elements per thread and step: one packed 4-byte store (this pass is pure memory traffic)
  const long long n4 = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(q)) & 15) ? 0 : n / 4;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
    float v[4];
    if constexpr (sizeof(T) == 4) {
      const float4 f = reinterpret_cast<const float4*>(x)[i];
      v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    } else {
      const uint2 w = reinterpret_cast<const uint2*>(x)[i];
      const T* h = reinterpret_cast<const T*>(&w);
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = to_f32(h[j]);
    }
    uint32_t packed = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) packed |= static_cast<uint32_t>(to_e4m3(v[j], scale, fmt)) << (8 * j);
    reinterpret_cast<uint32_t*>(q)[i] = packed;
  }
  for (long long i = 4 * n4 + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    q[i] = to_e4m3(to_f32(x[i]), scale, fmt);
}

// w[e][k][n] -> q_t[e][n][k] through a 32 x 32 shared-memory tile (both sides coalesced);
// scales[e] = scale, scales[E + e] = amax.
template <typename T>
__global__ void quantize_transpose_kernel(const T* __restrict__ w, int K, int N, int E,
                                          const unsigned int* __restrict__ amax_bits,
                                          uint8_t* __restrict__ q_t, float* __restrict__ scales, int fmt) {
  __shared__ float tile[32][33];
  const int e = blockIdx.z;
  const float amax = __uint_as_float(amax_bits[e]);
  const float scale = scale_from_amax(amax, fmt);
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
    if (n < N && k < K) qe[static_cast<long long>(n) * K + k] = to_e4m3(tile[threadIdx.x][r], scale, fmt);
  }
}

template <typename T>
int quantize_t(const void* x, long long n, void* q, float* scale_out, unsigned int* amax_bits,
               bool have_amax, cudaStream_t st, int fmt) {
  const int blocks = (int)std::min<long long>((n / 4 + 255) / 256 + 1, 148 * 16);
  if (!have_amax) {
    TSB_CUDA_OK(cudaMemsetAsync(amax_bits, 0, sizeof(unsigned int), st));
    amax_kernel<T><<<dim3(blocks, 1), 256, 0, st>>>(static_cast<const T*>(x), n, amax_bits);
    TSB_CUDA_OK(cudaGetLastError());
    note_launch();
  }
  quantize_kernel<T><<<blocks, 256, 0, st>>>(static_cast<const T*>(x), n, amax_bits,
                                            static_cast<uint8_t*>(q), scale_out, fmt);
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  return kOk;
}

template <typename T>
int quantize_weights_t(const void* w, int E, int K, int N, void* q_t, float* scales,
                       cudaStream_t st, int fmt) {
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
                                                            static_cast<uint8_t*>(q_t), scales, fmt);
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  return kOk;
}

// ---- NVFP4: blocks of 16 along the last axis, e2m1 codes, one e4m3 scale per block --------------
// The arithmetic of the reference's quantize_nvfp4 (python/tessera/__init__.py:3472-3500 ->
// python/tessera/compiler/microscaling.py:319-362), all in fp32:
//     scale = e4m3(max(amax(|block|) / 6, 1e-30))   (round to nearest even, subnormals kept);
//     code  = e2m1(x / (scale == 0 ? 1 : scale))    (round to nearest even, saturating at +-6);
//     dequantised value = e2m1(code) * scale        (so a block whose scale rounds to 0 reads as 0).
// e2m1 magnitudes: 0, 0.5, 1, 1.5, 2, 3, 4, 6 (codes 0..7), sign in bit 3. Two codes per byte,
// the even element in the low nibble.
__device__ __forceinline__ uint8_t to_e2m1(float x) {
  const float a = fabsf(x);
  // ties go to the code with an even mantissa bit: 0.25 -> 0, 0.75 -> 1, 1.25 -> 1, 1.75 -> 2,
  // 2.5 -> 2, 3.5 -> 4, 5 -> 4
  uint8_t c = a <= 0.25f ? 0 : a < 0.75f ? 1 : a <= 1.25f ? 2 : a < 1.75f ? 3 : a <= 2.5f ? 4
            : a < 3.5f ? 5 : a <= 5.0f ? 6 : 7;
  if (!(a == a)) c = 7;  // NaN cannot be stored; keep the sign and saturate
  return static_cast<uint8_t>(c | (x < 0.f ? 8 : 0));
}
__device__ __forceinline__ float from_e2m1(uint8_t c) {
  // magnitudes 0, 0.5, 1, 1.5, 2, 3, 4, 6: exponent field e = bits 1-2, mantissa bit m = bit 0;
  // e == 0 is the subnormal pair {0, 0.5}, otherwise (1 + m/2) * 2^(e-1)
  const int e = (c >> 1) & 3, mb = c & 1;
  const float m = e ? __int_as_float((126 + e) << 23) * (1.f + 0.5f * mb) : 0.5f * mb;
  return (c & 8) ? -m : m;
}
__device__ __forceinline__ float e4m3_to_f32(uint8_t b) {
  return __half2float(__half(__nv_cvt_fp8_to_halfraw(b, __NV_E4M3)));
}

template <typename T>
__global__ void nvfp4_quantize_kernel(const T* __restrict__ x, long long nblocks,
                                      uint8_t* __restrict__ codes, uint8_t* __restrict__ scales) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= nblocks) return;
  float v[16];
  float amax = 0.f;
  // a block is 16 consecutive elements: 16-byte loads when the base allows (cols % 16 == 0 keeps
  // every block 16-element aligned relative to it)
  if ((reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    constexpr int kPer = 16 / sizeof(T);          // elements per 16-byte load
    const uint4* src = reinterpret_cast<const uint4*>(x + i * 16);
#pragma unroll
    for (int q = 0; q < 16 / kPer; ++q) {
      const uint4 w4 = src[q];
      const T* h = reinterpret_cast<const T*>(&w4);
#pragma unroll
      for (int j = 0; j < kPer; ++j) v[q * kPer + j] = to_f32(h[j]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = to_f32(x[i * 16 + j]);
  }
#pragma unroll
  for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(v[j]));
  const uint8_t sb = __nv_cvt_float_to_fp8(fmaxf(__fdiv_rn(amax, 6.0f), 1e-30f), __NV_SATFINITE, __NV_E4M3);
  float sf = e4m3_to_f32(sb);
  if (sf == 0.f) sf = 1.f;
  uint32_t w[2] = {0u, 0u};
#pragma unroll
  for (int j = 0; j < 16; ++j) w[j >> 3] |= static_cast<uint32_t>(to_e2m1(__fdiv_rn(v[j], sf))) << (4 * (j & 7));
  *reinterpret_cast<uint2*>(codes + i * 8) = make_uint2(w[0], w[1]);
  scales[i] = sb;
}

template <typename OutT>
__global__ void nvfp4_dequantize_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ scales,
                                        long long nblocks, OutT* __restrict__ out) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= nblocks) return;
  const uint2 w = *reinterpret_cast<const uint2*>(codes + i * 8);
  const float sf = e4m3_to_f32(scales[i]);
  alignas(16) OutT vals[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const uint32_t word = j < 8 ? w.x : w.y;
    vals[j] = static_cast<OutT>(from_e2m1((word >> (4 * (j & 7))) & 15u) * sf);
  }
  if ((reinterpret_cast<uintptr_t>(out) & 15) == 0) {   // 16-byte stores
    uint4* dst = reinterpret_cast<uint4*>(out + i * 16);
    const uint4* srcv = reinterpret_cast<const uint4*>(vals);
#pragma unroll
    for (int q = 0; q < static_cast<int>(sizeof(OutT)) * 16 / 16; ++q) dst[q] = srcv[q];
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) out[i * 16 + j] = vals[j];
  }
}

// e4m3 bytes -> the same values as bf16 (exact: 4 significant bits into 8)
__global__ void fp8_to_bf16_kernel(const uint8_t* __restrict__ q, long long n, __nv_bfloat16* __restrict__ out,
                                   int fmt) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    out[i] = __float2bfloat16_rn(fmt ? __half2float(__half(__nv_cvt_fp8_to_halfraw(q[i], __NV_E5M2))) : e4m3_to_f32(q[i]));
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
  return tessera_sm100_quantize_fp8_fmt_device(x, n, dtype, TESSERA_SM100_FP8_E4M3, q, scale_out, amax_in, stream);
}
// The same with the 8-bit format as an argument: 0 = e4m3 (scale = amax / 448), 1 = e5m2 (amax / 57344).
int tessera_sm100_quantize_fp8_fmt_device(const void* x, long long n, int dtype, int fmt, void* q,
                                          float* scale_out, const unsigned int* amax_in, void* stream) {
  if (fmt != TESSERA_SM100_FP8_E4M3 && fmt != TESSERA_SM100_FP8_E5M2) {
    set_last_error("quantize_fp8: format must be 0 (e4m3) or 1 (e5m2), got %d", fmt);
    return kBadArg;
  }
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
    case TESSERA_SM100_F32: return quant::quantize_t<float>(x, n, q, scale_out, bits, have, st, fmt);
    case TESSERA_SM100_BF16: return quant::quantize_t<__nv_bfloat16>(x, n, q, scale_out, bits, have, st, fmt);
    case TESSERA_SM100_F16: return quant::quantize_t<__half>(x, n, q, scale_out, bits, have, st, fmt);
    default: break;
  }
  set_last_error("quantize_fp8: unsupported dtype %d", dtype);
  return kBadArg;
}

// w [E, K, N] -> q_t [E, N, K] e4m3 with one scale per expert. scales: 3E device floats — [0, E)
// scales, [E, 2E) amax, [2E, 3E) scratch.
int tessera_sm100_quantize_fp8_weights_device(const void* w, int E, int K, int N, int dtype,
                                              void* q_t, float* scales, void* stream) {
  return tessera_sm100_quantize_fp8_weights_fmt_device(w, E, K, N, dtype, TESSERA_SM100_FP8_E4M3, q_t, scales, stream);
}
int tessera_sm100_quantize_fp8_weights_fmt_device(const void* w, int E, int K, int N, int dtype, int fmt,
                                                  void* q_t, float* scales, void* stream) {
  if (fmt != TESSERA_SM100_FP8_E4M3 && fmt != TESSERA_SM100_FP8_E5M2) {
    set_last_error("quantize_fp8_weights: format must be 0 (e4m3) or 1 (e5m2), got %d", fmt);
    return kBadArg;
  }
  if (!w || !q_t || !scales || E <= 0 || K <= 0 || N <= 0) {
    set_last_error("quantize_fp8_weights: null pointer or non-positive size");
    return kBadArg;
  }
  if (int rc = ensure_device()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case TESSERA_SM100_F32: return quant::quantize_weights_t<float>(w, E, K, N, q_t, scales, st, fmt);
    case TESSERA_SM100_BF16: return quant::quantize_weights_t<__nv_bfloat16>(w, E, K, N, q_t, scales, st, fmt);
    case TESSERA_SM100_F16: return quant::quantize_weights_t<__half>(w, E, K, N, q_t, scales, st, fmt);
    default: break;
  }
  set_last_error("quantize_fp8_weights: unsupported dtype %d", dtype);
  return kBadArg;
}

// x [rows, cols] (cols a multiple of 16; dtype code) -> codes [rows, cols/2] bytes and scales
// [rows, cols/16] e4m3 bytes. For expert weights [E, K, N] pass rows = E*K, cols = N: the blocks
// run along N, as the reference quantises each expert's (K, N) matrix along its last axis.
int tessera_sm100_quantize_nvfp4_device(const void* x, long long rows, long long cols, int dtype,
                                        void* codes, void* scales, void* stream) {
  if (!x || !codes || !scales || rows < 0 || cols < 0 || (cols % 16)) {
    set_last_error("quantize_nvfp4: null pointer, negative size, or last dim %lld not divisible by 16", cols);
    return kBadArg;
  }
  const long long nblocks = rows * (cols / 16);
  if (nblocks == 0) return kOk;
  if (int rc = ensure_device()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>((nblocks + 127) / 128);
  auto c8 = static_cast<uint8_t*>(codes);
  auto s8 = static_cast<uint8_t*>(scales);
  switch (dtype) {
    case TESSERA_SM100_F32:
      quant::nvfp4_quantize_kernel<float><<<grid, 128, 0, st>>>(static_cast<const float*>(x), nblocks, c8, s8);
      break;
    case TESSERA_SM100_BF16:
      quant::nvfp4_quantize_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(static_cast<const __nv_bfloat16*>(x), nblocks, c8, s8);
      break;
    case TESSERA_SM100_F16:
      quant::nvfp4_quantize_kernel<__half><<<grid, 128, 0, st>>>(static_cast<const __half*>(x), nblocks, c8, s8);
      break;
    default:
      set_last_error("quantize_nvfp4: unsupported dtype %d", dtype);
      return kBadArg;
  }
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  return kOk;
}

// codes + scales -> the dequantised values as bf16 (exact: at most 5 significant bits) or f32.
int tessera_sm100_dequantize_nvfp4_device(const void* codes, const void* scales, long long rows,
                                          long long cols, void* out, int out_dtype, void* stream) {
  if (!codes || !scales || !out || rows < 0 || cols < 0 || (cols % 16)) {
    set_last_error("dequantize_nvfp4: null pointer, negative size, or last dim %lld not divisible by 16", cols);
    return kBadArg;
  }
  const long long nblocks = rows * (cols / 16);
  if (nblocks == 0) return kOk;
  if (int rc = ensure_device()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>((nblocks + 127) / 128);
  auto c8 = static_cast<const uint8_t*>(codes);
  auto s8 = static_cast<const uint8_t*>(scales);
  if (out_dtype == TESSERA_SM100_BF16)
    quant::nvfp4_dequantize_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(c8, s8, nblocks, static_cast<__nv_bfloat16*>(out));
  else if (out_dtype == TESSERA_SM100_F32)
    quant::nvfp4_dequantize_kernel<float><<<grid, 128, 0, st>>>(c8, s8, nblocks, static_cast<float*>(out));
  else {
    set_last_error("dequantize_nvfp4: output dtype must be bf16 or f32");
    return kBadArg;
  }
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  return kOk;
}

// 8-bit floats (fmt 0 = e4m3, 1 = e5m2) -> bf16 holding the same values (the activation operand of
// the fp8 x fp4 GEMM).
int tessera_sm100_fp8_to_bf16_device(const void* q, long long n, int fmt, void* out, void* stream) {
  if (!q || !out || n < 0 || (fmt != TESSERA_SM100_FP8_E4M3 && fmt != TESSERA_SM100_FP8_E5M2)) {
    set_last_error("fp8_to_bf16: null pointer, negative size or unknown format");
    return kBadArg;
  }
  if (n == 0) return kOk;
  if (int rc = ensure_device()) return rc;
  const int blocks = (int)std::min<long long>((n + 255) / 256, 148 * 8);
  quant::fp8_to_bf16_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(q), n, static_cast<__nv_bfloat16*>(out), fmt);
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  return kOk;
}

}  // extern "C"
