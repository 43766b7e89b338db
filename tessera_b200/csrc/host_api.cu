// Host-pointer entry points for attention and the MoE layer (upload -> kernels -> download),
// the attention dispatcher that picks the decode or the prefill kernel, and silu_mul.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cmath>

#include "../../include/tessera_sm100.h"
#include "device_ctx.h"

using namespace tsb;

namespace {

size_t esize(int dt) { return dt == TESSERA_SM100_F32 ? 4 : 2; }

struct PoolBuf {
  void* p = nullptr;
  explicit PoolBuf(size_t bytes) : p(pool_alloc(bytes)) {}
  ~PoolBuf() { pool_free_after_all(p); }  // safe on early exits that leave work queued
  PoolBuf(const PoolBuf&) = delete;
  PoolBuf& operator=(const PoolBuf&) = delete;
};

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ a, const T* __restrict__ b,
                                T* __restrict__ o, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float x = static_cast<float>(a[i]);
    o[i] = static_cast<T>((x / (1.0f + expf(-x))) * static_cast<float>(b[i]));
  }
}

template <typename T>
int silu_mul_launch(const void* a, const void* b, void* o, long long n, cudaStream_t st) {
  const int grid = (int)std::min<long long>((n + 255) / 256, 148 * 16);
  silu_mul_kernel<T><<<grid, 256, 0, st>>>(static_cast<const T*>(a), static_cast<const T*>(b),
                                           static_cast<T*>(o), n);
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  return kOk;
}

int finish_sync(cudaStream_t st, const char* what) {
  cudaError_t e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) {
    set_last_error("%s: synchronise failed: %s", what, cudaGetErrorString(e));
    cudaGetLastError();
    return kDeviceFailed;
  }
  int w[4];
  if (consume_device_err(w) != 0) {
    set_last_error("%s: kernel wait expired (code %d, block %d, detail %d)", what, w[0], w[1], w[2]);
    return kDeviceFailed;
  }
  return kOk;
}

}  // namespace

extern "C" {

int tessera_sm100_silu_mul_device(const void* a, const void* b, void* out, long long n, int dtype,
                                  void* stream) {
  if (!a || !b || !out || n < 0) {
    set_last_error("silu_mul: bad arguments");
    return kBadArg;
  }
  if (n == 0) return kOk;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case TESSERA_SM100_F32: return silu_mul_launch<float>(a, b, out, n, st);
    case TESSERA_SM100_BF16: return silu_mul_launch<__nv_bfloat16>(a, b, out, n, st);
    case TESSERA_SM100_F16: return silu_mul_launch<__half>(a, b, out, n, st);
    default: break;
  }
  set_last_error("silu_mul: unsupported dtype %d", dtype);
  return kBadArg;
}

// Device-pointer attention forward: one query token per sequence goes to the split-KV decode
// kernel (scratch from the library's pool), anything else to the tcgen05 prefill kernel.
int tessera_sm100_flash_attn_device(const void* Q, const void* K, const void* V, void* O, int B,
                                    int Hq, int Hkv, int Sq, int Sk, int D, float scale, int causal,
                                    void* stream) {
  if (Sq == 1) {
    const int splits = tessera_sm100_attn_decode_splits(B, Hq, Hkv, Sk);
    if (splits <= 1)
      return tessera_sm100_attn_decode_device(Q, K, V, O, B, Hq, Hkv, Sk, D, scale, 1, nullptr,
                                              stream);
    // Pool blocks are recycled in stream order; callers that overlap attention calls on
    // several streams should pass their own scratch to tessera_sm100_attn_decode_device.
    PoolBuf scratch(tessera_sm100_attn_decode_scratch_bytes(B, Hq, splits));
    if (!scratch.p) return kDeviceFailed;
    return tessera_sm100_attn_decode_device(Q, K, V, O, B, Hq, Hkv, Sk, D, scale, splits, scratch.p,
                                            stream);
  }
  return tessera_sm100_flash_attn_fwd_device(Q, K, V, O, B, Hq, Hkv, Sq, Sk, D, scale, causal,
                                             stream);
}

int tessera_sm100_flash_attn(const void* Q, const void* K, const void* V, void* O, int B, int Hq,
                             int Hkv, int Sq, int Sk, int D, float scale, int causal) {
  if (!Q || !K || !V || !O || B <= 0 || Hq <= 0 || Hkv <= 0 || Sq <= 0 || Sk <= 0 || D <= 0) {
    set_last_error("flash_attn: null pointer or non-positive size");
    return kBadArg;
  }
  if (int rc = ensure_device()) return rc;
  const size_t nq = (size_t)B * Hq * Sq * D * 2, nkv = (size_t)B * Hkv * Sk * D * 2;
  PoolBuf dq(nq), dk(nkv), dv(nkv), dout(nq);
  if (!dq.p || !dk.p || !dv.p || !dout.p) return kDeviceFailed;
  cudaStream_t st = nullptr;
  TSB_CUDA_OK(cudaMemcpyAsync(dq.p, Q, nq, cudaMemcpyHostToDevice, st));
  TSB_CUDA_OK(cudaMemcpyAsync(dk.p, K, nkv, cudaMemcpyHostToDevice, st));
  TSB_CUDA_OK(cudaMemcpyAsync(dv.p, V, nkv, cudaMemcpyHostToDevice, st));
  int rc = tessera_sm100_flash_attn_device(dq.p, dk.p, dv.p, dout.p, B, Hq, Hkv, Sq, Sk, D, scale,
                                           causal, st);
  if (rc == kOk) {
    TSB_CUDA_OK(cudaMemcpyAsync(O, dout.p, nq, cudaMemcpyDeviceToHost, st));
  }
  const int rs = finish_sync(st, "flash_attn");
  return rc ? rc : rs;
}

// Host-pointer MoE layer. Optional outputs (may be null): assignment [T,top_k] int32 and
// weights [T,top_k] f32 after capacity drops, group_sizes [E] int32, token_of_slot [T*top_k] int32.
int tessera_sm100_moe_layer(const void* x, const float* logits, const void* w_gate,
                            const void* w_up, const void* w_down, void* out, int T, int H, int F,
                            int E, int top_k, int normalize, int capacity, int dtype, int out_dtype,
                            int* assignment_out, float* weights_out, int* group_sizes_out,
                            int* token_of_slot_out) {
  if (!x || !logits || !w_gate || !w_up || !w_down || !out || T <= 0 || H <= 0 || F <= 0 ||
      E <= 0 || top_k <= 0) {
    set_last_error("moe_layer: null pointer or non-positive size");
    return kBadArg;
  }
  if (int rc = ensure_device()) return rc;
  const size_t nx = (size_t)T * H * esize(dtype), nl = (size_t)T * E * 4;
  const size_t nw1 = (size_t)E * H * F * esize(dtype);
  const size_t nout = (size_t)T * H * esize(out_dtype);
  const size_t nws = tessera_sm100_moe_workspace_bytes(T, H, F, E, top_k);
  PoolBuf dx(nx), dl(nl), dg(nw1), du(nw1), dd(nw1), dout(nout), ws(nws);
  if (!dx.p || !dl.p || !dg.p || !du.p || !dd.p || !dout.p || !ws.p) return kDeviceFailed;
  cudaStream_t st = nullptr;
  TSB_CUDA_OK(cudaMemcpyAsync(dx.p, x, nx, cudaMemcpyHostToDevice, st));
  TSB_CUDA_OK(cudaMemcpyAsync(dl.p, logits, nl, cudaMemcpyHostToDevice, st));
  TSB_CUDA_OK(cudaMemcpyAsync(dg.p, w_gate, nw1, cudaMemcpyHostToDevice, st));
  TSB_CUDA_OK(cudaMemcpyAsync(du.p, w_up, nw1, cudaMemcpyHostToDevice, st));
  TSB_CUDA_OK(cudaMemcpyAsync(dd.p, w_down, nw1, cudaMemcpyHostToDevice, st));
  int rc = tessera_sm100_moe_layer_device(dx.p, static_cast<const float*>(dl.p), dg.p, du.p, dd.p,
                                          dout.p, T, H, F, E, top_k, normalize, capacity, dtype,
                                          out_dtype, ws.p, st);
  if (rc == kOk) {
    TSB_CUDA_OK(cudaMemcpyAsync(out, dout.p, nout, cudaMemcpyDeviceToHost, st));
    void *a = nullptr, *w = nullptr, *tok = nullptr, *gs = nullptr;
    tessera_sm100_moe_workspace_views(ws.p, T, H, F, E, top_k, &a, &w, &tok, nullptr, nullptr, &gs,
                                      nullptr, nullptr);
    const size_t S = (size_t)T * top_k;
    if (assignment_out) TSB_CUDA_OK(cudaMemcpyAsync(assignment_out, a, S * 4, cudaMemcpyDeviceToHost, st));
    if (weights_out) TSB_CUDA_OK(cudaMemcpyAsync(weights_out, w, S * 4, cudaMemcpyDeviceToHost, st));
    if (token_of_slot_out) TSB_CUDA_OK(cudaMemcpyAsync(token_of_slot_out, tok, S * 4, cudaMemcpyDeviceToHost, st));
    if (group_sizes_out) TSB_CUDA_OK(cudaMemcpyAsync(group_sizes_out, gs, (size_t)E * 4, cudaMemcpyDeviceToHost, st));
  }
  const int rs = finish_sync(st, "moe_layer");
  return rc ? rc : rs;
}

}  // extern "C"
