// Library management and the device / stream / event helpers of the C ABI.
#include "../../include/tessera_sm100.h"
#include "device_ctx.h"
#include "sm100_ptx.cuh"

using namespace tsb;

namespace {
constexpr size_t kFlushBytes = 256ull << 20;  // larger than the 126 MB L2

__global__ void flush_kernel(uint4* buf, size_t n, uint32_t tag) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n;
       i += (size_t)gridDim.x * blockDim.x)
    buf[i] = make_uint4(tag, tag, tag, tag);
}

// One warp waits, through the same bounded wait the kernels use, on a barrier that nobody arrives
// on. When the limit runs out the waiter records the error word and the kernel ends normally.
__global__ void wait_expiry_kernel(long long limit_cycles, int* err, int* gave_up) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const bool ok = mbar_wait_limit(smem_u32(&bar), 0, &abort_flag, err, kErrWaitOther, 77, limit_cycles);
    if (gave_up) *gave_up = ok ? 0 : 1;
  }
  __syncthreads();
}
}  // namespace

extern "C" {

// Self-test of the failure path: a bounded device wait that is certain to run out (at most 2^28
// cycles, about 0.15 s). Afterwards tessera_sm100_consume_device_error reports {5, 0, 77}.
int tessera_sm100_selftest_wait_expiry(long long limit_cycles, void* stream) {
  if (limit_cycles <= 0 || limit_cycles > (1ll << 28)) {
    set_last_error("selftest_wait_expiry: limit_cycles must be in (0, 2^28]");
    return kBadArg;
  }
  if (int rc = ensure_device()) return rc;
  int* err = device_err_word();
  if (!err) return kDeviceFailed;
  wait_expiry_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(limit_cycles, err, nullptr);
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  return kOk;
}

const char* tessera_sm100_version(void) { return "tessera-sm100 0.1.0 (sm_100a, tcgen05/TMA)"; }
const char* tessera_sm100_last_error(void) { return last_error(); }

int tessera_sm100_device_count(int* count) {
  if (!count) return kBadArg;
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    n = 0;
  }
  *count = n;
  return kOk;
}
int tessera_sm100_set_device(int index) {
  if (cudaSetDevice(index) != cudaSuccess) {
    set_last_error("cudaSetDevice(%d) failed: %s", index, cudaGetErrorString(cudaGetLastError()));
    return kNoDevice;
  }
  return ensure_device();
}
int tessera_sm100_sm_count(int* count) {
  if (!count) return kBadArg;
  if (int rc = ensure_device()) return rc;
  *count = sm_count();
  return kOk;
}
int tessera_sm100_consume_device_error(int out[4]) {
  if (int rc = ensure_device()) return rc;
  TSB_CUDA_OK(cudaDeviceSynchronize());
  int code = consume_device_err(out);
  return code < 0 ? kDeviceFailed : kOk;
}
long long tessera_sm100_launch_count(void) { return launch_count(); }

int tessera_sm100_device_alloc(void** out, size_t bytes) {
  if (!out) return kBadArg;
  if (int rc = ensure_device()) return rc;
  TSB_CUDA_OK(cudaMalloc(out, bytes ? bytes : 1));
  return kOk;
}
int tessera_sm100_device_free(void* ptr) {
  if (!ptr) return kOk;
  TSB_CUDA_OK(cudaFree(ptr));
  return kOk;
}
// Caching allocator shared with the host-pointer entry points: freed blocks are kept and handed
// out again, so steady-state loops make no cudaMalloc/cudaFree calls (each of which synchronises
// the device). Free a block once the work that uses it has been ENQUEUED: pool_free orders its
// reuse after everything queued so far on the legacy default stream and on every stream made by
// tessera_sm100_stream_create / tsrCreateStream; pool_free_async after one given stream only
// (cheaper, and the form for a stream this library did not create).
int tessera_sm100_pool_alloc(void** out, size_t bytes) {
  if (!out) return kBadArg;
  if (int rc = ensure_device()) return rc;
  *out = pool_alloc(bytes);
  return *out ? kOk : kDeviceFailed;
}
int tessera_sm100_pool_free(void* ptr) {
  pool_free_after_all(ptr);
  return kOk;
}
int tessera_sm100_pool_free_async(void* ptr, void* stream) {
  pool_free_after(ptr, static_cast<cudaStream_t>(stream));
  return kOk;
}
int tessera_sm100_pool_release(void) {
  pool_release_all();
  return kOk;
}
int tessera_sm100_device_memset(void* ptr, int value, size_t bytes, void* stream) {
  if (!ptr) return kBadArg;
  TSB_CUDA_OK(cudaMemsetAsync(ptr, value, bytes, static_cast<cudaStream_t>(stream)));
  return kOk;
}
int tessera_sm100_device_upload(void* dst, const void* src, size_t bytes, void* stream) {
  if (!dst || !src) return kBadArg;
  TSB_CUDA_OK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice,
                              static_cast<cudaStream_t>(stream)));
  return kOk;
}
int tessera_sm100_device_download(void* dst, const void* src, size_t bytes, void* stream) {
  if (!dst || !src) return kBadArg;
  TSB_CUDA_OK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost,
                              static_cast<cudaStream_t>(stream)));
  return kOk;
}
int tessera_sm100_device_copy(void* dst, const void* src, size_t bytes, void* stream) {
  if (!dst || !src) return kBadArg;
  TSB_CUDA_OK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice,
                              static_cast<cudaStream_t>(stream)));
  return kOk;
}
int tessera_sm100_device_copy_2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch,
                                 size_t width_bytes, size_t rows, void* stream) {
  if (!dst || !src) return kBadArg;
  if (width_bytes == 0 || rows == 0) return kOk;
  TSB_CUDA_OK(cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, rows,
                                cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream)));
  return kOk;
}
// Rows of `width_bytes` from device memory (pitch src_pitch) into host memory (pitch dst_pitch).
int tessera_sm100_device_download_2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch,
                                     size_t width_bytes, size_t rows, void* stream) {
  if (!dst || !src) return kBadArg;
  if (width_bytes == 0 || rows == 0) return kOk;
  TSB_CUDA_OK(cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, rows,
                                cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)));
  return kOk;
}
int tessera_sm100_host_alloc(void** out, size_t bytes) {
  if (!out) return kBadArg;
  if (int rc = ensure_device()) return rc;
  TSB_CUDA_OK(cudaMallocHost(out, bytes ? bytes : 1));
  return kOk;
}
int tessera_sm100_host_free(void* ptr) {
  if (!ptr) return kOk;
  TSB_CUDA_OK(cudaFreeHost(ptr));
  return kOk;
}
int tessera_sm100_stream_create(void** out) {
  if (!out) return kBadArg;
  if (int rc = ensure_device()) return rc;
  cudaStream_t s;
  TSB_CUDA_OK(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  pool_note_stream(s, true);
  *out = s;
  return kOk;
}
int tessera_sm100_stream_destroy(void* stream) {
  if (!stream) return kOk;
  pool_note_stream(static_cast<cudaStream_t>(stream), false);
  TSB_CUDA_OK(cudaStreamDestroy(static_cast<cudaStream_t>(stream)));
  return kOk;
}
int tessera_sm100_stream_synchronize(void* stream) {
  TSB_CUDA_OK(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  return kOk;
}
int tessera_sm100_device_synchronize(void) {
  TSB_CUDA_OK(cudaDeviceSynchronize());
  return kOk;
}
int tessera_sm100_event_create(void** out) {
  if (!out) return kBadArg;
  if (int rc = ensure_device()) return rc;
  cudaEvent_t e;
  TSB_CUDA_OK(cudaEventCreate(&e));
  *out = e;
  return kOk;
}
int tessera_sm100_event_destroy(void* event) {
  if (!event) return kOk;
  TSB_CUDA_OK(cudaEventDestroy(static_cast<cudaEvent_t>(event)));
  return kOk;
}
int tessera_sm100_event_record(void* event, void* stream) {
  if (!event) return kBadArg;
  TSB_CUDA_OK(cudaEventRecord(static_cast<cudaEvent_t>(event), static_cast<cudaStream_t>(stream)));
  return kOk;
}
// Work enqueued on `stream` after this call waits for `event` (recorded on another stream).
int tessera_sm100_stream_wait_event(void* stream, void* event) {
  if (!event) return kBadArg;
  TSB_CUDA_OK(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), static_cast<cudaEvent_t>(event), 0));
  return kOk;
}
int tessera_sm100_event_synchronize(void* event) {
  if (!event) return kBadArg;
  TSB_CUDA_OK(cudaEventSynchronize(static_cast<cudaEvent_t>(event)));
  return kOk;
}
int tessera_sm100_event_elapsed_ms(void* start, void* stop, float* ms) {
  if (!start || !stop || !ms) return kBadArg;
  TSB_CUDA_OK(cudaEventElapsedTime(ms, static_cast<cudaEvent_t>(start),
                                   static_cast<cudaEvent_t>(stop)));
  return kOk;
}
int tessera_sm100_flush_l2(void* stream) {
  if (int rc = ensure_device()) return rc;
  static thread_local void* buf = nullptr;
  static thread_local int buf_dev = -1;
  static thread_local uint32_t tag = 0;
  if (!buf || buf_dev != current_device()) {
    TSB_CUDA_OK(cudaMalloc(&buf, kFlushBytes));
    buf_dev = current_device();
  }
  flush_kernel<<<148 * 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<uint4*>(buf), kFlushBytes / sizeof(uint4), ++tag);
  TSB_CUDA_OK(cudaGetLastError());
  return kOk;
}

}  // extern "C"
