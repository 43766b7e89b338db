// Host-side plumbing shared by every op in the library: device selection, the thread-local
// error string, the per-device error word kernels write when a bounded wait expires, a
// caching device allocator for the host-pointer entry points, and tensor-map encoding
// through the driver entry point (no link-time dependency on libcuda).
#pragma once
#include <cstddef>
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

namespace tsb {

// Return codes of the op entry points (same convention as the reference's shipped GEMM
// symbols): 0 ok, 1 bad shape / null pointer, 2 no usable GPU, 3 a device operation failed.
enum Rc : int { kOk = 0, kBadArg = 1, kNoDevice = 2, kDeviceFailed = 3 };

void set_last_error(const char* fmt, ...);
const char* last_error();

// Makes sure a CUDA device is usable on this thread; returns kOk or kNoDevice.
int ensure_device();
int current_device();
int sm_count();

// Process-wide count of kernels this library launched (reported by the benchmark).
void note_launch(int n = 1);
long long launch_count();

// int[4] in device memory, zero on creation: {code, block, detail, 0}. One per device.
int* device_err_word();
// Reads and clears the word (synchronises the device). Returns the code.
int consume_device_err(int out[4]);

// Caching allocator: blocks are kept for reuse until pool_release_all(). A freed block carries
// the events after which it may be handed out again, so freeing right after enqueueing the work
// that uses it is safe on any stream:
//   pool_free(p)            nothing queued uses p any more (the caller synchronised)
//   pool_free_after(p, s)   work queued on stream s may still use p
//   pool_free_after_all(p)  the stream is not known: ordered after the legacy default stream and
//                           every stream this library created on the device (pool_note_stream)
void* pool_alloc(size_t bytes);
void pool_free(void* p);
void pool_free_after(void* p, cudaStream_t stream);
void pool_free_after_all(void* p);
void pool_note_stream(cudaStream_t stream, bool created);
void pool_release_all();

// rank <= 5. dims[0] is the innermost extent (elements); strides_bytes[i] is the byte stride
// of dimension i+1. Returns false and sets the error string on failure.
bool encode_tmap(CUtensorMap* out, CUtensorMapDataType dtype, int rank, const void* base,
                 const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                 CUtensorMapSwizzle swizzle);

#define TSB_CUDA_OK(expr)                                                              \
  do {                                                                                 \
    cudaError_t _e = (expr);                                                           \
    if (_e != cudaSuccess) {                                                           \
      ::tsb::set_last_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),    \
                            __FILE__, __LINE__);                                       \
      return ::tsb::kDeviceFailed;                                                     \
    }                                                                                  \
  } while (0)

}  // namespace tsb
