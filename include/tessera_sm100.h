/* C ABI of libtessera_sm100.so: hand-written sm_100a (B200) kernels behind the entry points
 * the Tessera Python runtime binds with ctypes.
 *
 * Conventions (the same as the reference's shipped NVIDIA GEMM library,
 * src/compiler/codegen/tessera_gpu_backend_NVIDIA/runtime/cuda/tessera_nvidia_gemm.cpp:19-20):
 *   return 0 ok, 1 bad shape / null pointer, 2 no usable GPU, 3 a device operation failed.
 * tessera_sm100_last_error() returns a thread-local description of the last non-zero return.
 * Entry points without a `_device` suffix take HOST pointers and do
 * upload -> kernel -> synchronise -> download; `_device` entry points take DEVICE pointers
 * plus a cudaStream_t (as void*), are asynchronous and do not synchronise.
 * All matrices are dense row-major.
 */
#ifndef TESSERA_SM100_H_
#define TESSERA_SM100_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* dtype codes */
#define TESSERA_SM100_F32 0
#define TESSERA_SM100_BF16 1
#define TESSERA_SM100_F16 2

/* ---- library / device management ------------------------------------------------------ */
const char* tessera_sm100_version(void);
const char* tessera_sm100_last_error(void);
int tessera_sm100_device_count(int* count);
int tessera_sm100_set_device(int index);
int tessera_sm100_sm_count(int* count);
/* Synchronises the device and reports the error word kernels set when a bounded wait
 * expired: out[0] code (0 = none), out[1] block, out[2] detail. Clears it. */
int tessera_sm100_consume_device_error(int out[4]);
/* Number of kernels of this library launched by the calling process so far. */
long long tessera_sm100_launch_count(void);

/* Helpers with the shape of tessera_nvidia_device_alloc ... tessera_nvidia_event_destroy
 * (tessera_nvidia_gemm.cpp:617-697). */
int tessera_sm100_device_alloc(void** out, size_t bytes);
int tessera_sm100_device_free(void* ptr);
int tessera_sm100_device_memset(void* ptr, int value, size_t bytes, void* stream);
int tessera_sm100_device_upload(void* dst, const void* src, size_t bytes, void* stream);
int tessera_sm100_device_download(void* dst, const void* src, size_t bytes, void* stream);
int tessera_sm100_device_copy(void* dst, const void* src, size_t bytes, void* stream);
int tessera_sm100_host_alloc(void** out, size_t bytes); /* pinned host memory */
int tessera_sm100_host_free(void* ptr);
int tessera_sm100_stream_create(void** out);
int tessera_sm100_stream_destroy(void* stream);
int tessera_sm100_stream_synchronize(void* stream);
int tessera_sm100_device_synchronize(void);
int tessera_sm100_event_create(void** out);
int tessera_sm100_event_destroy(void* event);
int tessera_sm100_event_record(void* event, void* stream);
int tessera_sm100_event_synchronize(void* event);
int tessera_sm100_event_elapsed_ms(void* start, void* stop, float* ms);
/* Writes `bytes` of a scratch buffer (device memory) to evict the L2 cache between timed runs. */
int tessera_sm100_flush_l2(void* stream);

/* ---- GEMM ------------------------------------------------------------------------------
 * D[M,N] f32 = A[M,K] * B[K,N], 16-bit inputs, f32 accumulate, ragged sizes allowed.
 * Replaces tessera_nvidia_mma_gemm_bf16 / _f16 and their _device twins
 * (tessera_nvidia_gemm.cpp:546-551, 569-586), which back tessera.ops.gemm
 * (python/tessera/__init__.py:239-254). */
int tessera_sm100_mma_gemm_bf16(const void* A, const void* B, void* D, int M, int N, int K);
int tessera_sm100_mma_gemm_f16(const void* A, const void* B, void* D, int M, int N, int K);
int tessera_sm100_mma_gemm_bf16_device(const void* A, const void* B, void* D, int M, int N, int K,
                                       void* stream);
int tessera_sm100_mma_gemm_f16_device(const void* A, const void* B, void* D, int M, int N, int K,
                                      void* stream);
/* Batched form with a selectable output dtype: A[batch,M,K], B[batch,K,N], D[batch,M,N].
 * Covers tessera.ops.batched_gemm (python/tessera/__init__.py:252-254). */
int tessera_sm100_gemm(const void* A, const void* B, void* D, int batch, int M, int N, int K,
                       int in_dtype, int out_dtype);
int tessera_sm100_gemm_device(const void* A, const void* B, void* D, int batch, int M, int N,
                              int K, int in_dtype, int out_dtype, void* stream);
/* Explicit leading dimensions and batch strides (elements); every stride must be a 16-byte
 * multiple. Used for the column-parallel N-split, where each rank writes a column block of
 * Y (python/tessera/compiler/tensor_parallel.py:118-123). */
int tessera_sm100_gemm_strided_device(const void* A, const void* B, void* D, int batch, int M,
                                      int N, int K, long long lda, long long ldb, long long ldd,
                                      long long strideA, long long strideB, long long strideD,
                                      int in_dtype, int out_dtype, void* stream);

/* ---- MoE grouped GEMM ------------------------------------------------------------------
 * out[T,N] = rows of group e of x[T,K] times w[e] (w is [E,K,N]); offsets[E+1] int32 row
 * offsets in device memory. Same argument order as the reference's emitted grouped GEMM ABI
 * (x, w, off[E+1], o, T, K, N, E) (python/tessera/compiler/emit/nvidia_cuda.py:1526-1532);
 * semantics of tessera.ops.grouped_gemm (python/tessera/__init__.py:291-351).
 * K and N must be multiples of 8. */
int tessera_sm100_grouped_gemm_device(const void* x, const void* w, const int* offsets, void* out,
                                      int T, int K, int N, int E, int in_dtype, int out_dtype,
                                      void* stream);
/* out[T,F] = silu(x_e * w_gate[e]) * (x_e * w_up[e]) in one kernel: the first two grouped GEMMs
 * and the silu_mul of tessera.ops.moe_swiglu_block (python/tessera/__init__.py:592-616). */
int tessera_sm100_grouped_swiglu_device(const void* x, const void* w_gate, const void* w_up,
                                        const int* offsets, void* out, int T, int K, int F, int E,
                                        int in_dtype, int out_dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TESSERA_SM100_H_ */
