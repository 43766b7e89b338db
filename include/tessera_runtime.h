/* Runtime C ABI (`tsr*`) of the B200 backend: the same entry points, handle types, status codes
 * and struct layouts as the reference runtime (src/runtime/include/tessera/tessera_runtime.h:14-147,
 * tsr_types.h, tsr_status.h), implemented on CUDA for sm_100a. Where the reference's CUDA backend
 * stops at memory/stream/event wrappers and answers UNIMPLEMENTED for launches
 * (src/runtime/src/backend/cuda_backend.cpp:253-268), tsrLaunchKernel here routes GPU artifact
 * kernels to a launcher registered with tsrRegisterGpuLauncher; the library registers a built-in
 * launcher for target "nvidia_sm100" that maps kernel names to the hand-written kernels.
 *
 * Every function returns a TsrStatus; the text of the last failure is thread-local
 * (tsrGetLastError) and valid until the next call on that thread. Handles are owned by the
 * caller. tsrShutdown refuses (TSR_STATUS_INVALID_ARGUMENT) while streams, events or buffers are
 * alive (src/runtime/src/tessera_runtime.cpp:435-474). The host-tile (CPU) kernel entry points of
 * the reference are not part of this library: there is no CPU execution path.
 */
#ifndef TESSERA_RUNTIME_H_
#define TESSERA_RUNTIME_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  TSR_STATUS_SUCCESS = 0,
  TSR_STATUS_INVALID_ARGUMENT = 1,
  TSR_STATUS_NOT_FOUND = 2,
  TSR_STATUS_ALREADY_EXISTS = 3,
  TSR_STATUS_OUT_OF_MEMORY = 4,
  TSR_STATUS_UNIMPLEMENTED = 5,
  TSR_STATUS_INTERNAL = 6,
  TSR_STATUS_DEVICE_ERROR = 7
} TsrStatus;

typedef struct tsrDevice_t* tsrDevice;
typedef struct tsrStream_t* tsrStream;
typedef struct tsrEvent_t* tsrEvent;
typedef struct tsrBuffer_t* tsrBuffer;
typedef struct tsrArtifact_t* tsrArtifact;
typedef struct tsrKernel_t* tsrKernel;

typedef enum { TSR_DEVICE_CPU = 0, TSR_DEVICE_CUDA = 1, TSR_DEVICE_HIP = 2 } TsrDeviceKind;

typedef struct {
  TsrDeviceKind kind;
  char name[128];
  uint32_t logical_tile_threads_max;
  uint32_t concurrent_tiles_hint;
} tsrDeviceProps;

typedef enum {
  TSR_MEMCPY_HOST_TO_DEVICE,
  TSR_MEMCPY_DEVICE_TO_HOST,
  TSR_MEMCPY_DEVICE_TO_DEVICE,
  TSR_MEMCPY_HOST_TO_HOST
} TsrMemcpyKind;

typedef enum { TSR_PROFILE_RUNTIME_API = 0, TSR_PROFILE_DEVICE_ACTIVITY = 1 } TsrProfileEventKind;

/* payload_json is owned by the runtime and valid only during the callback; value is 0.0 for
 * runtime-API events and elapsed microseconds for device-activity events. */
typedef void (*tsrProfileEventFn)(TsrProfileEventKind kind, const char* name,
                                  const char* payload_json, double value, void* user);

typedef struct {
  const char* target;
  const char* options_json;
} tsrCompileOptions;

/* Ordered buffer pointers and scalar dims of one GPU kernel launch; the order is the kernel's
 * own ABI (a GEMM is buffers = {A, B, D}, dims = {M, N, K}). */
typedef struct {
  void** buffers;
  size_t num_buffers;
  const int64_t* dims;
  size_t num_dims;
} tsrGpuLaunchParams;

typedef TsrStatus (*tsrGpuLauncherFn)(const char* target, const char* kernel_name,
                                      const tsrGpuLaunchParams* params, void* user);

const char* tsrStatusString(TsrStatus status);
const char* tsrGetLastError(void);
void tsrClearLastError(void);
void tsrGetVersion(int* major, int* minor, int* patch);

TsrStatus tsrInit(void);
TsrStatus tsrShutdown(void);
TsrStatus tsrIsInitialized(int* out);

TsrStatus tsrGetDeviceCount(int* count);
TsrStatus tsrGetDevice(int index, tsrDevice* out);
TsrStatus tsrGetDeviceProps(tsrDevice dev, tsrDeviceProps* props);

TsrStatus tsrCreateStream(tsrDevice dev, tsrStream* out);
TsrStatus tsrDestroyStream(tsrStream s);
TsrStatus tsrStreamSynchronize(tsrStream s);

TsrStatus tsrCreateEvent(tsrDevice dev, tsrEvent* out);
TsrStatus tsrRecordEvent(tsrEvent e, tsrStream s);
TsrStatus tsrWaitEvent(tsrEvent e, tsrStream s);
TsrStatus tsrEventSynchronize(tsrEvent e);
TsrStatus tsrDestroyEvent(tsrEvent e);
/* Nanoseconds since process start at which the event completed (host steady clock). */
TsrStatus tsrEventGetTimestamp(tsrEvent e, uint64_t* ns_out);
/* Device time between two recorded events, in milliseconds (CUDA events). */
TsrStatus tsrEventElapsedMs(tsrEvent start, tsrEvent stop, float* ms_out);

TsrStatus tsrSetProfileEventCallback(tsrProfileEventFn fn, void* user);
TsrStatus tsrEnableProfiling(int enabled);

TsrStatus tsrMalloc(tsrDevice dev, size_t bytes, tsrBuffer* out);
TsrStatus tsrFree(tsrBuffer b);
TsrStatus tsrMemset(tsrBuffer b, int value, size_t bytes);
/* Buffer-to-buffer copy as in the reference (both operands are buffer handles); host data moves
 * through tsrMap/tsrUnmap or through the two explicit host forms below. */
TsrStatus tsrMemcpy(tsrBuffer dst, const tsrBuffer src, size_t bytes, TsrMemcpyKind kind);
TsrStatus tsrMemcpyFromHost(tsrBuffer dst, const void* src, size_t bytes);
TsrStatus tsrMemcpyToHost(void* dst, const tsrBuffer src, size_t bytes);
TsrStatus tsrMap(tsrBuffer b, void** host_ptr, size_t* bytes);
TsrStatus tsrUnmap(tsrBuffer b);
/* Raw device pointer and size of a buffer (for passing it to a kernel launch). */
TsrStatus tsrBufferGetPointer(tsrBuffer b, void** device_ptr, size_t* bytes);

/* module_ir is a comma-separated list of kernel names; options->target selects the launcher
 * target ("nvidia_sm100" and its aliases). */
TsrStatus tsrCompileArtifact(const char* module_ir, const tsrCompileOptions* options,
                             tsrArtifact* out);
TsrStatus tsrLoadArtifact(const void* bytes, size_t bytes_len, tsrArtifact* out);
TsrStatus tsrDestroyArtifact(tsrArtifact artifact);
TsrStatus tsrGetArtifactBytes(tsrArtifact artifact, const void** out_bytes, size_t* out_len);
TsrStatus tsrGetArtifactTarget(tsrArtifact artifact, const char** out);
TsrStatus tsrGetKernel(tsrArtifact artifact, const char* name, tsrKernel* out);
TsrStatus tsrDestroyKernel(tsrKernel kernel);
/* args[0] = const tsrGpuLaunchParams*; nargs >= 1. Routed to the registered launcher;
 * TSR_STATUS_UNIMPLEMENTED when none handles (target, kernel name). The built-in launcher
 * enqueues the work on `s` (NULL = the default stream), so tsrStreamSynchronize(s),
 * tsrRecordEvent(e, s) and tsrWaitEvent(e, s) order with it. */
TsrStatus tsrLaunchKernel(tsrStream s, tsrKernel kernel, void** args, size_t nargs);
/* The launcher signature carries no stream: a launcher registered with tsrRegisterGpuLauncher reads
 * the cudaStream_t of the tsrLaunchKernel call that is running it here (NULL = default stream). */
void* tessera_sm100_current_launch_stream(void);
TsrStatus tsrRegisterGpuLauncher(tsrGpuLauncherFn fn, void* user);
/* The library's own launcher for target "nvidia_sm100" (kernel names tessera.sm100.*), exported
 * so that a runtime with the same registry, such as the reference's libtessera_runtime
 * (src/runtime/src/tessera_runtime.cpp:1210-1222), can register it. */
TsrStatus tessera_sm100_gpu_launcher(const char* target, const char* kernel_name,
                                     const tsrGpuLaunchParams* params, void* user);

#ifdef __cplusplus
}
#endif
#endif /* TESSERA_RUNTIME_H_ */
