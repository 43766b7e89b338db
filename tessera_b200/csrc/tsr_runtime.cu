// `tsr*` runtime C ABI on CUDA for sm_100a (declared in include/tessera_runtime.h).
//
// Structure: a process-wide registry behind one mutex (initialisation state, live-handle
// counts, the GPU launcher, the profiling sink); no lock is held across a device operation or a
// launcher call. Errors never escape as C++ exceptions. The built-in launcher maps kernel names
// on target "nvidia_sm100" to the library's op entry points.
#include <atomic>
#include <chrono>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "../../include/tessera_runtime.h"
#include "../../include/tessera_sm100.h"
#include "device_ctx.h"

struct tsrDevice_t {
  int ordinal;
};
struct tsrStream_t {
  cudaStream_t stream;
  int device;
};
struct tsrEvent_t {
  cudaEvent_t event;
  int device;
  bool recorded;
};
struct tsrBuffer_t {
  void* ptr;
  size_t bytes;
  int device;
  void* host_shadow;  // pinned copy while mapped
};
struct tsrArtifact_t {
  std::string target;
  std::vector<std::string> kernels;
  std::string payload;
};
struct tsrKernel_t {
  std::string target;
  std::string name;
};

namespace {

thread_local std::string g_err;
std::mutex g_mu;
bool g_init = false;
std::vector<tsrDevice_t*> g_devices;
std::atomic<long> g_live_streams{0}, g_live_events{0}, g_live_buffers{0};
tsrGpuLauncherFn g_launcher = nullptr;
void* g_launcher_user = nullptr;
tsrProfileEventFn g_profile_fn = nullptr;
void* g_profile_user = nullptr;
bool g_profile_enabled = true;
std::atomic<int> g_profile_in_flight{0};
thread_local bool g_in_callback = false;
const auto g_t0 = std::chrono::steady_clock::now();

uint64_t now_ns() {
  return (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(
             std::chrono::steady_clock::now() - g_t0).count();
}

TsrStatus fail(TsrStatus st, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_err = buf;
  return st;
}

TsrStatus cuda_fail(cudaError_t e, const char* what) {
  cudaGetLastError();
  return fail(e == cudaErrorMemoryAllocation ? TSR_STATUS_OUT_OF_MEMORY : TSR_STATUS_DEVICE_ERROR,
              "%s: %s", what, cudaGetErrorString(e));
}

// Emits one profile event. Re-entrant calls from inside a callback are dropped; shutdown and
// callback replacement wait for callbacks in flight.
void emit(TsrProfileEventKind kind, const char* name, uint64_t start_ns, TsrStatus st,
          const std::string& extra = "") {
  tsrProfileEventFn fn;
  void* user;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_profile_fn || !g_profile_enabled || g_in_callback) return;
    fn = g_profile_fn;
    user = g_profile_user;
    g_profile_in_flight.fetch_add(1);
  }
  const uint64_t end = now_ns();
  char head[256];
  snprintf(head, sizeof(head), "{\"start_ns\":%llu,\"end_ns\":%llu,\"status\":\"%s\"%s",
           (unsigned long long)start_ns, (unsigned long long)end, tsrStatusString(st),
           extra.empty() ? "" : ",");
  std::string payload = std::string(head) + extra + "}";
  g_in_callback = true;
  fn(kind, name, payload.c_str(),
     kind == TSR_PROFILE_DEVICE_ACTIVITY ? (double)(end - start_ns) / 1000.0 : 0.0, user);
  g_in_callback = false;
  g_profile_in_flight.fetch_sub(1);
}

void drain_callbacks() {
  while (g_profile_in_flight.load() > 0) std::this_thread::yield();
}

TsrStatus need_init() {
  std::lock_guard<std::mutex> lk(g_mu);
  return g_init ? TSR_STATUS_SUCCESS : fail(TSR_STATUS_INVALID_ARGUMENT, "runtime is not initialised");
}

std::string normalize_target(const std::string& t) {
  static const char* aliases[] = {"nvidia_sm100", "sm100", "sm_100", "sm100a", "sm_100a",
                                  "blackwell", "b200"};
  for (const char* a : aliases)
    if (t == a) return "nvidia_sm100";
  return t;
}

// The CUDA stream of the tsrLaunchKernel call in progress on this thread. The launcher signature
// (target, kernel, params, user) carries no stream, so tsrLaunchKernel publishes it here and the
// built-in launcher enqueues on it; a launcher registered by someone else reads it through
// tessera_sm100_current_launch_stream().
thread_local void* t_launch_stream = nullptr;

// Built-in launcher: kernel name -> op entry point. buffers/dims follow each op's own ABI. The
// work is enqueued on the stream given to tsrLaunchKernel.
TsrStatus builtin_launcher(const char* target, const char* name, const tsrGpuLaunchParams* p,
                           void* /*user*/) {
  if (normalize_target(target ? target : "") != "nvidia_sm100") return TSR_STATUS_NOT_FOUND;
  const std::string k = name ? name : "";
  auto need = [&](size_t nb, size_t nd) {
    return p && p->num_buffers >= nb && p->num_dims >= nd && p->buffers && (nd == 0 || p->dims);
  };
  int rc = -1;
  if (k == "tessera.sm100.gemm.bf16" || k == "tessera.sm100.gemm.f16") {
    // buffers {A, B, D(f32)}, dims {M, N, K}
    if (!need(3, 3)) return fail(TSR_STATUS_INVALID_ARGUMENT, "%s wants 3 buffers and 3 dims", name);
    rc = tessera_sm100_gemm_device(p->buffers[0], p->buffers[1], p->buffers[2], 1, (int)p->dims[0],
                                   (int)p->dims[1], (int)p->dims[2],
                                   k == "tessera.sm100.gemm.bf16" ? TESSERA_SM100_BF16
                                                                  : TESSERA_SM100_F16,
                                   TESSERA_SM100_F32, t_launch_stream);
  } else if (k == "tessera.sm100.gemm.bf16.bf16out") {
    if (!need(3, 3)) return fail(TSR_STATUS_INVALID_ARGUMENT, "%s wants 3 buffers and 3 dims", name);
    rc = tessera_sm100_gemm_device(p->buffers[0], p->buffers[1], p->buffers[2], 1, (int)p->dims[0],
                                   (int)p->dims[1], (int)p->dims[2], TESSERA_SM100_BF16,
                                   TESSERA_SM100_BF16, t_launch_stream);
  } else if (k == "tessera.sm100.flash_attn.bf16") {
    // buffers {Q, K, V, O}, dims {B, Hq, Hkv, Sq, Sk, D, causal}; scale = 1/sqrt(D)
    if (!need(4, 7)) return fail(TSR_STATUS_INVALID_ARGUMENT, "%s wants 4 buffers and 7 dims", name);
    const float scale = 1.0f / sqrtf((float)p->dims[5]);
    rc = tessera_sm100_flash_attn_device(p->buffers[0], p->buffers[1], p->buffers[2], p->buffers[3],
                                         (int)p->dims[0], (int)p->dims[1], (int)p->dims[2],
                                         (int)p->dims[3], (int)p->dims[4], (int)p->dims[5], scale,
                                         (int)p->dims[6], t_launch_stream);
  } else if (k == "tessera.sm100.grouped_gemm.bf16") {
    // buffers {x, w, offsets(int32[E+1]), out}, dims {T, K, N, E}
    if (!need(4, 4)) return fail(TSR_STATUS_INVALID_ARGUMENT, "%s wants 4 buffers and 4 dims", name);
    rc = tessera_sm100_grouped_gemm_device(p->buffers[0], p->buffers[1],
                                           static_cast<const int*>(p->buffers[2]), p->buffers[3],
                                           (int)p->dims[0], (int)p->dims[1], (int)p->dims[2],
                                           (int)p->dims[3], TESSERA_SM100_BF16, TESSERA_SM100_BF16,
                                           t_launch_stream);
  } else {
    return TSR_STATUS_NOT_FOUND;
  }
  if (rc == 0) return TSR_STATUS_SUCCESS;
  g_err = tessera_sm100_last_error();
  return rc == 1 ? TSR_STATUS_INVALID_ARGUMENT : TSR_STATUS_DEVICE_ERROR;
}

}  // namespace

extern "C" {

const char* tsrStatusString(TsrStatus s) {
  switch (s) {
    case TSR_STATUS_SUCCESS: return "success";
    case TSR_STATUS_INVALID_ARGUMENT: return "invalid_argument";
    case TSR_STATUS_NOT_FOUND: return "not_found";
    case TSR_STATUS_ALREADY_EXISTS: return "already_exists";
    case TSR_STATUS_OUT_OF_MEMORY: return "out_of_memory";
    case TSR_STATUS_UNIMPLEMENTED: return "unimplemented";
    case TSR_STATUS_INTERNAL: return "internal";
    case TSR_STATUS_DEVICE_ERROR: return "device_error";
  }
  return "unknown";
}
const char* tsrGetLastError(void) { return g_err.c_str(); }
void tsrClearLastError(void) { g_err.clear(); }
void tsrGetVersion(int* major, int* minor, int* patch) {
  if (major) *major = 0;
  if (minor) *minor = 1;
  if (patch) *patch = 0;
}

TsrStatus tsrInit(void) {
  const uint64_t t = now_ns();
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    n = 0;
  }
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_init) {
      for (int i = 0; i < n; ++i) g_devices.push_back(new tsrDevice_t{i});
      if (!g_launcher) {
        g_launcher = builtin_launcher;
        g_launcher_user = nullptr;
      }
      g_init = true;
    }
  }
  emit(TSR_PROFILE_RUNTIME_API, "tsrInit", t, TSR_STATUS_SUCCESS);
  return TSR_STATUS_SUCCESS;
}

TsrStatus tsrShutdown(void) {
  const uint64_t t = now_ns();
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_init) return TSR_STATUS_SUCCESS;
    if (g_live_streams.load() || g_live_events.load() || g_live_buffers.load())
      return fail(TSR_STATUS_INVALID_ARGUMENT,
                  "shutdown refused: %ld stream(s), %ld event(s), %ld buffer(s) still alive",
                  g_live_streams.load(), g_live_events.load(), g_live_buffers.load());
  }
  emit(TSR_PROFILE_RUNTIME_API, "tsrShutdown", t, TSR_STATUS_SUCCESS);
  drain_callbacks();
  std::lock_guard<std::mutex> lk(g_mu);
  for (auto* d : g_devices) delete d;
  g_devices.clear();
  if (g_launcher == builtin_launcher) g_launcher = nullptr;
  g_init = false;
  return TSR_STATUS_SUCCESS;
}

TsrStatus tsrIsInitialized(int* out) {
  if (!out) return fail(TSR_STATUS_INVALID_ARGUMENT, "out==NULL");
  std::lock_guard<std::mutex> lk(g_mu);
  *out = g_init ? 1 : 0;
  return TSR_STATUS_SUCCESS;
}

TsrStatus tsrGetDeviceCount(int* count) {
  if (!count) return fail(TSR_STATUS_INVALID_ARGUMENT, "count==NULL");
  if (TsrStatus st = need_init()) return st;
  std::lock_guard<std::mutex> lk(g_mu);
  *count = (int)g_devices.size();
  return TSR_STATUS_SUCCESS;
}

TsrStatus tsrGetDevice(int index, tsrDevice* out) {
  if (!out) return fail(TSR_STATUS_INVALID_ARGUMENT, "out==NULL");
  if (TsrStatus st = need_init()) return st;
  std::lock_guard<std::mutex> lk(g_mu);
  if (index < 0 || index >= (int)g_devices.size())
    return fail(TSR_STATUS_NOT_FOUND, "device index %d out of range (%zu device(s))", index,
                g_devices.size());
  *out = g_devices[index];
  return TSR_STATUS_SUCCESS;
}

TsrStatus tsrGetDeviceProps(tsrDevice dev, tsrDeviceProps* props) {
  if (!dev || !props) return fail(TSR_STATUS_INVALID_ARGUMENT, "dev/props==NULL");
  cudaDeviceProp p;
  cudaError_t e = cudaGetDeviceProperties(&p, dev->ordinal);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDeviceProperties");
  memset(props, 0, sizeof(*props));
  props->kind = TSR_DEVICE_CUDA;
  snprintf(props->name, sizeof(props->name), "%s (sm_%d%d)", p.name, p.major, p.minor);
  props->logical_tile_threads_max = (uint32_t)p.maxThreadsPerBlock;
  props->concurrent_tiles_hint = (uint32_t)p.multiProcessorCount;
  return TSR_STATUS_SUCCESS;
}

TsrStatus tsrCreateStream(tsrDevice dev, tsrStream* out) {
  const uint64_t t = now_ns();
  if (!dev || !out) return fail(TSR_STATUS_INVALID_ARGUMENT, "dev/out==NULL");
  cudaError_t e = cudaSetDevice(dev->ordinal);
  cudaStream_t s = nullptr;
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
  if (e != cudaSuccess) return cuda_fail(e, "stream creation");
  tsb::pool_note_stream(s, true);
  *out = new tsrStream_t{s, dev->ordinal};
  g_live_streams.fetch_add(1);
  emit(TSR_PROFILE_RUNTIME_API, "tsrCreateStream", t, TSR_STATUS_SUCCESS);
  return TSR_STATUS_SUCCESS;
}
TsrStatus tsrDestroyStream(tsrStream s) {
  if (!s) return TSR_STATUS_SUCCESS;
  tsb::pool_note_stream(s->stream, false);
  cudaStreamDestroy(s->stream);
  delete s;
  g_live_streams.fetch_sub(1);
  return TSR_STATUS_SUCCESS;
}
TsrStatus tsrStreamSynchronize(tsrStream s) {
  const uint64_t t = now_ns();
  cudaError_t e = cudaStreamSynchronize(s ? s->stream : nullptr);
  TsrStatus st = e == cudaSuccess ? TSR_STATUS_SUCCESS : cuda_fail(e, "cudaStreamSynchronize");
  emit(TSR_PROFILE_RUNTIME_API, "tsrStreamSynchronize", t, st);
  return st;
}

TsrStatus tsrCreateEvent(tsrDevice dev, tsrEvent* out) {
  if (!dev || !out) return fail(TSR_STATUS_INVALID_ARGUMENT, "dev/out==NULL");
  cudaError_t e = cudaSetDevice(dev->ordinal);
  cudaEvent_t ev = nullptr;
  if (e == cudaSuccess) e = cudaEventCreate(&ev);
  if (e != cudaSuccess) return cuda_fail(e, "event creation");
  *out = new tsrEvent_t{ev, dev->ordinal, false};
  g_live_events.fetch_add(1);
  return TSR_STATUS_SUCCESS;
}
TsrStatus tsrRecordEvent(tsrEvent e, tsrStream s) {
  if (!e) return fail(TSR_STATUS_INVALID_ARGUMENT, "event==NULL");
  cudaError_t r = cudaEventRecord(e->event, s ? s->stream : nullptr);
  if (r != cudaSuccess) return cuda_fail(r, "cudaEventRecord");
  e->recorded = true;
  return TSR_STATUS_SUCCESS;
}
TsrStatus tsrWaitEvent(tsrEvent e, tsrStream s) {
  if (!e) return fail(TSR_STATUS_INVALID_ARGUMENT, "event==NULL");
  cudaError_t r = cudaStreamWaitEvent(s ? s->stream : nullptr, e->event, 0);
  return r == cudaSuccess ? TSR_STATUS_SUCCESS : cuda_fail(r, "cudaStreamWaitEvent");
}
TsrStatus tsrEventSynchronize(tsrEvent e) {
  if (!e) return fail(TSR_STATUS_INVALID_ARGUMENT, "event==NULL");
  cudaError_t r = cudaEventSynchronize(e->event);
  return r == cudaSuccess ? TSR_STATUS_SUCCESS : cuda_fail(r, "cudaEventSynchronize");
}
TsrStatus tsrDestroyEvent(tsrEvent e) {
  if (!e) return TSR_STATUS_SUCCESS;
  cudaEventDestroy(e->event);
  delete e;
  g_live_events.fetch_sub(1);
  return TSR_STATUS_SUCCESS;
}
TsrStatus tsrEventGetTimestamp(tsrEvent e, uint64_t* ns_out) {
  if (!e || !ns_out) return fail(TSR_STATUS_INVALID_ARGUMENT, "event/ns_out==NULL");
  if (!e->recorded) return fail(TSR_STATUS_INVALID_ARGUMENT, "event was never recorded");
  cudaError_t r = cudaEventSynchronize(e->event);
  if (r != cudaSuccess) return cuda_fail(r, "cudaEventSynchronize");
  *ns_out = now_ns();
  return TSR_STATUS_SUCCESS;
}
TsrStatus tsrEventElapsedMs(tsrEvent start, tsrEvent stop, float* ms_out) {
  if (!start || !stop || !ms_out) return fail(TSR_STATUS_INVALID_ARGUMENT, "null argument");
  cudaError_t r = cudaEventElapsedTime(ms_out, start->event, stop->event);
  return r == cudaSuccess ? TSR_STATUS_SUCCESS : cuda_fail(r, "cudaEventElapsedTime");
}

TsrStatus tsrSetProfileEventCallback(tsrProfileEventFn fn, void* user) {
  drain_callbacks();
  std::lock_guard<std::mutex> lk(g_mu);
  g_profile_fn = fn;
  g_profile_user = user;
  return TSR_STATUS_SUCCESS;
}
TsrStatus tsrEnableProfiling(int enabled) {
  std::lock_guard<std::mutex> lk(g_mu);
  g_profile_enabled = enabled != 0;
  return TSR_STATUS_SUCCESS;
}

TsrStatus tsrMalloc(tsrDevice dev, size_t bytes, tsrBuffer* out) {
  const uint64_t t = now_ns();
  if (!dev || !out) return fail(TSR_STATUS_INVALID_ARGUMENT, "dev/out==NULL");
  cudaError_t e = cudaSetDevice(dev->ordinal);
  void* p = nullptr;
  if (e == cudaSuccess) e = cudaMalloc(&p, bytes ? bytes : 1);
  if (e != cudaSuccess) {
    TsrStatus st = cuda_fail(e, "cudaMalloc");
    emit(TSR_PROFILE_RUNTIME_API, "tsrMalloc", t, st);
    return st;
  }
  *out = new tsrBuffer_t{p, bytes, dev->ordinal, nullptr};
  g_live_buffers.fetch_add(1);
  char extra[64];
  snprintf(extra, sizeof(extra), "\"bytes\":%zu", bytes);
  emit(TSR_PROFILE_RUNTIME_API, "tsrMalloc", t, TSR_STATUS_SUCCESS, extra);
  return TSR_STATUS_SUCCESS;
}
TsrStatus tsrFree(tsrBuffer b) {
  if (!b) return TSR_STATUS_SUCCESS;
  if (b->host_shadow) cudaFreeHost(b->host_shadow);
  cudaFree(b->ptr);
  delete b;
  g_live_buffers.fetch_sub(1);
  return TSR_STATUS_SUCCESS;
}
TsrStatus tsrMemset(tsrBuffer b, int value, size_t bytes) {
  if (!b) return fail(TSR_STATUS_INVALID_ARGUMENT, "b==NULL");
  if (bytes > b->bytes) return fail(TSR_STATUS_INVALID_ARGUMENT, "memset of %zu bytes exceeds the buffer (%zu)", bytes, b->bytes);
  cudaError_t e = cudaMemset(b->ptr, value, bytes);
  return e == cudaSuccess ? TSR_STATUS_SUCCESS : cuda_fail(e, "cudaMemset");
}
TsrStatus tsrMemcpy(tsrBuffer dst, const tsrBuffer src, size_t bytes, TsrMemcpyKind kind) {
  const uint64_t t = now_ns();
  if (!dst || !src) return fail(TSR_STATUS_INVALID_ARGUMENT, "dst/src==NULL");
  if (bytes > dst->bytes || bytes > src->bytes)
    return fail(TSR_STATUS_INVALID_ARGUMENT, "copy of %zu bytes exceeds a buffer", bytes);
  (void)kind;  // both operands live in device memory here
  cudaError_t e = cudaMemcpy(dst->ptr, src->ptr, bytes, cudaMemcpyDefault);
  TsrStatus st = e == cudaSuccess ? TSR_STATUS_SUCCESS : cuda_fail(e, "cudaMemcpy");
  char extra[64];
  snprintf(extra, sizeof(extra), "\"bytes\":%zu", bytes);
  emit(TSR_PROFILE_DEVICE_ACTIVITY, "tsrMemcpy", t, st, extra);
  return st;
}
TsrStatus tsrMemcpyFromHost(tsrBuffer dst, const void* src, size_t bytes) {
  if (!dst || !src) return fail(TSR_STATUS_INVALID_ARGUMENT, "dst/src==NULL");
  if (bytes > dst->bytes) return fail(TSR_STATUS_INVALID_ARGUMENT, "copy exceeds the buffer");
  cudaError_t e = cudaMemcpy(dst->ptr, src, bytes, cudaMemcpyHostToDevice);
  return e == cudaSuccess ? TSR_STATUS_SUCCESS : cuda_fail(e, "cudaMemcpy H2D");
}
TsrStatus tsrMemcpyToHost(void* dst, const tsrBuffer src, size_t bytes) {
  if (!dst || !src) return fail(TSR_STATUS_INVALID_ARGUMENT, "dst/src==NULL");
  if (bytes > src->bytes) return fail(TSR_STATUS_INVALID_ARGUMENT, "copy exceeds the buffer");
  cudaError_t e = cudaMemcpy(dst, src->ptr, bytes, cudaMemcpyDeviceToHost);
  return e == cudaSuccess ? TSR_STATUS_SUCCESS : cuda_fail(e, "cudaMemcpy D2H");
}
TsrStatus tsrMap(tsrBuffer b, void** host_ptr, size_t* bytes) {
  if (!b || !host_ptr) return fail(TSR_STATUS_INVALID_ARGUMENT, "b/host_ptr==NULL");
  if (!b->host_shadow) {
    cudaError_t e = cudaMallocHost(&b->host_shadow, b->bytes ? b->bytes : 1);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMallocHost");
    e = cudaMemcpy(b->host_shadow, b->ptr, b->bytes, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpy D2H");
  }
  *host_ptr = b->host_shadow;
  if (bytes) *bytes = b->bytes;
  return TSR_STATUS_SUCCESS;
}
TsrStatus tsrUnmap(tsrBuffer b) {
  if (!b) return fail(TSR_STATUS_INVALID_ARGUMENT, "b==NULL");
  if (!b->host_shadow) return TSR_STATUS_SUCCESS;
  cudaError_t e = cudaMemcpy(b->ptr, b->host_shadow, b->bytes, cudaMemcpyHostToDevice);
  cudaFreeHost(b->host_shadow);
  b->host_shadow = nullptr;
  return e == cudaSuccess ? TSR_STATUS_SUCCESS : cuda_fail(e, "cudaMemcpy H2D");
}
TsrStatus tsrBufferGetPointer(tsrBuffer b, void** device_ptr, size_t* bytes) {
  if (!b || !device_ptr) return fail(TSR_STATUS_INVALID_ARGUMENT, "b/device_ptr==NULL");
  *device_ptr = b->ptr;
  if (bytes) *bytes = b->bytes;
  return TSR_STATUS_SUCCESS;
}

// Artifact payload: "TSRART2\ntarget\t<t>\nkernel\t<name>\n..." (text, round-trips via
// tsrLoadArtifact).
static std::string make_payload(const tsrArtifact_t& a) {
  std::string s = "TSRART2\ntarget\t" + a.target + "\n";
  for (const auto& k : a.kernels) s += "kernel\t" + k + "\n";
  return s;
}

TsrStatus tsrCompileArtifact(const char* module_ir, const tsrCompileOptions* options,
                             tsrArtifact* out) {
  if (!module_ir || !out) return fail(TSR_STATUS_INVALID_ARGUMENT, "module_ir/out==NULL");
  auto* a = new tsrArtifact_t();
  a->target = normalize_target(options && options->target ? options->target : "nvidia_sm100");
  std::string cur;
  for (const char* c = module_ir;; ++c) {
    if (*c == ',' || *c == '\0') {
      size_t b = cur.find_first_not_of(" \t\n"), e = cur.find_last_not_of(" \t\n");
      if (b != std::string::npos) a->kernels.push_back(cur.substr(b, e - b + 1));
      cur.clear();
      if (*c == '\0') break;
    } else {
      cur.push_back(*c);
    }
  }
  if (a->kernels.empty()) {
    delete a;
    return fail(TSR_STATUS_INVALID_ARGUMENT, "module_ir names no kernel");
  }
  a->payload = make_payload(*a);
  *out = a;
  return TSR_STATUS_SUCCESS;
}

TsrStatus tsrLoadArtifact(const void* bytes, size_t len, tsrArtifact* out) {
  if (!bytes || !out) return fail(TSR_STATUS_INVALID_ARGUMENT, "bytes/out==NULL");
  std::string text(static_cast<const char*>(bytes), len);
  if (text.compare(0, 8, "TSRART2\n") != 0)
    return fail(TSR_STATUS_INVALID_ARGUMENT, "not a TSRART2 artifact payload");
  auto* a = new tsrArtifact_t();
  size_t pos = 8;
  while (pos < text.size()) {
    size_t eol = text.find('\n', pos);
    if (eol == std::string::npos) eol = text.size();
    std::string line = text.substr(pos, eol - pos);
    pos = eol + 1;
    size_t tab = line.find('\t');
    if (tab == std::string::npos) continue;
    std::string key = line.substr(0, tab), val = line.substr(tab + 1);
    if (key == "target") a->target = val;
    else if (key == "kernel") a->kernels.push_back(val);
  }
  if (a->target.empty() || a->kernels.empty()) {
    delete a;
    return fail(TSR_STATUS_INVALID_ARGUMENT, "artifact payload lacks a target or kernels");
  }
  a->payload = make_payload(*a);
  *out = a;
  return TSR_STATUS_SUCCESS;
}

TsrStatus tsrDestroyArtifact(tsrArtifact a) {
  delete a;
  return TSR_STATUS_SUCCESS;
}
TsrStatus tsrGetArtifactBytes(tsrArtifact a, const void** out_bytes, size_t* out_len) {
  if (!a || !out_bytes || !out_len) return fail(TSR_STATUS_INVALID_ARGUMENT, "null argument");
  *out_bytes = a->payload.data();
  *out_len = a->payload.size();
  return TSR_STATUS_SUCCESS;
}
TsrStatus tsrGetArtifactTarget(tsrArtifact a, const char** out) {
  if (!a || !out) return fail(TSR_STATUS_INVALID_ARGUMENT, "null argument");
  *out = a->target.c_str();
  return TSR_STATUS_SUCCESS;
}
TsrStatus tsrGetKernel(tsrArtifact a, const char* name, tsrKernel* out) {
  if (!a || !name || !out) return fail(TSR_STATUS_INVALID_ARGUMENT, "null argument");
  for (const auto& k : a->kernels)
    if (k == name) {
      *out = new tsrKernel_t{a->target, k};
      return TSR_STATUS_SUCCESS;
    }
  return fail(TSR_STATUS_NOT_FOUND, "artifact has no kernel named %s", name);
}
TsrStatus tsrDestroyKernel(tsrKernel k) {
  delete k;
  return TSR_STATUS_SUCCESS;
}

// The built-in launcher as a public symbol, so another runtime that implements the same
// registry (the reference's libtessera_runtime) can register it.
TsrStatus tessera_sm100_gpu_launcher(const char* target, const char* kernel_name,
                                     const tsrGpuLaunchParams* params, void* user) {
  return builtin_launcher(target, kernel_name, params, user);
}

// The cudaStream_t of the tsrLaunchKernel call that is running the calling launcher (NULL = the
// default stream, also outside a launch).
void* tessera_sm100_current_launch_stream(void) { return t_launch_stream; }

TsrStatus tsrRegisterGpuLauncher(tsrGpuLauncherFn fn, void* user) {
  std::lock_guard<std::mutex> lk(g_mu);
  g_launcher = fn ? fn : (g_init ? builtin_launcher : nullptr);
  g_launcher_user = fn ? user : nullptr;
  return TSR_STATUS_SUCCESS;
}

TsrStatus tsrLaunchKernel(tsrStream s, tsrKernel kernel, void** args, size_t nargs) {
  const uint64_t t = now_ns();
  if (!kernel || !args || nargs < 1 || !args[0])
    return fail(TSR_STATUS_INVALID_ARGUMENT, "kernel/args==NULL or nargs < 1");
  tsrGpuLauncherFn fn;
  void* user;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    fn = g_launcher;
    user = g_launcher_user;
  }
  TsrStatus st;
  if (!fn) {
    st = fail(TSR_STATUS_UNIMPLEMENTED, "no GPU launcher is registered (call tsrInit)");
  } else {
    if (s) cudaSetDevice(s->device);
    t_launch_stream = s ? static_cast<void*>(s->stream) : nullptr;
    st = fn(kernel->target.c_str(), kernel->name.c_str(),
            static_cast<const tsrGpuLaunchParams*>(args[0]), user);
    t_launch_stream = nullptr;
    if (st == TSR_STATUS_NOT_FOUND)
      st = fail(TSR_STATUS_UNIMPLEMENTED, "no launcher handles kernel %s on target %s",
                kernel->name.c_str(), kernel->target.c_str());
  }
  std::string extra = "\"kernel\":\"" + kernel->name + "\",\"target\":\"" + kernel->target + "\"";
  emit(TSR_PROFILE_RUNTIME_API, "tsrLaunchKernel", t, st, extra);
  emit(TSR_PROFILE_DEVICE_ACTIVITY, kernel->name.c_str(), t, st, extra);
  return st;
}

}  // extern "C"
