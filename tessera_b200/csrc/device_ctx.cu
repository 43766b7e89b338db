#include "device_ctx.h"

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <atomic>
#include <vector>

namespace tsb {

namespace {
thread_local std::string g_last_error;

// A cached block and the events that must have completed before it may be handed out again
// (none: free for any stream).
struct FreeBlock {
  void* ptr = nullptr;
  std::vector<cudaEvent_t> pending;
};
struct DeviceState {
  int* err_word = nullptr;
  int sm_count = 0;
  std::multimap<size_t, FreeBlock> free_blocks;  // size -> block
  std::map<void*, size_t> live_blocks;           // block -> size
  std::vector<cudaEvent_t> spare_events;         // recycled (timing disabled)
  std::vector<cudaStream_t> streams;             // streams the library created on this device
};
std::mutex g_mu;
std::atomic<long long> g_launches{0};
std::map<int, DeviceState> g_devices;

DeviceState& state_locked(int dev) { return g_devices[dev]; }

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
std::once_flag g_encode_once;

void resolve_encode() {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &fn, 12000, cudaEnableDefault,
                                       &q) == cudaSuccess &&
      q == cudaDriverEntryPointSuccess) {
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
}
}  // namespace

void set_last_error(const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_last_error = buf;
}
const char* last_error() { return g_last_error.c_str(); }

void note_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
long long launch_count() { return g_launches.load(std::memory_order_relaxed); }

int ensure_device() {
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n <= 0) {
    cudaGetLastError();
    set_last_error("no usable CUDA device (%s)", e == cudaSuccess ? "count is 0"
                                                                   : cudaGetErrorString(e));
    return kNoDevice;
  }
  e = cudaFree(nullptr);  // forces context creation on the current device
  if (e != cudaSuccess) {
    cudaGetLastError();
    set_last_error("CUDA context creation failed: %s", cudaGetErrorString(e));
    return kNoDevice;
  }
  return kOk;
}

int current_device() {
  int d = 0;
  cudaGetDevice(&d);
  return d;
}

int sm_count() {
  int dev = current_device();
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceState& s = state_locked(dev);
  if (s.sm_count == 0) {
    cudaDeviceGetAttribute(&s.sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (s.sm_count <= 0) s.sm_count = 148;
  }
  return s.sm_count;
}

int* device_err_word() {
  int dev = current_device();
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceState& s = state_locked(dev);
  if (!s.err_word) {
    if (cudaMalloc(&s.err_word, 4 * sizeof(int)) != cudaSuccess) {
      cudaGetLastError();
      s.err_word = nullptr;
      return nullptr;
    }
    cudaMemset(s.err_word, 0, 4 * sizeof(int));
  }
  return s.err_word;
}

int consume_device_err(int out[4]) {
  int* w = device_err_word();
  int host[4] = {0, 0, 0, 0};
  if (!w) return 0;
  if (cudaMemcpy(host, w, sizeof(host), cudaMemcpyDeviceToHost) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  if (host[0] != 0) cudaMemset(w, 0, sizeof(host));
  if (out) memcpy(out, host, sizeof(host));
  return host[0];
}

namespace {
// True once every pending event of the block has completed; completed events are recycled.
bool block_ready_locked(DeviceState& s, FreeBlock& b) {
  while (!b.pending.empty()) {
    if (cudaEventQuery(b.pending.back()) != cudaSuccess) {
      cudaGetLastError();  // cudaErrorNotReady is not sticky, but clear it anyway
      return false;
    }
    s.spare_events.push_back(b.pending.back());
    b.pending.pop_back();
  }
  return true;
}
}  // namespace

void* pool_alloc(size_t bytes) {
  if (bytes == 0) bytes = 256;
  bytes = (bytes + 255) & ~size_t(255);
  int dev = current_device();
  {
    std::lock_guard<std::mutex> lk(g_mu);
    DeviceState& s = state_locked(dev);
    // Reuse a cached block unless it would waste more than half of itself; skip blocks whose
    // last use has not finished on the stream it was freed on.
    for (auto it = s.free_blocks.lower_bound(bytes); it != s.free_blocks.end() && it->first <= 2 * bytes; ++it) {
      if (!block_ready_locked(s, it->second)) continue;
      void* p = it->second.ptr;
      s.live_blocks[p] = it->first;
      s.free_blocks.erase(it);
      return p;
    }
  }
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    pool_release_all();
    e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) {
      cudaGetLastError();
      set_last_error("cudaMalloc(%zu) failed: %s", bytes, cudaGetErrorString(e));
      return nullptr;
    }
  }
  std::lock_guard<std::mutex> lk(g_mu);
  state_locked(dev).live_blocks[p] = bytes;
  return p;
}

namespace {
// Moves a live block to the free list; `streams` are the streams whose queued work may still use it.
void pool_free_on(void* p, const cudaStream_t* streams, int n, bool all_known) {
  if (!p) return;
  int dev = current_device();
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceState& s = state_locked(dev);
  auto it = s.live_blocks.find(p);
  if (it == s.live_blocks.end()) return;
  FreeBlock b;
  b.ptr = p;
  auto mark = [&](cudaStream_t st) {
    cudaEvent_t ev = nullptr;
    if (!s.spare_events.empty()) {
      ev = s.spare_events.back();
      s.spare_events.pop_back();
    } else if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) {
      cudaGetLastError();
      ev = nullptr;
    }
    if (ev && cudaEventRecord(ev, st) == cudaSuccess) {
      b.pending.push_back(ev);
    } else {
      // No event to order the reuse by: wait for the stream here instead.
      cudaGetLastError();
      if (ev) s.spare_events.push_back(ev);
      cudaStreamSynchronize(st);
    }
  };
  for (int i = 0; i < n; ++i) mark(streams[i]);
  if (all_known) {
    mark(nullptr);  // the legacy default stream (it also waits for every blocking stream)
    for (cudaStream_t st : s.streams) mark(st);
  }
  s.free_blocks.emplace(it->second, std::move(b));
  s.live_blocks.erase(it);
}
}  // namespace

void pool_free(void* p) { pool_free_on(p, nullptr, 0, false); }
void pool_free_after(void* p, cudaStream_t stream) { pool_free_on(p, &stream, 1, false); }
void pool_free_after_all(void* p) { pool_free_on(p, nullptr, 0, true); }

void pool_note_stream(cudaStream_t stream, bool created) {
  int dev = current_device();
  std::lock_guard<std::mutex> lk(g_mu);
  auto& v = state_locked(dev).streams;
  if (created) {
    v.push_back(stream);
  } else {
    for (auto& kv : g_devices) {
      auto& w = kv.second.streams;
      for (size_t i = 0; i < w.size(); ++i)
        if (w[i] == stream) {
          w.erase(w.begin() + i);
          break;
        }
    }
  }
}

void pool_release_all() {
  int dev = current_device();
  std::vector<FreeBlock> victims;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    DeviceState& s = state_locked(dev);
    for (auto& kv : s.free_blocks) victims.push_back(std::move(kv.second));
    s.free_blocks.clear();
  }
  for (FreeBlock& b : victims) {
    for (cudaEvent_t ev : b.pending) {
      cudaEventSynchronize(ev);
      cudaEventDestroy(ev);
    }
    cudaFree(b.ptr);
  }
}

bool encode_tmap(CUtensorMap* out, CUtensorMapDataType dtype, int rank, const void* base,
                 const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                 CUtensorMapSwizzle swizzle) {
  std::call_once(g_encode_once, resolve_encode);
  if (!g_encode) {
    set_last_error("cuTensorMapEncodeTiled is not available from the driver");
    return false;
  }
  cuuint64_t gdims[5];
  cuuint64_t gstrides[4];
  cuuint32_t gbox[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
  }
  for (int i = 0; i + 1 < rank; ++i) gstrides[i] = strides_bytes[i];
  CUresult r = g_encode(out, dtype, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdims,
                        gstrides, gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error(
        "cuTensorMapEncodeTiled failed (CUresult %d): rank %d base %p dims [%llu,%llu,%llu] "
        "stride0 %llu box [%u,%u,%u]",
        static_cast<int>(r), rank, base, (unsigned long long)dims[0],
        (unsigned long long)(rank > 1 ? dims[1] : 0), (unsigned long long)(rank > 2 ? dims[2] : 0),
        (unsigned long long)(rank > 1 ? strides_bytes[0] : 0), box[0], rank > 1 ? box[1] : 0,
        rank > 2 ? box[2] : 0);
    return false;
  }
  return true;
}

}  // namespace tsb
