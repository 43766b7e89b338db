// Chunk-submission runtime for collectives: a bounded number of chunks in flight (QoS tokens), a
// size/path policy tag per chunk, and a Chrome/Perfetto trace of every chunk's life — the C hooks
// the reference's lowered QoS ops call (src/collectives/include/tessera/Dialect/Collective/
// Runtime/Execution.h:103-121; behaviour of lib/Dialect/Collective/Runtime/Execution.cpp).
//
// What differs from the reference: a chunk submitted for a (device, stream id) that has a CUDA
// stream bound to it (tessera_sm100_comm_bind_stream) completes when that stream reaches the
// submission point (cudaLaunchHostFunc), so the token count really bounds the chunks queued on
// the GPU; with no stream bound a chunk completes at once, as the reference's adapters do.
//
// Lifetime: the runtime is a process singleton behind a shared_ptr. The slot mutex is held only
// to read or replace the pointer, never across a submission (a submitter may block on a token),
// and every pending completion owns a reference, so tessera_shutdown_runtime() during a
// submission is safe and the next call builds a fresh runtime.
#include <cuda_runtime.h>

#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/tessera_collectives.h"

namespace tsb {
namespace comm_rt {

class TokenLimiter {
 public:
  explicit TokenLimiter(int tokens) : max_(tokens < 1 ? 1 : tokens) {}
  void set(int tokens) {
    std::lock_guard<std::mutex> g(mu_);
    max_ = tokens < 1 ? 1 : tokens;
    cv_.notify_all();
  }
  void acquire() {
    std::unique_lock<std::mutex> lk(mu_);
    cv_.wait(lk, [&] { return inflight_ < max_; });
    ++inflight_;
    if (inflight_ > peak_) peak_ = inflight_;
  }
  void release() {
    std::lock_guard<std::mutex> g(mu_);
    if (inflight_ > 0) --inflight_;
    cv_.notify_one();
  }
  void snapshot(int* max, int* inflight, int* peak) {
    std::lock_guard<std::mutex> g(mu_);
    *max = max_;
    *inflight = inflight_;
    *peak = peak_;
  }

 private:
  int max_, inflight_ = 0, peak_ = 0;
  std::mutex mu_;
  std::condition_variable cv_;
};

// Size classes and link choice, overridable from the environment like the reference's Policy
// (Policy.h:22-52): TESSERA_COMM_SMALL_MAX, TESSERA_COMM_LARGE_MIN, TESSERA_COMM_INTRA_PATH.
struct Policy {
  uint64_t small_max = 256ull << 10, large_min = 8ull << 20;
  bool intra_nvlink = true;
  static Policy from_env() {
    Policy p;
    if (const char* s = std::getenv("TESSERA_COMM_SMALL_MAX")) p.small_max = std::strtoull(s, nullptr, 10);
    if (const char* s = std::getenv("TESSERA_COMM_LARGE_MIN")) p.large_min = std::strtoull(s, nullptr, 10);
    if (const char* s = std::getenv("TESSERA_COMM_INTRA_PATH")) p.intra_nvlink = std::string(s) != "pcie";
    return p;
  }
  const char* algo(uint64_t bytes) const { return bytes >= large_min ? "ring" : "tree"; }
  const char* path() const { return intra_nvlink ? "NVLINK" : "PCIE"; }
};

struct Event {
  char ph;  // 'B', 'E', 'C'
  int pid, tid;
  double ts_us;
  uint64_t bytes;
  const char* algo;
  const char* path;
};

class Trace {
 public:
  void add(char ph, int pid, int tid, uint64_t bytes = 0, const char* algo = "", const char* path = "") {
    const double ts = std::chrono::duration<double, std::micro>(
                          std::chrono::steady_clock::now().time_since_epoch()).count();
    std::lock_guard<std::mutex> g(mu_);
    events_.push_back(Event{ph, pid, tid, ts, bytes, algo, path});
  }
  bool write(const char* file) {
    std::vector<Event> ev;
    {
      std::lock_guard<std::mutex> g(mu_);
      ev = events_;
    }
    FILE* f = std::fopen(file, "w");
    if (!f) return false;
    std::fprintf(f, "{\"traceEvents\":[");
    bool first = true;
    for (const Event& e : ev) {
      std::fprintf(f, "%s\n", first ? "" : ",");
      first = false;
      if (e.ph == 'C') {
        std::fprintf(f, "{\"name\":\"chunk_bytes\",\"cat\":\"counter\",\"ph\":\"C\",\"pid\":%d,\"tid\":%d,"
                        "\"ts\":%.3f,\"args\":{\"value\":%llu}}",
                     e.pid, e.tid, e.ts_us, (unsigned long long)e.bytes);
      } else if (e.ph == 'B') {
        std::fprintf(f, "{\"name\":\"CommChunk\",\"cat\":\"comm\",\"ph\":\"B\",\"pid\":%d,\"tid\":%d,"
                        "\"ts\":%.3f,\"args\":{\"schema\":\"tessera.telemetry.v1\","
                        "\"source\":\"collective_runtime\",\"op\":\"collective\","
                        "\"kernel_id\":\"collective_chunk\",\"status\":\"ok\",\"path\":\"%s\","
                        "\"algo\":\"%s\",\"memory_bytes\":%llu}}",
                     e.pid, e.tid, e.ts_us, e.path, e.algo, (unsigned long long)e.bytes);
      } else {
        std::fprintf(f, "{\"name\":\"CommChunk\",\"cat\":\"comm\",\"ph\":\"E\",\"pid\":%d,\"tid\":%d,"
                        "\"ts\":%.3f}",
                     e.pid, e.tid, e.ts_us);
      }
    }
    std::fprintf(f, "\n],\"displayTimeUnit\":\"ns\"}\n");
    return std::fclose(f) == 0;
  }
  size_t size() {
    std::lock_guard<std::mutex> g(mu_);
    return events_.size();
  }

 private:
  std::mutex mu_;
  std::vector<Event> events_;
};

struct Runtime {
  explicit Runtime(int tokens) : limiter(tokens), policy(Policy::from_env()) {}
  TokenLimiter limiter;
  Policy policy;
  Trace trace;
  std::mutex mu;                                   // guards `streams`
  std::map<std::pair<int, int>, cudaStream_t> streams;
  static constexpr int kPidBase = 1000;
};

std::mutex g_slot_mu;
std::shared_ptr<Runtime> g_slot;

std::shared_ptr<Runtime> grab(int tokens) {
  std::lock_guard<std::mutex> lk(g_slot_mu);
  if (!g_slot) g_slot = std::make_shared<Runtime>(tokens);
  return g_slot;
}

struct Pending {
  std::shared_ptr<Runtime> rt;  // keeps limiter and trace alive until the chunk completes
  int pid, tid;
};

void complete(Pending* p) {
  p->rt->trace.add('E', p->pid, p->tid);
  p->rt->limiter.release();
  delete p;
}

void CUDART_CB on_stream(void* user) { complete(static_cast<Pending*>(user)); }

}  // namespace comm_rt
}  // namespace tsb

using namespace tsb::comm_rt;

extern "C" {

void tessera_qos_limit_set(int tokens) {
  if (tokens < 1) tokens = 1;  // zero tokens would block every later submitter for good
  grab(tokens)->limiter.set(tokens);
}

void tessera_qos_acquire() { (void)grab(1); }  // tokens are taken by the submission itself

void tessera_qos_release() {}  // and returned by its completion

void tessera_submit_chunk_async(const void* ptr, uint64_t bytes, int device, int stream) {
  (void)ptr;
  std::shared_ptr<Runtime> rt = grab(1);  // slot mutex released here
  rt->limiter.acquire();                  // may block; no global lock is held
  const int pid = Runtime::kPidBase + device, tid = stream;
  rt->trace.add('B', pid, tid, bytes, rt->policy.algo(bytes), rt->policy.path());
  rt->trace.add('C', pid, tid, bytes);
  cudaStream_t bound = nullptr;
  bool has = false;
  {
    std::lock_guard<std::mutex> g(rt->mu);
    auto it = rt->streams.find({device, stream});
    if (it != rt->streams.end()) {
      bound = it->second;
      has = true;
    }
  }
  Pending* p = new Pending{rt, pid, tid};
  if (has && cudaLaunchHostFunc(bound, on_stream, p) == cudaSuccess) return;
  if (has) cudaGetLastError();
  complete(p);
}

int tessera_trace_write_status(const char* path) {
  std::shared_ptr<Runtime> rt;
  {
    std::lock_guard<std::mutex> lk(g_slot_mu);
    rt = g_slot;
  }
  if (!rt || !path) return 2;
  return rt->trace.write(path) ? 0 : 3;
}

void tessera_trace_write(const char* path) { (void)tessera_trace_write_status(path); }

void tessera_shutdown_runtime() {
  std::shared_ptr<Runtime> old;
  {
    std::lock_guard<std::mutex> lk(g_slot_mu);
    old.swap(g_slot);
  }
  // `old` dies here unless completions still hold it
}

int tessera_sm100_comm_bind_stream(int device, int stream_id, void* stream) {
  std::shared_ptr<Runtime> rt = grab(1);
  std::lock_guard<std::mutex> g(rt->mu);
  if (stream)
    rt->streams[{device, stream_id}] = static_cast<cudaStream_t>(stream);
  else
    rt->streams.erase({device, stream_id});
  return 0;
}

int tessera_sm100_qos_state(int* limit, int* inflight, int* peak_inflight, long long* trace_events) {
  std::shared_ptr<Runtime> rt;
  {
    std::lock_guard<std::mutex> lk(g_slot_mu);
    rt = g_slot;
  }
  int a = 0, b = 0, c = 0;
  if (rt) rt->limiter.snapshot(&a, &b, &c);
  if (limit) *limit = a;
  if (inflight) *inflight = b;
  if (peak_inflight) *peak_inflight = c;
  if (trace_events) *trace_events = rt ? (long long)rt->trace.size() : 0;
  return rt ? 0 : 2;
}

}  // extern "C"
