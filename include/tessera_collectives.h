/* Chunk-submission hooks for collectives: QoS tokens, policy tags and a trace of every chunk.
 *
 * These are the extern "C" entry points the reference's lowered QoS ops call
 * (src/collectives/include/tessera/Dialect/Collective/Runtime/Execution.h:103-121, implemented in
 * src/collectives/lib/Dialect/Collective/Runtime/Execution.cpp); same names, argument meaning and
 * void returns. The NCCL collectives themselves are in tessera_sm100.h.
 *
 * All functions are thread-safe; none throws; none needs a GPU unless a CUDA stream was bound. */
#ifndef TESSERA_COLLECTIVES_H
#define TESSERA_COLLECTIVES_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* At most `tokens` chunks in flight (values below 1 are taken as 1: zero would block every later
 * submitter). Shrinking below the number in flight takes effect as chunks complete
 * (TokenLimiter.h:11-22). Creates the runtime on first use. */
void tessera_qos_limit_set(int tokens);
/* Kept for symmetry with the lowered ops: a token is taken by tessera_submit_chunk_async itself
 * and returned when that chunk completes (Execution.cpp:73-81). */
void tessera_qos_acquire(void);
void tessera_qos_release(void);

/* Submits one chunk of a transfer: blocks until a token is free, records a "CommChunk" begin
 * event (pid 1000 + device, tid stream; args: path NVLINK|PCIE, algo tree|ring by size, bytes) and
 * a chunk_bytes counter, and records the end event and returns the token when the chunk
 * completes. Completion is immediate (as with the reference's adapters, Adapters.h:396-400)
 * unless a CUDA stream is bound to (device, stream) — then it happens when that stream reaches
 * this point, so the limit bounds the chunks actually queued on the GPU.
 * Environment (read when the runtime is created, Policy.h:30-41): TESSERA_COMM_SMALL_MAX,
 * TESSERA_COMM_LARGE_MIN (bytes), TESSERA_COMM_INTRA_PATH=nvlink|pcie. */
void tessera_submit_chunk_async(const void* ptr, uint64_t bytes, int device, int stream);

/* Writes the events recorded so far as Chrome-trace JSON ({"traceEvents":[...]}). A no-op when no
 * runtime exists. tessera_trace_write_status is the same with a result: 0 written, 2 no runtime or
 * null path, 3 the file could not be written (no reference counterpart: the reference returns
 * void). */
void tessera_trace_write(const char* path);
int tessera_trace_write_status(const char* path);

/* Drops the process-wide runtime (no-op if there is none). Safe while other threads submit: each
 * pending chunk keeps the old runtime alive until it completes; the next call builds a fresh one
 * (Execution.h:108-119). */
void tessera_shutdown_runtime(void);

/* No reference counterpart. Binds a CUDA stream handle to the (device, stream id) pair used by
 * tessera_submit_chunk_async (NULL unbinds). The caller keeps the stream alive while bound. */
int tessera_sm100_comm_bind_stream(int device, int stream_id, void* stream);
/* No reference counterpart. Current token limit, chunks in flight, the highest in-flight count
 * seen and the number of trace events; returns 2 (and zeros) when no runtime exists. */
int tessera_sm100_qos_state(int* limit, int* inflight, int* peak_inflight, long long* trace_events);

#ifdef __cplusplus
}
#endif
#endif
