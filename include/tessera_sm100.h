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
#define TESSERA_SM100_U8 3  /* collectives only */
#define TESSERA_SM100_I32 4 /* collectives only */

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
/* Self-test of the failure path every kernel shares: one warp waits, through the kernels' bounded
 * mbarrier wait, on a barrier nobody arrives on; after limit_cycles SM cycles (at most 2^28) it
 * gives up, records {5, block 0, detail 77} in the error word and the kernel ends normally. */
int tessera_sm100_selftest_wait_expiry(long long limit_cycles, void* stream);

/* Helpers with the shape of tessera_nvidia_device_alloc ... tessera_nvidia_event_destroy
 * (tessera_nvidia_gemm.cpp:617-697). */
int tessera_sm100_device_alloc(void** out, size_t bytes);
int tessera_sm100_device_free(void* ptr);
/* Caching device allocator: blocks are recycled without cudaFree. A block may be freed as soon as
 * the work that uses it has been ENQUEUED; it is handed out again only when that work has finished:
 * pool_free orders the reuse after everything queued so far on the legacy default stream and on
 * every stream made by tessera_sm100_stream_create / tsrCreateStream, pool_free_async after the one
 * given stream (cheaper; the form for a stream this library did not create). */
int tessera_sm100_pool_alloc(void** out, size_t bytes);
int tessera_sm100_pool_free(void* ptr);
int tessera_sm100_pool_free_async(void* ptr, void* stream);
int tessera_sm100_pool_release(void);
int tessera_sm100_device_memset(void* ptr, int value, size_t bytes, void* stream);
int tessera_sm100_device_upload(void* dst, const void* src, size_t bytes, void* stream);
int tessera_sm100_device_download(void* dst, const void* src, size_t bytes, void* stream);
int tessera_sm100_device_copy(void* dst, const void* src, size_t bytes, void* stream);
/* Strided device-to-device copy of `rows` rows of `width_bytes` bytes. */
int tessera_sm100_device_copy_2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch,
                                 size_t width_bytes, size_t rows, void* stream);
/* rows x width_bytes from device memory (pitch src_pitch) into host memory (pitch dst_pitch). */
int tessera_sm100_device_download_2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch,
                                     size_t width_bytes, size_t rows, void* stream);
int tessera_sm100_host_alloc(void** out, size_t bytes); /* pinned host memory */
int tessera_sm100_host_free(void* ptr);
int tessera_sm100_stream_create(void** out);
int tessera_sm100_stream_destroy(void* stream);
int tessera_sm100_stream_synchronize(void* stream);
int tessera_sm100_device_synchronize(void);
int tessera_sm100_event_create(void** out);
int tessera_sm100_event_destroy(void* event);
int tessera_sm100_event_record(void* event, void* stream);
int tessera_sm100_stream_wait_event(void* stream, void* event);
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
 * Covers tessera.ops.batched_gemm (python/tessera/__init__.py:252-254).
 * Problems of 32 MB and more are cut into row chunks (batch entries when batch > 1) that flow
 * through upload, compute and download streams, so with page-locked host buffers the call costs
 * about the larger transfer direction instead of upload + kernel + download.
 * TESSERA_SM100_HOST_GEMM_CHUNKS=<1..32> in the environment fixes the number of row chunks. */
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
/* The exchange of the column-parallel GEMM on its own: this rank's column block of its copy of the
 * row-major matrix [rows, N_total] is stored into every other rank's copy with 16-byte SM stores
 * (copies[i]: base of rank i's copy, a peer pointer for i != rank). What bench.py times, all ranks
 * at once, to get the exchange floor of the fused kernel on the machine it runs on. */
int tessera_sm100_allgather_columns_device(void* const* copies, int world, int rank, int rows,
                                           long long n_total, int elem_bytes, void* stream);
/* SM cycles per tcgen05.mma (K 16, M 128 per CTA) issued back to back on resident shared-memory
 * operands, the maximum over the issuing CTAs of one full-GPU launch: the arithmetic rate the GEMM
 * and attention main loops are measured against. pair != 0: cta_group::2 on clusters of two (M 256).
 * N: 64, 128 or 256 (128 or 256 for pairs). b_mn_major: layout of the B operand. Synchronous. */
int tessera_sm100_probe_mma_rate(int pair, int N, int b_mn_major, int reps, double* cycles_per_mma);
/* D[M,N] = act(A*B + bias[col] + residual[row,col]) with the bias / residual / activation applied in
 * the kernel epilogue: tessera.ops.gemm(A, B, epilogue={...}) -> fused_epilogue
 * (python/tessera/__init__.py:239-248, 2658-2675; the reference's GPU lane for it is the emitted
 * tessera_nvidia_mma_fused kernel, python/tessera/compiler/emit/nvidia_cuda.py:3446-3548).
 * bias: fp32 [N] or NULL. residual: [M,N] in the output dtype or NULL. activation: 0 none, 1 relu,
 * 2 gelu (tanh form), 3 silu. K and N multiples of 8. */
int tessera_sm100_gemm_epilogue_device(const void* A, const void* B, void* D, int M, int N, int K,
                                       int in_dtype, int out_dtype, const float* bias,
                                       const void* residual, int activation, void* stream);
/* Column-parallel GEMM with the all-gather of Y fused into the epilogue
 * (Y = all_gather(A @ W_r, axis=1), python/tessera/compiler/tensor_parallel.py:118-123): rank r
 * multiplies columns [r*N/world, (r+1)*N/world) of the full B[K,N] and TMA-stores every output
 * tile into all `world` copies of Y. Y_ptrs[i] is rank i's Y base (a CUDA-IPC-mapped peer pointer
 * for i != rank, see tessera_sm100_ipc_*). Each copy is complete once every rank's kernel has
 * finished, so ranks synchronise their streams and then meet at a host barrier. world <= 8.
 * With at most four ranks, fewer than four waves of tiles and at least 16 k-blocks of 64, the first
 * wave of work units are half-K units shared by two neighbouring CTA pairs (fp32 partial sums through a workspace taken
 * from the library's pool for the duration of the launch), so the first stores leave after half a
 * tile time. */
int tessera_sm100_gemm_allgather_device(const void* A, const void* B, void* const* Y_ptrs, int world,
                                        int rank, int M, int N_total, int K, int in_dtype,
                                        int out_dtype, void* stream);
/* The same with only this rank's column block resident: B_block is [K, N_total / world] with leading
 * dimension ldb (elements, a multiple of 8), as ParallelLinear holds its weight shard
 * (python/tessera/compiler/tensor_parallel.py:87-89). */
int tessera_sm100_gemm_allgather_block_device(const void* A, const void* B_block, long long ldb,
                                              void* const* Y_ptrs, int world, int rank, int M, int N_total,
                                              int K, int in_dtype, int out_dtype, void* stream);

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

/* ---- fp8 (e4m3) operands -------------------------------------------------------------------
 * The quantised grouped GEMM of tessera.ops.grouped_gemm(..., quant="fp8_e4m3")
 * (python/tessera/__init__.py:337-342; python/tessera/compiler/grouped_layout.py:353-392): the
 * reference quantises x per tensor and each expert's weights per expert with quantize_fp8
 * (python/tessera/__init__.py:3340-3374), dequantises on the host and runs an f32 GEMM. Here the
 * e4m3 bytes go to the tensor cores (tcgen05 kind::f8f6f4, f32 accumulate) and the two scales are
 * applied in the epilogue; the result differs from the reference's only by fp32 summation order.
 *
 * tessera_sm100_quantize_fp8_device: x (n elements of `dtype`) -> q (n bytes). scale_out holds 3
 * device floats: [0] scale = max(amax/448, 1e-12), [1] amax, [2] scratch. amax_in (optional): a
 * device uint32 with the bits of a known amax, which skips the reduction pass.
 * tessera_sm100_quantize_fp8_weights_device: w [E,K,N] -> q_t [E,N,K] (TRANSPOSED: both GEMM
 * operands are K-major), one scale per expert; scales holds 3E device floats: [0,E) scales,
 * [E,2E) amax, [2E,3E) scratch. Weights are static: quantise once, reuse.
 * GEMMs: xq [T,K] / Aq [M,K] bytes, wq_t [E,N,K] / Bq_t [N,K] bytes, K a multiple of 16, N of 8;
 * scale_x one device float, scale_w one per expert. The SwiGLU form writes the 16-bit hidden
 * activation silu(x Wg) * (x Wu) and, when amax_out is given (device uint32, zeroed by the
 * caller), max |hidden| as stored, ready for the next quantisation. */
/* 8-bit float formats of the *_fmt_device entry points (quantize_fp8(format=...),
 * python/tessera/__init__.py:3340-3374; grouped quant "fp8_e5m2"): the plain entry points are e4m3. */
#define TESSERA_SM100_FP8_E4M3 0
#define TESSERA_SM100_FP8_E5M2 1
int tessera_sm100_quantize_fp8_fmt_device(const void* x, long long n, int dtype, int fmt, void* q,
                                          float* scale_out, const unsigned int* amax_in, void* stream);
int tessera_sm100_quantize_fp8_weights_fmt_device(const void* w, int E, int K, int N, int dtype, int fmt,
                                                  void* q_t, float* scales, void* stream);
int tessera_sm100_gemm_fp8_fmt_device(const void* Aq, const void* Bq_t, void* D, int M, int N, int K,
                                      const float* scale_a, const float* scale_b, int out_dtype, int fmt,
                                      void* stream);
int tessera_sm100_grouped_gemm_fp8_fmt_device(const void* xq, const void* wq_t, const int* offsets,
                                              void* out, int T, int K, int N, int E, const float* scale_x,
                                              const float* scale_w, int out_dtype, int fmt, void* stream);
int tessera_sm100_grouped_swiglu_fp8_fmt_device(const void* xq, const void* wgq_t, const void* wuq_t,
                                                const int* offsets, void* hidden, int T, int K, int F,
                                                int E, const float* scale_x, const float* scale_wg,
                                                const float* scale_wu, int out_dtype,
                                                unsigned int* amax_out, int fmt, void* stream);
int tessera_sm100_quantize_fp8_device(const void* x, long long n, int dtype, void* q,
                                      float* scale_out, const unsigned int* amax_in, void* stream);
int tessera_sm100_quantize_fp8_weights_device(const void* w, int E, int K, int N, int dtype,
                                              void* q_t, float* scales, void* stream);
int tessera_sm100_gemm_fp8_device(const void* Aq, const void* Bq_t, void* D, int M, int N, int K,
                                  const float* scale_a, const float* scale_b, int out_dtype,
                                  void* stream);
int tessera_sm100_grouped_gemm_fp8_device(const void* xq, const void* wq_t, const int* offsets,
                                          void* out, int T, int K, int N, int E,
                                          const float* scale_x, const float* scale_w,
                                          int out_dtype, void* stream);
int tessera_sm100_grouped_swiglu_fp8_device(const void* xq, const void* wgq_t, const void* wuq_t,
                                            const int* offsets, void* hidden, int T, int K, int F,
                                            int E, const float* scale_x, const float* scale_wg,
                                            const float* scale_wu, int out_dtype,
                                            unsigned int* amax_out, void* stream);

/* ---- NVFP4 expert weights (quant = "nvfp4", "fp8xfp4") ----------------------------------------
 * The reference's grouped GEMM with quant="nvfp4" / "fp8xfp4" quantises and dequantises on the host
 * and multiplies in f32 (python/tessera/__init__.py:337-351; python/tessera/compiler/grouped_layout.py:
 * 319-392): NVFP4 = e2m1 codes in blocks of 16 along the LAST axis with one e4m3 scale per block,
 * scale = e4m3(max(amax/6, 1e-30)) (python/tessera/compiler/microscaling.py:319-362); for expert
 * weights [E,K,N] the blocks therefore run along N, which no block-scaled MMA consumes, so the
 * weights are kept packed at rest (4.5 bits per element) and expanded to bf16 for the GEMM: an e2m1
 * value times an e4m3 scale has at most 5 significant bits, so bf16 holds it exactly and the bf16
 * tensor-core GEMM forms exactly the reference's products. e4m3 activations ride as bf16 too
 * (tessera_sm100_fp8_to_bf16_device, fmt 0 = e4m3, 1 = e5m2) with their per-tensor scale applied to the fp32 accumulators by
 * the *_scaled_device grouped GEMMs (scale_a: one device float, or NULL for 1).
 * quantize: x [rows, cols] (cols % 16 == 0) -> codes [rows, cols/2] (two codes per byte, even element
 * in the low nibble) and scales [rows, cols/16] e4m3 bytes; weights: rows = E*K, cols = N. */
int tessera_sm100_quantize_nvfp4_device(const void* x, long long rows, long long cols, int dtype,
                                        void* codes, void* scales, void* stream);
int tessera_sm100_dequantize_nvfp4_device(const void* codes, const void* scales, long long rows,
                                          long long cols, void* out, int out_dtype, void* stream);
int tessera_sm100_fp8_to_bf16_device(const void* q, long long n, int fmt, void* out, void* stream);
int tessera_sm100_grouped_gemm_scaled_device(const void* x, const void* w, const int* offsets, void* out,
                                             int T, int K, int N, int E, int in_dtype, int out_dtype,
                                             const float* scale_a, void* stream);
int tessera_sm100_grouped_swiglu_scaled_device(const void* x, const void* w_gate, const void* w_up,
                                               const int* offsets, void* out, int T, int K, int F, int E,
                                               int in_dtype, int out_dtype, const float* scale_a,
                                               void* stream);

/* ---- MoE layer pieces --------------------------------------------------------------------
 * Router: top-k over f32 gate logits [T,E]; selection order and tie rule of route_tokens
 * (python/tessera/distributed/moe.py:160-172: descending, the higher expert index first on a
 * tie); weights are f32 softmax probabilities, renormalised over the top-k when `normalize`.
 * assignment [T,top_k] int32, weights [T,top_k] f32. */
int tessera_sm100_moe_route_device(const float* logits, int T, int E, int top_k, int normalize,
                                   int* assignment, float* weights, void* stream);
/* Stable expert sort of the token-major slots with the capacity rule of route_tokens
 * (python/tessera/distributed/moe.py:185-199; capacity < 0 = unlimited; dropped slots get
 * assignment -1 / weight 0 in place). Outputs are the canonical int32 transport arrays
 * (python/tessera/compiler/moe_transport.py:75-134): token_of_slot, expert_of_slot,
 * weight_of_slot (length = kept slots), group_sizes[E], group_offsets[E+1], plus
 * slot_of_assignment[T*top_k] (sorted position of each slot, -1 if dropped). E <= 256. */
int tessera_sm100_moe_permute_device(int* assignment, float* weights, int T, int top_k, int E,
                                     int capacity, int* token_of_slot, int* expert_of_slot,
                                     float* weight_of_slot, int* group_sizes, int* group_offsets,
                                     int* slot_of_assignment, void* stream);
/* o[s,:] = x[tok[s],:]: the dispatch gather, argument order of tessera_nvidia_moe_dispatch_f32
 * (x, tok, o, T, S, H) (python/tessera/compiler/emit/nvidia_cuda.py:1530). */
int tessera_sm100_moe_dispatch_device(const void* x, const int* tok, void* o, int T, int S, int H,
                                      int dtype, void* stream);
/* out[t,:] = sum_j weights[t,j] * y[slot_of_assignment[t,j],:] in j order (deterministic); the
 * combine of python/tessera/nn/functional.py:487-490. */
int tessera_sm100_moe_combine_device(const void* y, const int* slot_of_assignment,
                                     const float* weights, void* out, int T, int top_k, int H,
                                     int y_dtype, int out_dtype, void* stream);
/* o[tok[s],:] += w[s] * x[s,:] after zeroing o: tessera_nvidia_moe_combine_f32's contract
 * (x, tok, w, o, T, S, H) (python/tessera/compiler/emit/nvidia_cuda.py:1531) on device memory. */
int tessera_sm100_moe_combine_scatter_f32_device(const float* x, const int* tok, const float* w,
                                                 float* o, int T, int S, int H, void* stream);
/* Whole layer: route -> permute -> dispatch -> grouped SwiGLU GEMM -> grouped down GEMM ->
 * combine (python/tessera/nn/functional.py:403-490 with the router logits given). x [T,H],
 * w_gate/w_up [E,H,F], w_down [E,F,H] in `dtype` (bf16/f16), logits f32 [T,E], out [T,H].
 * `workspace` is device scratch of tessera_sm100_moe_workspace_bytes() bytes; the routing
 * products stay in it and can be located with tessera_sm100_moe_workspace_views(). */
size_t tessera_sm100_moe_workspace_bytes(int T, int H, int F, int E, int top_k);
int tessera_sm100_moe_layer_device(const void* x, const float* logits, const void* w_gate,
                                   const void* w_up, const void* w_down, void* out, int T, int H,
                                   int F, int E, int top_k, int normalize, int capacity, int dtype,
                                   int out_dtype, void* workspace, void* stream);
int tessera_sm100_moe_workspace_views(void* workspace, int T, int H, int F, int E, int top_k,
                                      void** assignment, void** weights, void** token_of_slot,
                                      void** expert_of_slot, void** weight_of_slot,
                                      void** group_sizes, void** group_offsets,
                                      void** slot_of_assignment);

/* ---- expert-parallel MoE exchange over peer memory ---------------------------------------------
 * Device-side dispatch and combine for the expert-parallel forward of
 * python/tessera/distributed/moe.py:358-483 (rank r owns experts [r*E/world, (r+1)*E/world)),
 * with no host round trip and no capacity padding. Per rank: sort the local slots by GLOBAL expert
 * with tessera_sm100_moe_permute_device, all-gather its group_sizes[E] into all_counts[world][E],
 * then
 *   ep_plan      -> group_offsets_local[E/world + 1] of the rows this rank will receive
 *                   (expert-major, source-major inside an expert) and dst_base[E]: the first row,
 *                   in the owner's receive buffer, of this rank's block for each expert;
 *   ep_dispatch  -> stores every kept token row into its owner's receive buffer (recv_bufs[i] is
 *                   rank i's buffer, a CUDA-IPC peer pointer for i != rank);
 *   (all ranks run the grouped GEMMs on their receive buffer into y_bufs[rank]);
 *   ep_combine   -> out[t] = sum_j w[t,j] * y_bufs[owner][row of slot (t,j)], j ascending.
 * Ranks must be ordered between the phases (dispatch -> expert GEMMs -> combine -> next dispatch),
 * e.g. by a small stream-ordered NCCL all-reduce. capacity_rows bounds the rows of each buffer. */
int tessera_sm100_ep_plan_device(const int* all_counts, int world, int rank, int E,
                                 int* group_offsets_local, int* dst_base, void* stream);
int tessera_sm100_ep_dispatch_device(const void* x, const int* token_of_slot,
                                     const int* expert_of_slot, const int* my_offsets,
                                     const int* dst_base, void* const* recv_bufs, int world, int E,
                                     int max_slots, int capacity_rows, int H, int dtype, void* stream);
int tessera_sm100_ep_combine_device(void* const* y_bufs, const int* assignment,
                                    const int* slot_of_assignment, const float* weights,
                                    const int* my_offsets, const int* dst_base, void* out, int T,
                                    int top_k, int world, int E, int capacity_rows, int H, int dtype,
                                    void* stream);
/* The same exchange with the ranks ordered by flags in peer memory instead of collectives: the
 * form of the reference's planned device-initiated exchange (its mock transport orders the phases
 * with thread barriers, python/tessera/distributed/moe.py:358-483). Every rank allocates one control
 * block of tessera_sm100_ep_ctrl_bytes() bytes, ZEROED ONCE, and maps every peer's block
 * (ctrl_ptrs[i] = rank i's block). `epoch` is 1 on the first forward call and one higher on every
 * following call, the same on all ranks. Per forward, on one stream:
 *   ep_route_publish    route + stable expert sort of the Tl local tokens (one launch; outputs as
 *                       tessera_sm100_moe_route_device + tessera_sm100_moe_permute_device with no
 *                       capacity drop) and this rank's per-expert counts stored into every rank's
 *                       control block;
 *   ep_dispatch_signal  waits for all ranks' counts and for the end of their previous call, writes
 *                       group_offsets_local[E/world + 1] and dst_base[E] (as ep_plan), stores the token
 *                       rows into the owners' receive buffers; when the kernel ends every rank's rows
 *                       for THIS rank have landed, so the grouped GEMMs can follow in the stream;
 *   ep_combine_signal   (after the GEMMs) announces this rank's outputs, waits for the owners', reads
 *                       the result rows back and forms the weighted sums; announces the end of the call.
 * `counter` is one zeroed device int per call site (dispatch and combine each need their own).
 * Waits give up after wait_limit_ms (<= 0: 10 s) and record code 5 in the device error word
 * (detail 100+r counts, 200+r previous call, 300+r rows, 400+r outputs of rank r); the kernels then
 * run to their end without the data. Never run two ranks of one group on the same GPU. */
size_t tessera_sm100_ep_ctrl_bytes(void);
int tessera_sm100_ep_route_publish_device(const float* logits, int Tl, int E, int top_k, int normalize,
                                          int* assignment, float* weights, int* token_of_slot,
                                          int* expert_of_slot, float* weight_of_slot, int* group_sizes,
                                          int* my_offsets, int* slot_of_assignment, void* const* ctrl_ptrs,
                                          int world, int rank, int epoch, void* stream);
int tessera_sm100_ep_dispatch_signal_device(const void* x, const int* token_of_slot,
                                            const int* expert_of_slot, const int* my_offsets,
                                            void* const* ctrl_ptrs, void* const* recv_bufs, int world,
                                            int rank, int E, int max_slots, int capacity_rows, int H,
                                            int dtype, int epoch, int* group_offsets_local, int* dst_base,
                                            int* counter, int wait_limit_ms, void* stream);
int tessera_sm100_ep_combine_signal_device(void* const* y_bufs, void* const* ctrl_ptrs,
                                           const int* assignment, const int* slot_of_assignment,
                                           const float* weights, const int* my_offsets,
                                           const int* dst_base, void* out, int T, int top_k, int world,
                                           int rank, int E, int capacity_rows, int H, int dtype, int epoch,
                                           int* counter, int wait_limit_ms, void* stream);

/* ---- decode attention --------------------------------------------------------------------
 * One query token per sequence against a KV cache: Q,O [B,Hq,1,D], K,V [B,Hkv,Sk,D] bf16,
 * D = 128, query head hq reads KV head hq / (Hq/Hkv) (python/tessera/nn/functional.py:349-356;
 * the reference's CUDA lane has the same mapping, python/tessera/compiler/emit/nvidia_cuda.py:265).
 * splits <= 0 lets the library choose; with more than one split `scratch` must hold
 * tessera_sm100_attn_decode_scratch_bytes(B, Hq, splits) bytes of device memory. */
int tessera_sm100_attn_decode_splits(int B, int Hq, int Hkv, int Sk);
size_t tessera_sm100_attn_decode_scratch_bytes(int B, int Hq, int splits);
int tessera_sm100_attn_decode_device(const void* Q, const void* K, const void* V, void* O, int B,
                                     int Hq, int Hkv, int Sk, int D, float scale, int splits,
                                     void* scratch, void* stream);
/* Decode attention for callers that must not allocate (this entry point has no counterpart in the
 * reference). Same arguments and result as tessera_sm100_attn_decode_device, but the split-KV
 * partials live in a static device array inside the library (8 MiB per GPU, held from library
 * load to process exit) and neither the first call nor any later one calls cudaMalloc, cudaFree
 * or an allocating library routine. It is meant for serving loops whose device-memory budget is
 * fixed at start-up, and for latency-critical decode steps that cannot afford the device-wide
 * synchronisation an allocation implies.
 *  - Limit: B * Hq * splits * 130 * 4 bytes <= 8 MiB when splits > 1 (batch 8 x 32 heads x 4
 *    splits needs 0.5 MiB; the benchmark shape, batch 64, runs as one split and needs none). splits <= 0 picks the library's split count, lowered
 *    until the partials fit; an explicit split count that does not fit returns 1 with an error
 *    text naming the required and the available bytes.
 *  - The first call on each device creates the context if none exists yet (a null cudaFree, the only
 *    allocator call this entry point ever makes, and only then) and resolves the array's device
 *    address with that device current; issue that first call outside any stream capture. Later
 *    calls use the cached address and make no such call.
 *  - All calls share the one array. Calls ordered on a stream are safe; calls that overlap on the
 *    GPU (different streams without ordering) race on it. Nothing in it needs clearing between
 *    calls: every partial a launch reads it has written itself.
 *  - check_previous != 0 first synchronises `stream` and returns 3 if an earlier launch of this
 *    entry point gave up a bounded wait (the error word is static too), clearing the record. */
int tessera_sm100_attn_decode_static_device(const void* Q, const void* K, const void* V, void* O,
                                            int B, int Hq, int Hkv, int Sk, int D, float scale,
                                            int splits, int check_previous, void* stream);

/* General attention forward: the contract of the reference's CUDA attention lane
 * (python/tessera/compiler/emit/nvidia_cuda.py:251-276, ABI :274: q,k,v,bias|NULL,o, B,Hq,Hkv,Sq,Sk,
 * D,Dv, scale, causal, wl, wr, softcap) on device pointers, for f32 / f16 / bf16 storage (dtype
 * code), D and Dv up to 512. bias: f32 [B,Hq,Sq,Sk] or NULL, added after the scale; softcap > 0
 * applies softcap*tanh(s/softcap); key n is masked for query m when (causal && n > m +
 * causal_shift) || (wl >= 0 && n < m - wl) || (wr >= 0 && n > m + wr); a fully masked row gives
 * zeros. causal_shift 0 is the lane's mask, max(Sk - Sq, 0) the bottom-right alignment of
 * tessera.ops.flash_attn. Q [B,Hq,Sq,D], K [B,Hkv,Sk,D], V [B,Hkv,Sk,Dv], O [B,Hq,Sq,Dv], dense. */
int tessera_sm100_flash_attn_general_device(const void* q, const void* k, const void* v,
                                            const float* bias, void* o, long long B, int Hq, int Hkv,
                                            long long Sq, long long Sk, int D, int Dv, float scale,
                                            int causal, long long causal_shift, long long window_left,
                                            long long window_right, float softcap, int dtype,
                                            void* stream);

/* Attention backward (VJP): (dO, Q, K, V [, bias]) -> (dQ, dK, dV), the contract of the reference's
 * CUDA lane (python/tessera/compiler/emit/nvidia_cuda.py:590-635, entry tessera_nvidia_flash_attn_bwd;
 * tests/device/nvidia/test_flash_attention_backward.py:23-50). Masks, bias, soft-cap and head mapping
 * as tessera_sm100_flash_attn_general_device; ds = p (dO.v - delta) (1 - tanh^2) with delta = dO.o;
 * dQ = sum ds scale k, dK = sum over the group's query heads and rows of ds scale q, dV = sum p dO.
 * f32 / f16 / bf16 storage (dtype code), fp32 math, gradients in the storage type, D and Dv up to
 * 256 (the reference's cap). Every output row is summed by one warp in a fixed order: the result is
 * deterministic (the reference's default route uses atomics) and the outputs need no clearing.
 * dO [B,Hq,Sq,Dv], dQ like Q, dK like K, dV like V. workspace: device memory of
 * tessera_sm100_flash_attn_bwd_workspace_bytes(B, Hq, Sq) bytes (softmax statistics per row).
 * tessera_sm100_flash_attn_bwd is the host-pointer form with the reference entry's argument order
 * (upload, run, synchronise, download); its causal mask is the lane's (key n > query m). */
size_t tessera_sm100_flash_attn_bwd_workspace_bytes(long long B, int Hq, long long Sq);
int tessera_sm100_flash_attn_bwd_device(const void* dO, const void* Q, const void* K, const void* V,
                                        const float* bias, void* dQ, void* dK, void* dV, long long B,
                                        int Hq, int Hkv, long long Sq, long long Sk, int D, int Dv,
                                        float scale, int causal, long long causal_shift,
                                        long long window_left, long long window_right, float softcap,
                                        int dtype, void* workspace, void* stream);
int tessera_sm100_flash_attn_bwd(const void* dO, const void* Q, const void* K, const void* V,
                                 const float* bias, void* dQ, void* dK, void* dV, long long B, int Hq,
                                 int Hkv, long long Sq, long long Sk, int D, int Dv, float scale,
                                 int causal, long long window_left, long long window_right,
                                 float softcap, int dtype);

/* The same gradients on the tensor cores for the training shape: bf16, D = Dv = 128, no bias /
 * window / soft-cap, causal with the bottom-right alignment of tessera.ops.flash_attn (key n legal
 * for query m when n <= m + max(Sk - Sq, 0); the lane's mask when Sq >= Sk). It runs the forward
 * kernel once more to get O and each row's log-sum-exp (into the workspace), then delta = dO.O, a
 * dQ kernel (one CTA per 128 query rows) and a dK/dV kernel (one CTA per 128 keys, over the query
 * heads of the KV head): tcgen05 MMA with TMEM accumulators, no atomics, bit-identical reruns
 * workspace: tessera_sm100_flash_attn_bwd_bf16_workspace_bytes(B, Hq, Sq) bytes.
 * tessera_sm100_flash_attn_fwd_lse_device is that forward pass on its own: O plus lse2[B,Hq,Sq] =
 * log2(sum_n exp2(scale*log2(e)*s_n)) over the legal keys (multiply by ln 2 for the natural-log LSE). */
size_t tessera_sm100_flash_attn_bwd_bf16_workspace_bytes(int B, int Hq, int Sq);
int tessera_sm100_flash_attn_bwd_bf16_device(const void* dO, const void* Q, const void* K, const void* V,
                                             void* dQ, void* dK, void* dV, int B, int Hq, int Hkv, int Sq,
                                             int Sk, float scale, int causal, void* workspace,
                                             void* stream);
int tessera_sm100_flash_attn_fwd_lse_device(const void* Q, const void* K, const void* V, void* O,
                                            float* lse2, int B, int Hq, int Hkv, int Sq, int Sk, int D,
                                            float scale, int causal, void* stream);
/* The backward of a step that kept O and lse2 from tessera_sm100_flash_attn_fwd_lse_device: no
 * forward recompute. delta_scratch: B*Hq*Sq device floats. Same gradients, bit for bit. */
int tessera_sm100_flash_attn_bwd_bf16_saved_device(const void* dO, const void* Q, const void* K,
                                                   const void* V, const void* O, const float* lse2,
                                                   void* dQ, void* dK, void* dV, int B, int Hq, int Hkv,
                                                   int Sq, int Sk, float scale, int causal,
                                                   float* delta_scratch, void* stream);

/* ---- max-shifted attention states -----------------------------------------------------------
 * ops.softmax_merge / softmax_finalize (python/tessera/_block_attnres_ops.py:104-146): a state is
 * (o [rows, Dv] = sum e^{s-m} v, m [rows] = max s, l [rows] = sum e^{s-m}), fp32; merging is
 * associative, so attention over a key set that is split (KV splits inside one GPU, KV shards on
 * several GPUs) is merge-then-finalize of the per-part states.
 * tessera_sm100_attn_decode_state_device is the decode kernel stopping before the division: Q
 * [B,Hq,128], K/V [B,Hkv,Sk,128] bf16 -> o_state [B,Hq,128], m_state, l_state [B,Hq] (m in natural
 * log units of the scaled scores). scratch: tessera_sm100_attn_decode_scratch_bytes(B, Hq,
 * max(splits,1)) bytes, always required here. */
int tessera_sm100_attn_decode_state_device(const void* Q, const void* K, const void* V,
                                           float* o_state, float* m_state, float* l_state, int B,
                                           int Hq, int Hkv, int Sk, int D, float scale, int splits,
                                           void* scratch, void* stream);
int tessera_sm100_softmax_merge_device(const float* oa, const float* ma, const float* la,
                                       const float* ob, const float* mb, const float* lb, float* o,
                                       float* m, float* l, long long rows, int Dv, void* stream);
int tessera_sm100_softmax_finalize_device(const float* o, const float* l, void* out, long long rows,
                                          int Dv, int out_dtype, void* stream);

/* ---- int8 KV cache --------------------------------------------------------------------------
 * KVCacheHandle(quantize_bits=8) stores K and V as int8 with one fp32 scale per token, shared by
 * all heads (python/tessera/cache/handle.py:72-215; quantize_kv / dequantize_kv,
 * python/tessera/__init__.py:3196-3265), and reads dequantise. Here decode attention reads the
 * 8-bit values directly — half the bytes of a bf16 cache on a bandwidth-bound kernel. STORAGE
 * FORM: each quantised value q in [-127, 127] is kept as the unsigned byte q + 128 (an int8 array
 * of the reference becomes this with one xor 0x80 per byte). A byte placed under an f16 exponent
 * is then already the f16 number q + 1152, so widening costs two byte permutes per four values;
 * the constant is removed from the dot products in fp32 (exactly linear), and the per-token
 * scales fold into the scores (K) and into P before P.V (V), so the result equals attention
 * over the dequantised cache.
 * Dense: Kq, Vq [B,Hkv,Sk,128] bytes, k_scale, v_scale [B,Sk]. Paged: pages
 * [num_pages,page_size,Hkv,128] bytes, scale pages [num_pages,page_size]; other arguments as the
 * 16-bit entry points. tessera_sm100_quantize_kv_int8_device: k, v [T, row] (row = heads*dim) ->
 * byte rows (q + 128) and scales with the reference's arithmetic (scale = max(amax/127, 1e-12),
 * q = clip(rint(x/scale), -127, 127)); dst_rows (optional device int64[T]) sends token t to row
 * dst_rows[t] of the outputs (a page slot), negative = skip. */
/* The split count the 8-bit kernels pick for splits <= 0 (they want more, shorter CTAs than the
 * 16-bit kernels); size the scratch with tessera_sm100_attn_decode_scratch_bytes(B, Hq, that). */
int tessera_sm100_attn_decode_int8_splits(int B, int Hq, int Hkv, int Sk);
int tessera_sm100_attn_decode_int8_device(const void* Q, const void* Kq, const void* Vq,
                                          const float* k_scale, const float* v_scale, void* O,
                                          int B, int Hq, int Hkv, int Sk, int D, float scale,
                                          int splits, void* scratch, void* stream);
int tessera_sm100_paged_attn_decode_int8_device(const void* Q, const void* k_pages,
                                                const void* v_pages, const float* k_scale,
                                                const float* v_scale, const int* page_table,
                                                const int* seq_lens, void* O, int B, int Hq, int Hkv,
                                                int D, int page_size, int num_pages, int max_pages,
                                                int max_seq_len, float scale, int splits,
                                                void* scratch, void* stream);
int tessera_sm100_quantize_kv_int8_device(const void* k, const void* v, void* kq, void* vq,
                                          float* k_scale, float* v_scale, const long long* dst_rows,
                                          long long T, int row, int dtype, void* stream);

/* Attention forward over strided operands: the same kernels with the layouts described by element
 * strides, one (batch, head, position) triple per tensor; the head dimension (128) is contiguous
 * and every stride is a multiple of 8 elements. Serves nn.functional.multi_head_attention
 * (python/tessera/nn/functional.py:493-548), whose [B, S, H*D] operands the reference reshapes
 * and transposes to [B, H, S, D] and back: here Q, K, V and O are read and written in place
 * (strides {S*H*D, D, H*D}), as are the column slices of a fused QKV projection. Sq == 1 runs the
 * decode kernel, anything else the prefill kernel (tessera_sm100_flash_attn_fwd_strided_device
 * is the prefill kernel alone). */
int tessera_sm100_flash_attn_strided_device(const void* Q, const void* K, const void* V, void* O,
                                            int B, int Hq, int Hkv, int Sq, int Sk, int D,
                                            const long long* q_strides, const long long* k_strides,
                                            const long long* v_strides, const long long* o_strides,
                                            float scale, int causal, void* stream);
int tessera_sm100_flash_attn_fwd_strided_device(const void* Q, const void* K, const void* V, void* O,
                                                int B, int Hq, int Hkv, int Sq, int Sk, int D,
                                                const long long* q_strides,
                                                const long long* k_strides,
                                                const long long* v_strides,
                                                const long long* o_strides, float scale, int causal,
                                                void* stream);

/* ---- paged KV cache ------------------------------------------------------------------------
 * The page ABI of python/tessera/cache/paged_kv.py:91-140 (PagedKVBufferABI): K and V pages are
 * [physical_page, page_offset, head, dim] and page_table[logical_page] names the physical page;
 * attention never infers placement from a logical token index. Storage here is bf16 (the
 * reference's version 1 is f32), head_dim 128, page_size a power of two in [8, 1024], and the
 * table is per sequence so a whole decode batch is one launch: page_table [B, max_pages] int32,
 * seq_lens [B] int32.
 *
 * tessera_sm100_paged_attn_decode_device: one query token per sequence against its pages; replaces
 * ops.paged_attention / cache.paged_kv.paged_attention(backend="nvidia")
 * (python/tessera/__init__.py:1291-1302, python/tessera/cache/paged_kv.py:480-559, 772-788) and
 * the reference's tessera_nvidia_resident_paged_attention
 * (python/tessera/compiler/emit/nvidia_cuda.py:2522, 2533). Q, O [B, Hq, 128] bf16. Every
 * seq_lens[b] must be in [1, max_seq_len]; max_seq_len <= max_pages * page_size sizes the grid.
 * splits / scratch as for tessera_sm100_attn_decode_device (use tessera_sm100_attn_decode_splits
 * with Sk = max_seq_len). A table entry outside [0, num_pages) is read as zeros and recorded in
 * the device error word (tessera_sm100_consume_device_error), never dereferenced. */
int tessera_sm100_paged_attn_decode_device(const void* Q, const void* k_pages, const void* v_pages,
                                           const int* page_table, const int* seq_lens, void* O,
                                           int B, int Hq, int Hkv, int D, int page_size,
                                           int num_pages, int max_pages, int max_seq_len,
                                           float scale, int splits, void* scratch, void* stream);

/* Appends one token per sequence (k_new, v_new [B, Hkv, D] bf16) at position seq_lens[b] and adds
 * one to seq_lens[b] on the device: KVCacheHandle.append for a decode step
 * (python/tessera/cache/handle.py:156-215) against paged storage. A sequence whose table is full
 * is left unchanged and recorded in the device error word. */
int tessera_sm100_paged_kv_append_device(const void* k_new, const void* v_new, void* k_pages,
                                         void* v_pages, const int* page_table, int* seq_lens, int B,
                                         int Hkv, int D, int page_size, int num_pages,
                                         int max_pages, void* stream);

/* out[x, h, :] = pages[page_table[idx[x] / page_size], idx[x] % page_size, h, :] for idx[T] int64,
 * in caller order: PagedKVBufferABI.gather (python/tessera/cache/paged_kv.py:130-140), the
 * reference's tessera_nvidia_resident_paged / tessera_nvidia_paged_kv_read_f32
 * (python/tessera/compiler/emit/nvidia_cuda.py:1883, 2521, 2532). bf16, H * D a multiple of 8. */
int tessera_sm100_paged_kv_gather_device(const void* pages, const int* page_table,
                                         const long long* idx, void* out, long long T, int H, int D,
                                         int page_size, int num_pages, int max_pages, void* stream);

/* ---- flash-attention forward (prefill) ----------------------------------------------------
 * O = softmax(scale * Q K^T [+ bottom-right causal mask]) V with fp32 statistics:
 * tessera.ops.flash_attn (python/tessera/__init__.py:1304-1356). Q,O [B,Hq,Sq,D], K,V [B,Hkv,Sk,D]
 * bf16, D = 128, query head h reads KV head h / (Hq/Hkv) (python/tessera/nn/functional.py:349-356).
 * Argument order follows the reference's flash-forward ABI (q,k,v,o,B,Hq,Hkv,Sq,Sk,D,scale,causal)
 * (python/tessera/compiler/emit/nvidia_cuda.py:274), without its bias/window/softcap extras. */
int tessera_sm100_flash_attn_fwd_device(const void* Q, const void* K, const void* V, void* O, int B,
                                        int Hq, int Hkv, int Sq, int Sk, int D, float scale,
                                        int causal, void* stream);

/* Attention forward that picks the kernel: Sq == 1 -> split-KV decode (scratch taken from the
 * library's pool, recycled in stream order), otherwise the tcgen05 prefill kernel. The
 * host-pointer form uploads Q,K,V, runs, synchronises and downloads O; it is what the Python
 * tessera.ops.flash_attn / nn.functional.gqa_attention binding calls
 * (python/tessera/__init__.py:1304-1356, python/tessera/nn/functional.py:349-356), in the manner
 * of run_flash_attention_forward (python/tessera/compiler/emit/nvidia_cuda.py:313-361). */
int tessera_sm100_flash_attn_device(const void* Q, const void* K, const void* V, void* O, int B,
                                    int Hq, int Hkv, int Sq, int Sk, int D, float scale, int causal,
                                    void* stream);
int tessera_sm100_flash_attn(const void* Q, const void* K, const void* V, void* O, int B, int Hq,
                             int Hkv, int Sq, int Sk, int D, float scale, int causal);

/* Host-pointer MoE layer (upload, tessera_sm100_moe_layer_device, download): the GPU lane of
 * tessera.nn.functional.moe_layer (python/tessera/nn/functional.py:403-490). Optional outputs
 * may be null. */
int tessera_sm100_moe_layer(const void* x, const float* logits, const void* w_gate,
                            const void* w_up, const void* w_down, void* out, int T, int H, int F,
                            int E, int top_k, int normalize, int capacity, int dtype, int out_dtype,
                            int* assignment_out, float* weights_out, int* group_sizes_out,
                            int* token_of_slot_out);

/* out = silu(a) * b elementwise: tessera.ops.silu_mul (python/tessera/__init__.py:559-574). */
int tessera_sm100_silu_mul_device(const void* a, const void* b, void* out, long long n, int dtype,
                                  void* stream);

/* ---- collectives (NCCL over NVLink / NVSwitch) ---------------------------------------------
 * Device-resident, typed, asynchronous on the given stream. They stand where the reference has
 * NCCLAdapter::all_reduce / reduce_scatter / all_gather / all_to_all
 * (src/collectives/include/tessera/Dialect/Collective/Runtime/Adapters.h:295-394) and the ctypes
 * executor of python/tessera/collectives.py:516-628. A communicator handle is created either per
 * process (unique id + init_rank; the current CUDA device is the rank's GPU) or for several
 * devices of one process (init_all). Reduction op: 0 sum, 1 max, 2 min, 3 prod. */
int tessera_sm100_nccl_version(int* version);
int tessera_sm100_comm_unique_id(void* out128);
int tessera_sm100_comm_init_rank(const void* id128, int world, int rank, void** comm_out);
int tessera_sm100_comm_init_all(int ndev, const int* devices, void** comms_out);
int tessera_sm100_comm_destroy(void* comm);
int tessera_sm100_comm_abort(void* comm);
int tessera_sm100_comm_info(void* comm, int* rank, int* world, int* device);
int tessera_sm100_comm_async_error(void* comm);
int tessera_sm100_group_start(void);
int tessera_sm100_group_end(void);
int tessera_sm100_all_gather(void* comm, const void* send, void* recv, size_t count_per_rank,
                             int dtype, void* stream);
int tessera_sm100_all_reduce(void* comm, const void* send, void* recv, size_t count, int dtype,
                             int op, void* stream);
int tessera_sm100_reduce_scatter(void* comm, const void* send, void* recv, size_t recv_count,
                                 int dtype, int op, void* stream);
int tessera_sm100_all_to_all(void* comm, const void* send, void* recv, size_t bytes_per_peer,
                             void* stream);
/* Ragged all-to-all in bytes; the four arrays are host arrays of length world. Expert-parallel
 * MoE dispatch/combine need it (python/tessera/distributed/moe.py:252-315 gives the counts). */
int tessera_sm100_all_to_all_v(void* comm, const void* send, const size_t* send_bytes,
                               const size_t* send_offs, void* recv, const size_t* recv_bytes,
                               const size_t* recv_offs, void* stream);
/* CUDA IPC handles (64 bytes) so that one rank's kernel can store into another rank's buffer. */
int tessera_sm100_ipc_get_handle(void* device_ptr, void* handle64);
int tessera_sm100_ipc_open_handle(const void* handle64, void** device_ptr);
int tessera_sm100_ipc_close_handle(void* device_ptr);

#ifdef __cplusplus
}
#endif
#endif /* TESSERA_SM100_H_ */
