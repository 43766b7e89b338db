// MoE layer for sm_100a: router top-k, stable expert permutation, dispatch gather, the two
// grouped tcgen05 GEMMs (gate+up fused with SiLU*mul, then down) and a deterministic weighted
// combine. Integer outputs (assignment, permutation, group sizes) reproduce the reference's
// numpy routing bit for bit; see python/tessera/distributed/moe.py:119-206 and
// python/tessera/nn/functional.py:461-490.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cfloat>

#include "../../include/tessera_sm100.h"
#include "device_ctx.h"

namespace tsb {
namespace gemm {
int launch_grouped(const void* x, const void* w, const void* w2, const int* offsets, void* out,
                   int T, int K, int N, int E, int in_dtype, int out_dtype, bool swiglu,
                   cudaStream_t stream, const float* scale_a = nullptr);
}

namespace moe {

constexpr int kMaxExperts = 256;
constexpr int kMaxTopK = 8;

// ------------------------------------------------------------------------- router
// One thread per token. Selection runs on the logits (softmax is monotonic) with the
// reference's tie rule: among equal values the HIGHER expert index ranks first
// (np.argsort(...)[:, -k:][:, ::-1]). Weights are the f32 softmax probabilities, renormalised
// over the selected experts when `normalize` is set and top_k > 1.
__device__ __forceinline__ void route_token(const float* __restrict__ logits, int t, int E, int top_k,
                                            int normalize, int* __restrict__ assignment,
                                            float* __restrict__ weights) {
  const float* row = logits + (long long)t * E;
  float mx = -FLT_MAX;
  for (int e = 0; e < E; ++e) mx = fmaxf(mx, row[e]);
  float denom = 0.f;
  for (int e = 0; e < E; ++e) denom += expf(row[e] - mx);
  int chosen[kMaxTopK];
  float wsel[kMaxTopK];
  float wsum = 0.f;
  for (int j = 0; j < top_k; ++j) {
    int best = -1;
    float bv = 0.f;
    for (int e = 0; e < E; ++e) {
      bool taken = false;
      for (int q = 0; q < j; ++q) taken |= (chosen[q] == e);
      if (taken) continue;
      const float v = row[e];
      if (best < 0 || v >= bv) {  // >= : later (higher) index wins ties
        best = e;
        bv = v;
      }
    }
    chosen[j] = best;
    wsel[j] = expf(bv - mx) / denom;
    wsum += wsel[j];
  }
  const bool renorm = normalize && top_k > 1;
  const float inv = renorm ? (wsum > 0.f ? wsum : 1.f) : 1.f;
  for (int j = 0; j < top_k; ++j) {
    assignment[(long long)t * top_k + j] = chosen[j];
    weights[(long long)t * top_k + j] = renorm ? wsel[j] / inv : wsel[j];
  }
}

__global__ void route_topk_kernel(const float* __restrict__ logits, int T, int E, int top_k,
                                  int normalize, int* __restrict__ assignment,
                                  float* __restrict__ weights) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t < T) route_token(logits, t, E, top_k, normalize, assignment, weights);
}

// ------------------------------------------------------------------------- permutation
// Single CTA of 1024 threads: stable counting sort of the token-major slots by expert.
// Slot s = t * top_k + j. A slot whose rank inside its expert reaches `capacity` is dropped
// (assignment := -1, weight := 0), which is exactly the reference's token-major fill order.
// Outputs follow the canonical int32 device ABI of
// python/tessera/compiler/moe_transport.py:75-134.
__device__ void permute_block(int* __restrict__ assignment, float* __restrict__ weights, int S, int E,
                              int capacity, int* __restrict__ token_of_slot,
                              int* __restrict__ expert_of_slot, float* __restrict__ weight_of_slot,
                              int* __restrict__ group_sizes, int* __restrict__ group_offsets,
                              int* __restrict__ slot_of_assignment, int top_k) {
  __shared__ int s_count[kMaxExperts];       // kept slots per expert
  __shared__ int s_offset[kMaxExperts + 1];  // exclusive scan of s_count
  __shared__ int s_running[kMaxExperts];     // slots of each expert seen in earlier chunks
  __shared__ int s_warp[32][kMaxExperts];    // per-warp counts inside the current chunk
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  for (int e = tid; e < E; e += blockDim.x) {
    s_count[e] = 0;
    s_running[e] = 0;
  }
  __syncthreads();
  // pass 1: histogram (capped by capacity)
  for (int s = tid; s < S; s += blockDim.x) {
    const int e = assignment[s];
    if (e >= 0 && e < E) atomicAdd(&s_count[e], 1);
  }
  __syncthreads();
  if (tid == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) {
      const int c = (capacity >= 0) ? min(s_count[e], capacity) : s_count[e];
      s_count[e] = c;
      s_offset[e] = acc;
      group_sizes[e] = c;
      group_offsets[e] = acc;
      acc += c;
    }
    s_offset[E] = acc;
    group_offsets[E] = acc;
  }
  __syncthreads();
  // pass 2: ranks, chunk by chunk in slot order
  for (int base = 0; base < S; base += blockDim.x) {
    const int s = base + tid;
    const int e = (s < S) ? assignment[s] : -1;
    const bool live = (e >= 0 && e < E);
    for (int i = tid; i < 32 * E; i += blockDim.x) (&s_warp[0][0])[(i / E) * kMaxExperts + (i % E)] = 0;
    __syncthreads();
    const unsigned peers = __match_any_sync(0xffffffffu, live ? e : -1 - lane);
    const int local_rank = __popc(peers & ((1u << lane) - 1u));
    if (live && local_rank == 0) s_warp[warp][e] = __popc(peers);
    __syncthreads();
    // exclusive prefix over warps, per expert; also advances the running totals
    for (int x = tid; x < E; x += blockDim.x) {
      int acc = s_running[x];
      for (int w = 0; w < 32; ++w) {
        const int c = s_warp[w][x];
        s_warp[w][x] = acc;
        acc += c;
      }
      s_running[x] = acc;
    }
    __syncthreads();
    if (s < S) {
      int pos = -1;
      if (live) {
        const int rank = s_warp[warp][e] + local_rank;
        if (capacity < 0 || rank < capacity) pos = s_offset[e] + rank;
      }
      if (pos >= 0) {
        token_of_slot[pos] = s / top_k;
        expert_of_slot[pos] = e;
        weight_of_slot[pos] = weights[s];
      } else if (live) {  // dropped by capacity
        assignment[s] = -1;
        weights[s] = 0.f;
      }
      slot_of_assignment[s] = pos;
    }
    __syncthreads();
  }
}

__global__ void __launch_bounds__(1024, 1)
permute_kernel(int* __restrict__ assignment, float* __restrict__ weights, int S, int E,
               int capacity, int* __restrict__ token_of_slot, int* __restrict__ expert_of_slot,
               float* __restrict__ weight_of_slot, int* __restrict__ group_sizes,
               int* __restrict__ group_offsets, int* __restrict__ slot_of_assignment, int top_k) {
  permute_block(assignment, weights, S, E, capacity, token_of_slot, expert_of_slot, weight_of_slot,
                group_sizes, group_offsets, slot_of_assignment, top_k);
}

// ------------------------------------------------------------------------- dispatch / combine
// o[s,:] = x[tok[s],:]   rows of `row_bytes` bytes (a multiple of 16).
__global__ void gather_rows_kernel(const uint4* __restrict__ x, const int* __restrict__ tok,
                                   uint4* __restrict__ o, const int* __restrict__ num_slots_ptr,
                                   int max_slots, int vec_per_row) {
  const int S = num_slots_ptr ? min(*num_slots_ptr, max_slots) : max_slots;
  const long long total = (long long)S * vec_per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int s = (int)(i / vec_per_row);
    const int c = (int)(i - (long long)s * vec_per_row);
    o[i] = x[(long long)tok[s] * vec_per_row + c];
  }
}

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

// out[t,:] = sum_j w[t,j] * y[slot_of_assignment[t,j],:], j ascending, f32 accumulate.
// No atomics: the sum order is fixed, so the result is deterministic.
template <typename YT, typename OT>
__global__ void combine_kernel(const YT* __restrict__ y, const int* __restrict__ slot_of,
                               const float* __restrict__ w, OT* __restrict__ out, int T, int top_k,
                               int H) {
  const int t = blockIdx.x;
  if (t >= T) return;
  for (int c = threadIdx.x * 4; c < H; c += blockDim.x * 4) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < top_k; ++j) {
      const int s = slot_of[(long long)t * top_k + j];
      if (s < 0) continue;
      const float wj = w[(long long)t * top_k + j];
      const YT* row = y + (long long)s * H + c;
#pragma unroll
      for (int q = 0; q < 4; ++q)
        if (c + q < H) acc[q] += wj * to_f32<YT>(row[q]);
    }
#pragma unroll
    for (int q = 0; q < 4; ++q)
      if (c + q < H) out[(long long)t * H + c + q] = from_f32<OT>(acc[q]);
  }
}

// Reference-shaped scatter combine: o[tok[s],:] += w[s] * x[s,:]  (o zeroed by the caller).
// f32 atomics: deterministic for top_k <= 2 (two commutative addends per element).
__global__ void combine_scatter_kernel(const float* __restrict__ x, const int* __restrict__ tok,
                                       const float* __restrict__ w, float* __restrict__ o, int S,
                                       int H) {
  const long long total = (long long)S * H;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int s = (int)(i / H);
    const int h = (int)(i - (long long)s * H);
    atomicAdd(&o[(long long)tok[s] * H + h], w[s] * x[i]);
  }
}


// ------------------------------------------------------------------------- expert parallel
// Device-side expert-parallel exchange over peer memory (no host round trip, no padding):
//   * every rank sorts its slots by GLOBAL expert (permute_kernel) and all-gathers its per-expert
//     counts, so each rank knows cnt[src][e] for all sources;
//   * ep_plan_kernel turns that table into (a) the group offsets of this rank's local experts
//     (rows arrive expert-major, source-major inside an expert: the stable expert sort of the
//     single-device layer) and (b) for every global expert e the first row, inside the owner's
//     receive buffer, of the block this rank contributes;
//   * ep_dispatch_kernel stores each token row straight into its owner's receive buffer
//     (plain 16-byte stores to a peer pointer), already in grouped order;
//   * ep_combine_kernel reads each slot's result row back from the owner's output buffer (plain
//     peer loads) and forms the weighted sum per token in slot order.
// Partitioning follows megamoe_forward (python/tessera/distributed/moe.py:358-483).
struct PeerPtrs {
  void* p[8];
};

__global__ void ep_plan_kernel(const int* __restrict__ cnt, int world, int rank, int E,
                               int* __restrict__ group_offsets_local, int* __restrict__ dst_base) {
  const int Ep = E / world;
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    int acc = 0;
    for (int el = 0; el < Ep; ++el) {
      group_offsets_local[el] = acc;
      for (int s = 0; s < world; ++s) acc += cnt[s * E + rank * Ep + el];
    }
    group_offsets_local[Ep] = acc;
  }
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int d = e / Ep;
    int base = 0;
    for (int e2 = d * Ep; e2 < e; ++e2)
      for (int s = 0; s < world; ++s) base += cnt[s * E + e2];
    for (int s = 0; s < rank; ++s) base += cnt[s * E + e];
    dst_base[e] = base;
  }
}

__global__ void ep_dispatch_kernel(const uint4* __restrict__ x, const int* __restrict__ token_of_slot,
                                   const int* __restrict__ expert_of_slot,
                                   const int* __restrict__ my_offsets, const int* __restrict__ dst_base,
                                   PeerPtrs recv, int E, int Ep, int capacity_rows, int vec_per_row) {
  const int S = my_offsets[E];  // kept slots of this rank
  const long long total = (long long)S * vec_per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int s = (int)(i / vec_per_row);
    const int c = (int)(i - (long long)s * vec_per_row);
    const int e = expert_of_slot[s];
    const int row = dst_base[e] + (s - my_offsets[e]);
    if (row < capacity_rows) {
      uint4* dst = static_cast<uint4*>(recv.p[e / Ep]);
      dst[(long long)row * vec_per_row + c] = x[(long long)token_of_slot[s] * vec_per_row + c];
    }
  }
}

template <typename YT, typename OT>
__global__ void ep_combine_kernel(PeerPtrs ybufs, const int* __restrict__ assignment,
                                  const int* __restrict__ slot_of, const float* __restrict__ w,
                                  const int* __restrict__ my_offsets, const int* __restrict__ dst_base,
                                  OT* __restrict__ out, int T, int top_k, int Ep, int capacity_rows,
                                  int H) {
  const int t = blockIdx.x;
  if (t >= T) return;
  for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
    float acc[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) acc[q] = 0.f;
    for (int j = 0; j < top_k; ++j) {
      const int s = slot_of[(long long)t * top_k + j];
      if (s < 0) continue;
      const int e = assignment[(long long)t * top_k + j];
      const int row = dst_base[e] + (s - my_offsets[e]);
      if (row >= capacity_rows) continue;
      const float wj = w[(long long)t * top_k + j];
      const YT* src = static_cast<const YT*>(ybufs.p[e / Ep]) + (long long)row * H + c;
      if constexpr (sizeof(YT) == 2) {
        const uint4 v = *reinterpret_cast<const uint4*>(src);   // 8 x 16-bit, H % 8 == 0
        const YT* h = reinterpret_cast<const YT*>(&v);
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[q] += wj * to_f32<YT>(h[q]);
      } else {
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[q] += wj * to_f32<YT>(src[q]);
      }
    }
#pragma unroll
    for (int q = 0; q < 8; ++q) out[(long long)t * H + c + q] = from_f32<OT>(acc[q]);
  }
}


// ---- the same exchange with the ranks ordered by flags in peer memory instead of collectives -----
// Every rank owns one EpCtrl block that all peers can write (CUDA IPC). A forward call carries an
// epoch number, the same on all ranks and one higher on every call; a flag is "up" once it has
// reached the epoch, so nothing is ever reset. Three launches surround the two grouped GEMMs:
//   ep_route_publish   route + stable expert sort of the local slots (one CTA), then this rank's E
//                      per-expert counts are stored into counts[rank][] of every rank's block and
//                      counts_ready[rank] goes up there;
//   ep_dispatch_signal waits for every source's counts (and for done[] of the previous epoch: the
//                      peers no longer read the buffers this call overwrites), derives the plan,
//                      stores the token rows into the owners' receive buffers, and the CTA that
//                      finishes last raises rows_ready[rank] everywhere and then waits for every
//                      source's rows_ready, so that the kernel's end means "all my rows are here";
//   ep_combine_signal  raises y_ready[rank] everywhere (the GEMMs before it in the stream are
//                      done), waits for every owner's y_ready, reads the result rows back, and the
//                      CTA that finishes last raises done[rank].
// Waits are bounded by wall-clock time (%globaltimer); on expiry the error word is set and the
// kernel carries on to its end without the data, so the context stays usable.
constexpr int kEpMaxWorld = 8;
struct EpCtrl {
  int counts[kEpMaxWorld][kMaxExperts];  // [source rank][global expert], written by the source
  int counts_ready[32];                  // [source rank] epoch; each flag array on its own line
  int rows_ready[32];
  int y_ready[32];
  int done[32];
};

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.b32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_relaxed_sys(const int* p) {
  int v;
  asm volatile("ld.relaxed.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Waits until *flag has reached `want` (epochs compare by signed difference). Returns false, with
// the error word set to {kErrWaitOther, block, detail}, when `limit_ns` runs out first.
__device__ bool ep_wait_flag(const int* flag, int want, unsigned long long limit_ns, int* err,
                             int detail) {
  if (ld_acquire_sys(flag) - want >= 0) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (;;) {
    if (ld_acquire_sys(flag) - want >= 0) return true;
    if (globaltimer_ns() - t0 > limit_ns) {
      if (atomicCAS(err, 0, 5 /* kErrWaitOther */) == 0) {
        err[1] = static_cast<int>(blockIdx.x);
        err[2] = detail;
      }
      __threadfence();
      return false;
    }
    __nanosleep(100);
  }
}

__global__ void __launch_bounds__(1024, 1)
ep_route_publish_kernel(const float* __restrict__ logits, int Tl, int E, int top_k, int normalize,
                        int* __restrict__ assignment, float* __restrict__ weights,
                        int* __restrict__ token_of_slot, int* __restrict__ expert_of_slot,
                        float* __restrict__ weight_of_slot, int* __restrict__ group_sizes,
                        int* __restrict__ my_offsets, int* __restrict__ slot_of, PeerPtrs ctrl,
                        int world, int rank, int epoch) {
  for (int t = threadIdx.x; t < Tl; t += blockDim.x)
    route_token(logits, t, E, top_k, normalize, assignment, weights);
  __syncthreads();
  permute_block(assignment, weights, Tl * top_k, E, -1, token_of_slot, expert_of_slot, weight_of_slot,
                group_sizes, my_offsets, slot_of, top_k);
  __syncthreads();
  for (int i = threadIdx.x; i < world * E; i += blockDim.x) {
    const int dst = i / E, e = i - dst * E;
    static_cast<EpCtrl*>(ctrl.p[dst])->counts[rank][e] = group_sizes[e];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < world)
    st_release_sys(&static_cast<EpCtrl*>(ctrl.p[threadIdx.x])->counts_ready[rank], epoch);
}

__global__ void ep_dispatch_signal_kernel(const uint4* __restrict__ x, const int* __restrict__ token_of_slot,
                                          const int* __restrict__ expert_of_slot,
                                          const int* __restrict__ my_offsets, PeerPtrs ctrl, PeerPtrs recv,
                                          int world, int rank, int E, int capacity_rows, int vec_per_row,
                                          int epoch, int* __restrict__ group_offsets_local,
                                          int* __restrict__ dst_base_out, int* __restrict__ counter,
                                          unsigned long long limit_ns, int* __restrict__ err) {
  __shared__ int s_base[kMaxExperts];
  __shared__ int s_last;
  const int Ep = E / world;
  const EpCtrl* mine = static_cast<const EpCtrl*>(ctrl.p[rank]);
  if (threadIdx.x < world) {
    ep_wait_flag(&mine->counts_ready[threadIdx.x], epoch, limit_ns, err, 100 + threadIdx.x);
    ep_wait_flag(&mine->done[threadIdx.x], epoch - 1, limit_ns, err, 200 + threadIdx.x);
  }
  __syncthreads();
  // The plan: for every global expert the first row, in its owner's receive buffer, of the block
  // this rank contributes (rows arrive expert-major, source-major inside an expert).
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int d = e / Ep;
    int base = 0;
    for (int e2 = d * Ep; e2 < e; ++e2)
      for (int sr = 0; sr < world; ++sr) base += ld_relaxed_sys(&mine->counts[sr][e2]);
    for (int sr = 0; sr < rank; ++sr) base += ld_relaxed_sys(&mine->counts[sr][e]);
    s_base[e] = base;
    if (blockIdx.x == 0) dst_base_out[e] = base;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    int acc = 0;
    for (int el = 0; el < Ep; ++el) {
      group_offsets_local[el] = acc;
      for (int sr = 0; sr < world; ++sr) acc += ld_relaxed_sys(&mine->counts[sr][rank * Ep + el]);
    }
    group_offsets_local[Ep] = acc;
  }
  __syncthreads();
  // One warp per kept slot: the row's source token and destination are looked up once, then the
  // lanes copy it with four 16-byte loads in flight each (a row of 4096 bf16 is 512 vectors).
  const int S = my_offsets[E];  // kept slots of this rank
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  for (int sl = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); sl < S; sl += gridDim.x * warps_per_cta) {
    const int e = expert_of_slot[sl];
    const int row = s_base[e] + (sl - my_offsets[e]);
    if (row >= capacity_rows) continue;
    const uint4* src = x + (long long)token_of_slot[sl] * vec_per_row;
    uint4* dst = static_cast<uint4*>(recv.p[e / Ep]) + (long long)row * vec_per_row;
    int c = lane;
    for (; c + 96 < vec_per_row; c += 128) {
      const uint4 v0 = src[c], v1 = src[c + 32], v2 = src[c + 64], v3 = src[c + 96];
      dst[c] = v0;
      dst[c + 32] = v1;
      dst[c + 64] = v2;
      dst[c + 96] = v3;
    }
    for (; c < vec_per_row; c += 32) dst[c] = src[c];
  }
  // The CTA that finishes last tells every rank that this rank's rows have landed.
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(counter, 1) == static_cast<int>(gridDim.x) - 1);
  __syncthreads();
  if (s_last) {
    if (threadIdx.x == 0) *counter = 0;
    __threadfence_system();
    if (threadIdx.x < world) {
      st_release_sys(&static_cast<EpCtrl*>(ctrl.p[threadIdx.x])->rows_ready[rank], epoch);
      ep_wait_flag(&mine->rows_ready[threadIdx.x], epoch, limit_ns, err, 300 + threadIdx.x);
    }
  }
}

template <typename YT, typename OT>
__global__ void ep_combine_signal_kernel(PeerPtrs ybufs, PeerPtrs ctrl, const int* __restrict__ assignment,
                                         const int* __restrict__ slot_of, const float* __restrict__ w,
                                         const int* __restrict__ my_offsets, const int* __restrict__ dst_base,
                                         OT* __restrict__ out, int T, int top_k, int world, int rank, int Ep,
                                         int capacity_rows, int H, int epoch, int* __restrict__ counter,
                                         unsigned long long limit_ns, int* __restrict__ err) {
  __shared__ int s_last;
  const EpCtrl* mine = static_cast<const EpCtrl*>(ctrl.p[rank]);
  if (threadIdx.x < world) {
    if (blockIdx.x == 0) {
      __threadfence_system();
      st_release_sys(&static_cast<EpCtrl*>(ctrl.p[threadIdx.x])->y_ready[rank], epoch);
    }
    ep_wait_flag(&mine->y_ready[threadIdx.x], epoch, limit_ns, err, 400 + threadIdx.x);
  }
  __syncthreads();
  // The token's k result rows: located once per CTA, then every thread issues all of its 16-byte
  // peer loads (k per column vector) before it touches the values, so one NVLink round trip covers them.
  __shared__ const YT* s_row[kMaxTopK];
  __shared__ float s_w[kMaxTopK];
  const int t = blockIdx.x;
  if (threadIdx.x < top_k) {
    const int j = threadIdx.x;
    const int sl = slot_of[(long long)t * top_k + j];
    const YT* rowp = nullptr;
    if (sl >= 0) {
      const int e = assignment[(long long)t * top_k + j];
      const int row = dst_base[e] + (sl - my_offsets[e]);
      if (row < capacity_rows) rowp = static_cast<const YT*>(ybufs.p[e / Ep]) + (long long)row * H;
    }
    s_row[j] = rowp;
    s_w[j] = w[(long long)t * top_k + j];
  }
  __syncthreads();
  constexpr int kVecsPerThread = 2;
  for (int c0 = threadIdx.x * 8; c0 < H; c0 += blockDim.x * 8 * kVecsPerThread) {
    uint4 v[kVecsPerThread][kMaxTopK];
#pragma unroll
    for (int u = 0; u < kVecsPerThread; ++u) {
      const int c = c0 + u * blockDim.x * 8;
#pragma unroll
      for (int j = 0; j < kMaxTopK; ++j)
        if (j < top_k && c < H && s_row[j]) v[u][j] = __ldcg(reinterpret_cast<const uint4*>(s_row[j] + c));
    }
#pragma unroll
    for (int u = 0; u < kVecsPerThread; ++u) {
      const int c = c0 + u * blockDim.x * 8;
      if (c >= H) break;
      float acc[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[q] = 0.f;
#pragma unroll
      for (int j = 0; j < kMaxTopK; ++j) {
        if (j >= top_k || !s_row[j]) continue;
        const float wj = s_w[j];
        const YT* hp = reinterpret_cast<const YT*>(&v[u][j]);
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[q] += wj * to_f32<YT>(hp[q]);
      }
#pragma unroll
      for (int q = 0; q < 8; ++q) out[(long long)t * H + c + q] = from_f32<OT>(acc[q]);
    }
  }
  // The CTA that finishes last tells every rank that this rank no longer reads their buffers.
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(counter, 1) == static_cast<int>(gridDim.x) - 1);
  __syncthreads();
  if (s_last) {
    if (threadIdx.x == 0) *counter = 0;
    __threadfence_system();
    if (threadIdx.x < world)
      st_release_sys(&static_cast<EpCtrl*>(ctrl.p[threadIdx.x])->done[rank], epoch);
  }
}

size_t dtype_size(int dt) { return dt == TESSERA_SM100_F32 ? 4 : 2; }

int route(const float* logits, int T, int E, int top_k, int normalize, int* assignment,
          float* weights, cudaStream_t st) {
  if (!logits || !assignment || !weights || T < 0 || E <= 0 || top_k <= 0 || top_k > E ||
      top_k > kMaxTopK) {
    set_last_error("moe_route: bad arguments (T %d E %d top_k %d; top_k <= %d)", T, E, top_k,
                   kMaxTopK);
    return kBadArg;
  }
  if (T == 0) return kOk;
  route_topk_kernel<<<(T + 127) / 128, 128, 0, st>>>(logits, T, E, top_k, normalize, assignment,
                                                      weights);
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  return kOk;
}

int permute(int* assignment, float* weights, int T, int top_k, int E, int capacity,
            int* token_of_slot, int* expert_of_slot, float* weight_of_slot, int* group_sizes,
            int* group_offsets, int* slot_of_assignment, cudaStream_t st) {
  if (!assignment || !weights || !token_of_slot || !expert_of_slot || !weight_of_slot ||
      !group_sizes || !group_offsets || !slot_of_assignment || T < 0 || top_k <= 0 || E <= 0 ||
      E > kMaxExperts) {
    set_last_error("moe_permute: bad arguments (T %d top_k %d E %d; E <= %d)", T, top_k, E,
                   kMaxExperts);
    return kBadArg;
  }
  permute_kernel<<<1, 1024, 0, st>>>(assignment, weights, T * top_k, E, capacity, token_of_slot,
                                     expert_of_slot, weight_of_slot, group_sizes, group_offsets,
                                     slot_of_assignment, top_k);
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  return kOk;
}

int dispatch(const void* x, const int* tok, void* o, const int* num_slots_ptr, int T, int S, int H,
             int dtype, cudaStream_t st) {
  const size_t row_bytes = (size_t)H * dtype_size(dtype);
  if (!x || !tok || !o || T < 0 || S < 0 || H <= 0 || (row_bytes % 16) ||
      (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(o) & 15)) {
    set_last_error("moe_dispatch: bad arguments (rows must be 16-byte multiples and aligned)");
    return kBadArg;
  }
  if (S == 0) return kOk;
  const int vec = (int)(row_bytes / 16);
  const long long total = (long long)S * vec;
  const int grid = (int)std::min<long long>((total + 255) / 256, 148 * 16);
  gather_rows_kernel<<<grid, 256, 0, st>>>(static_cast<const uint4*>(x), tok,
                                           static_cast<uint4*>(o), num_slots_ptr, S, vec);
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  return kOk;
}

template <typename YT>
int combine_out(const void* y, const int* slot_of, const float* w, void* out, int T, int top_k,
                int H, int out_dtype, cudaStream_t st) {
  const int block = 256;
  switch (out_dtype) {
    case TESSERA_SM100_F32:
      combine_kernel<YT, float><<<T, block, 0, st>>>(static_cast<const YT*>(y), slot_of, w,
                                                     static_cast<float*>(out), T, top_k, H);
      break;
    case TESSERA_SM100_BF16:
      combine_kernel<YT, __nv_bfloat16><<<T, block, 0, st>>>(
          static_cast<const YT*>(y), slot_of, w, static_cast<__nv_bfloat16*>(out), T, top_k, H);
      break;
    case TESSERA_SM100_F16:
      combine_kernel<YT, __half><<<T, block, 0, st>>>(static_cast<const YT*>(y), slot_of, w,
                                                      static_cast<__half*>(out), T, top_k, H);
      break;
    default:
      set_last_error("moe_combine: unsupported output dtype %d", out_dtype);
      return kBadArg;
  }
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  return kOk;
}

int combine(const void* y, const int* slot_of, const float* w, void* out, int T, int top_k, int H,
            int y_dtype, int out_dtype, cudaStream_t st) {
  if (!y || !slot_of || !w || !out || T < 0 || top_k <= 0 || H <= 0) {
    set_last_error("moe_combine: bad arguments");
    return kBadArg;
  }
  if (T == 0) return kOk;
  switch (y_dtype) {
    case TESSERA_SM100_F32: return combine_out<float>(y, slot_of, w, out, T, top_k, H, out_dtype, st);
    case TESSERA_SM100_BF16:
      return combine_out<__nv_bfloat16>(y, slot_of, w, out, T, top_k, H, out_dtype, st);
    case TESSERA_SM100_F16: return combine_out<__half>(y, slot_of, w, out, T, top_k, H, out_dtype, st);
    default: break;
  }
  set_last_error("moe_combine: unsupported input dtype %d", y_dtype);
  return kBadArg;
}

// Workspace layout for one MoE layer call (all offsets 256-byte aligned).
struct Workspace {
  size_t assignment, weights, token_of_slot, expert_of_slot, weight_of_slot, group_sizes,
      group_offsets, slot_of, x_perm, hidden, y, total;
};

Workspace plan_workspace(int T, int H, int F, int E, int top_k) {
  Workspace w{};
  size_t off = 0;
  auto take = [&](size_t bytes) {
    size_t at = off;
    off += (bytes + 255) & ~size_t(255);
    return at;
  };
  const size_t S = (size_t)T * top_k;
  w.assignment = take(S * 4);
  w.weights = take(S * 4);
  w.token_of_slot = take(S * 4);
  w.expert_of_slot = take(S * 4);
  w.weight_of_slot = take(S * 4);
  w.group_sizes = take((size_t)E * 4);
  w.group_offsets = take((size_t)(E + 1) * 4);
  w.slot_of = take(S * 4);
  w.x_perm = take(S * H * 2);
  w.hidden = take(S * F * 2);
  w.y = take(S * H * 2);
  w.total = off;
  return w;
}

// Full layer on device pointers. `ws` is caller-provided scratch of plan_workspace().total bytes.
int layer(const void* x, const float* logits, const void* w_gate, const void* w_up,
          const void* w_down, void* out, int T, int H, int F, int E, int top_k, int normalize,
          int capacity, int dtype, int out_dtype, uint8_t* ws, cudaStream_t st) {
  if (!x || !logits || !w_gate || !w_up || !w_down || !out || !ws || T <= 0 || H <= 0 || F <= 0) {
    set_last_error("moe_layer: null pointer or bad size");
    return kBadArg;
  }
  if ((H % 8) || (F % 8)) {
    set_last_error("moe_layer: hidden (%d) and FFN (%d) sizes must be multiples of 8", H, F);
    return kBadArg;
  }
  const Workspace w = plan_workspace(T, H, F, E, top_k);
  int* assignment = reinterpret_cast<int*>(ws + w.assignment);
  float* weights = reinterpret_cast<float*>(ws + w.weights);
  int* token_of_slot = reinterpret_cast<int*>(ws + w.token_of_slot);
  int* expert_of_slot = reinterpret_cast<int*>(ws + w.expert_of_slot);
  float* weight_of_slot = reinterpret_cast<float*>(ws + w.weight_of_slot);
  int* group_sizes = reinterpret_cast<int*>(ws + w.group_sizes);
  int* group_offsets = reinterpret_cast<int*>(ws + w.group_offsets);
  int* slot_of = reinterpret_cast<int*>(ws + w.slot_of);
  void* x_perm = ws + w.x_perm;
  void* hidden = ws + w.hidden;
  void* y = ws + w.y;
  const int S = T * top_k;
  int rc;
  if ((rc = route(logits, T, E, top_k, normalize, assignment, weights, st))) return rc;
  if ((rc = permute(assignment, weights, T, top_k, E, capacity, token_of_slot, expert_of_slot,
                    weight_of_slot, group_sizes, group_offsets, slot_of, st)))
    return rc;
  // Kept slots = group_offsets[E] (device value); dropped slots leave a tail that is never read.
  if ((rc = dispatch(x, token_of_slot, x_perm, group_offsets + E, T, S, H, dtype, st))) return rc;
  if ((rc = gemm::launch_grouped(x_perm, w_gate, w_up, group_offsets, hidden, S, H, F, E, dtype,
                                 dtype, true, st)))
    return rc;
  if ((rc = gemm::launch_grouped(hidden, w_down, nullptr, group_offsets, y, S, F, H, E, dtype,
                                 dtype, false, st)))
    return rc;
  return combine(y, slot_of, weights, out, T, top_k, H, dtype, out_dtype, st);
}

}  // namespace moe
}  // namespace tsb

using namespace tsb;

extern "C" {

int tessera_sm100_moe_route_device(const float* logits, int T, int E, int top_k, int normalize,
                                   int* assignment, float* weights, void* stream) {
  return moe::route(logits, T, E, top_k, normalize, assignment, weights,
                    static_cast<cudaStream_t>(stream));
}

int tessera_sm100_moe_permute_device(int* assignment, float* weights, int T, int top_k, int E,
                                     int capacity, int* token_of_slot, int* expert_of_slot,
                                     float* weight_of_slot, int* group_sizes, int* group_offsets,
                                     int* slot_of_assignment, void* stream) {
  return moe::permute(assignment, weights, T, top_k, E, capacity, token_of_slot, expert_of_slot,
                      weight_of_slot, group_sizes, group_offsets, slot_of_assignment,
                      static_cast<cudaStream_t>(stream));
}

int tessera_sm100_moe_dispatch_device(const void* x, const int* tok, void* o, int T, int S, int H,
                                      int dtype, void* stream) {
  return moe::dispatch(x, tok, o, nullptr, T, S, H, dtype, static_cast<cudaStream_t>(stream));
}

int tessera_sm100_moe_combine_device(const void* y, const int* slot_of_assignment,
                                     const float* weights, void* out, int T, int top_k, int H,
                                     int y_dtype, int out_dtype, void* stream) {
  return moe::combine(y, slot_of_assignment, weights, out, T, top_k, H, y_dtype, out_dtype,
                      static_cast<cudaStream_t>(stream));
}

int tessera_sm100_moe_combine_scatter_f32_device(const float* x, const int* tok, const float* w,
                                                 float* o, int T, int S, int H, void* stream) {
  if (!x || !tok || !w || !o || T < 0 || S < 0 || H <= 0) {
    set_last_error("moe_combine_scatter: bad arguments");
    return kBadArg;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  TSB_CUDA_OK(cudaMemsetAsync(o, 0, (size_t)T * H * 4, st));
  if (S == 0) return kOk;
  const long long total = (long long)S * H;
  const int grid = (int)std::min<long long>((total + 255) / 256, 148 * 16);
  moe::combine_scatter_kernel<<<grid, 256, 0, st>>>(x, tok, w, o, S, H);
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  return kOk;
}

size_t tessera_sm100_moe_workspace_bytes(int T, int H, int F, int E, int top_k) {
  return moe::plan_workspace(T, H, F, E, top_k).total;
}

int tessera_sm100_moe_layer_device(const void* x, const float* logits, const void* w_gate,
                                   const void* w_up, const void* w_down, void* out, int T, int H,
                                   int F, int E, int top_k, int normalize, int capacity, int dtype,
                                   int out_dtype, void* workspace, void* stream) {
  return moe::layer(x, logits, w_gate, w_up, w_down, out, T, H, F, E, top_k, normalize, capacity,
                    dtype, out_dtype, static_cast<uint8_t*>(workspace),
                    static_cast<cudaStream_t>(stream));
}

// Copies the routing products of the last layer call out of its workspace (device pointers
// into `workspace`); any output pointer may be null.
int tessera_sm100_moe_workspace_views(void* workspace, int T, int H, int F, int E, int top_k,
                                      void** assignment, void** weights, void** token_of_slot,
                                      void** expert_of_slot, void** weight_of_slot,
                                      void** group_sizes, void** group_offsets,
                                      void** slot_of_assignment) {
  if (!workspace) return kBadArg;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  const moe::Workspace w = moe::plan_workspace(T, H, F, E, top_k);
  if (assignment) *assignment = ws + w.assignment;
  if (weights) *weights = ws + w.weights;
  if (token_of_slot) *token_of_slot = ws + w.token_of_slot;
  if (expert_of_slot) *expert_of_slot = ws + w.expert_of_slot;
  if (weight_of_slot) *weight_of_slot = ws + w.weight_of_slot;
  if (group_sizes) *group_sizes = ws + w.group_sizes;
  if (group_offsets) *group_offsets = ws + w.group_offsets;
  if (slot_of_assignment) *slot_of_assignment = ws + w.slot_of;
  return kOk;
}

// ---- expert-parallel exchange over peer memory -------------------------------------------------
int tessera_sm100_ep_plan_device(const int* all_counts, int world, int rank, int E,
                                 int* group_offsets_local, int* dst_base, void* stream) {
  if (!all_counts || !group_offsets_local || !dst_base || world <= 0 || world > 8 || rank < 0 ||
      rank >= world || E <= 0 || E % world) {
    set_last_error("ep_plan: bad arguments (world %d rank %d E %d; world <= 8, E %% world == 0)", world,
                   rank, E);
    return kBadArg;
  }
  moe::ep_plan_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(all_counts, world, rank, E,
                                                                        group_offsets_local, dst_base);
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  return kOk;
}

int tessera_sm100_ep_dispatch_device(const void* x, const int* token_of_slot,
                                     const int* expert_of_slot, const int* my_offsets,
                                     const int* dst_base, void* const* recv_bufs, int world, int E,
                                     int max_slots, int capacity_rows, int H, int dtype, void* stream) {
  const size_t row_bytes = (size_t)H * moe::dtype_size(dtype);
  if (!x || !token_of_slot || !expert_of_slot || !my_offsets || !dst_base || !recv_bufs ||
      world <= 0 || world > 8 || E % world || (row_bytes % 16) || max_slots < 0) {
    set_last_error("ep_dispatch: bad arguments (rows must be 16-byte multiples, world <= 8)");
    return kBadArg;
  }
  if (max_slots == 0) return kOk;
  moe::PeerPtrs pp{};
  for (int i = 0; i < world; ++i) {
    if (!recv_bufs[i]) {
      set_last_error("ep_dispatch: receive buffer %d is null", i);
      return kBadArg;
    }
    pp.p[i] = recv_bufs[i];
  }
  const int vec = (int)(row_bytes / 16);
  const long long total = (long long)max_slots * vec;
  const int grid = (int)std::min<long long>((total + 255) / 256, 148 * 16);
  moe::ep_dispatch_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x), token_of_slot, expert_of_slot, my_offsets, dst_base, pp, E,
      E / world, capacity_rows, vec);
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  return kOk;
}

int tessera_sm100_ep_combine_device(void* const* y_bufs, const int* assignment,
                                    const int* slot_of_assignment, const float* weights,
                                    const int* my_offsets, const int* dst_base, void* out, int T,
                                    int top_k, int world, int E, int capacity_rows, int H, int dtype,
                                    void* stream) {
  if (!y_bufs || !assignment || !slot_of_assignment || !weights || !my_offsets || !dst_base || !out ||
      world <= 0 || world > 8 || E % world || (H % 8) || T < 0) {
    set_last_error("ep_combine: bad arguments (H must be a multiple of 8, world <= 8)");
    return kBadArg;
  }
  if (T == 0) return kOk;
  moe::PeerPtrs pp{};
  for (int i = 0; i < world; ++i) {
    if (!y_bufs[i]) {
      set_last_error("ep_combine: output buffer %d is null", i);
      return kBadArg;
    }
    pp.p[i] = y_bufs[i];
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int Ep = E / world;
  if (dtype == TESSERA_SM100_BF16)
    moe::ep_combine_kernel<__nv_bfloat16, __nv_bfloat16><<<T, 128, 0, st>>>(
        pp, assignment, slot_of_assignment, weights, my_offsets, dst_base,
        static_cast<__nv_bfloat16*>(out), T, top_k, Ep, capacity_rows, H);
  else if (dtype == TESSERA_SM100_F16)
    moe::ep_combine_kernel<__half, __half><<<T, 128, 0, st>>>(
        pp, assignment, slot_of_assignment, weights, my_offsets, dst_base, static_cast<__half*>(out),
        T, top_k, Ep, capacity_rows, H);
  else {
    set_last_error("ep_combine: dtype must be bf16 or f16");
    return kBadArg;
  }
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  return kOk;
}

// ---- the exchange ordered by flags in peer memory (no collective) ------------------------------
size_t tessera_sm100_ep_ctrl_bytes(void) { return sizeof(moe::EpCtrl); }

namespace {
bool ep_peer_ptrs(moe::PeerPtrs& pp, void* const* ptrs, int world, const char* what) {
  for (int i = 0; i < world; ++i) {
    if (!ptrs[i]) {
      set_last_error("%s: pointer %d of a per-rank array is null", what, i);
      return false;
    }
    pp.p[i] = ptrs[i];
  }
  return true;
}
unsigned long long ep_limit_ns(int wait_limit_ms) {
  return (unsigned long long)(wait_limit_ms > 0 ? wait_limit_ms : 10000) * 1000000ull;
}
}  // namespace

int tessera_sm100_ep_route_publish_device(const float* logits, int Tl, int E, int top_k, int normalize,
                                          int* assignment, float* weights, int* token_of_slot,
                                          int* expert_of_slot, float* weight_of_slot, int* group_sizes,
                                          int* my_offsets, int* slot_of_assignment, void* const* ctrl_ptrs,
                                          int world, int rank, int epoch, void* stream) {
  if (!logits || !assignment || !weights || !token_of_slot || !expert_of_slot || !weight_of_slot ||
      !group_sizes || !my_offsets || !slot_of_assignment || !ctrl_ptrs || Tl <= 0 || E <= 0 ||
      E > moe::kMaxExperts || top_k <= 0 || top_k > E || top_k > moe::kMaxTopK || world <= 0 ||
      world > moe::kEpMaxWorld || rank < 0 || rank >= world || E % world) {
    set_last_error("ep_route_publish: bad arguments (Tl %d E %d top_k %d world %d rank %d)", Tl, E, top_k,
                   world, rank);
    return kBadArg;
  }
  moe::PeerPtrs cp{};
  if (!ep_peer_ptrs(cp, ctrl_ptrs, world, "ep_route_publish")) return kBadArg;
  moe::ep_route_publish_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(
      logits, Tl, E, top_k, normalize, assignment, weights, token_of_slot, expert_of_slot, weight_of_slot,
      group_sizes, my_offsets, slot_of_assignment, cp, world, rank, epoch);
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  return kOk;
}

int tessera_sm100_ep_dispatch_signal_device(const void* x, const int* token_of_slot,
                                            const int* expert_of_slot, const int* my_offsets,
                                            void* const* ctrl_ptrs, void* const* recv_bufs, int world,
                                            int rank, int E, int max_slots, int capacity_rows, int H,
                                            int dtype, int epoch, int* group_offsets_local, int* dst_base,
                                            int* counter, int wait_limit_ms, void* stream) {
  const size_t row_bytes = (size_t)H * moe::dtype_size(dtype);
  if (!x || !token_of_slot || !expert_of_slot || !my_offsets || !ctrl_ptrs || !recv_bufs ||
      !group_offsets_local || !dst_base || !counter || world <= 0 || world > moe::kEpMaxWorld ||
      rank < 0 || rank >= world || E <= 0 || E > moe::kMaxExperts || E % world || (row_bytes % 16) ||
      max_slots <= 0) {
    set_last_error("ep_dispatch_signal: bad arguments (rows must be 16-byte multiples, world <= 8)");
    return kBadArg;
  }
  moe::PeerPtrs cp{}, rp{};
  if (!ep_peer_ptrs(cp, ctrl_ptrs, world, "ep_dispatch_signal") ||
      !ep_peer_ptrs(rp, recv_bufs, world, "ep_dispatch_signal"))
    return kBadArg;
  int* err = device_err_word();
  if (!err) return kDeviceFailed;
  const int vec = (int)(row_bytes / 16);
  // one warp per slot, 16 warps per CTA, at most two CTAs per SM (one wave: the flag waits of the
  // prologue are paid once)
  const int grid = (int)std::min<long long>(((long long)max_slots + 15) / 16, 2ll * sm_count());
  moe::ep_dispatch_signal_kernel<<<grid, 512, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x), token_of_slot, expert_of_slot, my_offsets, cp, rp, world, rank, E,
      capacity_rows, vec, epoch, group_offsets_local, dst_base, counter, ep_limit_ns(wait_limit_ms), err);
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  return kOk;
}

int tessera_sm100_ep_combine_signal_device(void* const* y_bufs, void* const* ctrl_ptrs,
                                           const int* assignment, const int* slot_of_assignment,
                                           const float* weights, const int* my_offsets,
                                           const int* dst_base, void* out, int T, int top_k, int world,
                                           int rank, int E, int capacity_rows, int H, int dtype, int epoch,
                                           int* counter, int wait_limit_ms, void* stream) {
  if (!y_bufs || !ctrl_ptrs || !assignment || !slot_of_assignment || !weights || !my_offsets ||
      !dst_base || !out || !counter || world <= 0 || world > moe::kEpMaxWorld || rank < 0 ||
      rank >= world || E % world || (H % 8) || T <= 0) {
    set_last_error("ep_combine_signal: bad arguments (H must be a multiple of 8, world <= 8, T > 0)");
    return kBadArg;
  }
  moe::PeerPtrs yp{}, cp{};
  if (!ep_peer_ptrs(yp, y_bufs, world, "ep_combine_signal") ||
      !ep_peer_ptrs(cp, ctrl_ptrs, world, "ep_combine_signal"))
    return kBadArg;
  int* err = device_err_word();
  if (!err) return kDeviceFailed;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int Ep = E / world;
  const unsigned long long lim = ep_limit_ns(wait_limit_ms);
  if (dtype == TESSERA_SM100_BF16)
    moe::ep_combine_signal_kernel<__nv_bfloat16, __nv_bfloat16><<<T, 256, 0, st>>>(
        yp, cp, assignment, slot_of_assignment, weights, my_offsets, dst_base,
        static_cast<__nv_bfloat16*>(out), T, top_k, world, rank, Ep, capacity_rows, H, epoch, counter, lim,
        err);
  else if (dtype == TESSERA_SM100_F16)
    moe::ep_combine_signal_kernel<__half, __half><<<T, 256, 0, st>>>(
        yp, cp, assignment, slot_of_assignment, weights, my_offsets, dst_base, static_cast<__half*>(out), T,
        top_k, world, rank, Ep, capacity_rows, H, epoch, counter, lim, err);
  else {
    set_last_error("ep_combine_signal: dtype must be bf16 or f16");
    return kBadArg;
  }
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  return kOk;
}

}  // extern "C"
