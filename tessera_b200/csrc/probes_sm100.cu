// Measurement probes that back the roofline figures: the issue rate of tcgen05.mma on resident
// operands, and the rate at which SM-issued stores fill the peers' copies of a column block (the
// exchange of the column-parallel GEMM on its own). Both are ordinary bounded kernels.
#include <algorithm>

#include "../../include/tessera_sm100.h"
#include "device_ctx.h"
#include "sm100_ptx.cuh"

namespace tsb {
namespace probes {

// `reps` groups of four back-to-back MMAs (M 128 per CTA, N given, K 16) on shared-memory operands
// that never change; the issuing thread times the whole run with clock64. kPair: cluster of two,
// cta_group::2 (M 256 over the pair, each CTA holding half of the B columns).
template <bool kPair>
__global__ void __launch_bounds__(128, 1)
mma_rate_kernel(int N, int b_mn_major, int reps, int stages, long long* out, int* err) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  __shared__ __align__(8) uint64_t bar_store;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const uint32_t bar = smem_u32(&bar_store);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b_cols = kPair ? N / 2 : N;  // B columns held by this CTA
  const int a_bytes = 128 * 64 * 2, b_bytes = 64 * b_cols * 2;
  const int stage_bytes = a_bytes + b_bytes;
  for (int i = threadIdx.x; i < stages * stage_bytes / 4; i += blockDim.x)
    reinterpret_cast<uint32_t*>(gen)[i] = 0x3c003c00u;  // small bf16 values
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(bar, 1);
    fence_mbar_init();
  }
  fence_proxy_async_smem();
  if (warp == 0) {
    if (kPair) {
      tmem_alloc_2cta(smem_u32(&tmem_slot), 512);
      tmem_relinquish_2cta();
    } else {
      tmem_alloc(smem_u32(&tmem_slot), 512);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (kPair) {
    cluster_arrive();
    cluster_wait();
  }
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const uint32_t rank = kPair ? cluster_ctarank() : 0;
  if (warp == 1 && lane == 0 && rank == 0) {
    const uint32_t idesc = make_idesc_f16(true, false, b_mn_major != 0, kPair ? 256 : 128, N);
    const uint32_t hi = smem_desc_hi(1024);
    const long long t0 = clock64();
    int s = 0;
    for (int r = 0; r < reps; ++r) {
      const uint32_t sa = base + s * stage_bytes, sb = sa + a_bytes;
      const uint32_t a_lo = smem_desc_lo(sa, 16);
      const uint32_t b_lo = smem_desc_lo(sb, b_mn_major ? 8192 : 16);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint32_t bl = b_lo + (b_mn_major ? k * 128 : k * 2);
        if (kPair)
          umma_f16_ss_parts_2cta(tmem, a_lo + k * 2, hi, bl, hi, idesc, 1u);
        else
          umma_f16_ss_parts(tmem, a_lo + k * 2, hi, bl, hi, idesc, 1u);
      }
      if (++s == stages) s = 0;
    }
    if (kPair)
      umma_commit_2cta(bar, 1);
    else
      umma_commit(bar);
    mbar_wait(bar, 0, &abort_flag, err, kErrWaitOther, 88);
    out[blockIdx.x] = clock64() - t0;
  }
  tc_fence_before();
  __syncthreads();
  if (kPair) {
    cluster_arrive();
    cluster_wait();
  }
  if (warp == 0) {
    tc_fence_after();
    if (kPair)
      tmem_dealloc_2cta(tmem, 512);
    else
      tmem_dealloc(tmem, 512);
  }
}

struct Copies {
  void* p[8];
};

// Every rank's column block [rows, row_bytes] of a row-major matrix (pitch bytes per row) copied
// from this rank's copy into all other ranks' copies with 16-byte stores: the all-gather of the
// column-parallel GEMM without the GEMM. `c.p[i]` is the block's first byte in rank i's copy.
__global__ void allgather_columns_kernel(Copies c, long long pitch, int rows, int row_bytes, int world,
                                         int rank) {
  const int vec_per_row = row_bytes / 16;
  const long long total = static_cast<long long>(rows) * vec_per_row;
  const uint8_t* mine = static_cast<const uint8_t*>(c.p[rank]);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vec_per_row;
    const long long off = r * pitch + (i - r * vec_per_row) * 16;
    const uint4 v = *reinterpret_cast<const uint4*>(mine + off);
    for (int k = 1; k < world; ++k) {
      const int dst = (rank + k) % world;  // every rank starts at a different peer
      *reinterpret_cast<uint4*>(static_cast<uint8_t*>(c.p[dst]) + off) = v;
    }
  }
}

}  // namespace probes
}  // namespace tsb

using namespace tsb;

extern "C" {

// SM cycles per tcgen05.mma (K 16, M 128 per CTA) issued back to back on resident operands, the
// maximum over all issuing CTAs of one full-GPU launch. pair != 0: cta_group::2 on clusters of two.
// N: 64..256 (a multiple of 16; 128 or 256 for pairs). b_mn_major: B operand layout. Returns the
// cycles in *cycles_per_mma.
int tessera_sm100_probe_mma_rate(int pair, int N, int b_mn_major, int reps, double* cycles_per_mma) {
  if (!cycles_per_mma || reps <= 0 || reps > 100000 || N < 64 || N > 256 || (N % 64) ||
      (pair && N < 128)) {
    set_last_error("probe_mma_rate: N must be 64, 128, 192 or 256 (128 or 256 for pairs), reps in (0, 100000]");
    return kBadArg;
  }
  if (N == 192) {
    set_last_error("probe_mma_rate: N = 192 is not laid out by this probe");
    return kBadArg;
  }
  if (int rc = ensure_device()) return rc;
  int* err = device_err_word();
  if (!err) return kDeviceFailed;
  const int sms = sm_count();
  const int stages = 4;
  const int b_cols = pair ? N / 2 : N;
  const int smem = stages * (16384 + 64 * b_cols * 2) + 2048;
  long long* out = static_cast<long long*>(pool_alloc(sizeof(long long) * sms));
  if (!out) return kDeviceFailed;
  auto done = [&](int rc) {
    pool_free_after_all(out);
    return rc;
  };
  if (cudaMemset(out, 0, sizeof(long long) * sms) != cudaSuccess) return done(kDeviceFailed);
  cudaError_t e;
  if (pair) {
    e = cudaFuncSetAttribute(probes::mma_rate_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    cudaLaunchConfig_t cfg{};
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    cfg.gridDim = dim3(2 * (sms / 2));
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = smem;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    if (e == cudaSuccess)
      e = cudaLaunchKernelEx(&cfg, probes::mma_rate_kernel<true>, N, b_mn_major, reps, stages, out, err);
  } else {
    e = cudaFuncSetAttribute(probes::mma_rate_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e == cudaSuccess) {
      probes::mma_rate_kernel<false><<<sms, 128, smem>>>(N, b_mn_major, reps, stages, out, err);
      e = cudaGetLastError();
    }
  }
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    set_last_error("probe_mma_rate: %s", cudaGetErrorString(e));
    cudaGetLastError();
    return done(kDeviceFailed);
  }
  note_launch();
  long long host[256] = {0};
  if (cudaMemcpy(host, out, sizeof(long long) * std::min(sms, 256), cudaMemcpyDeviceToHost) != cudaSuccess)
    return done(kDeviceFailed);
  long long worst = 0;
  for (int i = 0; i < std::min(sms, 256); ++i) worst = std::max(worst, host[i]);
  *cycles_per_mma = static_cast<double>(worst) / (4.0 * reps);
  return done(kOk);
}

// The exchange of the column-parallel GEMM on its own: this rank's column block of its copy of the
// row-major matrix [rows, N_total] (copies[rank]) is stored into every other copy (copies[i]: base of
// rank i's copy, a peer pointer for i != rank; a host array). Asynchronous on `stream`.
int tessera_sm100_allgather_columns_device(void* const* copies, int world, int rank, int rows,
                                           long long n_total, int elem_bytes, void* stream) {
  if (!copies || world <= 0 || world > 8 || rank < 0 || rank >= world || rows <= 0 || n_total <= 0 ||
      n_total % world || elem_bytes <= 0) {
    set_last_error("allgather_columns: bad arguments (world %d rank %d rows %d N %lld)", world, rank, rows,
                   n_total);
    return kBadArg;
  }
  const long long row_bytes = n_total / world * elem_bytes;
  if (row_bytes % 16 || row_bytes > (1ll << 30)) {
    set_last_error("allgather_columns: a rank's row segment (%lld bytes) must be a multiple of 16", row_bytes);
    return kBadArg;
  }
  if (world == 1) return kOk;
  probes::Copies c{};
  for (int i = 0; i < world; ++i) {
    if (!copies[i] || (reinterpret_cast<uintptr_t>(copies[i]) & 15)) {
      set_last_error("allgather_columns: copy %d is null or not 16-byte aligned", i);
      return kBadArg;
    }
    c.p[i] = static_cast<uint8_t*>(copies[i]) + rank * row_bytes;
  }
  const long long total = static_cast<long long>(rows) * (row_bytes / 16);
  const int grid = (int)std::min<long long>((total + 255) / 256, 148 * 8);
  probes::allgather_columns_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      c, n_total * elem_bytes, rows, (int)row_bytes, world, rank);
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  return kOk;
}

}  // extern "C"
