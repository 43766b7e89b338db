// Host side of the tcgen05 GEMM: tensor-map construction, launch, and the C entry points.
#include "gemm_sm100.cuh"
#include "gemm2_sm100.cuh"
#include "gemm_ag_sm100.cuh"

#include <algorithm>
#include <cstdlib>
#include <mutex>

#include "../../include/tessera_sm100.h"
#include "device_ctx.h"

namespace tsb {
namespace gemm {

namespace {

size_t out_size(int out_dtype) { return out_dtype == TESSERA_SM100_F32 ? 4 : 2; }

template <typename OutT, int kMode>
int launch_kernel(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tB2,
                  const CUtensorMap& tD, const Params& p, int grid, cudaStream_t stream) {
  // The attribute is per device; setting it on every call is cheap and keeps multi-device
  // processes correct.
  TSB_CUDA_OK(cudaFuncSetAttribute(gemm_kernel<OutT, kMode>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_ALLOC));
  gemm_kernel<OutT, kMode><<<grid, NUM_THREADS, SMEM_ALLOC, stream>>>(tA, tB, tB2, tD, p);
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  return kOk;
}

template <int kMode>
int dispatch_out(int out_dtype, const CUtensorMap& tA, const CUtensorMap& tB,
                 const CUtensorMap& tB2, const CUtensorMap& tD, const Params& p, int grid,
                 cudaStream_t stream) {
  switch (out_dtype) {
    case TESSERA_SM100_F32:
      return launch_kernel<float, kMode>(tA, tB, tB2, tD, p, grid, stream);
    case TESSERA_SM100_BF16:
      return launch_kernel<__nv_bfloat16, kMode>(tA, tB, tB2, tD, p, grid, stream);
    case TESSERA_SM100_F16:
      return launch_kernel<__half, kMode>(tA, tB, tB2, tD, p, grid, stream);
    default:
      break;
  }
  set_last_error("unsupported output dtype %d for this GEMM mode", out_dtype);
  return kBadArg;
}

// CTA-pair kernel: cluster of two, as many clusters as the device can hold at once.
template <typename OutT, int kMode>
int launch_pair_kernel(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tB2,
                       const CUtensorMap& tD, const Params& p, long long pair_tiles,
                       cudaStream_t stream) {
  TSB_CUDA_OK(cudaFuncSetAttribute(gemm2::gemm2_kernel<OutT, kMode>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, gemm2::SMEM_ALLOC));
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(gemm2::NUM_THREADS);
  cfg.dynamicSmemBytes = gemm2::SMEM_ALLOC;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  // How many clusters fit at once (GPCs with an odd SM count leave one SM unpaired).
  static int max_clusters[64] = {};
  const int dev = current_device();
  int mc = (dev >= 0 && dev < 64) ? max_clusters[dev] : 0;
  if (mc == 0) {
    cfg.gridDim = dim3(2 * (sm_count() / 2));
    if (cudaOccupancyMaxActiveClusters(&mc, gemm2::gemm2_kernel<OutT, kMode>, &cfg) != cudaSuccess ||
        mc <= 0) {
      cudaGetLastError();
      mc = sm_count() / 2;
    }
    if (dev >= 0 && dev < 64) max_clusters[dev] = mc;
  }
  const int clusters = (int)std::min<long long>(pair_tiles, mc);
  cfg.gridDim = dim3(2 * clusters);
  TSB_CUDA_OK(cudaLaunchKernelEx(&cfg, gemm2::gemm2_kernel<OutT, kMode>, tA, tB, tB2, tD, p));
  note_launch();
  return kOk;
}

// The all-gather GEMM: 256 x 256 pair tiles, every piece stored into all copies of the output; with
// p.ksplit = 2 the first wave of units are half-K units (workspace from the pool, reusable once this
// launch has finished on `stream`).
template <typename OutT>
int launch_ag_kernel(const CUtensorMap& tA, const CUtensorMap& tB, const PeerMaps& peers,
                     Params p, long long tiles, cudaStream_t stream) {
  TSB_CUDA_OK(cudaFuncSetAttribute(gemm_ag::gemm_ag_kernel<OutT>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, gemm_ag::SMEM_ALLOC));
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(gemm_ag::NUM_THREADS);
  cfg.dynamicSmemBytes = gemm_ag::SMEM_ALLOC;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  static int max_clusters[64] = {};
  const int dev = current_device();
  int mc = (dev >= 0 && dev < 64) ? max_clusters[dev] : 0;
  if (mc == 0) {
    cfg.gridDim = dim3(2 * (sm_count() / 2));
    if (cudaOccupancyMaxActiveClusters(&mc, gemm_ag::gemm_ag_kernel<OutT>, &cfg) != cudaSuccess || mc <= 0) {
      cudaGetLastError();
      mc = sm_count() / 2;
    }
    if (dev >= 0 && dev < 64) max_clusters[dev] = mc;
  }
  // With the first wave split, clusters 2t and 2t+1 share tile t: an even cluster count, and fp32
  // partial sums plus flags for those clusters / 2 tiles.
  int clusters = (int)std::min<long long>(tiles * p.ksplit, mc);
  if (p.ksplit == 2) {
    clusters &= ~1;
    if (clusters < 2) {
      p.ksplit = 1;
      clusters = (int)std::min<long long>(tiles, mc);
    }
  }
  void* ws = nullptr;
  if (p.ksplit == 2) {
    const size_t split_tiles = (size_t)clusters / 2;
    const size_t partial_bytes = split_tiles * gemm_ag::PARTIAL_BYTES_PER_TILE;
    const size_t flag_bytes = split_tiles * gemm_ag::FLAGS_PER_TILE * sizeof(int);
    ws = pool_alloc(partial_bytes + flag_bytes);
    if (!ws) return kDeviceFailed;
    p.partial = static_cast<float*>(ws);
    p.flags = reinterpret_cast<int*>(static_cast<char*>(ws) + partial_bytes);
    if (cudaMemsetAsync(p.flags, 0, flag_bytes, stream) != cudaSuccess) {
      set_last_error("gemm_allgather: clearing the flags failed: %s", cudaGetErrorString(cudaGetLastError()));
      pool_free_after(ws, stream);
      return kDeviceFailed;
    }
  }
  cfg.gridDim = dim3(2 * clusters);
  const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_ag::gemm_ag_kernel<OutT>, tA, tB, peers, p);
  if (ws) pool_free_after(ws, stream);
  if (e != cudaSuccess) {
    set_last_error("gemm_allgather: launch failed: %s", cudaGetErrorString(e));
    return kDeviceFailed;
  }
  note_launch();
  return kOk;
}

// TESSERA_SM100_GEMM_2CTA=0 keeps every GEMM on the single-CTA kernel.
bool pair_kernel_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("TESSERA_SM100_GEMM_2CTA");
    return !(e && e[0] == '0');
  }();
  return on;
}

CUtensorMapDataType tm_dtype(int dt) {
  switch (dt) {
    case TESSERA_SM100_BF16: return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    case TESSERA_SM100_F16: return CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    default: return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

// Dense (optionally batched) GEMM on device pointers with explicit leading dimensions and
// batch strides, all in elements. Every stride must make a 16-byte multiple.
int launch_plain(const void* A, const void* B, void* D, int batch, int M, int N, int K,
                 long long lda, long long ldb, long long ldd, long long sA, long long sB,
                 long long sD, int in_dtype, int out_dtype, cudaStream_t stream,
                 void* const* peer_D = nullptr, int num_peers = 0, const float* bias = nullptr,
                 const void* residual = nullptr, long long ldr = 0, int activation = 0,
                 int peer_first = 0) {
  if (!A || !B || !D || batch <= 0 || M <= 0 || N <= 0 || K <= 0) {
    set_last_error("gemm: null pointer or non-positive size (batch %d M %d N %d K %d)", batch, M,
                   N, K);
    return kBadArg;
  }
  if (in_dtype != TESSERA_SM100_BF16 && in_dtype != TESSERA_SM100_F16) {
    set_last_error("gemm: input dtype must be bf16 or f16");
    return kBadArg;
  }
  const size_t osz = out_size(out_dtype);
  if (!aligned16(A) || !aligned16(B) || !aligned16(D) || (lda * 2) % 16 || (ldb * 2) % 16 ||
      (ldd * (long long)osz) % 16 || (sA * 2) % 16 || (sB * 2) % 16 || (sD * (long long)osz) % 16) {
    set_last_error("gemm: operands must be 16-byte aligned with 16-byte-multiple strides");
    return kBadArg;
  }
  if (batch == 1) {  // any legal stride will do for a single batch
    sA = (long long)M * lda;
    sB = (long long)K * ldb;
    sD = (long long)M * ldd;
  }
  CUtensorMap tA, tB, tD;
  {
    uint64_t dims[3] = {(uint64_t)K, (uint64_t)M, (uint64_t)batch};
    uint64_t str[2] = {(uint64_t)lda * 2, (uint64_t)sA * 2};
    uint32_t box[3] = {BK, BM, 1};
    if (!encode_tmap(&tA, tm_dtype(in_dtype), 3, A, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return kBadArg;
  }
  {
    uint64_t dims[3] = {(uint64_t)N, (uint64_t)K, (uint64_t)batch};
    uint64_t str[2] = {(uint64_t)ldb * 2, (uint64_t)sB * 2};
    uint32_t box[3] = {64, BK, 1};
    if (!encode_tmap(&tB, tm_dtype(in_dtype), 3, B, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return kBadArg;
  }
  {
    uint64_t dims[3] = {(uint64_t)N, (uint64_t)M, (uint64_t)batch};
    uint64_t str[2] = {(uint64_t)ldd * osz, (uint64_t)sD * osz};
    uint32_t box[3] = {(uint32_t)(128 / osz), 32, 1};
    if (!encode_tmap(&tD, tm_dtype(out_dtype), 3, D, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return kBadArg;
  }
  // Large dense problems take the CTA-pair kernel (256 x 256 tiles, M = 256 MMAs): at least one
  // full wave of clusters.
  const long long pair_tiles =
      (long long)(((M + BM - 1) / BM + 1) / 2) * ((N + BN - 1) / BN) * batch;
  const bool use_pairs = pair_kernel_enabled() && M >= 2 * BM && pair_tiles >= sm_count() / 2;
  PeerMaps peer_maps;
  if (num_peers > 0) {
    // Column-parallel GEMM with the all-gather in the epilogue: one output map per copy of Y.
    if (num_peers > MAX_PEERS || !peer_D || batch != 1 || bias || residual || activation) {
      set_last_error("gemm: at most %d output copies, one batch and no fused epilogue", MAX_PEERS);
      return kBadArg;
    }
    uint64_t dims[3] = {(uint64_t)N, (uint64_t)M, (uint64_t)batch};
    uint64_t str[2] = {(uint64_t)ldd * osz, (uint64_t)sD * osz};
    uint32_t box[3] = {(uint32_t)(128 / osz), 32, 1};
    for (int i = 0; i < num_peers; ++i) {
      if (!peer_D[i] || !aligned16(peer_D[i])) {
        set_last_error("gemm: output copy %d is null or not 16-byte aligned", i);
        return kBadArg;
      }
      if (!encode_tmap(&peer_maps.m[i], tm_dtype(out_dtype), 3, peer_D[i], dims, str, box,
                       CU_TENSOR_MAP_SWIZZLE_128B))
        return kBadArg;
    }
    for (int i = num_peers; i < MAX_PEERS; ++i) peer_maps.m[i] = peer_maps.m[0];
  }
  Params p{};
  p.M = M;
  p.N = N;
  p.K = K;
  p.batch = batch;
  p.num_peers = num_peers;
  p.bias = bias;
  p.residual = residual;
  p.ldr = ldr;
  p.activation = activation;
  p.m_tiles = (M + BM - 1) / BM;
  p.n_tiles = (N + BN - 1) / BN;
  p.idesc = make_idesc_f16(in_dtype == TESSERA_SM100_BF16, false, true, BM, BN);
  p.group_offsets = nullptr;
  p.D = D;
  p.ldd = ldd;
  p.err = device_err_word();
  if (!p.err) return kDeviceFailed;
  const long long total = (long long)p.m_tiles * p.n_tiles * batch;
  if (num_peers > 0) {
    Params pa = p;
    pa.idesc = make_idesc_f16(in_dtype == TESSERA_SM100_BF16, false, true, 2 * BM, BN);
    pa.peer_first = peer_first;
    // Split K in the first wave when (a) there are fewer than four waves of whole tiles, so the first
    // tile time weighs on the step, (b) the K loop has at least 16 k-blocks, so each half still fills
    // the TMA ring, and (c) there are at most four copies. With more copies a CTA has more bytes to
    // store per tile than the tile takes to compute, the step is bound by how evenly the stores are
    // spread over the SMs, and the split (whose first wave stores from half of the CTAs) loses:
    // measured on eight GPUs 465 us against 250 us unsplit; on four 248 us against 273 us.
    const long long ag_tiles = (long long)((p.m_tiles + 1) / 2) * p.n_tiles;
    pa.ksplit = ((K + BK - 1) / BK >= 16 && ag_tiles < 4ll * (sm_count() / 2) && num_peers <= 4) ? 2 : 1;
    switch (out_dtype) {
      case TESSERA_SM100_F32: return launch_ag_kernel<float>(tA, tB, peer_maps, pa, ag_tiles, stream);
      case TESSERA_SM100_BF16: return launch_ag_kernel<__nv_bfloat16>(tA, tB, peer_maps, pa, ag_tiles, stream);
      case TESSERA_SM100_F16: return launch_ag_kernel<__half>(tA, tB, peer_maps, pa, ag_tiles, stream);
      default: break;
    }
  }
  if (use_pairs) {
    Params p2 = p;
    p2.idesc = make_idesc_f16(in_dtype == TESSERA_SM100_BF16, false, true, 2 * BM, BN);
    switch (out_dtype) {
      case TESSERA_SM100_F32:
        return launch_pair_kernel<float, kPlain>(tA, tB, tB, tD, p2, pair_tiles, stream);
      case TESSERA_SM100_BF16:
        return launch_pair_kernel<__nv_bfloat16, kPlain>(tA, tB, tB, tD, p2, pair_tiles, stream);
      case TESSERA_SM100_F16:
        return launch_pair_kernel<__half, kPlain>(tA, tB, tB, tD, p2, pair_tiles, stream);
      default: break;
    }
  }
  const int grid = (int)std::min<long long>(total, sm_count());
  return dispatch_out<kPlain>(out_dtype, tA, tB, tB, tD, p, grid, stream);
}

// Ragged grouped GEMM on device pointers. x[T,K] rows sorted by group, w[E,K,N] (and w2 for
// the SwiGLU form), offsets[E+1] int32 in device memory, out[T,N]. K and N multiples of 8.
int launch_grouped(const void* x, const void* w, const void* w2, const int* offsets, void* out,
                   int T, int K, int N, int E, int in_dtype, int out_dtype, bool swiglu,
                   cudaStream_t stream, const float* scale_a) {
  if (!x || !w || !offsets || !out || (swiglu && !w2) || T < 0 || K <= 0 || N <= 0 || E <= 0) {
    set_last_error("grouped_gemm: null pointer or bad size (T %d K %d N %d E %d)", T, K, N, E);
    return kBadArg;
  }
  if (T == 0) return kOk;
  if (in_dtype != TESSERA_SM100_BF16 && in_dtype != TESSERA_SM100_F16) {
    set_last_error("grouped_gemm: input dtype must be bf16 or f16");
    return kBadArg;
  }
  const size_t osz = out_size(out_dtype);
  if ((K % 8) || (N % 8) || !aligned16(x) || !aligned16(w) || !aligned16(out) ||
      (swiglu && !aligned16(w2))) {
    set_last_error("grouped_gemm: K and N must be multiples of 8 and pointers 16-byte aligned");
    return kBadArg;
  }
  CUtensorMap tA, tB, tB2, tD;
  {
    uint64_t dims[3] = {(uint64_t)K, (uint64_t)T, 1};
    uint64_t str[2] = {(uint64_t)K * 2, (uint64_t)T * K * 2};
    uint32_t box[3] = {BK, BM, 1};
    if (!encode_tmap(&tA, tm_dtype(in_dtype), 3, x, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return kBadArg;
  }
  {
    uint64_t dims[3] = {(uint64_t)N, (uint64_t)K, (uint64_t)E};
    uint64_t str[2] = {(uint64_t)N * 2, (uint64_t)K * N * 2};
    uint32_t box[3] = {64, BK, 1};
    if (!encode_tmap(&tB, tm_dtype(in_dtype), 3, w, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return kBadArg;
    if (swiglu) {
      if (!encode_tmap(&tB2, tm_dtype(in_dtype), 3, w2, dims, str, box,
                       CU_TENSOR_MAP_SWIZZLE_128B))
        return kBadArg;
    } else {
      tB2 = tB;
    }
  }
  {
    uint64_t dims[3] = {(uint64_t)N, (uint64_t)T, 1};
    uint64_t str[2] = {(uint64_t)N * osz, (uint64_t)T * N * osz};
    uint32_t box[3] = {(uint32_t)(128 / osz), 32, 1};
    if (!encode_tmap(&tD, tm_dtype(out_dtype), 3, out, dims, str, box,
                     CU_TENSOR_MAP_SWIZZLE_128B))
      return kBadArg;
  }
  Params p{};
  p.M = T;
  p.N = N;
  p.K = K;
  p.batch = E;
  const int out_w = swiglu ? BN / 2 : BN;
  p.m_tiles = 0;
  p.n_tiles = (N + out_w - 1) / out_w;
  p.idesc = make_idesc_f16(in_dtype == TESSERA_SM100_BF16, false, true, BM, BN);
  p.group_offsets = offsets;
  p.D = out;
  p.ldd = N;
  p.scale_a = scale_a;
  p.err = device_err_word();
  if (!p.err) return kDeviceFailed;
  // Upper bound on the number of tiles: every group may add one partial m-tile.
  const long long max_tiles = ((long long)(T + BM - 1) / BM + E) * p.n_tiles;
  const int grid = (int)std::min<long long>(max_tiles, sm_count());
  // Enough rows for at least one wave of 256-row pair tiles: the CTA-pair kernel.
  const long long max_pair_tiles = ((long long)(T + 2 * BM - 1) / (2 * BM) + E) * p.n_tiles;
  if (pair_kernel_enabled() && (long long)(T / (2 * BM)) * p.n_tiles >= sm_count() / 2) {
    Params p2 = p;
    p2.idesc = make_idesc_f16(in_dtype == TESSERA_SM100_BF16, false, true, 2 * BM, BN);
    if (swiglu) {
      if (out_dtype == TESSERA_SM100_F32)
        return launch_pair_kernel<float, kGroupedSwiGLU>(tA, tB, tB2, tD, p2, max_pair_tiles,
                                                         stream);
      if (out_dtype == TESSERA_SM100_BF16)
        return launch_pair_kernel<__nv_bfloat16, kGroupedSwiGLU>(tA, tB, tB2, tD, p2,
                                                                 max_pair_tiles, stream);
      if (out_dtype == TESSERA_SM100_F16)
        return launch_pair_kernel<__half, kGroupedSwiGLU>(tA, tB, tB2, tD, p2,
                                                          max_pair_tiles, stream);
    } else {
      if (out_dtype == TESSERA_SM100_F32)
        return launch_pair_kernel<float, kGrouped>(tA, tB, tB2, tD, p2, max_pair_tiles,
                                                   stream);
      if (out_dtype == TESSERA_SM100_BF16)
        return launch_pair_kernel<__nv_bfloat16, kGrouped>(tA, tB, tB2, tD, p2,
                                                           max_pair_tiles, stream);
      if (out_dtype == TESSERA_SM100_F16)
        return launch_pair_kernel<__half, kGrouped>(tA, tB, tB2, tD, p2, max_pair_tiles,
                                                    stream);
    }
  }
  if (swiglu)
    return dispatch_out<kGroupedSwiGLU>(out_dtype, tA, tB, tB2, tD, p, grid, stream);
  return dispatch_out<kGrouped>(out_dtype, tA, tB, tB2, tD, p, grid, stream);
}

// ---------------------------------------------------------------------------------------
// Row-pitch conversion kernels for operands whose natural row stride is not a 16-byte
// multiple (the TMA requirement). `esz` is the element size in bytes.
__global__ void repitch_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                               long long rows, long long row_bytes, long long src_pitch,
                               long long dst_pitch) {
  const long long total = rows * row_bytes;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / row_bytes;
    const long long c = i - r * row_bytes;
    dst[r * dst_pitch + c] = src[r * src_pitch + c];
  }
}

int repitch(const void* src, void* dst, long long rows, long long row_bytes, long long src_pitch,
            long long dst_pitch, cudaStream_t stream) {
  const long long total = rows * row_bytes;
  if (total == 0) return kOk;
  const int block = 256;
  const int grid = (int)std::min<long long>((total + block - 1) / block, 148 * 16);
  repitch_kernel<<<grid, block, 0, stream>>>(static_cast<const uint8_t*>(src),
                                             static_cast<uint8_t*>(dst), rows, row_bytes,
                                             src_pitch, dst_pitch);
  TSB_CUDA_OK(cudaGetLastError());
  note_launch();
  return kOk;
}

long long round_up8(long long v) { return (v + 7) & ~7ll; }

// Dense row-major batched GEMM on device pointers; pads through scratch when K or N is not
// a multiple of 8 (that path synchronises the stream before it frees the scratch).
int gemm_device(const void* A, const void* B, void* D, int batch, int M, int N, int K,
                int in_dtype, int out_dtype, cudaStream_t stream) {
  if (!A || !B || !D || batch <= 0 || M <= 0 || N <= 0 || K <= 0) {
    set_last_error("gemm: null pointer or non-positive size (batch %d M %d N %d K %d)", batch, M,
                   N, K);
    return kBadArg;
  }
  const size_t osz = out_size(out_dtype);
  const bool direct = (K % 8 == 0) && (N % 8 == 0) && aligned16(A) && aligned16(B) && aligned16(D);
  if (direct) {
    return launch_plain(A, B, D, batch, M, N, K, K, N, N, (long long)M * K, (long long)K * N,
                        (long long)M * N, in_dtype, out_dtype, stream);
  }
  const long long Kp = round_up8(K), Np = round_up8(N);
  void* pA = pool_alloc((size_t)batch * M * Kp * 2);
  void* pB = pool_alloc((size_t)batch * K * Np * 2);
  void* pD = pool_alloc((size_t)batch * M * Np * osz);
  int rc = kOk;
  if (!pA || !pB || !pD) rc = kDeviceFailed;
  if (rc == kOk) rc = repitch(A, pA, (long long)batch * M, (long long)K * 2, (long long)K * 2, Kp * 2, stream);
  if (rc == kOk) rc = repitch(B, pB, (long long)batch * K, (long long)N * 2, (long long)N * 2, Np * 2, stream);
  if (rc == kOk)
    rc = launch_plain(pA, pB, pD, batch, M, N, K, Kp, Np, Np, (long long)M * Kp,
                      (long long)K * Np, (long long)M * Np, in_dtype, out_dtype, stream);
  if (rc == kOk)
    rc = repitch(pD, D, (long long)batch * M, (long long)N * osz, Np * (long long)osz,
                 (long long)N * osz, stream);
  if (cudaStreamSynchronize(stream) != cudaSuccess && rc == kOk) {
    set_last_error("gemm: stream synchronise failed: %s", cudaGetErrorString(cudaGetLastError()));
    rc = kDeviceFailed;
  }
  pool_free(pA);
  pool_free(pB);
  pool_free(pD);
  return rc;
}

// Streams and events of the pipelined host-pointer form, created once per device.
constexpr int kMaxChunks = 32;
struct HostPipe {
  cudaStream_t up = nullptr, comp = nullptr, down = nullptr;
  cudaEvent_t b_ready = nullptr, up_done[kMaxChunks] = {}, comp_done[kMaxChunks] = {};
  bool ok = false;
  std::mutex busy;  // one pipelined call at a time per device: the events above are shared
};
HostPipe g_pipes[64];
std::mutex g_pipe_mu;

HostPipe* host_pipe() {
  const int dev = current_device();
  if (dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(g_pipe_mu);
  HostPipe& p = g_pipes[dev];
  if (!p.ok) {
    bool good = cudaStreamCreateWithFlags(&p.up, cudaStreamNonBlocking) == cudaSuccess &&
                cudaStreamCreateWithFlags(&p.comp, cudaStreamNonBlocking) == cudaSuccess &&
                cudaStreamCreateWithFlags(&p.down, cudaStreamNonBlocking) == cudaSuccess &&
                cudaEventCreateWithFlags(&p.b_ready, cudaEventDisableTiming) == cudaSuccess;
    for (int i = 0; good && i < kMaxChunks; ++i)
      good = cudaEventCreateWithFlags(&p.up_done[i], cudaEventDisableTiming) == cudaSuccess &&
             cudaEventCreateWithFlags(&p.comp_done[i], cudaEventDisableTiming) == cudaSuccess;
    if (!good) {
      cudaGetLastError();
      return nullptr;
    }
    p.ok = true;
  }
  return &p;
}

// Host-pointer form: upload (re-pitching rows on the way), run, download.
//
// Large problems are cut into chunks that flow through three streams — upload, compute,
// download — so the transfer of chunk i+1 to the device, the GEMM of chunk i and the transfer of
// chunk i-1 back to the host overlap (the link is full duplex; with page-locked host buffers the
// call then costs about the larger of the two transfer directions instead of their sum plus the
// kernel). A chunk is a block of rows of A and D (one batch entry when batch > 1); B is uploaded
// first (per entry when batched). Small problems take one chunk.
int gemm_host(const void* A, const void* B, void* D, int batch, int M, int N, int K, int in_dtype,
              int out_dtype) {
  if (!A || !B || !D || batch <= 0 || M <= 0 || N <= 0 || K <= 0) {
    set_last_error("gemm: null pointer or non-positive size (batch %d M %d N %d K %d)", batch, M,
                   N, K);
    return kBadArg;
  }
  if (int rc = ensure_device()) return rc;
  const size_t osz = out_size(out_dtype);
  const long long Kp = round_up8(K), Np = round_up8(N);
  const size_t bytes = ((size_t)batch * M * K + (size_t)batch * K * N) * 2 + (size_t)batch * M * N * osz;
  // Chunk plan: rows of one matrix, or whole batch entries.
  int chunks = 1;
  int row_start[kMaxChunks + 1] = {0};  // row chunks: [row_start[c], row_start[c + 1])
  HostPipe* pipe = nullptr;
  if (bytes >= (size_t)(32u << 20) && (pipe = host_pipe()) != nullptr) {
    if (batch > 1) {
      chunks = std::min(batch, kMaxChunks);
    } else {
      chunks = std::max(1, std::min({M / 820, kMaxChunks, 16}));  // 10 chunks at 8192 rows
      // Tuning override: TESSERA_SM100_HOST_GEMM_CHUNKS=<1..32> fixes the number of row chunks.
      if (const char* env = std::getenv("TESSERA_SM100_HOST_GEMM_CHUNKS")) {
        const int v = std::atoi(env);
        if (v >= 1) chunks = std::min({v, kMaxChunks, std::max(1, M / 128)});
      }
      // Chunk sizes fall off linearly (weights c+1, c, ..., 2): what cannot overlap with anything is
      // the GEMM and the download of the LAST chunk, so that one is small, while early chunks are
      // large enough to keep per-chunk overheads off the upload stream. Multiples of 128 rows.
      const long long wsum = (long long)chunks * (chunks + 3) / 2;
      int n = 0, r = 0;
      for (int c = 0; c < chunks && r < M; ++c) {
        long long rows = (long long)M * (chunks + 1 - c) / wsum;
        rows = std::max<long long>(128, (rows + 64) / 128 * 128);
        r = (int)std::min<long long>(M, r + rows);
        row_start[++n] = r;
      }
      row_start[n] = M;  // rounding leftovers go to the last chunk
      chunks = n;
    }
  }
  void* pA = pool_alloc((size_t)batch * M * Kp * 2);
  void* pB = pool_alloc((size_t)batch * K * Np * 2);
  void* pD = pool_alloc((size_t)batch * M * Np * osz);
  int rc = (pA && pB && pD) ? kOk : kDeviceFailed;
  auto fail = [&](const char* what) {
    set_last_error("gemm: %s failed: %s", what, cudaGetErrorString(cudaGetLastError()));
    rc = kDeviceFailed;
  };
  auto up2d = [&](void* dst, long long dpitch, const void* src, long long cols, long long rows,
                  cudaStream_t st, const char* what) {
    if (rc != kOk) return;
    const cudaError_t e =
        dpitch == cols  // contiguous on both sides: one linear copy
            ? cudaMemcpyAsync(dst, src, (size_t)rows * cols * 2, cudaMemcpyHostToDevice, st)
            : cudaMemcpy2DAsync(dst, dpitch * 2, src, (size_t)cols * 2, (size_t)cols * 2,
                                (size_t)rows, cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) fail(what);
  };
  auto down2d = [&](void* dst, const void* src, long long rows, cudaStream_t st) {
    if (rc != kOk) return;
    const cudaError_t e =
        Np == N ? cudaMemcpyAsync(dst, src, (size_t)rows * N * osz, cudaMemcpyDeviceToHost, st)
                : cudaMemcpy2DAsync(dst, (size_t)N * osz, src, Np * osz, (size_t)N * osz,
                                    (size_t)rows, cudaMemcpyDeviceToHost, st);
    if (e != cudaSuccess) fail("download of D");
  };
  const char* hA = static_cast<const char*>(A);
  const char* hB = static_cast<const char*>(B);
  char* hD = static_cast<char*>(D);
  char* dA = static_cast<char*>(pA);
  char* dB = static_cast<char*>(pB);
  char* dD = static_cast<char*>(pD);
  if (chunks <= 1) {
    cudaStream_t st = nullptr;
    up2d(pA, Kp, A, K, (long long)batch * M, st, "upload of A");
    up2d(pB, Np, B, N, (long long)batch * K, st, "upload of B");
    if (rc == kOk)
      rc = launch_plain(pA, pB, pD, batch, M, N, K, Kp, Np, Np, (long long)M * Kp,
                        (long long)K * Np, (long long)M * Np, in_dtype, out_dtype, st);
    down2d(D, pD, (long long)batch * M, st);
    if (cudaStreamSynchronize(st) != cudaSuccess && rc == kOk) fail("synchronise");
  } else {
    // Work queued earlier on the default stream (none by this library's host forms, which all
    // synchronise before returning) is not waited for: the three streams are non-blocking.
    std::lock_guard<std::mutex> one_at_a_time(pipe->busy);
    if (batch == 1) {
      up2d(pB, Np, B, N, K, pipe->up, "upload of B");
      if (rc == kOk && cudaEventRecord(pipe->b_ready, pipe->up) != cudaSuccess) fail("event record");
      if (rc == kOk && cudaStreamWaitEvent(pipe->comp, pipe->b_ready, 0) != cudaSuccess)
        fail("stream wait");
    }
    for (int c = 0; c < chunks && rc == kOk; ++c) {
      // chunk c: batch entries [e0, e1) x rows [r0, r1)
      int e0 = 0, e1 = 1, r0 = 0, r1 = M;
      if (batch > 1) {
        e0 = (int)((long long)batch * c / chunks);
        e1 = (int)((long long)batch * (c + 1) / chunks);
      } else {
        r0 = row_start[c];
        r1 = row_start[c + 1];
      }
      const long long a_off = (long long)e0 * M + r0;  // first row of A / D in this chunk
      const long long rows = batch > 1 ? (long long)(e1 - e0) * M : (r1 - r0);
      up2d(dA + a_off * Kp * 2, Kp, hA + a_off * K * 2, K, rows, pipe->up, "upload of A");
      if (batch > 1)
        up2d(dB + (long long)e0 * K * Np * 2, Np, hB + (long long)e0 * K * N * 2, N,
             (long long)(e1 - e0) * K, pipe->up, "upload of B");
      if (rc == kOk && cudaEventRecord(pipe->up_done[c], pipe->up) != cudaSuccess) fail("event record");
      if (rc == kOk && cudaStreamWaitEvent(pipe->comp, pipe->up_done[c], 0) != cudaSuccess)
        fail("stream wait");
      if (rc == kOk)
        rc = launch_plain(dA + a_off * Kp * 2, dB + (batch > 1 ? (long long)e0 * K * Np * 2 : 0),
                          dD + a_off * Np * osz, batch > 1 ? e1 - e0 : 1, batch > 1 ? M : r1 - r0, N,
                          K, Kp, Np, Np, (long long)M * Kp, (long long)K * Np, (long long)M * Np,
                          in_dtype, out_dtype, pipe->comp);
      if (rc == kOk && cudaEventRecord(pipe->comp_done[c], pipe->comp) != cudaSuccess)
        fail("event record");
      if (rc == kOk && cudaStreamWaitEvent(pipe->down, pipe->comp_done[c], 0) != cudaSuccess)
        fail("stream wait");
      down2d(hD + a_off * N * osz, dD + a_off * Np * osz, rows, pipe->down);
    }
    // Drain all three streams whatever happened, so the pooled buffers can be reused.
    const bool s1 = cudaStreamSynchronize(pipe->up) == cudaSuccess;
    const bool s2 = cudaStreamSynchronize(pipe->comp) == cudaSuccess;
    const bool s3 = cudaStreamSynchronize(pipe->down) == cudaSuccess;
    if (!(s1 && s2 && s3) && rc == kOk) fail("synchronise");
  }
  if (rc == kOk) {
    int e[4];
    if (consume_device_err(e) != 0) {
      set_last_error("gemm: kernel wait expired (code %d, block %d, detail %d)", e[0], e[1], e[2]);
      rc = kDeviceFailed;
    }
  }
  pool_free(pA);
  pool_free(pB);
  pool_free(pD);
  return rc;
}

// fp8 (e4m3) operands, both K-major: Aq[T or M, K] bytes and Bq_t[E or 1][N, K] bytes (B
// transposed). offsets == nullptr: one dense product (batch 1); otherwise ragged groups, with
// `swiglu` the fused gate/up form (Bq2_t = up weights). scale_a: one device float; scale_b /
// scale_b2: one device float per group. amax_out (optional, device uint32 zeroed by the caller)
// receives max |out| as stored.
template <typename OutT, int kMode>
int launch_fp8_kernel(bool pairs, const CUtensorMap& tA, const CUtensorMap& tB,
                      const CUtensorMap& tB2, const CUtensorMap& tD, const Params& p,
                      long long tiles, cudaStream_t stream) {
  if (pairs) {
    TSB_CUDA_OK(cudaFuncSetAttribute(gemm2::gemm2_kernel<OutT, kMode, true>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     gemm2::SMEM_ALLOC));
    cudaLaunchConfig_t cfg{};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.blockDim = dim3(gemm2::NUM_THREADS);
    cfg.dynamicSmemBytes = gemm2::SMEM_ALLOC;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const int clusters = (int)std::min<long long>(tiles, sm_count() / 2);
    cfg.gridDim = dim3(2 * clusters);
    TSB_CUDA_OK(cudaLaunchKernelEx(&cfg, gemm2::gemm2_kernel<OutT, kMode, true>, tA, tB, tB2, tD, p));
  } else {
    TSB_CUDA_OK(cudaFuncSetAttribute(gemm_kernel<OutT, kMode, true>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_ALLOC));
    const int grid = (int)std::min<long long>(tiles, sm_count());
    gemm_kernel<OutT, kMode, true><<<grid, NUM_THREADS, SMEM_ALLOC, stream>>>(tA, tB, tB2, tD, p);
    TSB_CUDA_OK(cudaGetLastError());
  }
  note_launch();
  return kOk;
}

int launch_fp8(const void* Aq, const void* Bq_t, const void* Bq2_t, const int* offsets, void* out,
               int T, int K, int N, int E, const float* scale_a, const float* scale_b,
               const float* scale_b2, int out_dtype, bool swiglu, unsigned int* amax_out,
               cudaStream_t stream, int fmt = 0) {
  const bool grouped = offsets != nullptr;
  if (fmt != TESSERA_SM100_FP8_E4M3 && fmt != TESSERA_SM100_FP8_E5M2) {
    set_last_error("gemm_fp8: format must be 0 (e4m3) or 1 (e5m2), got %d", fmt);
    return kBadArg;
  }
  if (!Aq || !Bq_t || !out || !scale_a || !scale_b || (swiglu && (!Bq2_t || !scale_b2 || !grouped)) ||
      T < 0 || K <= 0 || N <= 0 || E <= 0) {
    set_last_error("gemm_fp8: null pointer or bad size (T %d K %d N %d E %d)", T, K, N, E);
    return kBadArg;
  }
  if (T == 0) return kOk;
  const size_t osz = out_size(out_dtype);
  if ((K % 16) || (N % 8) || !aligned16(Aq) || !aligned16(Bq_t) || !aligned16(out) ||
      (swiglu && !aligned16(Bq2_t))) {
    set_last_error("gemm_fp8: K must be a multiple of 16, N of 8, pointers 16-byte aligned");
    return kBadArg;
  }
  CUtensorMap tA, tB, tB2, tD;
  {
    uint64_t dims[3] = {(uint64_t)K, (uint64_t)T, 1};
    uint64_t str[2] = {(uint64_t)K, (uint64_t)T * K};
    uint32_t box[3] = {128, BM, 1};
    if (!encode_tmap(&tA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, Aq, dims, str, box,
                     CU_TENSOR_MAP_SWIZZLE_128B))
      return kBadArg;
  }
  {
    uint64_t dims[3] = {(uint64_t)K, (uint64_t)N, (uint64_t)E};
    uint64_t str[2] = {(uint64_t)K, (uint64_t)N * K};
    uint32_t box[3] = {128, 128, 1};
    if (!encode_tmap(&tB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, Bq_t, dims, str, box,
                     CU_TENSOR_MAP_SWIZZLE_128B))
      return kBadArg;
    tB2 = tB;
    if (swiglu && !encode_tmap(&tB2, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, Bq2_t, dims, str, box,
                               CU_TENSOR_MAP_SWIZZLE_128B))
      return kBadArg;
  }
  {
    uint64_t dims[3] = {(uint64_t)N, (uint64_t)T, 1};
    uint64_t str[2] = {(uint64_t)N * osz, (uint64_t)T * N * osz};
    uint32_t box[3] = {(uint32_t)(128 / osz), 32, 1};
    if (!encode_tmap(&tD, tm_dtype(out_dtype), 3, out, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return kBadArg;
  }
  Params p{};
  p.M = T;
  p.N = N;
  p.K = K;
  p.batch = grouped ? E : 1;
  const int out_w = swiglu ? BN / 2 : BN;
  p.m_tiles = grouped ? 0 : (T + BM - 1) / BM;
  p.n_tiles = (N + out_w - 1) / out_w;
  p.group_offsets = offsets;
  p.D = out;
  p.ldd = N;
  p.scale_a = scale_a;
  p.scale_b = scale_b;
  p.scale_b2 = scale_b2;
  p.amax_out = amax_out;
  p.err = device_err_word();
  if (!p.err) return kDeviceFailed;
  const bool pairs = pair_kernel_enabled() && (long long)(T / (2 * BM)) * p.n_tiles >= sm_count() / 2;
  p.idesc = make_idesc_f8(pairs ? 2 * BM : BM, BN, fmt);
  const long long tiles =
      pairs ? ((long long)(T + 2 * BM - 1) / (2 * BM) + (grouped ? E : 0)) * p.n_tiles
            : ((long long)(T + BM - 1) / BM + (grouped ? E : 0)) * p.n_tiles;
#define TSB_FP8_CASE(OUT, MODE) return launch_fp8_kernel<OUT, MODE>(pairs, tA, tB, tB2, tD, p, tiles, stream)
  if (swiglu) {
    if (out_dtype == TESSERA_SM100_F32) TSB_FP8_CASE(float, kGroupedSwiGLU);
    if (out_dtype == TESSERA_SM100_BF16) TSB_FP8_CASE(__nv_bfloat16, kGroupedSwiGLU);
    if (out_dtype == TESSERA_SM100_F16) TSB_FP8_CASE(__half, kGroupedSwiGLU);
  } else if (grouped) {
    if (out_dtype == TESSERA_SM100_F32) TSB_FP8_CASE(float, kGrouped);
    if (out_dtype == TESSERA_SM100_BF16) TSB_FP8_CASE(__nv_bfloat16, kGrouped);
    if (out_dtype == TESSERA_SM100_F16) TSB_FP8_CASE(__half, kGrouped);
  } else {
    if (out_dtype == TESSERA_SM100_F32) TSB_FP8_CASE(float, kPlain);
    if (out_dtype == TESSERA_SM100_BF16) TSB_FP8_CASE(__nv_bfloat16, kPlain);
    if (out_dtype == TESSERA_SM100_F16) TSB_FP8_CASE(__half, kPlain);
  }
#undef TSB_FP8_CASE
  set_last_error("gemm_fp8: unsupported output dtype %d", out_dtype);
  return kBadArg;
}

}  // namespace gemm
}  // namespace tsb

using namespace tsb;

extern "C" {

int tessera_sm100_gemm_fp8_device(const void* Aq, const void* Bq_t, void* D, int M, int N, int K,
                                  const float* scale_a, const float* scale_b, int out_dtype,
                                  void* stream) {
  return gemm::launch_fp8(Aq, Bq_t, nullptr, nullptr, D, M, K, N, 1, scale_a, scale_b, nullptr,
                          out_dtype, false, nullptr, static_cast<cudaStream_t>(stream));
}
// The same three with the operand format as an argument: 0 = e4m3, 1 = e5m2 (both operands).
int tessera_sm100_gemm_fp8_fmt_device(const void* Aq, const void* Bq_t, void* D, int M, int N, int K,
                                      const float* scale_a, const float* scale_b, int out_dtype, int fmt,
                                      void* stream) {
  return gemm::launch_fp8(Aq, Bq_t, nullptr, nullptr, D, M, K, N, 1, scale_a, scale_b, nullptr,
                          out_dtype, false, nullptr, static_cast<cudaStream_t>(stream), fmt);
}
int tessera_sm100_grouped_gemm_fp8_fmt_device(const void* xq, const void* wq_t, const int* offsets,
                                              void* out, int T, int K, int N, int E, const float* scale_x,
                                              const float* scale_w, int out_dtype, int fmt, void* stream) {
  if (!offsets) {
    set_last_error("grouped_gemm_fp8: null offsets");
    return kBadArg;
  }
  return gemm::launch_fp8(xq, wq_t, nullptr, offsets, out, T, K, N, E, scale_x, scale_w, nullptr,
                          out_dtype, false, nullptr, static_cast<cudaStream_t>(stream), fmt);
}
int tessera_sm100_grouped_swiglu_fp8_fmt_device(const void* xq, const void* wgq_t, const void* wuq_t,
                                                const int* offsets, void* hidden, int T, int K, int F,
                                                int E, const float* scale_x, const float* scale_wg,
                                                const float* scale_wu, int out_dtype,
                                                unsigned int* amax_out, int fmt, void* stream) {
  if (!offsets) {
    set_last_error("grouped_swiglu_fp8: null offsets");
    return kBadArg;
  }
  return gemm::launch_fp8(xq, wgq_t, wuq_t, offsets, hidden, T, K, F, E, scale_x, scale_wg, scale_wu,
                          out_dtype, true, amax_out, static_cast<cudaStream_t>(stream), fmt);
}
int tessera_sm100_grouped_gemm_fp8_device(const void* xq, const void* wq_t, const int* offsets,
                                          void* out, int T, int K, int N, int E,
                                          const float* scale_x, const float* scale_w,
                                          int out_dtype, void* stream) {
  if (!offsets) {
    set_last_error("grouped_gemm_fp8: null offsets");
    return kBadArg;
  }
  return gemm::launch_fp8(xq, wq_t, nullptr, offsets, out, T, K, N, E, scale_x, scale_w, nullptr,
                          out_dtype, false, nullptr, static_cast<cudaStream_t>(stream));
}
int tessera_sm100_grouped_swiglu_fp8_device(const void* xq, const void* wgq_t, const void* wuq_t,
                                            const int* offsets, void* hidden, int T, int K, int F,
                                            int E, const float* scale_x, const float* scale_wg,
                                            const float* scale_wu, int out_dtype,
                                            unsigned int* amax_out, void* stream) {
  if (!offsets) {
    set_last_error("grouped_swiglu_fp8: null offsets");
    return kBadArg;
  }
  return gemm::launch_fp8(xq, wgq_t, wuq_t, offsets, hidden, T, K, F, E, scale_x, scale_wg, scale_wu,
                          out_dtype, true, amax_out, static_cast<cudaStream_t>(stream));
}

int tessera_sm100_mma_gemm_bf16(const void* A, const void* B, void* D, int M, int N, int K) {
  return gemm::gemm_host(A, B, D, 1, M, N, K, TESSERA_SM100_BF16, TESSERA_SM100_F32);
}
int tessera_sm100_mma_gemm_f16(const void* A, const void* B, void* D, int M, int N, int K) {
  return gemm::gemm_host(A, B, D, 1, M, N, K, TESSERA_SM100_F16, TESSERA_SM100_F32);
}
int tessera_sm100_mma_gemm_bf16_device(const void* A, const void* B, void* D, int M, int N, int K,
                                       void* stream) {
  return gemm::gemm_device(A, B, D, 1, M, N, K, TESSERA_SM100_BF16, TESSERA_SM100_F32,
                           static_cast<cudaStream_t>(stream));
}
int tessera_sm100_mma_gemm_f16_device(const void* A, const void* B, void* D, int M, int N, int K,
                                      void* stream) {
  return gemm::gemm_device(A, B, D, 1, M, N, K, TESSERA_SM100_F16, TESSERA_SM100_F32,
                           static_cast<cudaStream_t>(stream));
}
int tessera_sm100_gemm(const void* A, const void* B, void* D, int batch, int M, int N, int K,
                       int in_dtype, int out_dtype) {
  return gemm::gemm_host(A, B, D, batch, M, N, K, in_dtype, out_dtype);
}
int tessera_sm100_gemm_device(const void* A, const void* B, void* D, int batch, int M, int N,
                              int K, int in_dtype, int out_dtype, void* stream) {
  return gemm::gemm_device(A, B, D, batch, M, N, K, in_dtype, out_dtype,
                           static_cast<cudaStream_t>(stream));
}
int tessera_sm100_gemm_strided_device(const void* A, const void* B, void* D, int batch, int M,
                                      int N, int K, long long lda, long long ldb, long long ldd,
                                      long long strideA, long long strideB, long long strideD,
                                      int in_dtype, int out_dtype, void* stream) {
  return gemm::launch_plain(A, B, D, batch, M, N, K, lda, ldb, ldd, strideA, strideB, strideD,
                            in_dtype, out_dtype, static_cast<cudaStream_t>(stream));
}
// Column-parallel GEMM with the all-gather fused into the epilogue. B is the full [K, N_total]
// weight (rank r multiplies its columns [r*nb, (r+1)*nb), nb = N_total / world); Y_ptrs[i] is the
// base of rank i's [M, N_total] output (peer pointers for i != rank). Every tile is stored into
// all `world` copies, so when every rank's kernel has finished each copy holds the whole Y.
static int gemm_allgather(const void* A, const void* B_block, long long ldb, void* const* Y_ptrs,
                          int world, int rank, int M, int N_total, int K, int in_dtype, int out_dtype,
                          void* stream) {
  if (!Y_ptrs || world <= 0 || world > gemm::MAX_PEERS || rank < 0 || rank >= world ||
      N_total % world) {
    set_last_error("gemm_allgather: bad arguments (world %d rank %d N %d; world <= %d, N %% world == 0)",
                   world, rank, N_total, gemm::MAX_PEERS);
    return kBadArg;
  }
  const int nb = N_total / world;
  const size_t osz = out_dtype == TESSERA_SM100_F32 ? 4 : 2;
  if (nb % 8 || ldb < nb) {
    set_last_error("gemm_allgather: N / world (%d) must be a multiple of 8 and ldb (%lld) at least that", nb,
                   ldb);
    return kBadArg;
  }
  void* outs[gemm::MAX_PEERS];
  for (int i = 0; i < world; ++i) {
    if (!Y_ptrs[i]) {
      set_last_error("gemm_allgather: Y_ptrs[%d] is null", i);
      return kBadArg;
    }
    outs[i] = static_cast<char*>(Y_ptrs[i]) + (size_t)rank * nb * osz;
  }
  return gemm::launch_plain(A, B_block, outs[rank], 1, M, nb, K, K, ldb, N_total, 0, 0, 0, in_dtype,
                            out_dtype, static_cast<cudaStream_t>(stream), outs, world, nullptr, nullptr, 0, 0,
                            rank + 1);
}
int tessera_sm100_gemm_allgather_device(const void* A, const void* B, void* const* Y_ptrs, int world,
                                        int rank, int M, int N_total, int K, int in_dtype,
                                        int out_dtype, void* stream) {
  if (!B || world <= 0 || rank < 0 || N_total % world) {
    set_last_error("gemm_allgather: bad arguments");
    return kBadArg;
  }
  const char* Bblk = static_cast<const char*>(B) + (size_t)rank * (N_total / world) * 2;
  return gemm_allgather(A, Bblk, N_total, Y_ptrs, world, rank, M, N_total, K, in_dtype, out_dtype, stream);
}
// The same with only this rank's column block of B resident: B_block is [K, N_total / world] with
// leading dimension ldb (elements).
int tessera_sm100_gemm_allgather_block_device(const void* A, const void* B_block, long long ldb,
                                              void* const* Y_ptrs, int world, int rank, int M, int N_total,
                                              int K, int in_dtype, int out_dtype, void* stream) {
  return gemm_allgather(A, B_block, ldb, Y_ptrs, world, rank, M, N_total, K, in_dtype, out_dtype, stream);
}
// D = act(A*B + bias + residual): the GEMM with the reference's fused_epilogue applied in the
// kernel epilogue. bias is fp32 [N] or null; residual is [M,N] in the output dtype or null;
// activation 0 none, 1 relu, 2 gelu (tanh form), 3 silu. K and N must be multiples of 8.
int tessera_sm100_gemm_epilogue_device(const void* A, const void* B, void* D, int M, int N, int K,
                                       int in_dtype, int out_dtype, const float* bias,
                                       const void* residual, int activation, void* stream) {
  if ((K % 8) || (N % 8)) {
    set_last_error("gemm_epilogue: K (%d) and N (%d) must be multiples of 8", K, N);
    return kBadArg;
  }
  if (activation < 0 || activation > 3) {
    set_last_error("gemm_epilogue: activation must be 0 (none), 1 (relu), 2 (gelu) or 3 (silu)");
    return kBadArg;
  }
  if (out_dtype == TESSERA_SM100_F32 && residual && (reinterpret_cast<uintptr_t>(residual) & 3)) {
    set_last_error("gemm_epilogue: residual is misaligned");
    return kBadArg;
  }
  return gemm::launch_plain(A, B, D, 1, M, N, K, K, N, N, 0, 0, 0, in_dtype, out_dtype,
                            static_cast<cudaStream_t>(stream), nullptr, 0, bias, residual, N,
                            activation);
}
int tessera_sm100_grouped_gemm_device(const void* x, const void* w, const int* offsets, void* out,
                                      int T, int K, int N, int E, int in_dtype, int out_dtype,
                                      void* stream) {
  return gemm::launch_grouped(x, w, nullptr, offsets, out, T, K, N, E, in_dtype, out_dtype, false,
                              static_cast<cudaStream_t>(stream), nullptr);
}
// The same two with one fp32 scale (a device float) applied to the accumulators: operands that
// hold quantised values exactly (e4m3 activations as bf16 against dequantised NVFP4 weights).
int tessera_sm100_grouped_gemm_scaled_device(const void* x, const void* w, const int* offsets, void* out,
                                             int T, int K, int N, int E, int in_dtype, int out_dtype,
                                             const float* scale_a, void* stream) {
  return gemm::launch_grouped(x, w, nullptr, offsets, out, T, K, N, E, in_dtype, out_dtype, false,
                              static_cast<cudaStream_t>(stream), scale_a);
}
int tessera_sm100_grouped_swiglu_scaled_device(const void* x, const void* w_gate, const void* w_up,
                                               const int* offsets, void* out, int T, int K, int F, int E,
                                               int in_dtype, int out_dtype, const float* scale_a,
                                               void* stream) {
  return gemm::launch_grouped(x, w_gate, w_up, offsets, out, T, K, F, E, in_dtype, out_dtype, true,
                              static_cast<cudaStream_t>(stream), scale_a);
}
int tessera_sm100_grouped_swiglu_device(const void* x, const void* w_gate, const void* w_up,
                                        const int* offsets, void* out, int T, int K, int F, int E,
                                        int in_dtype, int out_dtype, void* stream) {
  return gemm::launch_grouped(x, w_gate, w_up, offsets, out, T, K, F, E, in_dtype, out_dtype, true,
                              static_cast<cudaStream_t>(stream), nullptr);
}

}  // extern "C"
