// NCCL-backed collectives behind the C ABI: the B200 counterpart of the reference's
// NCCLAdapter (src/collectives/include/tessera/Dialect/Collective/Runtime/Adapters.h:261-511)
// and of the one-process/multi-device ctypes executor (python/tessera/collectives.py:117-634).
//
// Differences that matter on NVLink 5 / NVSwitch:
//   * buffers are device resident and typed (bf16/f16/f32/bytes); nothing is staged through
//     the host and nothing synchronises the stream (the reference synchronises after every call)
//   * all_to_all_v takes per-peer byte counts, which expert-parallel MoE needs (the reference
//     supports equal shards only, Adapters.h:337-394)
//   * both process models are supported: one communicator per process
//     (unique id + init_rank, for one-process-per-GPU jobs) and init_all for a single process
//     that drives several GPUs.
// NCCL is resolved with dlopen at first use, so single-GPU users need no NCCL at all. C++
// exceptions never cross the ABI; every failure is a return code plus the thread-local error
// string.
#include <dlfcn.h>
#include <nccl.h>

#include <cstring>
#include <mutex>
#include <vector>

#include "../../include/tessera_sm100.h"
#include "device_ctx.h"

using namespace tsb;

namespace {

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommInitAll)(ncclComm_t*, int, const int*) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  ncclResult_t (*GetVersion)(int*) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*ReduceScatter)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  bool ok = false;
};

NcclApi g_nccl;
std::once_flag g_nccl_once;

void load_nccl() {
  const char* env = getenv("TESSERA_SM100_NCCL_LIB");
  const char* names[] = {env, "libnccl.so.2", "libnccl.so"};
  for (const char* n : names) {
    if (!n || !*n) continue;
    g_nccl.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    if (g_nccl.handle) break;
  }
  if (!g_nccl.handle) return;
  bool ok = true;
  auto sym = [&](const char* name) {
    void* p = dlsym(g_nccl.handle, name);
    if (!p) ok = false;
    return p;
  };
#define TSB_LOAD(field, name) g_nccl.field = reinterpret_cast<decltype(g_nccl.field)>(sym(name))
  TSB_LOAD(GetUniqueId, "ncclGetUniqueId");
  TSB_LOAD(CommInitRank, "ncclCommInitRank");
  TSB_LOAD(CommInitAll, "ncclCommInitAll");
  TSB_LOAD(CommDestroy, "ncclCommDestroy");
  TSB_LOAD(CommAbort, "ncclCommAbort");
  TSB_LOAD(CommGetAsyncError, "ncclCommGetAsyncError");
  TSB_LOAD(GetErrorString, "ncclGetErrorString");
  TSB_LOAD(GetVersion, "ncclGetVersion");
  TSB_LOAD(AllGather, "ncclAllGather");
  TSB_LOAD(AllReduce, "ncclAllReduce");
  TSB_LOAD(ReduceScatter, "ncclReduceScatter");
  TSB_LOAD(Send, "ncclSend");
  TSB_LOAD(Recv, "ncclRecv");
  TSB_LOAD(GroupStart, "ncclGroupStart");
  TSB_LOAD(GroupEnd, "ncclGroupEnd");
#undef TSB_LOAD
  g_nccl.ok = ok;
}

bool nccl_ready() {
  std::call_once(g_nccl_once, load_nccl);
  if (!g_nccl.ok) set_last_error("NCCL is not loadable (set TESSERA_SM100_NCCL_LIB to libnccl.so.2)");
  return g_nccl.ok;
}

struct Comm {
  ncclComm_t comm = nullptr;
  int rank = 0, world = 1, device = 0;
};

int fail(ncclResult_t r, const char* what) {
  set_last_error("%s failed: %s", what, g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "?");
  return kDeviceFailed;
}
#define TSB_NCCL_OK(expr)                       \
  do {                                          \
    ncclResult_t _r = (expr);                   \
    if (_r != ncclSuccess) return fail(_r, #expr); \
  } while (0)

bool nccl_dtype(int dt, ncclDataType_t* out, size_t* esz) {
  switch (dt) {
    case TESSERA_SM100_F32: *out = ncclFloat32; *esz = 4; return true;
    case TESSERA_SM100_BF16: *out = ncclBfloat16; *esz = 2; return true;
    case TESSERA_SM100_F16: *out = ncclFloat16; *esz = 2; return true;
    case TESSERA_SM100_U8: *out = ncclUint8; *esz = 1; return true;
    case TESSERA_SM100_I32: *out = ncclInt32; *esz = 4; return true;
    default: return false;
  }
}

bool red_op(int op, ncclRedOp_t* out) {
  switch (op) {
    case 0: *out = ncclSum; return true;
    case 1: *out = ncclMax; return true;
    case 2: *out = ncclMin; return true;
    case 3: *out = ncclProd; return true;
    default: return false;
  }
}

Comm* as_comm(void* h) { return static_cast<Comm*>(h); }

}  // namespace

extern "C" {

int tessera_sm100_nccl_version(int* version) {
  if (!version) return kBadArg;
  if (!nccl_ready()) return kNoDevice;
  TSB_NCCL_OK(g_nccl.GetVersion(version));
  return kOk;
}

int tessera_sm100_comm_unique_id(void* out128) {
  if (!out128) return kBadArg;
  if (!nccl_ready()) return kNoDevice;
  static_assert(sizeof(ncclUniqueId) == 128, "unique id size");
  ncclUniqueId id;
  TSB_NCCL_OK(g_nccl.GetUniqueId(&id));
  memcpy(out128, &id, sizeof(id));
  return kOk;
}

// One communicator for the calling process; the current CUDA device is the rank's GPU.
int tessera_sm100_comm_init_rank(const void* id128, int world, int rank, void** comm_out) {
  if (!id128 || !comm_out || world <= 0 || rank < 0 || rank >= world) {
    set_last_error("comm_init_rank: bad arguments (world %d rank %d)", world, rank);
    return kBadArg;
  }
  if (!nccl_ready()) return kNoDevice;
  if (int rc = ensure_device()) return rc;
  ncclUniqueId id;
  memcpy(&id, id128, sizeof(id));
  Comm* c = new Comm();
  c->rank = rank;
  c->world = world;
  c->device = current_device();
  ncclResult_t r = g_nccl.CommInitRank(&c->comm, world, id, rank);
  if (r != ncclSuccess) {
    delete c;
    return fail(r, "ncclCommInitRank");
  }
  *comm_out = c;
  return kOk;
}

// `ndev` communicators inside one process, rank i on devices[i] (ncclCommInitAll).
int tessera_sm100_comm_init_all(int ndev, const int* devices, void** comms_out) {
  if (ndev <= 0 || !devices || !comms_out) {
    set_last_error("comm_init_all: bad arguments");
    return kBadArg;
  }
  if (!nccl_ready()) return kNoDevice;
  std::vector<ncclComm_t> comms(ndev);
  TSB_NCCL_OK(g_nccl.CommInitAll(comms.data(), ndev, devices));
  for (int i = 0; i < ndev; ++i) {
    Comm* c = new Comm();
    c->comm = comms[i];
    c->rank = i;
    c->world = ndev;
    c->device = devices[i];
    comms_out[i] = c;
  }
  return kOk;
}

int tessera_sm100_comm_destroy(void* comm) {
  if (!comm) return kOk;
  Comm* c = as_comm(comm);
  if (g_nccl.ok && c->comm) g_nccl.CommDestroy(c->comm);
  delete c;
  return kOk;
}

// Tears the communicator down without waiting for outstanding operations (used after a peer
// was reported lost on the host side).
int tessera_sm100_comm_abort(void* comm) {
  if (!comm) return kOk;
  Comm* c = as_comm(comm);
  if (g_nccl.ok && c->comm) g_nccl.CommAbort(c->comm);
  delete c;
  return kOk;
}

int tessera_sm100_comm_info(void* comm, int* rank, int* world, int* device) {
  if (!comm) return kBadArg;
  Comm* c = as_comm(comm);
  if (rank) *rank = c->rank;
  if (world) *world = c->world;
  if (device) *device = c->device;
  return kOk;
}

// 0 when the communicator reports no asynchronous error, 3 otherwise (text in last_error).
int tessera_sm100_comm_async_error(void* comm) {
  if (!comm) return kBadArg;
  if (!nccl_ready()) return kNoDevice;
  ncclResult_t state = ncclSuccess;
  TSB_NCCL_OK(g_nccl.CommGetAsyncError(as_comm(comm)->comm, &state));
  if (state != ncclSuccess && state != ncclInProgress) return fail(state, "communicator");
  return kOk;
}

int tessera_sm100_group_start(void) {
  if (!nccl_ready()) return kNoDevice;
  TSB_NCCL_OK(g_nccl.GroupStart());
  return kOk;
}
int tessera_sm100_group_end(void) {
  if (!nccl_ready()) return kNoDevice;
  TSB_NCCL_OK(g_nccl.GroupEnd());
  return kOk;
}

int tessera_sm100_all_gather(void* comm, const void* send, void* recv, size_t count_per_rank,
                             int dtype, void* stream) {
  ncclDataType_t dt;
  size_t esz;
  if (!comm || !send || !recv || !nccl_dtype(dtype, &dt, &esz)) {
    set_last_error("all_gather: bad arguments");
    return kBadArg;
  }
  if (!nccl_ready()) return kNoDevice;
  TSB_NCCL_OK(g_nccl.AllGather(send, recv, count_per_rank, dt, as_comm(comm)->comm,
                               static_cast<cudaStream_t>(stream)));
  return kOk;
}

int tessera_sm100_all_reduce(void* comm, const void* send, void* recv, size_t count, int dtype,
                             int op, void* stream) {
  ncclDataType_t dt;
  size_t esz;
  ncclRedOp_t rop;
  if (!comm || !send || !recv || !nccl_dtype(dtype, &dt, &esz) || !red_op(op, &rop)) {
    set_last_error("all_reduce: bad arguments");
    return kBadArg;
  }
  if (!nccl_ready()) return kNoDevice;
  TSB_NCCL_OK(g_nccl.AllReduce(send, recv, count, dt, rop, as_comm(comm)->comm,
                               static_cast<cudaStream_t>(stream)));
  return kOk;
}

int tessera_sm100_reduce_scatter(void* comm, const void* send, void* recv, size_t recv_count,
                                 int dtype, int op, void* stream) {
  ncclDataType_t dt;
  size_t esz;
  ncclRedOp_t rop;
  if (!comm || !send || !recv || !nccl_dtype(dtype, &dt, &esz) || !red_op(op, &rop)) {
    set_last_error("reduce_scatter: bad arguments");
    return kBadArg;
  }
  if (!nccl_ready()) return kNoDevice;
  TSB_NCCL_OK(g_nccl.ReduceScatter(send, recv, recv_count, dt, rop, as_comm(comm)->comm,
                                   static_cast<cudaStream_t>(stream)));
  return kOk;
}

// Ragged all-to-all in bytes: peer p receives send[send_offs[p] .. +send_bytes[p]) and this rank
// receives recv_bytes[p] bytes from peer p at recv + recv_offs[p]. The four arrays are HOST
// arrays of length world. Equal shards are the special case the reference's all_to_all covers.
int tessera_sm100_all_to_all_v(void* comm, const void* send, const size_t* send_bytes,
                               const size_t* send_offs, void* recv, const size_t* recv_bytes,
                               const size_t* recv_offs, void* stream) {
  if (!comm || !send_bytes || !send_offs || !recv_bytes || !recv_offs) {
    set_last_error("all_to_all_v: bad arguments");
    return kBadArg;
  }
  if (!nccl_ready()) return kNoDevice;
  Comm* c = as_comm(comm);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  TSB_NCCL_OK(g_nccl.GroupStart());
  for (int p = 0; p < c->world; ++p) {
    if (send_bytes[p]) {
      ncclResult_t r = g_nccl.Send(static_cast<const char*>(send) + send_offs[p], send_bytes[p],
                                   ncclUint8, p, c->comm, st);
      if (r != ncclSuccess) {
        g_nccl.GroupEnd();
        return fail(r, "ncclSend");
      }
    }
    if (recv_bytes[p]) {
      ncclResult_t r = g_nccl.Recv(static_cast<char*>(recv) + recv_offs[p], recv_bytes[p],
                                   ncclUint8, p, c->comm, st);
      if (r != ncclSuccess) {
        g_nccl.GroupEnd();
        return fail(r, "ncclRecv");
      }
    }
  }
  TSB_NCCL_OK(g_nccl.GroupEnd());
  return kOk;
}

int tessera_sm100_all_to_all(void* comm, const void* send, void* recv, size_t bytes_per_peer,
                             void* stream) {
  if (!comm) return kBadArg;
  const int world = as_comm(comm)->world;
  std::vector<size_t> counts(world, bytes_per_peer), offs(world);
  for (int p = 0; p < world; ++p) offs[p] = (size_t)p * bytes_per_peer;
  return tessera_sm100_all_to_all_v(comm, send, counts.data(), offs.data(), recv, counts.data(),
                                    offs.data(), stream);
}

// ---- peer memory (CUDA IPC) for kernels that store straight into another GPU's buffer ----
int tessera_sm100_ipc_get_handle(void* device_ptr, void* handle64) {
  if (!device_ptr || !handle64) return kBadArg;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "ipc handle size");
  cudaIpcMemHandle_t h;
  TSB_CUDA_OK(cudaIpcGetMemHandle(&h, device_ptr));
  memcpy(handle64, &h, sizeof(h));
  return kOk;
}
int tessera_sm100_ipc_open_handle(const void* handle64, void** device_ptr) {
  if (!handle64 || !device_ptr) return kBadArg;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  TSB_CUDA_OK(cudaIpcOpenMemHandle(device_ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return kOk;
}
int tessera_sm100_ipc_close_handle(void* device_ptr) {
  if (!device_ptr) return kOk;
  TSB_CUDA_OK(cudaIpcCloseMemHandle(device_ptr));
  return kOk;
}

}  // extern "C"
