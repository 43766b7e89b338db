"""Multi-GPU forms of the hot path, one process per GPU.

* ``tp_column_range`` / ``TensorParallelGemm`` — column-parallel GEMM: W split on N, A replicated,
  ``Y = all_gather(A @ W_r, axis=1)`` (python/tessera/compiler/tensor_parallel.py:118-123).
* ``ep_plan`` / ``ExpertParallelMoE`` — expert-parallel MoE forward partitioned like
  ``megamoe_forward`` (python/tessera/distributed/moe.py:358-483): tokens row-sharded, rank r owns
  experts [r*Ep, (r+1)*Ep), a dispatch exchange, the local expert FFN, a combine exchange and a
  weighted sum per token. Unlike the reference nothing is padded to a capacity: the exchanges are
  ragged, sized from the routing histogram (``plan_all_to_all``, :252-315).

The planning code is plain numpy and independent of where the arithmetic runs. ``ExpertParallelMoE``
takes a *transport* (how ranks exchange rows) and a *compute backend* (how rows are gathered and
the expert FFN is evaluated); on a GPU job these are NCCL + the sm_100a kernels
(``NcclTransport`` / ``GpuMoeBackend``), while the CPU tests drive the very same planning and
sequencing with ``torch.distributed`` (gloo) and a numpy backend.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Protocol, Sequence

import numpy as np


# ---------------------------------------------------------------------------- tensor parallel
def tp_column_range(n: int, world: int, rank: int) -> tuple:
    """Column block of rank ``rank`` when N is split evenly over ``world`` ranks."""
    if n % world:
        raise ValueError(f"N={n} is not divisible by the tensor-parallel size {world}")
    nb = n // world
    return rank * nb, nb


class TensorParallelGemm:
    """Column-parallel GEMM whose epilogue is the all-gather: rank r multiplies its column block of
    W and stores every output tile into every rank's Y over NVLink
    (``tessera_sm100_gemm_allgather_device``). ``gather_host`` exchanges the 64-byte CUDA IPC
    handles of the Y buffers (e.g. ``torch.distributed.all_gather_object`` over gloo). After a
    call, synchronise the stream and pass a host barrier before reading ``self.Y``.

    ``run_host`` is the host-operand form: A is replicated data, so each rank uploads only M / world
    of its rows (plus its own column block of W), the rows are all-gathered over NVLink into every
    rank's device copy of A, the fused GEMM runs, and the rank's own block of Y comes back."""

    def __init__(self, M: int, N: int, K: int, world: int, rank: int, gather_host, dtype, out_dtype):
        import ctypes
        from . import _lib, device
        from .device import DeviceArray
        tp_column_range(N, world, rank)
        self.M, self.N, self.K, self.world, self.rank = M, N, K, world, rank
        self.dtype, self.out_dtype = np.dtype(dtype), np.dtype(out_dtype)
        self._in, self._out = device.dtype_code(dtype), device.dtype_code(out_dtype)
        self.Y = DeviceArray.zeros((M, N), out_dtype)
        self._A = self._Wb = None            # device operands of run_host, made on first use
        device.synchronize()
        handle = ctypes.create_string_buffer(64)
        _lib.call("tessera_sm100_ipc_get_handle", self.Y.ptr, handle)
        handles = gather_host(handle.raw)
        self._opened = []
        ptrs = []
        for r in range(world):
            if r == rank:
                ptrs.append(self.Y.ptr)
            else:
                p = ctypes.c_void_p()
                _lib.call("tessera_sm100_ipc_open_handle", ctypes.c_char_p(handles[r]), ctypes.byref(p))
                self._opened.append(p.value)
                ptrs.append(p.value)
        self._ptrs = (ctypes.c_void_p * world)(*ptrs)

    def __call__(self, A, W_full, stream=None) -> None:
        from . import _lib, device
        _lib.call("tessera_sm100_gemm_allgather_device", A.ptr, W_full.ptr, self._ptrs, self.world,
                  self.rank, self.M, self.N, self.K, self._in, self._out, device._stream_handle(stream))

    def exchange_only(self, stream=None) -> None:
        """The all-gather without the GEMM: this rank's column block of ``self.Y`` stored into every other
        rank's Y by a plain copy kernel. Timed on all ranks at once it gives the exchange floor of the
        fused kernel on the machine at hand."""
        from . import _lib, device
        _lib.call("tessera_sm100_allgather_columns_device", self._ptrs, self.world, self.rank, self.M, self.N,
                  self.out_dtype.itemsize, device._stream_handle(stream))

    def run_host(self, A_rows: np.ndarray, W_block: np.ndarray, Y_block: np.ndarray, comm, stream=None) -> None:
        """``A_rows``: rows [rank*M/world, (rank+1)*M/world) of A, ``W_block``: this rank's (K, N/world)
        columns of W, ``Y_block``: (M, N/world) host array that receives this rank's columns of Y
        (page-locked arrays make the copies asynchronous). ``comm`` is a ``collectives.Communicator``.
        Returns after this rank's block has arrived; the other ranks' blocks of ``self.Y`` are
        complete once every rank has returned."""
        from . import _lib, device
        from .device import DeviceArray
        M, N, K, W, r = self.M, self.N, self.K, self.world, self.rank
        if M % W:
            raise ValueError(f"M={M} is not divisible by the tensor-parallel size {W}")
        mb, nb = M // W, N // W
        if A_rows.shape != (mb, K) or W_block.shape != (K, nb) or Y_block.shape != (M, nb):
            raise ValueError("run_host: operand shapes do not match this rank's shard")
        if self._A is None:
            from .device import Event, Stream
            self._A, self._Wb = DeviceArray((M, K), self.dtype), DeviceArray((K, nb), self.dtype)
            self._Yb = DeviceArray((M, nb), self.out_dtype)          # this rank's block of Y, contiguous
            self._side, self._w_ready = Stream(), Event()
        sh = device._stream_handle(stream)
        isz, osz = self.dtype.itemsize, self.out_dtype.itemsize
        mine = self._A.view((mb, K), r * mb * K)
        # the rows of A go up first (the all-gather waits for nothing else); the block of W goes up on a
        # second stream while the all-gather runs
        _lib.call("tessera_sm100_device_upload", mine.ptr, A_rows.ctypes.data, mb * K * isz, sh)
        _lib.call("tessera_sm100_device_upload", self._Wb.ptr, W_block.ctypes.data, K * nb * isz, self._side.handle)
        self._w_ready.record(self._side)
        if W > 1:
            comm.all_gather(mine, self._A, stream)            # in place: block r of A is already there
        _lib.call("tessera_sm100_stream_wait_event", sh, self._w_ready.handle)
        _lib.call("tessera_sm100_gemm_allgather_block_device", self._A.ptr, self._Wb.ptr, nb, self._ptrs, W, r,
                  M, N, K, self._in, self._out, sh)
        # the rank's column block is strided in Y: compact it on the device, then one contiguous copy down
        _lib.call("tessera_sm100_device_copy_2d", self._Yb.ptr, nb * osz, self.Y.ptr + r * nb * osz, N * osz,
                  nb * osz, M, sh)
        _lib.call("tessera_sm100_device_download", Y_block.ctypes.data, self._Yb.ptr, M * nb * osz, sh)
        _lib.call("tessera_sm100_stream_synchronize", sh)

    def close(self) -> None:
        from . import _lib
        for p in self._opened:
            _lib.call("tessera_sm100_ipc_close_handle", p)
        self._opened = []
        if self._A is not None:
            self._side.close()
            self._w_ready.close()
            self._A = None


# ---------------------------------------------------------------------------- expert parallel
@dataclass
class EPPlan:
    world: int
    rank: int
    experts_per_rank: int
    top_k: int
    # send side (this rank's tokens)
    send_token: np.ndarray          # (Ssend,) int32 local token of each sent row, in send order
    send_counts: np.ndarray         # (world,) rows sent to each destination rank
    slot_of_assignment: np.ndarray  # (Tl, k) int32 position in send order of slot (t, j), -1 dropped
    send_expert_counts: np.ndarray  # (world, Ep) rows per destination and local expert


def ep_plan(assignment: np.ndarray, num_experts: int, world: int, rank: int) -> EPPlan:
    """Send-side plan from this rank's routing table (``assignment`` (Tl, k), -1 = dropped).
    Rows go out ordered by (destination rank, expert, token-major slot), so every receiver gets
    from every source a block that is already sorted by its local expert id."""
    assignment = np.asarray(assignment)
    if num_experts % world:
        raise ValueError(f"num_experts={num_experts} must be divisible by world_size={world}")
    Ep = num_experts // world
    Tl, k = assignment.shape
    flat = assignment.reshape(-1).astype(np.int64)
    kept = np.nonzero(flat >= 0)[0]
    order = kept[np.argsort(flat[kept], kind="stable")]      # by expert == by (dst, local expert)
    send_token = (order // k).astype(np.int32)
    slot_of = np.full(Tl * k, -1, np.int32)
    slot_of[order] = np.arange(order.shape[0], dtype=np.int32)
    counts = np.bincount(flat[order], minlength=num_experts).reshape(world, Ep).astype(np.int64)
    return EPPlan(world, rank, Ep, k, send_token, counts.sum(axis=1), slot_of.reshape(Tl, k), counts)


@dataclass
class EPRecvPlan:
    recv_counts: np.ndarray    # (world,) rows received from each source
    group_sizes: np.ndarray    # (Ep,) rows per local expert
    group_offsets: np.ndarray  # (Ep+1,) int32
    to_grouped: np.ndarray     # (Srecv,) int32: grouped row i comes from received row to_grouped[i]
    from_grouped: np.ndarray   # (Srecv,) int32: received row i sits at grouped row from_grouped[i]


def ep_recv_plan(all_expert_counts: np.ndarray, rank: int) -> EPRecvPlan:
    """Receive-side plan from the gathered ``send_expert_counts`` of every rank
    (shape (world_src, world_dst, Ep)). Received rows arrive source-major; the expert FFN wants
    them expert-major (source-major inside an expert), which is the stable expert sort the
    single-device layer applies."""
    counts = np.asarray(all_expert_counts)[:, rank, :]        # (src, Ep) rows bound for this rank
    world, Ep = counts.shape
    recv_counts = counts.sum(axis=1)
    total = int(recv_counts.sum())
    src_base = np.concatenate(([0], np.cumsum(recv_counts)[:-1]))
    in_src = np.concatenate((np.zeros((world, 1), np.int64), np.cumsum(counts, axis=1)[:, :-1]), axis=1)
    to_grouped = np.empty(total, np.int32)
    pos = 0
    for e in range(Ep):
        for s in range(world):
            n = int(counts[s, e])
            start = int(src_base[s] + in_src[s, e])
            to_grouped[pos:pos + n] = np.arange(start, start + n, dtype=np.int32)
            pos += n
    from_grouped = np.empty(total, np.int32)
    from_grouped[to_grouped] = np.arange(total, dtype=np.int32)
    group_sizes = counts.sum(axis=0).astype(np.int32)
    offsets = np.zeros(Ep + 1, np.int32)
    offsets[1:] = np.cumsum(group_sizes)
    return EPRecvPlan(recv_counts, group_sizes, offsets, to_grouped, from_grouped)


class Transport(Protocol):
    rank: int
    world: int

    def all_gather_small(self, arr: np.ndarray) -> np.ndarray: ...
    def exchange_rows(self, rows, send_counts: Sequence[int], recv_counts: Sequence[int]): ...


class MoeBackend(Protocol):
    def route(self, logits: np.ndarray, top_k: int, normalize: bool): ...       # -> (assignment, weights) host
    def gather_rows(self, rows, index: np.ndarray): ...
    def expert_ffn(self, rows, group_offsets: np.ndarray): ...
    def combine(self, rows, slot_of: np.ndarray, weights: np.ndarray, num_tokens: int): ...


class ExpertParallelMoE:
    """Sequencing of the expert-parallel forward for ONE rank."""

    def __init__(self, num_experts: int, top_k: int, transport: Transport, backend: MoeBackend,
                 normalize_weights: bool = True) -> None:
        if num_experts % transport.world:
            raise ValueError("num_experts must be divisible by the number of ranks")
        self.E, self.k = num_experts, top_k
        self.t, self.b = transport, backend
        self.normalize = normalize_weights

    def forward(self, x_local, logits_local: np.ndarray):
        """``x_local`` (Tl, H) rows of this rank, ``logits_local`` (Tl, E) router logits. Returns
        the (Tl, H) output rows of this rank (backend array type)."""
        t, b = self.t, self.b
        assignment, weights = b.route(logits_local, self.k, self.normalize)
        plan = ep_plan(assignment, self.E, t.world, t.rank)
        all_counts = t.all_gather_small(plan.send_expert_counts)          # (world, world, Ep)
        rplan = ep_recv_plan(all_counts, t.rank)
        send_rows = b.gather_rows(x_local, plan.send_token)               # dispatch pack
        recv_rows = t.exchange_rows(send_rows, plan.send_counts, rplan.recv_counts)
        grouped = b.gather_rows(recv_rows, rplan.to_grouped)              # expert-major
        y_grouped = b.expert_ffn(grouped, rplan.group_offsets)
        y_recv_order = b.gather_rows(y_grouped, rplan.from_grouped)       # back to source-major
        y_back = t.exchange_rows(y_recv_order, rplan.recv_counts, plan.send_counts)
        return b.combine(y_back, plan.slot_of_assignment, weights, int(np.asarray(logits_local).shape[0]))


# ---------------------------------------------------------------------------- GPU pieces
class NcclTransport:
    """Row exchange over a ``collectives.Communicator``; small host metadata travels through a
    caller-supplied ``gather_host`` (e.g. ``torch.distributed.all_gather_object`` over gloo)."""

    def __init__(self, comm, gather_host, stream=None) -> None:
        self.comm, self.rank, self.world = comm, comm.rank, comm.world
        self._gather_host = gather_host
        self.stream = stream

    def all_gather_small(self, arr: np.ndarray) -> np.ndarray:
        """Small integer metadata over NCCL (one upload, one all-gather, one download)."""
        from .device import DeviceArray
        a = np.ascontiguousarray(arr, np.int32)
        send = DeviceArray.from_host(a, pooled=True)
        recv = DeviceArray((self.world,) + a.shape, np.int32, pooled=True)
        self.comm.all_gather(send, recv, self.stream)
        return recv.download(stream=self.stream).astype(np.int64)

    def exchange_rows(self, rows, send_counts, recv_counts):
        from .device import DeviceArray
        width = rows.shape[1]
        row_bytes = width * rows.dtype.itemsize
        out = DeviceArray((int(np.sum(recv_counts)), width), rows.dtype, pooled=True)
        self.comm.all_to_all_v(rows.ptr, [int(c) * row_bytes for c in send_counts], out.ptr,
                               [int(c) * row_bytes for c in recv_counts], self.stream)
        return out


class GpuMoeBackend:
    """Expert FFN and row movement on the sm_100a kernels for one rank's local experts."""

    def __init__(self, w_gate, w_up, w_down, stream=None) -> None:
        from . import device
        self.wg, self.wu, self.wd = w_gate, w_up, w_down          # DeviceArrays (Ep, H, F) / (Ep, F, H)
        self.stream = stream
        self._code = device.dtype_code(w_gate.dtype)

    def route(self, logits, top_k, normalize):
        from . import _lib
        from .device import DeviceArray, _stream_handle
        logits = np.ascontiguousarray(logits, np.float32)
        T, E = logits.shape
        dl = DeviceArray.from_host(logits, pooled=True)
        da, dw = DeviceArray((T, top_k), np.int32, pooled=True), DeviceArray((T, top_k), np.float32, pooled=True)
        _lib.call("tessera_sm100_moe_route_device", dl.ptr, T, E, top_k, int(normalize), da.ptr, dw.ptr,
                  _stream_handle(self.stream))
        return da.download(), dw.download()

    def gather_rows(self, rows, index):
        from . import _lib
        from .device import DeviceArray, _stream_handle
        index = np.ascontiguousarray(index, np.int32)
        S, H = int(index.shape[0]), rows.shape[1]
        out = DeviceArray((S, H), rows.dtype, pooled=True)
        if S:
            didx = DeviceArray.from_host(index, pooled=True)
            _lib.call("tessera_sm100_moe_dispatch_device", rows.ptr, didx.ptr, out.ptr, rows.shape[0], S,
                      H, self._code, _stream_handle(self.stream))
        return out

    def expert_ffn(self, rows, group_offsets):
        from . import _lib
        from .device import DeviceArray, _stream_handle
        S, H = rows.shape
        Ep, _, F = self.wg.shape
        doff = DeviceArray.from_host(np.ascontiguousarray(group_offsets, np.int32), pooled=True)
        hidden = DeviceArray((max(S, 1), F), rows.dtype, pooled=True)
        out = DeviceArray((S, self.wd.shape[2]), rows.dtype, pooled=True)
        if S:
            sh = _stream_handle(self.stream)
            _lib.call("tessera_sm100_grouped_swiglu_device", rows.ptr, self.wg.ptr, self.wu.ptr, doff.ptr,
                      hidden.ptr, S, H, F, Ep, self._code, self._code, sh)
            _lib.call("tessera_sm100_grouped_gemm_device", hidden.ptr, self.wd.ptr, doff.ptr, out.ptr, S, F,
                      self.wd.shape[2], Ep, self._code, self._code, sh)
        return out

    def combine(self, rows, slot_of, weights, num_tokens):
        from . import _lib
        from .device import DeviceArray, _stream_handle
        k = slot_of.shape[1]
        H = rows.shape[1]
        dso = DeviceArray.from_host(np.ascontiguousarray(slot_of, np.int32), pooled=True)
        dw = DeviceArray.from_host(np.ascontiguousarray(weights, np.float32), pooled=True)
        out = DeviceArray((num_tokens, H), rows.dtype, pooled=True)
        _lib.call("tessera_sm100_moe_combine_device", rows.ptr, dso.ptr, dw.ptr, out.ptr, num_tokens, k, H,
                  self._code, self._code, _stream_handle(self.stream))
        return out


class DeviceExpertParallelMoE:
    """Expert-parallel MoE forward with the exchange done by the kernels themselves: token rows are
    stored straight into the owning rank's receive buffer over NVLink, results are read back from
    the owner's output buffer, and the ranks are ordered by flags the kernels raise in each other's
    memory (``tessera_sm100_ep_{route_publish,dispatch_signal,combine_signal}_device``): no
    collective, no host round trip, five launches per forward (route + sort + publish, plan +
    dispatch, the two grouped GEMMs, combine). Buffers are sized for the worst case (every slot of
    every rank on one rank). Every rank must call ``forward`` the same number of times.

    ``comm`` only supplies ``rank`` and ``world``; ``gather_host`` exchanges CUDA IPC handles once at
    construction (``torch.distributed.all_gather_object`` over gloo, or a list of one for a single
    rank). ``wait_limit_ms`` bounds every device-side wait for a peer."""

    def __init__(self, comm, gather_host, w_gate, w_up, w_down, tokens_per_rank: int, top_k: int,
                 num_experts: int, normalize_weights: bool = True, stream=None, wait_limit_ms: int = 10000) -> None:
        import ctypes
        from . import _lib, device
        from .device import DeviceArray
        self.world, self.rank = comm.world, comm.rank
        if num_experts % self.world:
            raise ValueError("num_experts must be divisible by the number of ranks")
        self.E, self.k, self.Tl = num_experts, top_k, tokens_per_rank
        self.Ep = num_experts // self.world
        self.wg, self.wu, self.wd = w_gate, w_up, w_down
        self.H, self.F = w_gate.shape[1], w_gate.shape[2]
        self.normalize = normalize_weights
        self.stream = stream
        self.dtype = w_gate.dtype
        self._code = device.dtype_code(self.dtype)
        self.capacity = self.Tl * self.k * self.world
        self.wait_limit_ms = int(wait_limit_ms)
        self.epoch = 0
        S = self.Tl * self.k
        i32, f32 = np.int32, np.float32
        self.assignment = DeviceArray((self.Tl, self.k), i32)
        self.weights = DeviceArray((self.Tl, self.k), f32)
        self.token_of_slot, self.expert_of_slot = DeviceArray((S,), i32), DeviceArray((S,), i32)
        self.weight_of_slot = DeviceArray((S,), f32)
        self.group_sizes, self.my_offsets = DeviceArray((self.E,), i32), DeviceArray((self.E + 1,), i32)
        self.slot_of = DeviceArray((S,), i32)
        self.local_offsets, self.dst_base = DeviceArray((self.Ep + 1,), i32), DeviceArray((self.E,), i32)
        self.counters = DeviceArray.zeros((2,), i32)                             # dispatch, combine
        self.ctrl = DeviceArray.zeros((int(_lib.load().tessera_sm100_ep_ctrl_bytes()),), np.uint8)   # peers raise flags here
        self.recv = DeviceArray.zeros((self.capacity, self.H), self.dtype)      # peers store here
        self.hidden = DeviceArray((self.capacity, self.F), self.dtype)
        self.y = DeviceArray.zeros((self.capacity, self.H), self.dtype)         # peers read here
        device.synchronize()
        self._opened = []

        def exchange(buf):
            h = ctypes.create_string_buffer(64)
            _lib.call("tessera_sm100_ipc_get_handle", buf.ptr, h)
            handles = gather_host(h.raw)
            ptrs = []
            for r in range(self.world):
                if r == self.rank:
                    ptrs.append(buf.ptr)
                else:
                    p = ctypes.c_void_p()
                    _lib.call("tessera_sm100_ipc_open_handle", ctypes.c_char_p(handles[r]), ctypes.byref(p))
                    self._opened.append(p.value)
                    ptrs.append(p.value)
            return (ctypes.c_void_p * self.world)(*ptrs)

        self._recv_ptrs = exchange(self.recv)
        self._y_ptrs = exchange(self.y)
        self._ctrl_ptrs = exchange(self.ctrl)

    # The forward in three stages, each on the stream it is given: exchange in, experts, exchange out.
    def _stage_dispatch(self, x_local, logits_local, stream) -> None:
        from . import _lib, device
        sh = device._stream_handle(stream)
        Tl, k, E, H = self.Tl, self.k, self.E, self.H
        self.epoch += 1
        _lib.call("tessera_sm100_ep_route_publish_device", logits_local.ptr, Tl, E, k, int(self.normalize),
                  self.assignment.ptr, self.weights.ptr, self.token_of_slot.ptr, self.expert_of_slot.ptr,
                  self.weight_of_slot.ptr, self.group_sizes.ptr, self.my_offsets.ptr, self.slot_of.ptr,
                  self._ctrl_ptrs, self.world, self.rank, self.epoch, sh)
        _lib.call("tessera_sm100_ep_dispatch_signal_device", x_local.ptr, self.token_of_slot.ptr,
                  self.expert_of_slot.ptr, self.my_offsets.ptr, self._ctrl_ptrs, self._recv_ptrs, self.world,
                  self.rank, E, Tl * k, self.capacity, H, self._code, self.epoch, self.local_offsets.ptr,
                  self.dst_base.ptr, self.counters.ptr, self.wait_limit_ms, sh)

    def _stage_experts(self, stream) -> None:
        from . import _lib, device
        sh = device._stream_handle(stream)
        _lib.call("tessera_sm100_grouped_swiglu_device", self.recv.ptr, self.wg.ptr, self.wu.ptr,
                  self.local_offsets.ptr, self.hidden.ptr, self.capacity, self.H, self.F, self.Ep, self._code,
                  self._code, sh)
        _lib.call("tessera_sm100_grouped_gemm_device", self.hidden.ptr, self.wd.ptr, self.local_offsets.ptr,
                  self.y.ptr, self.capacity, self.F, self.H, self.Ep, self._code, self._code, sh)

    def _stage_combine(self, out, stream) -> None:
        from . import _lib, device
        sh = device._stream_handle(stream)
        _lib.call("tessera_sm100_ep_combine_signal_device", self._y_ptrs, self._ctrl_ptrs, self.assignment.ptr,
                  self.slot_of.ptr, self.weights.ptr, self.my_offsets.ptr, self.dst_base.ptr, out.ptr, self.Tl,
                  self.k, self.world, self.rank, self.E, self.capacity, self.H, self._code, self.epoch,
                  self.counters.ptr + 4, self.wait_limit_ms, sh)

    def forward(self, x_local, logits_local, out=None):
        """``x_local`` (Tl, H) and ``logits_local`` (Tl, E) fp32 DeviceArrays; returns a (Tl, H)
        DeviceArray. Everything is enqueued on one stream; the caller synchronises."""
        from .device import DeviceArray
        if out is None:
            out = DeviceArray((self.Tl, self.H), self.dtype, pooled=True)
        self._stage_dispatch(x_local, logits_local, self.stream)
        self._stage_experts(self.stream)
        self._stage_combine(out, self.stream)
        return out

    def close(self) -> None:
        from . import _lib
        for p in self._opened:
            _lib.call("tessera_sm100_ipc_close_handle", p)
        self._opened = []
