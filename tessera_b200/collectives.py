"""Collectives for the B200 backend.

Two layers:

* ``Communicator`` — one NCCL communicator of THIS process (one process per GPU). Operates on
  ``DeviceArray``s, asynchronously on a stream. Created from a 128-byte unique id that rank 0
  produces and the launcher distributes (``torch.distributed`` store, a file, MPI ...).
* ``CollectiveAdapter`` / ``adapter(backend="nccl", world_size=N)`` — the reference's
  one-process/multi-device surface (python/tessera/collectives.py:657-817): per-rank host arrays
  in, per-rank host arrays out. Where the reference stages fp32 through ``cudaMalloc`` +
  ``cudaMemcpy`` per call (:415-474) this keeps the storage dtype and issues the grouped NCCL
  calls through the C ABI. ``backend="single_process"`` with world_size 1 passes values through.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Any, List, Optional, Sequence

import numpy as np

from . import _lib, device
from .device import DeviceArray

_OPS = {"sum": 0, "max": 1, "min": 2, "prod": 3}


def _coll_dtype(dt) -> int:
    dt = np.dtype(dt)
    if dt == np.uint8 or dt == np.int8:
        return _lib.U8
    if dt == np.int32:
        return _lib.I32
    return device.dtype_code(dt)


def nccl_version() -> int:
    v = ctypes.c_int(0)
    _lib.call("tessera_sm100_nccl_version", ctypes.byref(v))
    return v.value


class Communicator:
    """NCCL communicator of the calling process; the current CUDA device is this rank's GPU."""

    def __init__(self, handle: int, rank: int, world: int) -> None:
        self.handle, self.rank, self.world = handle, rank, world

    @staticmethod
    def unique_id() -> bytes:
        buf = ctypes.create_string_buffer(128)
        _lib.call("tessera_sm100_comm_unique_id", buf)
        return buf.raw

    @classmethod
    def from_unique_id(cls, uid: bytes, world: int, rank: int) -> "Communicator":
        if len(uid) != 128:
            raise ValueError("NCCL unique id must be 128 bytes")
        h = ctypes.c_void_p()
        _lib.call("tessera_sm100_comm_init_rank", ctypes.c_char_p(uid), int(world), int(rank),
                  ctypes.byref(h))
        return cls(h.value, rank, world)

    def all_gather(self, send: DeviceArray, recv: DeviceArray, stream=None) -> None:
        if recv.nbytes != send.nbytes * self.world:
            raise ValueError("all_gather: recv must hold world * send elements")
        _lib.call("tessera_sm100_all_gather", self.handle, send.ptr, recv.ptr, send.size,
                  _coll_dtype(send.dtype), device._stream_handle(stream))

    def all_reduce(self, send: DeviceArray, recv: DeviceArray, op: str = "sum", stream=None) -> None:
        _lib.call("tessera_sm100_all_reduce", self.handle, send.ptr, recv.ptr, send.size,
                  _coll_dtype(send.dtype), _OPS[op], device._stream_handle(stream))

    def reduce_scatter(self, send: DeviceArray, recv: DeviceArray, op: str = "sum", stream=None) -> None:
        _lib.call("tessera_sm100_reduce_scatter", self.handle, send.ptr, recv.ptr, recv.size,
                  _coll_dtype(send.dtype), _OPS[op], device._stream_handle(stream))

    def all_to_all_v(self, send_ptr: int, send_bytes: Sequence[int], recv_ptr: int,
                     recv_bytes: Sequence[int], stream=None) -> None:
        """Ragged exchange; blocks are laid out back to back in rank order on both sides."""
        arr = ctypes.c_size_t * self.world
        sb, rb = arr(*map(int, send_bytes)), arr(*map(int, recv_bytes))
        so = arr(*np.concatenate(([0], np.cumsum(send_bytes)[:-1])).astype(np.int64).tolist())
        ro = arr(*np.concatenate(([0], np.cumsum(recv_bytes)[:-1])).astype(np.int64).tolist())
        _lib.call("tessera_sm100_all_to_all_v", self.handle, send_ptr, sb, so, recv_ptr, rb, ro,
                  device._stream_handle(stream))

    def async_error(self) -> Optional[str]:
        rc = _lib.load().tessera_sm100_comm_async_error(self.handle)
        return None if rc == 0 else _lib.last_error()

    def abort(self) -> None:
        if self.handle:
            _lib.call("tessera_sm100_comm_abort", self.handle)
            self.handle = None

    def close(self) -> None:
        if self.handle:
            _lib.call("tessera_sm100_comm_destroy", self.handle)
            self.handle = None


# ------------------------------------------------------------------ reference-shaped adapter
@dataclass(frozen=True)
class CollectiveTopology:
    backend: str
    world_size: int
    device_ordinals: tuple
    rank_order: tuple
    cta_policy: str = "default"

    def __post_init__(self) -> None:
        if self.backend not in {"nccl"}:
            raise ValueError("native collective topology requires nccl")
        if self.world_size < 2:
            raise ValueError("native multi-rank topology requires world_size >= 2")
        if len(self.device_ordinals) != self.world_size or len(set(self.device_ordinals)) != self.world_size:
            raise ValueError("collective topology requires one unique device ordinal per rank")
        if self.rank_order != tuple(range(self.world_size)):
            raise ValueError("collective rank order must be the canonical contiguous order")
        if any(d < 0 for d in self.device_ordinals):
            raise ValueError("collective device ordinals must be nonnegative")


def collective_topology(*, backend: str, world_size: int, device_ordinals=None,
                        cta_policy: str = "default") -> CollectiveTopology:
    devs = tuple(range(world_size)) if device_ordinals is None else tuple(device_ordinals)
    return CollectiveTopology(backend, int(world_size), devs, tuple(range(int(world_size))), cta_policy)


@dataclass(frozen=True)
class CollectiveBackendStatus:
    backend: str
    status: str
    reason: str = ""
    world_size: int = 1

    @property
    def available(self) -> bool:
        return self.status in {"single_process", "hardware_runtime"}

    def to_dict(self) -> dict:
        return {"backend": self.backend, "status": self.status, "reason": self.reason,
                "world_size": self.world_size, "available": self.available}


def _per_rank(values, world: int) -> List[np.ndarray]:
    if isinstance(values, (list, tuple)):
        if len(values) != world:
            raise ValueError(f"expected {world} per-rank values, got {len(values)}")
        return [np.ascontiguousarray(v) for v in values]
    return [np.ascontiguousarray(values) for _ in range(world)]


class CollectiveAdapter:
    def __init__(self, *, backend: str = "single_process", world_size: int = 1, mesh_axes=None,
                 device_ordinals=None, cta_policy: str = "default") -> None:
        self.backend = backend
        self.world_size = int(world_size)
        if self.world_size < 1:
            raise ValueError("collective adapter world_size must be positive")
        self.mesh_axes = dict(mesh_axes or {"dp": self.world_size})
        self._topology = (collective_topology(backend=backend, world_size=self.world_size,
                                              device_ordinals=device_ordinals, cta_policy=cta_policy)
                          if backend == "nccl" and self.world_size > 1 else None)
        self._comms: Optional[list] = None

    def status(self) -> CollectiveBackendStatus:
        if self.world_size == 1 and self.backend in {"single_process", "nccl", "mock"}:
            return CollectiveBackendStatus(self.backend, "single_process", world_size=1)
        if self.backend == "nccl":
            try:
                n = device.device_count()
                nccl_version()
            except Exception as exc:
                return CollectiveBackendStatus(self.backend, "backend_unavailable", reason=str(exc),
                                               world_size=self.world_size)
            need = max(self._topology.device_ordinals) + 1
            if n < need:
                return CollectiveBackendStatus(
                    self.backend, "backend_unavailable", world_size=self.world_size,
                    reason=f"topology requires CUDA device ordinal {need - 1}, but only {n} device(s) are visible")
            return CollectiveBackendStatus(self.backend, "hardware_runtime", world_size=self.world_size)
        return CollectiveBackendStatus(self.backend, "backend_unavailable", world_size=self.world_size,
                                       reason=f"{self.backend!r} collectives are not part of this backend "
                                              f"(NCCL only)")

    # -- native plumbing
    def _ensure(self) -> list:
        st = self.status()
        if not st.available:
            raise RuntimeError(st.reason)
        if self._comms is None:
            devs = (ctypes.c_int * self.world_size)(*self._topology.device_ordinals)
            handles = (ctypes.c_void_p * self.world_size)()
            _lib.call("tessera_sm100_comm_init_all", self.world_size, devs, handles)
            self._comms = [Communicator(handles[i], i, self.world_size) for i in range(self.world_size)]
        return self._comms

    def _run(self, kind: str, values, op: str = "sum"):
        arrs = _per_rank(values, self.world_size)
        if self.world_size == 1:
            return [arrs[0]]
        comms = self._ensure()
        devs = self._topology.device_ordinals
        W = self.world_size
        first = arrs[0]
        if any(a.shape != first.shape or a.dtype != first.dtype for a in arrs):
            raise ValueError(f"{kind}: rank inputs must have identical shapes and dtypes")
        sends, recvs, outs = [], [], []
        for r in range(W):
            device.set_device(devs[r])
            sends.append(DeviceArray.from_host(arrs[r]))
            if kind == "all_gather":
                shape = (W * first.shape[0],) + first.shape[1:]
            elif kind == "reduce_scatter":
                if first.shape[0] % W:
                    raise ValueError("reduce_scatter: leading dimension must divide by world_size")
                shape = (first.shape[0] // W,) + first.shape[1:]
            else:
                shape = first.shape
            recvs.append(DeviceArray(shape, first.dtype))
        if kind == "all_to_all" and first.shape[0] % W:
            raise ValueError("all_to_all: leading dimension must divide by world_size")
        _lib.call("tessera_sm100_group_start")
        try:
            for r in range(W):
                device.set_device(devs[r])
                if kind == "all_gather":
                    comms[r].all_gather(sends[r], recvs[r])
                elif kind == "all_reduce":
                    comms[r].all_reduce(sends[r], recvs[r], op)
                elif kind == "reduce_scatter":
                    comms[r].reduce_scatter(sends[r], recvs[r], op)
                elif kind == "all_to_all":
                    per = sends[r].nbytes // W
                    comms[r].all_to_all_v(sends[r].ptr, [per] * W, recvs[r].ptr, [per] * W)
        finally:
            _lib.call("tessera_sm100_group_end")
        for r in range(W):
            device.set_device(devs[r])
            outs.append(recvs[r].download())
        device.set_device(devs[0])
        return outs

    def all_reduce(self, values, *, op: str = "sum"):
        return self._run("all_reduce", values, op)

    def reduce_scatter(self, values, *, axis: int = 0, op: str = "sum"):
        if axis != 0:
            raise ValueError("NCCL reduce_scatter v1 requires axis=0")
        return self._run("reduce_scatter", values, op)

    def all_gather(self, values, *, axis: int = 0):
        if axis == 0 or self.world_size == 1:
            return self._run("all_gather", values)
        # gather along another axis = gather along 0 of the moved array, then move back
        arrs = [np.moveaxis(a, axis, 0) for a in _per_rank(values, self.world_size)]
        return [np.ascontiguousarray(np.moveaxis(o, 0, axis)) for o in self._run("all_gather", arrs)]

    def collective_permute(self, values, *, pairs):
        """Rank ``source`` sends its whole value to rank ``target`` for every ``(source, target)``
        pair; ranks that are nobody's target get zeros (python/tessera/collectives.py:746-767).
        On NCCL this is one ragged all-to-all in which each rank sends to at most one peer."""
        pairs = tuple((int(a), int(b)) for a, b in pairs)
        sources = tuple(a for a, _ in pairs)
        targets = tuple(b for _, b in pairs)
        if not pairs:
            raise ValueError("collective_permute requires a non-empty peer map")
        if len(set(sources)) != len(sources) or len(set(targets)) != len(targets):
            raise ValueError("collective_permute sources and targets must be unique")
        if any(p < 0 or p >= self.world_size for p in (*sources, *targets)):
            raise ValueError("collective_permute peer is outside the communicator")
        arrs = _per_rank(values, self.world_size)
        if any(a.shape != arrs[0].shape for a in arrs):
            raise ValueError("collective_permute rank inputs must have identical shapes")
        W = self.world_size
        if W == 1:
            return [np.array(arrs[0], copy=True)]
        comms = self._ensure()
        devs = self._topology.device_ordinals
        send_to = dict(pairs)
        recv_from = {t: s for s, t in pairs}
        nbytes = arrs[0].nbytes
        sends, recvs = [], []
        for r in range(W):
            device.set_device(devs[r])
            sends.append(DeviceArray.from_host(arrs[r]))
            recvs.append(DeviceArray.zeros(arrs[0].shape, arrs[0].dtype))
        device.synchronize()
        _lib.call("tessera_sm100_group_start")
        try:
            for r in range(W):
                device.set_device(devs[r])
                sb = [nbytes if send_to.get(r) == p else 0 for p in range(W)]
                rb = [nbytes if recv_from.get(r) == p else 0 for p in range(W)]
                comms[r].all_to_all_v(sends[r].ptr, sb, recvs[r].ptr, rb)
        finally:
            _lib.call("tessera_sm100_group_end")
        outs = []
        for r in range(W):
            device.set_device(devs[r])
            outs.append(recvs[r].download())
        device.set_device(devs[0])
        return outs

    def all_to_all(self, values, *, scatter_axis: int = 0, gather_axis: int = 0):
        if scatter_axis != 0 or gather_axis != 0:
            raise ValueError("NCCL all_to_all v1 requires scatter_axis=gather_axis=0")
        return self._run("all_to_all", values)

    def close(self) -> None:
        if self._comms:
            for c in self._comms:
                c.close()
            self._comms = None


def adapter(*, backend: str = "single_process", world_size: int = 1, **kw: Any) -> CollectiveAdapter:
    return CollectiveAdapter(backend=backend, world_size=world_size, **kw)


# ------------------------------------------------------------------ chunk-submission hooks
def qos_limit_set(tokens: int) -> None:
    """At most ``tokens`` chunks in flight (``tessera_qos_limit_set``)."""
    _lib.load().tessera_qos_limit_set(int(tokens))


def submit_chunk_async(ptr: int, nbytes: int, device_index: int = 0, stream_id: int = 0) -> None:
    """Submit one transfer chunk through the token limiter and the trace (``tessera_submit_chunk_async``)."""
    _lib.load().tessera_submit_chunk_async(ctypes.c_void_p(int(ptr)), ctypes.c_uint64(int(nbytes)),
                                           int(device_index), int(stream_id))


def bind_chunk_stream(device_index: int, stream_id: int, stream) -> None:
    """Chunks submitted for ``(device_index, stream_id)`` complete when ``stream`` reaches them."""
    _lib.call("tessera_sm100_comm_bind_stream", int(device_index), int(stream_id),
              device._stream_handle(stream) if stream is not None else None)


def qos_state() -> dict:
    lim, inf, peak, ev = ctypes.c_int(), ctypes.c_int(), ctypes.c_int(), ctypes.c_longlong()
    rc = _lib.load().tessera_sm100_qos_state(ctypes.byref(lim), ctypes.byref(inf), ctypes.byref(peak),
                                             ctypes.byref(ev))
    return {"exists": rc == 0, "limit": lim.value, "inflight": inf.value, "peak_inflight": peak.value,
            "trace_events": ev.value}


def trace_write(path: str) -> None:
    rc = _lib.load().tessera_trace_write_status(str(path).encode())
    if rc == 3:
        raise OSError(f"could not write the collective trace to {path}")


def shutdown_runtime() -> None:
    _lib.load().tessera_shutdown_runtime()
