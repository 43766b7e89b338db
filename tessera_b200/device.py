"""Device memory, streams and events on top of the C ABI (no PyTorch, no CUDA Python)."""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import numpy as np

from . import _lib

try:  # bf16 host arrays
    import ml_dtypes

    bfloat16 = np.dtype(ml_dtypes.bfloat16)
except Exception:  # pragma: no cover - ml_dtypes ships with the image
    ml_dtypes = None
    bfloat16 = None


def dtype_code(dt) -> int:
    dt = np.dtype(dt)
    if dt == np.float32:
        return _lib.F32
    if dt == np.float16:
        return _lib.F16
    if bfloat16 is not None and dt == bfloat16:
        return _lib.BF16
    raise TypeError(f"unsupported dtype {dt}; expected float32, float16 or bfloat16")


def code_dtype(code: int) -> np.dtype:
    return {_lib.F32: np.dtype(np.float32), _lib.F16: np.dtype(np.float16), _lib.BF16: bfloat16}[code]


def set_device(index: int) -> None:
    _lib.call("tessera_sm100_set_device", int(index))


def device_count() -> int:
    n = ctypes.c_int(0)
    _lib.call("tessera_sm100_device_count", ctypes.byref(n))
    return n.value


def synchronize() -> None:
    _lib.call("tessera_sm100_device_synchronize")


def consume_device_error() -> tuple[int, int, int]:
    out = (ctypes.c_int * 4)()
    _lib.call("tessera_sm100_consume_device_error", out)
    return out[0], out[1], out[2]


def check_device_error(where: str = "") -> None:
    code, a, b = consume_device_error()
    if code == 6:
        raise _lib.BackendError(where or "kernel", 3,
                                f"a paged-KV page-table entry is outside the page pool (sequence or row {a}, "
                                f"logical page {b}); it was read as zeros")
    if code:
        raise _lib.BackendError(where or "kernel", 3,
                                f"a bounded wait expired on the device (code {code}, block {a}, "
                                f"detail {b})")


def launch_count() -> int:
    return int(_lib.load().tessera_sm100_launch_count())


class Stream:
    def __init__(self):
        h = ctypes.c_void_p()
        _lib.call("tessera_sm100_stream_create", ctypes.byref(h))
        self.handle = h

    def synchronize(self) -> None:
        _lib.call("tessera_sm100_stream_synchronize", self.handle)

    def wait_event(self, event: "Event") -> None:
        """Work enqueued on this stream from now on waits for ``event``."""
        _lib.call("tessera_sm100_stream_wait_event", self.handle, event.handle)

    def close(self) -> None:
        if self.handle:
            _lib.call("tessera_sm100_stream_destroy", self.handle)
            self.handle = None


def _stream_handle(stream) -> ctypes.c_void_p:
    if stream is None:
        return ctypes.c_void_p(None)
    if isinstance(stream, Stream):
        return stream.handle
    return ctypes.c_void_p(int(stream))


class Event:
    def __init__(self):
        h = ctypes.c_void_p()
        _lib.call("tessera_sm100_event_create", ctypes.byref(h))
        self.handle = h

    def record(self, stream=None) -> None:
        _lib.call("tessera_sm100_event_record", self.handle, _stream_handle(stream))

    def synchronize(self) -> None:
        _lib.call("tessera_sm100_event_synchronize", self.handle)

    def elapsed_ms(self, stop: "Event") -> float:
        ms = ctypes.c_float(0)
        _lib.call("tessera_sm100_event_elapsed_ms", self.handle, stop.handle, ctypes.byref(ms))
        return ms.value

    def close(self) -> None:
        if self.handle:
            _lib.call("tessera_sm100_event_destroy", self.handle)
            self.handle = None


class DeviceArray:
    """A dense row-major array in device memory (shape + dtype + pointer)."""

    def __init__(self, shape: Sequence[int], dtype, ptr: Optional[int] = None, owner=None,
                 pooled: bool = False):
        self.shape = tuple(int(s) for s in shape)
        self.dtype = np.dtype(dtype)
        self.nbytes = int(np.prod(self.shape, dtype=np.int64)) * self.dtype.itemsize
        self._owner = owner
        self._pooled = bool(pooled) and ptr is None
        if ptr is None:
            h = ctypes.c_void_p()
            _lib.call("tessera_sm100_pool_alloc" if self._pooled else "tessera_sm100_device_alloc",
                      ctypes.byref(h), max(self.nbytes, 1))
            self.ptr = int(h.value)
            self._owns = True
        else:
            self.ptr = int(ptr)
            self._owns = False

    @property
    def size(self) -> int:
        return int(np.prod(self.shape, dtype=np.int64))

    @property
    def ndim(self) -> int:
        return len(self.shape)

    @classmethod
    def from_host(cls, arr: np.ndarray, stream=None, pooled: bool = False) -> "DeviceArray":
        arr = np.ascontiguousarray(arr)
        out = cls(arr.shape, arr.dtype, pooled=pooled)
        out.upload(arr, stream)
        return out

    @classmethod
    def zeros(cls, shape, dtype, stream=None) -> "DeviceArray":
        out = cls(shape, dtype)
        _lib.call("tessera_sm100_device_memset", out.ptr, 0, out.nbytes, _stream_handle(stream))
        return out

    def upload(self, arr: np.ndarray, stream=None) -> None:
        arr = np.ascontiguousarray(arr)
        if arr.nbytes != self.nbytes:
            raise ValueError(f"upload size mismatch: {arr.nbytes} != {self.nbytes}")
        _lib.call("tessera_sm100_device_upload", self.ptr, arr.ctypes.data, self.nbytes,
                  _stream_handle(stream))
        if stream is None:
            _lib.call("tessera_sm100_stream_synchronize", None)

    def download(self, out: Optional[np.ndarray] = None, stream=None) -> np.ndarray:
        if out is None:
            out = np.empty(self.shape, dtype=self.dtype)
        _lib.call("tessera_sm100_device_download", out.ctypes.data, self.ptr, self.nbytes,
                  _stream_handle(stream))
        _lib.call("tessera_sm100_stream_synchronize", _stream_handle(stream))
        return out

    def view(self, shape, offset_elems: int = 0) -> "DeviceArray":
        """A non-owning view of a contiguous sub-range."""
        return DeviceArray(shape, self.dtype, ptr=self.ptr + offset_elems * self.dtype.itemsize,
                           owner=self)

    def numpy(self) -> np.ndarray:
        return self.download()

    def free(self) -> None:
        if self._owns and self.ptr:
            _lib.call("tessera_sm100_pool_free" if self._pooled else "tessera_sm100_device_free", self.ptr)
            self.ptr = 0
            self._owns = False

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class StridedView:
    """A window into a :class:`DeviceArray` whose last dimension is contiguous: pointer, shape and
    element strides. What a column slice of a fused projection output is (``qkv[..., a:b]``);
    the strided attention entry point reads such windows in place."""

    def __init__(self, base: DeviceArray, ptr: int, shape, strides):
        self.base, self.ptr = base, int(ptr)
        self.shape = tuple(int(x) for x in shape)
        self.strides = tuple(int(x) for x in strides)
        self.dtype = base.dtype
        if self.strides[-1] != 1:
            raise ValueError("StridedView: the last dimension must be contiguous")

    @property
    def ndim(self) -> int:
        return len(self.shape)

    def contiguous(self, stream=None) -> DeviceArray:
        """Copy into a dense array (rows of the last dimension are moved with 2-D copies)."""
        rows = int(np.prod(self.shape[:-1], dtype=np.int64))
        out = DeviceArray(self.shape, self.dtype)
        if len(self.shape) >= 2:
            lead = self.strides[-2]
            for k in range(len(self.shape) - 2):  # leading dims must nest for one 2-D copy
                if self.strides[k] != self.strides[k + 1] * self.shape[k + 1]:
                    raise ValueError("StridedView.contiguous: leading dimensions are not nested")
        else:
            lead = self.shape[-1]
        item = self.dtype.itemsize
        _lib.call("tessera_sm100_device_copy_2d", out.ptr, self.shape[-1] * item, self.ptr, lead * item,
                  self.shape[-1] * item, rows, _stream_handle(stream))
        return out

    def download(self) -> np.ndarray:
        return self.contiguous().download()


def slice_last(x, start: int, stop: int) -> StridedView:
    """``x[..., start:stop]`` of a dense device array as a view (no copy). ``start`` must keep the
    window 16-byte aligned."""
    if isinstance(x, StridedView):
        base, ptr, shape, strides = x.base, x.ptr, x.shape, x.strides
    else:
        base, ptr, shape = x, x.ptr, x.shape
        strides, acc = [], 1
        for n in reversed(shape):
            strides.append(acc)
            acc *= n
        strides = tuple(reversed(strides))
    if not (0 <= start < stop <= shape[-1]):
        raise ValueError(f"slice_last: [{start}:{stop}] outside the last dimension {shape[-1]}")
    item = np.dtype(base.dtype).itemsize
    if (start * item) % 16:
        raise ValueError("slice_last: the window must start on a 16-byte boundary")
    return StridedView(base, ptr + start * item, tuple(shape[:-1]) + (stop - start,), strides)


class PinnedArray:
    """Page-locked host memory exposed as a numpy array (``.array``)."""

    def __init__(self, shape, dtype):
        self.shape = tuple(int(s) for s in shape)
        self.dtype = np.dtype(dtype)
        self.nbytes = int(np.prod(self.shape, dtype=np.int64)) * self.dtype.itemsize
        h = ctypes.c_void_p()
        _lib.call("tessera_sm100_host_alloc", ctypes.byref(h), max(self.nbytes, 1))
        self.ptr = int(h.value)
        buf = (ctypes.c_uint8 * max(self.nbytes, 1)).from_address(self.ptr)
        self.array = np.frombuffer(buf, dtype=np.uint8, count=self.nbytes).view(self.dtype).reshape(
            self.shape)

    def free(self) -> None:
        if self.ptr:
            self.array = None
            _lib.call("tessera_sm100_host_free", self.ptr)
            self.ptr = 0


def flush_l2(stream=None) -> None:
    _lib.call("tessera_sm100_flush_l2", _stream_handle(stream))
