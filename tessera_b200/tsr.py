"""ctypes view of the ``tsr*`` runtime C ABI (include/tessera_runtime.h) and a small
``TesseraRuntime`` convenience wrapper in the manner of the reference's
(python/tessera/runtime.py:332-1077): status codes become ``TsrError`` exceptions and a bounded
deque keeps the profile events the runtime emits."""
from __future__ import annotations

import collections
import ctypes
import json
from ctypes import (CFUNCTYPE, POINTER, Structure, c_char, c_char_p, c_double, c_float, c_int, c_int64,
                    c_size_t, c_uint32, c_uint64, c_void_p)

from . import _lib
from .runtime import TsrStatus


class tsrDeviceProps(Structure):
    _fields_ = [("kind", c_int), ("name", c_char * 128), ("logical_tile_threads_max", c_uint32),
                ("concurrent_tiles_hint", c_uint32)]


class tsrCompileOptions(Structure):
    _fields_ = [("target", c_char_p), ("options_json", c_char_p)]


class tsrGpuLaunchParams(Structure):
    _fields_ = [("buffers", POINTER(c_void_p)), ("num_buffers", c_size_t), ("dims", POINTER(c_int64)),
                ("num_dims", c_size_t)]


PROFILE_FN = CFUNCTYPE(None, c_int, c_char_p, c_char_p, c_double, c_void_p)
LAUNCHER_FN = CFUNCTYPE(c_int, c_char_p, c_char_p, POINTER(tsrGpuLaunchParams), c_void_p)

_SIGS = {
    "tsrStatusString": (c_char_p, [c_int]), "tsrGetLastError": (c_char_p, []),
    "tsrClearLastError": (None, []), "tsrGetVersion": (None, [POINTER(c_int)] * 3),
    "tsrInit": (c_int, []), "tsrShutdown": (c_int, []), "tsrIsInitialized": (c_int, [POINTER(c_int)]),
    "tsrGetDeviceCount": (c_int, [POINTER(c_int)]), "tsrGetDevice": (c_int, [c_int, POINTER(c_void_p)]),
    "tsrGetDeviceProps": (c_int, [c_void_p, POINTER(tsrDeviceProps)]),
    "tsrCreateStream": (c_int, [c_void_p, POINTER(c_void_p)]), "tsrDestroyStream": (c_int, [c_void_p]),
    "tsrStreamSynchronize": (c_int, [c_void_p]),
    "tsrCreateEvent": (c_int, [c_void_p, POINTER(c_void_p)]), "tsrRecordEvent": (c_int, [c_void_p, c_void_p]),
    "tsrWaitEvent": (c_int, [c_void_p, c_void_p]), "tsrEventSynchronize": (c_int, [c_void_p]),
    "tsrDestroyEvent": (c_int, [c_void_p]), "tsrEventGetTimestamp": (c_int, [c_void_p, POINTER(c_uint64)]),
    "tsrEventElapsedMs": (c_int, [c_void_p, c_void_p, POINTER(c_float)]),
    "tsrSetProfileEventCallback": (c_int, [PROFILE_FN, c_void_p]), "tsrEnableProfiling": (c_int, [c_int]),
    "tsrMalloc": (c_int, [c_void_p, c_size_t, POINTER(c_void_p)]), "tsrFree": (c_int, [c_void_p]),
    "tsrMemset": (c_int, [c_void_p, c_int, c_size_t]),
    "tsrMemcpy": (c_int, [c_void_p, c_void_p, c_size_t, c_int]),
    "tsrMemcpyFromHost": (c_int, [c_void_p, c_void_p, c_size_t]),
    "tsrMemcpyToHost": (c_int, [c_void_p, c_void_p, c_size_t]),
    "tsrMap": (c_int, [c_void_p, POINTER(c_void_p), POINTER(c_size_t)]), "tsrUnmap": (c_int, [c_void_p]),
    "tsrBufferGetPointer": (c_int, [c_void_p, POINTER(c_void_p), POINTER(c_size_t)]),
    "tsrCompileArtifact": (c_int, [c_char_p, POINTER(tsrCompileOptions), POINTER(c_void_p)]),
    "tsrLoadArtifact": (c_int, [c_void_p, c_size_t, POINTER(c_void_p)]),
    "tsrDestroyArtifact": (c_int, [c_void_p]),
    "tsrGetArtifactBytes": (c_int, [c_void_p, POINTER(c_void_p), POINTER(c_size_t)]),
    "tsrGetArtifactTarget": (c_int, [c_void_p, POINTER(c_char_p)]),
    "tsrGetKernel": (c_int, [c_void_p, c_char_p, POINTER(c_void_p)]), "tsrDestroyKernel": (c_int, [c_void_p]),
    "tsrLaunchKernel": (c_int, [c_void_p, c_void_p, POINTER(c_void_p), c_size_t]),
    "tsrRegisterGpuLauncher": (c_int, [LAUNCHER_FN, c_void_p]),
}

_bound = False


def lib() -> ctypes.CDLL:
    global _bound
    l = _lib.load()
    if not _bound:
        for name, (res, args) in _SIGS.items():
            fn = getattr(l, name)
            fn.restype, fn.argtypes = res, args
        _bound = True
    return l


class TsrError(RuntimeError):
    def __init__(self, fn: str, status: int, detail: str):
        self.status = TsrStatus(status)
        super().__init__(f"{fn}: {self.status.name}: {detail}")


def check(fn: str, status: int) -> None:
    if status != 0:
        raise TsrError(fn, status, (lib().tsrGetLastError() or b"").decode())


class TesseraRuntime:
    """Thin object wrapper: ``with TesseraRuntime() as rt: dev = rt.device(0); buf = rt.malloc(dev, n)``."""

    def __init__(self, telemetry_capacity: int = 256) -> None:
        self._l = lib()
        self.telemetry = collections.deque(maxlen=telemetry_capacity)
        self._cb = PROFILE_FN(self._on_event)
        check("tsrInit", self._l.tsrInit())
        check("tsrSetProfileEventCallback", self._l.tsrSetProfileEventCallback(self._cb, None))

    def _on_event(self, kind, name, payload, value, _user):
        try:
            data = json.loads(payload.decode()) if payload else {}
        except Exception:
            data = {}
        self.telemetry.append({"kind": int(kind), "name": name.decode() if name else "", "value": value,
                               **data})

    def device_count(self) -> int:
        n = c_int(0)
        check("tsrGetDeviceCount", self._l.tsrGetDeviceCount(ctypes.byref(n)))
        return n.value

    def device(self, index: int = 0) -> c_void_p:
        h = c_void_p()
        check("tsrGetDevice", self._l.tsrGetDevice(index, ctypes.byref(h)))
        return h

    def device_props(self, dev) -> dict:
        p = tsrDeviceProps()
        check("tsrGetDeviceProps", self._l.tsrGetDeviceProps(dev, ctypes.byref(p)))
        return {"kind": p.kind, "name": p.name.decode(), "logical_tile_threads_max": p.logical_tile_threads_max,
                "concurrent_tiles_hint": p.concurrent_tiles_hint}

    def malloc(self, dev, nbytes: int) -> c_void_p:
        h = c_void_p()
        check("tsrMalloc", self._l.tsrMalloc(dev, nbytes, ctypes.byref(h)))
        return h

    def free(self, buf) -> None:
        check("tsrFree", self._l.tsrFree(buf))

    def upload(self, buf, arr) -> None:
        check("tsrMemcpyFromHost", self._l.tsrMemcpyFromHost(buf, arr.ctypes.data, arr.nbytes))

    def download(self, arr, buf) -> None:
        check("tsrMemcpyToHost", self._l.tsrMemcpyToHost(arr.ctypes.data, buf, arr.nbytes))

    def pointer(self, buf) -> int:
        p, n = c_void_p(), c_size_t()
        check("tsrBufferGetPointer", self._l.tsrBufferGetPointer(buf, ctypes.byref(p), ctypes.byref(n)))
        return p.value

    def launch(self, target: str, kernel_name: str, buffers, dims, stream=None) -> None:
        art, ker = c_void_p(), c_void_p()
        opts = tsrCompileOptions(target.encode(), None)
        check("tsrCompileArtifact", self._l.tsrCompileArtifact(kernel_name.encode(), ctypes.byref(opts),
                                                               ctypes.byref(art)))
        try:
            check("tsrGetKernel", self._l.tsrGetKernel(art, kernel_name.encode(), ctypes.byref(ker)))
            bufs = (c_void_p * len(buffers))(*[self.pointer(b) for b in buffers])
            dd = (c_int64 * len(dims))(*dims)
            params = tsrGpuLaunchParams(bufs, len(buffers), dd, len(dims))
            args = (c_void_p * 1)(ctypes.cast(ctypes.pointer(params), c_void_p))
            check("tsrLaunchKernel", self._l.tsrLaunchKernel(stream, ker, args, 1))
        finally:
            self._l.tsrDestroyKernel(ker)
            self._l.tsrDestroyArtifact(art)

    def synchronize(self) -> None:
        check("tsrStreamSynchronize", self._l.tsrStreamSynchronize(None))

    def close(self) -> None:
        self._l.tsrSetProfileEventCallback(PROFILE_FN(0), None)
        check("tsrShutdown", self._l.tsrShutdown())

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False
