"""The tsr* runtime C ABI on a machine without a GPU: lifecycle, errors, artifacts, the launcher
registry and the profiling callback (after src/runtime's tests and
tests/unit/test_runtime_abi.py in the reference)."""
import ctypes
from ctypes import c_char_p, c_int, c_size_t, c_void_p

import pytest

from tessera_b200 import tsr
from tessera_b200.runtime import TsrStatus


@pytest.fixture()
def rt(lib):
    l = tsr.lib()
    assert l.tsrInit() == 0
    yield l
    l.tsrRegisterGpuLauncher(tsr.LAUNCHER_FN(0), None)
    l.tsrSetProfileEventCallback(tsr.PROFILE_FN(0), None)
    assert l.tsrShutdown() == 0


def test_lifecycle_and_status_strings(lib):
    l = tsr.lib()
    flag = c_int(-1)
    assert l.tsrIsInitialized(ctypes.byref(flag)) == 0 and flag.value == 0
    n = c_int(-1)
    assert l.tsrGetDeviceCount(ctypes.byref(n)) == TsrStatus.INVALID_ARGUMENT   # before tsrInit
    assert b"not initialised" in l.tsrGetLastError()
    assert l.tsrInit() == 0 and l.tsrInit() == 0                                # idempotent
    assert l.tsrIsInitialized(ctypes.byref(flag)) == 0 and flag.value == 1
    assert l.tsrGetDeviceCount(ctypes.byref(n)) == 0 and n.value >= 0
    assert l.tsrShutdown() == 0 and l.tsrShutdown() == 0
    assert l.tsrIsInitialized(ctypes.byref(flag)) == 0 and flag.value == 0
    assert l.tsrStatusString(7) == b"device_error" and l.tsrStatusString(5) == b"unimplemented"
    major, minor, patch = c_int(), c_int(), c_int()
    l.tsrGetVersion(ctypes.byref(major), ctypes.byref(minor), ctypes.byref(patch))
    assert (major.value, minor.value) >= (0, 1)
    l.tsrClearLastError()
    assert l.tsrGetLastError() == b""


def test_artifact_round_trip(rt):
    art = c_void_p()
    opts = tsr.tsrCompileOptions(b"sm_100a", None)
    assert rt.tsrCompileArtifact(b"tessera.sm100.gemm.bf16, tessera.sm100.flash_attn.bf16",
                                 ctypes.byref(opts), ctypes.byref(art)) == 0
    target = c_char_p()
    assert rt.tsrGetArtifactTarget(art, ctypes.byref(target)) == 0 and target.value == b"nvidia_sm100"
    data, size = c_void_p(), c_size_t()
    assert rt.tsrGetArtifactBytes(art, ctypes.byref(data), ctypes.byref(size)) == 0
    payload = ctypes.string_at(data.value, size.value)
    assert payload.startswith(b"TSRART2\n")
    again = c_void_p()
    assert rt.tsrLoadArtifact(payload, len(payload), ctypes.byref(again)) == 0
    ker = c_void_p()
    assert rt.tsrGetKernel(again, b"tessera.sm100.flash_attn.bf16", ctypes.byref(ker)) == 0
    assert rt.tsrGetKernel(again, b"nope", ctypes.byref(c_void_p())) == TsrStatus.NOT_FOUND
    assert rt.tsrLoadArtifact(b"garbage", 7, ctypes.byref(c_void_p())) == TsrStatus.INVALID_ARGUMENT
    assert rt.tsrCompileArtifact(b" , ", None, ctypes.byref(c_void_p())) == TsrStatus.INVALID_ARGUMENT
    rt.tsrDestroyKernel(ker)
    rt.tsrDestroyArtifact(again)
    rt.tsrDestroyArtifact(art)


def test_launcher_registry_and_profile_events(rt):
    seen, events = [], []

    @tsr.LAUNCHER_FN
    def fake(target, name, params, user):
        seen.append((target, name, params.contents.num_buffers, [params.contents.dims[i] for i in range(3)]))
        return 0 if name == b"my.kernel" else int(TsrStatus.NOT_FOUND)

    @tsr.PROFILE_FN
    def sink(kind, name, payload, value, user):
        events.append((kind, name, payload))

    assert rt.tsrRegisterGpuLauncher(fake, None) == 0
    assert rt.tsrSetProfileEventCallback(sink, None) == 0
    art, ker, other = c_void_p(), c_void_p(), c_void_p()
    opts = tsr.tsrCompileOptions(b"custom_target", None)
    assert rt.tsrCompileArtifact(b"my.kernel,unknown.kernel", ctypes.byref(opts), ctypes.byref(art)) == 0
    assert rt.tsrGetKernel(art, b"my.kernel", ctypes.byref(ker)) == 0
    assert rt.tsrGetKernel(art, b"unknown.kernel", ctypes.byref(other)) == 0
    bufs = (c_void_p * 2)(1, 2)
    dims = (ctypes.c_int64 * 3)(4, 5, 6)
    params = tsr.tsrGpuLaunchParams(bufs, 2, dims, 3)
    args = (c_void_p * 1)(ctypes.cast(ctypes.pointer(params), c_void_p))
    assert rt.tsrLaunchKernel(None, ker, args, 1) == 0
    assert seen[-1] == (b"custom_target", b"my.kernel", 2, [4, 5, 6])
    assert rt.tsrLaunchKernel(None, other, args, 1) == TsrStatus.UNIMPLEMENTED   # never a silent success
    assert b"unknown.kernel" in rt.tsrGetLastError()
    assert rt.tsrLaunchKernel(None, ker, args, 0) == TsrStatus.INVALID_ARGUMENT
    names = [e[1] for e in events]
    assert b"tsrLaunchKernel" in names and b"my.kernel" in names
    assert any(b'"status":"unimplemented"' in e[2] for e in events)
    n = len(events)
    assert rt.tsrEnableProfiling(0) == 0
    rt.tsrLaunchKernel(None, ker, args, 1)
    assert len(events) == n
    rt.tsrEnableProfiling(1)
    # with the built-in launcher restored an unknown target reports UNIMPLEMENTED as well
    assert rt.tsrRegisterGpuLauncher(tsr.LAUNCHER_FN(0), None) == 0
    assert rt.tsrLaunchKernel(None, ker, args, 1) == TsrStatus.UNIMPLEMENTED
    for h in (ker, other):
        rt.tsrDestroyKernel(h)
    rt.tsrDestroyArtifact(art)


def test_null_arguments_are_rejected(rt):
    assert rt.tsrGetDevice(99, ctypes.byref(c_void_p())) == TsrStatus.NOT_FOUND
    assert rt.tsrMalloc(None, 16, ctypes.byref(c_void_p())) == TsrStatus.INVALID_ARGUMENT
    assert rt.tsrMemset(None, 0, 4) == TsrStatus.INVALID_ARGUMENT
    assert rt.tsrRecordEvent(None, None) == TsrStatus.INVALID_ARGUMENT
    assert rt.tsrFree(None) == 0 and rt.tsrDestroyStream(None) == 0
