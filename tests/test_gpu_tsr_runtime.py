"""tsr* runtime on the GPU: buffers, streams, events, shutdown refusal with live handles, and a
GEMM launched by kernel name through the built-in sm_100 launcher."""
import ctypes
from ctypes import c_float, c_void_p

import numpy as np
import pytest

from oracle import tessera_oracle as orc
from tessera_b200 import tsr
from tessera_b200.device import bfloat16
from tessera_b200.runtime import TsrStatus

pytestmark = pytest.mark.gpu


def test_runtime_objects_and_named_gemm_launch():
    rt = tsr.TesseraRuntime()
    l = tsr.lib()
    assert rt.device_count() >= 1
    dev = rt.device(0)
    props = rt.device_props(dev)
    assert props["kind"] == 1 and "sm_100" in props["name"] and props["concurrent_tiles_hint"] >= 100
    rng = np.random.default_rng(0)
    M, N, K = 200, 264, 136
    A = (rng.standard_normal((M, K), dtype=np.float32) / 11).astype(bfloat16)
    B = rng.standard_normal((K, N), dtype=np.float32).astype(bfloat16)
    D = np.zeros((M, N), np.float32)
    bA, bB, bD = rt.malloc(dev, A.nbytes), rt.malloc(dev, B.nbytes), rt.malloc(dev, D.nbytes)
    assert l.tsrShutdown() == TsrStatus.INVALID_ARGUMENT        # live buffers
    assert b"buffer" in l.tsrGetLastError()
    rt.upload(bA, A)
    rt.upload(bB, B)
    stream, e0, e1 = c_void_p(), c_void_p(), c_void_p()
    assert l.tsrCreateStream(dev, ctypes.byref(stream)) == 0
    assert l.tsrCreateEvent(dev, ctypes.byref(e0)) == 0 and l.tsrCreateEvent(dev, ctypes.byref(e1)) == 0
    assert l.tsrRecordEvent(e0, None) == 0
    rt.launch("blackwell", "tessera.sm100.gemm.bf16", [bA, bB, bD], [M, N, K])
    assert l.tsrRecordEvent(e1, None) == 0 and l.tsrEventSynchronize(e1) == 0
    ms = c_float(-1)
    assert l.tsrEventElapsedMs(e0, e1, ctypes.byref(ms)) == 0 and ms.value >= 0
    rt.synchronize()
    rt.download(D, bD)
    assert orc.max_rel_err(D, orc.gemm(A, B)) < 1e-4
    with pytest.raises(tsr.TsrError) as info:
        rt.launch("nvidia_sm100", "tessera.sm100.not_a_kernel", [bA], [1])
    assert info.value.status == TsrStatus.UNIMPLEMENTED
    # map / unmap round trip
    hp, nb = c_void_p(), ctypes.c_size_t()
    assert l.tsrMap(bD, ctypes.byref(hp), ctypes.byref(nb)) == 0 and nb.value == D.nbytes
    view = np.ctypeslib.as_array(ctypes.cast(hp, ctypes.POINTER(c_float)), shape=(M * N,))
    np.testing.assert_array_equal(view.reshape(M, N), D)
    view[:] = 1.0
    assert l.tsrUnmap(bD) == 0
    rt.download(D, bD)
    assert (D == 1.0).all()
    names = {e["name"] for e in rt.telemetry}
    assert {"tsrMalloc", "tsrLaunchKernel", "tessera.sm100.gemm.bf16"} <= names
    for h in (e0, e1):
        l.tsrDestroyEvent(h)
    l.tsrDestroyStream(stream)
    for b in (bA, bB, bD):
        rt.free(b)
    rt.close()


def test_named_launch_runs_on_the_stream_it_is_given():
    """tsrLaunchKernel(s, ...) enqueues on `s`: synchronising `s` alone makes the result readable,
    and events recorded on `s` bracket the kernel (a GEMM large enough that its device time cannot
    be mistaken for an empty interval)."""
    rt = tsr.TesseraRuntime()
    l = tsr.lib()
    dev = rt.device(0)
    rng = np.random.default_rng(1)
    M = N = K = 4096
    A = (rng.standard_normal((M, K), dtype=np.float32) / 64).astype(bfloat16)
    B = rng.standard_normal((K, N), dtype=np.float32).astype(bfloat16)
    bA, bB, bD = rt.malloc(dev, A.nbytes), rt.malloc(dev, B.nbytes), rt.malloc(dev, M * N * 4)
    rt.upload(bA, A)
    rt.upload(bB, B)
    stream, e0, e1 = c_void_p(), c_void_p(), c_void_p()
    assert l.tsrCreateStream(dev, ctypes.byref(stream)) == 0
    assert l.tsrCreateEvent(dev, ctypes.byref(e0)) == 0 and l.tsrCreateEvent(dev, ctypes.byref(e1)) == 0
    rt.launch("nvidia_sm100", "tessera.sm100.gemm.bf16", [bA, bB, bD], [M, N, K], stream=stream)   # warm-up
    assert l.tsrStreamSynchronize(stream) == 0
    assert l.tsrRecordEvent(e0, stream) == 0
    rt.launch("nvidia_sm100", "tessera.sm100.gemm.bf16", [bA, bB, bD], [M, N, K], stream=stream)
    assert l.tsrRecordEvent(e1, stream) == 0
    assert l.tsrStreamSynchronize(stream) == 0          # this stream only: no device-wide synchronise
    ms = c_float(-1)
    assert l.tsrEventElapsedMs(e0, e1, ctypes.byref(ms)) == 0
    assert ms.value > 0.05, f"events on the launch stream bracket {ms.value} ms: the kernel ran elsewhere"
    # only that stream was synchronised; the copy below orders with nothing else
    out = np.empty((M, N), np.float32)
    rt.download(out, bD)
    rows = [0, 1234, M - 1]
    ref = A[rows].astype(np.float32) @ B.astype(np.float32)
    assert orc.max_rel_err(out[rows], ref) < 1e-4
    for h in (e0, e1):
        l.tsrDestroyEvent(h)
    l.tsrDestroyStream(stream)
    for b in (bA, bB, bD):
        rt.free(b)
    rt.close()
