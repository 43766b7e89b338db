"""Times the reference's own GPU GEMM (`tessera_nvidia_mma_gemm_bf16_device`, the mma.sync kernel of
src/compiler/codegen/tessera_gpu_backend_NVIDIA/runtime/cuda/tessera_nvidia_gemm.cpp:42-60, which the
library NVRTC-compiles for the live device) on this GPU, with the reference's own event helpers
(`tessera_nvidia_event_*`, tessera_nvidia_gemm.cpp:668-697). The library is built by
build_ref_gemm.sh into baseline/_ref/. A context number beside bench.py's, never a target: the kernel
is one warp per 16 x 8 output tile with scalar global loads.

    python baseline/time_ref_gemm.py [size ...]        (default: 1024 8192)
"""
import ctypes
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from tessera_b200 import device  # noqa: E402
from tessera_b200.device import DeviceArray, bfloat16  # noqa: E402


def main():
    sizes = [int(a) for a in sys.argv[1:]] or [1024, 8192]
    path = os.path.join(ROOT, "baseline", "_ref", "libtessera_nvidia_gemm.so")
    if not os.path.exists(path):
        print(json.dumps({"impl": "reference-gpu", "unavailable": "baseline/_ref/libtessera_nvidia_gemm.so not built"}))
        return
    device.set_device(0)
    lib = ctypes.CDLL(path)
    gemm = lib.tessera_nvidia_mma_gemm_bf16_device
    gemm.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int] * 3 + [ctypes.c_void_p]
    gemm.restype = ctypes.c_int
    for name in ("create", "record", "synchronize", "elapsed_ms", "destroy"):
        getattr(lib, "tessera_nvidia_event_" + name).restype = ctypes.c_int
    lib.tessera_nvidia_event_create.argtypes = [ctypes.POINTER(ctypes.c_void_p)]
    lib.tessera_nvidia_event_record.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    lib.tessera_nvidia_event_synchronize.argtypes = [ctypes.c_void_p]
    lib.tessera_nvidia_event_elapsed_ms.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(ctypes.c_float)]
    lib.tessera_nvidia_event_destroy.argtypes = [ctypes.c_void_p]
    for n in sizes:
        rng = np.random.default_rng(n)
        a = (rng.standard_normal((n, n), dtype=np.float32) / np.sqrt(n)).astype(bfloat16)
        b = (rng.standard_normal((n, n), dtype=np.float32) / np.sqrt(n)).astype(bfloat16)
        da, db = DeviceArray.from_host(a), DeviceArray.from_host(b)
        dd = DeviceArray.zeros((n, n), np.float32)
        rc = gemm(da.ptr, db.ptr, dd.ptr, n, n, n, None)      # first call compiles the kernel
        device.synchronize()
        if rc != 0:
            print(json.dumps({"impl": "reference-gpu", "size": n, "unavailable": f"the reference's launch returned {rc}"}))
            return
        e0, e1 = ctypes.c_void_p(), ctypes.c_void_p()
        assert lib.tessera_nvidia_event_create(ctypes.byref(e0)) == 0
        assert lib.tessera_nvidia_event_create(ctypes.byref(e1)) == 0
        times = []
        for _ in range(2):
            lib.tessera_nvidia_event_record(e0, None)
            rc = gemm(da.ptr, db.ptr, dd.ptr, n, n, n, None)
            lib.tessera_nvidia_event_record(e1, None)
            lib.tessera_nvidia_event_synchronize(e1)
            ms = ctypes.c_float()
            lib.tessera_nvidia_event_elapsed_ms(e0, e1, ctypes.byref(ms))
            times.append(ms.value)
        lib.tessera_nvidia_event_destroy(e0)
        lib.tessera_nvidia_event_destroy(e1)
        rows = [0, n // 3, n - 1]
        got = dd.numpy()[rows]
        want = a[rows].astype(np.float32) @ b.astype(np.float32)
        err = float(np.abs(got - want).max() / np.abs(want).max())
        ms = min(times)
        print(json.dumps({"impl": "reference-gpu", "kernel": "tessera_nvidia_mma_gemm_bf16_device", "size": n,
                          "ms": ms, "tflops": 2.0 * n ** 3 / ms / 1e9, "rc": rc, "max_rel_err_3_rows": err}), flush=True)


if __name__ == "__main__":
    main()
