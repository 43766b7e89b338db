"""Shared helpers for the GPU parity tests (they call the kernels through the C ABI)."""
import ctypes

import numpy as np

from tessera_b200 import _lib, device
from tessera_b200.device import DeviceArray, bfloat16

TOL = 1e-2  # max|y - ref| / max|ref|, computed in fp32 (the stated parity tolerance)


def rel_err(y, ref):
    y = np.asarray(y).astype(np.float32)
    ref = np.asarray(ref).astype(np.float32)
    return float(np.abs(y - ref).max() / max(float(np.abs(ref).max()), 1e-30))


def no_device_error():
    code, block, detail = device.consume_device_error()
    assert code == 0, f"a bounded device wait expired: code {code}, block {block}, detail {detail}"


def gemm_device(A, B, out_dtype=np.float32):
    """A [..,M,K], B [..,K,N] host arrays -> host result through tessera_sm100_gemm_device."""
    batch = int(np.prod(A.shape[:-2], dtype=np.int64)) if A.ndim > 2 else 1
    M, K, N = A.shape[-2], A.shape[-1], B.shape[-1]
    dA, dB = DeviceArray.from_host(A), DeviceArray.from_host(B)
    dD = DeviceArray.zeros(A.shape[:-2] + (M, N), out_dtype)
    _lib.call("tessera_sm100_gemm_device", dA.ptr, dB.ptr, dD.ptr, batch, M, N, K,
              device.dtype_code(A.dtype), device.dtype_code(out_dtype), None)
    out = dD.download()
    no_device_error()
    return out


def attn_device(q, k, v, causal, scale=None, decode_splits=None):
    B, Hq, Sq, D = q.shape
    _, Hkv, Sk, _ = k.shape
    scale = 1.0 / np.sqrt(D) if scale is None else scale
    dq, dk, dv = (DeviceArray.from_host(t) for t in (q, k, v))
    do = DeviceArray.zeros(q.shape, bfloat16)
    if decode_splits is not None:
        lib = _lib.load()
        ns = decode_splits if decode_splits > 0 else lib.tessera_sm100_attn_decode_splits(B, Hq, Hkv, Sk)
        scr = DeviceArray((max(1, lib.tessera_sm100_attn_decode_scratch_bytes(B, Hq, max(ns, 1))),), np.uint8)
        _lib.call("tessera_sm100_attn_decode_device", dq.ptr, dk.ptr, dv.ptr, do.ptr, B, Hq, Hkv, Sk, D,
                  ctypes.c_float(scale), decode_splits, scr.ptr, None)
    else:
        _lib.call("tessera_sm100_flash_attn_fwd_device", dq.ptr, dk.ptr, dv.ptr, do.ptr, B, Hq, Hkv, Sq,
                  Sk, D, ctypes.c_float(scale), int(causal), None)
    out = do.download()
    no_device_error()
    return out
