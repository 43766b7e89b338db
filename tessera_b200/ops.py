"""``tessera.ops`` for the B200 backend: the dense-contraction ops, executed on the GPU.

Same names, arguments and error behaviour as the reference's numpy ops
(python/tessera/__init__.py:239-254 ``gemm``/``matmul``/``batched_gemm``, :291-351
``grouped_gemm``, :559-616 ``silu_mul``/``swiglu``/``moe_swiglu_block``, :1304-1356 ``flash_attn``,
python/tessera/nn/functional.py:349-356 ``gqa_attention``), but every op here calls the sm_100a
kernels through the C ABI. There is no CPU fallback: without the shared library or a GPU the
call raises ``BackendError``.

Host arrays (numpy, or anything with ``._data`` / ``.numpy()``) go in and numpy arrays come out;
``DeviceArray`` inputs stay on the device and produce ``DeviceArray`` outputs, so a chain of ops
moves no data across PCIe.

Differences from the numpy reference, all on the side of what its own GPU lanes do:
* 16-bit GEMM operands accumulate in fp32 and the result is float32 unless ``out_dtype`` is
  given (the reference's shipped GEMM symbols return fp32,
  src/compiler/codegen/tessera_gpu_backend_NVIDIA/runtime/cuda/tessera_nvidia_gemm.cpp:41-60).
* float32 host operands are not accepted by the tensor-core ops unless ``compute_dtype`` says
  which 16-bit format to round them to.
"""
from __future__ import annotations

import ctypes
from typing import Any, Optional

import numpy as np

from . import _lib, device
from .device import DeviceArray, StridedView, bfloat16

GROUPED_KINDS = ("contiguous", "dense", "masked", "k_grouped")
SUPPORTED_GROUPED_KINDS = ("contiguous", "dense")


def _unwrap(x: Any) -> Any:
    """DeviceArray stays; everything else becomes a numpy array (reference `_as_numpy`,
    python/tessera/runtime.py:44377-44384)."""
    if isinstance(x, (DeviceArray, StridedView)):
        return x
    if hasattr(x, "_data"):
        return np.asarray(x._data)
    if hasattr(x, "numpy") and callable(x.numpy):
        return np.asarray(x.numpy())
    return np.asarray(x)


def _storage_dtype(arrs, compute_dtype: Optional[str], op: str) -> np.dtype:
    dts = {np.dtype(a.dtype) for a in arrs}
    if compute_dtype is not None:
        name = {"bf16": bfloat16, "bfloat16": bfloat16, "f16": np.dtype(np.float16),
                "fp16": np.dtype(np.float16), "float16": np.dtype(np.float16)}.get(compute_dtype)
        if name is None:
            raise ValueError(f"{op}: compute_dtype must be 'bf16' or 'f16', got {compute_dtype!r}")
        return np.dtype(name)
    if len(dts) != 1:
        raise TypeError(f"{op}: operands must share one dtype, got {sorted(map(str, dts))}")
    dt = dts.pop()
    if dt == np.float16 or dt == bfloat16:
        return dt
    raise TypeError(f"{op}: operands must be float16 or bfloat16 (got {dt}); pass "
                    f"compute_dtype='bf16' to round float32 operands")


def _to_device(x, dt: np.dtype) -> DeviceArray:
    if isinstance(x, DeviceArray):
        if x.dtype != dt:
            raise TypeError(f"device operand has dtype {x.dtype}, expected {dt}")
        return x
    return DeviceArray.from_host(np.ascontiguousarray(x).astype(dt, copy=False))


def _any_device(*xs) -> bool:
    return any(isinstance(x, DeviceArray) for x in xs)


def _out_code(out_dtype, default: int) -> int:
    if out_dtype is None:
        return default
    return device.dtype_code(out_dtype)


# --------------------------------------------------------------------------------- GEMM
def gemm(A, B, epilogue=None, *, out_dtype=None, compute_dtype: Optional[str] = None, stream=None,
         out=None):
    """Matrix multiply ``A @ B``; leading dimensions are a batch (python/tessera/__init__.py:239-248).
    ``out`` (host operands only) is an optional preallocated result array, e.g. pinned memory."""
    if epilogue:
        return _gemm_fused(A, B, dict(epilogue), out_dtype, compute_dtype, stream)
    A, B = _unwrap(A), _unwrap(B)
    if A.ndim < 2 or B.ndim < 2:
        raise ValueError(f"gemm: operands must be at least 2-D, got {A.shape} @ {B.shape}")
    if A.shape[-1] != B.shape[-2]:
        raise ValueError(f"gemm: K mismatch — {A.shape} @ {B.shape}")
    dt = _storage_dtype((A, B), compute_dtype, "gemm")
    in_code = device.dtype_code(dt)
    out_code = _out_code(out_dtype, _lib.F32)
    M, K, N = A.shape[-2], A.shape[-1], B.shape[-1]
    batch_shape = A.shape[:-2]
    if B.shape[:-2] != batch_shape:
        if _any_device(A, B):
            raise ValueError("gemm: device operands must have identical batch dimensions")
        bs = np.broadcast_shapes(A.shape[:-2], B.shape[:-2])
        A = np.broadcast_to(A, bs + A.shape[-2:])
        B = np.broadcast_to(B, bs + B.shape[-2:])
        batch_shape = bs
    batch = int(np.prod(batch_shape, dtype=np.int64)) if batch_shape else 1
    out_shape = tuple(batch_shape) + (M, N)
    if batch == 0 or M == 0 or N == 0:
        return np.zeros(out_shape, device.code_dtype(out_code))
    if K == 0:
        return np.zeros(out_shape, device.code_dtype(out_code))
    if _any_device(A, B):
        dA, dB = _to_device(A, dt), _to_device(B, dt)
        out = DeviceArray(out_shape, device.code_dtype(out_code))
        _lib.call("tessera_sm100_gemm_device", dA.ptr, dB.ptr, out.ptr, batch, M, N, K, in_code,
                  out_code, device._stream_handle(stream))
        return out
    a = np.ascontiguousarray(A).astype(dt, copy=False)
    b = np.ascontiguousarray(B).astype(dt, copy=False)
    if out is None:
        out = np.empty(out_shape, device.code_dtype(out_code))
    elif out.shape != out_shape or out.dtype != device.code_dtype(out_code) or not out.flags.c_contiguous:
        raise ValueError(f"gemm: out must be a contiguous {device.code_dtype(out_code)} array of shape {out_shape}")
    _lib.call("tessera_sm100_gemm", a.ctypes.data, b.ctypes.data, out.ctypes.data, batch, M, N, K,
              in_code, out_code)
    return out


_ACTIVATIONS = {"linear": 0, "none": 0, None: 0, "relu": 1, "gelu": 2, "silu": 3}


def _gemm_fused(A, B, epilogue: dict, out_dtype, compute_dtype, stream):
    """``fused_epilogue(A @ B, **epilogue)`` (python/tessera/__init__.py:2658-2675) with bias,
    residual and activation applied inside the GEMM kernel's epilogue."""
    bias = epilogue.pop("bias", None)
    activation = epilogue.pop("activation", "linear")
    residual = epilogue.pop("residual", None)
    dropout_p = epilogue.pop("dropout_p", 0.0)
    cast_dtype = epilogue.pop("cast_dtype", None)
    if dropout_p:
        raise NotImplementedError("gemm: dropout in the fused epilogue is not part of this backend")
    if epilogue:
        raise TypeError(f"gemm: unknown epilogue key(s) {sorted(epilogue)}")
    if activation not in _ACTIVATIONS:
        raise ValueError(f"gemm: activation must be one of linear/relu/gelu/silu, got {activation!r}")
    A, B = _unwrap(A), _unwrap(B)
    if A.ndim != 2 or B.ndim != 2:
        raise ValueError("gemm: the fused epilogue takes 2-D operands")
    if A.shape[1] != B.shape[0]:
        raise ValueError(f"gemm: K mismatch — {A.shape} @ {B.shape}")
    M, K, N = A.shape[0], A.shape[1], B.shape[1]
    dt = _storage_dtype((A, B), compute_dtype, "gemm")
    out_code = _out_code(cast_dtype if cast_dtype is not None else out_dtype, _lib.F32)
    out_dt = device.code_dtype(out_code)
    on_device = _any_device(A, B)
    dA, dB = _to_device(A, dt), _to_device(B, dt)
    dbias = dres = None
    if bias is not None:
        b = np.ascontiguousarray(np.broadcast_to(np.asarray(_unwrap(bias), np.float32), (N,)))
        dbias = DeviceArray.from_host(b)
    if residual is not None:
        r = _unwrap(residual)
        if isinstance(r, DeviceArray):
            if r.shape != (M, N) or r.dtype != out_dt:
                raise ValueError(f"gemm: device residual must be {(M, N)} {out_dt}")
            dres = r
        else:
            dres = DeviceArray.from_host(np.ascontiguousarray(np.broadcast_to(np.asarray(r), (M, N))).astype(out_dt))
    out = DeviceArray((M, N), out_dt)
    _lib.call("tessera_sm100_gemm_epilogue_device", dA.ptr, dB.ptr, out.ptr, M, N, K, device.dtype_code(dt),
              out_code, dbias.ptr if dbias else None, dres.ptr if dres else None, _ACTIVATIONS[activation],
              device._stream_handle(stream))
    return out if on_device else _finish(out)


def matmul(A, B, epilogue=None, **kw):
    return gemm(A, B, epilogue=epilogue, **kw)


def batched_gemm(A, B, epilogue=None, **kw):
    return gemm(A, B, epilogue=epilogue, **kw)


# --------------------------------------------------------------------------------- attention
def flash_attn(Q, K=None, V=None, scale=None, causal: bool = False, cache=None,
               dropout_p: float = 0.0, params=None, deterministic=None, seed=None, attn_bias=None,
               kv_state=None, *, window=None, softcap=None, causal_alignment: str = "bottom_right",
               stream=None):
    """``softmax(scale * Q K^T [+ attn_bias], causal) V`` (python/tessera/__init__.py:1304-1356). Q
    [B,Hq,Sq,D], K [B,Hkv,Sk,D], V [B,Hkv,Sk,Dv]; Hkv may divide Hq (grouped-query attention).

    bfloat16 operands with D = Dv = 128 and no bias / window / soft-cap run on the tcgen05 prefill
    kernel or the split-KV decode kernel; every other combination (float32 / float16 / bfloat16
    storage, any head dimension up to 512, ``attn_bias`` broadcastable to [B,Hq,Sq,Sk], ``window``
    = n or (left, right), ``softcap``) runs on the general kernel with the semantics of the
    reference's CUDA lane (python/tessera/compiler/emit/nvidia_cuda.py:251-276).
    ``causal_alignment``: "bottom_right" masks key j > i + max(Sk - Sq, 0) as the reference op does;
    "top_left" masks j > i as the reference's launch executor does."""
    if kv_state is not None:  # python/tessera/__init__.py:1318-1321
        return paged_attention(Q, kv_state, scale=scale, causal=causal)
    if cache is not None:
        raise NotImplementedError("flash_attn: cache= is not part of this backend; pass kv_state=")
    if not 0.0 <= dropout_p < 1.0:
        raise ValueError("dropout_p must be in [0.0, 1.0)")
    if dropout_p > 0.0:
        raise NotImplementedError("flash_attn: dropout is not part of this backend")
    if causal_alignment not in ("bottom_right", "top_left"):
        raise ValueError("causal_alignment must be 'bottom_right' or 'top_left'")
    if K is None or V is None:
        raise ValueError("flash_attn: K and V are required")
    Q, K, V = _unwrap(Q), _unwrap(K), _unwrap(V)
    squeeze = 0
    while Q.ndim < 4:  # (S, D) or (H, S, D) like numpy broadcasting would accept
        if _any_device(Q, K, V):
            raise ValueError("flash_attn: device operands must be 4-D [B, H, S, D]")
        Q, K, V = Q[None], K[None], V[None]
        squeeze += 1
    if Q.ndim != 4 or K.ndim != 4 or V.ndim != 4:
        raise ValueError(f"flash_attn: expected [B, H, S, D] operands, got {Q.shape}, {K.shape}, {V.shape}")
    Bq, Hq, Sq, D = Q.shape
    Bk, Hkv, Sk, Dk = K.shape
    Dv = V.shape[3]
    if tuple(V.shape[:3]) != tuple(K.shape[:3]) or Bk != Bq or Dk != D:
        raise ValueError(f"flash_attn: incompatible shapes Q {Q.shape}, K {K.shape}, V {V.shape}")
    if Hq % Hkv:
        raise ValueError("num_query_heads must be divisible by num_kv_heads")
    dts = {np.dtype(t.dtype) for t in (Q, K, V)}
    if len(dts) != 1:
        raise TypeError(f"flash_attn: operands must share one dtype, got {sorted(map(str, dts))}")
    dt = dts.pop()
    if dt not in (np.dtype(np.float32), np.dtype(np.float16), bfloat16):
        raise TypeError(f"flash_attn: operands must be float32, float16 or bfloat16 (got {dt})")
    if scale is None:
        scale = 1.0 / np.sqrt(D)
    cscale = ctypes.c_float(float(scale))
    wl = wr = -1
    if window is not None:
        wl, wr = (window if isinstance(window, (tuple, list)) else (window, window))
        wl = -1 if wl is None else int(wl)
        wr = -1 if wr is None else int(wr)
        if (wl < 0 and wl != -1) or (wr < 0 and wr != -1):
            raise ValueError("window bounds must be >= 0")
    cap = 0.0 if softcap is None else float(softcap)
    if cap < 0:
        raise ValueError("softcap must be >= 0")
    shift = max(Sk - Sq, 0) if causal_alignment == "bottom_right" else 0
    fast = (dt == bfloat16 and D == 128 and Dv == 128 and attn_bias is None and wl < 0 and wr < 0 and cap == 0.0
            and (not causal or shift == max(Sk - Sq, 0)))
    on_device = _any_device(Q, K, V)
    if fast and on_device:
        dq, dk, dv = _to_device(Q, dt), _to_device(K, dt), _to_device(V, dt)
        out = DeviceArray(Q.shape, dt)
        _lib.call("tessera_sm100_flash_attn_device", dq.ptr, dk.ptr, dv.ptr, out.ptr, Bq, Hq, Hkv, Sq,
                  Sk, D, cscale, int(bool(causal)), device._stream_handle(stream))
        return out
    if fast:
        q, k, v = (np.ascontiguousarray(t) for t in (Q, K, V))
        out = np.empty(q.shape, dt)
        _lib.call("tessera_sm100_flash_attn", q.ctypes.data, k.ctypes.data, v.ctypes.data, out.ctypes.data,
                  Bq, Hq, Hkv, Sq, Sk, D, cscale, int(bool(causal)))
    else:
        if D > 512 or Dv > 512:
            raise ValueError(f"flash_attn: head dimensions up to 512 are served (got D={D}, Dv={Dv})")
        dbias = None
        if attn_bias is not None:
            b = _unwrap(attn_bias)
            if isinstance(b, DeviceArray):
                if b.shape != (Bq, Hq, Sq, Sk) or b.dtype != np.float32:
                    raise ValueError("flash_attn: a device attn_bias must be float32 [B, Hq, Sq, Sk]")
                dbias = b
            else:
                try:
                    full = np.broadcast_to(np.asarray(b, np.float32), (Bq, Hq, Sq, Sk))
                except ValueError:
                    raise ValueError(f"flash_attn: attn_bias {np.shape(b)} does not broadcast to "
                                     f"{(Bq, Hq, Sq, Sk)}") from None
                dbias = DeviceArray.from_host(np.ascontiguousarray(full), pooled=True)
        dq, dk, dv = _to_device(Q, dt), _to_device(K, dt), _to_device(V, dt)
        dout = DeviceArray((Bq, Hq, Sq, Dv), dt)
        _lib.call("tessera_sm100_flash_attn_general_device", dq.ptr, dk.ptr, dv.ptr,
                  dbias.ptr if dbias is not None else None, dout.ptr, Bq, Hq, Hkv, Sq, Sk, D, Dv, cscale,
                  int(bool(causal)), shift, wl, wr, ctypes.c_float(cap), device.dtype_code(dt),
                  device._stream_handle(stream))
        if on_device:
            return dout
        out = _finish(dout)
    for _ in range(squeeze):
        out = out[0]
    return out


def flash_attn_backward(dO, Q, K, V, *, scale=None, causal: bool = False, window=None, attn_bias=None,
                        softcap=None, causal_alignment: str = "top_left", stream=None):
    """Gradients ``(dQ, dK, dV)`` of ``flash_attn`` with respect to Q, K and V for the output
    gradient ``dO``: the contract of the reference's CUDA backward lane
    (python/tessera/compiler/emit/nvidia_cuda.py:590-635, 675-750). dO [B,Hq,Sq,Dv], Q [B,Hq,Sq,D],
    K [B,Hkv,Sk,D], V [B,Hkv,Sk,Dv] in one of float32 / float16 / bfloat16; the gradients come back
    in that dtype (fp32 math). ``causal_alignment`` defaults to the lane's "top_left" (key j > i
    masked); "bottom_right" is the mask of ``ops.flash_attn``. Device operands give device
    results. Deterministic: every gradient row is summed in a fixed order."""
    if causal_alignment not in ("bottom_right", "top_left"):
        raise ValueError("causal_alignment must be 'bottom_right' or 'top_left'")
    dO, Q, K, V = _unwrap(dO), _unwrap(Q), _unwrap(K), _unwrap(V)
    if any(t.ndim != 4 for t in (dO, Q, K, V)):
        raise ValueError("flash_attn_backward requires rank-4 dO/Q/K/V tensors")
    Bq, Hq, Sq, D = Q.shape
    Bk, Hkv, Sk, Dk = K.shape
    Dv = V.shape[3]
    if (tuple(V.shape[:3]) != tuple(K.shape[:3]) or Bk != Bq or Dk != D or tuple(dO.shape) != (Bq, Hq, Sq, Dv)
            or Hq % Hkv or max(D, Dv) > 256):
        raise ValueError("invalid flash_attn_backward Q/K/V/dO shape or head mapping")
    dts = {np.dtype(t.dtype) for t in (dO, Q, K, V)}
    if len(dts) != 1 or next(iter(dts)) not in (np.dtype(np.float32), np.dtype(np.float16), bfloat16):
        raise TypeError("flash_attn_backward requires matching float32, float16 or bfloat16 dO/Q/K/V storage")
    dt = dts.pop()
    if scale is None:
        scale = 1.0 / np.sqrt(D)
    wl = wr = -1
    if window is not None:
        wl, wr = (window if isinstance(window, (tuple, list)) else (window, window))
        wl = -1 if wl is None else int(wl)
        wr = -1 if wr is None else int(wr)
    cap = 0.0 if softcap is None else float(softcap)
    if wl < -1 or wr < -1 or cap < 0.0:
        raise ValueError("window bounds must be >= 0 and softcap must be >= 0")
    dbias = None
    if attn_bias is not None:
        b = _unwrap(attn_bias)
        if isinstance(b, DeviceArray):
            if b.shape != (Bq, Hq, Sq, Sk) or b.dtype != np.float32:
                raise ValueError("flash_attn_backward: a device attn_bias must be float32 [B, Hq, Sq, Sk]")
            dbias = b
        else:
            b = np.asarray(b)
            if b.dtype != np.float32 or b.shape != (Bq, Hq, Sq, Sk):
                raise ValueError("flash_attn_backward bias must be float32 with shape [B,Hq,Sq,Sk]")
            dbias = DeviceArray.from_host(np.ascontiguousarray(b), pooled=True)
    shift = max(Sk - Sq, 0) if causal_alignment == "bottom_right" else 0
    on_device = _any_device(dO, Q, K, V)
    dgo, dq_, dk_, dv_ = (_to_device(t, dt) for t in (dO, Q, K, V))
    gq, gk, gv = DeviceArray(Q.shape, dt), DeviceArray(K.shape, dt), DeviceArray(V.shape, dt)
    # the training shape runs on the tensor cores (its causal mask is the bottom-right one)
    if (dt == bfloat16 and D == 128 and Dv == 128 and dbias is None and wl < 0 and wr < 0 and cap == 0.0
            and (not causal or shift == max(Sk - Sq, 0))):
        nws = int(_lib.load().tessera_sm100_flash_attn_bwd_bf16_workspace_bytes(Bq, Hq, Sq))
        ws = DeviceArray((nws,), np.uint8, pooled=True)
        _lib.call("tessera_sm100_flash_attn_bwd_bf16_device", dgo.ptr, dq_.ptr, dk_.ptr, dv_.ptr, gq.ptr, gk.ptr,
                  gv.ptr, Bq, Hq, Hkv, Sq, Sk, ctypes.c_float(float(scale)), int(bool(causal)), ws.ptr,
                  device._stream_handle(stream))
        if on_device:
            return gq, gk, gv
        return _finish(gq), _finish(gk), _finish(gv)
    nws = int(_lib.load().tessera_sm100_flash_attn_bwd_workspace_bytes(Bq, Hq, Sq))
    ws = DeviceArray((nws,), np.uint8, pooled=True)
    _lib.call("tessera_sm100_flash_attn_bwd_device", dgo.ptr, dq_.ptr, dk_.ptr, dv_.ptr,
              dbias.ptr if dbias is not None else None, gq.ptr, gk.ptr, gv.ptr, Bq, Hq, Hkv, Sq, Sk, D, Dv,
              ctypes.c_float(float(scale)), int(bool(causal)), shift, wl, wr, ctypes.c_float(cap),
              device.dtype_code(dt), ws.ptr, device._stream_handle(stream))
    if on_device:
        return gq, gk, gv
    return _finish(gq), _finish(gk), _finish(gv)


def paged_attention(Q, kv_state, *, scale=None, causal: bool = False, token_indices=None):
    """Attention over a paged KV state (python/tessera/__init__.py:1291-1302): ``Q`` is
    ``(num_heads, q_len, 128)``; the pages are read in place by the paged decode kernel."""
    from .cache import paged_attention as _pa
    return _pa(_unwrap(Q), kv_state, scale=scale, causal=causal, token_indices=token_indices)


def _f32_device(x) -> DeviceArray:
    if isinstance(x, DeviceArray):
        if x.dtype != np.float32:
            raise TypeError("attention states are float32")
        return x
    return DeviceArray.from_host(np.ascontiguousarray(x, np.float32))


def softmax_merge(output_a, maximum_a, normalizer_a, output_b, maximum_b, normalizer_b, *, stream=None):
    """Associative merge of two max-shifted attention states ``(o, m, l)``
    (python/tessera/_block_attnres_ops.py:104-131). Host states are checked like the reference
    (matching shapes, strictly positive normalisers); device states are taken as they are."""
    ins = [_unwrap(t) for t in (output_a, maximum_a, normalizer_a, output_b, maximum_b, normalizer_b)]
    on_device = _any_device(*ins)
    oa, ma, la, ob, mb, lb = ins
    for name, (o, m, l) in (("state_a", (oa, ma, la)), ("state_b", (ob, mb, lb))):
        if len(o.shape) < 1 or tuple(o.shape[:-1]) != tuple(m.shape):
            raise ValueError(f"{name} output prefix {tuple(o.shape[:-1])} must match maximum shape {tuple(m.shape)}")
        if tuple(l.shape) != tuple(m.shape):
            raise ValueError(f"{name} normalizer shape {tuple(l.shape)} must match maximum shape {tuple(m.shape)}")
        if not isinstance(l, DeviceArray) and np.any(np.asarray(l) <= 0.0):
            raise ValueError(f"{name} normalizer must be strictly positive")
    if tuple(oa.shape) != tuple(ob.shape) or tuple(ma.shape) != tuple(mb.shape):
        raise ValueError("softmax_merge states must have identical shapes")
    d = [_f32_device(t) for t in ins]
    rows, Dv = int(np.prod(ma.shape, dtype=np.int64)), int(oa.shape[-1])
    o, m, l = DeviceArray(oa.shape, np.float32), DeviceArray(ma.shape, np.float32), DeviceArray(ma.shape, np.float32)
    _lib.call("tessera_sm100_softmax_merge_device", *(t.ptr for t in d), o.ptr, m.ptr, l.ptr, rows, Dv,
              device._stream_handle(stream))
    if on_device:
        return o, m, l
    return o.download(), m.download(), l.download()


def softmax_finalize(output, normalizer, *, out_dtype=None, stream=None):
    """``output / l`` (python/tessera/_block_attnres_ops.py:134-146)."""
    o, l = _unwrap(output), _unwrap(normalizer)
    if len(o.shape) < 1 or tuple(o.shape[:-1]) != tuple(l.shape):
        raise ValueError(f"output prefix {tuple(o.shape[:-1])} must match normalizer shape {tuple(l.shape)}")
    if not isinstance(l, DeviceArray) and np.any(np.asarray(l) <= 0.0):
        raise ValueError("normalizer must be strictly positive")
    on_device = _any_device(o, l)
    do, dl = _f32_device(o), _f32_device(l)
    code = _out_code(out_dtype, _lib.F32)
    out = DeviceArray(o.shape, device.code_dtype(code))
    _lib.call("tessera_sm100_softmax_finalize_device", do.ptr, dl.ptr, out.ptr,
              int(np.prod(l.shape, dtype=np.int64)), int(o.shape[-1]), code, device._stream_handle(stream))
    return out if on_device else out.download()


def attn_decode_state(Q, K, V, *, scale=None, stream=None):
    """Decode attention of ``Q`` ``[B, Hq, 1, 128]`` over ``K``, ``V`` ``[B, Hkv, Sk, 128]`` stopped
    before the division: the state ``(o [B,Hq,128], m [B,Hq], l [B,Hq])`` of this key set. States of
    disjoint key sets (KV shards) combine with :func:`softmax_merge` and :func:`softmax_finalize`."""
    q, k, v = _unwrap(Q), _unwrap(K), _unwrap(V)
    on_device = _any_device(q, k, v)
    if len(q.shape) != 4 or q.shape[2] != 1 or len(k.shape) != 4 or tuple(k.shape) != tuple(v.shape):
        raise ValueError("attn_decode_state: Q must be [B, Hq, 1, D] and K, V equal-shape [B, Hkv, Sk, D]")
    B, Hq, _, D = q.shape
    Hkv, Sk = k.shape[1], k.shape[2]
    if Hq % Hkv:
        raise ValueError("num_query_heads must be divisible by num_kv_heads")
    dq, dk, dv = _to_device(q, bfloat16), _to_device(k, bfloat16), _to_device(v, bfloat16)
    lib = _lib.load()
    splits = max(1, int(lib.tessera_sm100_attn_decode_splits(B, Hq, Hkv, Sk)))
    scratch = DeviceArray((int(lib.tessera_sm100_attn_decode_scratch_bytes(B, Hq, splits)),), np.uint8, pooled=True)
    o, m, l = (DeviceArray((B, Hq, D), np.float32), DeviceArray((B, Hq), np.float32),
               DeviceArray((B, Hq), np.float32))
    sc = float(1.0 / np.sqrt(D) if scale is None else scale)
    _lib.call("tessera_sm100_attn_decode_state_device", dq.ptr, dk.ptr, dv.ptr, o.ptr, m.ptr, l.ptr, B, Hq, Hkv,
              Sk, D, sc, splits, scratch.ptr, device._stream_handle(stream))
    if on_device:
        return o, m, l
    res = (o.download(), m.download(), l.download())
    device.check_device_error("attn_decode_state")
    return res


def gqa_attention(Q, K, V, num_query_heads: int, num_kv_heads: int, **kwargs):
    """Grouped-query attention (python/tessera/nn/functional.py:349-356). The KV heads are shared
    inside the kernel instead of being repeated in memory."""
    if num_query_heads % num_kv_heads != 0:
        raise ValueError("num_query_heads must be divisible by num_kv_heads")
    q, k = _unwrap(Q), _unwrap(K)
    if q.shape[1] != num_query_heads or k.shape[1] != num_kv_heads:
        raise ValueError(f"gqa_attention: Q has {q.shape[1]} heads and K has {k.shape[1]}, expected "
                         f"{num_query_heads} and {num_kv_heads}")
    return flash_attn(Q, K, V, **kwargs)


def mqa_attention(Q, K, V, **kwargs):
    return gqa_attention(Q, K, V, num_query_heads=_unwrap(Q).shape[1], num_kv_heads=1, **kwargs)


# --------------------------------------------------------------------------------- MoE
def _group_offsets(group_sizes, T: int, op: str) -> np.ndarray:
    gs = np.asarray(group_sizes).astype(np.int64).reshape(-1)
    if int(gs.sum()) != T:
        raise ValueError(f"{op}: group_sizes sum {int(gs.sum())} != T={T}")
    if np.any(gs < 0):
        raise ValueError(f"{op}: group_sizes must be non-negative")
    off = np.zeros(gs.shape[0] + 1, np.int32)
    off[1:] = np.cumsum(gs)
    return off


# quant names of the reference (python/tessera/compiler/grouped_layout.py:319-350) -> 8-bit format code
# (tessera_sm100.h: 0 = e4m3, 1 = e5m2), and the activation format of the schemes with NVFP4 weights
_FP8_QUANTS = {"fp8": 0, "fp8_e4m3": 0, "fp8_e5m2": 1}
_FP4_QUANTS = {"nvfp4": "nvfp4", "fp8xfp4": 0, "fp8_e4m3xnvfp4": 0, "fp8_e5m2xnvfp4": 1}
_OTHER_QUANTS = ()


def _check_kind(kind: str, alignment, group_sizes, quant, op: str) -> None:
    if kind not in GROUPED_KINDS:
        raise ValueError(f"{op}: unknown kind {kind!r}; expected one of {GROUPED_KINDS}")
    if kind not in SUPPORTED_GROUPED_KINDS:
        raise NotImplementedError(f"{op}: kind={kind!r} is not implemented yet")
    if quant is not None and str(quant).lower() not in tuple(_FP8_QUANTS) + tuple(_FP4_QUANTS):
        raise ValueError(f"{op}: quant {quant!r} has no grouped path; expected one of "
                         f"{tuple(_FP8_QUANTS) + tuple(_FP4_QUANTS)}")
    if alignment is not None:
        gs = np.asarray(group_sizes).astype(np.int64).reshape(-1)
        if np.any(gs % int(alignment)):
            raise ValueError(f"{op}: every group size must be a multiple of alignment={alignment}")


class Fp8Tensor:
    """8-bit floats (``fmt`` 0 = e4m3, 1 = e5m2) on the device with their scale(s): ``q`` uint8,
    ``scales`` float32 device array whose first element(s) are the scale(s)
    (``tessera_sm100_quantize_fp8*_device`` layouts)."""

    def __init__(self, q: DeviceArray, scales: DeviceArray, shape, per_expert: bool, fmt: int = 0):
        self.q, self.scales, self.shape, self.per_expert, self.fmt = q, scales, tuple(shape), per_expert, int(fmt)

    def scale_values(self) -> np.ndarray:
        n = self.shape[0] if self.per_expert else 1
        return self.scales.download()[:n]


def _fp8_fmt(format) -> int:
    if format in (0, 1):
        return int(format)
    try:
        return {"e4m3": 0, "e5m2": 1}[str(format).lower()]
    except KeyError:
        raise ValueError(f"format must be 'e4m3' or 'e5m2'; got {format!r}") from None


def quantize_fp8_activations(x, *, amax_bits: Optional[DeviceArray] = None, format="e4m3", stream=None) -> Fp8Tensor:
    """Per-tensor 8-bit float quantisation of ``x`` (any shape; float32 / float16 / bfloat16) on the
    device: ``scale = max(amax/max_normal, 1e-12)`` with ``max_normal`` 448 (e4m3) or 57344 (e5m2),
    ``q = fp8(x / scale)`` (python/tessera/__init__.py:3340-3374)."""
    fmt = _fp8_fmt(format)
    xa = _unwrap(x)
    dx = xa if isinstance(xa, DeviceArray) else DeviceArray.from_host(np.ascontiguousarray(xa), pooled=True)
    q = DeviceArray(dx.shape, np.uint8)
    scales = DeviceArray((3,), np.float32)
    _lib.call("tessera_sm100_quantize_fp8_fmt_device", dx.ptr, int(dx.size), device.dtype_code(dx.dtype), fmt, q.ptr,
              scales.ptr, amax_bits.ptr if amax_bits is not None else None, device._stream_handle(stream))
    return Fp8Tensor(q, scales, dx.shape, False, fmt)


def quantize_fp8_experts(weights, *, format="e4m3", stream=None) -> Fp8Tensor:
    """Per-expert 8-bit float quantisation of ``weights`` (E, K, N), stored transposed as (E, N, K) so both
    GEMM operands are K-major (python/tessera/compiler/grouped_layout.py:371-392). Expert weights are
    static: quantise once and pass the result wherever weights are expected."""
    w = _unwrap(weights)
    if len(w.shape) != 3:
        raise ValueError(f"quantize_fp8_experts: weights must be (E, K, N); got {tuple(w.shape)}")
    dw = w if isinstance(w, DeviceArray) else DeviceArray.from_host(np.ascontiguousarray(w), pooled=True)
    E, K, N = dw.shape
    q = DeviceArray((E, N, K), np.uint8)
    scales = DeviceArray((3 * E,), np.float32)
    fmt = _fp8_fmt(format)
    _lib.call("tessera_sm100_quantize_fp8_weights_fmt_device", dw.ptr, E, K, N, device.dtype_code(dw.dtype), fmt,
              q.ptr, scales.ptr, device._stream_handle(stream))
    return Fp8Tensor(q, scales, (E, K, N), True, fmt)


def _as_fp8_experts(w, fmt, stream) -> Fp8Tensor:
    if isinstance(w, Fp8Tensor):
        if w.fmt != fmt:
            raise ValueError("pre-quantised weights are in a different 8-bit format than the one asked for")
        return w
    return quantize_fp8_experts(w, format=fmt, stream=stream)


class Nvfp4Tensor:
    """NVFP4 storage on the device: ``codes`` uint8, two e2m1 codes per byte along the last axis
    (even element in the low nibble), ``scales`` uint8 e4m3, one per block of 16; ``shape`` is the
    logical shape. 4.5 bits per element."""

    def __init__(self, codes: DeviceArray, scales: DeviceArray, shape):
        self.codes, self.scales, self.shape = codes, scales, tuple(int(d) for d in shape)

    def dequantize(self, dtype=bfloat16, *, stream=None) -> DeviceArray:
        rows = int(np.prod(self.shape[:-1], dtype=np.int64))
        out = DeviceArray(self.shape, dtype, pooled=True)
        _lib.call("tessera_sm100_dequantize_nvfp4_device", self.codes.ptr, self.scales.ptr, rows, self.shape[-1],
                  out.ptr, device.dtype_code(np.dtype(dtype)), device._stream_handle(stream))
        return out


def quantize_nvfp4(x, *, block_size: int = 16, stream=None) -> Nvfp4Tensor:
    """Block-scaled e2m1 quantisation along the last axis with the reference's arithmetic
    (python/tessera/__init__.py:3472-3500, python/tessera/compiler/microscaling.py:319-362): one e4m3
    scale ``max(amax/6, 1e-30)`` per 16 elements. For expert weights (E, K, N) the blocks run along
    N, as the reference quantises each expert's matrix."""
    if block_size != 16:
        raise NotImplementedError("quantize_nvfp4: block_size 16 (the NVFP4 layout) is the one served")
    xa = _unwrap(x)
    if xa.shape[-1] % 16:
        raise ValueError(f"last dim {xa.shape[-1]} must be divisible by block_size 16 for NVFP4")
    dx = xa if isinstance(xa, DeviceArray) else DeviceArray.from_host(np.ascontiguousarray(xa), pooled=True)
    rows = int(np.prod(xa.shape[:-1], dtype=np.int64))
    cols = int(xa.shape[-1])
    codes = DeviceArray(tuple(xa.shape[:-1]) + (cols // 2,), np.uint8)
    scales = DeviceArray(tuple(xa.shape[:-1]) + (cols // 16,), np.uint8)
    _lib.call("tessera_sm100_quantize_nvfp4_device", dx.ptr, rows, cols, device.dtype_code(dx.dtype), codes.ptr,
              scales.ptr, device._stream_handle(stream))
    return Nvfp4Tensor(codes, scales, xa.shape)


def dequantize_nvfp4(t: Nvfp4Tensor, *, dtype=np.float32, stream=None):
    """The values an :class:`Nvfp4Tensor` stands for, on the host."""
    return _finish(t.dequantize(dtype, stream=stream))


def _fp4_operand(x, act: str, stream):
    """x -> (bf16 device array holding the quantised values exactly, device scale or None)."""
    if act == "nvfp4":
        return quantize_nvfp4(x, stream=stream).dequantize(bfloat16, stream=stream), None
    xq = quantize_fp8_activations(x, format=act, stream=stream)
    vals = DeviceArray(tuple(xq.q.shape), bfloat16, pooled=True)
    _lib.call("tessera_sm100_fp8_to_bf16_device", xq.q.ptr, int(xq.q.size), xq.fmt, vals.ptr,
              device._stream_handle(stream))
    return vals, xq.scales


def _fp4_weights(w, stream) -> DeviceArray:
    t = w if isinstance(w, Nvfp4Tensor) else quantize_nvfp4(w, stream=stream)
    if len(t.shape) != 3:
        raise ValueError(f"grouped weights must be (E, K, N); got {t.shape}")
    return t.dequantize(bfloat16, stream=stream)


def _grouped_gemm_fp4(x, weights, group_sizes, act, out_dtype, stream):
    """Grouped GEMM with NVFP4 weights and nvfp4 or e4m3 activations. Both operands are turned into
    bf16 arrays that hold the quantised values exactly (e2m1 x e4m3-scale has at most 5 significant
    bits, an e4m3 value 4), multiplied on the bf16 tensor-core path with fp32 accumulation, and the
    per-tensor activation scale of the fp8 scheme is applied to the accumulators: the products are
    those of the reference's dequantise-then-f32-matmul."""
    xa = _unwrap(x)
    if len(xa.shape) != 2:
        raise ValueError(f"grouped_gemm: x must be (T, K); got {tuple(xa.shape)}")
    T, K = xa.shape
    on_device = isinstance(xa, DeviceArray)
    wd = _fp4_weights(weights, stream)
    E, Kw, N = wd.shape
    if Kw != K:
        raise ValueError(f"grouped_gemm: K mismatch — x K={K}, weights K={Kw}")
    off = _group_offsets(group_sizes, T, "grouped_gemm")
    if off.shape[0] != E + 1:
        raise ValueError(f"grouped_gemm: weights {wd.shape} must be (E, K, N) with E == len(group_sizes)="
                         f"{off.shape[0] - 1}")
    xv, xs = _fp4_operand(xa, act, stream)
    odt = np.dtype(out_dtype) if out_dtype is not None else np.dtype(xa.dtype)
    out = DeviceArray((T, N), odt)
    doff = DeviceArray.from_host(off, pooled=True)
    _lib.call("tessera_sm100_grouped_gemm_scaled_device", xv.ptr, wd.ptr, doff.ptr, out.ptr, T, K, N, E, _lib.BF16,
              device.dtype_code(odt), xs.ptr if xs is not None else None, device._stream_handle(stream))
    return out if on_device else _finish(out)


def _moe_swiglu_block_fp4(x, w_gate, w_up, w_down, group_sizes, act, stream):
    """Expert FFN with NVFP4 weights: as the fp8 block, every grouped GEMM quantises its activation
    operand (python/tessera/__init__.py:592-616); the hidden activation stays fp32 in between."""
    xa = _unwrap(x)
    if len(xa.shape) != 2:
        raise ValueError("moe_swiglu_block: expected x (T,K)")
    T, K = xa.shape
    on_device = isinstance(xa, DeviceArray)
    gd, ud, dd = (_fp4_weights(w, stream) for w in (w_gate, w_up, w_down))
    E, Kw, F = gd.shape
    if ud.shape != gd.shape or dd.shape[0] != E or dd.shape[1] != F or Kw != K:
        raise ValueError(f"moe_swiglu_block: shape mismatch x {tuple(xa.shape)}, w_gate {gd.shape}, "
                         f"w_down {dd.shape}")
    N = dd.shape[2]
    off = _group_offsets(group_sizes, T, "moe_swiglu_block")
    if off.shape[0] != E + 1:
        raise ValueError(f"moe_swiglu_block: len(group_sizes)={off.shape[0] - 1} != E={E}")
    sh = device._stream_handle(stream)
    doff = DeviceArray.from_host(off, pooled=True)
    xv, xs = _fp4_operand(xa, act, stream)
    hidden = DeviceArray((T, F), np.float32, pooled=True)
    _lib.call("tessera_sm100_grouped_swiglu_scaled_device", xv.ptr, gd.ptr, ud.ptr, doff.ptr, hidden.ptr, T, K, F, E,
              _lib.BF16, _lib.F32, xs.ptr if xs is not None else None, sh)
    hv, hs = _fp4_operand(hidden, act, stream)
    odt = np.dtype(xa.dtype)
    out = DeviceArray((T, N), odt)
    _lib.call("tessera_sm100_grouped_gemm_scaled_device", hv.ptr, dd.ptr, doff.ptr, out.ptr, T, F, N, E, _lib.BF16,
              device.dtype_code(odt), hs.ptr if hs is not None else None, sh)
    return out if on_device else _finish(out)


def _grouped_gemm_fp8(x, weights, group_sizes, out_dtype, stream, fmt=None):
    xa = _unwrap(x)
    if len(xa.shape) != 2:
        raise ValueError(f"grouped_gemm: x must be (T, K); got {tuple(xa.shape)}")
    if fmt is None:
        fmt = weights.fmt if isinstance(weights, Fp8Tensor) else 0
    wq = _as_fp8_experts(weights, fmt, stream)
    E, K, N = wq.shape
    T = xa.shape[0]
    if xa.shape[1] != K:
        raise ValueError(f"grouped_gemm: K mismatch — x K={xa.shape[1]}, weights K={K}")
    off = _group_offsets(group_sizes, T, "grouped_gemm")
    if off.shape[0] != E + 1:
        raise ValueError(f"grouped_gemm: weights {wq.shape} must be (E, K, N) with E == len(group_sizes)="
                         f"{off.shape[0] - 1}")
    if K % 16 or N % 8:
        raise ValueError("grouped_gemm: the fp8 path needs K a multiple of 16 and N a multiple of 8")
    on_device = isinstance(xa, DeviceArray)
    xq = quantize_fp8_activations(xa, format=fmt, stream=stream)
    odt = np.dtype(out_dtype) if out_dtype is not None else np.dtype(xa.dtype)
    out = DeviceArray((T, N), odt)      # group sizes sum to T: every row is written
    doff = DeviceArray.from_host(off, pooled=True)
    _lib.call("tessera_sm100_grouped_gemm_fp8_fmt_device", xq.q.ptr, wq.q.ptr, doff.ptr, out.ptr, T, K, N, E,
              xq.scales.ptr, wq.scales.ptr, device.dtype_code(odt), fmt, device._stream_handle(stream))
    return out if on_device else _finish(out)


def grouped_gemm(x, weights, group_sizes, *, kind="contiguous", alignment=None, quant=None,
                 out_dtype=None, stream=None):
    """Ragged grouped matmul: row block e of ``x`` (T, K) times ``weights[e]`` (E, K, N)
    (python/tessera/__init__.py:291-351). Output dtype follows ``x``. ``quant="fp8_e4m3"`` quantises
    ``x`` per tensor and each expert's weights per expert and multiplies the e4m3 values on the
    tensor cores (the reference dequantises on the host and multiplies in f32); ``weights`` may be
    an :class:`Fp8Tensor` from :func:`quantize_fp8_experts`."""
    _check_kind(kind, alignment, group_sizes, quant, "grouped_gemm")
    if isinstance(weights, Nvfp4Tensor) or (quant is not None and str(quant).lower() in _FP4_QUANTS):
        act = _FP4_QUANTS[str(quant).lower()] if quant is not None else 0
        return _grouped_gemm_fp4(x, weights, group_sizes, act, out_dtype, stream)
    if quant is not None or isinstance(weights, Fp8Tensor):
        return _grouped_gemm_fp8(x, weights, group_sizes, out_dtype, stream,
                                 _FP8_QUANTS[str(quant).lower()] if quant is not None else None)
    x, w = _unwrap(x), _unwrap(weights)
    if x.ndim != 2:
        raise ValueError(f"grouped_gemm: x must be (T, K); got {x.shape}")
    gs_len = np.asarray(group_sizes).reshape(-1).shape[0]
    if w.ndim != 3 or w.shape[0] != gs_len:
        raise ValueError(f"grouped_gemm: weights {w.shape} must be (E, K, N) with "
                         f"E == len(group_sizes)={gs_len}")
    if w.shape[1] != x.shape[1]:
        raise ValueError(f"grouped_gemm: K mismatch — x K={x.shape[1]}, weights K={w.shape[1]}")
    T, K = x.shape
    E, _, N = w.shape
    off = _group_offsets(group_sizes, T, "grouped_gemm")
    dt = _storage_dtype((x, w), None, "grouped_gemm")
    out_code = _out_code(out_dtype, device.dtype_code(dt))
    on_device = _any_device(x, w)
    dx, dw = _to_device(x, dt), _to_device(w, dt)
    doff = DeviceArray.from_host(off)
    out = DeviceArray.zeros((T, N), device.code_dtype(out_code))
    _lib.call("tessera_sm100_grouped_gemm_device", dx.ptr, dw.ptr, doff.ptr, out.ptr, T, K, N, E,
              device.dtype_code(dt), out_code, device._stream_handle(stream))
    return out if on_device else _finish(out)


def _finish(out: DeviceArray) -> np.ndarray:
    host = out.download()
    device.check_device_error("kernel")
    return host


def silu_mul(a, b, *, stream=None):
    """``silu(a) * b`` elementwise (python/tessera/__init__.py:559-574)."""
    a, b = _unwrap(a), _unwrap(b)
    if a.shape != b.shape:
        raise ValueError(f"silu_mul: shape mismatch {a.shape} vs {b.shape}")
    on_device = _any_device(a, b)
    dt = np.dtype(a.dtype)
    da, db = _to_device(a, dt), _to_device(b, dt)
    out = DeviceArray(a.shape, dt)
    _lib.call("tessera_sm100_silu_mul_device", da.ptr, db.ptr, out.ptr, int(da.size),
              device.dtype_code(dt), device._stream_handle(stream))
    return out if on_device else _finish(out)


def moe_swiglu_block(x, w_gate, w_up, w_down, group_sizes, *, kind="contiguous", alignment=None,
                     quant=None, stream=None):
    """Expert FFN over grouped tokens: gate and up grouped GEMMs fused with ``silu_mul`` in one
    kernel, then the down grouped GEMM (python/tessera/__init__.py:592-616)."""
    _check_kind(kind, alignment, group_sizes, quant, "moe_swiglu_block")
    if isinstance(w_gate, Nvfp4Tensor) or (quant is not None and str(quant).lower() in _FP4_QUANTS):
        act = _FP4_QUANTS[str(quant).lower()] if quant is not None else 0
        return _moe_swiglu_block_fp4(x, w_gate, w_up, w_down, group_sizes, act, stream)
    if quant is not None or isinstance(w_gate, Fp8Tensor):
        return _moe_swiglu_block_fp8(x, w_gate, w_up, w_down, group_sizes, stream,
                                     _FP8_QUANTS[str(quant).lower()] if quant is not None else None)
    x, wg, wu, wd = _unwrap(x), _unwrap(w_gate), _unwrap(w_up), _unwrap(w_down)
    if x.ndim != 2 or wg.ndim != 3 or wu.shape != wg.shape or wd.ndim != 3:
        raise ValueError("moe_swiglu_block: expected x (T,K), w_gate/w_up (E,K,F), w_down (E,F,N)")
    T, K = x.shape
    E, Kw, F = wg.shape
    if Kw != K or wd.shape[0] != E or wd.shape[1] != F:
        raise ValueError(f"moe_swiglu_block: shape mismatch x {x.shape}, w_gate {wg.shape}, "
                         f"w_down {wd.shape}")
    N = wd.shape[2]
    off = _group_offsets(group_sizes, T, "moe_swiglu_block")
    if off.shape[0] != E + 1:
        raise ValueError(f"moe_swiglu_block: len(group_sizes)={off.shape[0] - 1} != E={E}")
    dt = _storage_dtype((x, wg, wu, wd), None, "moe_swiglu_block")
    code = device.dtype_code(dt)
    on_device = _any_device(x, wg, wu, wd)
    dx, dg, du, dd = (_to_device(t, dt) for t in (x, wg, wu, wd))
    doff = DeviceArray.from_host(off)
    hidden = DeviceArray.zeros((T, F), dt)
    out = DeviceArray.zeros((T, N), dt)
    sh = device._stream_handle(stream)
    _lib.call("tessera_sm100_grouped_swiglu_device", dx.ptr, dg.ptr, du.ptr, doff.ptr, hidden.ptr, T,
              K, F, E, code, code, sh)
    _lib.call("tessera_sm100_grouped_gemm_device", hidden.ptr, dd.ptr, doff.ptr, out.ptr, T, F, N, E,
              code, code, sh)
    return out if on_device else _finish(out)


def _moe_swiglu_block_fp8(x, w_gate, w_up, w_down, group_sizes, stream, fmt=None):
    """fp8 expert FFN: x quantised once, gate and up GEMMs fused with silu_mul (16-bit hidden plus its
    amax from the epilogue), hidden quantised per tensor, down GEMM — the reference applies ``quant``
    to every grouped GEMM of the block (python/tessera/__init__.py:592-616)."""
    xa = _unwrap(x)
    if len(xa.shape) != 2:
        raise ValueError("moe_swiglu_block: expected x (T,K)")
    if fmt is None:
        fmt = w_gate.fmt if isinstance(w_gate, Fp8Tensor) else 0
    gq, uq, dq = (_as_fp8_experts(w, fmt, stream) for w in (w_gate, w_up, w_down))
    E, K, F = gq.shape
    if uq.shape != gq.shape or dq.shape[0] != E or dq.shape[1] != F or xa.shape[1] != K:
        raise ValueError(f"moe_swiglu_block: shape mismatch x {tuple(xa.shape)}, w_gate {gq.shape}, "
                         f"w_down {dq.shape}")
    N = dq.shape[2]
    T = xa.shape[0]
    off = _group_offsets(group_sizes, T, "moe_swiglu_block")
    if off.shape[0] != E + 1:
        raise ValueError(f"moe_swiglu_block: len(group_sizes)={off.shape[0] - 1} != E={E}")
    if K % 16 or F % 16 or N % 8:
        raise ValueError("moe_swiglu_block: the fp8 path needs K and F multiples of 16 and N of 8")
    on_device = isinstance(xa, DeviceArray)
    odt = np.dtype(xa.dtype)
    # The hidden activation stays fp32 between the two GEMMs: e4m3 keeps 3 mantissa bits, so rounding
    # it to 16 bits first would move about one element in 32 across a quantisation boundary.
    hdt = np.dtype(np.float32)
    sh = device._stream_handle(stream)
    xq = quantize_fp8_activations(xa, format=fmt, stream=stream)
    doff = DeviceArray.from_host(off, pooled=True)
    hidden = DeviceArray((T, F), hdt, pooled=True)
    amax = DeviceArray.zeros((1,), np.uint32)
    _lib.call("tessera_sm100_grouped_swiglu_fp8_fmt_device", xq.q.ptr, gq.q.ptr, uq.q.ptr, doff.ptr, hidden.ptr, T,
              K, F, E, xq.scales.ptr, gq.scales.ptr, uq.scales.ptr, device.dtype_code(hdt), amax.ptr, fmt, sh)
    hq = quantize_fp8_activations(hidden, amax_bits=amax, format=fmt, stream=stream)
    out = DeviceArray((T, N), odt)
    _lib.call("tessera_sm100_grouped_gemm_fp8_fmt_device", hq.q.ptr, dq.q.ptr, doff.ptr, out.ptr, T, F, N, E,
              hq.scales.ptr, dq.scales.ptr, device.dtype_code(odt), fmt, sh)
    return out if on_device else _finish(out)


def swiglu(x, W_gate, W_up, W_down, *, stream=None):
    """Dense SwiGLU MLP ``(silu(x Wg) * (x Wu)) Wd`` (python/tessera/__init__.py:576-590), run as a
    one-expert ``moe_swiglu_block`` so gate, up and the activation share a kernel."""
    x_, wg, wu, wd = _unwrap(x), _unwrap(W_gate), _unwrap(W_up), _unwrap(W_down)
    lead = x_.shape[:-1]
    x2 = x_.reshape((-1, x_.shape[-1]))
    out = moe_swiglu_block(x2, wg.reshape((1,) + tuple(wg.shape)), wu.reshape((1,) + tuple(wu.shape)),
                           wd.reshape((1,) + tuple(wd.shape)), [x2.shape[0]], stream=stream)
    return out.reshape(tuple(lead) + (wd.shape[-1],)) if isinstance(out, np.ndarray) else out


def moe_layer_from_logits(x, logits, W_gate, W_up, W_down, *, top_k: int = 1,
                          normalize_weights: bool = True, capacity: Optional[int] = None,
                          out_dtype=None, return_routing: bool = False):
    """Route (given router logits) -> permute -> expert FFN -> combine, all on the GPU. Returns
    the (T, N) output, plus a dict of routing products when ``return_routing`` is set."""
    x, wg, wu, wd = _unwrap(x), _unwrap(W_gate), _unwrap(W_up), _unwrap(W_down)
    logits = np.ascontiguousarray(_unwrap(logits), dtype=np.float32)
    T, H = x.shape
    E, Hw, F = wg.shape
    if Hw != H or wu.shape != wg.shape or wd.shape != (E, F, H) or logits.shape != (T, E):
        raise ValueError(f"moe_layer: shape mismatch x {x.shape}, logits {logits.shape}, w_gate "
                         f"{wg.shape}, w_up {wu.shape}, w_down {wd.shape}")
    if not 1 <= top_k <= E:
        raise ValueError(f"top_k must be in [1, num_experts={E}], got {top_k}")
    dt = _storage_dtype((x, wg, wu, wd), None, "moe_layer")
    code = device.dtype_code(dt)
    out_code = _out_code(out_dtype, code)
    xh, g, u, d = (np.ascontiguousarray(t) for t in (x, wg, wu, wd))
    out = np.empty((T, H), device.code_dtype(out_code))
    assignment = np.empty((T, top_k), np.int32)
    weights = np.empty((T, top_k), np.float32)
    group_sizes = np.empty((E,), np.int32)
    token_of_slot = np.empty((T * top_k,), np.int32)
    _lib.call("tessera_sm100_moe_layer", xh.ctypes.data, logits.ctypes.data, g.ctypes.data,
              u.ctypes.data, d.ctypes.data, out.ctypes.data, T, H, F, E, int(top_k),
              int(bool(normalize_weights)), -1 if capacity is None else int(capacity), code, out_code,
              assignment.ctypes.data, weights.ctypes.data, group_sizes.ctypes.data,
              token_of_slot.ctypes.data)
    if not return_routing:
        return out
    kept = int(group_sizes.sum())
    return out, dict(assignment=assignment.astype(np.int64), weights=weights,
                     group_sizes=group_sizes, token_of_slot=token_of_slot[:kept])


_RUNTIME_KERNELS: dict[str, Any] = {}


def register_runtime_kernel(name: str, fn) -> None:
    """Op registry seam (python/tessera/__init__.py:182-186): expose ``fn`` as ``ops.<name>``."""
    if not callable(fn):
        raise TypeError("runtime kernel must be callable")
    _RUNTIME_KERNELS[name] = fn
    globals()[name] = fn
