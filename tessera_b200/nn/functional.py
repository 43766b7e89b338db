"""``tessera.nn.functional`` entries on the hot path (python/tessera/nn/functional.py:349-490)."""
from __future__ import annotations

import numpy as np

import ctypes

from .. import _lib, device, ops
from ..device import DeviceArray, StridedView, bfloat16, slice_last


def linear(x, W, bias=None, *, out_dtype=None, activation: str = "linear"):
    """``y = x @ W (+ bias)`` over the last dimension of ``x`` (python/tessera/nn/functional.py:33-44),
    bias (and an optional activation) applied inside the GEMM kernel. ``x`` may be ``[..., K]``, host
    or device; the result keeps ``x``'s storage dtype unless ``out_dtype`` says otherwise, so layers
    chain without conversions."""
    xa = ops._unwrap(x)
    lead = tuple(xa.shape[:-1])
    K = xa.shape[-1]
    if isinstance(xa, DeviceArray):
        x2 = xa.view((int(np.prod(lead, dtype=np.int64)), K))
    else:
        x2 = np.asarray(xa).reshape(-1, K)
    odt = out_dtype if out_dtype is not None else xa.dtype
    if bias is None and activation == "linear":
        y = ops.gemm(x2, W, out_dtype=odt)
    else:
        ep = {"activation": activation}
        if bias is not None:
            ep["bias"] = ops._unwrap(bias)
        y = ops.gemm(x2, W, epilogue=ep, out_dtype=odt)
    N = y.shape[-1]
    return y.view(lead + (N,)) if isinstance(y, DeviceArray) else y.reshape(lead + (N,))


def split_last(x, sizes):
    """``x[..., a:b]`` windows of consecutive widths ``sizes`` — views for a device array (nothing is
    copied; the strided attention call reads them in place), slices for a host array."""
    xa = ops._unwrap(x)
    out, a = [], 0
    for n in sizes:
        out.append(slice_last(xa, a, a + n) if isinstance(xa, (DeviceArray, StridedView)) else xa[..., a:a + n])
        a += n
    if a != xa.shape[-1]:
        raise ValueError(f"split_last: sizes sum to {a}, last dimension is {xa.shape[-1]}")
    return out


def _bsx_strides(t, heads: int, D: int):
    """(batch, head, position) element strides of a [B, S, heads*D] operand."""
    if isinstance(t, StridedView):
        return (t.strides[0], D, t.strides[1])
    return (t.shape[1] * heads * D, D, heads * D)


def multi_head_attention(Q, K, V, num_heads: int, scale=None, causal: bool = False, dropout_p: float = 0.0,
                         seed=None, *, num_kv_heads=None, stream=None):
    """Attention over ``[B, S, H*D]`` operands (python/tessera/nn/functional.py:493-548). The
    reference reshapes to ``[B, H, S, D]``, calls ``ops.flash_attn`` and transposes back; here the
    kernels read and write the ``[B, S, H, D]`` layout directly through strided tensor maps, so
    nothing is transposed. ``num_kv_heads`` (default ``num_heads``) allows grouped-query K/V of
    width ``num_kv_heads * D``. Device operands may be views made by :func:`split_last`."""
    if dropout_p:
        raise NotImplementedError("multi_head_attention: dropout is not part of this backend")
    q, k, v = (ops._unwrap(t) for t in (Q, K, V))
    if q.ndim != 3 or k.ndim != 3 or v.ndim != 3:
        raise ValueError("multi_head_attention expects [B, S, H*D] inputs; for raw [B, H, S, D] tensors, "
                         "call tessera.ops.flash_attn directly")
    Hkv = int(num_kv_heads) if num_kv_heads else int(num_heads)
    B, Sq, hd = q.shape
    Sk = k.shape[1]
    if k.shape[0] != B or v.shape[0] != B:
        raise ValueError("Q/K/V must share batch dim")
    if v.shape[1] != Sk:
        raise ValueError(f"K and V must share sequence length; got {Sk} vs {v.shape[1]}")
    if hd % num_heads:
        raise ValueError(f"hidden dim {hd} not divisible by num_heads {num_heads}")
    D = hd // num_heads
    if k.shape[2] != Hkv * D or v.shape[2] != Hkv * D:
        raise ValueError("Q/K/V must share hidden dim" if Hkv == num_heads else
                         f"K/V hidden dim must be num_kv_heads*D = {Hkv * D}")
    if num_heads % Hkv:
        raise ValueError("num_heads must be divisible by num_kv_heads")
    if D != 128:
        raise ValueError(f"multi_head_attention: head dimension must be 128 on this backend; got {D}")
    on_device = any(isinstance(t, (DeviceArray, StridedView)) for t in (q, k, v))

    def dev(t):
        if isinstance(t, (DeviceArray, StridedView)):
            if t.dtype != bfloat16:
                raise TypeError("multi_head_attention: device operands must be bfloat16")
            return t
        return DeviceArray.from_host(np.ascontiguousarray(t).astype(bfloat16), pooled=True)

    dq, dk, dv = dev(q), dev(k), dev(v)
    out = DeviceArray((B, Sq, hd), bfloat16)
    arr = lambda t: (ctypes.c_longlong * 3)(*t)
    sc = float(1.0 / np.sqrt(D) if scale is None else scale)
    _lib.call("tessera_sm100_flash_attn_strided_device", dq.ptr, dk.ptr, dv.ptr, out.ptr, B, num_heads, Hkv, Sq,
              Sk, D, arr(_bsx_strides(dq, num_heads, D)), arr(_bsx_strides(dk, Hkv, D)),
              arr(_bsx_strides(dv, Hkv, D)), arr(_bsx_strides(out, num_heads, D)), sc, int(bool(causal)),
              device._stream_handle(stream))
    if on_device:
        return out
    host = out.download()
    device.check_device_error("multi_head_attention")
    return host


def gqa_attention(Q, K, V, num_query_heads: int, num_kv_heads: int, **kwargs):
    return ops.gqa_attention(Q, K, V, num_query_heads, num_kv_heads, **kwargs)


def mqa_attention(Q, K, V, **kwargs):
    return ops.mqa_attention(Q, K, V, **kwargs)


def swiglu(x, W_gate, W_up, W_down):
    return ops.swiglu(x, W_gate, W_up, W_down)


def moe_layer(x, W_router, W_gate, W_up, W_down, *, top_k: int = 1, normalize_weights: bool = True,
              capacity_factor: float = 0.0, kind: str = "contiguous", alignment=None, quant=None):
    """Single-device top-k SwiGLU MoE layer: router GEMM -> top-k -> permute -> expert FFN ->
    combine (python/tessera/nn/functional.py:403-490), every step on the GPU. ``capacity_factor
    <= 0`` means no capacity drop, as in the reference (:447-452)."""
    if kind not in ops.SUPPORTED_GROUPED_KINDS or quant is not None or alignment is not None:
        raise NotImplementedError("moe_layer: only the contiguous, unquantised layout is implemented")
    xa = ops._unwrap(x)
    logits = np.asarray(ops.gemm(xa, W_router), dtype=np.float32)
    T, E = logits.shape
    capacity = None
    if capacity_factor > 0:
        capacity = int(np.ceil(capacity_factor * T / max(1, E)))
    return ops.moe_layer_from_logits(xa, logits, W_gate, W_up, W_down, top_k=top_k,
                                     normalize_weights=normalize_weights, capacity=capacity)
