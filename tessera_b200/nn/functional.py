"""``tessera.nn.functional`` entries on the hot path (python/tessera/nn/functional.py:349-490)."""
from __future__ import annotations

import numpy as np

from .. import ops


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
