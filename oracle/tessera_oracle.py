"""CPU oracle for the dense-contraction hot path. TEST INFRASTRUCTURE ONLY.

This module restates, in plain numpy, what the reference's CPU path computes for GEMM,
flash attention (prefill and GQA decode) and the MoE layer. It is the checker the parity
tests and the benchmark's CPU-baseline leg use; nothing in ``tessera_b200`` imports it and it
must never be on a product path.

Parity status: PINNED. ``tests/golden/*.npz`` were produced by importing the reference package
itself (``tests/golden/make_golden.py``) and ``tests/test_oracle_golden.py`` checks every
function here against them.

Each function cites the reference file:line it follows (paths relative to the reference
project root).
"""
from __future__ import annotations

from typing import NamedTuple, Optional

import numpy as np

try:
    import ml_dtypes

    _BF16 = np.dtype(ml_dtypes.bfloat16)
except Exception:  # pragma: no cover
    ml_dtypes = None
    _BF16 = None


# ----------------------------------------------------------------------------- storage rounding
def round_to_storage(x, dtype: str) -> np.ndarray:
    """Round f32 ``x`` to 16-bit storage and back (python/tessera/compiler/fusion_core.py:348-362)."""
    a = np.ascontiguousarray(x, np.float32)
    if dtype in ("float16", "f16"):
        return a.astype(np.float16).astype(np.float32)
    if dtype in ("bfloat16", "bf16"):
        if _BF16 is not None:
            return a.astype(_BF16).astype(np.float32)
        u = a.view(np.uint32).astype(np.uint64)
        bits = (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16).astype(np.uint32)
        return bits.view(np.float32)
    if dtype in ("float32", "f32"):
        return a
    raise ValueError(f"unsupported storage dtype {dtype!r}")


def storage_name(arr) -> str:
    dt = np.asarray(arr).dtype
    if dt == np.float16:
        return "f16"
    if _BF16 is not None and dt == _BF16:
        return "bf16"
    return "f32"


def _f32(x) -> np.ndarray:
    return np.asarray(x).astype(np.float32)


# ----------------------------------------------------------------------------- GEMM
def gemm(A, B) -> np.ndarray:
    """``A @ B`` with leading dims broadcast as batch; 16-bit operands are taken at their stored
    values and multiplied in f32 (python/tessera/__init__.py:239-254 ``gemm``/``batched_gemm``;
    f32 accumulation of rounded operands as in ``MatmulRegion.reference``,
    python/tessera/compiler/fusion_core.py:398-405)."""
    return np.matmul(_f32(A), _f32(B)).astype(np.float32)


def fused_epilogue(x, bias=None, activation="linear", residual=None) -> np.ndarray:
    """bias, residual, then activation (python/tessera/__init__.py:2658-2675; gelu is the tanh
    form of :487-497, silu :554-557, relu :549-552), in f32."""
    x = np.asarray(x, np.float32)
    if bias is not None:
        x = x + np.asarray(bias, np.float32)
    if residual is not None:
        x = x + _f32(residual)
    if activation == "gelu":
        k = float(np.sqrt(2.0 / np.pi))
        x = x * 0.5 * (1.0 + np.tanh(k * (x + 0.044715 * x ** 3)))
    elif activation == "relu":
        x = np.maximum(0, x)
    elif activation == "silu":
        x = x / (1.0 + np.exp(-x))
    return x.astype(np.float32)


def gated_matmul(A, Wg, Wu) -> np.ndarray:
    """``silu(A @ Wg) * (A @ Wu)`` (``GatedMatmulRegion.reference``,
    python/tessera/compiler/fusion_core.py:773-781)."""
    a = _f32(A)
    g = a @ _f32(Wg)
    return ((g / (1.0 + np.exp(-g))) * (a @ _f32(Wu))).astype(np.float32)


def attention_region(Q, K, V, scale: float = 1.0, causal: bool = False) -> np.ndarray:
    """Single-head ``softmax(scale Q K^T) V`` with keys ``n > m`` masked when causal
    (``AttentionRegion.reference``, python/tessera/compiler/fusion_core.py:672-727)."""
    s = (_f32(Q) @ _f32(K).T) * np.float32(scale)
    if causal:
        m = np.arange(s.shape[0])[:, None]
        n = np.arange(s.shape[1])[None, :]
        s = np.where(n > m, -np.inf, s)
    return (softmax(s) @ _f32(V)).astype(np.float32)


# ----------------------------------------------------------------------------- attention
def softmax(x, axis: int = -1) -> np.ndarray:
    """python/tessera/__init__.py:450-454."""
    e = np.exp(x - x.max(axis=axis, keepdims=True))
    return e / e.sum(axis=axis, keepdims=True)


def flash_attn(Q, K, V, scale: Optional[float] = None, causal: bool = False,
               q_block: int = 1024) -> np.ndarray:
    """``softmax(scale * Q K^T, causal) V`` per (batch, head), f32 math
    (python/tessera/__init__.py:1304-1356). The causal mask is bottom-right aligned:
    key j is masked for query i when ``j > i + max(Sk - Sq, 0)`` (``np.triu(k=1+max(Sk-Sq,0))``,
    :1344-1349). The reference materialises the whole [B,H,Sq,Sk] score tensor; this walks
    (b, h) slices and query blocks instead, which changes memory use but not a single value.
    """
    Q, K, V = _f32(Q), _f32(K), _f32(V)
    B, H, Sq, D = Q.shape
    Sk = K.shape[-2]
    if scale is None:
        scale = 1.0 / np.sqrt(D)
    scale = np.float32(scale)
    out = np.empty((B, H, Sq, V.shape[-1]), np.float32)
    shift = max(Sk - Sq, 0)
    for b in range(B):
        for h in range(H):
            kT = K[b, h].T
            for q0 in range(0, Sq, q_block):
                q1 = min(Sq, q0 + q_block)
                scores = np.matmul(Q[b, h, q0:q1], kT) * scale
                if causal:
                    i = np.arange(q0, q1)[:, None]
                    j = np.arange(Sk)[None, :]
                    scores = np.where(j > i + shift, -np.inf, scores)
                out[b, h, q0:q1] = np.matmul(softmax(scores), V[b, h])
    return out


def attention_lane(q, k, v, *, scale, causal: bool = False, window=None, bias=None, softcap=None,
                   causal_shift: int = 0) -> np.ndarray:
    """The CUDA attention lane's contract (python/tessera/compiler/emit/nvidia_cuda.py:251-276), as
    the reference's device test restates it (tests/device/nvidia/test_flash_attention.py:23-58):
    ``s = scale q.k (+ bias)``, ``s = softcap tanh(s / softcap)``, keys ``n > m + causal_shift``
    (causal), ``n < m - wl``, ``n > m + wr`` masked (the mask wins over the soft-cap), softmax, ``@ v``;
    ``hk = hq // (Hq / Hkv)``; ``D`` and ``Dv`` may differ; a fully masked row gives zeros.
    ``causal_shift`` 0 is the lane (top-left); ``max(Sk - Sq, 0)`` is ``ops.flash_attn``."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    B, Hq, Sq, D = q.shape
    _, Hkv, Sk, _ = k.shape
    rep = Hq // Hkv
    if window is None:
        wl = wr = None
    elif isinstance(window, (tuple, list)):
        wl, wr = window
    else:
        wl = wr = window
    m = np.arange(Sq)[:, None]
    n = np.arange(Sk)[None, :]
    keep = np.ones((Sq, Sk), bool)
    if causal:
        keep &= n <= m + causal_shift
    if wl is not None and wl >= 0:
        keep &= n >= m - wl
    if wr is not None and wr >= 0:
        keep &= n <= m + wr
    out = np.zeros((B, Hq, Sq, v.shape[-1]), np.float32)
    for b in range(B):
        for hq in range(Hq):
            hk = hq // rep
            s = (q[b, hq] @ k[b, hk].T) * np.float32(scale)
            if bias is not None:
                s = s + np.asarray(bias, np.float32)[b, hq]
            if softcap:
                s = softcap * np.tanh(s / softcap)
            s = np.where(keep, s, -np.inf)
            mx = s.max(-1, keepdims=True)
            mx = np.where(np.isfinite(mx), mx, 0.0)
            p = np.exp(s - mx)
            den = p.sum(-1, keepdims=True)
            out[b, hq] = (p / np.where(den > 0, den, 1.0)) @ v[b, hk]
    return out


def attention_lane_backward(do, q, k, v, *, scale, causal: bool = False, window=None, bias=None,
                            softcap=None, causal_shift: int = 0):
    """Gradients ``(dQ, dK, dV)`` of :func:`attention_lane`: the CUDA backward lane's contract
    (python/tessera/compiler/emit/nvidia_cuda.py:590-635) as the reference's device test restates it
    (tests/device/nvidia/test_flash_attention_backward.py:23-50): ``p`` = softmax over the legal
    keys, ``delta = dO . o``, ``ds = p (dO . v - delta) (1 - tanh^2(raw / softcap))``,
    ``dQ += ds scale k``, ``dK += ds scale q`` and ``dV += p dO`` summed over the query heads of a
    KV head; a row with no legal key contributes nothing (the device lane's ``z > 0`` guard)."""
    do, q, k, v = _f32(do), _f32(q), _f32(k), _f32(v)
    B, Hq, Sq, D = q.shape
    _, Hkv, Sk, _ = k.shape
    rep = Hq // Hkv
    if window is None:
        wl = wr = None
    elif isinstance(window, (tuple, list)):
        wl, wr = window
    else:
        wl = wr = window
    m = np.arange(Sq)[:, None]
    n = np.arange(Sk)[None, :]
    keep = np.ones((Sq, Sk), bool)
    if causal:
        keep &= n <= m + causal_shift
    if wl is not None and wl >= 0:
        keep &= n >= m - wl
    if wr is not None and wr >= 0:
        keep &= n <= m + wr
    dq, dk, dv = np.zeros_like(q), np.zeros_like(k), np.zeros_like(v)
    sc = np.float32(scale)
    for b in range(B):
        for hq in range(Hq):
            hk = hq // rep
            raw = (q[b, hq] @ k[b, hk].T) * sc
            if bias is not None:
                raw = raw + np.asarray(bias, np.float32)[b, hq]
            deriv = np.ones_like(raw)
            s = raw
            if softcap:
                t = np.tanh(raw / softcap)
                s = softcap * t
                deriv = 1 - t * t
            s = np.where(keep, s, -np.inf)
            mx = s.max(-1, keepdims=True)
            mx = np.where(np.isfinite(mx), mx, 0.0)
            e = np.exp(s - mx)
            den = e.sum(-1, keepdims=True)
            p = e / np.where(den > 0, den, 1.0)
            dp = do[b, hq] @ v[b, hk].T
            delta = (p * dp).sum(-1, keepdims=True)
            ds = p * (dp - delta) * deriv
            dq[b, hq] = (ds @ k[b, hk]) * sc
            dk[b, hk] += (ds.T @ q[b, hq]) * sc
            dv[b, hk] += p.T @ do[b, hq]
    return dq, dk, dv


def gqa_attention(Q, K, V, num_query_heads: int, num_kv_heads: int, **kwargs) -> np.ndarray:
    """Query head ``hq`` reads KV head ``hq // (Hq/Hkv)``: the reference repeats each KV head
    ``Hq/Hkv`` times along the head axis and calls ``flash_attn``
    (python/tessera/nn/functional.py:345-356)."""
    if num_query_heads % num_kv_heads != 0:
        raise ValueError("num_query_heads must be divisible by num_kv_heads")
    rep = num_query_heads // num_kv_heads
    return flash_attn(Q, np.repeat(np.asarray(K), rep, axis=1), np.repeat(np.asarray(V), rep, axis=1),
                      **kwargs)


def multi_head_attention(Q, K, V, num_heads: int, scale=None, causal: bool = False,
                         num_kv_heads: Optional[int] = None) -> np.ndarray:
    """``[B, S, H*D]`` operands: reshape to ``[B, H, S, D]``, ``flash_attn``, transpose back
    (python/tessera/nn/functional.py:493-548). ``num_kv_heads`` (not in the reference, which takes
    equal widths) repeats K/V heads as ``gqa_attention`` does."""
    Q, K, V = _f32(Q), _f32(K), _f32(V)
    B, Sq, hd = Q.shape
    D = hd // num_heads
    Hkv = num_kv_heads or num_heads

    def split(t, h):
        return t.reshape(B, t.shape[1], h, D).transpose(0, 2, 1, 3)

    q, k, v = split(Q, num_heads), split(K, Hkv), split(V, Hkv)
    if Hkv != num_heads:
        out = gqa_attention(q, k, v, num_heads, Hkv, scale=scale, causal=causal)
    else:
        out = flash_attn(q, k, v, scale=scale, causal=causal)
    return np.ascontiguousarray(out.transpose(0, 2, 1, 3)).reshape(B, Sq, hd)


def linear(x, W, bias=None) -> np.ndarray:
    """``x @ W (+ bias)`` (python/tessera/nn/functional.py:33-44)."""
    y = np.matmul(_f32(x), _f32(W))
    return (y + np.asarray(bias, np.float32)).astype(np.float32) if bias is not None else y.astype(np.float32)


def softmax_merge(oa, ma, la, ob, mb, lb):
    """Associative merge of two max-shifted partial attention states
    (python/tessera/_block_attnres_ops.py:104-131)."""
    m = np.maximum(ma, mb)
    sa = np.exp(ma - m).astype(np.float32)
    sb = np.exp(mb - m).astype(np.float32)
    return ((sa[..., None] * oa + sb[..., None] * ob).astype(np.float32), m.astype(np.float32),
            (sa * la + sb * lb).astype(np.float32))


def softmax_finalize(o, l) -> np.ndarray:
    """python/tessera/_block_attnres_ops.py:134-146."""
    return np.asarray(o / l[..., None], dtype=np.float32)


# ----------------------------------------------------------------------------- fp8 quantisation
def quantize_fp8(x, format: str = "e4m3"):
    """Per-tensor symmetric 8-bit float quantisation, returned dequantised: ``scale =
    max(amax/max_normal, 1e-12)`` with ``max_normal`` 448 (e4m3) or 57344 (e5m2), ``q =
    fp8(clip(x/scale, -max_normal, max_normal))``, result ``q * scale`` and ``scale``, all in
    float32 (python/tessera/__init__.py:3340-3374)."""
    x = np.asarray(x, np.float32)
    top, dt = {"e4m3": (448.0, ml_dtypes.float8_e4m3fn), "e5m2": (57344.0, ml_dtypes.float8_e5m2)}[format]
    amax = np.max(np.abs(x)) if x.size else np.float32(0)
    scale = np.float32(np.maximum(np.float32(amax) / np.float32(top), np.float32(1e-12)))
    scaled = np.clip(x / scale, -top, top)
    q = scaled.astype(dt).astype(np.float32)
    return (q * scale).astype(np.float32), scale


def grouped_gemm_fp8(x, w, group_sizes, format: str = "e4m3") -> np.ndarray:
    """``grouped_gemm(..., quant="fp8_e4m3")``: x quantised per tensor, each expert's weights per
    expert, then the f32 grouped GEMM (python/tessera/__init__.py:337-351,
    python/tessera/compiler/grouped_layout.py:371-392)."""
    xq = quantize_fp8(_f32(x), format)[0]
    wq = np.stack([quantize_fp8(_f32(w)[e], format)[0] for e in range(np.asarray(w).shape[0])])
    return grouped_gemm(xq, wq, group_sizes)


def moe_swiglu_block_fp8(x, w_gate, w_up, w_down, group_sizes, format: str = "e4m3") -> np.ndarray:
    """``moe_swiglu_block(..., quant="fp8_e4m3")``: every grouped GEMM of the block quantises its
    operands (python/tessera/__init__.py:592-616)."""
    gate = grouped_gemm_fp8(x, w_gate, group_sizes, format)
    up = grouped_gemm_fp8(x, w_up, group_sizes, format)
    return grouped_gemm_fp8(silu_mul(gate, up), w_down, group_sizes, format)


def quantize_nvfp4(x, block_size: int = 16):
    """NVFP4 along the last axis: per block of 16, ``scale = e4m3(max(amax/6, 1e-30))`` and
    ``code = e2m1(x / (scale or 1))``; returns ``(dequantised, scales, codes)`` as float32, the
    dequantised value being ``code * scale`` (python/tessera/__init__.py:3472-3500,
    python/tessera/compiler/microscaling.py:319-384)."""
    x = np.asarray(x, np.float32)
    n = x.shape[-1]
    if n % block_size:
        raise ValueError(f"last dim {n} must be divisible by block_size {block_size} for NVFP4")
    blocks = x.reshape(x.shape[:-1] + (n // block_size, block_size))
    amax = np.abs(blocks).max(axis=-1)
    raw = np.maximum(amax / np.float32(6.0), np.float32(1e-30)).astype(np.float32)
    scale = raw.astype(ml_dtypes.float8_e4m3fn).astype(np.float32)
    safe = np.where(scale == 0.0, np.float32(1.0), scale)[..., None]
    codes = (blocks / safe).astype(ml_dtypes.float4_e2m1fn).astype(np.float32)
    dq = (codes * scale[..., None]).reshape(x.shape).astype(np.float32)
    return dq, scale, codes.reshape(x.shape)


def _fp4_scheme(quant: str):
    q = str(quant).lower()
    return {"nvfp4": ("nvfp4", "nvfp4"), "fp8xfp4": ("fp8_e4m3", "nvfp4"),
            "fp8_e4m3xnvfp4": ("fp8_e4m3", "nvfp4"), "fp8_e5m2xnvfp4": ("fp8_e5m2", "nvfp4")}[q]


def _qdq(a, fmt: str):
    if fmt == "nvfp4":
        return quantize_nvfp4(a)[0]
    return quantize_fp8(a, "e5m2" if fmt == "fp8_e5m2" else "e4m3")[0]


def grouped_gemm_fp4(x, w, group_sizes, quant: str = "fp8xfp4") -> np.ndarray:
    """``grouped_gemm(..., quant="nvfp4" | "fp8xfp4")``: x and each expert's (K, N) weights are
    quantised and dequantised per the scheme's formats, then the f32 grouped GEMM
    (python/tessera/compiler/grouped_layout.py:319-392)."""
    act, wf = _fp4_scheme(quant)
    w = _f32(w)
    return grouped_gemm(_qdq(_f32(x), act), np.stack([_qdq(w[e], wf) for e in range(w.shape[0])]), group_sizes)


def moe_swiglu_block_fp4(x, w_gate, w_up, w_down, group_sizes, quant: str = "fp8xfp4") -> np.ndarray:
    """``moe_swiglu_block(..., quant=...)`` with NVFP4 weights: every grouped GEMM of the block
    quantises its operands (python/tessera/__init__.py:592-616)."""
    gate = grouped_gemm_fp4(x, w_gate, group_sizes, quant)
    up = grouped_gemm_fp4(x, w_up, group_sizes, quant)
    return grouped_gemm_fp4(silu_mul(gate, up), w_down, group_sizes, quant)


def quantize_kv(k, v, bits: int = 8):
    """Per-token symmetric integer quantisation of ``(seq, heads, dim)`` K and V: one scale per
    token and tensor, ``scale = max(amax / qmax, 1e-12)``, ``q = clip(round(x / scale), -qmax,
    qmax)`` with ``qmax = 2^(bits-1) - 1``; returns ``(k_q, v_q, scale)`` with ``scale`` of shape
    ``(2, seq, 1, 1)`` (python/tessera/__init__.py:3196-3249)."""
    k, v = np.asarray(k, np.float32), np.asarray(v, np.float32)
    qmax = (1 << (bits - 1)) - 1
    ks = np.maximum(np.max(np.abs(k), axis=(1, 2), keepdims=True) / qmax, 1e-12).astype(np.float32)
    vs = np.maximum(np.max(np.abs(v), axis=(1, 2), keepdims=True) / qmax, 1e-12).astype(np.float32)
    kq = np.clip(np.round(k / ks), -qmax, qmax).astype(np.int8)
    vq = np.clip(np.round(v / vs), -qmax, qmax).astype(np.int8)
    return kq, vq, np.stack([ks, vs], axis=0)


def dequantize_kv(k_q, v_q, scale):
    """``q * scale`` per token (python/tessera/__init__.py:3251-3265)."""
    scale = np.asarray(scale, np.float32)
    return (np.asarray(k_q).astype(np.float32) * scale[0], np.asarray(v_q).astype(np.float32) * scale[1])


# ----------------------------------------------------------------------------- paged KV
def paged_pack(k, v, page_size: int):
    """Tokens ``[n, H, D]`` -> identity-mapped pages ``[P, L, H, D]`` + table
    (``materialize_paged_kv_abi``, python/tessera/cache/paged_kv.py:421-454)."""
    k, v = _f32(k), _f32(v)
    n, H, D = k.shape
    pages = max(1, (n + page_size - 1) // page_size)
    kp = np.zeros((pages, page_size, H, D), np.float32)
    vp = np.zeros((pages, page_size, H, D), np.float32)
    kp.reshape(-1, H, D)[:n] = k
    vp.reshape(-1, H, D)[:n] = v
    return kp, vp, np.arange(pages, dtype=np.int32)


def paged_gather(k_pages, v_pages, page_table, logical_length: int, token_indices):
    """``PagedKVBufferABI.gather`` (python/tessera/cache/paged_kv.py:130-140): caller order,
    logical page -> physical page through the table."""
    idx = np.asarray(token_indices, np.int64).reshape(-1)
    if idx.size and (idx.min() < 0 or idx.max() >= logical_length):
        raise IndexError(f"paged KV token index outside [0, {logical_length})")
    L = np.asarray(k_pages).shape[1]
    lp, off = np.divmod(idx, L)
    pp = np.asarray(page_table)[lp]
    return _f32(np.asarray(k_pages)[pp, off]), _f32(np.asarray(v_pages)[pp, off])


def paged_attention(Q, k_pages, v_pages, page_table, logical_length: int, scale=None,
                    causal: bool = False, token_indices=None) -> np.ndarray:
    """``paged_attention`` (python/tessera/cache/paged_kv.py:480-559) over the page ABI: gather
    the requested tokens (all of ``[0, logical_length)`` by default), repeat KV heads for
    grouped queries and run ``_reference_attention`` (:457-477). Q ``(Hq, q_len, D)``."""
    Q = _f32(Q)
    idx = np.arange(logical_length) if token_indices is None else np.asarray(token_indices, np.int64)
    gk, gv = paged_gather(k_pages, v_pages, page_table, logical_length, idx)
    K, V = np.transpose(gk, (1, 0, 2)), np.transpose(gv, (1, 0, 2))
    if K.shape[0] != Q.shape[0]:
        if K.shape[0] < 1 or Q.shape[0] % K.shape[0]:
            raise ValueError("attention query heads must be divisible by KV heads")
        rep = Q.shape[0] // K.shape[0]
        K, V = np.repeat(K, rep, axis=0), np.repeat(V, rep, axis=0)
    if scale is None:
        scale = 1.0 / np.sqrt(Q.shape[-1])
    scores = np.matmul(Q, K.swapaxes(-1, -2)) * scale
    if causal:
        q_len, k_len = scores.shape[-2], scores.shape[-1]
        mask = np.triu(np.ones((q_len, k_len), dtype=bool), k=1 + max(k_len - q_len, 0))
        scores = np.where(mask, -np.inf, scores)
    scores = scores - scores.max(axis=-1, keepdims=True)
    w = np.exp(scores)
    w = w / w.sum(axis=-1, keepdims=True)
    return np.matmul(w, V).astype(np.float32)


# ----------------------------------------------------------------------------- MoE
class Routing(NamedTuple):
    assignment: np.ndarray  # (T, k) int64, -1 = dropped
    weights: np.ndarray     # (T, k) float32
    load: np.ndarray        # (E,) int64 (before capacity drops)
    overflow: int


def route_tokens(scores, top_k: int, normalize_weights: bool = True,
                 capacity: Optional[int] = None) -> Routing:
    """Top-k routing on f32 softmax probabilities (python/tessera/distributed/moe.py:119-206).
    ``np.argsort(probs)[:, -k:][:, ::-1]``: on equal probabilities the HIGHER expert index
    comes first. Capacity is applied in token-major slot order; ``None`` means no drops."""
    scores = np.asarray(scores)
    if scores.ndim != 2:
        raise ValueError(f"scores must be 2D (num_tokens, num_experts), got shape {scores.shape}")
    T, E = scores.shape
    exp_scores = np.exp(scores - scores.max(axis=1, keepdims=True))
    probs = exp_scores / exp_scores.sum(axis=1, keepdims=True)
    idx = np.argsort(probs, axis=1)[:, -top_k:][:, ::-1]
    w = np.take_along_axis(probs, idx, axis=1)
    if normalize_weights and top_k > 1:
        s = w.sum(axis=1, keepdims=True)
        s = np.where(s > 0, s, 1.0)
        w = w / s
    load = np.bincount(idx.reshape(-1), minlength=E).astype(np.int64)
    assignment = idx.astype(np.int64).copy()
    weights = w.astype(np.float32).copy()
    overflow = 0
    if capacity is not None:
        fill = np.zeros(E, np.int64)
        for t in range(T):
            for s_ in range(top_k):
                e = idx[t, s_]
                if fill[e] >= capacity:
                    assignment[t, s_] = -1
                    weights[t, s_] = 0.0
                    overflow += 1
                else:
                    fill[e] += 1
    return Routing(assignment, weights, load, overflow)


class Permutation(NamedTuple):
    token_of_slot: np.ndarray    # (S,) int32: source token of each expert-sorted slot
    expert_of_slot: np.ndarray   # (S,) int32, non-decreasing
    weight_of_slot: np.ndarray   # (S,) float32
    group_sizes: np.ndarray      # (E,) int32
    group_offsets: np.ndarray    # (E+1,) int32
    slot_of_assignment: np.ndarray  # (T, k) int32: sorted position of slot (t, j), -1 if dropped


def moe_permutation(assignment, weights, num_experts: int) -> Permutation:
    """Token-major slots, kept slots stably sorted by expert
    (python/tessera/nn/functional.py:461-477); int32 arrays as in the canonical device ABI
    (python/tessera/compiler/moe_transport.py:75-273)."""
    assignment = np.asarray(assignment)
    T, k = assignment.shape
    slot_token = np.repeat(np.arange(T, dtype=np.int64), k)
    slot_expert = assignment.reshape(-1)
    slot_weight = np.asarray(weights, np.float32).reshape(-1)
    keep = slot_expert >= 0
    kept_idx = np.nonzero(keep)[0]
    order = np.argsort(slot_expert[keep], kind="stable")
    src = kept_idx[order]
    group_sizes = np.bincount(slot_expert[src], minlength=num_experts).astype(np.int32)
    offsets = np.zeros(num_experts + 1, np.int32)
    offsets[1:] = np.cumsum(group_sizes)
    slot_of = np.full(T * k, -1, np.int32)
    slot_of[src] = np.arange(len(src), dtype=np.int32)
    return Permutation(slot_token[src].astype(np.int32), slot_expert[src].astype(np.int32),
                       slot_weight[src], group_sizes, offsets, slot_of.reshape(T, k))


def grouped_gemm(x, weights, group_sizes) -> np.ndarray:
    """Row block e of ``x`` times ``weights[e]`` (python/tessera/__init__.py:291-351), f32."""
    x, w = _f32(x), _f32(weights)
    gs = np.asarray(group_sizes).astype(np.int64).reshape(-1)
    if int(gs.sum()) != x.shape[0]:
        raise ValueError(f"grouped_gemm: group_sizes sum {int(gs.sum())} != T={x.shape[0]}")
    out = np.zeros((x.shape[0], w.shape[2]), np.float32)
    off = 0
    for e in range(w.shape[0]):
        n = int(gs[e])
        if n:
            out[off:off + n] = x[off:off + n] @ w[e]
        off += n
    return out


def silu_mul(a, b) -> np.ndarray:
    """``silu(a) * b`` (python/tessera/__init__.py:559-574)."""
    a = np.asarray(a, np.float32)
    return (a / (1.0 + np.exp(-a))) * np.asarray(b, np.float32)


def moe_swiglu_block(x, w_gate, w_up, w_down, group_sizes) -> np.ndarray:
    """gate/up grouped GEMMs -> silu_mul -> down grouped GEMM (python/tessera/__init__.py:592-616)."""
    gate = grouped_gemm(x, w_gate, group_sizes)
    up = grouped_gemm(x, w_up, group_sizes)
    return grouped_gemm(silu_mul(gate, up), w_down, group_sizes)


def moe_layer_from_logits(x, logits, w_gate, w_up, w_down, top_k: int,
                          normalize_weights: bool = True, capacity: Optional[int] = None):
    """``nn.functional.moe_layer`` (python/tessera/nn/functional.py:403-490) with the router
    logits supplied instead of ``x @ W_router``. Returns (out, routing, permutation)."""
    x = _f32(x)
    E = np.asarray(w_gate).shape[0]
    route = route_tokens(np.asarray(logits, np.float32), top_k, normalize_weights, capacity)
    perm = moe_permutation(route.assignment, route.weights, E)
    x_perm = x[perm.token_of_slot]
    y_perm = moe_swiglu_block(x_perm, w_gate, w_up, w_down, perm.group_sizes)
    out = np.zeros((x.shape[0], y_perm.shape[1]), np.float32)
    np.add.at(out, perm.token_of_slot, y_perm * perm.weight_of_slot[:, None])
    return out, route, perm


def moe_layer(x, W_router, w_gate, w_up, w_down, top_k: int = 1, normalize_weights: bool = True):
    """python/tessera/nn/functional.py:403-490 (no capacity drop)."""
    logits = gemm(x, W_router)
    return moe_layer_from_logits(x, logits, w_gate, w_up, w_down, top_k, normalize_weights)[0]


def expert_parallel_moe(x, logits, w_gate, w_up, w_down, top_k: int, world_size: int,
                        normalize_weights: bool = True) -> np.ndarray:
    """Expert-parallel forward partitioned as ``megamoe_forward``
    (python/tessera/distributed/moe.py:358-483): tokens row-sharded T/R per rank, rank r owns
    experts [r*Ep, (r+1)*Ep), dispatch exchange, local expert FFN, combine exchange, weighted sum
    in (token, slot) order. Unpadded (the reference pads every (source, expert) bucket to a fixed
    capacity with zero rows; when nothing is dropped the results are identical)."""
    x = _f32(x)
    logits = np.asarray(logits, np.float32)
    T, _ = x.shape
    E = np.asarray(w_gate).shape[0]
    R = world_size
    if T % R or E % R:
        raise ValueError("T and num_experts must be divisible by world_size")
    Tl, Ep = T // R, E // R
    N = np.asarray(w_down).shape[2]
    # per source rank: routing and send buckets
    routes = [route_tokens(logits[r * Tl:(r + 1) * Tl], top_k, normalize_weights) for r in range(R)]
    sends = [[None] * R for _ in range(R)]  # sends[src][dst] = (rows, expert_local, (t, j))
    for src in range(R):
        a = routes[src].assignment
        for dst in range(R):
            ts, js = np.nonzero((a // Ep) == dst)  # token-major order
            sends[src][dst] = (x[src * Tl + ts], a[ts, js] - dst * Ep, ts, js)
    y = np.zeros((T, N), np.float32)
    back = [[None] * R for _ in range(R)]
    for dst in range(R):
        rows = np.concatenate([sends[src][dst][0] for src in range(R)], axis=0)
        el = np.concatenate([sends[src][dst][1] for src in range(R)], axis=0)
        order = np.argsort(el, kind="stable")
        gs = np.bincount(el, minlength=Ep)
        out_sorted = moe_swiglu_block(rows[order], w_gate[dst * Ep:(dst + 1) * Ep],
                                      w_up[dst * Ep:(dst + 1) * Ep],
                                      w_down[dst * Ep:(dst + 1) * Ep], gs)
        out = np.empty_like(out_sorted)
        out[order] = out_sorted
        pos = 0
        for src in range(R):
            n = len(sends[src][dst][1])
            back[dst][src] = out[pos:pos + n]
            pos += n
    for src in range(R):
        w = routes[src].weights
        contrib = {}
        for dst in range(R):
            _, _, ts, js = sends[src][dst]
            for i, (t, j) in enumerate(zip(ts, js)):
                contrib[(int(t), int(j))] = back[dst][src][i]
        for t in range(Tl):
            for j in range(top_k):
                if (t, j) in contrib:
                    y[src * Tl + t] += w[t, j] * contrib[(t, j)]
    return y


# ----------------------------------------------------------------------------- error metrics
def max_rel_err(y, ref) -> float:
    """``max|y - ref| / max|ref|`` in f32: the parity metric (tolerance 1e-2)."""
    y, ref = _f32(y), _f32(ref)
    return float(np.abs(y - ref).max() / max(float(np.abs(ref).max()), 1e-30))


def fro_rel_err(y, ref) -> float:
    y, ref = _f32(y).astype(np.float64), _f32(ref).astype(np.float64)
    return float(np.linalg.norm(y - ref) / max(np.linalg.norm(ref), 1e-30))


# ----------------------------------------------------------------------------- seeded inputs
def make_inputs(config: str, scale_down: int = 1, seed: Optional[int] = None) -> dict:
    """Seeded synthetic inputs with the shapes and distributions of the five benchmark
    configurations (one ``default_rng(seed)``, tensors drawn in the order listed). ``scale_down``
    divides the large dimensions for CPU-sized cases."""
    bf16 = _BF16
    if config == "gemm_f16_batched":       # A[4,1024,1024] x W[4,1024,1024] f16
        rng = np.random.default_rng(1001 if seed is None else seed)
        n = 1024 // scale_down
        A = (rng.standard_normal((4, n, n), dtype=np.float32) / np.sqrt(n)).astype(np.float16)
        W = (rng.standard_normal((4, n, n), dtype=np.float32) / np.sqrt(n)).astype(np.float16)
        return dict(A=A, W=W)
    if config == "gemm_bf16":              # M=N=K=8192
        rng = np.random.default_rng(1002 if seed is None else seed)
        n = 8192 // scale_down
        A = (rng.standard_normal((n, n), dtype=np.float32) / np.sqrt(n)).astype(bf16)
        B = (rng.standard_normal((n, n), dtype=np.float32) / np.sqrt(n)).astype(bf16)
        return dict(A=A, B=B)
    if config == "attn_prefill":           # B=8 H=32 S=4096 D=128 causal
        rng = np.random.default_rng(1003 if seed is None else seed)
        B, H, S, D = max(1, 8 // scale_down), max(1, 32 // scale_down), 4096 // scale_down, 128
        q, k, v = (rng.standard_normal((B, H, S, D), dtype=np.float32).astype(bf16) for _ in range(3))
        return dict(Q=q, K=k, V=v, scale=1.0 / np.sqrt(D), causal=True)
    if config == "attn_decode":            # batch 64, Hq 32, Hkv 8, D 128, KV 8192
        rng = np.random.default_rng(1004 if seed is None else seed)
        B, Hq, Hkv, S, D = max(1, 64 // scale_down), 32, 8, 8192 // scale_down, 128
        q = rng.standard_normal((B, Hq, 1, D), dtype=np.float32).astype(bf16)
        k = rng.standard_normal((B, Hkv, S, D), dtype=np.float32).astype(bf16)
        v = rng.standard_normal((B, Hkv, S, D), dtype=np.float32).astype(bf16)
        return dict(Q=q, K=k, V=v, Hq=Hq, Hkv=Hkv, scale=1.0 / np.sqrt(D))
    if config == "moe":                    # 8192 tokens, hidden 4096, FFN 14336, 8 experts, top-2
        rng = np.random.default_rng(1005 if seed is None else seed)
        T, H, F, E = 8192 // scale_down, 4096 // scale_down, 14336 // scale_down, 8
        x = rng.standard_normal((T, H), dtype=np.float32)
        logits = rng.standard_normal((T, E), dtype=np.float32)
        wg = (rng.standard_normal((E, H, F), dtype=np.float32) / np.sqrt(H)).astype(bf16)
        wu = (rng.standard_normal((E, H, F), dtype=np.float32) / np.sqrt(H)).astype(bf16)
        wd = (rng.standard_normal((E, F, H), dtype=np.float32) / np.sqrt(F)).astype(bf16)
        return dict(x=x.astype(bf16), logits=logits, w_gate=wg, w_up=wu, w_down=wd, top_k=2)
    raise ValueError(f"unknown config {config!r}")
