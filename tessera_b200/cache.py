"""Paged KV cache for the decode path: the page ABI of the reference
(python/tessera/cache/paged_kv.py) with the pages resident in device memory.

Two layers:

* the descriptors the reference defines — :class:`PageTier`, :class:`KVKind`, :class:`KVGeometry`,
  :class:`PageTableEntry`, :class:`PagedKVBufferABI` (pages ``[physical_page, page_offset, head,
  dim]``, ``page_table[logical_page] -> physical page``) and :func:`materialize_paged_kv_abi`;
* :class:`PagedKVCache`, a batched device-resident cache (one page table row and one length per
  sequence, bf16 pages) that the paged decode kernel reads in place and the append kernel writes.

``paged_attention`` here is the GPU consumer; there is no host fallback.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Any, Optional, Sequence

import numpy as np

from . import _lib, device
from .device import DeviceArray, bfloat16

HEAD_DIM = 128          # the decode kernel's head dimension
GATHER_PAGE = 64        # page size of the compact pages a token_indices gather produces


class PageTier(enum.Enum):
    """Where a logical page lives (python/tessera/cache/paged_kv.py:40-49)."""
    RESIDENT = "resident"
    HOST = "host"
    OFFLOAD = "offload"


class KVKind(enum.Enum):
    """Storage family of a KV state (python/tessera/cache/paged_kv.py:52-62)."""
    FULL = "full"
    LATENT = "latent"
    LOW_RANK = "low_rank"
    QUANTIZED_TAIL = "quantized_tail"


@dataclass(frozen=True)
class KVGeometry:
    num_heads: int
    head_dim: int
    max_seq: int
    page_size: int
    dtype: str = "fp32"


@dataclass(frozen=True)
class PageTableEntry:
    page_id: int
    tier: PageTier
    shared_with: tuple = ()


@dataclass(frozen=True)
class PagedKVBufferABI:
    """Physical-page view handed to a device backend (python/tessera/cache/paged_kv.py:91-140):
    ``k_pages``/``v_pages`` are ``[P, L, H, D]`` host arrays (float32 as in the reference, or
    float16/bfloat16), ``page_table`` is rank-1 int32 and ``logical_length`` the token count."""

    k_pages: np.ndarray
    v_pages: np.ndarray
    page_table: np.ndarray
    logical_length: int
    abi_version: int = 1
    layout: str = "PLHD"

    def __post_init__(self) -> None:
        k, v, table = np.asarray(self.k_pages), np.asarray(self.v_pages), np.asarray(self.page_table)
        if self.abi_version != 1 or self.layout != "PLHD":
            raise ValueError("unsupported paged KV buffer ABI version/layout")
        ok_dtypes = [np.dtype(np.float32), np.dtype(np.float16)] + ([bfloat16] if bfloat16 is not None else [])
        if k.dtype not in ok_dtypes or k.dtype != v.dtype or k.ndim != 4 or k.shape != v.shape:
            raise ValueError("paged KV ABI requires equal rank-4 f32/f16/bf16 K/V pages")
        if table.dtype != np.int32 or table.ndim != 1 or table.size < 1:
            raise ValueError("paged KV ABI page_table must be non-empty rank-1 i32")
        if np.any(table < 0) or np.any(table >= k.shape[0]):
            raise ValueError("paged KV ABI page_table references an invalid physical page")
        if self.logical_length < 0 or self.logical_length > int(table.size) * int(k.shape[1]):
            raise ValueError("paged KV ABI logical_length exceeds table capacity")

    @property
    def page_size(self) -> int:
        return int(np.asarray(self.k_pages).shape[1])

    def gather(self, token_indices) -> tuple[np.ndarray, np.ndarray]:
        """Host gather through the page table in caller order (a descriptor utility, used to
        build and inspect caches; attention never goes through it)."""
        idx = np.asarray(token_indices, dtype=np.int64).reshape(-1)
        if idx.size and (idx.min() < 0 or idx.max() >= self.logical_length):
            raise IndexError(f"paged KV token index outside [0, {self.logical_length})")
        lp, off = np.divmod(idx, self.page_size)
        pp = np.asarray(self.page_table)[lp]
        return (np.asarray(self.k_pages)[pp, off].astype(np.float32),
                np.asarray(self.v_pages)[pp, off].astype(np.float32))


def materialize_paged_kv_abi(kv_state: Any) -> PagedKVBufferABI:
    """Any paged KV state -> :class:`PagedKVBufferABI` (python/tessera/cache/paged_kv.py:421-454):
    a state's own ``paged_kv_abi()`` wins; otherwise its tokens are gathered once through the
    protocol (``kv_geometry`` / ``seq_len`` / ``gather``) into identity-mapped pages."""
    if isinstance(kv_state, PagedKVBufferABI):
        return kv_state
    native = getattr(kv_state, "paged_kv_abi", None)
    if callable(native):
        abi = native()
        if isinstance(abi, PagedKVBufferABI):
            return abi
        # a reference-side PagedKVBufferABI: same fields, different class
        return PagedKVBufferABI(np.asarray(abi.k_pages), np.asarray(abi.v_pages),
                                np.asarray(abi.page_table), int(abi.logical_length))
    for attr in ("kv_geometry", "seq_len", "gather"):
        if not callable(getattr(kv_state, attr, None)):
            raise TypeError(f"{type(kv_state).__name__} does not satisfy the paged KV protocol "
                            f"(missing {attr}())")
    geo = kv_state.kv_geometry()
    n = int(kv_state.seq_len())
    L, H, D = int(geo.page_size), int(geo.num_heads), int(geo.head_dim)
    pages = max(1, (n + L - 1) // L)
    k_pages = np.zeros((pages, L, H, D), np.float32)
    v_pages = np.zeros((pages, L, H, D), np.float32)
    if n:
        k, v = kv_state.gather(range(n))
        k_pages.reshape(-1, H, D)[:n] = np.asarray(k, np.float32)
        v_pages.reshape(-1, H, D)[:n] = np.asarray(v, np.float32)
    return PagedKVBufferABI(k_pages, v_pages, np.arange(pages, dtype=np.int32), n)


def _check_page_size(page_size: int) -> None:
    if page_size < 8 or page_size > 1024 or page_size & (page_size - 1):
        raise ValueError(f"page_size must be a power of two in [8, 1024]; got {page_size}")


class PagedKVCache:
    """Device-resident paged KV for a batch of sequences.

    ``k_pages`` / ``v_pages``: ``[num_pages, page_size, num_kv_heads, 128]`` bf16;
    ``page_table``: ``[num_seqs, max_pages]`` int32; ``seq_lens``: ``[num_seqs]`` int32.
    Page allocation is host bookkeeping (a free list); token data only moves on the device.
    """

    kind = KVKind.FULL

    def __init__(self, num_seqs: int, num_kv_heads: int, head_dim: int = HEAD_DIM, *, page_size: int = 64,
                 num_pages: int, max_pages_per_seq: Optional[int] = None, quantize_bits: Optional[int] = None):
        if head_dim != HEAD_DIM:
            raise ValueError(f"PagedKVCache: head_dim must be {HEAD_DIM}; got {head_dim}")
        if num_seqs <= 0 or num_kv_heads <= 0 or num_pages <= 0:
            raise ValueError("PagedKVCache: num_seqs / num_kv_heads / num_pages must be positive")
        _check_page_size(page_size)
        self.num_seqs, self.num_kv_heads, self.head_dim = int(num_seqs), int(num_kv_heads), int(head_dim)
        self.page_size, self.num_pages = int(page_size), int(num_pages)
        self.max_pages = int(max_pages_per_seq) if max_pages_per_seq else max(1, num_pages // num_seqs)
        if quantize_bits not in (None, 8):
            raise ValueError("PagedKVCache: quantize_bits must be None or 8")
        # quantize_bits=8: 8-bit pages (each value stored as the byte q + 128, the form the decode
        # kernel widens for free) with one fp32 scale per token for K and for V, shared by the
        # heads (KVCacheHandle(quantize_bits=8), python/tessera/cache/handle.py:72-137)
        self.quantize_bits = quantize_bits
        shape = (self.num_pages, self.page_size, self.num_kv_heads, self.head_dim)
        page_dtype = np.uint8 if quantize_bits else bfloat16
        self.k_pages = DeviceArray.zeros(shape, page_dtype)
        self.v_pages = DeviceArray.zeros(shape, page_dtype)
        self.k_scales = self.v_scales = None
        if quantize_bits:
            self.k_scales = DeviceArray.zeros((self.num_pages, self.page_size), np.float32)
            self.v_scales = DeviceArray.zeros((self.num_pages, self.page_size), np.float32)
        self._table = np.zeros((self.num_seqs, self.max_pages), np.int32)
        self._owned = np.zeros(self.num_seqs, np.int64)          # pages assigned per sequence
        self._lens = np.zeros(self.num_seqs, np.int32)
        self._free = list(range(self.num_pages - 1, -1, -1))     # pop() hands out page 0 first
        self.page_table = DeviceArray.from_host(self._table)
        self.seq_lens = DeviceArray.from_host(self._lens)

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_abi(cls, abi: PagedKVBufferABI) -> "PagedKVCache":
        """One sequence from a host page descriptor, placement and table kept as given."""
        k = np.asarray(abi.k_pages)
        P, L, H, D = k.shape
        self = cls.__new__(cls)
        self.quantize_bits, self.k_scales, self.v_scales = None, None, None
        if D != HEAD_DIM:
            raise ValueError(f"PagedKVCache: head_dim must be {HEAD_DIM}; got {D}")
        _check_page_size(L)
        self.num_seqs, self.num_kv_heads, self.head_dim = 1, H, D
        self.page_size, self.num_pages = L, P
        table = np.asarray(abi.page_table, np.int32).reshape(1, -1)
        self.max_pages = table.shape[1]
        self.k_pages = DeviceArray.from_host(k.astype(bfloat16))
        self.v_pages = DeviceArray.from_host(np.asarray(abi.v_pages).astype(bfloat16))
        self._table = table.copy()
        self._lens = np.array([abi.logical_length], np.int32)
        self._owned = np.array([table.shape[1]], np.int64)
        self._free = sorted(set(range(P)) - set(table.reshape(-1).tolist()), reverse=True)
        self.page_table = DeviceArray.from_host(self._table)
        self.seq_lens = DeviceArray.from_host(self._lens)
        return self

    @classmethod
    def from_dense(cls, K, V, *, page_size: int = 64, seq_lens: Optional[Sequence[int]] = None,
                   num_pages: Optional[int] = None, page_order: Optional[Sequence[int]] = None,
                   max_pages_per_seq: Optional[int] = None, quantize_bits: Optional[int] = None) -> "PagedKVCache":
        """Build from dense host ``K``, ``V`` ``[B, S, Hkv, 128]``; sequence b keeps its first
        ``seq_lens[b]`` tokens. ``page_order`` (a permutation of the physical pages) scatters the
        pages so the table is not the identity."""
        K, V = np.asarray(K), np.asarray(V)
        if K.ndim != 4 or K.shape != V.shape:
            raise ValueError("from_dense: K and V must be equal-shape [B, S, Hkv, D]")
        B, S, H, D = K.shape
        lens = np.full(B, S, np.int64) if seq_lens is None else np.asarray(seq_lens, np.int64)
        if lens.shape != (B,) or lens.min() < 0 or lens.max() > S:
            raise ValueError("from_dense: seq_lens must be B values in [0, S]")
        per_seq = np.maximum(1, (lens + page_size - 1) // page_size)
        need = int(per_seq.sum())
        P = int(num_pages) if num_pages else need
        if P < need:
            raise ValueError(f"from_dense: {need} pages needed, num_pages={P}")
        self = cls(B, H, D, page_size=page_size, num_pages=P,
                   max_pages_per_seq=max_pages_per_seq or int(per_seq.max()), quantize_bits=quantize_bits)
        order = list(range(P)) if page_order is None else [int(x) for x in page_order]
        if sorted(order) != list(range(P)):
            raise ValueError("from_dense: page_order must be a permutation of range(num_pages)")
        self._free = order[::-1]
        for b in range(B):
            for lp in range(int(per_seq[b])):
                self._table[b, lp] = self._free.pop()
            self._owned[b] = per_seq[b]
        self._lens[:] = lens
        if quantize_bits:
            # tokens go to their page slots through the quantisation kernel itself
            toks_k = np.concatenate([K[b, :int(lens[b])] for b in range(B)]).reshape(-1, H * D)
            toks_v = np.concatenate([V[b, :int(lens[b])] for b in range(B)]).reshape(-1, H * D)
            rows = np.concatenate([self._slot_rows(b, np.arange(int(lens[b]))) for b in range(B)])
            self._quantize_into_pages(toks_k, toks_v, rows)
        else:
            hk = np.zeros((P, page_size, H, D), bfloat16)
            hv = np.zeros((P, page_size, H, D), bfloat16)
            for b in range(B):
                n = int(lens[b])
                for lp in range(int(per_seq[b])):
                    pp = int(self._table[b, lp])
                    t0, t1 = lp * page_size, min(n, (lp + 1) * page_size)
                    if t1 > t0:
                        hk[pp, :t1 - t0] = K[b, t0:t1].astype(bfloat16)
                        hv[pp, :t1 - t0] = V[b, t0:t1].astype(bfloat16)
            self.k_pages.upload(hk)
            self.v_pages.upload(hv)
        self.page_table.upload(self._table)
        self.seq_lens.upload(self._lens)
        return self

    def _slot_rows(self, b: int, positions: np.ndarray) -> np.ndarray:
        """Row index (physical page * page_size + offset) of each position of sequence ``b``."""
        lp, off = np.divmod(np.asarray(positions, np.int64), self.page_size)
        return self._table[b, lp].astype(np.int64) * self.page_size + off

    def _quantize_into_pages(self, k_rows, v_rows, dst_rows: np.ndarray, stream=None) -> None:
        """Per-token int8 quantisation of ``[T, Hkv*D]`` rows straight into their page slots."""
        T, row = k_rows.shape
        if T == 0:
            return
        dk = k_rows if isinstance(k_rows, DeviceArray) else DeviceArray.from_host(np.ascontiguousarray(k_rows), pooled=True)
        dv = v_rows if isinstance(v_rows, DeviceArray) else DeviceArray.from_host(np.ascontiguousarray(v_rows), pooled=True)
        drows = DeviceArray.from_host(np.ascontiguousarray(dst_rows, np.int64), pooled=True)
        _lib.call("tessera_sm100_quantize_kv_int8_device", dk.ptr, dv.ptr, self.k_pages.ptr, self.v_pages.ptr,
                  self.k_scales.ptr, self.v_scales.ptr, drows.ptr, T, row, device.dtype_code(dk.dtype),
                  device._stream_handle(stream))
        if stream is None:
            device.synchronize()

    # ------------------------------------------------------------------ decode-step append
    def append(self, k_new, v_new, stream=None) -> "PagedKVCache":
        """One new token per sequence: ``k_new``, ``v_new`` ``[B, Hkv, 128]`` (host or device).
        Sequences that start a new page get one from the free list first; the rows are written and
        the lengths bumped by a kernel (KVCacheHandle.append, python/tessera/cache/handle.py:156-215)."""
        # Which sequences start a new page: checked for ALL of them before any state changes, so a
        # refusal leaves the host table, the free list and the device table as they were.
        need = [b for b in range(self.num_seqs) if int(self._lens[b]) >= int(self._owned[b]) * self.page_size]
        for b in need:
            if self._owned[b] >= self.max_pages:
                raise ValueError(f"PagedKVCache.append: sequence {b} would exceed its page table "
                                 f"({self.max_pages} pages of {self.page_size})")
        if len(need) > len(self._free):
            raise ValueError(f"PagedKVCache.append: no free pages ({len(need)} needed, {len(self._free)} free)")
        for b in need:
            self._table[b, self._owned[b]] = self._free.pop()
            self._owned[b] += 1
        if need:
            self.page_table.upload(self._table, stream)
        shape = (self.num_seqs, self.num_kv_heads, self.head_dim)
        if self.quantize_bits:
            # quantise the new rows straight into their slots, then publish the new lengths
            rows = np.array([self._slot_rows(b, np.array([int(self._lens[b])]))[0] for b in range(self.num_seqs)])
            row = self.num_kv_heads * self.head_dim
            kn = k_new.view((self.num_seqs, row)) if isinstance(k_new, DeviceArray) else \
                np.asarray(k_new).reshape(self.num_seqs, row)
            vn = v_new.view((self.num_seqs, row)) if isinstance(v_new, DeviceArray) else \
                np.asarray(v_new).reshape(self.num_seqs, row)
            self._quantize_into_pages(kn, vn, rows, stream)
            self._lens += 1
            self.seq_lens.upload(self._lens, stream)
            return self
        dk, dv = _as_device_bf16(k_new, shape, "k_new"), _as_device_bf16(v_new, shape, "v_new")
        _lib.call("tessera_sm100_paged_kv_append_device", dk.ptr, dv.ptr, self.k_pages.ptr, self.v_pages.ptr,
                  self.page_table.ptr, self.seq_lens.ptr, self.num_seqs, self.num_kv_heads, self.head_dim,
                  self.page_size, self.num_pages, self.max_pages, device._stream_handle(stream))
        self._lens += 1
        return self

    def release(self, b: int) -> None:
        """Return sequence ``b``'s pages to the free list and reset its length."""
        for lp in range(int(self._owned[b])):
            self._free.append(int(self._table[b, lp]))
        self._owned[b] = 0
        self._lens[b] = 0
        self._table[b] = 0
        self.page_table.upload(self._table)
        self.seq_lens.upload(self._lens)

    # ------------------------------------------------------------------ protocol (one sequence)
    def _single(self, what: str) -> None:
        if self.num_seqs != 1:
            raise ValueError(f"PagedKVCache.{what}: the one-sequence protocol needs num_seqs == 1")

    def kv_geometry(self) -> KVGeometry:
        return KVGeometry(self.num_kv_heads, self.head_dim, self.max_pages * self.page_size,
                          self.page_size, "bf16")

    def seq_len(self) -> int:
        self._single("seq_len")
        return int(self._lens[0])

    def lengths(self) -> np.ndarray:
        return self._lens.copy()

    def quant_bits(self):
        return None

    def page_table_entries(self) -> list:
        self._single("page_table_entries")
        n = (int(self._lens[0]) + self.page_size - 1) // self.page_size
        return [PageTableEntry(p, PageTier.RESIDENT) for p in range(n)]

    def tier(self, page_id: int) -> PageTier:
        return PageTier.RESIDENT

    def gather(self, token_indices, seq: int = 0, stream=None) -> tuple[np.ndarray, np.ndarray]:
        """K, V rows ``[T, Hkv, 128]`` (float32 host arrays) for logical tokens of sequence ``seq``,
        in caller order — gathered by a kernel (PagedKVBufferABI.gather,
        python/tessera/cache/paged_kv.py:130-140)."""
        dk, dv = self.gather_device(token_indices, seq, stream)
        k, v = dk.download().astype(np.float32), dv.download().astype(np.float32)
        device.check_device_error("paged_kv_gather")
        return k, v

    def gather_device(self, token_indices, seq: int = 0, stream=None, pad_to: int = 1):
        if self.quantize_bits:
            raise NotImplementedError("PagedKVCache.gather: not available for an int8 cache")
        idx = np.asarray(list(token_indices) if not isinstance(token_indices, np.ndarray) else token_indices,
                         dtype=np.int64).reshape(-1)
        n = int(self._lens[seq])
        if idx.size and (idx.min() < 0 or idx.max() >= n):
            raise IndexError(f"paged KV token index outside [0, {n})")
        T = int(idx.size)
        rows = max(pad_to, (T + pad_to - 1) // pad_to * pad_to)
        shape = (rows, self.num_kv_heads, self.head_dim)
        dk, dv = DeviceArray.zeros(shape, bfloat16, stream), DeviceArray.zeros(shape, bfloat16, stream)
        if T:
            didx = DeviceArray.from_host(idx, stream)
            table = self.page_table.view((self.max_pages,), seq * self.max_pages)
            for pages, out in ((self.k_pages, dk), (self.v_pages, dv)):
                _lib.call("tessera_sm100_paged_kv_gather_device", pages.ptr, table.ptr, didx.ptr, out.ptr, T,
                          self.num_kv_heads, self.head_dim, self.page_size, self.num_pages, self.max_pages,
                          device._stream_handle(stream))
        return dk, dv

    def paged_kv_abi(self) -> PagedKVBufferABI:
        """Download as a host descriptor (for inspection and tests)."""
        self._single("paged_kv_abi")
        used = max(1, int(self._owned[0]))
        return PagedKVBufferABI(self.k_pages.download(), self.v_pages.download(),
                                self._table[0, :used].copy(), int(self._lens[0]))


def _as_device_bf16(x, shape, name: str) -> DeviceArray:
    if isinstance(x, DeviceArray):
        if x.shape != tuple(shape) or x.dtype != bfloat16:
            raise ValueError(f"{name}: device array must be {tuple(shape)} bfloat16")
        return x
    a = np.asarray(x)
    if a.shape != tuple(shape):
        raise ValueError(f"{name}: expected shape {tuple(shape)}, got {a.shape}")
    return DeviceArray.from_host(a.astype(bfloat16), pooled=True)


def _decode(Q: DeviceArray, cache_like, table: DeviceArray, lens: DeviceArray, B: int, Hq: int,
            max_pages: int, max_seq_len: int, scale: float, stream, scales=None) -> DeviceArray:
    k_pages, v_pages, Hkv, L, P = cache_like
    lib = _lib.load()
    pick = lib.tessera_sm100_attn_decode_int8_splits if scales is not None else lib.tessera_sm100_attn_decode_splits
    splits = int(pick(B, Hq, Hkv, max_seq_len))
    scratch = None
    if splits > 1:
        nbytes = int(lib.tessera_sm100_attn_decode_scratch_bytes(B, Hq, splits))
        scratch = DeviceArray((nbytes,), np.uint8, pooled=True)
    out = DeviceArray((B, Hq, HEAD_DIM), bfloat16)
    if scales is not None:
        _lib.call("tessera_sm100_paged_attn_decode_int8_device", Q.ptr, k_pages.ptr, v_pages.ptr, scales[0].ptr,
                  scales[1].ptr, table.ptr, lens.ptr, out.ptr, B, Hq, Hkv, HEAD_DIM, L, P, max_pages, max_seq_len,
                  float(scale), splits, scratch.ptr if scratch is not None else None,
                  device._stream_handle(stream))
        return out
    _lib.call("tessera_sm100_paged_attn_decode_device", Q.ptr, k_pages.ptr, v_pages.ptr, table.ptr, lens.ptr,
              out.ptr, B, Hq, Hkv, HEAD_DIM, L, P, max_pages, max_seq_len, float(scale), splits,
              scratch.ptr if scratch is not None else None, device._stream_handle(stream))
    return out


def paged_decode(Q, cache: PagedKVCache, *, scale: Optional[float] = None, stream=None):
    """One decode step for the whole batch: ``Q`` ``[B, Hq, 128]`` against ``cache``; returns
    ``[B, Hq, 128]`` (bf16 device array for a device ``Q``, float32 host array otherwise)."""
    on_device = isinstance(Q, DeviceArray)
    q = Q if on_device else np.asarray(getattr(Q, "_data", Q))
    if len(q.shape) != 3 or q.shape[0] != cache.num_seqs or q.shape[2] != HEAD_DIM:
        raise ValueError(f"paged_decode: Q must be ({cache.num_seqs}, Hq, {HEAD_DIM}); got {tuple(q.shape)}")
    Hq = int(q.shape[1])
    if Hq % cache.num_kv_heads:
        raise ValueError("paged_decode: query heads must be divisible by KV heads; got "
                         f"Q={Hq} KV={cache.num_kv_heads}")
    lens = cache.lengths()
    if lens.min() < 1:
        raise ValueError("paged_decode: every sequence needs at least one cached token")
    dq = _as_device_bf16(q, q.shape, "Q")
    sc = 1.0 / np.sqrt(HEAD_DIM) if scale is None else float(scale)
    out = _decode(dq, (cache.k_pages, cache.v_pages, cache.num_kv_heads, cache.page_size, cache.num_pages),
                  cache.page_table, cache.seq_lens, cache.num_seqs, Hq, cache.max_pages, int(lens.max()), sc,
                  stream, scales=(cache.k_scales, cache.v_scales) if cache.quantize_bits else None)
    if on_device:
        return out
    host = out.download().astype(np.float32)
    device.check_device_error("paged_attn_decode")
    return host


def paged_attention(Q, kv_state, *, scale: Optional[float] = None, causal: bool = False,
                    token_indices: Optional[Sequence[int]] = None, backend: str = "nvidia",
                    return_execution: bool = False, stream=None):
    """Attention over a paged KV state (python/tessera/cache/paged_kv.py:480-559). ``Q`` is
    ``(num_heads, q_len, 128)``; returns float32 ``(num_heads, q_len, 128)``.

    The pages are read in place by the decode kernel. The ``q_len`` query rows of a head ride as
    extra query heads of its KV head (non-causal), or as ``q_len`` batch entries whose lengths
    realise the reference's bottom-right causal mask. ``token_indices`` first gathers the chosen
    tokens on the device into compact pages. ``backend`` accepts "nvidia" (this kernel) only."""
    if backend not in ("nvidia", "nvidia_sm100"):
        raise ValueError(f"unknown backend {backend!r}; this package runs paged attention on 'nvidia' only")
    q = np.asarray(getattr(Q, "_data", Q))
    if q.ndim != 3:
        raise ValueError(f"Q must be (num_heads, q_len, head_dim); got {q.shape}")
    Hq, q_len, D = q.shape
    if D != HEAD_DIM:
        raise ValueError(f"paged_attention: head_dim must be {HEAD_DIM}; got {D}")
    cache = kv_state if isinstance(kv_state, PagedKVCache) else PagedKVCache.from_abi(
        materialize_paged_kv_abi(kv_state))
    cache._single("paged_attention")
    Hkv = cache.num_kv_heads
    if Hkv < 1 or Hq % Hkv:
        raise ValueError(f"attention query heads must be divisible by KV heads; got Q={Hq} KV={Hkv}")
    sc = 1.0 / np.sqrt(D) if scale is None else float(scale)
    scales = (cache.k_scales, cache.v_scales) if cache.quantize_bits else None
    if token_indices is None:
        n = cache.seq_len()
        pages = (cache.k_pages, cache.v_pages, Hkv, cache.page_size, cache.num_pages)
        table_row, max_pages = cache._table[0], cache.max_pages
        keep = None
    else:
        idx = np.asarray(list(token_indices), np.int64)
        n = int(idx.size)
        dk, dv = cache.gather_device(idx, 0, stream, pad_to=GATHER_PAGE)
        P = dk.shape[0] // GATHER_PAGE
        pages = (dk, dv, Hkv, GATHER_PAGE, P)
        table_row, max_pages = np.arange(P, dtype=np.int32), P
        keep = (dk, dv)
    if n < 1:
        raise ValueError("paged_attention: the KV state holds no tokens")
    if causal and q_len > 1:
        # row i sees keys j <= i + max(n - q_len, 0): one batch entry per row
        B = q_len
        lens = np.minimum(n, np.arange(q_len) + max(n - q_len, 0) + 1).astype(np.int32)
        qd = np.ascontiguousarray(q.transpose(1, 0, 2))                    # [q_len, Hq, D]
        heads = Hq
    else:
        B = 1
        lens = np.array([n], np.int32)
        qd = np.ascontiguousarray(q.reshape(1, Hq * q_len, D))             # head hq, row qi -> hq*q_len+qi
        heads = Hq * q_len
    table = DeviceArray.from_host(np.ascontiguousarray(np.broadcast_to(table_row, (B, max_pages))).astype(np.int32),
                                  pooled=True)
    dl = DeviceArray.from_host(lens, pooled=True)
    dq = DeviceArray.from_host(qd.astype(bfloat16), pooled=True)
    out = _decode(dq, pages, table, dl, B, heads, max_pages, int(lens.max()), sc, stream,
                  scales=scales if token_indices is None else None)
    host = out.download().astype(np.float32)
    device.check_device_error("paged_attention")
    del keep
    res = host.transpose(1, 0, 2) if (causal and q_len > 1) else host.reshape(Hq, q_len, D)
    res = np.ascontiguousarray(res)
    return (res, "native_gpu") if return_execution else res


__all__ = ["PageTier", "KVKind", "KVGeometry", "PageTableEntry", "PagedKVBufferABI", "PagedKVCache",
           "materialize_paged_kv_abi", "paged_attention", "paged_decode"]
