"""Kernel candidates for the reference's arbiter seam (python/tessera/compiler/emit/candidate.py:
110-236): one :class:`Candidate` per op kind, each bound to the hand-written sm_100a kernel for
that op, plus a registry and a tier-priority ``arbitrate`` / ``run_arbitrated`` pair.

Regions are read by attribute (``epilogue``, ``residual``, ``reduction``, ``scale``, ``causal``,
``gate_act``, ``storage_dtype`` ...), so the reference's own ``fusion_core`` region objects and
the light descriptors defined here both work. A candidate never computes on the host: when it
cannot serve a region or a shape it says so (``applies_to`` is false, or ``run`` raises
``ValueError``) and the arbiter moves on. The accuracy gate (the reference's
``verify_candidate``, candidate.py:285-330) stays with whoever registers these candidates in
the reference; it is not re-implemented here.
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from dataclasses import dataclass
from enum import IntEnum
from typing import Any, Callable, Optional

import numpy as np

from . import _lib, device, ops
from .device import DeviceArray, bfloat16

EXECUTION_TAG = "nvidia_sm100_tcgen05"   # a real device kernel ran (not a reference execution)


class Tier(IntEnum):
    SYNTHESIZED = 1
    EMITTED = 2
    HAND_TUNED = 3


OP_FUSED_REGION = "fused_region"
OP_ATTENTION = "attention"
OP_GATED_MATMUL = "gated_matmul"
OP_MATMUL = "matmul"
_OPS = (OP_FUSED_REGION, OP_ATTENTION, OP_GATED_MATMUL, OP_MATMUL)


# ------------------------------------------------------------------ region descriptors
@dataclass(frozen=True)
class MatmulRegion:
    """``D = A @ B`` on 16-bit storage (python/tessera/compiler/fusion_core.py:365-405)."""
    dtype: str = "bfloat16"


@dataclass(frozen=True)
class FusedRegion:
    """Matmul + ordered pointwise epilogue (fusion_core.py:226-345): ``bias`` then at most one of
    ``relu`` / ``gelu`` / ``silu``; ``residual`` is added after the chain."""
    epilogue: tuple = ()
    reduction: Optional[str] = None
    residual: bool = False
    prologue: tuple = ()
    bias_name: Optional[str] = None
    storage_dtype: str = "bf16"


@dataclass(frozen=True)
class AttentionRegion:
    """Single-head ``softmax(scale Q K^T) V`` with keys ``n > m`` masked when causal
    (fusion_core.py:672-727)."""
    scale: float = 1.0
    causal: bool = False
    storage_dtype: str = "bf16"


@dataclass(frozen=True)
class GatedMatmulRegion:
    """``f(A @ Wg) * (A @ Wu)`` (fusion_core.py:747-782)."""
    gate_act: str = "silu"
    storage_dtype: str = "bf16"


_STORAGE = {"bf16": bfloat16, "bfloat16": bfloat16, "f16": np.dtype(np.float16), "fp16": np.dtype(np.float16),
            "float16": np.dtype(np.float16)}


def _storage(region, default="bf16") -> np.dtype:
    name = getattr(region, "storage_dtype", None) or getattr(region, "dtype", None) or default
    if name not in _STORAGE:
        raise ValueError(f"storage dtype {name!r} is not served by the sm_100a kernels (bf16 / f16 only)")
    return _STORAGE[name]


def _gpu_present() -> bool:
    try:
        return device.device_count() > 0
    except Exception:
        return False


# ------------------------------------------------------------------ the seam
class Candidate(ABC):
    name: str = ""
    tier: Tier = Tier.SYNTHESIZED
    target: str = ""
    op: str = OP_FUSED_REGION
    accuracy_atol: Optional[float] = None
    accuracy_rtol: Optional[float] = None
    mma_target: Optional[str] = None
    mma_arch: Optional[str] = None
    mma_prefer_shape: Optional[tuple] = None

    def available(self) -> bool:
        return True

    def applies_to(self, region: Any) -> bool:
        return True

    def measure_device_latency(self, region: Any, *inputs: Any, reps: int = 100, warmup: int = 10):
        return None

    @abstractmethod
    def run(self, region: Any, *inputs: Any, **kwargs: Any):
        """-> (output, execution_tag)"""


class _Sm100Candidate(Candidate):
    tier = Tier.HAND_TUNED
    target = "nvidia"
    mma_target = "nvidia"
    mma_arch = "sm_100a"
    accuracy_atol = 2e-2       # 16-bit operands against an f32 reference
    accuracy_rtol = 2e-2

    def available(self) -> bool:
        return _gpu_present()

    def measure_device_latency(self, region, *inputs, reps: int = 100, warmup: int = 10):
        """Mean device time in ms of ``run`` on device-resident operands (CUDA events)."""
        staged = [DeviceArray.from_host(np.ascontiguousarray(x).astype(_storage(region)))
                  if isinstance(x, np.ndarray) and x.ndim >= 2 else x for x in inputs]
        for _ in range(warmup):
            self._run_device(region, *staged)
        a, b = device.Event(), device.Event()
        a.record()
        for _ in range(reps):
            self._run_device(region, *staged)
        b.record()
        b.synchronize()
        return a.elapsed_ms(b) / reps

    def run(self, region, *inputs, **kwargs):
        out = self._run_device(region, *inputs, **kwargs)
        host = out.download() if isinstance(out, DeviceArray) else out
        device.check_device_error(self.name)
        return np.asarray(host, np.float32), EXECUTION_TAG


class Sm100Matmul(_Sm100Candidate):
    name = "sm100_tcgen05_gemm"
    op = OP_MATMUL
    mma_prefer_shape = (128, 256, 16)

    def _run_device(self, region, A, B, **_):
        dt = _storage(region)
        return ops.gemm(_as(A, dt), _as(B, dt), out_dtype=np.float32)


class Sm100FusedGemm(_Sm100Candidate):
    name = "sm100_tcgen05_gemm_epilogue"
    op = OP_FUSED_REGION
    mma_prefer_shape = (128, 256, 16)
    _ACTS = ("relu", "gelu", "silu")

    def applies_to(self, region) -> bool:
        ep = tuple(getattr(region, "epilogue", ()))
        if getattr(region, "reduction", None) or tuple(getattr(region, "prologue", ())):
            return False
        acts = [e for e in ep if e != "bias"]
        if any(a not in self._ACTS for a in acts) or len(acts) > 1 or ep.count("bias") > 1:
            return False
        if "bias" in ep and ep[0] != "bias":
            return False
        # the kernel adds the residual before the activation; the region adds it after
        if getattr(region, "residual", False) and acts:
            return False
        try:
            _storage(region)
        except ValueError:
            return False
        return True

    def _run_device(self, region, A, B, bias=None, residual=None, **_):
        if not self.applies_to(region):
            raise ValueError(f"{self.name}: region {region!r} is not served")
        dt = _storage(region)
        ep = tuple(getattr(region, "epilogue", ()))
        acts = [e for e in ep if e != "bias"]
        spec = {"activation": acts[0] if acts else "linear"}
        if "bias" in ep:
            if bias is None:
                raise ValueError(f"{self.name}: the region has a bias epilogue but no bias was given")
            spec["bias"] = bias
        if getattr(region, "residual", False):
            if residual is None:
                raise ValueError(f"{self.name}: the region has a residual but none was given")
            spec["residual"] = residual
        return ops.gemm(_as(A, dt), _as(B, dt), epilogue=spec, out_dtype=np.float32)


class Sm100Attention(_Sm100Candidate):
    name = "sm100_tcgen05_flash_attn"
    op = OP_ATTENTION

    def applies_to(self, region) -> bool:
        try:
            return _storage(region) == bfloat16 and not getattr(region, "q_transposed", False) \
                and not getattr(region, "k_transposed", False)
        except ValueError:
            return False

    def _run_device(self, region, Q, K, V, **_):
        q, k, v = (ops._unwrap(t) for t in (Q, K, V))
        if len(q.shape) != 2 or len(k.shape) != 2 or len(v.shape) != 2:
            raise ValueError(f"{self.name}: the region is single-head: Q (M,D), K (Nk,D), V (Nk,Dv)")
        if q.shape[1] != 128 or v.shape[1] != 128:
            raise ValueError(f"{self.name}: head dimension must be 128")
        causal = bool(getattr(region, "causal", False))
        if causal and q.shape[0] != k.shape[0]:
            # the region masks n > m (top-left); the kernel's mask is bottom-right aligned
            raise ValueError(f"{self.name}: causal regions need M == Nk")
        dq, dk, dv = (_as(t, bfloat16) for t in (q, k, v))
        out = DeviceArray((1, 1, q.shape[0], 128), bfloat16)
        _lib.call("tessera_sm100_flash_attn_device", dq.ptr, dk.ptr, dv.ptr, out.ptr, 1, 1, 1, q.shape[0],
                  k.shape[0], 128, float(getattr(region, "scale", 1.0)), int(causal), None)
        return out.view((q.shape[0], 128))


class Sm100GatedMatmul(_Sm100Candidate):
    name = "sm100_tcgen05_swiglu_gate"
    op = OP_GATED_MATMUL

    def applies_to(self, region) -> bool:
        try:
            _storage(region)
        except ValueError:
            return False
        return getattr(region, "gate_act", "silu") == "silu"

    def _run_device(self, region, A, Wg, Wu, **_):
        if not self.applies_to(region):
            raise ValueError(f"{self.name}: only the silu gate is served")
        dt = _storage(region)
        a, wg, wu = (_as(t, dt) for t in (A, Wg, Wu))
        M, K = a.shape
        H = wg.shape[1]
        if tuple(wg.shape) != (K, H) or tuple(wu.shape) != (K, H):
            raise ValueError(f"{self.name}: expected A (M,K), Wg and Wu (K,H)")
        off = DeviceArray.from_host(np.array([0, M], np.int32))
        out = DeviceArray((M, H), dt)
        code = device.dtype_code(dt)
        _lib.call("tessera_sm100_grouped_swiglu_device", a.ptr, wg.ptr, wu.ptr, off.ptr, out.ptr, M, K, H, 1,
                  code, code, None)
        return out


def _as(x, dt) -> DeviceArray:
    x = ops._unwrap(x)
    if isinstance(x, DeviceArray):
        if x.dtype != dt:
            raise TypeError(f"device operand has dtype {x.dtype}, expected {dt}")
        return x
    return DeviceArray.from_host(np.ascontiguousarray(x).astype(dt))


# ------------------------------------------------------------------ registry + arbiter
_CANDIDATES: dict = {}


class ArbiterError(RuntimeError):
    pass


def register_candidate(candidate: Candidate) -> None:
    """Same-name registration in an ``(target, op)`` bucket replaces (candidate.py:199-226)."""
    if not candidate.target or not candidate.name:
        raise ValueError("Candidate.target and Candidate.name must be non-empty")
    if candidate.op not in _OPS:
        raise ValueError(f"unknown Candidate.op {candidate.op!r}")
    bucket = _CANDIDATES.setdefault((candidate.target, candidate.op), [])
    for i, existing in enumerate(bucket):
        if existing.name == candidate.name:
            bucket[i] = candidate
            return
    bucket.append(candidate)


def candidates_for(target: str, op: str) -> list:
    return list(_CANDIDATES.get((target, op), ()))


def arbitrate(target: str, op: str, region: Any, *, measure: Optional[Callable[[Candidate], float]] = None,
              force: Optional[str] = None) -> Candidate:
    """Pick a candidate: ``force`` by name, else the lowest ``measure`` (e.g. device latency),
    else the highest tier among those available and applicable."""
    pool = [c for c in candidates_for(target, op) if c.available() and c.applies_to(region)]
    if force is not None:
        for c in pool:
            if c.name == force:
                return c
        raise ArbiterError(f"forced candidate {force!r} is not available for ({target}, {op})")
    if not pool:
        raise ArbiterError(f"no candidate can serve ({target}, {op}) for {region!r}")
    if measure is not None:
        return min(pool, key=measure)
    return max(pool, key=lambda c: int(c.tier))


def run_arbitrated(target: str, op: str, region: Any, *inputs: Any, **kwargs: Any):
    """-> (output, execution_tag, candidate_name)"""
    c = arbitrate(target, op, region, force=kwargs.pop("force", None))
    out, tag = c.run(region, *inputs, **kwargs)
    return out, tag, c.name


def register_sm100_candidates() -> list:
    """Register the four sm_100a candidates under target ``"nvidia"``; returns them."""
    cs = [Sm100Matmul(), Sm100FusedGemm(), Sm100Attention(), Sm100GatedMatmul()]
    for c in cs:
        register_candidate(c)
    return cs


__all__ = ["Tier", "Candidate", "ArbiterError", "MatmulRegion", "FusedRegion", "AttentionRegion",
           "GatedMatmulRegion", "Sm100Matmul", "Sm100FusedGemm", "Sm100Attention", "Sm100GatedMatmul",
           "register_candidate", "candidates_for", "arbitrate", "run_arbitrated", "register_sm100_candidates",
           "EXECUTION_TAG", "OP_MATMUL", "OP_FUSED_REGION", "OP_ATTENTION", "OP_GATED_MATMUL"]
