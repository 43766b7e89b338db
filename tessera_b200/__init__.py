"""B200-native backend for Tessera's dense-contraction hot path.

``import tessera_b200 as tessera`` gives the part of the reference's Python surface that sits on
that path — ``tessera.jit``, ``tessera.kernel``, ``tessera.index_launch``, ``tessera.ops.gemm`` /
``flash_attn`` / ``grouped_gemm`` / ``moe_swiglu_block``, ``tessera.runtime.launch`` — with every
op executed by hand-written sm_100a kernels through a ctypes C ABI. Nothing here imports
PyTorch, and there is no CPU fallback.
"""
from . import cache, collectives, device, native_artifact, nn, ops, runtime
from .distributed import (Block, Cyclic, DistributedArray, MeshSpec, Rect, Region, Replicated,
                          ShardSpec, array, dist, domain, index_launch, kernel)
from .jit import JitFn, TesseraJitError, jit

__version__ = "0.1.0"


class _DTypeSentinel:
    """Inert annotation sentinels such as ``tessera.f16[..., ...]``
    (python/tessera/__init__.py:6027-6145): dtype and mutability come from the arrays."""

    def __init__(self, name: str) -> None:
        self.name = name

    def __getitem__(self, _item) -> "_DTypeSentinel":
        return self

    def __repr__(self) -> str:
        return f"tessera.{self.name}"


f16 = _DTypeSentinel("f16")
bf16 = _DTypeSentinel("bf16")
f32 = _DTypeSentinel("f32")
mut_f16 = _DTypeSentinel("mut_f16")
mut_bf16 = _DTypeSentinel("mut_bf16")
mut_f32 = _DTypeSentinel("mut_f32")

__all__ = ["ops", "cache", "runtime", "native_artifact", "collectives", "device", "nn", "jit", "JitFn", "TesseraJitError",
           "kernel", "index_launch", "DistributedArray", "ShardSpec", "MeshSpec", "Rect", "Block",
           "Cyclic", "Replicated", "Region", "domain", "dist", "array", "f16", "bf16", "f32",
           "mut_f16", "mut_bf16", "mut_f32"]
