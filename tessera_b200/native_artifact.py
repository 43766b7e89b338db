"""Descriptor types of the native launch seam: what ``register_native_launcher``'s ``submit`` hook
receives and what ``runtime.launch`` checks before it calls the hook.

The contract follows the reference's ``python/tessera/compiler/native_artifact.py`` (types at
:250-470 and :466-760, ``LaunchDescriptor.validate_invocation`` at :997-1051; consumed by
``_launch_native_descriptor``, python/tessera/runtime.py:30905-30990): a native image names its entry
points and their ABI ids; a launch descriptor names one entry point and the buffers and scalars
it takes; before anything is submitted, the runtime checks that the descriptor belongs to the image
and that the caller's buffers match the bindings (names, dtype, rank, layout, address alignment,
shape guards). Violations raise :class:`ArtifactContractError` with the reference's diagnostic
codes, which ``launch`` turns into an ``invalid_artifact`` result. Only what this backend's seam
needs is modelled: no pipeline registry, resource records or device libraries.
"""
from __future__ import annotations

import hashlib
import json
from dataclasses import dataclass, field
from typing import Mapping, Optional, Tuple

import numpy as np

NATIVE_IMAGE_FORMATS = frozenset({"ptx", "cubin", "hsaco", "elf", "object", "shared_object", "metallib", "spirv"})
DIRECTIONS = frozenset({"input", "output", "inout"})
SHAPE_PREDICATES = {"eq": lambda d, v: d == v, "min": lambda d, v: d >= v, "max": lambda d, v: d <= v,
                    "multiple_of": lambda d, v: d % v == 0}
_DTYPES = {"fp32": "fp32", "f32": "fp32", "float32": "fp32", "fp16": "fp16", "f16": "fp16", "float16": "fp16",
           "bf16": "bf16", "bfloat16": "bf16", "int32": "int32", "i32": "int32", "int64": "int64", "i64": "int64",
           "int8": "int8", "uint8": "uint8", "bool": "bool", "fp8_e4m3": "fp8_e4m3", "fp8_e5m2": "fp8_e5m2"}


class ArtifactContractError(ValueError):
    """A descriptor, image or invocation breaks the launch contract; ``code`` is the diagnostic id."""

    def __init__(self, code: str, message: str) -> None:
        super().__init__(f"{code}: {message}")
        self.code = code


def canonical_dtype(name, code: str, what: str) -> str:
    key = str(np.dtype(name)) if not isinstance(name, str) else name
    try:
        return _DTYPES[key.lower()]
    except KeyError:
        raise ArtifactContractError(code, f"{what} has invalid dtype {name!r}") from None


def _natural(value, code: str, what: str, positive: bool = False) -> int:
    if not isinstance(value, int) or isinstance(value, bool) or value < (1 if positive else 0):
        raise ArtifactContractError(code, f"{what} must be a {'positive' if positive else 'non-negative'} integer")
    return value


def _digest(obj) -> str:
    return hashlib.sha256(json.dumps(obj, sort_keys=True, separators=(",", ":")).encode()).hexdigest()


@dataclass(frozen=True)
class NativeEntryPoint:
    symbol: str
    abi_id: str

    def __post_init__(self) -> None:
        if not self.symbol or not self.abi_id:
            raise ArtifactContractError("E_NATIVE_IMAGE_SCHEMA", "entry point needs a symbol and an ABI id")


@dataclass(frozen=True)
class NativeImageArtifact:
    target: str
    architecture: str
    binary_format: str
    payload: bytes
    entry_points: Tuple[NativeEntryPoint, ...]

    def __post_init__(self) -> None:
        from .runtime import normalize_target
        object.__setattr__(self, "target", normalize_target(self.target))
        if not self.architecture:
            raise ArtifactContractError("E_NATIVE_IMAGE_SCHEMA", "exact architecture must be non-empty")
        if self.binary_format not in NATIVE_IMAGE_FORMATS:
            raise ArtifactContractError("E_NATIVE_IMAGE_SCHEMA", f"binary format {self.binary_format!r} is not registered")
        if not isinstance(self.payload, bytes) or not self.payload:
            raise ArtifactContractError("E_NATIVE_IMAGE_SCHEMA", "native payload must be non-empty bytes")
        entries = tuple(self.entry_points)
        if not entries or any(not isinstance(e, NativeEntryPoint) for e in entries):
            raise ArtifactContractError("E_NATIVE_IMAGE_SCHEMA", "a native image needs NativeEntryPoint values")
        if len({e.symbol for e in entries}) != len(entries):
            raise ArtifactContractError("E_NATIVE_IMAGE_SCHEMA", "native image has duplicate entry symbols")
        object.__setattr__(self, "entry_points", entries)

    @property
    def image_digest(self) -> str:
        return _digest({"target": self.target, "architecture": self.architecture, "format": self.binary_format,
                        "payload": hashlib.sha256(self.payload).hexdigest(),
                        "entries": [[e.symbol, e.abi_id] for e in self.entry_points]})

    def entry_point(self, symbol: str) -> Optional[NativeEntryPoint]:
        return next((e for e in self.entry_points if e.symbol == symbol), None)


@dataclass(frozen=True)
class BufferBinding:
    ordinal: int
    name: str
    direction: str
    dtype: str
    rank: int
    layout: str
    alignment: int = 1

    def __post_init__(self) -> None:
        code = "E_LAUNCH_DESCRIPTOR_SCHEMA"
        _natural(self.ordinal, code, "buffer ordinal")
        if not isinstance(self.name, str) or not self.name:
            raise ArtifactContractError(code, "buffer name must be non-empty")
        if self.direction not in DIRECTIONS:
            raise ArtifactContractError(code, f"invalid buffer direction {self.direction!r}")
        object.__setattr__(self, "dtype", canonical_dtype(self.dtype, code, f"buffer {self.name}"))
        _natural(self.rank, code, "buffer rank")
        if not isinstance(self.layout, str) or not self.layout:
            raise ArtifactContractError(code, "buffer layout must be non-empty")
        _natural(self.alignment, code, "buffer alignment", positive=True)
        if self.alignment & (self.alignment - 1):
            raise ArtifactContractError(code, "buffer alignment must be a power of two")


@dataclass(frozen=True)
class ScalarArgument:
    ordinal: int
    name: str
    dtype: str

    def __post_init__(self) -> None:
        code = "E_LAUNCH_DESCRIPTOR_SCHEMA"
        _natural(self.ordinal, code, "scalar ordinal")
        if not isinstance(self.name, str) or not self.name:
            raise ArtifactContractError(code, "scalar name must be non-empty")
        object.__setattr__(self, "dtype", canonical_dtype(self.dtype, code, f"scalar {self.name}"))


@dataclass(frozen=True)
class ShapeGuard:
    binding: str
    dimension: int
    predicate: str
    value: int

    def __post_init__(self) -> None:
        code = "E_LAUNCH_DESCRIPTOR_SCHEMA"
        if not self.binding:
            raise ArtifactContractError(code, "shape guard binding must be non-empty")
        _natural(self.dimension, code, "shape guard dimension")
        if self.predicate not in SHAPE_PREDICATES:
            raise ArtifactContractError(code, f"invalid shape predicate {self.predicate!r}")
        _natural(self.value, code, "shape guard value", positive=True)


@dataclass(frozen=True)
class BufferArgument:
    """What the runtime knows about one caller buffer before submission."""
    dtype: str
    shape: Tuple[int, ...]
    layout: str = "row_major"
    address_alignment: int = 1

    def __post_init__(self) -> None:
        code = "E_LAUNCH_BINDING_MISMATCH"
        object.__setattr__(self, "dtype", canonical_dtype(self.dtype, code, "runtime buffer"))
        object.__setattr__(self, "shape", tuple(int(d) for d in self.shape))
        if any(d < 0 for d in self.shape):
            raise ArtifactContractError(code, "runtime shape dimensions must be non-negative")
        if not self.layout:
            raise ArtifactContractError(code, "runtime layout must be non-empty")
        _natural(self.address_alignment, code, "runtime alignment", positive=True)

    @classmethod
    def of(cls, value) -> "BufferArgument":
        """Contract of a numpy array or a device array (dense row-major; alignment from its address)."""
        if hasattr(value, "ptr"):
            addr = int(value.ptr)
        else:
            value = np.asarray(value)
            addr = int(value.ctypes.data)
        align = (addr & -addr) if addr else 1 << 12
        return cls(dtype=str(np.dtype(value.dtype)), shape=tuple(value.shape), address_alignment=min(align, 1 << 12))


@dataclass(frozen=True)
class LaunchDescriptor:
    image_digest: str
    entry_symbol: str
    abi_id: str
    buffers: Tuple[BufferBinding, ...]
    scalars: Tuple[ScalarArgument, ...] = ()
    shape_guards: Tuple[ShapeGuard, ...] = ()
    provenance: Mapping[str, object] = field(default_factory=dict)

    def __post_init__(self) -> None:
        code = "E_LAUNCH_DESCRIPTOR_SCHEMA"
        if not self.entry_symbol or not self.abi_id:
            raise ArtifactContractError(code, "descriptor needs an entry symbol and an ABI id")
        buffers, scalars = tuple(self.buffers), tuple(self.scalars)
        if any(not isinstance(b, BufferBinding) for b in buffers) or any(not isinstance(s, ScalarArgument) for s in scalars):
            raise ArtifactContractError(code, "buffers / scalars must be BufferBinding / ScalarArgument values")
        ordinals = [b.ordinal for b in buffers] + [s.ordinal for s in scalars]
        if sorted(ordinals) != list(range(len(ordinals))):
            raise ArtifactContractError(code, "argument ordinals must be 0..n-1 without gaps or repeats")
        names = [b.name for b in buffers] + [s.name for s in scalars]
        if len(set(names)) != len(names):
            raise ArtifactContractError(code, "argument names must be unique")
        known = {b.name: b for b in buffers}
        for g in self.shape_guards:
            if g.binding not in known or g.dimension >= known[g.binding].rank:
                raise ArtifactContractError(code, f"shape guard names {g.binding}[{g.dimension}], which is not bound")
        object.__setattr__(self, "buffers", buffers)
        object.__setattr__(self, "scalars", scalars)
        object.__setattr__(self, "shape_guards", tuple(self.shape_guards))

    @property
    def descriptor_digest(self) -> str:
        return _digest({"image": self.image_digest, "entry": self.entry_symbol, "abi": self.abi_id,
                        "buffers": [[b.ordinal, b.name, b.direction, b.dtype, b.rank, b.layout, b.alignment]
                                    for b in self.buffers],
                        "scalars": [[s.ordinal, s.name, s.dtype] for s in self.scalars],
                        "guards": [[g.binding, g.dimension, g.predicate, g.value] for g in self.shape_guards]})

    def argument_names(self) -> list:
        """Buffer and scalar names in ordinal order (how positional ``launch`` arguments bind)."""
        return [n for _, n in sorted([(b.ordinal, b.name) for b in self.buffers]
                                     + [(s.ordinal, s.name) for s in self.scalars])]

    def validate_image(self, image: NativeImageArtifact) -> None:
        if self.image_digest != image.image_digest:
            raise ArtifactContractError("E_LAUNCH_STALE_IMAGE", "launch descriptor references a different native image")
        entry = image.entry_point(self.entry_symbol)
        if entry is None:
            raise ArtifactContractError("E_LAUNCH_STALE_IMAGE", f"entry symbol {self.entry_symbol!r} is absent from the image")
        if entry.abi_id != self.abi_id:
            raise ArtifactContractError("E_LAUNCH_STALE_IMAGE", "launch ABI id does not match the image's entry point")

    def validate_invocation(self, image: NativeImageArtifact, buffers: Mapping[str, BufferArgument],
                            scalars: Mapping[str, object]) -> None:
        """Everything that can be checked before a backend sees the call."""
        code = "E_LAUNCH_BINDING_MISMATCH"
        self.validate_image(image)
        want_b, want_s = {b.name for b in self.buffers}, {s.name for s in self.scalars}
        if set(buffers) != want_b:
            raise ArtifactContractError(code, f"buffer names differ: expected {sorted(want_b)}, got {sorted(buffers)}")
        if set(scalars) != want_s:
            raise ArtifactContractError(code, f"scalar names differ: expected {sorted(want_s)}, got {sorted(scalars)}")
        for b in self.buffers:
            got = buffers[b.name]
            if got.dtype != b.dtype:
                raise ArtifactContractError(code, f"buffer {b.name!r} dtype mismatch ({got.dtype} for {b.dtype})")
            if len(got.shape) != b.rank:
                raise ArtifactContractError(code, f"buffer {b.name!r} rank mismatch")
            if got.layout != b.layout:
                raise ArtifactContractError(code, f"buffer {b.name!r} layout mismatch")
            if got.address_alignment % b.alignment:
                raise ArtifactContractError(code, f"buffer {b.name!r} alignment mismatch")
        for s in self.scalars:
            v = scalars[s.name]
            if s.dtype.startswith(("int", "uint")) and (not isinstance(v, (int, np.integer)) or isinstance(v, bool)):
                raise ArtifactContractError(code, f"scalar {s.name!r} requires an integer")
            if s.dtype.startswith(("fp", "bf")) and (not isinstance(v, (int, float, np.number)) or isinstance(v, bool)):
                raise ArtifactContractError(code, f"scalar {s.name!r} requires a number")
            if s.dtype == "bool" and not isinstance(v, (bool, np.bool_)):
                raise ArtifactContractError(code, f"scalar {s.name!r} requires bool")
        for g in self.shape_guards:
            dim = buffers[g.binding].shape[g.dimension]
            if not SHAPE_PREDICATES[g.predicate](dim, g.value):
                raise ArtifactContractError(code, f"shape guard failed for {g.binding}[{g.dimension}]: "
                                                  f"{g.predicate} {g.value}, got {dim}")


__all__ = ["ArtifactContractError", "BufferArgument", "BufferBinding", "LaunchDescriptor", "NATIVE_IMAGE_FORMATS",
           "NativeEntryPoint", "NativeImageArtifact", "ScalarArgument", "ShapeGuard"]
