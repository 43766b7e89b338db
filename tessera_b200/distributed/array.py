"""``DistributedArray``: a host array plus shard metadata. API of
python/tessera/distributed/array.py:78-283, with two additions the README sketch of the reference
needs (its own class lacks them): ``__setitem__``/``__getitem__`` that write through to the
backing array, and a real bfloat16 backing store (the reference keeps "bf16" as float32,
:35-36) so shards can be handed to the GPU kernels without a conversion pass."""
from __future__ import annotations

from typing import Any, List, Optional, Tuple

import numpy as np

from ..device import bfloat16
from .domain import Distribution, Domain
from .shard import MeshSpec, ShardSpec

_ALIASES = {
    "bf16": "bf16", "bfloat16": "bf16",
    "fp16": "fp16", "f16": "fp16", "float16": "fp16", "half": "fp16",
    "fp32": "fp32", "f32": "fp32", "float32": "fp32",
    "fp64": "fp64", "f64": "fp64", "float64": "fp64",
    "int8": "int8", "i8": "int8", "int16": "int16", "i16": "int16",
    "int32": "int32", "i32": "int32", "int64": "int64", "i64": "int64",
    "uint8": "uint8", "u8": "uint8", "bool": "bool",
}
_DTYPE_MAP = {
    "bf16": bfloat16 if bfloat16 is not None else np.dtype(np.float32),
    "fp16": np.dtype(np.float16), "fp32": np.dtype(np.float32), "fp64": np.dtype(np.float64),
    "int8": np.dtype(np.int8), "int16": np.dtype(np.int16), "int32": np.dtype(np.int32),
    "int64": np.dtype(np.int64), "uint8": np.dtype(np.uint8), "bool": np.dtype(np.bool_),
}


def _normalize_dtype(dtype: str) -> str:
    try:
        return _ALIASES[str(dtype).lower()]
    except KeyError:
        raise ValueError(f"Tessera dtype {dtype!r} has no storage backing in this DistributedArray "
                         f"runtime. Backed dtypes: {sorted(_DTYPE_MAP)}.") from None


class DistributedArray:
    def __init__(self, data: np.ndarray, dtype: str, shard_spec: ShardSpec,
                 logical_shape: Optional[Tuple[int, ...]] = None) -> None:
        self.dtype = _normalize_dtype(dtype)
        self._data = data
        self.shard_spec = shard_spec
        self.shape: Tuple[int, ...] = tuple(logical_shape) if logical_shape is not None \
            else tuple(data.shape)
        self._mesh_size_cache: dict = {}

    @classmethod
    def from_domain(cls, domain: Domain, dtype: str, distribution: Distribution,
                    fill: str = "zeros", mesh: Optional[MeshSpec] = None) -> "DistributedArray":
        name = _normalize_dtype(dtype)
        spec = distribution.make_shard_spec(domain)
        if mesh is not None and not spec.replicated:
            for dim in spec.partition:
                spec.shard_size(dim, domain.shape[dim], mesh)  # raises when not divisible
        np_dtype = _DTYPE_MAP[name]
        shape = domain.shape
        if fill == "zeros":
            data = np.zeros(shape, np_dtype)
        elif fill == "ones":
            data = np.ones(shape, np_dtype)
        elif fill == "randn":
            data = np.random.randn(*shape).astype(np_dtype)
        elif fill == "empty":
            data = np.empty(shape, np_dtype)
        else:
            raise ValueError(f"Unknown fill strategy {fill!r}. Use 'zeros', 'ones', 'randn', 'empty'.")
        out = cls(data=data, dtype=name, shard_spec=spec, logical_shape=shape)
        if mesh is not None:
            out._bind_mesh(mesh)
        return out

    def _bind_mesh(self, mesh: MeshSpec) -> "DistributedArray":
        self._mesh_size_cache = {a: mesh.axis_size(a) for a in self.shard_spec.mesh_axes}
        return self

    def parts(self, axis: str) -> List["DistributedArray"]:
        """Per-rank shards along mesh axis ``axis``. Block shards are views of the backing array,
        so writing into a shard writes into the parent (``np.array_split`` semantics)."""
        spec = self.shard_spec
        if spec.replicated:
            return [self]
        if axis not in spec.mesh_axes:
            raise ValueError(f"Array is not partitioned over axis {axis!r}. Partitioned axes: "
                             f"{spec.mesh_axes}")
        dim = spec.partition[spec.mesh_axes.index(axis)]
        if axis not in self._mesh_size_cache:
            raise ValueError(f"Mesh axis {axis!r} has no bound size; bind the mesh (e.g. via "
                             f"_bind_mesh) before calling parts({axis!r}).")
        n = self._mesh_size_cache[axis]
        size = self.shape[dim]
        if spec.cyclic:
            subs = []
            for r in range(n):
                idx = list(range(r, size, n))
                if idx:
                    subs.append(np.take(self._data, idx, axis=dim))
                else:
                    shp = list(self._data.shape)
                    shp[dim] = 0
                    subs.append(np.empty(shp, self._data.dtype))
        else:
            if size % n:
                raise ValueError(f"Cannot evenly split dimension {dim} of size {size} into {n} parts "
                                 f"for axis {axis!r}")
            subs = np.array_split(self._data, n, axis=dim)
        return [DistributedArray(data=s, dtype=self.dtype, shard_spec=ShardSpec.replicate(),
                                 logical_shape=tuple(s.shape)) for s in subs]

    # write-through indexing (not in the reference class)
    def __setitem__(self, key, value) -> None:
        if hasattr(value, "_data"):
            value = value._data
        elif hasattr(value, "numpy") and callable(value.numpy):
            value = value.numpy()
        self._data[key] = np.asarray(value).astype(self._data.dtype, copy=False)

    def __getitem__(self, key) -> Any:
        return self._data[key]

    @property
    def ndim(self) -> int:
        return len(self.shape)

    @property
    def numel(self) -> int:
        return int(np.prod(self.shape, dtype=np.int64))

    def numpy(self) -> np.ndarray:
        return self._data

    def __repr__(self) -> str:
        return f"DistributedArray(shape={self.shape}, dtype={self.dtype!r}, shard={self.shard_spec})"
