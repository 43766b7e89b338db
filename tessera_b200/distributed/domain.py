"""Domains (logical shapes) and distributions (placement over a mesh). API of
python/tessera/distributed/domain.py:29-227: ``Block`` maps mesh axis i to tensor dimension i."""
from __future__ import annotations

from math import prod
from typing import Tuple

from .shard import ShardSpec


class Domain:
    @property
    def shape(self) -> Tuple[int, ...]:
        raise NotImplementedError

    @property
    def rank(self) -> int:
        return len(self.shape)


class Rect(Domain):
    """Dense rectangular domain."""

    def __init__(self, dims: Tuple[int, ...]) -> None:
        if not dims:
            raise ValueError("Rect domain must have at least one dimension")
        for i, d in enumerate(dims):
            if not isinstance(d, int) or isinstance(d, bool) or d < 1:
                raise ValueError(f"Rect dimension {i} must be a positive integer, got {d!r}")
        self._dims = tuple(dims)

    @property
    def shape(self) -> Tuple[int, ...]:
        return self._dims

    @property
    def numel(self) -> int:
        return prod(self._dims)

    def __eq__(self, other) -> bool:
        return isinstance(other, Rect) and other._dims == self._dims

    def __hash__(self) -> int:
        return hash(self._dims)

    def __repr__(self) -> str:
        return f"Rect({self._dims})"


class Distribution:
    def make_shard_spec(self, domain: Domain) -> ShardSpec:
        raise NotImplementedError

def _check_axes(mesh_axes, what: str) -> Tuple[str, ...]:
    if not mesh_axes:
        raise ValueError(f"{what} distribution requires at least one mesh axis")
    if isinstance(mesh_axes, str):
        raise TypeError(f"{what}: mesh_axes must be a tuple of axis names, not a string")
    return tuple(mesh_axes)


class Block(Distribution):
    """Contiguous blocks: tensor dimension i is split over ``mesh_axes[i]``."""

    def __init__(self, mesh_axes: Tuple[str, ...]) -> None:
        self.mesh_axes = _check_axes(mesh_axes, "Block")

    def make_shard_spec(self, domain: Domain) -> ShardSpec:
        if len(self.mesh_axes) > domain.rank:
            raise ValueError(f"Block has {len(self.mesh_axes)} mesh axes but the domain has rank "
                             f"{domain.rank}")
        return ShardSpec(partition=tuple(range(len(self.mesh_axes))), mesh_axes=self.mesh_axes)

    def __repr__(self) -> str:
        return f"Block(mesh_axes={self.mesh_axes})"


class Cyclic(Distribution):
    """Round-robin placement along the leading dimensions."""

    def __init__(self, mesh_axes: Tuple[str, ...]) -> None:
        self.mesh_axes = _check_axes(mesh_axes, "Cyclic")

    def make_shard_spec(self, domain: Domain) -> ShardSpec:
        if len(self.mesh_axes) > domain.rank:
            raise ValueError(f"Cyclic has {len(self.mesh_axes)} mesh axes but the domain has rank "
                             f"{domain.rank}")
        return ShardSpec.cyclic_shard(tuple(range(len(self.mesh_axes))), self.mesh_axes)

    def __repr__(self) -> str:
        return f"Cyclic(mesh_axes={self.mesh_axes})"


class Replicated(Distribution):
    def make_shard_spec(self, domain: Domain) -> ShardSpec:
        return ShardSpec.replicate()

    def __repr__(self) -> str:
        return "Replicated()"
