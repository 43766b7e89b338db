"""Distributed programming surface: regions, domains, distributions, arrays, index_launch
(python/tessera/distributed/__init__.py)."""
import types

from .array import DistributedArray
from .domain import Block, Cyclic, Rect, Replicated
from .launch import index_launch, kernel
from .region import Region
from .shard import MeshSpec, ShardSpec

domain = types.SimpleNamespace(Rect=Rect)
dist = types.SimpleNamespace(Block=Block, Cyclic=Cyclic, Replicated=Replicated)
array = types.SimpleNamespace(from_domain=DistributedArray.from_domain)

__all__ = ["Region", "ShardSpec", "MeshSpec", "Rect", "Block", "Cyclic", "Replicated",
           "DistributedArray", "index_launch", "kernel", "domain", "dist", "array"]
