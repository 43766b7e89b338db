"""``@kernel`` and ``index_launch``: fan a kernel out over the shards of a mesh axis
(python/tessera/distributed/launch.py:32-193).

The reference runs the per-rank calls one after another on the CPU. Here rank ``r`` runs with
CUDA device ``r mod device_count`` current, so ``ops`` calls inside the kernel body execute on
that rank's GPU; list-of-ndarray fan-out, scalar broadcast and the length checks are unchanged.
"""
from __future__ import annotations

import functools
from typing import Any, Callable, List, Optional

from .array import DistributedArray


class KernelFn:
    def __init__(self, fn: Callable, name: Optional[str] = None) -> None:
        self._fn = fn
        self.name = name or fn.__name__
        functools.update_wrapper(self, fn)

    def __call__(self, *args: Any, **kwargs: Any) -> Any:
        return self._fn(*args, **kwargs)

    def __repr__(self) -> str:
        return f"<TesseraKernel {self.name!r}>"


def kernel(fn: Callable) -> KernelFn:
    return KernelFn(fn)


def _device_count() -> int:
    try:
        from .. import device
        return device.device_count()
    except Exception:
        return 0


class _ShardDispatcher:
    def __init__(self, fn: Callable, axis: str) -> None:
        self._fn = fn
        self.axis = axis

    def __call__(self, *shard_lists: Any) -> List[Any]:
        lists: list = []
        for arg in shard_lists:
            if isinstance(arg, list):
                lists.append(arg)
            elif isinstance(arg, DistributedArray):
                lists.append(arg.parts(self.axis))
            else:
                lists.append(None)  # replicated to every rank
        n_ranks = next((len(p) for p in lists if p is not None), None)
        if n_ranks is None:
            raise ValueError("index_launch requires at least one list-of-shards argument")
        for i, p in enumerate(lists):
            if p is not None and len(p) != n_ranks:
                raise ValueError(f"Shard list {i} has {len(p)} entries but expected {n_ranks} "
                                 f"(from axis {self.axis!r})")
        ndev = _device_count()
        results = []
        for r in range(n_ranks):
            if ndev > 1:
                from .. import device
                device.set_device(r % ndev)
            args = [p[r] if p is not None else shard_lists[i] for i, p in enumerate(lists)]
            results.append(self._fn(*args))
        if ndev > 1:
            from .. import device
            device.set_device(0)
        return results

    def __repr__(self) -> str:
        name = getattr(self._fn, "name", getattr(self._fn, "__name__", "?"))
        return f"<ShardDispatcher kernel={name!r} axis={self.axis!r}>"


class IndexLauncher:
    def __init__(self, axis: str) -> None:
        self.axis = axis

    def __call__(self, fn: Callable) -> _ShardDispatcher:
        return _ShardDispatcher(fn=fn, axis=self.axis)

    def __repr__(self) -> str:
        return f"IndexLauncher(axis={self.axis!r})"


def index_launch(axis: str) -> IndexLauncher:
    return IndexLauncher(axis=axis)
