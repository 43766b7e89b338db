"""``@kernel`` and ``index_launch``: fan a kernel out over the shards of a mesh axis
(python/tessera/distributed/launch.py:32-193).

The reference runs the per-rank calls one after another on the CPU. Here rank ``r`` runs with
CUDA device ``r mod device_count`` current, so ``ops`` calls inside the kernel body execute on
that rank's GPU, and with more than one GPU the ranks are issued concurrently: one host thread
per GPU walks that GPU's ranks in order (the C ABI releases the interpreter lock, the current
device and the error string are per thread), and the call returns when every rank has finished.
Shards are independent by construction, so the results are those of the sequential loop;
list-of-ndarray fan-out, scalar broadcast and the length checks are unchanged.
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

        def rank_args(r):
            return [p[r] if p is not None else shard_lists[i] for i, p in enumerate(lists)]

        if ndev <= 1 or n_ranks <= 1:
            return [self._fn(*rank_args(r)) for r in range(n_ranks)]
        from concurrent.futures import ThreadPoolExecutor
        from .. import device
        results: list = [None] * n_ranks
        errors: list = [None] * n_ranks

        def run_device(d):
            device.set_device(d)
            for r in range(d, n_ranks, ndev):
                try:
                    results[r] = self._fn(*rank_args(r))
                except BaseException as exc:  # reported in rank order below
                    errors[r] = exc

        used = min(ndev, n_ranks)
        with ThreadPoolExecutor(max_workers=used) as pool:
            list(pool.map(run_device, range(used)))
        for exc in errors:
            if exc is not None:
                raise exc
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
