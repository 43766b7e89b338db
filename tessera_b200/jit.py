"""``@jit`` for the B200 backend (decorator surface of python/tessera/compiler/jit.py:2774-3103).

The reference lowers the function body to Graph IR and, for ``target="nvidia_sm100"``, stops at
Target-IR text. Here a ``JitFn`` executes the body with ``tessera.ops`` bound to the sm_100a
kernels: 16-bit array arguments are uploaded once, intermediates stay in device memory across
ops, and results are downloaded on return. ``runtime_artifact()`` stamps the same metadata keys
the reference's NVIDIA branch stamps (:2269-2295) so ``runtime.launch`` can run single-op bodies.
There is no CPU path: ``target="cpu"`` raises.
"""
from __future__ import annotations

import ast
import functools
import inspect
import textwrap
from typing import Any, Callable, Dict, Optional, Sequence

import numpy as np

from . import runtime as _rt
from .device import DeviceArray, bfloat16


class TesseraJitError(RuntimeError):
    pass


def _scan_ops(fn: Callable, source: Optional[str]) -> list:
    """Find ``<anything>.ops.<name>(...)`` calls in the body, in source order."""
    try:
        text = source if source is not None else textwrap.dedent(inspect.getsource(fn))
        tree = ast.parse(text)
    except (OSError, TypeError, SyntaxError, IndentationError):
        return []
    found = []
    for node in ast.walk(tree):
        if isinstance(node, ast.Call) and isinstance(node.func, ast.Attribute):
            owner = node.func.value
            if isinstance(owner, ast.Attribute) and owner.attr == "ops" or \
                    isinstance(owner, ast.Name) and owner.id == "ops":
                operands = [a.id for a in node.args if isinstance(a, ast.Name)]
                kwargs = {}
                for kw in node.keywords:
                    try:
                        kwargs[kw.arg] = ast.literal_eval(kw.value)
                    except Exception:
                        pass
                found.append({"op_name": f"tessera.{node.func.attr}", "operands": operands,
                              "kwargs": kwargs, "lineno": node.lineno})
    found.sort(key=lambda d: d["lineno"])
    for d in found:
        d.pop("lineno")
    return found


class JitFn:
    def __init__(self, fn: Callable, *, target: str, deterministic: bool, seed: Optional[int],
                 source: Optional[str]) -> None:
        self._fn = fn
        self.target = target
        self.deterministic = deterministic
        self.seed = seed
        self.name = fn.__name__
        self.arg_names = list(inspect.signature(fn).parameters)
        self.ops = _scan_ops(fn, source)
        self.execution_kind = "native_gpu"
        self.last_fallback_reason = None
        functools.update_wrapper(self, fn)

    def runtime_artifact(self) -> _rt.RuntimeArtifact:
        if len(self.ops) == 1:
            op = self.ops[0]
            try:
                return _rt.make_artifact(op["op_name"], self.arg_names, op["operands"], op["kwargs"])
            except ValueError:
                pass
        meta = {"target": _rt.TARGET, "compiler_path": "sm100_eager_graph", "executable": False,
                "execution_kind": "native_gpu", "arg_names": self.arg_names,
                "ops": [dict(o, result=f"v{i}") for i, o in enumerate(self.ops)],
                "reason": "multi-op bodies run through JitFn.__call__, not through launch()"}
        return _rt.RuntimeArtifact(metadata=meta, abi_signature=f"tessera.runtime.v1.{_rt.TARGET}")

    @staticmethod
    def _stage(value: Any) -> Any:
        data = value._data if hasattr(value, "_data") else value
        if isinstance(data, np.ndarray) and data.ndim >= 2 and data.dtype in (np.float16, bfloat16):
            return DeviceArray.from_host(data)
        return value

    @staticmethod
    def _unstage(value: Any) -> Any:
        from .device import StridedView
        if isinstance(value, (DeviceArray, StridedView)):
            from . import device
            host = value.download()
            device.check_device_error("jit")
            return host
        if isinstance(value, tuple):
            return tuple(JitFn._unstage(v) for v in value)
        if isinstance(value, list):
            return [JitFn._unstage(v) for v in value]
        return value

    def __call__(self, *args: Any, **kwargs: Any) -> Any:
        staged = [self._stage(a) for a in args]
        skw = {k: self._stage(v) for k, v in kwargs.items()}
        return self._unstage(self._fn(*staged, **skw))

    def __repr__(self) -> str:
        return f"<JitFn {self.name!r} target={self.target!r}>"


def jit(fn: Optional[Callable] = None, *, deterministic: bool = False, seed: Optional[int] = None,
        bindings: Optional[Dict[str, int]] = None, target: Optional[Any] = None,
        source: Optional[str] = None, **_ignored: Any) -> Any:
    """Decorator, usable bare or with arguments. ``target`` may be ``None`` or any spelling of the
    sm_100 family (``"nvidia_sm100"``, ``"sm_100a"``, ``"blackwell"`` ...)."""
    tname = _rt.TARGET if target is None else _rt.normalize_target(target)
    if tname != _rt.TARGET:
        raise TesseraJitError(f"target {target!r} is not served by the sm_100a backend (there is no "
                              f"CPU or other-GPU path here); use target={_rt.TARGET!r}")

    def decorate(f: Callable) -> JitFn:
        return JitFn(f, target=tname, deterministic=deterministic, seed=seed, source=source)

    return decorate(fn) if fn is not None else decorate
