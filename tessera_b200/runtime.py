"""Runtime dispatcher: ``RuntimeArtifact`` + ``launch()`` + the native-launcher registry, with an
execution row for ``target="nvidia_sm100"`` that the reference lacks (it stops at Target-IR text
and ``launch()`` answers ``missing_backend``; python/tessera/runtime.py:30993-31181,
python/tessera/compiler/capabilities.py:518-538).

Contracts kept from the reference:
* ``launch(kernel, args, stream=None)`` binds ``args`` (tuple/list by ``metadata["arg_names"]``,
  or a mapping by name; python/tessera/runtime.py:44363-44374), never raises for backend errors
  and returns a result dict with ``ok``, ``runtime_status``, ``compiler_path``,
  ``execution_kind``, ``artifact_hash``, ``output``/``reason`` (:31033-31077).
* executors raise; ``launch`` turns a raise into ``runtime_status="invalid_artifact"``.
* ``register_native_launcher(target, binary_formats=..., submit=...)`` (:279-299).
"""
from __future__ import annotations

import hashlib
import json
import time
from dataclasses import dataclass, field
from enum import IntEnum
from typing import Any, Callable, Mapping, Optional

import numpy as np

from . import _lib


class TsrStatus(IntEnum):
    """Status codes of the runtime C ABI (src/runtime/include/tessera/tsr_status.h)."""
    SUCCESS = 0
    INVALID_ARGUMENT = 1
    NOT_FOUND = 2
    ALREADY_EXISTS = 3
    OUT_OF_MEMORY = 4
    UNIMPLEMENTED = 5
    INTERNAL = 6
    DEVICE_ERROR = 7


@dataclass(frozen=True)
class RuntimeProfile:
    cpu_wall_ms: Optional[float] = None
    kernel_elapsed_ms: Optional[float] = None
    memory_bytes: Optional[int] = None
    launch_overhead_ms: Optional[float] = None


@dataclass(frozen=True)
class BackendCapability:
    name: str
    available: bool
    executable: bool
    reason: str = ""
    dtypes: tuple = ()
    features: tuple = ()


TARGET = "nvidia_sm100"
_TARGET_ALIASES = {
    "nvidia_sm100": TARGET, "sm100": TARGET, "sm_100": TARGET, "sm100a": TARGET,
    "sm_100a": TARGET, "blackwell": TARGET, "b200": TARGET,
}
COMPILER_PATHS = {
    "sm100_gemm": ("tessera.matmul", "tessera.gemm", "tessera.batched_gemm", "matmul", "gemm"),
    "sm100_flash_attn": ("tessera.flash_attn", "flash_attn", "tessera.gqa_attention"),
    "sm100_moe": ("tessera.grouped_gemm", "tessera.moe_swiglu_block", "tessera.moe_layer",
                  "tessera.moe_dispatch", "tessera.moe_combine"),
    "sm100_flash_attn_bwd": ("tessera.flash_attn", "flash_attn", "tessera.flash_attn_bwd",
                             "tessera.flash_attn_vjp"),
}


def normalize_target(target: Any) -> str:
    """Map a target spelling to its canonical name (python/tessera/compiler/capabilities.py:87-106).
    Only the sm_100 family normalises to this backend; ``None`` means the CPU path."""
    if target is None:
        return "cpu"
    name = str(getattr(target, "name", target)).lower()
    return _TARGET_ALIASES.get(name, name)


@dataclass(frozen=True)
class RuntimeArtifact:
    graph_ir: str = ""
    schedule_ir: str = ""
    tile_ir: str = ""
    target_ir: str = ""
    metadata: Optional[dict] = None
    abi_signature: str = ""
    native_image: Any = None
    launch_descriptor: Any = None

    def _payload(self) -> dict:
        return {"graph_ir": self.graph_ir, "schedule_ir": self.schedule_ir, "tile_ir": self.tile_ir,
                "target_ir": self.target_ir, "metadata": self.metadata or {},
                "abi_signature": self.abi_signature}

    @property
    def artifact_hash(self) -> str:
        return hashlib.sha256(json.dumps(self._payload(), sort_keys=True, default=str).encode()).hexdigest()

    def to_dict(self) -> dict:
        d = self._payload()
        d["artifact_hash"] = self.artifact_hash
        return d

    def to_json(self) -> str:
        return json.dumps(self.to_dict(), sort_keys=True, default=str)

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "RuntimeArtifact":
        meta = data.get("metadata") or {}
        if not isinstance(meta, Mapping):
            raise ValueError("runtime metadata must be an object")
        art = cls(graph_ir=data.get("graph_ir", ""), schedule_ir=data.get("schedule_ir", ""),
                  tile_ir=data.get("tile_ir", ""), target_ir=data.get("target_ir", ""),
                  metadata=dict(meta), abi_signature=data.get("abi_signature", ""))
        h = data.get("artifact_hash")
        if h is not None and h != art.artifact_hash:
            raise ValueError("runtime artifact hash does not match content")
        return art

    @classmethod
    def from_json(cls, payload) -> "RuntimeArtifact":
        if isinstance(payload, bytes):
            payload = payload.decode("utf-8")
        return cls.from_dict(json.loads(payload))


def load_artifact(kernel: Any) -> RuntimeArtifact:
    if isinstance(kernel, RuntimeArtifact):
        return kernel
    if hasattr(kernel, "runtime_artifact") and callable(kernel.runtime_artifact):
        return kernel.runtime_artifact()
    if isinstance(kernel, (str, bytes)):
        return RuntimeArtifact.from_json(kernel)
    if isinstance(kernel, Mapping):
        return RuntimeArtifact.from_dict(kernel)
    raise TypeError(f"cannot load a runtime artifact from {type(kernel).__name__}")


# --------------------------------------------------------------------------------- native launchers
@dataclass(frozen=True)
class NativeLauncherRegistration:
    target: str
    binary_formats: tuple
    submit: Callable


_native_launchers: dict = {}


def register_native_launcher(target: str, *, binary_formats: tuple, submit: Callable,
                             replace: bool = False) -> None:
    exact = normalize_target(target)
    if exact in _native_launchers and not replace:
        raise ValueError(f"native launcher already registered for {exact}")
    formats = tuple(binary_formats)
    if not formats or any(not isinstance(f, str) or not f for f in formats):
        raise ValueError("binary_formats must contain at least one non-empty format")
    _native_launchers[exact] = NativeLauncherRegistration(exact, formats, submit)


def unregister_native_launcher(target: str) -> None:
    _native_launchers.pop(normalize_target(target), None)


# --------------------------------------------------------------------------------- executors
def _bind_launch_args(args: Any, arg_names: list) -> dict:
    if isinstance(args, Mapping):
        return dict(args)
    if args is None:
        args = ()
    if not isinstance(args, (list, tuple)):
        args = (args,)
    values = {n: v for n, v in zip(arg_names, args)}
    if len(values) < len(arg_names):
        raise ValueError("launch args missing value(s): " + ", ".join(arg_names[len(values):]))
    return values


def _single_op(metadata: Mapping, accepted: tuple, who: str) -> Mapping:
    ops_list = list(metadata.get("ops") or [])
    if len(ops_list) != 1 or str(ops_list[0].get("op_name", "")) not in accepted:
        raise ValueError(f"{who} executor handles exactly one of {accepted}; got "
                         f"{[o.get('op_name') for o in ops_list]!r}")
    return ops_list[0]


def _execute_sm100_gemm(artifact: RuntimeArtifact, args: Any) -> Any:
    """One matmul/gemm op on the tcgen05 GEMM; returns the fp32 product like the reference's
    ``_execute_nvidia_mma_artifact`` (python/tessera/runtime.py:2264-2339)."""
    from . import ops
    meta = artifact.metadata or {}
    op = _single_op(meta, COMPILER_PATHS["sm100_gemm"], "sm100_gemm")
    names = [str(n) for n in op.get("operands", [])]
    if len(names) != 2:
        raise ValueError("matmul requires exactly two operands")
    values = _bind_launch_args(args, list(meta.get("arg_names") or []))
    kw = dict(op.get("kwargs") or {})
    return ops.gemm(values[names[0]], values[names[1]], out_dtype=kw.get("out_dtype"),
                    compute_dtype=kw.get("compute_dtype"))


def _execute_sm100_flash_attn(artifact: RuntimeArtifact, args: Any) -> Any:
    """One flash_attn op (python/tessera/runtime.py:9886-9932 for the argument conventions)."""
    from . import ops
    meta = artifact.metadata or {}
    op = _single_op(meta, COMPILER_PATHS["sm100_flash_attn"], "sm100_flash_attn")
    names = [str(n) for n in op.get("operands", [])]
    if len(names) not in (3, 4):
        raise ValueError("sm100 flash attention requires Q, K, V and optional bias")
    values = _bind_launch_args(args, list(meta.get("arg_names") or []))
    kw = dict(op.get("kwargs") or {})
    window = kw.get("window", None)
    if window is None and (kw.get("window_left") is not None or kw.get("window_right") is not None):
        window = (kw.get("window_left"), kw.get("window_right"))
    bias = values[names[3]] if len(names) == 4 else None
    if bias is not None and np.dtype(getattr(getattr(bias, "_data", bias), "dtype", np.float32)) != np.float32:
        raise ValueError("sm100 flash attention bias must use f32 storage")
    # the launch path masks key n > m (top-left), like the reference's executor and CUDA lane
    return ops.flash_attn(values[names[0]], values[names[1]], values[names[2]],
                          scale=kw.get("scale"), causal=bool(kw.get("causal", False)), attn_bias=bias,
                          window=window, softcap=kw.get("softcap", kw.get("logit_softcap", None)),
                          causal_alignment="top_left")


def _execute_sm100_flash_attn_bwd(artifact: RuntimeArtifact, args: Any) -> Any:
    """One attention VJP: operands ``(dO, Q, K, V[, bias])``, result ``(dQ, dK, dV)``
    (python/tessera/runtime.py:9935-9990)."""
    from . import ops
    meta = artifact.metadata or {}
    op = _single_op(meta, COMPILER_PATHS["sm100_flash_attn_bwd"], "sm100_flash_attn_bwd")
    names = [str(n) for n in op.get("operands", [])]
    if len(names) not in (4, 5):
        raise ValueError("sm100 flash backward requires dO, Q, K, V and optional bias")
    values = _bind_launch_args(args, list(meta.get("arg_names") or []))
    kw = dict(op.get("kwargs") or {})
    window = kw.get("window", None)
    if window is None and (kw.get("window_left") is not None or kw.get("window_right") is not None):
        window = (kw.get("window_left"), kw.get("window_right"))
    bias = values[names[4]] if len(names) == 5 else None
    if bias is not None and np.dtype(getattr(getattr(bias, "_data", bias), "dtype", np.float32)) != np.float32:
        raise ValueError("sm100 flash backward bias must use f32 storage")
    return ops.flash_attn_backward(values[names[0]], values[names[1]], values[names[2]], values[names[3]],
                                   scale=kw.get("scale"), causal=bool(kw.get("causal", False)), window=window,
                                   attn_bias=bias, softcap=kw.get("softcap", kw.get("logit_softcap", None)))


def _execute_sm100_moe(artifact: RuntimeArtifact, args: Any) -> Any:
    """grouped_gemm / moe_swiglu_block / moe_layer (python/tessera/runtime.py:9256-9281)."""
    from . import ops
    meta = artifact.metadata or {}
    op = _single_op(meta, COMPILER_PATHS["sm100_moe"], "sm100_moe")
    name = str(op.get("op_name"))
    values = _bind_launch_args(args, list(meta.get("arg_names") or []))
    kw = dict(op.get("kwargs") or {})
    if name == "tessera.grouped_gemm":
        return ops.grouped_gemm(values["x"], values["weights"], values["group_sizes"])
    if name == "tessera.moe_swiglu_block":
        return ops.moe_swiglu_block(values["x"], values["w_gate"], values["w_up"], values["w_down"],
                                    values["group_sizes"])
    if name == "tessera.moe_layer":
        return ops.moe_layer_from_logits(values["x"], values["logits"], values["w_gate"],
                                         values["w_up"], values["w_down"],
                                         top_k=int(kw.get("top_k", 1)),
                                         normalize_weights=bool(kw.get("normalize_weights", True)))
    raise ValueError(f"sm100_moe executor does not handle {name}")


def _executor_table() -> dict:
    return {"sm100_gemm": _execute_sm100_gemm, "sm100_flash_attn": _execute_sm100_flash_attn,
            "sm100_moe": _execute_sm100_moe, "sm100_flash_attn_bwd": _execute_sm100_flash_attn_bwd}


def backend_capabilities(target: Any) -> BackendCapability:
    name = normalize_target(target)
    if name != TARGET:
        return BackendCapability(name, False, False, reason=f"{name} is not served by this backend")
    try:
        _lib.load()
    except Exception as exc:
        return BackendCapability(name, False, False, reason=str(exc))
    import ctypes
    n = ctypes.c_int(0)
    _lib.load().tessera_sm100_device_count(ctypes.byref(n))
    if n.value <= 0:
        return BackendCapability(name, False, False, reason="no CUDA device visible",
                                 dtypes=("bf16", "fp16"))
    return BackendCapability(name, True, True, dtypes=("bf16", "fp16"),
                             features=("tcgen05", "tma", "tmem", "nccl"))


_last_profile = RuntimeProfile()


def get_last_profile() -> RuntimeProfile:
    return _last_profile


def _failure(artifact: RuntimeArtifact, status: str, reason: str, meta: Mapping, gate: Optional[str] = None) -> dict:
    return {"ok": False, "runtime_status": status,
            "compiler_path": str(meta.get("compiler_path", "artifact_only")),
            "execution_kind": str(meta.get("execution_kind", "artifact_only")),
            "artifact_hash": artifact.artifact_hash, "reason": reason,
            "first_failing_gate": gate, "first_failing_gate_detail": reason if gate else "",
            "telemetry": {"event": "runtime.launch", "status": status, "arch": meta.get("target")}}


def _launch_native_descriptor(artifact: "RuntimeArtifact", args: Any, stream: Any, t0: int, meta: Mapping) -> dict:
    """The descriptor seam (python/tessera/runtime.py:30905-30990): the invocation is checked against
    the descriptor and the image BEFORE the registered ``submit`` hook sees it, so a hook only ever
    receives buffers whose names, dtypes, ranks, layouts, alignments and guarded extents match."""
    from .native_artifact import ArtifactContractError, BufferArgument, LaunchDescriptor, NativeImageArtifact
    image, descriptor = artifact.native_image, artifact.launch_descriptor
    path = str(meta.get("compiler_path", "canonical_native_descriptor"))
    base = {"compiler_path": path, "artifact_hash": artifact.artifact_hash}
    try:
        if not isinstance(image, NativeImageArtifact) or not isinstance(descriptor, LaunchDescriptor):
            raise ArtifactContractError("E_LAUNCH_DESCRIPTOR_SCHEMA",
                                        "native_image / launch_descriptor must be NativeImageArtifact / LaunchDescriptor")
        values = dict(args) if isinstance(args, Mapping) else _bind_launch_args(args, descriptor.argument_names())
        buffer_names = {b.name for b in descriptor.buffers}
        buffers = {k: v for k, v in values.items() if k in buffer_names or hasattr(v, "shape") and getattr(v, "ndim", 0) > 0}
        scalars = {k: v for k, v in values.items() if k not in buffers}
        descriptor.validate_invocation(image, {k: BufferArgument.of(v) for k, v in buffers.items()}, scalars)
    except ArtifactContractError as exc:
        return {"ok": False, "runtime_status": "invalid_artifact", "execution_kind": "artifact_only",
                "diagnostic_code": exc.code, "reason": str(exc), **base}
    except Exception as exc:
        return {"ok": False, "runtime_status": "invalid_artifact", "execution_kind": "artifact_only",
                "reason": str(exc), **base}
    base.update(image_digest=image.image_digest, launch_descriptor_digest=descriptor.descriptor_digest)
    reg = _native_launchers.get(image.target)
    if reg is None or image.binary_format not in reg.binary_formats:
        return {"ok": False, "runtime_status": "unimplemented", "execution_kind": "artifact_only",
                "reason": f"no launcher registered for {image.target} accepts {image.binary_format!r}", **base}
    try:
        output = reg.submit(image, descriptor, buffers, scalars, stream)
    except Exception as exc:  # the submit hook raised
        return {"ok": False, "runtime_status": "device_error", "execution_kind": "native", "reason": str(exc), **base}
    ms = (time.perf_counter_ns() - t0) / 1e6
    return {"ok": True, "runtime_status": "success", "execution_kind": "native_gpu", "execution_mode": "descriptor",
            "output": output, "telemetry": {"event": "runtime.launch", "status": "ok"},
            "profile": {"launch_overhead_ms": ms, "kernel_elapsed_ms": ms, "cpu_wall_ms": None}, **base}


def launch(kernel: Any, args: Any, stream: Any = None) -> dict:
    """Run an executable artifact on the B200 backend, or return a structured non-success result."""
    global _last_profile
    t0 = time.perf_counter_ns()
    artifact = load_artifact(kernel)
    meta = artifact.metadata or {}
    target = normalize_target(meta.get("target", "cpu"))
    if artifact.launch_descriptor is not None:
        return _launch_native_descriptor(artifact, args, stream, t0, meta)
    if target != TARGET:
        cap = backend_capabilities(target)
        status = "unimplemented" if cap.available else "missing_backend"
        return _failure(artifact, status, f"{target} artifacts are not executed by the sm_100a "
                        f"backend (its target is {TARGET!r})", meta, gate="runtime_abi")
    path = str(meta.get("compiler_path", ""))
    table = _executor_table()
    if path not in table or meta.get("executable") is not True:
        return _failure(artifact, "unimplemented",
                        f"no executable row for ({target}, {path or 'artifact_only'})", meta,
                        gate="runtime_abi")
    cap = backend_capabilities(target)
    if not cap.available:
        return _failure(artifact, "missing_backend", cap.reason, meta, gate="runtime_abi")
    try:
        output = table[path](artifact, args)
    except _lib.BackendError as exc:
        _last_profile = RuntimeProfile(launch_overhead_ms=0.0)
        status = "device_error" if exc.rc == 3 else "invalid_artifact"
        return _failure(artifact, status, str(exc), meta)
    except Exception as exc:
        _last_profile = RuntimeProfile(launch_overhead_ms=0.0)
        return _failure(artifact, "invalid_artifact", str(exc), meta)
    ms = (time.perf_counter_ns() - t0) / 1e6
    _last_profile = RuntimeProfile(cpu_wall_ms=ms, launch_overhead_ms=ms)
    return {"ok": True, "runtime_status": "success", "compiler_path": path,
            "execution_kind": "native_gpu", "execution_mode": "sm100_tcgen05",
            "artifact_hash": artifact.artifact_hash, "output": output,
            "telemetry": {"event": "runtime.launch", "status": "ok", "arch": TARGET,
                          "latency_ms": ms, "kernel_id": str(meta.get("kernel_id", path))},
            "profile": {"cpu_wall_ms": ms, "launch_overhead_ms": ms}}


def make_artifact(op_name: str, arg_names: list, operands: Optional[list] = None,
                  kwargs: Optional[dict] = None, output_name: str = "out") -> RuntimeArtifact:
    """Metadata-only artifact for one op on this backend (the shape ``JitFn.runtime_artifact()``
    stamps for the NVIDIA lane, python/tessera/compiler/jit.py:2269-2295)."""
    path = next((p for p, names in COMPILER_PATHS.items() if op_name in names), None)
    if path is None:
        raise ValueError(f"{op_name} is not an op of the sm_100a backend")
    meta = {"target": TARGET, "compiler_path": path, "executable": True,
            "execution_kind": "native_gpu", "arg_names": list(arg_names), "output_name": output_name,
            "ops": [{"op_name": op_name, "result": output_name,
                     "operands": list(operands if operands is not None else arg_names),
                     "kwargs": dict(kwargs or {})}]}
    return RuntimeArtifact(metadata=meta, abi_signature=f"tessera.runtime.v1.{TARGET}")
