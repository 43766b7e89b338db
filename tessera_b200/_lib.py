"""ctypes binding of ``libtessera_sm100.so`` (the C ABI declared in ``include/tessera_sm100.h``).

There is no fallback: if the shared library is missing or a call returns non-zero, an exception
is raised. ``TESSERA_SM100_LIB`` overrides the library path (the same pattern as the reference's
``TESSERA_NVIDIA_GEMM_LIB``, python/tessera/runtime.py:2169).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_longlong, c_size_t, c_void_p
from pathlib import Path

_LIB = None

F32, BF16, F16, U8, I32 = 0, 1, 2, 3, 4


class BackendError(RuntimeError):
    """A C-ABI call returned a non-zero code."""

    def __init__(self, fn: str, rc: int, detail: str):
        self.fn, self.rc, self.detail = fn, rc, detail
        kind = {1: "bad argument", 2: "no usable GPU", 3: "device operation failed"}.get(rc, "error")
        super().__init__(f"{fn}: rc={rc} ({kind}): {detail}")


def lib_path() -> Path:
    env = os.environ.get("TESSERA_SM100_LIB")
    if env:
        return Path(env)
    return Path(__file__).resolve().parent / "lib" / "libtessera_sm100.so"


_VP = c_void_p
_SIGNATURES = {
    "tessera_sm100_version": (c_char_p, []),
    "tessera_sm100_last_error": (c_char_p, []),
    "tessera_sm100_device_count": (c_int, [POINTER(c_int)]),
    "tessera_sm100_set_device": (c_int, [c_int]),
    "tessera_sm100_sm_count": (c_int, [POINTER(c_int)]),
    "tessera_sm100_consume_device_error": (c_int, [POINTER(c_int)]),
    "tessera_sm100_launch_count": (c_longlong, []),
    "tessera_sm100_selftest_wait_expiry": (c_int, [c_longlong, _VP]),
    "tessera_sm100_device_alloc": (c_int, [POINTER(_VP), c_size_t]),
    "tessera_sm100_device_free": (c_int, [_VP]),
    "tessera_sm100_pool_alloc": (c_int, [POINTER(_VP), c_size_t]),
    "tessera_sm100_pool_free": (c_int, [_VP]),
    "tessera_sm100_pool_free_async": (c_int, [_VP, _VP]),
    "tessera_sm100_pool_release": (c_int, []),
    "tessera_sm100_device_memset": (c_int, [_VP, c_int, c_size_t, _VP]),
    "tessera_sm100_device_upload": (c_int, [_VP, _VP, c_size_t, _VP]),
    "tessera_sm100_device_download": (c_int, [_VP, _VP, c_size_t, _VP]),
    "tessera_sm100_device_copy": (c_int, [_VP, _VP, c_size_t, _VP]),
    "tessera_sm100_device_copy_2d": (c_int, [_VP, c_size_t, _VP, c_size_t, c_size_t, c_size_t, _VP]),
    "tessera_sm100_device_download_2d": (c_int, [_VP, c_size_t, _VP, c_size_t, c_size_t, c_size_t, _VP]),
    "tessera_sm100_host_alloc": (c_int, [POINTER(_VP), c_size_t]),
    "tessera_sm100_host_free": (c_int, [_VP]),
    "tessera_sm100_stream_create": (c_int, [POINTER(_VP)]),
    "tessera_sm100_stream_destroy": (c_int, [_VP]),
    "tessera_sm100_stream_synchronize": (c_int, [_VP]),
    "tessera_sm100_device_synchronize": (c_int, []),
    "tessera_sm100_event_create": (c_int, [POINTER(_VP)]),
    "tessera_sm100_event_destroy": (c_int, [_VP]),
    "tessera_sm100_event_record": (c_int, [_VP, _VP]),
    "tessera_sm100_stream_wait_event": (c_int, [_VP, _VP]),
    "tessera_sm100_event_synchronize": (c_int, [_VP]),
    "tessera_sm100_event_elapsed_ms": (c_int, [_VP, _VP, POINTER(c_float)]),
    "tessera_sm100_flush_l2": (c_int, [_VP]),
    "tessera_sm100_mma_gemm_bf16": (c_int, [_VP, _VP, _VP, c_int, c_int, c_int]),
    "tessera_sm100_mma_gemm_f16": (c_int, [_VP, _VP, _VP, c_int, c_int, c_int]),
    "tessera_sm100_mma_gemm_bf16_device": (c_int, [_VP, _VP, _VP, c_int, c_int, c_int, _VP]),
    "tessera_sm100_mma_gemm_f16_device": (c_int, [_VP, _VP, _VP, c_int, c_int, c_int, _VP]),
    "tessera_sm100_gemm": (c_int, [_VP, _VP, _VP, c_int, c_int, c_int, c_int, c_int, c_int]),
    "tessera_sm100_gemm_device": (c_int, [_VP, _VP, _VP, c_int, c_int, c_int, c_int, c_int, c_int,
                                          _VP]),
    "tessera_sm100_gemm_strided_device": (c_int, [_VP, _VP, _VP, c_int, c_int, c_int, c_int,
                                                  c_longlong, c_longlong, c_longlong, c_longlong,
                                                  c_longlong, c_longlong, c_int, c_int, _VP]),
    "tessera_sm100_gemm_epilogue_device": (c_int, [_VP, _VP, _VP, c_int, c_int, c_int, c_int, c_int, _VP,
                                                   _VP, c_int, _VP]),
    "tessera_sm100_gemm_allgather_device": (c_int, [_VP, _VP, POINTER(_VP), c_int, c_int, c_int, c_int,
                                                    c_int, c_int, c_int, _VP]),
    "tessera_sm100_allgather_columns_device": (c_int, [POINTER(_VP), c_int, c_int, c_int, c_longlong, c_int, _VP]),
    "tessera_sm100_probe_mma_rate": (c_int, [c_int, c_int, c_int, c_int, POINTER(ctypes.c_double)]),
    "tessera_sm100_gemm_allgather_block_device": (c_int, [_VP, _VP, c_longlong, POINTER(_VP), c_int, c_int, c_int,
                                                          c_int, c_int, c_int, c_int, _VP]),
    "tessera_sm100_grouped_gemm_device": (c_int, [_VP, _VP, _VP, _VP, c_int, c_int, c_int, c_int,
                                                  c_int, c_int, _VP]),
    "tessera_sm100_grouped_swiglu_device": (c_int, [_VP, _VP, _VP, _VP, _VP, c_int, c_int, c_int,
                                                    c_int, c_int, c_int, _VP]),
    "tessera_sm100_moe_route_device": (c_int, [_VP, c_int, c_int, c_int, c_int, _VP, _VP, _VP]),
    "tessera_sm100_moe_permute_device": (c_int, [_VP, _VP, c_int, c_int, c_int, c_int, _VP, _VP,
                                                 _VP, _VP, _VP, _VP, _VP]),
    "tessera_sm100_moe_dispatch_device": (c_int, [_VP, _VP, _VP, c_int, c_int, c_int, c_int, _VP]),
    "tessera_sm100_moe_combine_device": (c_int, [_VP, _VP, _VP, _VP, c_int, c_int, c_int, c_int,
                                                 c_int, _VP]),
    "tessera_sm100_moe_combine_scatter_f32_device": (c_int, [_VP, _VP, _VP, _VP, c_int, c_int,
                                                             c_int, _VP]),
    "tessera_sm100_moe_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int]),
    "tessera_sm100_moe_layer_device": (c_int, [_VP, _VP, _VP, _VP, _VP, _VP, c_int, c_int, c_int,
                                               c_int, c_int, c_int, c_int, c_int, c_int, _VP, _VP]),
    "tessera_sm100_moe_workspace_views": (c_int, [_VP, c_int, c_int, c_int, c_int, c_int]
                                          + [POINTER(_VP)] * 8),
    "tessera_sm100_ep_plan_device": (c_int, [_VP, c_int, c_int, c_int, _VP, _VP, _VP]),
    "tessera_sm100_ep_dispatch_device": (c_int, [_VP, _VP, _VP, _VP, _VP, POINTER(_VP), c_int, c_int,
                                                 c_int, c_int, c_int, c_int, _VP]),
    "tessera_sm100_ep_combine_device": (c_int, [POINTER(_VP), _VP, _VP, _VP, _VP, _VP, _VP, c_int, c_int,
                                                c_int, c_int, c_int, c_int, c_int, _VP]),
    "tessera_sm100_ep_ctrl_bytes": (c_size_t, []),
    "tessera_sm100_ep_route_publish_device": (c_int, [_VP, c_int, c_int, c_int, c_int, _VP, _VP, _VP, _VP, _VP, _VP,
                                                      _VP, _VP, POINTER(_VP), c_int, c_int, c_int, _VP]),
    "tessera_sm100_ep_dispatch_signal_device": (c_int, [_VP, _VP, _VP, _VP, POINTER(_VP), POINTER(_VP), c_int, c_int,
                                                        c_int, c_int, c_int, c_int, c_int, c_int, _VP, _VP, _VP,
                                                        c_int, _VP]),
    "tessera_sm100_ep_combine_signal_device": (c_int, [POINTER(_VP), POINTER(_VP), _VP, _VP, _VP, _VP, _VP, _VP,
                                                       c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                                       c_int, _VP, c_int, _VP]),
    "tessera_sm100_attn_decode_splits": (c_int, [c_int, c_int, c_int, c_int]),
    "tessera_sm100_attn_decode_int8_splits": (c_int, [c_int, c_int, c_int, c_int]),
    "tessera_sm100_attn_decode_scratch_bytes": (c_size_t, [c_int, c_int, c_int]),
    "tessera_sm100_attn_decode_device": (c_int, [_VP, _VP, _VP, _VP, c_int, c_int, c_int, c_int,
                                                 c_int, c_float, c_int, _VP, _VP]),
    "tessera_sm100_flash_attn_strided_device": (c_int, [_VP, _VP, _VP, _VP, c_int, c_int, c_int, c_int, c_int,
                                                        c_int, _VP, _VP, _VP, _VP, c_float, c_int, _VP]),
    "tessera_sm100_flash_attn_fwd_strided_device": (c_int, [_VP, _VP, _VP, _VP, c_int, c_int, c_int, c_int,
                                                            c_int, c_int, _VP, _VP, _VP, _VP, c_float, c_int,
                                                            _VP]),
    "tessera_qos_limit_set": (None, [c_int]),
    "tessera_qos_acquire": (None, []),
    "tessera_qos_release": (None, []),
    "tessera_submit_chunk_async": (None, [_VP, ctypes.c_uint64, c_int, c_int]),
    "tessera_trace_write": (None, [c_char_p]),
    "tessera_trace_write_status": (c_int, [c_char_p]),
    "tessera_shutdown_runtime": (None, []),
    "tessera_sm100_comm_bind_stream": (c_int, [c_int, c_int, _VP]),
    "tessera_sm100_qos_state": (c_int, [POINTER(c_int), POINTER(c_int), POINTER(c_int), POINTER(c_longlong)]),
    "tessera_sm100_attn_decode_state_device": (c_int, [_VP, _VP, _VP, _VP, _VP, _VP, c_int, c_int, c_int, c_int,
                                                       c_int, c_float, c_int, _VP, _VP]),
    "tessera_sm100_softmax_merge_device": (c_int, [_VP] * 9 + [c_longlong, c_int, _VP]),
    "tessera_sm100_softmax_finalize_device": (c_int, [_VP, _VP, _VP, c_longlong, c_int, c_int, _VP]),
    "tessera_sm100_flash_attn_general_device": (c_int, [_VP, _VP, _VP, _VP, _VP, c_longlong, c_int, c_int,
                                                        c_longlong, c_longlong, c_int, c_int, c_float, c_int,
                                                        c_longlong, c_longlong, c_longlong, c_float, c_int, _VP]),
    "tessera_sm100_flash_attn_bwd_workspace_bytes": (c_size_t, [c_longlong, c_int, c_longlong]),
    "tessera_sm100_flash_attn_bwd_device": (c_int, [_VP] * 8 + [c_longlong, c_int, c_int, c_longlong, c_longlong,
                                                    c_int, c_int, c_float, c_int, c_longlong, c_longlong,
                                                    c_longlong, c_float, c_int, _VP, _VP]),
    "tessera_sm100_flash_attn_bwd": (c_int, [_VP] * 8 + [c_longlong, c_int, c_int, c_longlong, c_longlong, c_int,
                                             c_int, c_float, c_int, c_longlong, c_longlong, c_float, c_int]),
    "tessera_sm100_flash_attn_bwd_bf16_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "tessera_sm100_flash_attn_bwd_bf16_device": (c_int, [_VP] * 7 + [c_int, c_int, c_int, c_int, c_int, c_float,
                                                         c_int, _VP, _VP]),
    "tessera_sm100_flash_attn_bwd_bf16_saved_device": (c_int, [_VP] * 9 + [c_int, c_int, c_int, c_int, c_int,
                                                               c_float, c_int, _VP, _VP]),
    "tessera_sm100_flash_attn_fwd_lse_device": (c_int, [_VP] * 5 + [c_int, c_int, c_int, c_int, c_int, c_int,
                                                        c_float, c_int, _VP]),
    "tessera_sm100_quantize_nvfp4_device": (c_int, [_VP, c_longlong, c_longlong, c_int, _VP, _VP, _VP]),
    "tessera_sm100_dequantize_nvfp4_device": (c_int, [_VP, _VP, c_longlong, c_longlong, _VP, c_int, _VP]),
    "tessera_sm100_fp8_to_bf16_device": (c_int, [_VP, c_longlong, c_int, _VP, _VP]),
    "tessera_sm100_quantize_fp8_fmt_device": (c_int, [_VP, c_longlong, c_int, c_int, _VP, _VP, _VP, _VP]),
    "tessera_sm100_quantize_fp8_weights_fmt_device": (c_int, [_VP, c_int, c_int, c_int, c_int, c_int, _VP, _VP, _VP]),
    "tessera_sm100_gemm_fp8_fmt_device": (c_int, [_VP, _VP, _VP, c_int, c_int, c_int, _VP, _VP, c_int, c_int, _VP]),
    "tessera_sm100_grouped_gemm_fp8_fmt_device": (c_int, [_VP, _VP, _VP, _VP, c_int, c_int, c_int, c_int, _VP, _VP,
                                                          c_int, c_int, _VP]),
    "tessera_sm100_grouped_swiglu_fp8_fmt_device": (c_int, [_VP, _VP, _VP, _VP, _VP, c_int, c_int, c_int, c_int,
                                                            _VP, _VP, _VP, c_int, _VP, c_int, _VP]),
    "tessera_sm100_grouped_gemm_scaled_device": (c_int, [_VP, _VP, _VP, _VP, c_int, c_int, c_int, c_int, c_int,
                                                         c_int, _VP, _VP]),
    "tessera_sm100_grouped_swiglu_scaled_device": (c_int, [_VP, _VP, _VP, _VP, _VP, c_int, c_int, c_int, c_int,
                                                           c_int, c_int, _VP, _VP]),
    "tessera_sm100_quantize_fp8_device": (c_int, [_VP, c_longlong, c_int, _VP, _VP, _VP, _VP]),
    "tessera_sm100_quantize_fp8_weights_device": (c_int, [_VP, c_int, c_int, c_int, c_int, _VP, _VP, _VP]),
    "tessera_sm100_gemm_fp8_device": (c_int, [_VP, _VP, _VP, c_int, c_int, c_int, _VP, _VP, c_int, _VP]),
    "tessera_sm100_grouped_gemm_fp8_device": (c_int, [_VP, _VP, _VP, _VP, c_int, c_int, c_int, c_int, _VP, _VP,
                                                      c_int, _VP]),
    "tessera_sm100_grouped_swiglu_fp8_device": (c_int, [_VP, _VP, _VP, _VP, _VP, c_int, c_int, c_int, c_int,
                                                        _VP, _VP, _VP, c_int, _VP, _VP]),
    "tessera_sm100_attn_decode_int8_device": (c_int, [_VP, _VP, _VP, _VP, _VP, _VP, c_int, c_int, c_int, c_int,
                                                      c_int, c_float, c_int, _VP, _VP]),
    "tessera_sm100_paged_attn_decode_int8_device": (c_int, [_VP, _VP, _VP, _VP, _VP, _VP, _VP, _VP, c_int, c_int,
                                                            c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                                            c_int, _VP, _VP]),
    "tessera_sm100_quantize_kv_int8_device": (c_int, [_VP, _VP, _VP, _VP, _VP, _VP, _VP, c_longlong, c_int, c_int,
                                                      _VP]),
    "tessera_sm100_paged_attn_decode_device": (c_int, [_VP, _VP, _VP, _VP, _VP, _VP, c_int, c_int, c_int,
                                                       c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                                                       _VP, _VP]),
    "tessera_sm100_paged_kv_append_device": (c_int, [_VP, _VP, _VP, _VP, _VP, _VP, c_int, c_int, c_int, c_int,
                                                     c_int, c_int, _VP]),
    "tessera_sm100_paged_kv_gather_device": (c_int, [_VP, _VP, _VP, _VP, ctypes.c_longlong, c_int, c_int,
                                                     c_int, c_int, c_int, _VP]),
    "tessera_sm100_attn_decode_static_device": (c_int, [_VP, _VP, _VP, _VP, c_int, c_int, c_int, c_int,
                                                        c_int, c_float, c_int, c_int, _VP]),
    "tessera_sm100_flash_attn_fwd_device": (c_int, [_VP, _VP, _VP, _VP, c_int, c_int, c_int, c_int,
                                                    c_int, c_int, c_float, c_int, _VP]),
    "tessera_sm100_flash_attn_device": (c_int, [_VP, _VP, _VP, _VP, c_int, c_int, c_int, c_int,
                                                c_int, c_int, c_float, c_int, _VP]),
    "tessera_sm100_flash_attn": (c_int, [_VP, _VP, _VP, _VP, c_int, c_int, c_int, c_int, c_int,
                                         c_int, c_float, c_int]),
    "tessera_sm100_moe_layer": (c_int, [_VP, _VP, _VP, _VP, _VP, _VP, c_int, c_int, c_int, c_int,
                                        c_int, c_int, c_int, c_int, c_int, _VP, _VP, _VP, _VP]),
    "tessera_sm100_silu_mul_device": (c_int, [_VP, _VP, _VP, c_longlong, c_int, _VP]),
    "tessera_sm100_nccl_version": (c_int, [POINTER(c_int)]),
    "tessera_sm100_comm_unique_id": (c_int, [_VP]),
    "tessera_sm100_comm_init_rank": (c_int, [_VP, c_int, c_int, POINTER(_VP)]),
    "tessera_sm100_comm_init_all": (c_int, [c_int, POINTER(c_int), POINTER(_VP)]),
    "tessera_sm100_comm_destroy": (c_int, [_VP]),
    "tessera_sm100_comm_abort": (c_int, [_VP]),
    "tessera_sm100_comm_info": (c_int, [_VP, POINTER(c_int), POINTER(c_int), POINTER(c_int)]),
    "tessera_sm100_comm_async_error": (c_int, [_VP]),
    "tessera_sm100_group_start": (c_int, []),
    "tessera_sm100_group_end": (c_int, []),
    "tessera_sm100_all_gather": (c_int, [_VP, _VP, _VP, c_size_t, c_int, _VP]),
    "tessera_sm100_all_reduce": (c_int, [_VP, _VP, _VP, c_size_t, c_int, c_int, _VP]),
    "tessera_sm100_reduce_scatter": (c_int, [_VP, _VP, _VP, c_size_t, c_int, c_int, _VP]),
    "tessera_sm100_all_to_all": (c_int, [_VP, _VP, _VP, c_size_t, _VP]),
    "tessera_sm100_all_to_all_v": (c_int, [_VP, _VP, POINTER(c_size_t), POINTER(c_size_t), _VP,
                                           POINTER(c_size_t), POINTER(c_size_t), _VP]),
    "tessera_sm100_ipc_get_handle": (c_int, [_VP, _VP]),
    "tessera_sm100_ipc_open_handle": (c_int, [_VP, POINTER(_VP)]),
    "tessera_sm100_ipc_close_handle": (c_int, [_VP]),
}


def load() -> ctypes.CDLL:
    """Load the shared library once; raise if it is not there."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = lib_path()
    if not path.exists():
        raise BackendError("load", 2, f"{path} not found; run `python -m tessera_b200.build`")
    lib = ctypes.CDLL(str(path))
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    _LIB = lib
    return lib


def exported_symbols() -> list[str]:
    return sorted(_SIGNATURES)


def last_error() -> str:
    return (load().tessera_sm100_last_error() or b"").decode("utf-8", "replace")


def check(fn_name: str, rc: int) -> None:
    if rc != 0:
        raise BackendError(fn_name, rc, last_error())


def call(fn_name: str, *args):
    """Call an int-returning entry point and raise on a non-zero code."""
    rc = getattr(load(), fn_name)(*args)
    check(fn_name, rc)
