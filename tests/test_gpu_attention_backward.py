"""Attention backward (dQ, dK, dV) on the GPU through ``runtime.launch``, ``ops.flash_attn_backward``
and the host-pointer C entry. Cases and tolerances are those of the reference's device test
(tests/device/nvidia/test_flash_attention_backward.py:53-110), checked against the fixture made
with that test's own numpy reference, and against the oracle at larger sizes."""
import ctypes
import os

import numpy as np
import pytest

from oracle import tessera_oracle as orc
from tests.gpu_util import no_device_error, rel_err

pytestmark = pytest.mark.gpu

import tessera_b200 as tessera  # noqa: E402
from tessera_b200 import _lib, runtime as rt  # noqa: E402
from tessera_b200.device import DeviceArray, bfloat16  # noqa: E402


def _artifact(with_bias: bool, **kwargs):
    names = ["do", "q", "k", "v"] + (["bias"] if with_bias else [])
    return rt.RuntimeArtifact(metadata={
        "target": "nvidia_sm100", "compiler_path": "sm100_flash_attn_bwd", "executable": True,
        "execution_kind": "native_gpu", "arg_names": names, "output_name": "grads",
        "ops": [{"op_name": "tessera.flash_attn", "result": "grads", "operands": names, "kwargs": kwargs}]})


def _kwargs(kw):
    scale, causal, wl, wr, cap = (float(x) for x in kw)
    out = dict(scale=scale)
    if causal:
        out["causal"] = True
    if wl >= 0 or wr >= 0:
        out["window"] = (int(wl), int(wr))
    if cap:
        out["softcap"] = cap
    return out


def test_launch_matches_the_backward_lane_fixture(golden_dir):
    g = np.load(os.path.join(golden_dir, "attention_bwd.npz"))
    for i in range(int(g["n"])):
        with_bias = f"b{i}" in g
        args = (g[f"do{i}"], g[f"q{i}"], g[f"k{i}"], g[f"v{i}"]) + ((g[f"b{i}"],) if with_bias else ())
        got = rt.launch(_artifact(with_bias, **_kwargs(g[f"kw{i}"])), args)
        assert got["ok"], got.get("reason")
        for name, actual in zip(("dq", "dk", "dv"), got["output"]):
            assert actual.dtype == np.float32
            np.testing.assert_allclose(actual, g[f"{name}{i}"], atol=1e-4, rtol=0, err_msg=f"case {i} {name}")
    no_device_error()


@pytest.mark.parametrize("dt,atol", [(np.float16, 3e-3), (bfloat16, 2.5e-2)])
def test_half_storage_accumulates_in_f32(dt, atol):
    rng = np.random.default_rng(923)
    q = rng.standard_normal((1, 2, 4, 4), dtype=np.float32).astype(dt)
    k = rng.standard_normal((1, 1, 5, 4), dtype=np.float32).astype(dt)
    v = rng.standard_normal((1, 1, 5, 3), dtype=np.float32).astype(dt)
    do = rng.standard_normal((1, 2, 4, 3), dtype=np.float32).astype(dt)
    got = rt.launch(_artifact(False, scale=.5), (do, q, k, v))
    assert got["ok"], got.get("reason")
    ref = orc.attention_lane_backward(do, q, k, v, scale=.5)
    for actual, expected in zip(got["output"], ref):
        assert actual.dtype == dt
        np.testing.assert_allclose(actual.astype(np.float32), expected, atol=atol, rtol=0)


@pytest.mark.parametrize("B,Hq,Hkv,Sq,Sk,D,Dv,kw", [
    (2, 8, 2, 200, 333, 128, 128, dict(causal=True, causal_alignment="bottom_right")),
    (1, 4, 4, 257, 129, 64, 96, dict(window=(40, 7))),
    (1, 6, 1, 90, 90, 256, 256, dict(causal=True, softcap=3.0)),
    (3, 2, 2, 31, 500, 72, 40, dict()),
])
def test_larger_shapes_against_the_oracle(B, Hq, Hkv, Sq, Sk, D, Dv, kw):
    rng = np.random.default_rng(Sq * 7 + Sk)
    q = rng.standard_normal((B, Hq, Sq, D), dtype=np.float32)
    k = rng.standard_normal((B, Hkv, Sk, D), dtype=np.float32)
    v = rng.standard_normal((B, Hkv, Sk, Dv), dtype=np.float32)
    do = rng.standard_normal((B, Hq, Sq, Dv), dtype=np.float32)
    bias = (rng.standard_normal((B, Hq, Sq, Sk)) * 0.3).astype(np.float32) if Sq == 257 else None
    scale = 1 / np.sqrt(D)
    got = tessera.ops.flash_attn_backward(do, q, k, v, scale=scale, attn_bias=bias, **kw)
    okw = {a: b for a, b in kw.items() if a != "causal_alignment"}
    shift = max(Sk - Sq, 0) if kw.get("causal_alignment") == "bottom_right" else 0
    ref = orc.attention_lane_backward(do, q, k, v, scale=scale, bias=bias, causal_shift=shift, **okw)
    for name, a, e in zip(("dq", "dk", "dv"), got, ref):
        assert rel_err(a, e) < 2e-4, name
    again = tessera.ops.flash_attn_backward(do, q, k, v, scale=scale, attn_bias=bias, **kw)
    for a, b2 in zip(got, again):
        np.testing.assert_array_equal(a, b2)   # fixed summation order: bit-identical reruns
    no_device_error()


def test_rows_without_legal_keys_and_device_operands():
    rng = np.random.default_rng(4)
    q = rng.standard_normal((1, 1, 10, 4), dtype=np.float32)
    k = rng.standard_normal((1, 1, 4, 4), dtype=np.float32)
    v = rng.standard_normal((1, 1, 4, 4), dtype=np.float32)
    do = rng.standard_normal((1, 1, 10, 4), dtype=np.float32)
    dev = [DeviceArray.from_host(t) for t in (do, q, k, v)]
    got = tessera.ops.flash_attn_backward(*dev, scale=0.5, causal=True, window=(1, 0))
    assert all(isinstance(gx, DeviceArray) for gx in got)
    ref = orc.attention_lane_backward(do, q, k, v, scale=0.5, causal=True, window=(1, 0))
    for a, e in zip(got, ref):
        np.testing.assert_allclose(a.download(), e, atol=1e-5, rtol=0)
    assert not got[0].download()[0, 0, 5:].any()


def test_host_pointer_entry_has_the_reference_argument_order():
    rng = np.random.default_rng(77)
    B, Hq, Hkv, Sq, Sk, D, Dv = 1, 4, 2, 7, 9, 8, 6
    q = rng.standard_normal((B, Hq, Sq, D), dtype=np.float32)
    k = rng.standard_normal((B, Hkv, Sk, D), dtype=np.float32)
    v = rng.standard_normal((B, Hkv, Sk, Dv), dtype=np.float32)
    do = rng.standard_normal((B, Hq, Sq, Dv), dtype=np.float32)
    dq, dk, dv = np.empty_like(q), np.empty_like(k), np.empty_like(v)
    _lib.call("tessera_sm100_flash_attn_bwd", do.ctypes.data, q.ctypes.data, k.ctypes.data, v.ctypes.data, None,
              dq.ctypes.data, dk.ctypes.data, dv.ctypes.data, B, Hq, Hkv, Sq, Sk, D, Dv,
              ctypes.c_float(8 ** -0.5), 1, -1, -1, ctypes.c_float(0.0), _lib.F32)
    ref = orc.attention_lane_backward(do, q, k, v, scale=8 ** -0.5, causal=True)
    for a, e in zip((dq, dk, dv), ref):
        np.testing.assert_allclose(a, e, atol=7e-5, rtol=0)
    lib = _lib.load()
    rc = lib.tessera_sm100_flash_attn_bwd(do.ctypes.data, q.ctypes.data, k.ctypes.data, v.ctypes.data, None,
                                          dq.ctypes.data, dk.ctypes.data, dv.ctypes.data, B, 3, Hkv, Sq, Sk, D, Dv,
                                          ctypes.c_float(1.0), 0, -1, -1, ctypes.c_float(0.0), _lib.F32)
    assert rc != 0   # Hq not divisible by Hkv


@pytest.mark.parametrize("B,Hq,Hkv,Sq,Sk,causal", [
    (1, 2, 2, 64, 64, False),
    (1, 2, 2, 64, 64, True),
    (2, 4, 2, 200, 200, True),
    (1, 8, 2, 130, 333, True),     # bottom-right mask, ragged tiles, grouped heads
    (1, 4, 1, 257, 100, False),
    (1, 2, 2, 300, 77, True),      # Sq > Sk: the lane's top-left mask
    (1, 4, 4, 1, 190, False),
])
def test_tensor_core_path_bf16_d128(B, Hq, Hkv, Sq, Sk, causal):
    """bf16, D = 128: the mma.sync kernels. The reference for bf16 storage is the fp32 oracle on the
    same bf16-rounded operands; the gradients are rounded to bf16 on output."""
    rng = np.random.default_rng(Sq * 13 + Sk + causal)
    D = 128
    q = rng.standard_normal((B, Hq, Sq, D), dtype=np.float32).astype(bfloat16)
    k = rng.standard_normal((B, Hkv, Sk, D), dtype=np.float32).astype(bfloat16)
    v = rng.standard_normal((B, Hkv, Sk, D), dtype=np.float32).astype(bfloat16)
    do = rng.standard_normal((B, Hq, Sq, D), dtype=np.float32).astype(bfloat16)
    scale = 1 / np.sqrt(D)
    got = tessera.ops.flash_attn_backward(do, q, k, v, scale=scale, causal=causal, causal_alignment="bottom_right")
    ref = orc.attention_lane_backward(do, q, k, v, scale=scale, causal=causal, causal_shift=max(Sk - Sq, 0))
    for name, a, e in zip(("dq", "dk", "dv"), got, ref):
        assert a.dtype == bfloat16
        assert rel_err(a.astype(np.float32), e) < 2e-2, name
    again = tessera.ops.flash_attn_backward(do, q, k, v, scale=scale, causal=causal, causal_alignment="bottom_right")
    for a, b2 in zip(got, again):
        np.testing.assert_array_equal(a.view(np.uint16), b2.view(np.uint16))
    no_device_error()


def test_forward_with_lse_matches_the_oracle():
    rng = np.random.default_rng(8)
    B, Hq, Hkv, Sq, Sk, D = 1, 4, 2, 150, 210, 128
    q = rng.standard_normal((B, Hq, Sq, D), dtype=np.float32).astype(bfloat16)
    k = rng.standard_normal((B, Hkv, Sk, D), dtype=np.float32).astype(bfloat16)
    v = rng.standard_normal((B, Hkv, Sk, D), dtype=np.float32).astype(bfloat16)
    dq_, dk_, dv_ = (DeviceArray.from_host(t) for t in (q, k, v))
    o, lse = DeviceArray((B, Hq, Sq, D), bfloat16), DeviceArray((B, Hq, Sq), np.float32)
    scale = 1 / np.sqrt(D)
    _lib.call("tessera_sm100_flash_attn_fwd_lse_device", dq_.ptr, dk_.ptr, dv_.ptr, o.ptr, lse.ptr, B, Hq, Hkv, Sq,
              Sk, D, ctypes.c_float(scale), 1, None)
    qf, kf = q.astype(np.float32), k.astype(np.float32)
    shift = Sk - Sq
    for h in range(Hq):
        s = qf[0, h] @ kf[0, h // 2].T * scale
        keep = np.arange(Sk)[None, :] <= np.arange(Sq)[:, None] + shift
        s = np.where(keep, s, -np.inf)
        want = (np.log(np.exp(s - s.max(-1, keepdims=True)).sum(-1)) + s.max(-1)) / np.log(2.0)
        np.testing.assert_allclose(lse.download()[0, h], want, atol=2e-3, rtol=0)
    assert rel_err(o.download().astype(np.float32),
                   orc.attention_lane(q, k, v, scale=scale, causal=True, causal_shift=shift)) < 2e-2


def test_backward_from_saved_forward_state_is_bit_identical():
    rng = np.random.default_rng(21)
    B, Hq, Hkv, Sq, Sk, D = 1, 4, 2, 200, 260, 128
    q, k, v, do = (rng.standard_normal(s, dtype=np.float32).astype(bfloat16)
                   for s in ((B, Hq, Sq, D), (B, Hkv, Sk, D), (B, Hkv, Sk, D), (B, Hq, Sq, D)))
    scale = 1 / np.sqrt(D)
    want = tessera.ops.flash_attn_backward(do, q, k, v, scale=scale, causal=True, causal_alignment="bottom_right")
    dq_, dk_, dv_, dg = (DeviceArray.from_host(t) for t in (q, k, v, do))
    o, lse = DeviceArray((B, Hq, Sq, D), bfloat16), DeviceArray((B, Hq, Sq), np.float32)
    _lib.call("tessera_sm100_flash_attn_fwd_lse_device", dq_.ptr, dk_.ptr, dv_.ptr, o.ptr, lse.ptr, B, Hq, Hkv, Sq,
              Sk, D, ctypes.c_float(scale), 1, None)
    gq, gk, gv = DeviceArray(q.shape, bfloat16), DeviceArray(k.shape, bfloat16), DeviceArray(v.shape, bfloat16)
    scr = DeviceArray((B, Hq, Sq), np.float32)
    _lib.call("tessera_sm100_flash_attn_bwd_bf16_saved_device", dg.ptr, dq_.ptr, dk_.ptr, dv_.ptr, o.ptr, lse.ptr,
              gq.ptr, gk.ptr, gv.ptr, B, Hq, Hkv, Sq, Sk, ctypes.c_float(scale), 1, scr.ptr, None)
    for a, e in zip((gq, gk, gv), want):
        np.testing.assert_array_equal(a.download().view(np.uint16), e.view(np.uint16))
    no_device_error()


