"""The general attention kernel (any head dimension, f32 / f16 / bf16 storage, bias, window,
soft-cap) through ``runtime.launch`` and ``ops.flash_attn``. The cases and tolerances are those of
the reference's device test (tests/device/nvidia/test_flash_attention.py:61-108), checked against
the fixture made with that test's own numpy reference and against the oracle."""
import os

import numpy as np
import pytest

from oracle import tessera_oracle as orc
from tests.gpu_util import TOL, no_device_error, rel_err

pytestmark = pytest.mark.gpu

import tessera_b200 as tessera  # noqa: E402
from tessera_b200 import runtime as rt  # noqa: E402
from tessera_b200.device import bfloat16  # noqa: E402


def _artifact(*, with_bias: bool, **kwargs):
    operands = ["q", "k", "v"] + (["bias"] if with_bias else [])
    return rt.RuntimeArtifact(metadata={
        "target": "nvidia_sm100", "compiler_path": "sm100_flash_attn", "executable": True,
        "execution_kind": "native_gpu", "arg_names": operands, "output_name": "o",
        "ops": [{"op_name": "tessera.flash_attn", "result": "o", "operands": operands, "kwargs": kwargs}]})


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


def test_launch_matches_the_lane_contract_fixture(golden_dir):
    g = np.load(os.path.join(golden_dir, "attention.npz"))
    for i in range(int(g["lane_n"])):
        has_bias = f"laneb{i}" in g
        args = (g[f"laneq{i}"], g[f"lanek{i}"], g[f"lanev{i}"]) + ((g[f"laneb{i}"],) if has_bias else ())
        got = rt.launch(_artifact(with_bias=has_bias, **_kwargs(g[f"lanekw{i}"])), args)
        assert got["ok"] is True, got.get("reason")
        assert got["output"].dtype == np.float32 and got["execution_kind"] == "native_gpu"
        np.testing.assert_allclose(got["output"], g[f"laneo{i}"], atol=4e-5, rtol=0, err_msg=f"case {i}")
    no_device_error()


def test_f16_and_bf16_storage_f32_accumulation():
    rng = np.random.default_rng(821)
    for dt, atol in ((np.float16, 2e-3), (bfloat16, 2e-2)):
        q = rng.standard_normal((1, 4, 5, 8), dtype=np.float32).astype(dt)
        k = rng.standard_normal((1, 2, 7, 8), dtype=np.float32).astype(dt)
        v = rng.standard_normal((1, 2, 7, 6), dtype=np.float32).astype(dt)
        scale = 1.0 / np.sqrt(8.0)
        got = rt.launch(_artifact(with_bias=False, scale=scale), (q, k, v))
        assert got["ok"] is True, got.get("reason")
        assert got["output"].dtype == dt
        np.testing.assert_allclose(got["output"].astype(np.float32), orc.attention_lane(q, k, v, scale=scale),
                                   atol=atol, rtol=0)


def test_ops_flash_attn_bias_and_odd_head_dims(golden_dir):
    g = np.load(os.path.join(golden_dir, "attention.npz"))
    Q, K, V = (g[n].astype(bfloat16) for n in ("biasQ", "biasK", "biasV"))
    got = tessera.ops.flash_attn(Q, K, V, causal=True, attn_bias=g["biasB"])
    assert got.dtype == bfloat16 and rel_err(got, g["biasO"]) < TOL
    rng = np.random.default_rng(9)
    # bottom-right causal alignment with Sq != Sk and head dimensions the tcgen05 kernels do not take
    for D, Dv, Sq, Sk in ((64, 64, 100, 260), (96, 160, 260, 100), (256, 256, 33, 33), (128, 128, 50, 90)):
        q = rng.standard_normal((2, 4, Sq, D), dtype=np.float32)
        k = rng.standard_normal((2, 2, Sk, D), dtype=np.float32)
        v = rng.standard_normal((2, 2, Sk, Dv), dtype=np.float32)
        got = tessera.ops.flash_attn(q, k, v, causal=True)
        ref = orc.attention_lane(q, k, v, scale=1 / np.sqrt(D), causal=True, causal_shift=max(Sk - Sq, 0))
        assert got.dtype == np.float32 and got.shape == (2, 4, Sq, Dv)
        assert rel_err(got, ref) < 1e-4, (D, Dv, Sq, Sk)
    # same shapes, the two kernels: bf16 D=128 goes to tcgen05, a window sends it to the general kernel
    q, k, v = (rng.standard_normal((1, 2, 300, 128), dtype=np.float32).astype(bfloat16) for _ in range(3))
    fast = tessera.ops.flash_attn(q, k, v, causal=True)
    general = tessera.ops.flash_attn(q, k, v, causal=True, window=(10 ** 6, 10 ** 6))
    assert rel_err(fast, general) < TOL
    no_device_error()


def test_fully_masked_rows_are_zero_and_bad_arguments_are_rejected():
    rng = np.random.default_rng(3)
    q, k, v = (rng.standard_normal((1, 1, 6, 16), dtype=np.float32) for _ in range(3))
    # window (0, 0) with a bias of -inf on the diagonal leaves nothing: the lane returns zeros
    got = rt.launch(_artifact(with_bias=False, scale=0.3, window=(0, 0)), (q, k[:, :, :3], v[:, :, :3]))
    assert got["ok"] and np.all(got["output"][0, 0, 3:] == 0) and np.all(np.isfinite(got["output"]))
    bad = rt.launch(_artifact(with_bias=True, scale=0.3), (q, k, v, np.zeros((1, 1, 6, 6), np.float64)))
    assert bad["ok"] is False and "f32" in bad["reason"]
    with pytest.raises(ValueError):
        tessera.ops.flash_attn(q, k, v, window=(-3, 1))
    with pytest.raises(ValueError):
        tessera.ops.flash_attn(q, k, v, attn_bias=np.zeros((5, 5), np.float32))
    with pytest.raises(TypeError):
        tessera.ops.flash_attn(q, k.astype(np.float16), v)
