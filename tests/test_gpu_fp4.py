"""NVFP4 expert weights on the GPU: the quantiser is bit-exact against the reference-made fixture
(codes and scales, including an all-zero block, a block whose scale underflows e4m3, and ties on
the e2m1 grid), and the grouped GEMM / expert FFN with quant="nvfp4" and "fp8xfp4" reproduce the
reference's dequantise-then-f32 results."""
import os

import ml_dtypes
import numpy as np
import pytest

from oracle import tessera_oracle as orc
from tests.gpu_util import no_device_error, rel_err

pytestmark = pytest.mark.gpu

import tessera_b200 as tessera  # noqa: E402
from tessera_b200 import ops  # noqa: E402
from tessera_b200.device import DeviceArray, bfloat16  # noqa: E402

_E2M1 = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0.0, -.5, -1, -1.5, -2, -3, -4, -6], np.float32)


def _unpack(t):
    codes = t.codes.download()
    lo, hi = codes & 15, codes >> 4
    vals = np.stack([_E2M1[lo], _E2M1[hi]], axis=-1).reshape(t.shape)
    scales = t.scales.download().view(ml_dtypes.float8_e4m3fn).astype(np.float32)
    return vals, scales


@pytest.mark.parametrize("dt", [np.float32, bfloat16])
def test_quantiser_is_bit_exact(golden_dir, dt):
    g = np.load(os.path.join(golden_dir, "quant4.npz"))
    x = g["n_x"].astype(dt)
    want_dq, want_sc, want_codes = orc.quantize_nvfp4(x)
    if dt == np.float32:
        np.testing.assert_array_equal(want_dq, g["n_dq"])
    t = ops.quantize_nvfp4(x)
    vals, scales = _unpack(t)
    np.testing.assert_array_equal(scales, want_sc)
    np.testing.assert_array_equal(vals, want_codes)
    np.testing.assert_array_equal(ops.dequantize_nvfp4(t), want_dq)
    np.testing.assert_array_equal(t.dequantize(bfloat16).download().astype(np.float32), want_dq)  # bf16 is exact


def test_e2m1_grid_ties_and_saturation():
    x = np.zeros((1, 16), np.float32)
    x[0] = [6.0, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25, -0.75, -5.0, 0.26, 0.74, 5.01, 4.99, -6.0]
    want = orc.quantize_nvfp4(x)[2]
    vals, scales = _unpack(ops.quantize_nvfp4(x))
    assert scales[0, 0] == 1.0
    np.testing.assert_array_equal(vals, want)


@pytest.mark.parametrize("quant", ["nvfp4", "fp8xfp4", "fp8_e5m2xnvfp4"])
def test_fixture_grouped_gemm_and_block(golden_dir, quant):
    g = np.load(os.path.join(golden_dir, "quant4.npz"))
    x = g["g_x"].astype(bfloat16)
    w, wg, wu, wd = (g[k].astype(bfloat16) for k in ("g_w", "g_wg", "g_wu", "g_wd"))
    got = ops.grouped_gemm(x, w, g["g_sizes"], quant=quant, out_dtype=np.float32)
    assert rel_err(got, g[f"gg_{quant}"]) < 1e-5
    blk = ops.moe_swiglu_block(x, wg, wu, wd, g["g_sizes"], quant=quant)
    assert rel_err(blk.astype(np.float32), g[f"blk_{quant}"]) < 8e-3     # bf16 output rounding
    no_device_error()


@pytest.mark.parametrize("quant", ["nvfp4", "fp8xfp4", "fp8_e5m2xnvfp4"])
def test_larger_ragged_groups_and_prequantised_weights(quant):
    rng = np.random.default_rng(12)
    T, K, N, E = 700, 512, 384, 5
    sizes = np.array([300, 0, 129, 256, 15])
    x = rng.standard_normal((T, K), dtype=np.float32).astype(bfloat16)
    w = (rng.standard_normal((E, K, N), dtype=np.float32) / 16).astype(bfloat16)
    ref = orc.grouped_gemm_fp4(x, w, sizes, quant)
    got = ops.grouped_gemm(x, w, sizes, quant=quant, out_dtype=np.float32)
    assert rel_err(got, ref) < 1e-5
    stored = ops.quantize_nvfp4(DeviceArray.from_host(w))        # 4.5 bits per weight at rest
    assert stored.codes.size == E * K * N // 2 and stored.scales.size == E * K * N // 16
    again = ops.grouped_gemm(x, stored, sizes, quant=quant, out_dtype=np.float32)
    np.testing.assert_array_equal(got, again)
    no_device_error()
