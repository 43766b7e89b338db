"""fp8 (e4m3) grouped GEMM on the GPU: the quantisation kernels reproduce the reference's
quantize_fp8 bit for bit, and the tensor-core GEMMs on the e4m3 bytes match the reference's
dequantise-then-f32-GEMM result (fixture made by the reference; oracle at larger sizes, including
sizes that take the CTA-pair kernel)."""
import os

import ml_dtypes
import numpy as np
import pytest

from oracle import tessera_oracle as orc
from tests.gpu_util import TOL, no_device_error, rel_err

pytestmark = pytest.mark.gpu

import tessera_b200 as tessera  # noqa: E402
from tessera_b200.device import bfloat16  # noqa: E402

E4 = ml_dtypes.float8_e4m3fn


def _bf(x):
    return np.asarray(x, np.float32).astype(bfloat16)


def test_quantisation_is_bit_exact(golden_dir):
    g = np.load(os.path.join(golden_dir, "moe.npz"))
    t = tessera.ops.quantize_fp8_activations(_bf(g["q_x"]))
    scale = t.scale_values()[0]
    assert scale == g["q_x_scale"]
    dq = t.q.download().view(E4).astype(np.float32) * scale
    np.testing.assert_array_equal(dq, g["q_x_dq"])
    # per-expert weights, stored transposed
    w = _bf(g["q_wg"])
    tw = tessera.ops.quantize_fp8_experts(w)
    q = tw.q.download().view(E4).astype(np.float32)        # (E, N, K)
    for e in range(w.shape[0]):
        ref_dq, ref_scale = orc.quantize_fp8(w[e])
        assert tw.scale_values()[e] == ref_scale
        np.testing.assert_array_equal(q[e].T * ref_scale, ref_dq)
    # float32 input and an all-zero tensor (scale floors at 1e-12)
    x32 = np.random.default_rng(1).standard_normal((37, 48)).astype(np.float32) * 1000
    t32 = tessera.ops.quantize_fp8_activations(x32)
    ref_dq, ref_scale = orc.quantize_fp8(x32)
    assert t32.scale_values()[0] == ref_scale
    np.testing.assert_array_equal(t32.q.download().view(E4).astype(np.float32) * ref_scale, ref_dq)
    tz = tessera.ops.quantize_fp8_activations(np.zeros((4, 16), np.float32))
    assert tz.scale_values()[0] == np.float32(1e-12) and not tz.q.download().any()


def test_fixture_grouped_gemm_and_block(golden_dir):
    g = np.load(os.path.join(golden_dir, "moe.npz"))
    x, wg, wu, wd, sizes = _bf(g["q_x"]), _bf(g["q_wg"]), _bf(g["q_wu"]), _bf(g["q_wd"]), g["q_sizes"]
    got = tessera.ops.grouped_gemm(x, wg, sizes, quant="fp8_e4m3", out_dtype=np.float32)
    assert rel_err(got, g["q_gg"]) < 1e-5      # same e4m3 values, f32 accumulation: only the order differs
    assert tessera.ops.grouped_gemm(x, wg, sizes, quant="fp8").dtype == bfloat16
    blk = tessera.ops.moe_swiglu_block(x, wg, wu, wd, sizes, quant="fp8_e4m3")
    assert rel_err(blk, g["q_block"]) < TOL    # the hidden activation is rounded to bf16 before its quantisation
    no_device_error()


@pytest.mark.parametrize("sizes,K,N", [([100, 0, 129, 33, 127], 192, 128), ([5, 300, 1, 0, 0, 700], 144, 528),
                                       ([300, 0, 777, 100, 871], 272, 2576), ([256, 512, 1280], 64, 2560)])
def test_grouped_fp8_against_oracle(sizes, K, N):
    rng = np.random.default_rng(len(sizes) + K)
    sizes = np.array(sizes)
    T, E = int(sizes.sum()), len(sizes)
    x = _bf(rng.standard_normal((T, K)))
    w = _bf(rng.standard_normal((E, K, N)) / np.sqrt(K))
    w2 = _bf(rng.standard_normal((E, K, N)) / np.sqrt(K))
    wd = _bf(rng.standard_normal((E, N, K)) / np.sqrt(N))
    got = tessera.ops.grouped_gemm(x, w, sizes, quant="fp8_e4m3", out_dtype=np.float32)
    assert rel_err(got, orc.grouped_gemm_fp8(x, w, sizes)) < 1e-5
    pre = tessera.ops.quantize_fp8_experts(w)              # quantise once, reuse
    again = tessera.ops.grouped_gemm(x, pre, sizes, out_dtype=np.float32)
    np.testing.assert_array_equal(got, again)
    blk = tessera.ops.moe_swiglu_block(x, w, w2, wd, sizes, quant="fp8_e4m3")
    assert rel_err(blk, orc.moe_swiglu_block_fp8(x, w, w2, wd, sizes)) < TOL
    no_device_error()


def test_unsupported_quant_names():
    x, w = np.zeros((8, 16), np.float32), np.zeros((1, 16, 8), np.float32)
    with pytest.raises(ValueError):          # the reference's message: NVFP4 blocks of 16 along N
        tessera.ops.grouped_gemm(x, w, [8], quant="nvfp4")
    with pytest.raises(ValueError):
        tessera.ops.grouped_gemm(x, w, [8], quant="int3")
    with pytest.raises(ValueError):
        tessera.ops.grouped_gemm(np.zeros((8, 24), np.float32), np.zeros((1, 24, 8), np.float32), [8], quant="fp8")


def test_e5m2_quantisation_and_grouped_gemm(golden_dir):
    """quant="fp8_e5m2": the same kernels with the e5m2 format code (scale = amax / 57344)."""
    g = np.load(os.path.join(golden_dir, "quant4.npz"))
    t = tessera.ops.quantize_fp8_activations(g["n_x"], format="e5m2")
    scale = t.scale_values()[0]
    assert scale == g["e5_scale"]
    np.testing.assert_array_equal(t.q.download().view(ml_dtypes.float8_e5m2).astype(np.float32) * scale, g["e5_dq"])
    x, w, wg, wu, wd = (_bf(g[k]) for k in ("g_x", "g_w", "g_wg", "g_wu", "g_wd"))
    got = tessera.ops.grouped_gemm(x, w, g["g_sizes"], quant="fp8_e5m2", out_dtype=np.float32)
    assert rel_err(got, g["gg_fp8_e5m2"]) < 1e-5
    blk = tessera.ops.moe_swiglu_block(x, wg, wu, wd, g["g_sizes"], quant="fp8_e5m2")
    assert rel_err(blk, g["blk_fp8_e5m2"]) < TOL
    # larger, ragged, CTA-pair sizes against the oracle
    rng = np.random.default_rng(3)
    sizes = np.array([300, 0, 777, 100, 871])
    xs = _bf(rng.standard_normal((int(sizes.sum()), 272)))
    ws = _bf(rng.standard_normal((5, 272, 2576)) / 16)
    got = tessera.ops.grouped_gemm(xs, ws, sizes, quant="fp8_e5m2", out_dtype=np.float32)
    assert rel_err(got, orc.grouped_gemm_fp8(xs, ws, sizes, "e5m2")) < 1e-5
    no_device_error()
