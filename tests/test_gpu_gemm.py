"""GEMM parity on the GPU: tcgen05 kernel vs the numpy oracle and the reference-made fixtures.
Shapes follow the reference's device test (tests/device/nvidia/test_mma_runtime_symbol.py:178)."""
import ctypes
import os

import numpy as np
import pytest

from oracle import tessera_oracle as orc
from tests.gpu_util import TOL, gemm_device, no_device_error, rel_err

pytestmark = pytest.mark.gpu

from tessera_b200.device import bfloat16  # noqa: E402

SHAPES = [(16, 8, 16), (32, 24, 48), (64, 64, 64), (17, 9, 31), (128, 128, 256), (130, 264, 72),
          (512, 1024, 512), (1, 1, 1), (129, 257, 65), (300, 40, 1000)]


def _rand(rng, shape, dt, scale=1.0):
    return (rng.standard_normal(shape, dtype=np.float32) * scale).astype(dt)


@pytest.mark.parametrize("dt", [bfloat16, np.float16], ids=["bf16", "f16"])
def test_reference_shaped_host_symbol_matches_oracle(lib, dt):
    fn = lib.tessera_sm100_mma_gemm_bf16 if dt == bfloat16 else lib.tessera_sm100_mma_gemm_f16
    rng = np.random.default_rng(20260625)
    for (M, N, K) in SHAPES:
        A, B = _rand(rng, (M, K), dt), _rand(rng, (K, N), dt)
        D = np.zeros((M, N), np.float32)
        rc = fn(A.ctypes.data, B.ctypes.data, D.ctypes.data, M, N, K)
        assert rc == 0, lib.tessera_sm100_last_error()
        assert rel_err(D, orc.gemm(A, B)) < 1e-4  # fp32 output: only the summation order differs


def test_bad_arguments_return_code_1(lib):
    z = np.zeros((4, 4), np.float16)
    assert lib.tessera_sm100_mma_gemm_f16(z.ctypes.data, z.ctypes.data, z.ctypes.data, 0, 4, 4) == 1
    assert lib.tessera_sm100_mma_gemm_f16(None, z.ctypes.data, z.ctypes.data, 4, 4, 4) == 1
    assert b"gemm" in lib.tessera_sm100_last_error()


@pytest.mark.parametrize("out_dt", [np.float32, bfloat16, np.float16], ids=["f32", "bf16", "f16"])
def test_output_dtypes_and_batches(out_dt):
    rng = np.random.default_rng(3)
    in_dt = np.float16 if out_dt == np.float16 else bfloat16
    for (b, M, N, K) in [(1, 384, 768, 1024), (3, 256, 512, 128), (4, 100, 72, 200), (2, 17, 9, 31)]:
        A = _rand(rng, (b, M, K), in_dt, 1 / np.sqrt(K))
        B = _rand(rng, (b, K, N), in_dt)
        got = gemm_device(A, B, out_dt)
        assert got.dtype == np.dtype(out_dt)
        assert rel_err(got, orc.gemm(A, B)) < (1e-4 if out_dt == np.float32 else TOL)


def test_golden_fixtures(golden_dir):
    g = np.load(os.path.join(golden_dir, "gemm.npz"))
    for i in range(int(g["n"])):
        dt = bfloat16 if str(g[f"dtype{i}"]) == "bf16" else np.float16
        got = gemm_device(g[f"A{i}"].astype(dt), g[f"B{i}"].astype(dt), np.float32)
        assert rel_err(got, g[f"Y{i}"]) < 1e-4


def test_config1_batched_f16_via_ops():
    """A[4,1024,1024] x W[4,1024,1024] f16 -> fp32 through the public op."""
    import tessera_b200 as tessera
    inp = orc.make_inputs("gemm_f16_batched")
    Y = tessera.ops.gemm(inp["A"], inp["W"])
    assert Y.dtype == np.float32 and Y.shape == (4, 1024, 1024)
    assert rel_err(Y, orc.gemm(inp["A"], inp["W"])) < 1e-4


def test_config2_full_size_properties():
    """8192^3 bf16: sampled rows against the oracle plus linearity in A (D(a1+a2) = D(a1)+D(a2) when
    the sum is exact in bf16)."""
    rng = np.random.default_rng(1002)
    n = 8192
    A = _rand(rng, (n, n), bfloat16, 1 / np.sqrt(n))
    B = _rand(rng, (n, n), bfloat16, 1 / np.sqrt(n))
    Y = gemm_device(A, B, bfloat16)
    rows = [0, 1, 127, 128, 4095, 8191, 5000]
    ref = A[rows].astype(np.float32) @ B.astype(np.float32)
    assert rel_err(Y[rows], ref) < TOL
    cols = [0, 255, 256, 8191]
    refc = A.astype(np.float32) @ B[:, cols].astype(np.float32)
    assert rel_err(Y[:, cols], refc) < TOL
    # linearity with exactly representable operands: small integers
    A1 = rng.integers(-4, 5, (512, 1024)).astype(np.float32).astype(bfloat16)
    A2 = rng.integers(-4, 5, (512, 1024)).astype(np.float32).astype(bfloat16)
    Bi = rng.integers(-4, 5, (1024, 768)).astype(np.float32).astype(bfloat16)
    s = (A1.astype(np.float32) + A2.astype(np.float32)).astype(bfloat16)
    np.testing.assert_array_equal(gemm_device(s, Bi), gemm_device(A1, Bi) + gemm_device(A2, Bi))
    no_device_error()


def test_strided_column_block_output(lib):
    """Each of g ranks writes its [M, N/g] block straight into the full row-major Y (ldd = N)."""
    from tessera_b200 import _lib, device
    from tessera_b200.device import DeviceArray
    rng = np.random.default_rng(9)
    M, N, K, g = 256, 1024, 512, 4
    A = _rand(rng, (M, K), bfloat16, 1 / np.sqrt(K))
    W = _rand(rng, (K, N), bfloat16)
    dA, dW = DeviceArray.from_host(A), DeviceArray.from_host(W)
    dY = DeviceArray.zeros((M, N), bfloat16)
    nb = N // g
    for r in range(g):
        _lib.call("tessera_sm100_gemm_strided_device", dA.ptr, dW.ptr + r * nb * 2, dY.ptr + r * nb * 2,
                  1, M, nb, K, K, N, N, 0, 0, 0, _lib.BF16, _lib.BF16, None)
    assert rel_err(dY.download(), orc.gemm(A, W)) < TOL
    no_device_error()


@pytest.mark.parametrize("act", ["linear", "relu", "gelu", "silu"])
def test_fused_epilogue(golden_dir, act):
    """ops.gemm(A, B, epilogue={bias, residual, activation}) against the reference-made fixture and
    the oracle at a multi-tile size, fp32 and bf16 outputs."""
    import tessera_b200 as tessera
    g = np.load(os.path.join(golden_dir, "gemm.npz"))
    A, B = g["epiA"].astype(bfloat16), g["epiB"].astype(bfloat16)
    got = tessera.ops.gemm(A, B, epilogue=dict(bias=g["epi_bias"], activation=act, residual=g["epi_res"]))
    assert rel_err(got, g[f"epi_{act}"]) < 1e-4
    rng = np.random.default_rng(17)
    M, N, K = 300, 520, 264
    A = (rng.standard_normal((M, K), dtype=np.float32) / 16).astype(bfloat16)
    B = rng.standard_normal((K, N), dtype=np.float32).astype(bfloat16)
    bias = rng.standard_normal(N, dtype=np.float32)
    res = rng.standard_normal((M, N), dtype=np.float32).astype(bfloat16)
    ref = orc.fused_epilogue(orc.gemm(A, B), bias=bias, activation=act, residual=res)
    got = tessera.ops.gemm(A, B, epilogue=dict(bias=bias, activation=act, residual=res), out_dtype=bfloat16)
    assert got.dtype == bfloat16 and rel_err(got, ref) < TOL
    got32 = tessera.ops.gemm(A, B, epilogue=dict(bias=bias, activation=act))
    assert rel_err(got32, orc.fused_epilogue(orc.gemm(A, B), bias=bias, activation=act)) < 1e-4
    no_device_error()


@pytest.mark.parametrize("batch,M,N,K,out_dt", [(1, 4352, 2048, 2048, np.float32), (3, 1536, 1536, 1536, np.float32),
                                                (1, 3100, 3080, 3064, bfloat16)])
def test_host_pointer_form_pipelined_chunks(lib, batch, M, N, K, out_dt):
    """Host-pointer GEMMs of 32 MB and more run as row (or batch-entry) chunks over three streams;
    the result must equal the device-pointer form bit for bit (same kernel, same tiles per row
    block) and the oracle within tolerance. The last case has a ragged last chunk and row pitches
    that are not multiples of 8 elements."""
    rng = np.random.default_rng(M + N)
    shapeA = (batch, M, K) if batch > 1 else (M, K)
    shapeB = (batch, K, N) if batch > 1 else (K, N)
    A = _rand(rng, shapeA, bfloat16, 1 / np.sqrt(K))
    B = _rand(rng, shapeB, bfloat16)
    D = np.zeros(shapeA[:-1] + (N,), out_dt)
    rc = lib.tessera_sm100_gemm(A.ctypes.data, B.ctypes.data, D.ctypes.data, batch, M, N, K, 1,
                                0 if out_dt == np.float32 else 1)
    assert rc == 0, lib.tessera_sm100_last_error()
    assert rel_err(D, orc.gemm(A, B)) < (1e-4 if out_dt == np.float32 else TOL)
    if N % 8 == 0 and K % 8 == 0:
        np.testing.assert_array_equal(D, gemm_device(A, B, out_dt))
    no_device_error()


@pytest.mark.parametrize("batch,M,N,K,out_dt", [(1, 2304, 4352, 520, np.float32), (1, 2200, 4360, 264, bfloat16),
                                                (2, 1280, 4096, 256, np.float16), (1, 8192, 1280, 128, np.float32)])
def test_cta_pair_kernel_shapes(batch, M, N, K, out_dt):
    """Shapes large enough for the CTA-pair kernel (256 x 256 tiles, cta_group::2 MMAs): an odd
    number of 128-row tiles (the last pair's second CTA has no rows), ragged M and N, batches."""
    rng = np.random.default_rng(M + N + K)
    dt = np.float16 if out_dt == np.float16 else bfloat16
    shapeA = (batch, M, K) if batch > 1 else (M, K)
    shapeB = (batch, K, N) if batch > 1 else (K, N)
    A, B = _rand(rng, shapeA, dt, 1 / np.sqrt(K)), _rand(rng, shapeB, dt)
    got = gemm_device(A, B, out_dt)
    assert rel_err(got, orc.gemm(A, B)) < (1e-4 if out_dt == np.float32 else TOL)
    no_device_error()


@pytest.mark.parametrize("M,N,K,out_dt,world", [(2048, 8192, 264, bfloat16, 2), (384, 1024, 512, bfloat16, 2),
                                                (2304, 8192, 128, np.float32, 2), (200, 1088, 72, bfloat16, 8),
                                                (1000, 2112, 520, np.float16, 4), (129, 48, 64, np.float32, 3),
                                                (512, 1024, 1088, bfloat16, 2), (2304, 2048, 2048, np.float32, 4),
                                                (200, 1088, 1032, bfloat16, 8), (4096, 4096, 4096, bfloat16, 4), (2048, 3072, 2048, np.float16, 3),
                                                (4864, 8192, 1024, bfloat16, 2)])
def test_fused_all_gather_epilogue_with_local_copies(lib, M, N, K, out_dt, world):
    """The column-parallel GEMM's epilogue stores each finished piece into every rank's Y. Here the
    "ranks" run one after the other on one GPU with all Y copies local, which exercises the per-copy
    stores and the rotation over the copies (ragged M, column blocks that are not a multiple of the
    tile width, an odd number of 128-row tiles, 2 to 8 ranks, 16-bit and fp32 outputs) and, with at
    most four copies, 16 k-blocks or more and fewer than four waves of tiles, the first wave of
    units split over the K loop between neighbouring clusters (an odd number of k-blocks, a ragged
    last one, whole tiles following the split wave; the last case has enough tiles to run unsplit
    with a long K loop); every copy must hold the complete product."""
    from tessera_b200 import _lib, device
    from tessera_b200.device import DeviceArray
    rng = np.random.default_rng(M + K)
    dt = np.float16 if out_dt == np.float16 else bfloat16
    A, B = _rand(rng, (M, K), dt, 1 / np.sqrt(K)), _rand(rng, (K, N), dt)
    dA, dB = DeviceArray.from_host(A), DeviceArray.from_host(B)
    ys = [DeviceArray.zeros((M, N), out_dt) for _ in range(world)]
    ptrs = (ctypes.c_void_p * world)(*[y.ptr for y in ys])
    for rank in range(world):
        _lib.call("tessera_sm100_gemm_allgather_device", dA.ptr, dB.ptr, ptrs, world, rank, M, N, K,
                  device.dtype_code(dt), device.dtype_code(out_dt), None)
    ref = orc.gemm(A, B)
    first = ys[0].download()
    assert rel_err(first, ref) < (1e-4 if out_dt == np.float32 else TOL)
    for y in ys[1:]:
        np.testing.assert_array_equal(y.download(), first)
    no_device_error()
