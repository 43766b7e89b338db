"""Multi-op chains that stay on the device: strided attention over [B, S, H*D] operands
(nn.functional.multi_head_attention), linear with the bias in the GEMM epilogue, and a
QKV-projection -> attention -> output-projection block under @jit, against the oracle and the
reference-made fixture."""
import os

import numpy as np
import pytest

from oracle import tessera_oracle as orc
from tests.gpu_util import TOL, no_device_error, rel_err

pytestmark = pytest.mark.gpu

import tessera_b200 as tessera  # noqa: E402
from tessera_b200 import device  # noqa: E402
from tessera_b200.device import DeviceArray, bfloat16, slice_last  # noqa: E402
from tessera_b200.nn import functional as F  # noqa: E402


def _bf(x):
    return np.asarray(x, np.float32).astype(bfloat16)


def test_multi_head_attention_fixture(golden_dir):
    g = np.load(os.path.join(golden_dir, "attention.npz"))
    for i in range(int(g["mha_n"])):
        B, H, Sq, Sk, causal = (int(x) for x in g[f"mhameta{i}"])
        got = F.multi_head_attention(_bf(g[f"mhaQ{i}"]), _bf(g[f"mhaK{i}"]), _bf(g[f"mhaV{i}"]), H,
                                     causal=bool(causal))
        assert got.shape == (B, Sq, H * 128)
        assert rel_err(got, g[f"mhaO{i}"]) < TOL, f"case {i}"
    y = F.linear(_bf(g["lin_x"]), _bf(g["lin_W"]), g["lin_b"])
    assert y.shape == (2, 24, 48) and y.dtype == bfloat16
    assert rel_err(y, g["lin_y"]) < TOL
    no_device_error()


@pytest.mark.parametrize("Sq,Sk,causal", [(300, 300, True), (1, 513, False), (130, 700, True)])
def test_strided_attention_equals_dense_kernel(Sq, Sk, causal):
    """[B, S, H, D] operands through strided tensor maps give the same bits as the dense
    [B, H, S, D] call on transposed copies (same kernel, same tiles)."""
    rng = np.random.default_rng(Sq + Sk)
    B, Hq, Hkv = 2, 4, 2
    q = _bf(rng.standard_normal((B, Sq, Hq * 128)))
    k = _bf(rng.standard_normal((B, Sk, Hkv * 128)))
    v = _bf(rng.standard_normal((B, Sk, Hkv * 128)))
    got = F.multi_head_attention(q, k, v, Hq, causal=causal, num_kv_heads=Hkv)
    t = lambda a, h: np.ascontiguousarray(a.reshape(B, a.shape[1], h, 128).transpose(0, 2, 1, 3))
    dense = tessera.ops.flash_attn(t(q, Hq), t(k, Hkv), t(v, Hkv), causal=causal)
    dense = np.ascontiguousarray(np.asarray(dense).transpose(0, 2, 1, 3)).reshape(B, Sq, Hq * 128)
    np.testing.assert_array_equal(np.asarray(got).view(np.uint16), dense.view(np.uint16))
    assert rel_err(got, orc.multi_head_attention(q, k, v, Hq, causal=causal, num_kv_heads=Hkv)) < TOL
    no_device_error()


def test_attention_block_stays_on_device_under_jit():
    """QKV projection -> attention on column windows of the projection output -> output
    projection: three launches, no transposes, no host round trips between them."""
    rng = np.random.default_rng(77)
    B, S, Hq, Hkv, hidden = 2, 256, 4, 2, 512
    wq, wkv = Hq * 128, Hkv * 128
    x = _bf(rng.standard_normal((B, S, hidden)) / 4)
    Wqkv = _bf(rng.standard_normal((hidden, wq + 2 * wkv)) / np.sqrt(hidden))
    bqkv = (rng.standard_normal(wq + 2 * wkv) / 4).astype(np.float32)
    Wo = _bf(rng.standard_normal((wq, hidden)) / np.sqrt(wq))
    seen = {}

    @tessera.jit(target="nvidia_sm100")
    def block(x, Wqkv, Wo):
        qkv = F.linear(x, Wqkv, bqkv)
        q, k, v = F.split_last(qkv, (wq, wkv, wkv))
        seen["types"] = (type(qkv).__name__, type(q).__name__)
        o = F.multi_head_attention(q, k, v, Hq, causal=True, num_kv_heads=Hkv)
        seen["launches_mid"] = device.launch_count()
        return F.linear(o, Wo)

    before = device.launch_count()
    y = block(x, Wqkv, Wo)
    assert seen["types"] == ("DeviceArray", "StridedView")
    assert device.launch_count() - before == 3           # GEMM, attention, GEMM
    qkv = _bf(orc.linear(x, Wqkv, bqkv))
    q, k, v = qkv[..., :wq], qkv[..., wq:wq + wkv], qkv[..., wq + wkv:]
    o = _bf(orc.multi_head_attention(q, k, v, Hq, causal=True, num_kv_heads=Hkv))
    ref = orc.linear(o, Wo)
    assert y.shape == (B, S, hidden) and y.dtype == bfloat16
    assert rel_err(y, ref) < 2 * TOL   # three bf16 roundings in the chain
    no_device_error()


def test_strided_view_copy_and_bad_strides(lib):
    rng = np.random.default_rng(1)
    a = _bf(rng.standard_normal((3, 5, 64)))
    d = DeviceArray.from_host(a)
    w = slice_last(d, 16, 48)
    np.testing.assert_array_equal(w.download().view(np.uint16), a[..., 16:48].view(np.uint16))
    with pytest.raises(ValueError):
        slice_last(d, 3, 48)       # not 16-byte aligned
    import ctypes
    bad = (ctypes.c_longlong * 3)(128 * 4, 128, 4)   # position stride of 4 elements: not 16 bytes
    ok = (ctypes.c_longlong * 3)(128 * 4, 128, 128)
    q = DeviceArray.zeros((1, 4, 1, 128), bfloat16)
    rc = lib.tessera_sm100_flash_attn_strided_device(q.ptr, q.ptr, q.ptr, q.ptr, 1, 1, 1, 4, 4, 128, bad, ok, ok,
                                                     ok, ctypes.c_float(0.1), 0, None)
    assert rc == 1
