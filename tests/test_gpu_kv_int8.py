"""int8 KV cache on the GPU: per-token quantisation is bit-exact against the reference's
quantize_kv, and decode attention over the int8 bytes equals the reference's attention over the
dequantised cache (fixture made by the reference's KVCacheHandle(quantize_bits=8); oracle at
larger sizes, dense and paged, ragged lengths, appends)."""
import ctypes
import os

import numpy as np
import pytest

from oracle import tessera_oracle as orc
from tests.gpu_util import TOL, no_device_error, rel_err

pytestmark = pytest.mark.gpu

from tessera_b200 import _lib, cache as pk, device  # noqa: E402
from tessera_b200.device import DeviceArray, bfloat16  # noqa: E402


def _bf(x):
    return np.asarray(x, np.float32).astype(bfloat16)


def _quantize(k, v):
    """k, v [T, H, D] host -> device 8-bit rows (stored as value + 128) + scales through the C ABI."""
    T, H, D = k.shape
    dk, dv = DeviceArray.from_host(k.reshape(T, H * D)), DeviceArray.from_host(v.reshape(T, H * D))
    kq, vq = DeviceArray((T, H, D), np.uint8), DeviceArray((T, H, D), np.uint8)
    ks, vs = DeviceArray((T,), np.float32), DeviceArray((T,), np.float32)
    _lib.call("tessera_sm100_quantize_kv_int8_device", dk.ptr, dv.ptr, kq.ptr, vq.ptr, ks.ptr, vs.ptr, None, T,
              H * D, device.dtype_code(k.dtype), None)
    return kq, vq, ks, vs


def test_quantisation_is_bit_exact(golden_dir):
    g = np.load(os.path.join(golden_dir, "paged.npz"))
    for dt in (bfloat16, np.float32):
        kq, vq, ks, vs = _quantize(g["q8_k"].astype(dt), g["q8_v"].astype(dt))
        np.testing.assert_array_equal(kq.download().astype(np.int16) - 128, g["q8_kq"])
        np.testing.assert_array_equal(vq.download().astype(np.int16) - 128, g["q8_vq"])
        np.testing.assert_array_equal(ks.download(), g["q8_scale"][0].reshape(-1))
        np.testing.assert_array_equal(vs.download(), g["q8_scale"][1].reshape(-1))


def test_fixture_paged_attention_over_int8_cache(golden_dir):
    g = np.load(os.path.join(golden_dir, "paged.npz"))
    k, v, Q = _bf(g["q8_k"]), _bf(g["q8_v"]), _bf(g["q8_Q"])
    cache = pk.PagedKVCache.from_dense(k[None], v[None], page_size=16, quantize_bits=8,
                                       page_order=np.random.default_rng(0).permutation(9))
    assert cache.k_pages.dtype == np.uint8
    got = pk.paged_attention(Q, cache)
    assert rel_err(got, g["q8_O"]) < TOL
    no_device_error()


@pytest.mark.parametrize("Sk,splits", [(1000, 1), (4096, 4), (77, 1), (2500, 0)])
def test_dense_int8_decode_against_oracle(Sk, splits):
    rng = np.random.default_rng(Sk)
    B, Hq, Hkv, D = 3, 16, 2, 128
    k = _bf(rng.standard_normal((B, Sk, Hkv, D)) * rng.uniform(0.1, 4.0, (B, Sk, 1, 1)))
    v = _bf(rng.standard_normal((B, Sk, Hkv, D)))
    q = _bf(rng.standard_normal((B, Hq, D)))
    kq = np.empty((B, Hkv, Sk, D), np.int8)
    vq = np.empty((B, Hkv, Sk, D), np.int8)
    ks, vs = np.empty((B, Sk), np.float32), np.empty((B, Sk), np.float32)
    ref = np.empty((B, Hq, D), np.float32)
    for b in range(B):
        a, c, sc = orc.quantize_kv(k[b], v[b], 8)
        kq[b], vq[b] = a.transpose(1, 0, 2), c.transpose(1, 0, 2)
        ks[b], vs[b] = sc[0].reshape(-1), sc[1].reshape(-1)
        kd, vd = orc.dequantize_kv(a, c, sc)
        ref[b] = orc.gqa_attention(q[b][None, :, None, :], kd.transpose(1, 0, 2)[None], vd.transpose(1, 0, 2)[None],
                                   Hq, Hkv)[0, :, 0]
    lib = _lib.load()
    ns = splits or lib.tessera_sm100_attn_decode_int8_splits(B, Hq, Hkv, Sk)
    scr = DeviceArray((max(1, lib.tessera_sm100_attn_decode_scratch_bytes(B, Hq, max(ns, 1))),), np.uint8)
    stored = [(t.astype(np.int16) + 128).astype(np.uint8) for t in (kq, vq)]   # the cache's byte form
    dq, dkq, dvq, dks, dvs = (DeviceArray.from_host(t) for t in (q, stored[0], stored[1], ks, vs))
    out = DeviceArray.zeros((B, Hq, D), bfloat16)
    _lib.call("tessera_sm100_attn_decode_int8_device", dq.ptr, dkq.ptr, dvq.ptr, dks.ptr, dvs.ptr, out.ptr, B, Hq,
              Hkv, Sk, D, ctypes.c_float(1 / np.sqrt(D)), ns, scr.ptr, None)
    assert rel_err(out.download(), ref) < TOL
    no_device_error()


@pytest.mark.parametrize("page_size", [8, 16, 64, 256])
def test_paged_int8_ragged_batch_and_append(page_size):
    rng = np.random.default_rng(page_size + 1)
    B, Hq, Hkv, S = 4, 8, 2, 600
    lens = np.array([599, 1, 64, 333])
    K = _bf(rng.standard_normal((B, S + 4, Hkv, 128)) * rng.uniform(0.2, 3.0, (B, S + 4, 1, 1)))
    V = _bf(rng.standard_normal((B, S + 4, Hkv, 128)))
    need = int(np.maximum(1, -(-(lens + 4) // page_size)).sum())
    cache = pk.PagedKVCache.from_dense(K, V, page_size=page_size, seq_lens=lens, num_pages=need + 3,
                                       page_order=rng.permutation(need + 3),
                                       max_pages_per_seq=int(-(-(S + 4) // page_size)), quantize_bits=8)

    def check(cur):
        Q = _bf(rng.standard_normal((B, Hq, 128)))
        got = pk.paged_decode(Q, cache)
        for b in range(B):
            n = int(cur[b])
            kq, vq, sc = orc.quantize_kv(K[b, :n], V[b, :n], 8)
            kd, vd = orc.dequantize_kv(kq, vq, sc)
            ref = orc.gqa_attention(Q[b][None, :, None, :], kd.transpose(1, 0, 2)[None], vd.transpose(1, 0, 2)[None],
                                    Hq, Hkv)[0, :, 0]
            assert rel_err(got[b], ref) < TOL, f"sequence {b}"

    check(lens)
    for step in range(3):   # decode-loop appends, across page edges for the short pages
        kn = np.stack([K[b, lens[b] + step] for b in range(B)])
        vn = np.stack([V[b, lens[b] + step] for b in range(B)])
        cache.append(kn, vn)
        np.testing.assert_array_equal(cache.seq_lens.download(), lens + step + 1)
        check(lens + step + 1)
    no_device_error()
