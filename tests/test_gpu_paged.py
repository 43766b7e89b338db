"""Paged KV on the GPU: the paged decode kernel, the append kernel and the gather kernel against
the oracle and the reference-made fixture. Cases follow tests/unit/test_paged_kv_native.py and
tests/integration/test_nvidia_paged_kv_native.py of the reference (full read, GQA, causal rows,
token subsets, non-identity tables) at the kernel's head dimension of 128."""
import os

import numpy as np
import pytest

from oracle import tessera_oracle as orc
from tests.gpu_util import TOL, no_device_error, rel_err

pytestmark = pytest.mark.gpu

import tessera_b200 as tessera  # noqa: E402
from tessera_b200 import cache as pk  # noqa: E402
from tessera_b200.device import DeviceArray, bfloat16  # noqa: E402


def _bf(x):
    return np.asarray(x, np.float32).astype(bfloat16)


def test_fixture_cases(golden_dir):
    g = np.load(os.path.join(golden_dir, "paged.npz"))
    for i in range(int(g["n"])):
        Hq, Hkv, q_len, n, L, causal = (int(x) for x in g[f"meta{i}"])
        kp, vp, table = orc.paged_pack(g[f"k{i}"], g[f"v{i}"], L)
        abi = pk.PagedKVBufferABI(kp, vp, table, n)
        idx = g[f"idx{i}"].tolist() if f"idx{i}" in g else None
        got, exe = pk.paged_attention(g[f"Q{i}"], abi, causal=bool(causal), token_indices=idx,
                                      return_execution=True)
        assert exe == "native_gpu" and got.shape == (Hq, q_len, 128)
        assert rel_err(got, g[f"O{i}"]) < TOL, f"case {i}"
    no_device_error()


def test_scattered_table_and_gather(golden_dir):
    g = np.load(os.path.join(golden_dir, "paged.npz"))
    n = int(g["sn"])
    abi = pk.PagedKVBufferABI(g["sk_pages"], g["sv_pages"], g["stable"], n)

    class State:  # a backend-native state exposing only its own page ABI
        def paged_kv_abi(self):
            return abi

    got = tessera.ops.paged_attention(g["sQ"], State())
    assert rel_err(got, g["sO"]) < TOL
    assert rel_err(tessera.ops.flash_attn(g["sQ"], kv_state=State()), g["sO"]) < TOL
    cache = pk.PagedKVCache.from_abi(abi)
    gk, gv = cache.gather(g["sgidx"])
    np.testing.assert_array_equal(gk, g["sgk"])   # stored values are bf16-exact: the gather is a copy
    np.testing.assert_array_equal(gv, g["sgv"])
    with pytest.raises(IndexError):
        cache.gather([n])
    no_device_error()


@pytest.mark.parametrize("page_size", [8, 16, 64, 128, 256])
def test_batched_decode_ragged_lengths(page_size):
    """Whole decode batch in one launch: per-sequence lengths and scattered pages."""
    rng = np.random.default_rng(page_size)
    B, Hq, Hkv, S = 5, 8, 2, 700
    lens = np.array([700, 1, 64, 333, 129])
    K = _bf(rng.standard_normal((B, S, Hkv, 128)))
    V = _bf(rng.standard_normal((B, S, Hkv, 128)))
    Q = _bf(rng.standard_normal((B, Hq, 128)))
    need = int(np.maximum(1, -(-lens // page_size)).sum())
    order = rng.permutation(need + 4)
    cache = pk.PagedKVCache.from_dense(K, V, page_size=page_size, seq_lens=lens, num_pages=need + 4,
                                       page_order=order)
    got = pk.paged_decode(Q, cache)
    for b in range(B):
        n = int(lens[b])
        ref = orc.gqa_attention(Q[b][None, :, None, :], K[b, :n].transpose(1, 0, 2)[None],
                                V[b, :n].transpose(1, 0, 2)[None], Hq, Hkv)[0, :, 0]
        assert rel_err(got[b], ref) < TOL, f"sequence {b}"
    no_device_error()


def test_stale_page_tail_is_ignored():
    """Whatever sits in a page beyond the sequence end (here NaN bit patterns) must not reach O."""
    rng = np.random.default_rng(3)
    n, L, H = 70, 64, 2
    k, v = _bf(rng.standard_normal((n, H, 128))), _bf(rng.standard_normal((n, H, 128)))
    kp, vp, table = orc.paged_pack(k, v, L)
    kp.reshape(-1, H, 128)[n:] = np.nan
    vp.reshape(-1, H, 128)[n:] = np.nan
    Q = _bf(rng.standard_normal((4, 1, 128)))
    got = pk.paged_attention(Q, pk.PagedKVBufferABI(kp, vp, table, n))
    assert np.isfinite(got).all()
    assert rel_err(got, orc.paged_attention(Q, *orc.paged_pack(k, v, L), n)) < TOL


def test_append_then_decode():
    """Decode loop: append a token per sequence on the device, attend, repeat across a page edge."""
    rng = np.random.default_rng(11)
    B, Hq, Hkv, L = 3, 4, 4, 8
    S0 = np.array([7, 8, 15])
    steps = 4
    K = _bf(rng.standard_normal((B, 32, Hkv, 128)))
    V = _bf(rng.standard_normal((B, 32, Hkv, 128)))
    cache = pk.PagedKVCache.from_dense(K, V, page_size=L, seq_lens=S0, num_pages=16, max_pages_per_seq=4,
                                       page_order=rng.permutation(16))
    for s in range(steps):
        kn = np.stack([K[b, S0[b] + s] for b in range(B)])
        vn = np.stack([V[b, S0[b] + s] for b in range(B)])
        cache.append(kn, vn)
        np.testing.assert_array_equal(cache.seq_lens.download(), S0 + s + 1)
        Q = _bf(rng.standard_normal((B, Hq, 128)))
        got = pk.paged_decode(Q, cache)
        for b in range(B):
            n = int(S0[b]) + s + 1
            ref = orc.flash_attn(Q[b][None, :, None, :], K[b, :n].transpose(1, 0, 2)[None],
                                 V[b, :n].transpose(1, 0, 2)[None])[0, :, 0]
            assert rel_err(got[b], ref) < TOL
    no_device_error()
    with pytest.raises(ValueError):   # sequence 2 now holds 19 tokens in 3 of 4 pages; fill and overflow
        for _ in range(20):
            cache.append(kn, vn)


def test_refused_append_changes_nothing():
    """Three sequences need a new page and two pages are free: the append is refused BEFORE any
    bookkeeping changes, so the host table, the free list and the device table still agree, and
    after a page is released the same append works and decodes correctly."""
    rng = np.random.default_rng(23)
    B, Hq, Hkv, L = 3, 4, 4, 8
    S0 = np.array([8, 8, 8])                      # every sequence sits exactly on a page edge
    K = _bf(rng.standard_normal((B, 16, Hkv, 128)))
    V = _bf(rng.standard_normal((B, 16, Hkv, 128)))
    cache = pk.PagedKVCache.from_dense(K, V, page_size=L, seq_lens=S0, num_pages=5, max_pages_per_seq=2)
    assert len(cache._free) == 2
    table0, owned0, free0 = cache._table.copy(), cache._owned.copy(), list(cache._free)
    kn = np.stack([K[b, S0[b]] for b in range(B)])
    vn = np.stack([V[b, S0[b]] for b in range(B)])
    with pytest.raises(ValueError, match="no free pages"):
        cache.append(kn, vn)
    np.testing.assert_array_equal(cache._table, table0)
    np.testing.assert_array_equal(cache._owned, owned0)
    assert list(cache._free) == free0
    np.testing.assert_array_equal(cache.page_table.download(), table0)
    np.testing.assert_array_equal(cache.seq_lens.download(), S0)
    cache.release(2)                              # sequence 2 gives its page back: three free pages
    assert len(cache._free) == 3
    cache.append(kn, vn)                          # 0 and 1 grow onto new pages, 2 restarts with one token
    np.testing.assert_array_equal(cache.seq_lens.download(), [9, 9, 1])
    Q = _bf(rng.standard_normal((B, Hq, 128)))
    got = pk.paged_decode(Q, cache)
    for b, n in ((0, 9), (1, 9)):
        ref = orc.flash_attn(Q[b][None, :, None, :], K[b, :n].transpose(1, 0, 2)[None],
                             V[b, :n].transpose(1, 0, 2)[None])[0, :, 0]
        assert rel_err(got[b], ref) < TOL
    no_device_error()


def test_device_resident_decode_matches_dense_kernel():
    """Same tokens through the paged kernel and the dense decode kernel: identical arithmetic
    order per tile, so the outputs agree bit for bit when the page size covers whole tiles."""
    rng = np.random.default_rng(21)
    B, Hq, Hkv, S = 4, 32, 8, 1024
    K = _bf(rng.standard_normal((B, S, Hkv, 128)))
    V = _bf(rng.standard_normal((B, S, Hkv, 128)))
    Q = _bf(rng.standard_normal((B, Hq, 128)))
    cache = pk.PagedKVCache.from_dense(K, V, page_size=64, page_order=rng.permutation(B * S // 64))
    paged = pk.paged_decode(DeviceArray.from_host(Q), cache).download()
    dense = tessera.ops.flash_attn(Q[:, :, None, :], np.ascontiguousarray(K.transpose(0, 2, 1, 3)),
                                   np.ascontiguousarray(V.transpose(0, 2, 1, 3)))[:, :, 0]
    np.testing.assert_array_equal(paged.view(np.uint16), np.asarray(dense).view(np.uint16))
    no_device_error()


def test_bad_table_entry_is_reported_not_dereferenced():
    rng = np.random.default_rng(5)
    K = _bf(rng.standard_normal((1, 64, 1, 128)))
    cache = pk.PagedKVCache.from_dense(K, K, page_size=16)
    cache._table[0, 2] = 999                       # outside [0, num_pages)
    cache.page_table.upload(cache._table)
    with pytest.raises(tessera._lib.BackendError):
        pk.paged_decode(_bf(rng.standard_normal((1, 1, 128))), cache)
    no_device_error()                              # the record was consumed by the failed call
