"""Attention parity on the GPU: prefill (tcgen05) and split-KV decode vs the oracle and the
reference-made fixtures. Cases follow tests/device/nvidia/test_flash_attention.py (MHA/GQA/MQA,
causal, ragged lengths)."""
import os

import numpy as np
import pytest

from oracle import tessera_oracle as orc
from tests.gpu_util import TOL, attn_device, rel_err

pytestmark = pytest.mark.gpu

from tessera_b200.device import bfloat16  # noqa: E402


def _qkv(rng, B, Hq, Hkv, Sq, Sk, D=128):
    q = rng.standard_normal((B, Hq, Sq, D), dtype=np.float32).astype(bfloat16)
    k = rng.standard_normal((B, Hkv, Sk, D), dtype=np.float32).astype(bfloat16)
    v = rng.standard_normal((B, Hkv, Sk, D), dtype=np.float32).astype(bfloat16)
    return q, k, v


def _ref(q, k, v, causal):
    Hq, Hkv = q.shape[1], k.shape[1]
    if Hq == Hkv:
        return orc.flash_attn(q, k, v, causal=causal)
    return orc.gqa_attention(q, k, v, Hq, Hkv, causal=causal)


PREFILL = [(1, 1, 1, 256, 256, False), (1, 1, 1, 256, 256, True), (1, 2, 2, 128, 128, True),
           (1, 2, 1, 384, 384, True), (2, 4, 2, 512, 512, True), (1, 2, 2, 300, 300, True),
           (1, 2, 2, 300, 300, False), (1, 2, 1, 128, 512, True), (1, 1, 1, 77, 1000, True),
           (1, 1, 1, 1000, 77, False), (1, 8, 1, 130, 130, True), (1, 1, 1, 5, 3, False),
           # the 64-key block walk: exactly one block, a second tile of one row, more query rows than keys
           # under the causal mask, and a key sequence long enough for every ring slot to wrap many times
           (1, 1, 1, 200, 64, True), (1, 2, 1, 257, 65, True), (1, 1, 1, 129, 129, True),
           (1, 1, 1, 1000, 77, True), (1, 2, 2, 64, 4096, True), (1, 1, 1, 320, 4096, False)]


@pytest.mark.parametrize("B,Hq,Hkv,Sq,Sk,causal", PREFILL)
def test_prefill_matches_oracle(B, Hq, Hkv, Sq, Sk, causal):
    q, k, v = _qkv(np.random.default_rng(Sq * 7 + Sk), B, Hq, Hkv, Sq, Sk)
    assert rel_err(attn_device(q, k, v, causal), _ref(q, k, v, causal)) < TOL


@pytest.mark.parametrize("causal", [False, True])
def test_prefill_raises_the_running_maximum_in_every_block(causal):
    """Scores that keep growing along the key axis (by more than 2^8 per 64 keys, at a rate that differs from
    row to row) make the kernel raise its running maximum and rescale the output accumulator in TMEM in
    block after block -- the path random data never takes after the first block."""
    rng = np.random.default_rng(11)
    B, H, Sq, Sk, D = 1, 2, 384, 1024, 128
    u = rng.standard_normal(D).astype(np.float32)
    u /= np.linalg.norm(u)
    row_gain = (1.0 + 3.0 * np.arange(Sq, dtype=np.float32) / Sq)[None, None, :, None]
    key_ramp = (np.arange(Sk, dtype=np.float32) / Sk)[None, None, :, None]
    q = (u * row_gain + 0.05 * rng.standard_normal((B, H, Sq, D), dtype=np.float32)).astype(bfloat16)
    k = (u * key_ramp * 424.0 + 0.05 * rng.standard_normal((B, H, Sk, D), dtype=np.float32)).astype(bfloat16)
    v = rng.standard_normal((B, H, Sk, D), dtype=np.float32).astype(bfloat16)
    # scale * q.k runs from 0 to about 37..150 over the keys: 3..13 (log2 units) per block of 64
    assert rel_err(attn_device(q, k, v, causal), _ref(q, k, v, causal)) < TOL


def test_golden_fixtures(golden_dir):
    g = np.load(os.path.join(golden_dir, "attention.npz"))
    for i in range(int(g["n"])):
        B, Hq, Hkv, Sq, Sk, D, causal = (int(x) for x in g[f"meta{i}"])
        q, k, v = (g[f"{n}{i}"].astype(bfloat16) for n in "QKV")
        splits = 0 if Sq == 1 else None
        assert rel_err(attn_device(q, k, v, bool(causal), decode_splits=splits), g[f"O{i}"]) < TOL


DECODE = [(2, 8, 2, 300, 1), (2, 8, 2, 300, 0), (3, 32, 8, 2048, 0), (1, 16, 1, 777, 3),
          (2, 4, 4, 64, 0), (1, 32, 8, 5000, 5), (1, 24, 2, 130, 2), (1, 8, 8, 1, 0)]


@pytest.mark.parametrize("B,Hq,Hkv,Sk,splits", DECODE)
def test_decode_matches_oracle(B, Hq, Hkv, Sk, splits):
    q, k, v = _qkv(np.random.default_rng(Sk + splits), B, Hq, Hkv, 1, Sk)
    got = attn_device(q, k, v, False, decode_splits=splits)
    assert rel_err(got, _ref(q, k, v, False)) < TOL


def test_decode_equals_prefill_kernel_on_one_token():
    q, k, v = _qkv(np.random.default_rng(4), 2, 8, 2, 1, 700)
    a = attn_device(q, k, v, False, decode_splits=0).astype(np.float32)
    b = attn_device(q, k, v, True).astype(np.float32)  # causal with Sq=1 masks nothing
    assert rel_err(a, b) < TOL


def test_config3_prefill_full_size_properties():
    """B=8 H=32 S=4096 D=128 causal: sampled heads against the oracle, and with V = 1 every output
    element is 1 (softmax rows sum to one)."""
    inp = orc.make_inputs("attn_prefill")
    q, k, v = inp["Q"], inp["K"], inp["V"]
    o = attn_device(q, k, v, True)
    for (b, h) in [(0, 0), (7, 31), (3, 17)]:
        ref = orc.flash_attn(q[b:b + 1, h:h + 1], k[b:b + 1, h:h + 1], v[b:b + 1, h:h + 1], causal=True)
        assert rel_err(o[b, h], ref[0, 0]) < TOL
    ones = np.ones_like(v)
    o1 = attn_device(q, k, ones, True).astype(np.float32)
    assert np.abs(o1 - 1.0).max() < TOL
    # row 0 of a causal head sees only key 0: the output is V[0]
    np.testing.assert_allclose(o[:, :, 0].astype(np.float32), v[:, :, 0].astype(np.float32), atol=TOL)


def test_config4_decode_full_size_properties():
    """batch 64, Hq 32, Hkv 8, KV 8192: sampled sequences against the oracle; V = 1 gives 1; the
    split count does not change the result beyond rounding."""
    inp = orc.make_inputs("attn_decode")
    q, k, v = inp["Q"], inp["K"], inp["V"]
    o = attn_device(q, k, v, False, decode_splits=0)
    for b in (0, 63, 31):
        ref = orc.gqa_attention(q[b:b + 1], k[b:b + 1], v[b:b + 1], 32, 8, causal=False)
        assert rel_err(o[b], ref[0]) < TOL
    o1 = attn_device(q, k, np.ones_like(v), False, decode_splits=0).astype(np.float32)
    assert np.abs(o1 - 1.0).max() < TOL
    o8 = attn_device(q, k, v, False, decode_splits=8)
    assert rel_err(o8, o) < TOL


def test_softmax_merge_and_finalize_fixture(golden_dir):
    """ops.softmax_merge / softmax_finalize on the GPU against the reference-made states."""
    import tessera_b200 as tessera
    g = np.load(os.path.join(golden_dir, "attention.npz"))
    o, m, l = tessera.ops.softmax_merge(g["merge_oa"], g["merge_ma"], g["merge_la"], g["merge_ob"], g["merge_mb"],
                                        g["merge_lb"])
    ro, rm, rl = orc.softmax_merge(g["merge_oa"], g["merge_ma"], g["merge_la"], g["merge_ob"], g["merge_mb"],
                                   g["merge_lb"])
    np.testing.assert_allclose(o, ro, rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(m, rm, rtol=0, atol=0)
    np.testing.assert_allclose(l, rl, rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(tessera.ops.softmax_finalize(o, l), orc.softmax_finalize(ro, rl), rtol=1e-6, atol=1e-6)
    with pytest.raises(ValueError):
        tessera.ops.softmax_merge(g["merge_oa"], g["merge_ma"], -g["merge_la"], g["merge_ob"], g["merge_mb"],
                                  g["merge_lb"])
    with pytest.raises(ValueError):
        tessera.ops.softmax_finalize(g["merge_oa"], g["merge_la"][:-1])


@pytest.mark.parametrize("cuts", [(700,), (64, 1000, 1001)])
def test_kv_sharded_decode_merges_to_full_attention(cuts):
    """Attention over a KV sequence cut into shards: per-shard states from the decode kernel,
    merged in any order, equal the unsharded result (the split-KV contract,
    python/tessera/_block_attnres_ops.py:104-146)."""
    import tessera_b200 as tessera
    rng = np.random.default_rng(sum(cuts))
    B, Hq, Hkv, Sk = 3, 8, 2, 1500
    q, k, v = _qkv(rng, B, Hq, Hkv, 1, Sk)
    edges = [0, *cuts, Sk]
    states = [tessera.ops.attn_decode_state(q, np.ascontiguousarray(k[:, :, a:b]), np.ascontiguousarray(v[:, :, a:b]))
              for a, b in zip(edges[:-1], edges[1:])]
    ref = orc.gqa_attention(q, k, v, Hq, Hkv)[:, :, 0]
    for order in (states, states[::-1]):
        o, m, l = order[0]
        for s in order[1:]:
            o, m, l = tessera.ops.softmax_merge(o, m, l, *s)
        assert rel_err(tessera.ops.softmax_finalize(o, l), ref) < TOL
    # the state itself: m is the row maximum of the scaled scores in natural-log units
    s0 = np.einsum("bhd,bhkd->bhk", np.asarray(q[:, :, 0], np.float32),
                   np.repeat(np.asarray(k[:, :, :edges[1]], np.float32), Hq // Hkv, axis=1)) / np.sqrt(128.0)
    np.testing.assert_allclose(states[0][1], s0.max(-1), rtol=1e-5, atol=1e-5)
