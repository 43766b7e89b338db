"""Pins the numpy oracle against fixtures produced by the reference implementation itself
(tests/golden/make_golden.py). Exact equality is expected wherever the oracle performs the same
numpy operations; attention is compared at 1e-6 because the oracle walks query blocks."""
import os

import numpy as np

from oracle import tessera_oracle as orc


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


def test_gemm_matches_reference(golden_dir):
    g = _load(golden_dir, "gemm.npz")
    for i in range(int(g["n"])):
        y = orc.gemm(g[f"A{i}"], g[f"B{i}"])
        np.testing.assert_array_equal(y, g[f"Y{i}"])
        np.testing.assert_array_equal(y, g[f"Yregion{i}"])
        # rounding to storage is idempotent on stored values
        dt = str(g[f"dtype{i}"])
        np.testing.assert_array_equal(orc.round_to_storage(g[f"A{i}"], dt), g[f"A{i}"])


def test_fused_epilogue_matches_reference(golden_dir):
    g = _load(golden_dir, "gemm.npz")
    y = orc.gemm(g["epiA"], g["epiB"])
    for act in ("linear", "relu", "gelu", "silu"):
        got = orc.fused_epilogue(y, bias=g["epi_bias"], activation=act, residual=g["epi_res"])
        np.testing.assert_allclose(got, g[f"epi_{act}"], rtol=1e-6, atol=1e-6)


def test_attention_matches_reference(golden_dir):
    g = _load(golden_dir, "attention.npz")
    for i in range(int(g["n"])):
        B, Hq, Hkv, Sq, Sk, D, causal = (int(v) for v in g[f"meta{i}"])
        if Hq == Hkv:
            o = orc.flash_attn(g[f"Q{i}"], g[f"K{i}"], g[f"V{i}"], causal=bool(causal), q_block=16)
        else:
            o = orc.gqa_attention(g[f"Q{i}"], g[f"K{i}"], g[f"V{i}"], Hq, Hkv, causal=bool(causal))
        np.testing.assert_allclose(o, g[f"O{i}"], rtol=0, atol=2e-6)


def test_softmax_merge_matches_reference(golden_dir):
    g = _load(golden_dir, "attention.npz")
    o, m, l = orc.softmax_merge(g["merge_oa"], g["merge_ma"], g["merge_la"], g["merge_ob"],
                                g["merge_mb"], g["merge_lb"])
    np.testing.assert_array_equal(o, g["merge_o"])
    np.testing.assert_array_equal(m, g["merge_m"])
    np.testing.assert_array_equal(l, g["merge_l"])
    np.testing.assert_array_equal(orc.softmax_finalize(o, l), g["merge_final"])


def test_routing_and_permutation_match_reference(golden_dir):
    g = _load(golden_dir, "moe.npz")
    for i in range(int(g["n_route"])):
        T, E, k, cap = (int(v) for v in g[f"meta{i}"])
        r = orc.route_tokens(g[f"logits{i}"], k, True, None if cap < 0 else cap)
        np.testing.assert_array_equal(r.assignment, g[f"assignment{i}"])
        np.testing.assert_array_equal(r.weights, g[f"weights{i}"])
        np.testing.assert_array_equal(r.load, g[f"load{i}"])
        assert r.overflow == int(g[f"overflow{i}"])
        p = orc.moe_permutation(r.assignment, r.weights, E)
        np.testing.assert_array_equal(p.token_of_slot, g[f"token_of_slot{i}"])
        np.testing.assert_array_equal(p.expert_of_slot, g[f"expert_of_slot{i}"])
        np.testing.assert_array_equal(p.weight_of_slot, g[f"combine_weights{i}"])
        np.testing.assert_array_equal(p.group_sizes, g[f"group_sizes{i}"])
        np.testing.assert_array_equal(p.group_offsets, g[f"group_offsets{i}"])
        assert p.token_of_slot.dtype == np.int32 and p.group_offsets.dtype == np.int32
        # slot_of_assignment is the inverse of the permutation
        kept = p.slot_of_assignment >= 0
        np.testing.assert_array_equal(kept, r.assignment >= 0)
        t_idx, _ = np.nonzero(kept)
        np.testing.assert_array_equal(p.token_of_slot[p.slot_of_assignment[kept]], t_idx)


def test_moe_compute_matches_reference(golden_dir):
    g = _load(golden_dir, "moe.npz")
    x, Wr, Wg, Wu, Wd, gs = (g[k] for k in ("x", "Wr", "Wg", "Wu", "Wd", "gs"))
    np.testing.assert_array_equal(orc.grouped_gemm(x, Wg, gs), g["grouped_gemm"])
    np.testing.assert_allclose(orc.moe_swiglu_block(x, Wg, Wu, Wd, gs), g["swiglu_block"],
                               rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(orc.moe_layer(x, Wr, Wg, Wu, Wd, top_k=1), g["moe_layer_k1"],
                               rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(orc.moe_layer(x, Wr, Wg, Wu, Wd, top_k=2), g["moe_layer_k2"],
                               rtol=1e-5, atol=1e-6)


def test_expert_parallel_matches_reference(golden_dir):
    g = _load(golden_dir, "moe.npz")
    x, Wr, Wg, Wu, Wd = (g[k] for k in ("x", "Wr", "Wg", "Wu", "Wd"))
    logits = orc.gemm(x, Wr)
    for R in (2, 4):
        assert int(g[f"megamoe_dropped_w{R}"]) == 0
        y = orc.expert_parallel_moe(x, logits, Wg, Wu, Wd, top_k=2, world_size=R)
        np.testing.assert_allclose(y, g[f"megamoe_w{R}"], rtol=1e-4, atol=1e-5)
    # and the expert-parallel form equals the single-device layer
    np.testing.assert_allclose(orc.expert_parallel_moe(x, logits, Wg, Wu, Wd, top_k=2, world_size=2),
                               g["moe_layer_k2"], rtol=1e-4, atol=1e-5)


def test_seeded_moe_routing_known_answer():
    """Per-expert slot counts of the 8192-token benchmark routing (seed 1005), as produced by the
    reference's route_tokens."""
    rng = np.random.default_rng(1005)
    rng.standard_normal((8192, 4096), dtype=np.float32)
    logits = rng.standard_normal((8192, 8), dtype=np.float32)
    r = orc.route_tokens(logits, 2)
    assert r.load.tolist() == [1994, 2066, 2065, 2092, 2074, 2036, 1965, 2092]
    srt = np.sort(logits, axis=1)
    assert (srt[:, -2] - srt[:, -3]).min() > 1e-5  # no near-ties: the top-2 choice is well-posed


def test_paged_attention_matches_reference(golden_dir):
    g = _load(golden_dir, "paged.npz")
    for i in range(int(g["n"])):
        Hq, Hkv, q_len, n, L, causal = (int(x) for x in g[f"meta{i}"])
        kp, vp, table = orc.paged_pack(g[f"k{i}"], g[f"v{i}"], L)
        np.testing.assert_array_equal(kp, g[f"kpages{i}"])
        np.testing.assert_array_equal(table, g[f"table{i}"])
        idx = g[f"idx{i}"] if f"idx{i}" in g else None
        o = orc.paged_attention(g[f"Q{i}"], kp, vp, table, n, causal=bool(causal), token_indices=idx)
        np.testing.assert_allclose(o, g[f"O{i}"], rtol=1e-6, atol=1e-6)
    # scattered physical placement
    n = int(g["sn"])
    gk, gv = orc.paged_gather(g["sk_pages"], g["sv_pages"], g["stable"], n, g["sgidx"])
    np.testing.assert_array_equal(gk, g["sgk"])
    np.testing.assert_array_equal(gv, g["sgv"])
    o = orc.paged_attention(g["sQ"], g["sk_pages"], g["sv_pages"], g["stable"], n)
    np.testing.assert_allclose(o, g["sO"], rtol=1e-6, atol=1e-6)


def test_multi_head_attention_and_linear_match_reference(golden_dir):
    g = _load(golden_dir, "attention.npz")
    for i in range(int(g["mha_n"])):
        B, H, Sq, Sk, causal = (int(x) for x in g[f"mhameta{i}"])
        o = orc.multi_head_attention(g[f"mhaQ{i}"], g[f"mhaK{i}"], g[f"mhaV{i}"], H, causal=bool(causal))
        np.testing.assert_allclose(o, g[f"mhaO{i}"], rtol=2e-6, atol=2e-6)
    np.testing.assert_allclose(orc.linear(g["lin_x"], g["lin_W"], g["lin_b"]), g["lin_y"], rtol=1e-6, atol=1e-6)


def test_region_oracles_match_reference(golden_dir):
    g = _load(golden_dir, "gemm.npz")
    np.testing.assert_allclose(orc.gated_matmul(g["gatedA"], g["gatedWg"], g["gatedWu"]), g["gatedO"],
                               rtol=1e-5, atol=1e-5)
    sc = float(1.0 / np.sqrt(128.0))
    np.testing.assert_allclose(orc.attention_region(g["regQ"], g["regK"], g["regV"], sc, False), g["regO"],
                               rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(orc.attention_region(g["regQ"], g["regK"], g["regV"], sc, True), g["regOc"],
                               rtol=1e-5, atol=1e-6)


def _lane_kwargs(kw):
    scale, causal, wl, wr, cap = (float(x) for x in kw)
    return dict(scale=scale, causal=bool(causal), window=None if wl < 0 and wr < 0 else (int(wl), int(wr)),
                softcap=cap or None)


def test_attention_lane_contract_matches_reference(golden_dir):
    g = _load(golden_dir, "attention.npz")
    for i in range(int(g["lane_n"])):
        bias = g[f"laneb{i}"] if f"laneb{i}" in g else None
        o = orc.attention_lane(g[f"laneq{i}"], g[f"lanek{i}"], g[f"lanev{i}"], bias=bias, **_lane_kwargs(g[f"lanekw{i}"]))
        np.testing.assert_allclose(o, g[f"laneo{i}"], rtol=1e-5, atol=2e-6)
    Sq, Sk = g["biasQ"].shape[2], g["biasK"].shape[2]
    o = orc.attention_lane(g["biasQ"], g["biasK"], g["biasV"], scale=1 / np.sqrt(32.0), causal=True,
                           bias=np.broadcast_to(g["biasB"], (2, 2, Sq, Sk)), causal_shift=max(Sk - Sq, 0))
    np.testing.assert_allclose(o, g["biasO"], rtol=1e-5, atol=2e-6)


def test_fp8_quantised_grouped_gemm_matches_reference(golden_dir):
    g = _load(golden_dir, "moe.npz")
    dq, sc = orc.quantize_fp8(g["q_x"])
    np.testing.assert_array_equal(dq, g["q_x_dq"])
    assert sc == g["q_x_scale"]
    np.testing.assert_allclose(orc.grouped_gemm_fp8(g["q_x"], g["q_wg"], g["q_sizes"]), g["q_gg"], rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(orc.moe_swiglu_block_fp8(g["q_x"], g["q_wg"], g["q_wu"], g["q_wd"], g["q_sizes"]),
                               g["q_block"], rtol=1e-5, atol=1e-6)


def test_int8_kv_cache_matches_reference(golden_dir):
    g = _load(golden_dir, "paged.npz")
    kq, vq, sc = orc.quantize_kv(g["q8_k"], g["q8_v"], 8)
    np.testing.assert_array_equal(kq, g["q8_kq"])
    np.testing.assert_array_equal(vq, g["q8_vq"])
    np.testing.assert_array_equal(sc, g["q8_scale"])
    kd, vd = orc.dequantize_kv(kq, vq, sc)
    kp, vp, table = orc.paged_pack(kd, vd, 16)
    o = orc.paged_attention(g["q8_Q"], kp, vp, table, kd.shape[0])
    np.testing.assert_allclose(o, g["q8_O"], rtol=1e-5, atol=1e-6)


def test_attention_backward_lane_matches_reference(golden_dir):
    g = _load(golden_dir, "attention_bwd.npz")
    for i in range(int(g["n"])):
        bias = g[f"b{i}"] if f"b{i}" in g else None
        got = orc.attention_lane_backward(g[f"do{i}"], g[f"q{i}"], g[f"k{i}"], g[f"v{i}"], bias=bias,
                                          **_lane_kwargs(g[f"kw{i}"]))
        for name, a in zip(("dq", "dk", "dv"), got):
            np.testing.assert_allclose(a, g[f"{name}{i}"], rtol=2e-5, atol=5e-6, err_msg=f"case {i} {name}")


def test_attention_backward_is_the_gradient_of_the_forward_lane():
    """Central differences of sum(O * dO) through the forward oracle, in float64."""
    rng = np.random.default_rng(3)
    q = rng.standard_normal((1, 2, 4, 3)); k = rng.standard_normal((1, 1, 5, 3)); v = rng.standard_normal((1, 1, 5, 2))
    do = rng.standard_normal((1, 2, 4, 2))
    bias = rng.standard_normal((1, 2, 4, 5)) * 0.2
    kw = dict(scale=0.6, causal=True, window=(3, 2), softcap=1.5, causal_shift=1)

    def loss(q_, k_, v_):
        # float64 forward with the same masks (the float32 oracle is too coarse to differentiate)
        m = np.arange(4)[:, None]; n = np.arange(5)[None, :]
        keep = (n <= m + 1) & (n >= m - 3) & (n <= m + 2)
        tot = 0.0
        for h in range(2):
            s = q_[0, h] @ k_[0, 0].T * 0.6 + bias[0, h]
            s = 1.5 * np.tanh(s / 1.5)
            s = np.where(keep, s, -np.inf)
            p = np.exp(s - s.max(-1, keepdims=True)); p /= p.sum(-1, keepdims=True)
            tot += ((p @ v_[0, 0]) * do[0, h]).sum()
        return tot

    dq, dk, dv = orc.attention_lane_backward(do, q, k, v, bias=bias, **kw)
    eps = 1e-5
    for arr, grad in ((q, dq), (k, dk), (v, dv)):
        num = np.zeros_like(arr)
        it = np.nditer(arr, flags=["multi_index"])
        for _ in it:
            idx = it.multi_index
            old = arr[idx]
            arr[idx] = old + eps; hi = loss(q, k, v)
            arr[idx] = old - eps; lo = loss(q, k, v)
            arr[idx] = old
            num[idx] = (hi - lo) / (2 * eps)
        np.testing.assert_allclose(grad, num, rtol=2e-3, atol=2e-4)


def test_attention_backward_rows_without_legal_keys_contribute_nothing():
    rng = np.random.default_rng(4)
    q = rng.standard_normal((1, 1, 10, 4), dtype=np.float32); k = rng.standard_normal((1, 1, 4, 4), dtype=np.float32)
    v = rng.standard_normal((1, 1, 4, 4), dtype=np.float32); do = rng.standard_normal((1, 1, 10, 4), dtype=np.float32)
    dq, dk, dv = orc.attention_lane_backward(do, q, k, v, scale=0.5, causal=True, window=(1, 0))
    assert np.isfinite(dq).all() and np.isfinite(dk).all() and np.isfinite(dv).all()
    assert not dq[0, 0, 5:].any()   # rows 5.. see only keys >= 4, which do not exist


def test_nvfp4_quantisation_and_grouped_gemms_match_reference(golden_dir):
    g = _load(golden_dir, "quant4.npz")
    dq, sc, _ = orc.quantize_nvfp4(g["n_x"])
    np.testing.assert_array_equal(dq, g["n_dq"])
    np.testing.assert_array_equal(sc, g["n_scales"])
    assert not dq[5, :16].any() and g["n_x"][5, :16].any()      # scale rounded to zero: block reads as 0
    dq5, sc5 = orc.quantize_fp8(g["n_x"], "e5m2")
    np.testing.assert_array_equal(dq5, g["e5_dq"])
    assert sc5 == g["e5_scale"]
    np.testing.assert_allclose(orc.grouped_gemm_fp8(g["g_x"], g["g_w"], g["g_sizes"], "e5m2"), g["gg_fp8_e5m2"],
                               rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(orc.moe_swiglu_block_fp8(g["g_x"], g["g_wg"], g["g_wu"], g["g_wd"], g["g_sizes"], "e5m2"),
                               g["blk_fp8_e5m2"], rtol=1e-5, atol=1e-6)
    for q in ("nvfp4", "fp8xfp4", "fp8_e5m2xnvfp4"):
        np.testing.assert_allclose(orc.grouped_gemm_fp4(g["g_x"], g["g_w"], g["g_sizes"], q), g[f"gg_{q}"],
                                   rtol=1e-6, atol=1e-6)
        np.testing.assert_allclose(orc.moe_swiglu_block_fp4(g["g_x"], g["g_wg"], g["g_wu"], g["g_wd"], g["g_sizes"], q),
                                   g[f"blk_{q}"], rtol=1e-5, atol=1e-6)
