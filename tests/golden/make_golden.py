"""Generates the golden fixtures in this directory by running the REFERENCE implementation.

Run it where the reference checkout is available (it cannot run on a machine without it):

    TESSERA_REFERENCE=/path/to/tessera python tests/golden/make_golden.py

It imports the reference's own ``tessera`` package (pure Python + numpy) and records inputs and
outputs of the hot-path functions at small sizes:

  gemm.npz        tessera.ops.gemm (plain and with epilogue=) / MatmulRegion.reference  (python/tessera/__init__.py:239-254, 2658-2675,
                                                                   python/tessera/compiler/fusion_core.py:398-405)
  attention.npz   tessera.ops.flash_attn, nn.functional.gqa_attention, softmax_merge/finalize
                                                                  (python/tessera/__init__.py:1304-1356,
                                                                   python/tessera/nn/functional.py:349-356,
                                                                   python/tessera/_block_attnres_ops.py:104-146)
  paged.npz       cache.paged_attention over KVCacheHandle, materialize_paged_kv_abi,
                  PagedKVBufferABI.gather                         (python/tessera/cache/paged_kv.py:91-140, 421-559)
  moe.npz         distributed.moe.route_tokens, stdlib.moe.plan_dispatch +
                  compiler.moe_transport.descriptor_from_dispatch_plan, ops.grouped_gemm,
                  ops.moe_swiglu_block, nn.functional.moe_layer, distributed.moe.megamoe_layer

The committed .npz files are what ``tests/test_oracle_golden.py`` pins the oracle against.
"""
import os
import sys

import numpy as np

REF = os.environ.get("TESSERA_REFERENCE")
if not REF or not os.path.isdir(os.path.join(REF, "python", "tessera")):
    raise SystemExit("set TESSERA_REFERENCE to a checkout of the reference project (it is imported to make the fixtures)")
sys.dont_write_bytecode = True
sys.path.insert(0, os.path.join(REF, "python"))
sys.path.insert(1, REF)

import ml_dtypes  # noqa: E402
import tessera  # noqa: E402  (the reference package)
from tessera.compiler import fusion_core  # noqa: E402
from tessera.compiler.moe_transport import descriptor_from_dispatch_plan  # noqa: E402
from tessera.distributed import moe as dmoe  # noqa: E402
from tessera.nn import functional as F  # noqa: E402
from tessera.stdlib import moe as smoe  # noqa: E402
from tessera._block_attnres_ops import softmax_finalize, softmax_merge  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
bf16 = ml_dtypes.bfloat16


def rt(x, dt):
    """Round to 16-bit storage and return float32 (what the reference holds for 'bf16')."""
    return np.asarray(x, np.float32).astype(dt).astype(np.float32)


def gemm():
    rng = np.random.default_rng(101)
    out = {}
    for i, (b, M, N, K, dt) in enumerate([(1, 17, 9, 31, "bf16"), (3, 48, 40, 56, "f16"),
                                          (1, 128, 128, 256, "bf16"), (2, 33, 64, 72, "bf16")]):
        st = bf16 if dt == "bf16" else np.float16
        A = rt(rng.standard_normal((b, M, K)) / np.sqrt(K), st)
        B = rt(rng.standard_normal((b, K, N)) / np.sqrt(K), st)
        Y = np.asarray(tessera.ops.gemm(A, B), np.float32)  # f32 arrays holding 16-bit values
        region = fusion_core.MatmulRegion(dtype="bfloat16" if dt == "bf16" else "float16")
        Yr = np.stack([region.reference(A[j], B[j]) for j in range(b)])
        out[f"A{i}"], out[f"B{i}"], out[f"Y{i}"], out[f"Yregion{i}"] = A, B, Y, Yr
        out[f"dtype{i}"] = np.array(dt)
    out["n"] = np.array(4)
    # fused epilogue: ops.gemm(A, B, epilogue={...}) -> fused_epilogue (python/tessera/__init__.py:2658-2675)
    A = rt(rng.standard_normal((40, 64)) / 8, bf16)
    B = rt(rng.standard_normal((64, 72)), bf16)
    bias = rng.standard_normal(72).astype(np.float32)
    res = rt(rng.standard_normal((40, 72)), bf16)
    out.update(epiA=A, epiB=B, epi_bias=bias, epi_res=res)
    for act in ("linear", "relu", "gelu", "silu"):
        out[f"epi_{act}"] = np.asarray(
            tessera.ops.gemm(A, B, epilogue=dict(bias=bias, activation=act, residual=res)), np.float32)
    # region oracles behind the arbiter seam (fusion_core.py:672-727, 747-782)
    A = rt(rng.standard_normal((70, 64)) / 8, bf16)
    Wg = rt(rng.standard_normal((64, 136)), bf16)
    Wu = rt(rng.standard_normal((64, 136)), bf16)
    out.update(gatedA=A, gatedWg=Wg, gatedWu=Wu,
               gatedO=fusion_core.GatedMatmulRegion(gate_act="silu").reference(A, Wg, Wu))
    Q = rt(rng.standard_normal((96, 128)), bf16)
    K = rt(rng.standard_normal((96, 128)), bf16)
    V = rt(rng.standard_normal((96, 128)), bf16)
    sc = float(1.0 / np.sqrt(128.0))
    out.update(regQ=Q, regK=K, regV=V,
               regO=fusion_core.AttentionRegion(scale=sc, causal=False).reference(Q, K, V),
               regOc=fusion_core.AttentionRegion(scale=sc, causal=True).reference(Q, K, V))
    np.savez_compressed(os.path.join(HERE, "gemm.npz"), **out)


def attention():
    rng = np.random.default_rng(202)
    out = {}
    cases = [(1, 2, 2, 40, 40, 128, True), (2, 2, 2, 33, 70, 128, True), (1, 2, 2, 70, 33, 128, True),
             (1, 3, 3, 50, 50, 128, False), (2, 4, 2, 1, 97, 128, False), (1, 8, 2, 24, 24, 128, True)]
    for i, (B, Hq, Hkv, Sq, Sk, D, causal) in enumerate(cases):
        Q = rt(rng.standard_normal((B, Hq, Sq, D)), bf16)
        K = rt(rng.standard_normal((B, Hkv, Sk, D)), bf16)
        V = rt(rng.standard_normal((B, Hkv, Sk, D)), bf16)
        if Hq == Hkv:
            O = tessera.ops.flash_attn(Q, K, V, causal=causal)
        else:
            O = F.gqa_attention(Q, K, V, Hq, Hkv, causal=causal)
        out[f"Q{i}"], out[f"K{i}"], out[f"V{i}"] = Q, K, V
        out[f"O{i}"] = np.asarray(O, np.float32)
        out[f"meta{i}"] = np.array([B, Hq, Hkv, Sq, Sk, D, int(causal)])
    out["n"] = np.array(len(cases))
    # [B, S, H*D] operands: nn.functional.multi_head_attention and linear (nn/functional.py:33-44, 493-548)
    for i, (B, H, Sq, Sk, causal) in enumerate([(2, 2, 96, 96, True), (1, 3, 40, 130, False), (2, 2, 1, 77, False)]):
        Q = rt(rng.standard_normal((B, Sq, H * 128)), bf16)
        K = rt(rng.standard_normal((B, Sk, H * 128)), bf16)
        V = rt(rng.standard_normal((B, Sk, H * 128)), bf16)
        out[f"mhaQ{i}"], out[f"mhaK{i}"], out[f"mhaV{i}"] = Q, K, V
        out[f"mhaO{i}"] = np.asarray(F.multi_head_attention(Q, K, V, H, causal=causal), np.float32)
        out[f"mhameta{i}"] = np.array([B, H, Sq, Sk, int(causal)])
    out["mha_n"] = np.array(3)
    x = rt(rng.standard_normal((2, 24, 64)) / 8, bf16)
    W = rt(rng.standard_normal((64, 48)), bf16)
    b = rng.standard_normal(48).astype(np.float32)
    out.update(lin_x=x, lin_W=W, lin_b=b, lin_y=np.asarray(F.linear(x, W, b), np.float32))
    # the CUDA lane's contract (bias, top-left causal, window, soft-cap, D != Dv), from the numpy
    # reference inside the reference's own device test (tests/device/nvidia/test_flash_attention.py:23-58)
    import importlib.util
    spec = importlib.util.spec_from_file_location(
        "ref_test_flash", os.path.join(REF, "tests", "device", "nvidia", "test_flash_attention.py"))
    ref_test = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref_test)
    lane = [  # B, Hq, Hkv, Sq, Sk, D, Dv, kwargs, with_bias
        (2, 4, 4, 5, 7, 8, 6, dict(scale=1 / np.sqrt(8.0)), False),
        (2, 4, 2, 5, 7, 8, 6, dict(scale=1 / np.sqrt(8.0)), False),
        (2, 4, 1, 5, 7, 8, 6, dict(scale=1 / np.sqrt(8.0)), False),
        (1, 4, 2, 6, 8, 8, 8, dict(scale=0.35, causal=True, window=(3, 1), softcap=1.7), True),
        (1, 2, 1, 70, 45, 40, 72, dict(scale=0.2, causal=True), False),
        (1, 2, 2, 33, 100, 64, 64, dict(scale=0.125, window=(10, 0)), True),
        (1, 1, 1, 9, 9, 16, 16, dict(scale=0.3, causal=True, window=(0, 0)), False),
    ]
    for i, (B, Hq, Hkv, Sq, Sk, D, Dv, kw, wb) in enumerate(lane):
        q = rng.standard_normal((B, Hq, Sq, D), dtype=np.float32)
        k = rng.standard_normal((B, Hkv, Sk, D), dtype=np.float32)
        v = rng.standard_normal((B, Hkv, Sk, Dv), dtype=np.float32)
        bias = (rng.standard_normal((B, Hq, Sq, Sk)) * 0.2).astype(np.float32) if wb else None
        out[f"laneq{i}"], out[f"lanek{i}"], out[f"lanev{i}"] = q, k, v
        if wb:
            out[f"laneb{i}"] = bias
        out[f"laneo{i}"] = ref_test._reference(q, k, v, bias=bias, **kw).astype(np.float32)
        out[f"lanekw{i}"] = np.array([kw.get("scale"), float(kw.get("causal", False)),
                                      -1 if "window" not in kw else kw["window"][0],
                                      -1 if "window" not in kw else kw["window"][1],
                                      kw.get("softcap", 0.0)], np.float64)
    out["lane_n"] = np.array(len(lane))
    # ops.flash_attn with attn_bias (added before the bottom-right causal mask, __init__.py:1340-1350)
    Q = rt(rng.standard_normal((2, 2, 20, 32)), bf16)
    K = rt(rng.standard_normal((2, 2, 50, 32)), bf16)
    V = rt(rng.standard_normal((2, 2, 50, 32)), bf16)
    ab = (rng.standard_normal((2, 1, 20, 50)) * 0.5).astype(np.float32)
    out.update(biasQ=Q, biasK=K, biasV=V, biasB=ab,
               biasO=np.asarray(tessera.ops.flash_attn(Q, K, V, causal=True, attn_bias=ab), np.float32))
    # split-KV merge states
    oa, ob = rng.standard_normal((2, 5, 16)).astype(np.float32)
    ma, mb = rng.standard_normal((2, 5)).astype(np.float32)
    la, lb = (rng.random((2, 5)) + 0.5).astype(np.float32)
    o, m, l = softmax_merge(oa, ma, la, ob, mb, lb)
    out.update(merge_oa=oa, merge_ob=ob, merge_ma=ma, merge_mb=mb, merge_la=la, merge_lb=lb,
               merge_o=o, merge_m=m, merge_l=l, merge_final=softmax_finalize(o, l))
    np.savez_compressed(os.path.join(HERE, "attention.npz"), **out)


def attention_backward():
    """(dQ, dK, dV) from the numpy reference inside the reference's own device test of the CUDA
    backward lane (tests/device/nvidia/test_flash_attention_backward.py:23-50), on that test's
    shapes and seeds plus larger ones."""
    import importlib.util
    spec = importlib.util.spec_from_file_location(
        "ref_test_flash_bwd", os.path.join(REF, "tests", "device", "nvidia", "test_flash_attention_backward.py"))
    ref_test = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref_test)
    out = {}
    cases = [  # seed, q shape, (Hkv, Sk), Dv, kwargs, with_bias
        (913, (1, 4, 4, 4), (2, 5), 3, dict(scale=.5), False),
        (912, (1, 4, 4, 4), (1, 5), 3, dict(scale=.5), False),
        (919, (1, 2, 5, 4), (1, 6), 3, dict(scale=.5, causal=True, window=(2, 1), softcap=1.4), True),
        (929, (1, 4, 7, 8), (2, 9), 6, dict(scale=8 ** -0.5, causal=True), False),
        (1001, (2, 4, 40, 40), (2, 70), 24, dict(scale=0.15, causal=True), False),
        (1002, (1, 2, 33, 128), (1, 50), 128, dict(scale=128 ** -0.5, window=(10, 5)), True),
        (1003, (1, 2, 12, 8), (2, 7), 8, dict(scale=0.3, window=(20, 3), softcap=2.0), False),
        (1004, (1, 3, 65, 16), (3, 65), 16, dict(scale=0.25, causal=True), False),
    ]
    for i, (seed, qs, (Hkv, Sk), Dv, kw, wb) in enumerate(cases):
        rng = np.random.default_rng(seed)
        B, Hq, Sq, D = qs
        q = rng.standard_normal(qs, dtype=np.float32)
        k = rng.standard_normal((B, Hkv, Sk, D), dtype=np.float32)
        v = rng.standard_normal((B, Hkv, Sk, Dv), dtype=np.float32)
        do = rng.standard_normal((B, Hq, Sq, Dv), dtype=np.float32)
        bias = (rng.standard_normal((B, Hq, Sq, Sk)) * .1).astype(np.float32) if wb else None
        dq, dk, dv = ref_test._ref(do, q, k, v, bias=bias, **kw)
        out[f"q{i}"], out[f"k{i}"], out[f"v{i}"], out[f"do{i}"] = q, k, v, do
        if wb:
            out[f"b{i}"] = bias
        out[f"dq{i}"], out[f"dk{i}"], out[f"dv{i}"] = (np.asarray(g, np.float32) for g in (dq, dk, dv))
        out[f"kw{i}"] = np.array([kw["scale"], float(kw.get("causal", False)),
                                  -1 if "window" not in kw else kw["window"][0],
                                  -1 if "window" not in kw else kw["window"][1],
                                  kw.get("softcap", 0.0)], np.float64)
    out["n"] = np.array(len(cases))
    np.savez_compressed(os.path.join(HERE, "attention_bwd.npz"), **out)


def moe():
    rng = np.random.default_rng(303)
    out = {}
    # routing + permutation, with and without capacity
    cases = [(64, 8, 2, None), (100, 8, 2, 20), (37, 4, 1, 6), (50, 16, 4, None)]
    for i, (T, E, k, cap) in enumerate(cases):
        logits = rng.standard_normal((T, E)).astype(np.float32)
        cfg = dmoe.MoEConfig(num_experts=E, top_k=k, capacity_factor=1e9)
        r = dmoe.route_tokens(logits, cfg, capacity=cap if cap is not None else T * k + 1)
        # the transport descriptor is built from the un-dropped routing plus the same capacity
        r0 = dmoe.route_tokens(logits, cfg, capacity=T * k + 1)
        plan = smoe.plan_dispatch(r0.assignment, r0.weights, E, capacity=cap)
        desc = descriptor_from_dispatch_plan(plan)
        out[f"logits{i}"] = logits
        out[f"meta{i}"] = np.array([T, E, k, -1 if cap is None else cap])
        out[f"assignment{i}"], out[f"weights{i}"] = r.assignment, r.weights
        out[f"load{i}"], out[f"overflow{i}"] = r.load, np.array(r.overflow)
        out[f"token_of_slot{i}"], out[f"expert_of_slot{i}"] = desc.token_of_slot, desc.expert_of_slot
        out[f"combine_weights{i}"] = desc.combine_weights
        out[f"group_sizes{i}"], out[f"group_offsets{i}"] = desc.group_sizes, desc.group_offsets
    out["n_route"] = np.array(len(cases))
    # grouped GEMM / SwiGLU block / full layer / expert-parallel layer
    T, H, Fdim, E, k = 48, 32, 64, 4, 2
    x = rt(rng.standard_normal((T, H)), bf16)
    Wr = rt(rng.standard_normal((H, E)) / np.sqrt(H), bf16)
    Wg = rt(rng.standard_normal((E, H, Fdim)) / np.sqrt(H), bf16)
    Wu = rt(rng.standard_normal((E, H, Fdim)) / np.sqrt(H), bf16)
    Wd = rt(rng.standard_normal((E, Fdim, H)) / np.sqrt(Fdim), bf16)
    gs = np.array([10, 0, 25, 13], np.int64)
    out.update(x=x, Wr=Wr, Wg=Wg, Wu=Wu, Wd=Wd, gs=gs)
    out["grouped_gemm"] = np.asarray(tessera.ops.grouped_gemm(x, Wg, gs), np.float32)
    out["swiglu_block"] = np.asarray(tessera.ops.moe_swiglu_block(x, Wg, Wu, Wd, gs), np.float32)
    out["moe_layer_k1"] = np.asarray(F.moe_layer(x, Wr, Wg, Wu, Wd, top_k=1), np.float32)
    out["moe_layer_k2"] = np.asarray(F.moe_layer(x, Wr, Wg, Wu, Wd, top_k=2), np.float32)
    cfg = dmoe.MoEConfig(num_experts=E, top_k=k, capacity_factor=1e9)
    for R in (2, 4):
        y, dropped = dmoe.megamoe_layer(x, Wr, Wg, Wu, Wd, world_size=R, config=cfg,
                                        capacity=T * k)
        out[f"megamoe_w{R}"] = np.asarray(y, np.float32)
        out[f"megamoe_dropped_w{R}"] = np.array(dropped)
    # quantised grouped GEMM (quant="fp8_e4m3"): per-tensor x, per-expert w (__init__.py:337-351, 3340-3374)
    sizes = np.array([40, 0, 100, 52])
    xq = rt(rng.standard_normal((192, 64)), bf16)
    wgq = rt(rng.standard_normal((4, 64, 96)) / 8, bf16)
    wuq = rt(rng.standard_normal((4, 64, 96)) / 8, bf16)
    wdq = rt(rng.standard_normal((4, 96, 48)) / 10, bf16)
    dq, sc = tessera.ops.quantize_fp8(xq)
    out.update(q_sizes=sizes, q_x=xq, q_wg=wgq, q_wu=wuq, q_wd=wdq, q_x_dq=np.asarray(dq, np.float32),
               q_x_scale=np.float32(sc),
               q_gg=np.asarray(tessera.ops.grouped_gemm(xq, wgq, sizes, quant="fp8_e4m3"), np.float32),
               q_block=np.asarray(tessera.ops.moe_swiglu_block(xq, wgq, wuq, wdq, sizes, quant="fp8_e4m3"),
                                  np.float32))
    np.savez_compressed(os.path.join(HERE, "moe.npz"), **out)


def quant4():
    """NVFP4 quantisation and the grouped GEMMs with quant="nvfp4" / "fp8xfp4", from the reference's
    own ops (python/tessera/__init__.py:291-351, 592-616, 3472-3500)."""
    import tessera
    rng = np.random.default_rng(4242)
    out = {}
    x = (rng.standard_normal((37, 64)) * np.exp(rng.standard_normal((37, 1)))).astype(np.float32)
    x[3, 16:32] = 0.0                      # an all-zero block
    x[5, :16] *= 1e-4                      # a block whose scale rounds to zero in e4m3
    x[7, 5] = 0.75 * 6 / 6 ; x[7, 0] = 6.0  # a tie on the e2m1 grid under scale 1
    dq, sc = tessera.ops.quantize_nvfp4(x)
    out.update(n_x=x, n_dq=np.asarray(dq, np.float32), n_scales=np.asarray(sc, np.float32))
    T, K, N, F, E = 96, 64, 48, 80, 3
    sizes = np.array([40, 0, 56])
    xs = rt(rng.standard_normal((T, K)), bf16)
    w = rt(rng.standard_normal((E, K, N)) / 8, bf16)
    wg = rt(rng.standard_normal((E, K, F)) / 8, bf16)
    wu = rt(rng.standard_normal((E, K, F)) / 8, bf16)
    wd = rt(rng.standard_normal((E, F, N)) / 9, bf16)
    out.update(g_x=xs, g_w=w, g_wg=wg, g_wu=wu, g_wd=wd, g_sizes=sizes)
    dq5, sc5 = tessera.ops.quantize_fp8(x, format="e5m2")
    out.update(e5_dq=np.asarray(dq5, np.float32), e5_scale=np.float32(sc5))
    for q in ("nvfp4", "fp8xfp4", "fp8_e5m2", "fp8_e5m2xnvfp4"):
        out[f"gg_{q}"] = np.asarray(tessera.ops.grouped_gemm(xs, w, sizes, quant=q), np.float32)
        out[f"blk_{q}"] = np.asarray(tessera.ops.moe_swiglu_block(xs, wg, wu, wd, sizes, quant=q), np.float32)
    np.savez_compressed(os.path.join(HERE, "quant4.npz"), **out)


def paged():
    """cache.paged_attention over a KVCacheHandle, and the page ABI it is materialised into
    (python/tessera/cache/paged_kv.py:421-559)."""
    from tessera.cache import KVCacheHandle, paged_attention
    from tessera.cache.paged_kv import PagedKVBufferABI, materialize_paged_kv_abi
    rng = np.random.default_rng(404)
    out = {}
    cases = [  # Hq, Hkv, q_len, n, page_size, causal, token_indices
        (4, 4, 1, 200, 16, False, None),
        (8, 2, 3, 150, 8, True, None),
        (8, 2, 2, 97, 32, False, None),
        (16, 2, 1, 333, 64, False, None),
        (4, 2, 4, 130, 16, True, "subset"),
        (4, 4, 5, 3, 8, True, None),
    ]
    for i, (Hq, Hkv, q_len, n, L, causal, ti) in enumerate(cases):
        h = KVCacheHandle(num_heads=Hkv, head_dim=128, max_seq=n + 8, page_size=L)
        k = rt(rng.standard_normal((n, Hkv, 128)), bf16)
        v = rt(rng.standard_normal((n, Hkv, 128)), bf16)
        h.append(k, v)
        Q = rt(rng.standard_normal((Hq, q_len, 128)), bf16)
        idx = None
        if ti == "subset":
            idx = rng.permutation(n)[: n // 2].astype(np.int64)
        o = paged_attention(Q, h, causal=causal, token_indices=None if idx is None else idx.tolist())
        abi = materialize_paged_kv_abi(h)
        out.update({f"Q{i}": Q, f"k{i}": k, f"v{i}": v, f"O{i}": np.asarray(o, np.float32),
                    f"meta{i}": np.array([Hq, Hkv, q_len, n, L, int(causal)]),
                    f"kpages{i}": abi.k_pages, f"table{i}": abi.page_table})
        if idx is not None:
            out[f"idx{i}"] = idx
    # a scattered table: the same tokens behind a permuted physical placement
    n, Hkv, L = 75, 2, 16
    k = rt(rng.standard_normal((n, Hkv, 128)), bf16)
    v = rt(rng.standard_normal((n, Hkv, 128)), bf16)
    pages = (n + L - 1) // L
    table = rng.permutation(pages + 3)[:pages].astype(np.int32)
    kp = np.zeros((pages + 3, L, Hkv, 128), np.float32)
    vp = np.zeros_like(kp)
    for t in range(n):
        kp[table[t // L], t % L] = k[t]
        vp[table[t // L], t % L] = v[t]
    abi = PagedKVBufferABI(kp, vp, table, n)

    class _State:  # a backend-native state: exposes only its own page ABI
        def paged_kv_abi(self):
            return abi
    gidx = rng.integers(0, n, 40)
    gk, gv = abi.gather(gidx)
    out.update(sk_pages=kp, sv_pages=vp, stable=table, sn=np.array(n), sgidx=gidx, sgk=gk, sgv=gv)
    Q = rt(rng.standard_normal((4, 2, 128)), bf16)
    kk, vv = abi.gather(np.arange(n))
    from tessera.cache.paged_kv import _reference_attention
    out.update(sQ=Q, sO=_reference_attention(Q, np.transpose(kk, (1, 0, 2)), np.transpose(vv, (1, 0, 2)),
                                             1.0 / np.sqrt(128.0), False).astype(np.float32))
    out["n"] = np.array(len(cases))
    # an int8 cache: KVCacheHandle(quantize_bits=8) quantises per token on append and dequantises on
    # read (python/tessera/cache/handle.py:72-215, python/tessera/__init__.py:3196-3265)
    n, Hkv, Hq = 140, 2, 8
    h8 = KVCacheHandle(num_heads=Hkv, head_dim=128, max_seq=n + 8, page_size=16, quantize_bits=8)
    k = rt(rng.standard_normal((n, Hkv, 128)) * np.linspace(0.2, 3.0, n)[:, None, None], bf16)
    v = rt(rng.standard_normal((n, Hkv, 128)), bf16)
    h8.append(k, v)
    Q = rt(rng.standard_normal((Hq, 1, 128)), bf16)
    kq, vq, sc, _ = tessera.ops.quantize_kv(k, v, bits=8)
    out.update(q8_k=k, q8_v=v, q8_Q=Q, q8_kq=kq, q8_vq=vq, q8_scale=np.asarray(sc, np.float32),
               q8_O=np.asarray(paged_attention(Q, h8), np.float32))
    np.savez_compressed(os.path.join(HERE, "paged.npz"), **out)


if __name__ == "__main__":
    # no arguments: every fixture; otherwise only the named generators (each owns one .npz)
    every = {"gemm": gemm, "attention": attention, "attention_backward": attention_backward, "moe": moe, "quant4": quant4,
             "paged": paged}
    for name in (sys.argv[1:] or list(every)):
        every[name]()
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))
