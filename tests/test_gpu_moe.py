"""MoE parity on the GPU: bit-exact routing and permutation, grouped GEMMs, whole layer.
Cases follow tests/unit/test_moe_layer.py, tests/device/nvidia/test_moe_transport.py (empty
group, dispatch bit-equality) and tests/unit/test_nvidia_moe_transport_contract.py (int32 ABI)."""
import os

import numpy as np
import pytest

from oracle import tessera_oracle as orc
from tests.gpu_util import TOL, no_device_error, rel_err

pytestmark = pytest.mark.gpu

from tessera_b200 import _lib, device  # noqa: E402
from tessera_b200.device import DeviceArray as DA, bfloat16  # noqa: E402


def _route_permute(logits, k, cap):
    T, E = logits.shape
    S = T * k
    dl = DA.from_host(logits)
    da, dw = DA.zeros((T, k), np.int32), DA.zeros((T, k), np.float32)
    _lib.call("tessera_sm100_moe_route_device", dl.ptr, T, E, k, 1, da.ptr, dw.ptr, None)
    tok, exp_, wos = DA.zeros((S,), np.int32), DA.zeros((S,), np.int32), DA.zeros((S,), np.float32)
    gs, go, so = DA.zeros((E,), np.int32), DA.zeros((E + 1,), np.int32), DA.zeros((S,), np.int32)
    _lib.call("tessera_sm100_moe_permute_device", da.ptr, dw.ptr, T, k, E, cap, tok.ptr, exp_.ptr,
              wos.ptr, gs.ptr, go.ptr, so.ptr, None)
    return dict(assignment=da.download(), weights=dw.download(), token_of_slot=tok.download(),
                expert_of_slot=exp_.download(), weight_of_slot=wos.download(), group_sizes=gs.download(),
                group_offsets=go.download(), slot_of=so.download().reshape(T, k))


@pytest.mark.parametrize("T,E,k,cap", [(257, 8, 2, -1), (1000, 8, 2, 200), (513, 16, 4, -1),
                                       (64, 4, 1, 10), (8192, 8, 2, -1), (3000, 64, 8, 300),
                                       (1, 8, 2, -1), (5000, 256, 2, -1)])
def test_routing_and_permutation_bit_exact(T, E, k, cap):
    logits = np.random.default_rng(T + E).standard_normal((T, E), dtype=np.float32)
    got = _route_permute(logits, k, cap)
    r = orc.route_tokens(logits, k, True, None if cap < 0 else cap)
    p = orc.moe_permutation(r.assignment, r.weights, E)
    kept = int(p.group_offsets[-1])
    np.testing.assert_array_equal(got["assignment"], r.assignment)
    np.testing.assert_array_equal(got["token_of_slot"][:kept], p.token_of_slot)
    np.testing.assert_array_equal(got["expert_of_slot"][:kept], p.expert_of_slot)
    np.testing.assert_array_equal(got["group_sizes"], p.group_sizes)
    np.testing.assert_array_equal(got["group_offsets"], p.group_offsets)
    np.testing.assert_array_equal(got["slot_of"], p.slot_of_assignment)
    assert np.abs(got["weights"] - r.weights).max() <= 1e-6
    assert np.abs(got["weight_of_slot"][:kept] - p.weight_of_slot).max() <= 1e-6
    assert np.all(np.diff(got["expert_of_slot"][:kept]) >= 0)  # non-decreasing expert ids


def test_routing_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "moe.npz"))
    for i in range(int(g["n_route"])):
        T, E, k, cap = (int(v) for v in g[f"meta{i}"])
        got = _route_permute(np.ascontiguousarray(g[f"logits{i}"]), k, cap)
        kept = int(g[f"group_offsets{i}"][-1])
        np.testing.assert_array_equal(got["assignment"], g[f"assignment{i}"])
        np.testing.assert_array_equal(got["token_of_slot"][:kept], g[f"token_of_slot{i}"])
        np.testing.assert_array_equal(got["expert_of_slot"][:kept], g[f"expert_of_slot{i}"])
        np.testing.assert_array_equal(got["group_sizes"], g[f"group_sizes{i}"])
        np.testing.assert_array_equal(got["group_offsets"], g[f"group_offsets{i}"])


@pytest.mark.parametrize("sizes,K,N", [([100, 0, 129, 33, 127], 192, 128), ([256, 128], 64, 256),
                                       ([5, 300, 1, 0, 0, 700], 136, 520), ([0, 0, 7], 8, 8),
                                       # large enough for the CTA-pair kernel: ragged tails in both CTAs
                                       # of a pair, an empty group, a group smaller than one CTA's rows
                                       ([300, 0, 777, 100, 871], 136, 2568), ([256, 512, 1280], 64, 2560)])
def test_grouped_gemm_and_swiglu(sizes, K, N):
    import tessera_b200 as tessera
    rng = np.random.default_rng(len(sizes) + K)
    sizes = np.array(sizes)
    T, E = int(sizes.sum()), len(sizes)
    x = rng.standard_normal((T, K), dtype=np.float32).astype(bfloat16)
    w = (rng.standard_normal((E, K, N), dtype=np.float32) / np.sqrt(K)).astype(bfloat16)
    w2 = (rng.standard_normal((E, K, N), dtype=np.float32) / np.sqrt(K)).astype(bfloat16)
    wd = (rng.standard_normal((E, N, K), dtype=np.float32) / np.sqrt(N)).astype(bfloat16)
    assert rel_err(tessera.ops.grouped_gemm(x, w, sizes, out_dtype=np.float32),
                   orc.grouped_gemm(x, w, sizes)) < 1e-4
    got = tessera.ops.grouped_gemm(x, w, sizes)
    assert got.dtype == bfloat16 and rel_err(got, orc.grouped_gemm(x, w, sizes)) < TOL
    assert rel_err(tessera.ops.moe_swiglu_block(x, w, w2, wd, sizes),
                   orc.moe_swiglu_block(x, w, w2, wd, sizes)) < TOL
    a = rng.standard_normal((T, N), dtype=np.float32)
    b = rng.standard_normal((T, N), dtype=np.float32)
    np.testing.assert_allclose(tessera.ops.silu_mul(a, b), orc.silu_mul(a, b), rtol=1e-5, atol=1e-6)
    no_device_error()


def test_dispatch_is_bit_exact_and_combine_matches():
    rng = np.random.default_rng(2)
    T, H, k, E = 257, 192, 2, 5
    x = rng.standard_normal((T, H), dtype=np.float32).astype(bfloat16)
    r = orc.route_tokens(rng.standard_normal((T, E), dtype=np.float32), k)
    p = orc.moe_permutation(r.assignment, r.weights, E)
    S = len(p.token_of_slot)
    dx, dtok = DA.from_host(x), DA.from_host(p.token_of_slot)
    dxp = DA.zeros((S, H), bfloat16)
    _lib.call("tessera_sm100_moe_dispatch_device", dx.ptr, dtok.ptr, dxp.ptr, T, S, H, _lib.BF16, None)
    xp = dxp.download()
    np.testing.assert_array_equal(xp.view(np.uint16), x[p.token_of_slot].view(np.uint16))
    y = rng.standard_normal((S, H), dtype=np.float32)
    dy, dso, dw = DA.from_host(y), DA.from_host(p.slot_of_assignment), DA.from_host(r.weights)
    dout = DA.zeros((T, H), np.float32)
    _lib.call("tessera_sm100_moe_combine_device", dy.ptr, dso.ptr, dw.ptr, dout.ptr, T, k, H, _lib.F32,
              _lib.F32, None)
    ref = np.zeros((T, H), np.float32)
    np.add.at(ref, p.token_of_slot, y * p.weight_of_slot[:, None])
    np.testing.assert_allclose(dout.download(), ref, rtol=1e-5, atol=1e-6)
    dsc = DA.zeros((T, H), np.float32)
    dwos = DA.from_host(p.weight_of_slot)
    _lib.call("tessera_sm100_moe_combine_scatter_f32_device", dy.ptr, dtok.ptr, dwos.ptr, dsc.ptr, T, S, H, None)
    np.testing.assert_allclose(dsc.download(), ref, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("top_k", [1, 2, 4])
def test_moe_layer_small(top_k):
    import tessera_b200 as tessera
    rng = np.random.default_rng(top_k)
    T, H, F, E = 512, 256, 512, 8
    x = rng.standard_normal((T, H), dtype=np.float32).astype(bfloat16)
    logits = rng.standard_normal((T, E), dtype=np.float32)
    wg = (rng.standard_normal((E, H, F), dtype=np.float32) / np.sqrt(H)).astype(bfloat16)
    wu = (rng.standard_normal((E, H, F), dtype=np.float32) / np.sqrt(H)).astype(bfloat16)
    wd = (rng.standard_normal((E, F, H), dtype=np.float32) / np.sqrt(F)).astype(bfloat16)
    out, routing = tessera.ops.moe_layer_from_logits(x, logits, wg, wu, wd, top_k=top_k,
                                                      out_dtype=np.float32, return_routing=True)
    ref, r, p = orc.moe_layer_from_logits(x, logits, wg, wu, wd, top_k)
    np.testing.assert_array_equal(routing["assignment"], r.assignment)
    np.testing.assert_array_equal(routing["group_sizes"], p.group_sizes)
    np.testing.assert_array_equal(routing["token_of_slot"], p.token_of_slot)
    assert rel_err(out, ref) < TOL
    # capacity drops follow the reference's token-major rule
    out_c, routing_c = tessera.ops.moe_layer_from_logits(x, logits, wg, wu, wd, top_k=top_k, capacity=40,
                                                          out_dtype=np.float32, return_routing=True)
    ref_c, r_c, _ = orc.moe_layer_from_logits(x, logits, wg, wu, wd, top_k, capacity=40)
    np.testing.assert_array_equal(routing_c["assignment"], r_c.assignment)
    assert rel_err(out_c, ref_c) < TOL


def test_moe_layer_golden(golden_dir):
    import tessera_b200 as tessera
    g = np.load(os.path.join(golden_dir, "moe.npz"))
    x, Wr, Wg, Wu, Wd = (g[k].astype(bfloat16) for k in ("x", "Wr", "Wg", "Wu", "Wd"))
    for k in (1, 2):
        got = tessera.nn.functional.moe_layer(x, Wr, Wg, Wu, Wd, top_k=k)
        assert rel_err(got, g[f"moe_layer_k{k}"]) < TOL
    assert rel_err(tessera.ops.moe_swiglu_block(x, Wg, Wu, Wd, g["gs"]), g["swiglu_block"]) < TOL


def test_config5_full_size():
    """8192 tokens, hidden 4096, FFN 14336, 8 experts, top-2: routing and permutation bit-exact
    against the oracle over all tokens; outputs of sampled tokens against a per-token fp32
    reference; group sizes equal the reference's known answer for the seed."""
    import tessera_b200 as tessera
    inp = orc.make_inputs("moe")
    x, logits, wg, wu, wd = inp["x"], inp["logits"], inp["w_gate"], inp["w_up"], inp["w_down"]
    out, routing = tessera.ops.moe_layer_from_logits(x, logits, wg, wu, wd, top_k=2,
                                                      out_dtype=np.float32, return_routing=True)
    r = orc.route_tokens(logits, 2)
    p = orc.moe_permutation(r.assignment, r.weights, 8)
    np.testing.assert_array_equal(routing["assignment"], r.assignment)
    np.testing.assert_array_equal(routing["token_of_slot"], p.token_of_slot)
    assert routing["group_sizes"].tolist() == [1994, 2066, 2065, 2092, 2074, 2036, 1965, 2092]
    assert np.abs(routing["weights"] - r.weights).max() <= 1e-6
    toks = [0, 1, 777, 4095, 8191, 5000]
    xf = x.astype(np.float32)
    ref = np.zeros((len(toks), x.shape[1]), np.float32)
    for i, t in enumerate(toks):
        for j in range(2):
            e = int(r.assignment[t, j])
            h = orc.silu_mul(xf[t] @ wg[e].astype(np.float32), xf[t] @ wu[e].astype(np.float32))
            ref[i] += r.weights[t, j] * (h @ wd[e].astype(np.float32))
    assert rel_err(out[toks], ref) < TOL
    assert not np.isnan(out).any()


def test_device_side_expert_parallel_exchange_on_one_rank():
    """The flag-ordered dispatch/combine kernels with a world of one (own buffers stand in for the
    peers'): the fused route + sort reproduces the reference's routing bit for bit, and the result
    equals the single-device layer, three times in a row (buffers and flags are reused, the epoch
    moves on)."""
    from types import SimpleNamespace
    from tessera_b200 import parallel
    rng = np.random.default_rng(31)
    T, H, F, E, k = 300, 128, 256, 8, 2
    x = rng.standard_normal((T, H), dtype=np.float32).astype(bfloat16)
    logits = rng.standard_normal((T, E), dtype=np.float32)
    wg = (rng.standard_normal((E, H, F), dtype=np.float32) / 11).astype(bfloat16)
    wu = (rng.standard_normal((E, H, F), dtype=np.float32) / 11).astype(bfloat16)
    wd = (rng.standard_normal((E, F, H), dtype=np.float32) / 16).astype(bfloat16)
    moe = parallel.DeviceExpertParallelMoE(SimpleNamespace(world=1, rank=0), lambda h: [h], DA.from_host(wg),
                                           DA.from_host(wu), DA.from_host(wd), T, k, E, wait_limit_ms=2000)
    dx, dl = DA.from_host(x), DA.from_host(logits)
    ref, routing, perm = orc.moe_layer_from_logits(x, logits, wg, wu, wd, k)
    for _ in range(3):
        y = moe.forward(dx, dl)
        device.synchronize()
        assert rel_err(y.download(), ref) < TOL
    assert moe.epoch == 3
    np.testing.assert_array_equal(moe.assignment.download(), routing.assignment.astype(np.int32))
    np.testing.assert_array_equal(moe.token_of_slot.download(), perm.token_of_slot)
    np.testing.assert_array_equal(moe.expert_of_slot.download(), perm.expert_of_slot)
    np.testing.assert_array_equal(moe.group_sizes.download(), perm.group_sizes)
    np.testing.assert_array_equal(moe.local_offsets.download(), perm.group_offsets)
    np.testing.assert_allclose(moe.weights.download(), routing.weights, rtol=0, atol=1e-6)
    no_device_error()
    moe.close()
