"""Host-side logic that needs no GPU: the distributed API, artifact plumbing, launch() failure
statuses and argument validation. Mirrors the reference's tests/unit/test_distributed_api.py
(fan-out :418-478) and test_runtime_launch_first_failing_gate.py."""
import numpy as np
import pytest

import tessera_b200 as tessera
from tessera_b200 import runtime as rt
from tessera_b200.distributed import Block, Cyclic, DistributedArray, MeshSpec, Rect, Replicated, ShardSpec


def test_mesh_and_shard_spec():
    mesh = MeshSpec({"dp": 4, "tp": 8})
    assert mesh.total_ranks == 32 and mesh.axis_size("tp") == 8
    with pytest.raises(KeyError):
        mesh.axis_size("pp")
    with pytest.raises(ValueError):
        MeshSpec({})
    spec = ShardSpec(partition=(1,), mesh_axes=("tp",))
    assert spec.shard_size(1, 8192, mesh) == 1024 and spec.shard_size(0, 8192, mesh) == 8192
    with pytest.raises(ValueError):
        spec.shard_size(1, 100, mesh)
    with pytest.raises(ValueError):
        ShardSpec(partition=(0, 1), mesh_axes=("tp",))
    assert ShardSpec.replicate().replicated


def test_block_maps_mesh_axis_i_to_dim_i():
    d = Rect((4, 128, 64))
    spec = Block(mesh_axes=("dp", "tp")).make_shard_spec(d)
    assert spec.partition == (0, 1) and spec.mesh_axes == ("dp", "tp")
    assert Replicated().make_shard_spec(d).replicated
    assert Cyclic(("dp",)).make_shard_spec(d).cyclic
    with pytest.raises(ValueError):
        Rect(())


def test_parts_needs_a_bound_mesh_and_returns_views():
    X = tessera.array.from_domain(Rect((8, 16)), "fp32", Block(("dp",)))
    with pytest.raises(ValueError):
        X.parts("dp")
    X._bind_mesh(MeshSpec({"dp": 4}))
    shards = X.parts("dp")
    assert len(shards) == 4 and shards[0].shape == (2, 16)
    shards[1]._data[:] = 7.0          # a block shard is a view of the parent
    assert (X.numpy()[2:4] == 7.0).all() and (X.numpy()[:2] == 0).all()
    with pytest.raises(ValueError):
        X.parts("tp")
    rep = tessera.array.from_domain(Rect((8, 16)), "fp32", Replicated())
    assert rep.parts("dp") == [rep]


def test_column_split_with_explicit_shard_spec_and_setitem():
    W = DistributedArray(np.arange(24, dtype=np.float32).reshape(4, 6), "fp32",
                         ShardSpec(partition=(1,), mesh_axes=("tp",)))
    W._bind_mesh(MeshSpec({"tp": 3}))
    cols = W.parts("tp")
    assert [c.shape for c in cols] == [(4, 2)] * 3
    cols[2][:] = np.zeros((4, 2))
    assert (W[:, 4:] == 0).all() and W[0, 0] == 0 and W[0, 1] == 1


def test_index_launch_fans_out_lists_and_broadcasts_scalars():
    calls = []

    @tessera.kernel
    def k(a, b, c, s):
        calls.append(s)
        c[:] = a @ b * s

    A = [np.full((2, 3), r + 1.0) for r in range(4)]
    B = [np.ones((3, 2)) for _ in range(4)]
    C = np.zeros((8, 2))
    outs = tessera.index_launch(axis="tp")(k)(A, B, np.array_split(C, 4, axis=0), 2.0)
    assert outs == [None] * 4 and calls == [2.0] * 4
    for r in range(4):
        assert (C[2 * r:2 * r + 2] == 6.0 * (r + 1)).all()
    with pytest.raises(ValueError):
        tessera.index_launch(axis="tp")(k)(A, B[:3], np.array_split(C, 4), 1.0)
    with pytest.raises(ValueError):
        tessera.index_launch(axis="tp")(k)(1, 2, 3, 4)


def test_artifact_roundtrip_and_hash():
    art = rt.make_artifact("tessera.matmul", ["a", "b"])
    assert art.metadata["target"] == "nvidia_sm100" and art.metadata["compiler_path"] == "sm100_gemm"
    again = rt.RuntimeArtifact.from_json(art.to_json())
    assert again.artifact_hash == art.artifact_hash
    bad = art.to_dict()
    bad["artifact_hash"] = "0" * 64
    with pytest.raises(ValueError):
        rt.RuntimeArtifact.from_dict(bad)
    with pytest.raises(ValueError):
        rt.make_artifact("tessera.conv2d", ["x"])


def test_target_aliases():
    for name in ("sm100", "sm_100", "sm100a", "sm_100a", "blackwell", "nvidia_sm100"):
        assert rt.normalize_target(name) == "nvidia_sm100"
    assert rt.normalize_target("cuda") == "cuda"  # an alias of sm_90 in the reference, not ours
    assert rt.normalize_target(None) == "cpu"


def test_launch_reports_structured_failures_and_never_raises():
    other = rt.RuntimeArtifact(metadata={"target": "nvidia_sm120", "compiler_path": "nvidia_mma",
                                         "executable": True})
    res = rt.launch(other, ())
    assert res["ok"] is False and res["runtime_status"] in ("missing_backend", "unimplemented")
    assert res["first_failing_gate"] == "runtime_abi"
    no_row = rt.RuntimeArtifact(metadata={"target": "nvidia_sm100", "compiler_path": "nope",
                                          "executable": True})
    assert rt.launch(no_row, ())["runtime_status"] == "unimplemented"
    not_exec = rt.RuntimeArtifact(metadata={"target": "sm_100a", "compiler_path": "sm100_gemm",
                                            "executable": False})
    assert rt.launch(not_exec, ())["ok"] is False


def _image_and_descriptor():
    from tessera_b200 import native_artifact as na
    abi = "tessera.nvidia.matmul.a_b_d_m_n_k.bf16.v1"
    image = na.NativeImageArtifact(target="blackwell", architecture="sm_100a", binary_format="cubin",
                                   payload=b"\x7fELF-stand-in", entry_points=(na.NativeEntryPoint("gemm_entry", abi),))
    desc = na.LaunchDescriptor(
        image_digest=image.image_digest, entry_symbol="gemm_entry", abi_id=abi,
        buffers=(na.BufferBinding(0, "a", "input", "fp32", 2, "row_major", 16),
                 na.BufferBinding(1, "d", "output", "fp32", 2, "row_major", 16)),
        scalars=(na.ScalarArgument(2, "n", "int32"),),
        shape_guards=(na.ShapeGuard("a", 1, "multiple_of", 8),))
    return image, desc


def test_native_launcher_registry():
    seen = {}

    def submit(image, descriptor, buffers, scalars, stream):
        seen.update(buffers=set(buffers), scalars=dict(scalars), symbol=descriptor.entry_symbol)
        return "ran"

    rt.register_native_launcher("blackwell", binary_formats=("cubin",), submit=submit, replace=True)
    with pytest.raises(ValueError):
        rt.register_native_launcher("sm_100a", binary_formats=("cubin",), submit=submit)
    with pytest.raises(ValueError):
        rt.register_native_launcher("sm_100a", binary_formats=(), submit=submit, replace=True)
    image, desc = _image_and_descriptor()
    assert image.target == "nvidia_sm100" and desc.argument_names() == ["a", "d", "n"]
    art = rt.RuntimeArtifact(metadata={"target": "nvidia_sm100"}, native_image=image, launch_descriptor=desc)
    a, d = np.zeros((4, 16), np.float32), np.zeros((4, 4), np.float32)
    res = rt.launch(art, (a, d, 5))
    assert res["ok"] and res["output"] == "ran" and res["execution_mode"] == "descriptor", res
    assert seen == {"buffers": {"a", "d"}, "scalars": {"n": 5}, "symbol": "gemm_entry"}
    assert res["image_digest"] == image.image_digest and res["launch_descriptor_digest"] == desc.descriptor_digest
    assert rt.launch(art, {"a": a, "d": d, "n": 7})["ok"]
    # objects that are not descriptor types never reach the hook
    bad = rt.RuntimeArtifact(metadata={"target": "nvidia_sm100"}, native_image=object(), launch_descriptor=object())
    assert rt.launch(bad, (a, d, 5))["runtime_status"] == "invalid_artifact"
    rt.unregister_native_launcher("nvidia_sm100")
    assert rt.launch(art, (a, d, 5))["runtime_status"] == "unimplemented"


def test_descriptor_invocation_is_validated_before_submission():
    """LaunchDescriptor.validate_invocation (python/tessera/compiler/native_artifact.py:997-1051):
    every mismatch is an invalid_artifact result with the reference's diagnostic code, and the
    submit hook is not called."""
    from tessera_b200 import native_artifact as na
    calls = []
    rt.register_native_launcher("nvidia_sm100", binary_formats=("cubin",),
                                submit=lambda *a: calls.append(a) or "ran", replace=True)
    image, desc = _image_and_descriptor()
    art = rt.RuntimeArtifact(metadata={"target": "nvidia_sm100"}, native_image=image, launch_descriptor=desc)
    a, d = np.zeros((4, 16), np.float32), np.zeros((4, 4), np.float32)

    def code(args):
        res = rt.launch(art, args)
        assert res["ok"] is False and res["runtime_status"] == "invalid_artifact", res
        return res.get("diagnostic_code")

    assert code({"a": a, "n": 5}) == "E_LAUNCH_BINDING_MISMATCH"                       # a buffer is missing
    assert code({"a": a, "d": d, "n": 5, "extra": 1}) == "E_LAUNCH_BINDING_MISMATCH"   # an unknown scalar
    assert code((a.astype(np.float16), d, 5)) == "E_LAUNCH_BINDING_MISMATCH"           # dtype
    assert code((a[0], d, 5)) == "E_LAUNCH_BINDING_MISMATCH"                           # rank
    assert code((np.zeros((4, 12), np.float32), d, 5)) == "E_LAUNCH_BINDING_MISMATCH"  # shape guard: 12 % 8
    assert code((a, d, 2.5)) == "E_LAUNCH_BINDING_MISMATCH"                            # int scalar given a float
    misaligned = np.zeros(4 * 16 + 1, np.float32)[1:].reshape(4, 16)                   # 4-byte aligned only
    assert code((misaligned, d, 5)) == "E_LAUNCH_BINDING_MISMATCH"
    other = na.NativeImageArtifact(target="sm100", architecture="sm_100a", binary_format="cubin", payload=b"other",
                                   entry_points=image.entry_points)
    stale = rt.RuntimeArtifact(metadata={"target": "nvidia_sm100"}, native_image=other, launch_descriptor=desc)
    res = rt.launch(stale, (a, d, 5))
    assert res["diagnostic_code"] == "E_LAUNCH_STALE_IMAGE"
    assert calls == []
    assert rt.launch(art, (a, d, 5))["ok"] and len(calls) == 1
    # schema errors are raised where the descriptor is built
    with pytest.raises(na.ArtifactContractError) as info:
        na.BufferBinding(0, "a", "sideways", "fp32", 2, "row_major")
    assert info.value.code == "E_LAUNCH_DESCRIPTOR_SCHEMA"
    with pytest.raises(na.ArtifactContractError):
        na.BufferBinding(0, "a", "input", "fp32", 2, "row_major", alignment=24)
    with pytest.raises(na.ArtifactContractError):
        na.LaunchDescriptor(image.image_digest, "gemm_entry", desc.abi_id,
                            buffers=(na.BufferBinding(0, "a", "input", "fp32", 2, "row_major"),
                                     na.BufferBinding(0, "d", "output", "fp32", 2, "row_major")))
    with pytest.raises(na.ArtifactContractError):
        na.NativeImageArtifact(target="sm100", architecture="sm_100a", binary_format="tarball", payload=b"x",
                               entry_points=image.entry_points)
    rt.unregister_native_launcher("nvidia_sm100")


def test_jit_rejects_targets_it_does_not_serve_and_scans_ops():
    with pytest.raises(tessera.TesseraJitError):
        tessera.jit(target="cpu")(lambda a: a)

    @tessera.jit(target="sm_100a")
    def step(A, W):
        return tessera.ops.gemm(A, W)

    art = step.runtime_artifact()
    assert art.metadata["compiler_path"] == "sm100_gemm"
    assert art.metadata["ops"][0]["operands"] == ["A", "W"]
    assert art.abi_signature == "tessera.runtime.v1.nvidia_sm100"


def test_op_argument_validation_happens_before_any_device_work():
    ops = tessera.ops
    a16 = np.zeros((4, 8), np.float16)
    with pytest.raises(ValueError):
        ops.gemm(a16, np.zeros((7, 4), np.float16))                    # K mismatch
    with pytest.raises(TypeError):
        ops.gemm(np.zeros((4, 8), np.float32), np.zeros((8, 4), np.float32))  # no tf32 path
    with pytest.raises(ValueError):
        ops.grouped_gemm(a16, np.zeros((2, 8, 8), np.float16), [1, 1])  # sizes do not sum to T
    with pytest.raises(ValueError):
        ops.grouped_gemm(a16, np.zeros((2, 8, 8), np.float16), [2, 2], kind="bogus")
    with pytest.raises(NotImplementedError):
        ops.grouped_gemm(a16, np.zeros((2, 8, 8), np.float16), [2, 2], kind="masked")
    with pytest.raises(ValueError):
        ops.gqa_attention(np.zeros((1, 6, 1, 128)), np.zeros((1, 4, 8, 128)), np.zeros((1, 4, 8, 128)), 6, 4)
    with pytest.raises(ValueError):
        ops.flash_attn(np.zeros((1, 2, 4, 128)), np.zeros((1, 2, 4, 128)), np.zeros((1, 2, 4, 128)),
                       dropout_p=1.5)
    assert ops.gemm(np.zeros((0, 8), np.float16), np.zeros((8, 4), np.float16)).shape == (0, 4)
    with pytest.raises(ValueError):
        ops.gemm(a16, np.zeros((8, 8), np.float16), epilogue={"activation": "swish"})
    with pytest.raises(NotImplementedError):
        ops.gemm(a16, np.zeros((8, 8), np.float16), epilogue={"dropout_p": 0.1})
    with pytest.raises(TypeError):
        ops.gemm(a16, np.zeros((8, 8), np.float16), epilogue={"bogus": 1})


def test_paged_kv_descriptors(golden_dir):
    """Page-ABI descriptors (python/tessera/cache/paged_kv.py:91-140, 421-454): validation, the
    host gather and materialisation through the protocol — no GPU involved."""
    import os
    from tessera_b200 import cache as pk
    g = np.load(os.path.join(golden_dir, "paged.npz"))
    n = int(g["sn"])
    abi = pk.PagedKVBufferABI(g["sk_pages"], g["sv_pages"], g["stable"], n)
    assert abi.page_size == 16
    gk, gv = abi.gather(g["sgidx"])
    np.testing.assert_array_equal(gk, g["sgk"])
    np.testing.assert_array_equal(gv, g["sgv"])
    with pytest.raises(IndexError):
        abi.gather([n])
    with pytest.raises(ValueError):
        pk.PagedKVBufferABI(g["sk_pages"], g["sv_pages"], g["stable"].astype(np.int64), n)
    with pytest.raises(ValueError):
        pk.PagedKVBufferABI(g["sk_pages"], g["sv_pages"], np.array([99], np.int32), 1)
    with pytest.raises(ValueError):
        pk.PagedKVBufferABI(g["sk_pages"], g["sv_pages"], g["stable"], 10 ** 6)
    with pytest.raises(ValueError):
        pk.PagedKVBufferABI(g["sk_pages"], g["sv_pages"][:1], g["stable"], n)

    class Handle:  # the protocol a contiguous cache satisfies
        def __init__(self, k, v, L):
            self.k, self.v, self.L = k, v, L

        def kv_geometry(self):
            return pk.KVGeometry(self.k.shape[1], self.k.shape[2], 4096, self.L)

        def seq_len(self):
            return self.k.shape[0]

        def gather(self, idx):
            idx = np.asarray(list(idx), np.int64)
            return self.k[idx], self.v[idx]

    m = pk.materialize_paged_kv_abi(Handle(g["k0"], g["v0"], 16))
    np.testing.assert_array_equal(m.k_pages, g["kpages0"])
    np.testing.assert_array_equal(m.page_table, g["table0"])
    assert m.logical_length == g["k0"].shape[0]
    with pytest.raises(TypeError):
        pk.materialize_paged_kv_abi(object())
    for bad in (0, 4, 24, 2048):
        with pytest.raises(ValueError):
            pk._check_page_size(bad)
    with pytest.raises(ValueError):
        pk.paged_attention(np.zeros((2, 1, 64), np.float32), abi)          # head_dim
    with pytest.raises(ValueError):
        pk.paged_attention(np.zeros((2, 1, 128), np.float32), abi, backend="rocm")
