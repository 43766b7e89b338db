"""The Python surface end to end on the GPU: @jit, runtime.launch, index_launch."""
import numpy as np
import pytest

from oracle import tessera_oracle as orc
from tests.gpu_util import TOL, rel_err

pytestmark = pytest.mark.gpu

import tessera_b200 as tessera  # noqa: E402
from tessera_b200 import runtime as rt  # noqa: E402
from tessera_b200.device import DeviceArray, bfloat16  # noqa: E402
from tessera_b200.distributed import DistributedArray, MeshSpec, ShardSpec  # noqa: E402


def test_launch_reaches_every_dtype():
    """tests/device/nvidia/test_mma_runtime_symbol.py:267-285, on target nvidia_sm100."""
    for dt in (bfloat16, np.float16):
        rng = np.random.default_rng(1200)
        a = rng.standard_normal((17, 31)).astype(np.float32).astype(dt)
        b = rng.standard_normal((31, 9)).astype(np.float32).astype(dt)
        art = rt.RuntimeArtifact(metadata={
            "target": "nvidia_sm100", "compiler_path": "sm100_gemm", "executable": True,
            "execution_kind": "native_gpu", "arg_names": ["a", "b"], "output_name": "d",
            "ops": [{"op_name": "tessera.matmul", "result": "d", "operands": ["a", "b"], "kwargs": {}}]})
        res = rt.launch(art, (a, b))
        assert res["ok"] is True, res.get("reason")
        assert res["execution_kind"] == "native_gpu" and res["runtime_status"] == "success"
        np.testing.assert_allclose(res["output"], orc.gemm(a, b), rtol=0, atol=1e-3)
    res = rt.launch(art, {"a": a, "b": np.zeros((30, 9), dt)})  # K mismatch -> structured failure
    assert res["ok"] is False and res["runtime_status"] == "invalid_artifact"


def test_launch_flash_attn_and_moe():
    rng = np.random.default_rng(5)
    q, k, v = (rng.standard_normal((1, 4, 200, 128), dtype=np.float32).astype(bfloat16) for _ in range(3))
    art = rt.make_artifact("tessera.flash_attn", ["Q", "K", "V"], kwargs={"causal": True})
    res = rt.launch(art, (q, k, v))
    assert res["ok"], res.get("reason")
    assert rel_err(res["output"], orc.flash_attn(q, k, v, causal=True)) < TOL
    x = rng.standard_normal((40, 64), dtype=np.float32).astype(bfloat16)
    w = rng.standard_normal((3, 64, 72), dtype=np.float32).astype(bfloat16)
    art = rt.make_artifact("tessera.grouped_gemm", ["x", "weights", "group_sizes"])
    res = rt.launch(art, {"x": x, "weights": w, "group_sizes": [10, 0, 30]})
    assert res["ok"], res.get("reason")
    assert rel_err(res["output"], orc.grouped_gemm(x, w, [10, 0, 30])) < TOL


def test_jit_keeps_intermediates_on_the_device():
    @tessera.jit(target="nvidia_sm100")
    def mlp(x, w1, w2):
        h = tessera.ops.gemm(x, w1, out_dtype=bfloat16)
        assert isinstance(h, DeviceArray)          # no download between the two GEMMs
        return tessera.ops.gemm(h, w2)

    rng = np.random.default_rng(8)
    x = (rng.standard_normal((64, 128), dtype=np.float32)).astype(bfloat16)
    w1 = (rng.standard_normal((128, 256), dtype=np.float32) / 11).astype(bfloat16)
    w2 = (rng.standard_normal((256, 64), dtype=np.float32) / 16).astype(bfloat16)
    y = mlp(x, w1, w2)
    h = orc.gemm(x, w1).astype(bfloat16)
    assert isinstance(y, np.ndarray) and rel_err(y, orc.gemm(h, w2)) < TOL


def test_index_launch_tensor_parallel_column_split():
    """The README sketch of the reference made runnable: W and Y split on N over axis "tp", A
    replicated, every rank's GEMM on the GPU, results landing in the shards of Y."""
    rng = np.random.default_rng(12)
    M, K, N, g = 64, 128, 256, 4
    A = (rng.standard_normal((M, K), dtype=np.float32) / np.sqrt(K)).astype(bfloat16)
    Wd = (rng.standard_normal((K, N), dtype=np.float32)).astype(bfloat16)
    mesh = MeshSpec({"tp": g})
    W = DistributedArray(Wd, "bf16", ShardSpec(partition=(1,), mesh_axes=("tp",)))._bind_mesh(mesh)
    Y = DistributedArray(np.zeros((M, N), np.float32), "fp32",
                         ShardSpec(partition=(1,), mesh_axes=("tp",)))._bind_mesh(mesh)

    @tessera.kernel
    def tp_gemm(a, w, y):
        y[:] = tessera.ops.gemm(a, w)

    tessera.index_launch(axis="tp")(tp_gemm)(A, W.parts("tp"), Y.parts("tp"))
    assert rel_err(Y.numpy(), orc.gemm(A, Wd)) < 1e-4


def test_chunk_submission_completes_in_stream_order(tmp_path):
    """A chunk submitted for a (device, stream id) with a CUDA stream bound completes when the
    stream reaches it: the token stays out while earlier work is queued and returns after it."""
    import json
    from tessera_b200 import collectives as coll, device
    coll.shutdown_runtime()
    coll.qos_limit_set(2)
    st = device.Stream()
    coll.bind_chunk_stream(0, 7, st)
    for _ in range(100):
        device.flush_l2(st)                       # ~10 ms of queued work ahead of the chunk
    coll.submit_chunk_async(0, 1 << 20, 0, 7)
    early = coll.qos_state()
    st.synchronize()
    late = coll.qos_state()
    assert early["peak_inflight"] == 1 and late["inflight"] == 0 and late["trace_events"] == 3
    coll.submit_chunk_async(0, 64, 0, 3)          # nothing bound to stream id 3: completes at once
    assert coll.qos_state()["inflight"] == 0
    out = tmp_path / "t.json"
    coll.trace_write(str(out))
    ev = json.loads(out.read_text())["traceEvents"]
    b = [e for e in ev if e["ph"] == "B" and e["tid"] == 7][0]
    e = [e for e in ev if e["ph"] == "E" and e["tid"] == 7][0]
    assert e["ts"] - b["ts"] > 1000               # microseconds: the end waited for the queued work
    coll.bind_chunk_stream(0, 7, None)
    coll.shutdown_runtime()
    st.close()
