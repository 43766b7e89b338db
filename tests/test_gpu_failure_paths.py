"""Failure paths on the GPU, made with waits that are certain to run out (a flag or barrier that
nothing ever signals) and short limits: the waiting kernel records the error word and ends by
itself, the host reads the code, and the next call works. Nothing here faults or hangs a GPU."""
import ctypes
from types import SimpleNamespace

import numpy as np
import pytest

from oracle import tessera_oracle as orc
from tessera_b200 import _lib, device, parallel
from tessera_b200 import runtime as rt
from tessera_b200.device import DeviceArray as DA, bfloat16

pytestmark = pytest.mark.gpu


def _gemm_artifact():
    return rt.make_artifact("tessera.matmul", ["a", "b"])


def test_expired_mbarrier_wait_surfaces_as_device_error_and_the_next_call_works():
    device.set_device(0)
    device.consume_device_error()
    rng = np.random.default_rng(7)
    a = rng.standard_normal((64, 96), dtype=np.float32).astype(bfloat16)
    b = rng.standard_normal((96, 40), dtype=np.float32).astype(bfloat16)
    # 1. straight through the C ABI: the kernel returns by itself and the word holds {5, 0, 77}
    _lib.call("tessera_sm100_selftest_wait_expiry", 1 << 20, None)          # about half a millisecond
    device.synchronize()
    assert device.consume_device_error() == (5, 0, 77)
    assert device.consume_device_error()[0] == 0                           # reading clears it
    # 2. through the op layer: the pending word turns the next host-facing op into rc 3 ...
    _lib.call("tessera_sm100_selftest_wait_expiry", 1 << 20, None)
    with pytest.raises(_lib.BackendError) as info:
        device.check_device_error("selftest")
    assert info.value.rc == 3 and "bounded wait expired" in str(info.value)
    # 3. ... and runtime.launch reports it as a structured device_error instead of raising
    _lib.call("tessera_sm100_selftest_wait_expiry", 1 << 20, None)
    res = rt.launch(_gemm_artifact(), (a, b))
    assert res["ok"] is False and res["runtime_status"] == "device_error", res
    # 4. the context is intact: the same launch now succeeds with the right numbers
    res = rt.launch(_gemm_artifact(), (a, b))
    assert res["ok"] is True, res.get("reason")
    np.testing.assert_allclose(res["output"], orc.gemm(a, b), rtol=0, atol=2e-3)
    with pytest.raises(_lib.BackendError):
        _lib.call("tessera_sm100_selftest_wait_expiry", 1 << 40, None)      # limit above the allowed maximum


def test_expert_parallel_wait_for_a_rank_that_never_arrives():
    """Rank 0 of a two-rank expert-parallel group whose rank 1 does not exist: its flags live in a
    second local control block that nothing ever raises. The dispatch and combine kernels give up
    after 30 ms each, record which wait ran out, and end; a one-rank forward afterwards is correct."""
    device.set_device(0)
    device.consume_device_error()
    rng = np.random.default_rng(11)
    T, H, F, E, k = 128, 128, 256, 4, 2
    x = rng.standard_normal((T, H), dtype=np.float32).astype(bfloat16)
    logits = rng.standard_normal((T, E), dtype=np.float32)
    wg = (rng.standard_normal((E, H, F), dtype=np.float32) / 11).astype(bfloat16)
    wu = (rng.standard_normal((E, H, F), dtype=np.float32) / 11).astype(bfloat16)
    wd = (rng.standard_normal((E, F, H), dtype=np.float32) / 16).astype(bfloat16)
    # the absent rank's buffers: plain local allocations handed over in place of IPC handles
    fake = {}
    half = E // 2
    # Built as a complete one-rank group first (no IPC handle is opened), then widened to a world of
    # two whose second rank is a set of stand-in buffers on this GPU.
    moe = parallel.DeviceExpertParallelMoE(SimpleNamespace(world=1, rank=0), lambda h: [h], DA.from_host(wg[:half]),
                                           DA.from_host(wu[:half]), DA.from_host(wd[:half]), T, k, half,
                                           wait_limit_ms=30)
    moe.world, moe.E, moe.Ep = 2, E, half
    moe.capacity = T * k * 2
    moe.group_sizes, moe.my_offsets = DA((E,), np.int32), DA((E + 1,), np.int32)
    moe.dst_base = DA((E,), np.int32)
    moe.recv = DA.zeros((moe.capacity, H), bfloat16)
    moe.hidden = DA((moe.capacity, F), bfloat16)
    moe.y = DA.zeros((moe.capacity, H), bfloat16)
    fake["recv"], fake["y"] = DA.zeros((moe.capacity, H), bfloat16), DA.zeros((moe.capacity, H), bfloat16)
    fake["ctrl"] = DA.zeros((moe.ctrl.nbytes,), np.uint8)
    device.synchronize()
    moe._recv_ptrs = (ctypes.c_void_p * 2)(moe.recv.ptr, fake["recv"].ptr)
    moe._y_ptrs = (ctypes.c_void_p * 2)(moe.y.ptr, fake["y"].ptr)
    moe._ctrl_ptrs = (ctypes.c_void_p * 2)(moe.ctrl.ptr, fake["ctrl"].ptr)
    out = moe.forward(DA.from_host(x), DA.from_host(logits))
    device.synchronize()                     # returns: every wait gave up after its 30 ms
    code, _block, detail = device.consume_device_error()
    assert code == 5 and detail == 101, (code, detail)      # first to expire: rank 1's counts
    assert out.shape == (T, H)
    # the flags this rank raised in the stand-in block are there (epoch 1): it did its own part
    ctrl1 = fake["ctrl"].download().view(np.int32)
    flags = ctrl1[8 * 256:]
    assert flags[0] == 1 and flags[32] == 1 and flags[64] == 1, flags[:96:32]     # counts, rows, outputs of rank 0
    moe.close()
    # a complete one-rank group on the same context works right after
    one = parallel.DeviceExpertParallelMoE(SimpleNamespace(world=1, rank=0), lambda h: [h], DA.from_host(wg),
                                           DA.from_host(wu), DA.from_host(wd), T, k, E, wait_limit_ms=2000)
    y = one.forward(DA.from_host(x), DA.from_host(logits))
    device.synchronize()
    assert device.consume_device_error()[0] == 0
    assert orc.max_rel_err(y.download(), orc.moe_layer_from_logits(x, logits, wg, wu, wd, k)[0]) < 1e-2
    one.close()
