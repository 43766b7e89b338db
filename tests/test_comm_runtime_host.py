"""The chunk-submission hooks (QoS tokens, trace, shutdown) without a GPU. The contract follows
the reference's smoke tool (src/collectives/tools/tessera-collective-runtime-smoke/
runtime_smoke.cpp): concurrent submitters, shutdown during submission, re-creation after
shutdown, and a trace whose begin and end events pair up."""
import ctypes
import json
import threading

import numpy as np
import pytest

from tessera_b200 import collectives as coll


@pytest.fixture(autouse=True)
def _fresh_runtime(lib):
    coll.shutdown_runtime()
    yield
    coll.shutdown_runtime()


def test_limit_is_clamped_and_state_reported():
    assert not coll.qos_state()["exists"]
    coll.qos_limit_set(0)                    # would block every submitter: taken as 1
    st = coll.qos_state()
    assert st["exists"] and st["limit"] == 1 and st["inflight"] == 0
    coll.qos_limit_set(5)
    assert coll.qos_state()["limit"] == 5


def test_concurrent_submitters_and_trace_pairs(tmp_path):
    coll.qos_limit_set(8)
    buf = np.zeros(16, np.uint8)
    threads = [threading.Thread(target=lambda d=d: [coll.submit_chunk_async(buf.ctypes.data, 1 << (10 + d), d, i % 3)
                                                    for i in range(100)]) for d in range(8)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    st = coll.qos_state()
    assert st["inflight"] == 0 and 1 <= st["peak_inflight"] <= 8
    assert st["trace_events"] == 8 * 100 * 3            # begin, counter, end per chunk
    out = tmp_path / "trace.json"
    coll.trace_write(str(out))
    ev = json.loads(out.read_text())["traceEvents"]
    begins = [e for e in ev if e["ph"] == "B"]
    ends = [e for e in ev if e["ph"] == "E"]
    assert len(begins) == len(ends) == 800
    assert {e["pid"] for e in begins} == {1000 + d for d in range(8)}
    assert all(e["args"]["schema"] == "tessera.telemetry.v1" and e["args"]["path"] == "NVLINK" for e in begins)
    big = [e for e in begins if e["args"]["memory_bytes"] >= 8 << 20]
    assert all(e["args"]["algo"] == "tree" for e in begins if e["args"]["memory_bytes"] < 8 << 20)
    assert all(e["args"]["algo"] == "ring" for e in big)
    with pytest.raises(OSError):
        coll.trace_write(str(tmp_path / "no_such_dir" / "t.json"))


def test_shutdown_while_submitting_then_reinit(lib):
    coll.qos_limit_set(4)
    stop = threading.Event()
    count = [0]

    def submitter():
        while not stop.is_set():
            lib.tessera_submit_chunk_async(None, ctypes.c_uint64(4096), 0, 0)
            count[0] += 1

    t = threading.Thread(target=submitter)
    t.start()
    for _ in range(200):
        coll.shutdown_runtime()
    stop.set()
    t.join()
    assert count[0] > 0
    coll.shutdown_runtime()
    assert not coll.qos_state()["exists"]
    lib.tessera_trace_write(b"/nonexistent/never_written.json")      # no runtime: a no-op
    coll.submit_chunk_async(0, 64)                                   # re-creates on demand
    st = coll.qos_state()
    assert st["exists"] and st["limit"] == 1 and st["trace_events"] == 3


def test_policy_from_environment(monkeypatch, tmp_path):
    monkeypatch.setenv("TESSERA_COMM_LARGE_MIN", "1000")
    monkeypatch.setenv("TESSERA_COMM_INTRA_PATH", "pcie")
    coll.shutdown_runtime()
    coll.submit_chunk_async(0, 2000)
    out = tmp_path / "t.json"
    coll.trace_write(str(out))
    b = [e for e in json.loads(out.read_text())["traceEvents"] if e["ph"] == "B"][0]
    assert b["args"]["algo"] == "ring" and b["args"]["path"] == "PCIE"


def test_collective_permute_validation():
    ad = coll.adapter(backend="single_process", world_size=1)
    out = ad.collective_permute(np.arange(4.0, dtype=np.float32), pairs=((0, 0),))
    np.testing.assert_array_equal(out[0], np.arange(4.0, dtype=np.float32))
    with pytest.raises(ValueError):
        ad.collective_permute(np.zeros(2, np.float32), pairs=())
    with pytest.raises(ValueError):
        ad.collective_permute(np.zeros(2, np.float32), pairs=((0, 1),))
    with pytest.raises(ValueError):
        ad.collective_permute(np.zeros(2, np.float32), pairs=((0, 0), (0, 0)))
