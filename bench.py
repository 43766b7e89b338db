"""Benchmark of the dense-contraction hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload ...]

Headline (one JSON line on stdout, rank 0): dense bf16 GEMM M=N=K=8192, fp32 accumulate, bf16
output. With N > 1 GPUs the GEMM is column-parallel (W split on N, A replicated) and followed by an
all-gather of Y, total work fixed ("strong" scaling). The same line carries, under "workloads",
the other configurations of the hot path (causal prefill attention, GQA decode attention, the MoE
layer), each with its own roofline entry.

A step is one pass over synthetic inputs that are resident in HBM before the timed region. Every
timed step is preceded (outside its CUDA-event bracket) by an L2 flush. Times are CUDA events on
the launching stream; with several ranks the per-step maximum over ranks is what counts.
``e2e`` is the same GEMM through the public ``tessera_b200.ops.gemm`` call with pinned host
buffers, host<->device copies inside the timed region.

``--impl reference`` times the reference's CPU implementation of the same configuration (its
numpy path, restated in oracle/) on the host cores of this machine.

Multi-GPU runs are launched as ``python -m torch.distributed.run --nproc-per-node N bench.py
--gpus N ...``; torch.distributed (gloo) is used for rank plumbing only.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) from the ncu captures
# summarised under profiles/. The GEMM capture is the benchmark size itself; the attention and MoE
# captures ran a quarter-size case (heads, batch, experts x slots) and are scaled x4, the traffic
# of these kernels being proportional to those counts. The MoE figure is the sum of its two
# grouped GEMM launches.
NCU_TRAFFIC_BYTES = {"gemm_8192": 1.209e9, "attn_prefill": 1.007e9, "attn_decode": 2.171e9, "attn_decode_paged": 2.166e9,
                     "attn_decode_int8": 1.093e9, "moe": 4.78e9}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return {k: float(d[k]) for k in FALLBACK_PEAKS}, "measured"
    except Exception:
        return dict(FALLBACK_PEAKS), "fallback"


# ------------------------------------------------------------------------------ clocks sampling
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.rows, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-i",
                 str(self.gpu), "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append(line.strip())

    def mark(self):
        return len(self.rows)

    def stop(self):
        if self.proc:
            self.proc.terminate()

    def summary(self, lo: int = 0, hi=None):
        sm, mx, reasons = [], [], set()
        for row in self.rows[lo:hi]:
            parts = [p.strip() for p in row.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                  "sw_power_cap"), parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------------ rank plumbing
class Ranks:
    def __init__(self, n_gpus: int):
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("gloo")
            self.dist = dist

    def barrier(self):
        if self.dist:
            self.dist.barrier()

    def gather(self, obj):
        if not self.dist:
            return [obj]
        out = [None] * self.world
        self.dist.all_gather_object(out, obj)
        return out

    def bcast(self, obj):
        if not self.dist:
            return obj
        box = [obj]
        self.dist.broadcast_object_list(box, src=0)
        return box[0]

    def close(self):
        if self.dist:
            self.dist.barrier()
            self.dist.destroy_process_group()


def timed_steps(ranks, device, fn, steps, warmup, flush=True):
    """W warm-ups, then K steps; each step bracketed by CUDA events on the launching stream, an
    L2 flush before every bracket. Returns per-step times (ms) as the max over ranks."""
    for _ in range(warmup):
        fn()
    device.synchronize()
    ranks.barrier()
    ev = [(device.Event(), device.Event()) for _ in range(steps)]
    for a, b in ev:
        if flush:
            device.flush_l2()
        a.record()
        fn()
        b.record()
    device.synchronize()
    ranks.barrier()
    mine = [a.elapsed_ms(b) for a, b in ev]
    device.check_device_error("bench")
    allr = ranks.gather(mine)
    return [max(r[i] for r in allr) for i in range(steps)]


def clock_probe(device, sampler, fn, seconds=0.4):
    """Runs `fn` back to back for `seconds` and returns the sampler marks around it: the clocks
    the GPU holds under this load (single timed steps are shorter than one nvidia-smi sample)."""
    fn()
    device.synchronize()
    time.sleep(0.05)
    m0 = sampler.mark()
    t0 = time.perf_counter()
    while time.perf_counter() - t0 < seconds:
        for _ in range(8):
            fn()
        device.synchronize()
    return m0, sampler.mark()


def tiled_normal(rng, shape, tile_axis_len, scale, dtype):
    """N(0,1)*scale values; drawn for `tile_axis_len` entries of axis 0 and repeated along it
    (same distribution, a fraction of the host time)."""
    base = (rng.standard_normal((tile_axis_len,) + tuple(shape[1:]), dtype=np.float32) * scale).astype(dtype)
    reps = -(-shape[0] // tile_axis_len)
    return np.concatenate([np.roll(base, r, axis=-1) for r in range(reps)], axis=0)[:shape[0]]


# ------------------------------------------------------------------------------ workloads
def bench_gemm(ranks, args, peaks, peak_kind, sampler):
    import tessera_b200 as tessera
    from tessera_b200 import _lib, collectives, device, parallel
    from tessera_b200.device import DeviceArray, PinnedArray, bfloat16
    n = 8192
    W = ranks.world
    rng = np.random.default_rng(1002)
    A = (rng.standard_normal((n, n), dtype=np.float32) / np.sqrt(n)).astype(bfloat16)
    B = (rng.standard_normal((n, n), dtype=np.float32) / np.sqrt(n)).astype(bfloat16)
    c0, nb = parallel.tp_column_range(n, W, ranks.rank)
    dA = DeviceArray.from_host(A)
    dB = DeviceArray.from_host(B)            # full W on every rank; a rank reads its column block
    dY = DeviceArray.zeros((n, n), bfloat16)
    comm = None
    stage = gathered = fused = None
    tp_mode = "single"
    if W > 1:
        uid = ranks.bcast(collectives.Communicator.unique_id() if ranks.rank == 0 else None)
        comm = collectives.Communicator.from_unique_id(uid, W, ranks.rank)
        stage = DeviceArray((n, nb), bfloat16)
        gathered = DeviceArray((W, n, nb), bfloat16)
        tp_mode = "nccl"
        if args.tp_mode == "fused":
            try:
                fused = parallel.TensorParallelGemm(n, n, n, W, ranks.rank, ranks.gather, bfloat16, bfloat16)
                dY = fused.Y
                tp_mode = "fused"
            except Exception as exc:
                fused = None
                tp_mode = f"nccl (fused set-up failed: {exc})"
            # every rank must take the same path
            modes = ranks.gather(tp_mode)
            if any(m != "fused" for m in modes):
                fused, tp_mode = None, next(m for m in modes if m != "fused")

    def gemm_only():
        if W == 1:
            _lib.call("tessera_sm100_gemm_device", dA.ptr, dB.ptr, dY.ptr, 1, n, n, n, _lib.BF16,
                      _lib.BF16, None)
        else:
            _lib.call("tessera_sm100_gemm_strided_device", dA.ptr, dB.ptr + c0 * 2, stage.ptr, 1, n, nb,
                      n, n, n, nb, 0, 0, 0, _lib.BF16, _lib.BF16, None)

    def step():
        if fused is not None:
            fused(dA, dB)
            return
        gemm_only()
        if W > 1:
            comm.all_gather(stage, gathered)
            for r in range(W):   # [W, M, nb] -> row-major Y[M, N]
                _lib.call("tessera_sm100_device_copy_2d", dY.ptr + r * nb * 2, n * 2,
                          gathered.ptr + r * n * nb * 2, nb * 2, nb * 2, n, None)

    l0 = device.launch_count()
    m0 = sampler.mark()
    times = timed_steps(ranks, device, step, args.steps, args.warmup)
    m1 = sampler.mark()
    launches = (device.launch_count() - l0) * args.steps // (args.steps + args.warmup)
    # kernel-only time for the roofline entry: at one GPU the step is the kernel; with several,
    # the GEMM without the exchange, timed the same way (before the clock probe heats the GPU)
    kernel_times = times if W == 1 else timed_steps(ranks, device, gemm_only, args.steps, args.warmup)
    probe_marks = clock_probe(device, sampler, step)
    flops = 2.0 * n * n * n
    ms = statistics.mean(times)
    k_ms = statistics.mean(kernel_times)
    achieved = flops / W / k_ms / 1e9        # per-GPU kernel TFLOP/s
    # correctness spot check of what was just timed
    rows = [0, 4097, n - 1]
    got = dY.download()[rows].astype(np.float32)
    ref = A[rows].astype(np.float32) @ B.astype(np.float32)
    rel = float(np.abs(got - ref).max() / np.abs(ref).max())

    # end to end through the public op with pinned host buffers
    e2e = None
    try:
        pA, pB = PinnedArray((n, n), bfloat16), PinnedArray((n, nb), bfloat16)
        pY = PinnedArray((n, nb), bfloat16)
        pA.array[...] = A
        pB.array[...] = B[:, c0:c0 + nb]
        e2e_steps = max(2, min(args.steps, 5))
        tessera.ops.gemm(pA.array, pB.array, out_dtype=bfloat16, out=pY.array)
        ranks.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            tessera.ops.gemm(pA.array, pB.array, out_dtype=bfloat16, out=pY.array)
        device.synchronize()
        dt = (time.perf_counter() - t0) / e2e_steps
        dt = max(ranks.gather(dt))
        e2e = {"value": flops / dt / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": int(pA.nbytes + pB.nbytes),
               "d2h_bytes_per_step": int(pY.nbytes), "ms_per_step": dt * 1e3,
               "api": "tessera_b200.ops.gemm(host, host) -> tessera_sm100_gemm",
               "note": "per rank: upload A and its column block of W, GEMM, download its block of Y"}
    except Exception as exc:  # keep the headline even if pinned allocation fails
        e2e = {"value": None, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
               "error": str(exc)}
    if comm:
        comm.close()
    return {
        "value": flops / ms / 1e9, "ms_per_step": ms, "gpu_launches": int(launches * W),
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"],
                     "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops"],
                     "traffic": NCU_TRAFFIC_BYTES["gemm_8192"], "peak_kind": f"burst cuBLAS bf16, of {peak_kind}",
                     "kernel_ms": k_ms, "kernel": ("gemm2_kernel<bf16> (tcgen05 cta_group::2, 256x256x64 per CTA pair, 6-stage TMA)"
                                if (n // 256) * (-(-nb // 256)) >= 74 else
                                "gemm_kernel<bf16,plain> (tcgen05 128x256x64, 4-stage TMA)")},
        "e2e": e2e, "check_max_rel_err": rel, "clock_marks": (m0, m1), "probe_marks": probe_marks,
        "tp_mode": tp_mode,
    }


def bench_attn_prefill(ranks, args, peaks, peak_kind):
    import ctypes
    from tessera_b200 import _lib, device
    from tessera_b200.device import DeviceArray, bfloat16
    B, H, S, D = 8, 32, 4096, 128
    W = ranks.world
    Hl = H // W
    rng = np.random.default_rng(1003 + ranks.rank)
    q, k, v = (tiled_normal(rng, (B, Hl, S, D), 2, 1.0, bfloat16) for _ in range(3))
    dq, dk, dv = (DeviceArray.from_host(t) for t in (q, k, v))
    do = DeviceArray.zeros((B, Hl, S, D), bfloat16)
    scale = ctypes.c_float(1.0 / np.sqrt(D))
    fn = lambda: _lib.call("tessera_sm100_flash_attn_fwd_device", dq.ptr, dk.ptr, dv.ptr, do.ptr, B, Hl,
                           Hl, S, S, D, scale, 1, None)
    times = timed_steps(ranks, device, fn, args.steps, args.warmup)
    ms = statistics.mean(times)
    flops = 4.0 * B * H * S * S * D / 2
    ach = flops / W / ms / 1e9
    return {"metric": "causal flash-attention forward TFLOP/s", "value": flops / ms / 1e9, "unit": "TFLOP/s",
            "ms_per_step": ms, "config": f"B={B} H={H} S={S} D={D} bf16 causal, heads sharded /{W}",
            "flops_convention": "4*B*H*S^2*D/2",
            "roofline": {"bound": "tensor", "achieved": ach, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": ach / peaks["bf16_tflops"], "traffic": NCU_TRAFFIC_BYTES["attn_prefill"],
                         "peak_kind": f"burst cuBLAS bf16, of {peak_kind}"}}


def bench_attn_backward(ranks, args, peaks, peak_kind):
    """Gradients of the prefill workload (same shape): forward recompute for O and the row
    log-sum-exps, delta, the dQ kernel and the dK/dV kernel, all inside the timed step."""
    import ctypes
    from tessera_b200 import _lib, device
    from tessera_b200.device import DeviceArray, bfloat16
    B, H, S, D = 8, 32, 4096, 128
    W = ranks.world
    Hl = H // W
    rng = np.random.default_rng(1010 + ranks.rank)
    q, k, v, g = (tiled_normal(rng, (B, Hl, S, D), 2, 1.0, bfloat16) for _ in range(4))
    dq, dk, dv, dg = (DeviceArray.from_host(t) for t in (q, k, v, g))
    gq, gk, gv = (DeviceArray.zeros((B, Hl, S, D), bfloat16) for _ in range(3))
    ws = DeviceArray((int(_lib.load().tessera_sm100_flash_attn_bwd_bf16_workspace_bytes(B, Hl, S)),), np.uint8)
    scale = ctypes.c_float(1.0 / np.sqrt(D))
    fn = lambda: _lib.call("tessera_sm100_flash_attn_bwd_bf16_device", dg.ptr, dq.ptr, dk.ptr, dv.ptr, gq.ptr,
                           gk.ptr, gv.ptr, B, Hl, Hl, S, S, scale, 1, ws.ptr, None)
    times = timed_steps(ranks, device, fn, args.steps, args.warmup)
    ms = statistics.mean(times)
    # the same gradients from a kept forward state (O and the row log-sum-exps): no recompute
    o = DeviceArray.zeros((B, Hl, S, D), bfloat16)
    lse = DeviceArray.zeros((B, Hl, S), np.float32)
    dscr = DeviceArray.zeros((B, Hl, S), np.float32)
    _lib.call("tessera_sm100_flash_attn_fwd_lse_device", dq.ptr, dk.ptr, dv.ptr, o.ptr, lse.ptr, B, Hl, Hl, S, S, D,
              scale, 1, None)
    fn2 = lambda: _lib.call("tessera_sm100_flash_attn_bwd_bf16_saved_device", dg.ptr, dq.ptr, dk.ptr, dv.ptr, o.ptr,
                            lse.ptr, gq.ptr, gk.ptr, gv.ptr, B, Hl, Hl, S, S, scale, 1, dscr.ptr, None)
    ms_saved = statistics.mean(timed_steps(ranks, device, fn2, args.steps, args.warmup))
    flops = 10.0 * B * H * S * S * D / 2
    ach = flops / W / ms / 1e9
    return {"metric": "causal flash-attention backward TFLOP/s", "value": flops / ms / 1e9, "unit": "TFLOP/s",
            "ms_per_step": ms, "ms_per_step_from_saved_forward_state": ms_saved,
            "tflops_from_saved_forward_state": flops / ms_saved / 1e9,
            "config": f"B={B} H={H} S={S} D={D} bf16 causal, heads sharded /{W}",
            "flops_convention": "10*B*H*S^2*D/2 (five S x S x D products; the kernels form seven, plus the "
                                "forward recompute, all inside the timed step)",
            "device_error": device.consume_device_error()[0],
            "roofline": {"bound": "tensor", "achieved": ach, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": ach / peaks["bf16_tflops"], "traffic": None,
                         "peak_kind": f"burst cuBLAS bf16, of {peak_kind}"}}


def bench_attn_decode(ranks, args, peaks, peak_kind):
    import ctypes
    from tessera_b200 import _lib, device
    from tessera_b200.device import DeviceArray, bfloat16
    B, Hq, Hkv, S, D = 64, 32, 8, 8192, 128
    W = ranks.world
    Bl = B // W
    rng = np.random.default_rng(1004 + ranks.rank)
    q = rng.standard_normal((Bl, Hq, 1, D), dtype=np.float32).astype(bfloat16)
    k = tiled_normal(rng, (Bl, Hkv, S, D), 2, 1.0, bfloat16)
    v = tiled_normal(rng, (Bl, Hkv, S, D), 2, 1.0, bfloat16)
    dq, dk, dv = (DeviceArray.from_host(t) for t in (q, k, v))
    do = DeviceArray.zeros((Bl, Hq, 1, D), bfloat16)
    lib = _lib.load()
    ns = lib.tessera_sm100_attn_decode_splits(Bl, Hq, Hkv, S)
    scr = DeviceArray((max(1, lib.tessera_sm100_attn_decode_scratch_bytes(Bl, Hq, ns)),), np.uint8)
    scale = ctypes.c_float(1.0 / np.sqrt(D))
    fn = lambda: _lib.call("tessera_sm100_attn_decode_device", dq.ptr, dk.ptr, dv.ptr, do.ptr, Bl, Hq, Hkv,
                           S, D, scale, ns, scr.ptr, None)
    times = timed_steps(ranks, device, fn, args.steps, args.warmup)
    ms = statistics.mean(times)
    nbytes = 2.0 * B * Hkv * S * D * 2
    ach = nbytes / W / ms / 1e6
    return {"metric": "GQA decode attention GB/s (K+V bytes)", "value": nbytes / ms / 1e6, "unit": "GB/s",
            "ms_per_step": ms, "config": f"batch={B} Hq={Hq} Hkv={Hkv} KV={S} D={D} bf16, batch sharded /{W}",
            "splits": ns,
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": ach / peaks["hbm_gbs"], "traffic": NCU_TRAFFIC_BYTES["attn_decode"],
                         "peak_kind": f"copy bandwidth, of {peak_kind}"}}


def bench_attn_decode_paged(ranks, args, peaks, peak_kind):
    """The decode workload with K/V behind a page table: pages [P, 64, Hkv, D] placed by a random
    permutation, one table row per sequence."""
    import ctypes
    from tessera_b200 import _lib, device
    from tessera_b200.device import DeviceArray, bfloat16
    B, Hq, Hkv, S, D, L = 64, 32, 8, 8192, 128, 64
    W = ranks.world
    Bl = B // W
    rng = np.random.default_rng(1006 + ranks.rank)
    per_seq = S // L
    P = Bl * per_seq
    q = rng.standard_normal((Bl, Hq, D), dtype=np.float32).astype(bfloat16)
    kp = tiled_normal(rng, (P, L, Hkv, D), 64, 1.0, bfloat16)
    vp = tiled_normal(rng, (P, L, Hkv, D), 64, 1.0, bfloat16)
    table = rng.permutation(P).astype(np.int32).reshape(Bl, per_seq)
    lens = np.full(Bl, S, np.int32)
    dq, dk, dv, dt, dl = (DeviceArray.from_host(t) for t in (q, kp, vp, table, lens))
    do = DeviceArray.zeros((Bl, Hq, D), bfloat16)
    lib = _lib.load()
    ns = lib.tessera_sm100_attn_decode_splits(Bl, Hq, Hkv, S)
    scr = DeviceArray((max(1, lib.tessera_sm100_attn_decode_scratch_bytes(Bl, Hq, ns)),), np.uint8)
    scale = ctypes.c_float(1.0 / np.sqrt(D))
    fn = lambda: _lib.call("tessera_sm100_paged_attn_decode_device", dq.ptr, dk.ptr, dv.ptr, dt.ptr, dl.ptr,
                           do.ptr, Bl, Hq, Hkv, D, L, P, per_seq, S, scale, ns, scr.ptr, None)
    times = timed_steps(ranks, device, fn, args.steps, args.warmup)
    ms = statistics.mean(times)
    code = device.consume_device_error()[0]
    nbytes = 2.0 * B * Hkv * S * D * 2
    ach = nbytes / W / ms / 1e6
    return {"metric": "paged GQA decode attention GB/s (K+V bytes)", "value": nbytes / ms / 1e6, "unit": "GB/s",
            "ms_per_step": ms, "device_error": code,
            "config": f"batch={B} Hq={Hq} Hkv={Hkv} KV={S} D={D} bf16, pages of {L} tokens [P,L,Hkv,D] in "
                      f"random physical order, batch sharded /{W}",
            "splits": ns,
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": ach / peaks["hbm_gbs"], "traffic": NCU_TRAFFIC_BYTES["attn_decode_paged"],
                         "peak_kind": f"copy bandwidth, of {peak_kind}"}}


def bench_attn_decode_int8(ranks, args, peaks, peak_kind):
    """The decode workload over an int8 KV cache (per-token scales): half the bytes of the bf16
    cache. The metric counts the bytes the kernel has to read (int8 K + V plus the scales)."""
    import ctypes
    from tessera_b200 import _lib, device
    from tessera_b200.device import DeviceArray, bfloat16
    B, Hq, Hkv, S, D = 64, 32, 8, 8192, 128
    W = ranks.world
    Bl = B // W
    rng = np.random.default_rng(1008 + ranks.rank)
    q = rng.standard_normal((Bl, Hq, D), dtype=np.float32).astype(bfloat16)
    base = rng.integers(1, 256, (2, Hkv, S, D), dtype=np.uint8)   # stored form: value + 128
    kq = np.concatenate([np.roll(base, r, axis=-1) for r in range(-(-Bl // 2))])[:Bl]
    vq = np.roll(kq, 3, axis=2)
    ks = rng.uniform(0.005, 0.03, (Bl, S)).astype(np.float32)
    vs = rng.uniform(0.005, 0.03, (Bl, S)).astype(np.float32)
    dq, dk, dv, dks, dvs = (DeviceArray.from_host(t) for t in (q, kq, vq, ks, vs))
    do = DeviceArray.zeros((Bl, Hq, D), bfloat16)
    lib = _lib.load()
    ns = lib.tessera_sm100_attn_decode_int8_splits(Bl, Hq, Hkv, S)
    scr = DeviceArray((max(1, lib.tessera_sm100_attn_decode_scratch_bytes(Bl, Hq, ns)),), np.uint8)
    scale = ctypes.c_float(1.0 / np.sqrt(D))
    fn = lambda: _lib.call("tessera_sm100_attn_decode_int8_device", dq.ptr, dk.ptr, dv.ptr, dks.ptr, dvs.ptr,
                           do.ptr, Bl, Hq, Hkv, S, D, scale, ns, scr.ptr, None)
    times = timed_steps(ranks, device, fn, args.steps, args.warmup)
    ms = statistics.mean(times)
    code = device.consume_device_error()[0]
    nbytes = 2.0 * B * Hkv * S * D + 2.0 * B * S * 4
    ach = nbytes / W / ms / 1e6
    return {"metric": "GQA decode attention over an int8 KV cache, GB/s (int8 K+V bytes + scales)",
            "value": nbytes / ms / 1e6, "unit": "GB/s", "ms_per_step": ms, "device_error": code,
            "config": f"batch={B} Hq={Hq} Hkv={Hkv} KV={S} D={D}, int8 K/V with per-token fp32 scales, "
                      f"batch sharded /{W}",
            "splits": ns, "equivalent_bf16_gbs": 2.0 * B * Hkv * S * D * 2 / ms / 1e6,
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": ach / peaks["hbm_gbs"], "traffic": NCU_TRAFFIC_BYTES["attn_decode_int8"] / W,
                         "peak_kind": f"copy bandwidth, of {peak_kind}"}}


def bench_moe(ranks, args, peaks, peak_kind):
    from tessera_b200 import _lib, collectives, device, parallel
    from tessera_b200.device import DeviceArray, bfloat16
    T, H, F, E, k = 8192, 4096, 14336, 8, 2
    W = ranks.world
    rng = np.random.default_rng(1005)
    x = rng.standard_normal((T, H), dtype=np.float32).astype(bfloat16)
    logits = rng.standard_normal((T, E), dtype=np.float32)
    Ep = E // W
    rngw = np.random.default_rng(2005 + ranks.rank)
    wg = tiled_normal(rngw, (Ep, H, F), 1, 1 / np.sqrt(H), bfloat16)
    wu = tiled_normal(rngw, (Ep, H, F), 1, 1 / np.sqrt(H), bfloat16)
    wd = tiled_normal(rngw, (Ep, F, H), 1, 1 / np.sqrt(F), bfloat16)
    dwg, dwu, dwd = (DeviceArray.from_host(t) for t in (wg, wu, wd))
    flops = 3 * 2.0 * T * k * H * F
    ep_mode = "single"
    if W == 1:
        dx, dl = DeviceArray.from_host(x), DeviceArray.from_host(logits)
        out = DeviceArray.zeros((T, H), bfloat16)
        ws = DeviceArray((_lib.load().tessera_sm100_moe_workspace_bytes(T, H, F, E, k),), np.uint8)
        fn = lambda: _lib.call("tessera_sm100_moe_layer_device", dx.ptr, dl.ptr, dwg.ptr, dwu.ptr, dwd.ptr,
                               out.ptr, T, H, F, E, k, 1, -1, _lib.BF16, _lib.BF16, ws.ptr, None)
        comm = None
    else:
        uid = ranks.bcast(collectives.Communicator.unique_id() if ranks.rank == 0 else None)
        comm = collectives.Communicator.from_unique_id(uid, W, ranks.rank)
        Tl = T // W
        sl = slice(ranks.rank * Tl, (ranks.rank + 1) * Tl)
        dxl = DeviceArray.from_host(x[sl])
        ll = np.ascontiguousarray(logits[sl])
        ep_mode = "device"
        try:
            moe = parallel.DeviceExpertParallelMoE(comm, ranks.gather, dwg, dwu, dwd, Tl, k, E)
            dll = DeviceArray.from_host(ll)
            out_l = DeviceArray.zeros((Tl, H), bfloat16)
            fn = lambda: moe.forward(dxl, dll, out=out_l)
        except Exception as exc:
            ep_mode = f"nccl all-to-all (device exchange set-up failed: {exc})"
        modes = ranks.gather(ep_mode)
        if any(m != "device" for m in modes):
            ep_mode = next(m for m in modes if m != "device")
            moe = parallel.ExpertParallelMoE(E, k, parallel.NcclTransport(comm, ranks.gather),
                                             parallel.GpuMoeBackend(dwg, dwu, dwd))
            fn = lambda: moe.forward(dxl, ll)
    times = timed_steps(ranks, device, fn, max(2, args.steps // 2), min(args.warmup, 3))
    ms = statistics.mean(times)
    pipelined = None
    if W > 1 and ep_mode == "device":
        # the same layer over micro-batches, exchange overlapping the expert GEMMs
        try:
            pm = parallel.PipelinedExpertParallelMoE(comm, ranks.gather, dwg, dwu, dwd, Tl, k, E, micro_batches=2)
            fnp = lambda: pm.forward(dxl, dll, out=out_l)
            pipelined = {"micro_batches": 2,
                         "ms_per_step": statistics.mean(timed_steps(ranks, device, fnp, max(2, args.steps // 2),
                                                                    min(args.warmup, 3)))}
            pm.close()
        except Exception as exc:
            pipelined = {"error": f"{type(exc).__name__}: {exc}"}
    if comm:
        comm.close()
    ach = flops / W / ms / 1e9
    return {"metric": "MoE FFN layer TFLOP/s (routed slots, unpadded)", "value": flops / ms / 1e9,
            "unit": "TFLOP/s", "ms_per_step": ms, "pipelined": pipelined,
            "config": f"T={T} H={H} F={F} E={E} top-{k} bf16, " + ("single GPU" if W == 1 else f"expert-parallel /{W}, exchange: {ep_mode}"),
            "roofline": {"bound": "tensor", "achieved": ach, "peak": peaks["bf16_tflops_sustained"],
                         "unit": "TFLOP/s", "frac": ach / peaks["bf16_tflops_sustained"],
                         "traffic": NCU_TRAFFIC_BYTES["moe"],
                         "peak_kind": f"sustained cuBLAS bf16 (two multi-ms GEMMs per step), of {peak_kind}"}}


def bench_moe_fp8(ranks, args, peaks, peak_kind):
    """The expert FFN of the MoE workload with e4m3 operands (quant="fp8_e4m3"): activations
    quantised per tensor inside the timed step, expert weights quantised once beforehand (they are
    static), gate/up GEMMs fused with silu_mul, hidden re-quantised, down GEMM. Single GPU."""
    import ctypes
    from tessera_b200 import _lib, device, ops
    from tessera_b200.device import DeviceArray, bfloat16
    if ranks.world != 1:
        return {"skipped": "single-GPU workload"}
    T, H, F, E, k = 8192, 4096, 14336, 8, 2
    S = T * k
    sizes = np.array([1994, 2066, 2065, 2092, 2074, 2036, 1965, 2092], np.int32)   # the seed-1005 routing
    off = np.zeros(E + 1, np.int32)
    off[1:] = np.cumsum(sizes)
    rng = np.random.default_rng(1007)
    xs = tiled_normal(rng, (S, H), 64, 1.0, bfloat16)
    wg = tiled_normal(rng, (E, H, F), 1, 1 / np.sqrt(H), bfloat16)
    wu = tiled_normal(rng, (E, H, F), 1, 1 / np.sqrt(H), bfloat16)
    wd = tiled_normal(rng, (E, F, H), 1, 1 / np.sqrt(F), bfloat16)
    gq, uq, dq = (ops.quantize_fp8_experts(w) for w in (wg, wu, wd))
    dx, doff = DeviceArray.from_host(xs), DeviceArray.from_host(off)
    xq, sx = DeviceArray((S, H), np.uint8), DeviceArray((3,), np.float32)
    hidden, hq, sh = DeviceArray((S, F), np.float32), DeviceArray((S, F), np.uint8), DeviceArray((3,), np.float32)
    amax = DeviceArray.zeros((1,), np.uint32)
    out = DeviceArray((S, H), bfloat16)

    def fn():
        _lib.call("tessera_sm100_quantize_fp8_device", dx.ptr, S * H, _lib.BF16, xq.ptr, sx.ptr, None, None)
        _lib.call("tessera_sm100_device_memset", amax.ptr, 0, 4, None)
        _lib.call("tessera_sm100_grouped_swiglu_fp8_device", xq.ptr, gq.q.ptr, uq.q.ptr, doff.ptr, hidden.ptr, S, H,
                  F, E, sx.ptr, gq.scales.ptr, uq.scales.ptr, _lib.F32, amax.ptr, None)
        _lib.call("tessera_sm100_quantize_fp8_device", hidden.ptr, S * F, _lib.F32, hq.ptr, sh.ptr, amax.ptr, None)
        _lib.call("tessera_sm100_grouped_gemm_fp8_device", hq.ptr, dq.q.ptr, doff.ptr, out.ptr, S, F, H, E, sh.ptr,
                  dq.scales.ptr, _lib.BF16, None)

    times = timed_steps(ranks, device, fn, max(2, args.steps // 2), min(args.warmup, 3))
    ms = statistics.mean(times)
    flops = 3 * 2.0 * S * H * F
    ach = flops / ms / 1e9
    return {"metric": "MoE expert FFN TFLOP/s, e4m3 operands (quant=fp8_e4m3)", "value": ach, "unit": "TFLOP/s",
            "ms_per_step": ms,
            "config": f"{S} routed slots in {E} ragged groups, H={H} F={F}; step = quantise x, fused gate/up GEMM + "
                      f"silu_mul (fp32 hidden, so its quantisation matches the reference's), quantise hidden, down GEMM (weights "
                      f"quantised once)",
            "roofline": {"bound": "tensor", "achieved": ach, "peak": 2 * peaks["bf16_tflops_sustained"],
                         "unit": "TFLOP/s", "frac": ach / (2 * peaks["bf16_tflops_sustained"]), "traffic": None,
                         "peak_kind": f"2 x sustained cuBLAS bf16 (no fp8 peak was measured: the dense fp8 rate is "
                                      f"nominally twice the bf16 rate), of {peak_kind}"}}


# ------------------------------------------------------------------------------ CPU baseline
def cpu_gemm_baseline(target_seconds: float = 10.0, max_reps: int = 10):
    from oracle import tessera_oracle as orc
    inp = orc.make_inputs("gemm_bf16")
    A, B = inp["A"].astype(np.float32), inp["B"].astype(np.float32)
    t0 = time.perf_counter()
    orc.gemm(A, B)
    first = time.perf_counter() - t0
    reps = int(min(max_reps, max(1, round(target_seconds / max(first, 1e-3)))))
    t0 = time.perf_counter()
    for _ in range(reps):
        orc.gemm(A, B)
    dt = (time.perf_counter() - t0) / reps
    flops = 2.0 * 8192 ** 3
    return {"value": flops / dt / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port",
            "sample": f"{reps} x full 8192^3 fp32 matmul of bf16-rounded operands (numpy, all host threads), "
                      f"{dt:.2f} s each", "seconds_per_step": dt}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import tessera_oracle as orc
    inp = orc.make_inputs("gemm_bf16")
    A, B = inp["A"].astype(np.float32), inp["B"].astype(np.float32)
    for _ in range(args.warmup):
        orc.gemm(A, B)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        orc.gemm(A, B)
    dt = (time.perf_counter() - t0) / args.steps
    val = 2.0 * 8192 ** 3 / dt / 1e12
    line = {"impl": "reference", "metric": "bf16 GEMM TFLOP/s (M=N=K=8192)", "value": val, "unit": "TFLOP/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": "gemm_bf16_8192: A[8192,8192] x B[8192,8192], bf16 operands, fp32 accumulate"},
            "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port",
                             "sample": "each step = the full 8192^3 product: the reference's tessera.ops.gemm "
                                       "(np.matmul) on fp32 arrays holding bf16 values, all host threads"},
            "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------ small cases for ncu
def profile_case(name: str) -> None:
    """One warm-up and two launches of one kernel on a small case (inputs larger than L2, well
    under a few GB): what `ncu --set full -k regex:<kernel> -c 2` is pointed at."""
    import ctypes
    from tessera_b200 import _lib, device
    from tessera_b200.device import DeviceArray, bfloat16
    device.set_device(0)
    rng = np.random.default_rng(1)

    def dev_normal(shape, scale=1.0):
        return DeviceArray.from_host(tiled_normal(rng, shape, min(shape[0], 2), scale, bfloat16))

    if name == "gemm":
        n = 8192
        a, b = dev_normal((n, n), 1 / np.sqrt(n)), dev_normal((n, n), 1 / np.sqrt(n))
        d = DeviceArray.zeros((n, n), bfloat16)
        fn = lambda: _lib.call("tessera_sm100_gemm_device", a.ptr, b.ptr, d.ptr, 1, n, n, n, _lib.BF16,
                               _lib.BF16, None)
    elif name == "attn_prefill":
        B, H, S, D = 4, 16, 4096, 128
        q, k, v = (dev_normal((B, H, S, D)) for _ in range(3))
        o = DeviceArray.zeros((B, H, S, D), bfloat16)
        fn = lambda: _lib.call("tessera_sm100_flash_attn_fwd_device", q.ptr, k.ptr, v.ptr, o.ptr, B, H, H, S,
                               S, D, ctypes.c_float(1 / np.sqrt(D)), 1, None)
    elif name == "attn_decode":
        B, Hq, Hkv, S, D = 16, 32, 8, 8192, 128
        q = dev_normal((B, Hq, 1, D))
        k, v = dev_normal((B, Hkv, S, D)), dev_normal((B, Hkv, S, D))
        o = DeviceArray.zeros((B, Hq, 1, D), bfloat16)
        lib = _lib.load()
        ns = lib.tessera_sm100_attn_decode_splits(B, Hq, Hkv, S)
        scr = DeviceArray((max(1, lib.tessera_sm100_attn_decode_scratch_bytes(B, Hq, ns)),), np.uint8)
        fn = lambda: _lib.call("tessera_sm100_attn_decode_device", q.ptr, k.ptr, v.ptr, o.ptr, B, Hq, Hkv, S,
                               D, ctypes.c_float(1 / np.sqrt(D)), ns, scr.ptr, None)
    elif name == "attn_decode_paged":
        B, Hq, Hkv, S, D, L = 16, 32, 8, 8192, 128, 64
        per_seq = S // L
        P = B * per_seq
        q = DeviceArray.from_host(rng.standard_normal((B, Hq, D), dtype=np.float32).astype(bfloat16))
        kp, vp = dev_normal((P, L, Hkv, D)), dev_normal((P, L, Hkv, D))
        table = DeviceArray.from_host(rng.permutation(P).astype(np.int32).reshape(B, per_seq))
        lens = DeviceArray.from_host(np.full(B, S, np.int32))
        o = DeviceArray.zeros((B, Hq, D), bfloat16)
        lib = _lib.load()
        ns = lib.tessera_sm100_attn_decode_splits(B, Hq, Hkv, S)
        scr = DeviceArray((max(1, lib.tessera_sm100_attn_decode_scratch_bytes(B, Hq, ns)),), np.uint8)
        fn = lambda: _lib.call("tessera_sm100_paged_attn_decode_device", q.ptr, kp.ptr, vp.ptr, table.ptr,
                               lens.ptr, o.ptr, B, Hq, Hkv, D, L, P, per_seq, S, ctypes.c_float(1 / np.sqrt(D)),
                               ns, scr.ptr, None)
    elif name == "gemm_fp8":
        n = 8192
        a8 = DeviceArray.from_host(rng.integers(0, 120, (n, n), dtype=np.uint8))      # e4m3 bytes, finite values
        b8 = DeviceArray.from_host(rng.integers(0, 120, (n, n), dtype=np.uint8))      # B given transposed [N, K]
        sa = DeviceArray.from_host(np.array([1e-3], np.float32))
        sb = DeviceArray.from_host(np.array([1e-3], np.float32))
        d = DeviceArray.zeros((n, n), bfloat16)
        fn = lambda: _lib.call("tessera_sm100_gemm_fp8_device", a8.ptr, b8.ptr, d.ptr, n, n, n, sa.ptr, sb.ptr,
                               _lib.BF16, None)
    elif name == "attn_backward":
        B, H, S, D = 2, 16, 4096, 128
        q, k, v, g = (dev_normal((B, H, S, D)) for _ in range(4))
        gq, gk, gv = (DeviceArray.zeros((B, H, S, D), bfloat16) for _ in range(3))
        ws = DeviceArray((int(_lib.load().tessera_sm100_flash_attn_bwd_bf16_workspace_bytes(B, H, S)),), np.uint8)
        fn = lambda: _lib.call("tessera_sm100_flash_attn_bwd_bf16_device", g.ptr, q.ptr, k.ptr, v.ptr, gq.ptr,
                               gk.ptr, gv.ptr, B, H, H, S, S, ctypes.c_float(1 / np.sqrt(D)), 1, ws.ptr, None)
    elif name == "attn_decode_int8":
        B, Hq, Hkv, S, D = 32, 32, 8, 8192, 128
        q = DeviceArray.from_host(rng.standard_normal((B, Hq, D), dtype=np.float32).astype(bfloat16))
        base = rng.integers(1, 256, (2, Hkv, S, D), dtype=np.uint8)
        kq = np.concatenate([base] * (B // 2))
        k, v = DeviceArray.from_host(kq), DeviceArray.from_host(np.roll(kq, 3, axis=2))
        ks = DeviceArray.from_host(rng.uniform(0.005, 0.03, (B, S)).astype(np.float32))
        vs = DeviceArray.from_host(rng.uniform(0.005, 0.03, (B, S)).astype(np.float32))
        o = DeviceArray.zeros((B, Hq, D), bfloat16)
        lib = _lib.load()
        ns = lib.tessera_sm100_attn_decode_int8_splits(B, Hq, Hkv, S)
        scr = DeviceArray((max(1, lib.tessera_sm100_attn_decode_scratch_bytes(B, Hq, ns)),), np.uint8)
        fn = lambda: _lib.call("tessera_sm100_attn_decode_int8_device", q.ptr, k.ptr, v.ptr, ks.ptr, vs.ptr, o.ptr,
                               B, Hq, Hkv, S, D, ctypes.c_float(1 / np.sqrt(D)), ns, scr.ptr, None)
    elif name == "moe":
        T, H, F, E, k = 2048, 4096, 14336, 2, 2
        x = dev_normal((T, H))
        logits = DeviceArray.from_host(rng.standard_normal((T, E), dtype=np.float32))
        wg, wu = dev_normal((E, H, F), 1 / np.sqrt(H)), dev_normal((E, H, F), 1 / np.sqrt(H))
        wd = dev_normal((E, F, H), 1 / np.sqrt(F))
        out = DeviceArray.zeros((T, H), bfloat16)
        ws = DeviceArray((_lib.load().tessera_sm100_moe_workspace_bytes(T, H, F, E, k),), np.uint8)
        fn = lambda: _lib.call("tessera_sm100_moe_layer_device", x.ptr, logits.ptr, wg.ptr, wu.ptr, wd.ptr,
                               out.ptr, T, H, F, E, k, 1, -1, _lib.BF16, _lib.BF16, ws.ptr, None)
    else:
        raise SystemExit(f"unknown profile case {name}")
    for _ in range(3):
        fn()
    device.synchronize()
    device.check_device_error("profile case")
    print(f"profile case {name}: 3 launches done")


# ------------------------------------------------------------------------------ main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="all", choices=["all", "gemm", "attn_prefill", "attn_backward", "attn_decode", "attn_decode_paged", "attn_decode_int8", "moe",
                             "moe_fp8"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--tp-mode", default="fused", choices=["fused", "nccl"],
                    help="N>1 GEMM: all-gather fused into the epilogue (peer TMA stores) or NCCL after it")
    ap.add_argument("--profile-case", default=None,
                    help="run three launches of one kernel on a small case and exit (for ncu)")
    args = ap.parse_args()
    if args.profile_case:
        profile_case(args.profile_case)
        return
    args.warmup = max(args.warmup, 3)

    if args.impl == "reference":
        run_reference(args)
        return

    if args.gpus > 1 and "WORLD_SIZE" not in os.environ:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29541", os.path.abspath(__file__)] + sys.argv[1:]
        sys.exit(subprocess.call(cmd))

    # NCCL writes its version/INFO lines to stdout by default; stdout carries the one JSON line.
    os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
    ranks = Ranks(args.gpus)
    from tessera_b200 import device
    device.set_device(ranks.local_rank)
    peaks, peak_kind = load_peaks()
    sampler = ClockSampler(ranks.local_rank)
    if ranks.rank == 0:
        sampler.start()
        time.sleep(0.3)

    g = bench_gemm(ranks, args, peaks, peak_kind, sampler)
    extras = {}
    if args.workload in ("all", "attn_prefill", "attn_backward", "attn_decode", "attn_decode_paged", "attn_decode_int8", "moe",
                         "moe_fp8"):
        for name, fn in (("attn_prefill", bench_attn_prefill), ("attn_backward", bench_attn_backward),
                         ("attn_decode", bench_attn_decode),
                         ("attn_decode_paged", bench_attn_decode_paged),
                         ("attn_decode_int8", bench_attn_decode_int8), ("moe", bench_moe),
                         ("moe_fp8", bench_moe_fp8)):
            if args.workload not in ("all", name):
                continue
            try:
                extras[name] = fn(ranks, args, peaks, peak_kind)
            except Exception as exc:
                extras[name] = {"error": f"{type(exc).__name__}: {exc}"}
    timed_marks, probe_marks = g.pop("clock_marks"), g.pop("probe_marks")
    clocks = None
    if ranks.rank == 0:
        under_load = sampler.summary(*probe_marks)
        in_steps = sampler.summary(*timed_marks)
        whole = sampler.summary()
        clocks = {"sm_mhz": under_load["sm_mhz"], "sm_max_mhz": under_load["sm_max_mhz"] or whole["sm_max_mhz"],
                  "reasons": sorted(set(under_load["reasons"]) | set(in_steps["reasons"]) | set(whole["reasons"])),
                  "samples": under_load["samples"],
                  "how": "median SM clock while the timed step runs back to back for 0.4 s right after the "
                         "timed region (one timed step is shorter than an nvidia-smi sample); reasons are the "
                         "union over the whole run",
                  "sm_mhz_during_timed_steps": in_steps["sm_mhz"], "samples_during_timed_steps": in_steps["samples"]}
    sampler.stop()

    cpu = None
    if ranks.rank == 0 and ranks.world == 1 and not args.no_cpu_baseline:
        cpu = cpu_gemm_baseline()

    if ranks.rank == 0:
        W = ranks.world
        line = {
            "metric": "bf16 GEMM TFLOP/s (M=N=K=8192)", "value": g["value"], "unit": "TFLOP/s",
            "n_gpus": W, "steps": args.steps, "warmup": args.warmup, "ms_per_step": g["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (seeded N(0,1)/sqrt(K) operands)",
            "config": {"workload": "gemm_bf16_8192: A[8192,8192] x B[8192,8192] -> Y bf16, fp32 accumulate",
                       "parallelism": "single GPU" if W == 1 else (
                           f"column-parallel tp{W}: W split on N, all-gather of Y fused into the GEMM "
                           f"epilogue (TMA stores into every rank's Y over NVLink)" if g["tp_mode"] == "fused"
                           else f"column-parallel tp{W}: W split on N, NCCL all-gather of Y + strided copies "
                                f"into row-major Y [{g['tp_mode']}]"),
                       "l2": "L2 flushed (256 MiB write) before every timed step, outside the event bracket",
                       "timing": "CUDA events per step on the launching stream, max over ranks, mean of steps"},
            "roofline": g["roofline"], "e2e": g["e2e"], "gpu_launches": g["gpu_launches"],
            "clocks": clocks, "check_max_rel_err": g["check_max_rel_err"], "workloads": extras,
        }
        if cpu:
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)
    ranks.close()


if __name__ == "__main__":
    main()
