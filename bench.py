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
``e2e`` is the same GEMM through the public host-operand call with pinned host buffers,
host<->device copies inside the timed region: ``tessera_b200.ops.gemm`` on one GPU,
``parallel.TensorParallelGemm.run_host`` on several (each rank uploads M/N rows of A and its block of
W, A is all-gathered over NVLink, the rank's block of Y comes back).

What was timed is checked: sampled outputs of every workload against the CPU reference on every
rank (``roofline.parity``); a mismatch is listed in ``parity_failures`` and the process exits 3.
``roofline.configs`` summarises configurations 1, 3, 4 and 5 (value, time, fraction of the roofline,
CPU value); with several GPUs ``roofline.exchange`` holds the exchange timed on its own, the GEMM
on its own and the step against the larger of the two.

``--impl reference`` times the reference's CPU implementation of the headline configuration (its
numpy path, restated in oracle/) on the host cores of this machine with every core's worth of BLAS
threads; single-GPU runs also time the CPU path of each configuration on a bounded sample
(``cpu_baseline`` of every workload).

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


def _all_host_threads_before_numpy():
    """The CPU legs (the reference arm, and the baselines of a single-GPU run) use every host core.
    torch.distributed.run exports OMP_NUM_THREADS=1 to its children, which would leave numpy's BLAS
    with one thread, so the thread counts are set here, before numpy is imported."""
    reference = any(a == "reference" or a == "--impl=reference" for a in sys.argv)
    if reference or int(os.environ.get("WORLD_SIZE", "1")) == 1:
        for var in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
            os.environ[var] = str(os.cpu_count() or 1)


_all_host_threads_before_numpy()

import numpy as np  # noqa: E402

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
WORKLOAD = "gemm_bf16_8192: A[8192,8192] x B[8192,8192] -> Y bf16, fp32 accumulate"
PARITY_TOL = 1e-2          # max|y - ref| / max|ref| in fp32, the stated parity tolerance
# Peer-store bandwidth of SM-issued stores measured on this pool (633-650 GB/s per direction with all
# ranks storing at once, profiles/column_exchange_8gpu.md): only the fallback denominator of the
# exchange floor; a multi-GPU run times the exchange itself.
PEER_STORE_GBS = 640.0


def blas_threads():
    """Threads numpy's BLAS will use, raised to all cores where the library allows it."""
    try:
        import threadpoolctl
        threadpoolctl.threadpool_limits(limits=os.cpu_count())
        info = threadpoolctl.threadpool_info()
        return max((int(i.get("num_threads", 1)) for i in info), default=1)
    except Exception:
        return int(os.environ.get("OMP_NUM_THREADS", "1"))

# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) from the ncu captures
# summarised under profiles/. The GEMM capture is the benchmark size itself; the attention and MoE
# captures ran a quarter-size case (heads, batch, experts x slots) and are scaled x4, the traffic
# of these kernels being proportional to those counts. The MoE figure is the sum of its two
# grouped GEMM launches.
NCU_TRAFFIC_BYTES = {"gemm_8192": 1.209e9, "attn_prefill": 1.005e9, "attn_decode": 2.171e9, "attn_decode_paged": 2.166e9,
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
    # Parity of what was just timed, on EVERY rank: sampled rows of its gathered Y against the fp32
    # product of the bf16 operands, over all columns, with the worst column block (one per
    # producing rank) reported separately.
    ranks.barrier()
    rows = [0, 255, 4097 + ranks.rank, n - 1]
    got = dY.download()[rows].astype(np.float32)
    ref = A[rows].astype(np.float32) @ B.astype(np.float32)
    scale = float(np.abs(ref).max())
    rel = float(np.abs(got - ref).max() / scale)
    blk = n // W
    worst_block = max(float(np.abs(got[:, r * blk:(r + 1) * blk] - ref[:, r * blk:(r + 1) * blk]).max() / scale)
                      for r in range(W))
    all_rel = ranks.gather(max(rel, worst_block))
    # kernel-only time for the roofline entry: at one GPU the step is the kernel; with several,
    # the GEMM without the exchange, timed the same way (before the clock probe heats the GPU)
    kernel_times = times if W == 1 else timed_steps(ranks, device, gemm_only, args.steps, args.warmup)
    # the exchange on its own (every rank storing its column block into the peers' Y, all at once):
    # the measured floor of the fused step on this machine
    exchange_ms = None
    if fused is not None:
        exchange_ms = statistics.mean(timed_steps(ranks, device, fused.exchange_only, args.steps, args.warmup))
    probe_marks = clock_probe(device, sampler, step)
    flops = 2.0 * n * n * n
    ms = statistics.mean(times)
    k_ms = statistics.mean(kernel_times)
    achieved = flops / W / k_ms / 1e9        # per-GPU kernel TFLOP/s

    # End to end through the public host-operand call with pinned buffers. One GPU: ops.gemm on the
    # whole problem. Several: A is replicated data, so each rank uploads M / W of its rows and its
    # own column block of W, the rows are all-gathered over NVLink, the fused GEMM runs and the
    # rank's block of Y comes back (TensorParallelGemm.run_host).
    e2e = None
    try:
        e2e_steps = max(2, min(args.steps, 5))
        if W == 1 or fused is None:
            pA, pB = PinnedArray((n, n), bfloat16), PinnedArray((n, nb), bfloat16)
            pY = PinnedArray((n, nb), bfloat16)
            pA.array[...] = A
            pB.array[...] = B[:, c0:c0 + nb]
            run = lambda: tessera.ops.gemm(pA.array, pB.array, out_dtype=bfloat16, out=pY.array)
            api = "tessera_b200.ops.gemm(host, host) -> tessera_sm100_gemm"
            note = "per rank: upload A and its column block of W, GEMM, download its block of Y"
            h2d = int(pA.nbytes + pB.nbytes)
        else:
            mb = n // W
            pA, pB = PinnedArray((mb, n), bfloat16), PinnedArray((n, nb), bfloat16)
            pY = PinnedArray((n, nb), bfloat16)
            pA.array[...] = A[ranks.rank * mb:(ranks.rank + 1) * mb]
            pB.array[...] = B[:, c0:c0 + nb]
            run = lambda: fused.run_host(pA.array, pB.array, pY.array, comm)
            api = "tessera_b200.parallel.TensorParallelGemm.run_host(host rows of A, host block of W) -> host block of Y"
            note = (f"per rank: upload M/{W} rows of A and its column block of W, all-gather A over NVLink (NCCL), "
                    f"fused GEMM + all-gather of Y, download its block of Y; bytes are the sum over ranks")
            h2d = int(pA.nbytes + pB.nbytes) * W
        run()
        ranks.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            run()
        device.synchronize()
        dt = (time.perf_counter() - t0) / e2e_steps
        dt = max(ranks.gather(dt))
        e2e_got = pY.array[rows].astype(np.float32)
        e2e_rel = float(np.abs(e2e_got - ref[:, c0:c0 + nb]).max() / scale)
        e2e = {"value": flops / dt / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": int(pY.nbytes) * (W if fused is not None and W > 1 else 1),
               "ms_per_step": dt * 1e3, "api": api, "note": note,
               "check_max_rel_err": max(ranks.gather(e2e_rel))}
    except Exception as exc:  # keep the headline even if pinned allocation fails
        e2e = {"value": None, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
               "error": f"{type(exc).__name__}: {exc}"}
    if comm:
        comm.close()
    roof = {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"],
            "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops"],
            "traffic": NCU_TRAFFIC_BYTES["gemm_8192"], "peak_kind": f"burst cuBLAS bf16, of {peak_kind}",
            "kernel_ms": k_ms, "kernel": ("gemm2_kernel<bf16> (tcgen05 cta_group::2, 256x256x64 per CTA pair, 6-stage TMA)"
                       if (n // 256) * (-(-nb // 256)) >= 74 else
                       "gemm_kernel<bf16,plain> (tcgen05 128x256x64, 4-stage TMA)")}
    if W > 1:
        # Every rank has to take in the other ranks' column blocks of Y over its NVLink ingress. The
        # floor is the exchange timed on its own just above (all ranks storing at once); the constant is
        # an earlier measurement on this pool, kept beside it for comparison.
        ingress = (W - 1) / W * n * n * 2
        floor_ms = exchange_ms if exchange_ms else ingress / (PEER_STORE_GBS * 1e9) * 1e3
        roof["exchange"] = {"ingress_bytes_per_rank": ingress,
                            "exchange_only_ms": exchange_ms,
                            "peer_store_gbs_measured": (ingress / exchange_ms / 1e6) if exchange_ms else None,
                            "peer_store_gbs_earlier_measurement": PEER_STORE_GBS,
                            "exchange_floor_ms": floor_ms, "compute_ms": k_ms,
                            "floor_ms": max(floor_ms, k_ms), "step_ms": ms,
                            "efficiency_vs_floor": max(floor_ms, k_ms) / ms,
                            "fused_kernel": "gemm_ag_kernel<bf16> (cta_group::2 256x256x64, TMA stores into every rank's Y; "
                                            "first wave of units split over K with at most four ranks)"
                                            if tp_mode == "fused" else None,
                            "note": "floor = max(the exchange alone, the GEMM alone); a perfectly overlapped step would "
                                    "take that long"}
    return {
        "value": flops / ms / 1e9, "ms_per_step": ms, "gpu_launches": int(launches * W),
        "roofline": roof,
        "e2e": e2e, "check_max_rel_err": max(all_rel), "check_per_rank": all_rel,
        "clock_marks": (m0, m1), "probe_marks": probe_marks,
        "tp_mode": tp_mode,
    }


def bench_gemm_batched(ranks, args, peaks, peak_kind):
    """Config 1: A[4,1024,1024] f16 x W[4,1024,1024] f16 -> Y f32, the case the reference runs on its
    CPU JIT path. Launch-bound on a B200 (3.8 us at the tensor peak): reported with its CPU time,
    not as a roofline target. With several GPUs every rank runs the same four products."""
    from oracle import tessera_oracle as orc
    from tessera_b200 import _lib, device
    from tessera_b200.device import DeviceArray
    rng = np.random.default_rng(1001)
    A = (rng.standard_normal((4, 1024, 1024), dtype=np.float32) / 32).astype(np.float16)
    Wt = (rng.standard_normal((4, 1024, 1024), dtype=np.float32) / 32).astype(np.float16)
    dA, dW = DeviceArray.from_host(A), DeviceArray.from_host(Wt)
    dY = DeviceArray.zeros((4, 1024, 1024), np.float32)
    fn = lambda: _lib.call("tessera_sm100_gemm_device", dA.ptr, dW.ptr, dY.ptr, 4, 1024, 1024, 1024, _lib.F16,
                           _lib.F32, None)
    times = timed_steps(ranks, device, fn, args.steps, args.warmup)
    ms = statistics.mean(times)
    flops = 2.0 * 4 * 1024 ** 3
    out = {"metric": "batched f16 GEMM 4 x 1024^3 -> f32, TFLOP/s", "value": flops / ms / 1e9, "unit": "TFLOP/s",
           "ms_per_step": ms, "config": "A[4,1024,1024] f16 x W[4,1024,1024] f16 -> Y f32, N(0,1)/sqrt(1024), seed 1001"
                                        + ("" if ranks.world == 1 else f" (replicated on {ranks.world} GPUs)"),
           "roofline": {"bound": "tensor", "achieved": flops / ms / 1e9, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                        "frac": flops / ms / 1e9 / peaks["bf16_tflops"], "traffic": None,
                        "peak_kind": f"burst cuBLAS bf16, of {peak_kind}; launch-bound size, not a roofline target"}}
    if ranks.rank == 0:
        blas_threads()
        ref = orc.gemm(A, Wt)
        t0 = time.perf_counter()
        reps = 5
        for _ in range(reps):
            orc.gemm(A, Wt)
        cpu_s = (time.perf_counter() - t0) / reps
        out["parity"] = {"max_rel_err": float(orc.max_rel_err(dY.download(), ref)), "tolerance": 1e-4}
        out["cpu_baseline"] = {"value": flops / cpu_s / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port",
                               "ms_per_step": cpu_s * 1e3,
                               "sample": f"{reps} x the whole configuration: fp32 matmul of the f16 operands "
                                         f"(numpy, {blas_threads()} BLAS threads), what the reference's CPU plan executes"}
    return out


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
    # parity of what was timed: two (batch, head) slices of this rank against the chunked fp32 reference
    from oracle import tessera_oracle as orc
    got = do.download()
    picks = [(0, 0), (B - 1, Hl - 1)]
    t0 = time.perf_counter()
    err = max(orc.max_rel_err(got[b:b + 1, h:h + 1], orc.flash_attn(q[b:b + 1, h:h + 1], k[b:b + 1, h:h + 1],
                                                                  v[b:b + 1, h:h + 1], causal=True)) for b, h in picks)
    cpu_s_per_head = (time.perf_counter() - t0) / len(picks)
    out = {"metric": "causal flash-attention forward TFLOP/s", "value": flops / ms / 1e9, "unit": "TFLOP/s",
           "ms_per_step": ms, "config": f"B={B} H={H} S={S} D={D} bf16 causal, heads sharded /{W}",
           "flops_convention": "4*B*H*S^2*D/2",
           "value_in_the_reference_benchmark_convention": {
               "value": 3.0 * B * H * S * S * D / ms / 1e9, "unit": "TFLOP/s",
               "convention": "3*B*H*S^2*D, what benchmarks/benchmark_attention.py:51-63 counts (no causal halving)"},
           "parity": {"max_rel_err": max(ranks.gather(float(err))), "tolerance": PARITY_TOL,
                      "sample": "2 (batch, head) slices per rank, all rows"},
           "roofline": {"bound": "tensor", "achieved": ach, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                        "frac": ach / peaks["bf16_tflops"], "traffic": NCU_TRAFFIC_BYTES["attn_prefill"],
                        "peak_kind": f"burst cuBLAS bf16, of {peak_kind}"}}
    if ranks.rank == 0 and W == 1 and not args.no_cpu_baseline:
        nthreads = blas_threads()
        out["cpu_baseline"] = {"value": flops / (cpu_s_per_head * B * H) / 1e12, "unit": "TFLOP/s",
                               "cores": os.cpu_count(), "kind": "port",
                               "seconds_for_the_whole_config_extrapolated": cpu_s_per_head * B * H,
                               "sample": f"{len(picks)} of {B * H} (batch, head) slices through the chunked numpy reference "
                                         f"(the reference's own form materialises a 17 GB score tensor), {nthreads} BLAS "
                                         f"threads, x{B * H // len(picks)} extrapolation"}
    return out


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
    from oracle import tessera_oracle as orc
    got = do.download()
    picks = [0, Bl - 1]
    t0 = time.perf_counter()
    err = max(orc.max_rel_err(got[b:b + 1], orc.gqa_attention(q[b:b + 1], k[b:b + 1], v[b:b + 1], Hq, Hkv)) for b in picks)
    cpu_s_per_seq = (time.perf_counter() - t0) / len(picks)
    out = {"metric": "GQA decode attention GB/s (K+V bytes)", "value": nbytes / ms / 1e6, "unit": "GB/s",
           "ms_per_step": ms, "config": f"batch={B} Hq={Hq} Hkv={Hkv} KV={S} D={D} bf16, batch sharded /{W}",
           "splits": ns,
           "parity": {"max_rel_err": max(ranks.gather(float(err))), "tolerance": PARITY_TOL,
                      "sample": "2 sequences per rank, all heads"},
           "roofline": {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                        "frac": ach / peaks["hbm_gbs"], "traffic": NCU_TRAFFIC_BYTES["attn_decode"],
                        "peak_kind": f"copy bandwidth, of {peak_kind}"}}
    if ranks.rank == 0 and W == 1 and not args.no_cpu_baseline:
        out["cpu_baseline"] = {"value": nbytes / (cpu_s_per_seq * B) / 1e9, "unit": "GB/s", "cores": os.cpu_count(),
                               "kind": "port", "seconds_for_the_whole_config_extrapolated": cpu_s_per_seq * B,
                               "sample": f"{len(picks)} of {B} sequences through the numpy reference (KV heads repeated x"
                                         f"{Hq // Hkv}, then attention in fp32), {blas_threads()} BLAS threads, "
                                         f"x{B // len(picks)} extrapolation"}
    return out


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
    from types import SimpleNamespace
    from oracle import tessera_oracle as orc
    from tessera_b200 import _lib, device, parallel
    from tessera_b200.device import DeviceArray, bfloat16
    T, H, F, E, k = 8192, 4096, 14336, 8, 2
    W = ranks.world
    rng = np.random.default_rng(1005)
    x = rng.standard_normal((T, H), dtype=np.float32).astype(bfloat16)
    logits = rng.standard_normal((T, E), dtype=np.float32)
    Ep = E // W
    # Expert e's matrices are one seeded N(0,1)/sqrt(fan-in) draw per kind rolled by 7e columns, so any
    # rank can rebuild any expert for the parity check without holding all 2.8 GB on the host.
    wrng = np.random.default_rng(2005)
    base_g = (wrng.standard_normal((H, F), dtype=np.float32) / np.sqrt(H)).astype(bfloat16)
    base_u = (wrng.standard_normal((H, F), dtype=np.float32) / np.sqrt(H)).astype(bfloat16)
    base_d = (wrng.standard_normal((F, H), dtype=np.float32) / np.sqrt(F)).astype(bfloat16)
    expert = lambda base, e: np.roll(base, 7 * e, axis=1)
    mine = range(ranks.rank * Ep, (ranks.rank + 1) * Ep)
    dwg = DeviceArray.from_host(np.stack([expert(base_g, e) for e in mine]))
    dwu = DeviceArray.from_host(np.stack([expert(base_u, e) for e in mine]))
    dwd = DeviceArray.from_host(np.stack([expert(base_d, e) for e in mine]))
    flops = 3 * 2.0 * T * k * H * F
    Tl = T // W
    sl = slice(ranks.rank * Tl, (ranks.rank + 1) * Tl)
    moe = None
    if W == 1:
        dx, dl = DeviceArray.from_host(x), DeviceArray.from_host(logits)
        out = DeviceArray.zeros((T, H), bfloat16)
        ws = DeviceArray((_lib.load().tessera_sm100_moe_workspace_bytes(T, H, F, E, k),), np.uint8)
        fn = lambda: _lib.call("tessera_sm100_moe_layer_device", dx.ptr, dl.ptr, dwg.ptr, dwu.ptr, dwd.ptr,
                               out.ptr, T, H, F, E, k, 1, -1, _lib.BF16, _lib.BF16, ws.ptr, None)
        mode = "single GPU"
    else:
        dxl = DeviceArray.from_host(x[sl])
        dll = DeviceArray.from_host(np.ascontiguousarray(logits[sl]))
        out = DeviceArray.zeros((Tl, H), bfloat16)
        moe = parallel.DeviceExpertParallelMoE(SimpleNamespace(world=W, rank=ranks.rank), ranks.gather, dwg, dwu,
                                               dwd, Tl, k, E)
        fn = lambda: moe.forward(dxl, dll, out=out)
        mode = (f"expert-parallel /{W}: token rows stored into the owners' buffers and results read back over "
                f"NVLink by the kernels, ranks ordered by flags in peer memory (no collective)")
    ranks.barrier()
    l0 = device.launch_count()
    steps, warm = max(2, args.steps // 2), min(args.warmup, 3)
    times = timed_steps(ranks, device, fn, steps, warm)
    launches = (device.launch_count() - l0) // (steps + warm)
    ms = statistics.mean(times)
    # Parity of what was timed, on every rank: routing bit-exact against the reference's router on
    # the same logits, and sampled tokens against the fp32 reference (hidden activation in bf16).
    route = orc.route_tokens(logits, k, True)
    if W == 1:
        views = [ctypes_void() for _ in range(8)]
        _lib.call("tessera_sm100_moe_workspace_views", ws.ptr, T, H, F, E, k, *[v_ref(v) for v in views])
        assign = DeviceArray((T, k), np.int32, ptr=views[0].value).download()
    else:
        assign = moe.assignment.download()
    routing_ok = bool(np.array_equal(assign, route.assignment[sl].astype(np.int32)))
    got = out.download().astype(np.float32)
    toks = [0, Tl // 2 + ranks.rank, Tl - 1]
    ref = np.zeros((len(toks), H), np.float32)
    xf = x.astype(np.float32)
    t0 = time.perf_counter()
    for i, t in enumerate(toks):
        g = ranks.rank * Tl + t
        for j in range(k):
            e = int(route.assignment[g, j])
            h = orc.silu_mul(xf[g] @ expert(base_g, e).astype(np.float32), xf[g] @ expert(base_u, e).astype(np.float32))
            h = h.astype(bfloat16).astype(np.float32)
            ref[i] += route.weights[g, j] * (h @ expert(base_d, e).astype(np.float32))
    err = float(np.abs(got[toks] - ref).max() / np.abs(ref).max())
    code = device.consume_device_error()[0]
    if moe is not None:
        ranks.barrier()
        moe.close()
    ach = flops / W / ms / 1e9
    res = {"metric": "MoE FFN layer TFLOP/s (routed slots, unpadded)", "value": flops / ms / 1e9,
           "unit": "TFLOP/s", "ms_per_step": ms, "gpu_launches_per_step": int(launches), "device_error": code,
           "config": f"T={T} H={H} F={F} E={E} top-{k} bf16, {mode}",
           "parity": {"max_rel_err": max(ranks.gather(err)), "routing_bit_exact": all(ranks.gather(routing_ok)),
                      "tolerance": PARITY_TOL, "sample": "3 tokens per rank, all columns; assignment of every local token"},
           "roofline": {"bound": "tensor", "achieved": ach, "peak": peaks["bf16_tflops_sustained"],
                        "unit": "TFLOP/s", "frac": ach / peaks["bf16_tflops_sustained"],
                        "traffic": NCU_TRAFFIC_BYTES["moe"],
                        "peak_kind": f"sustained cuBLAS bf16 (two multi-ms GEMMs per step), of {peak_kind}"}}
    if ranks.rank == 0 and W == 1 and not args.no_cpu_baseline:
        # the reference layer on a token subset (every expert still gets ~T/64 rows), extrapolated
        nthreads = blas_threads()
        sub = 1024
        wg_all = np.stack([expert(base_g, e) for e in range(E)]).astype(np.float32)
        wu_all = np.stack([expert(base_u, e) for e in range(E)]).astype(np.float32)
        wd_all = np.stack([expert(base_d, e) for e in range(E)]).astype(np.float32)
        t0 = time.perf_counter()
        orc.moe_layer_from_logits(xf[:sub], logits[:sub], wg_all, wu_all, wd_all, k)
        cpu_s = time.perf_counter() - t0
        res["cpu_baseline"] = {"value": flops * (sub / T) / cpu_s / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count(),
                               "kind": "port", "seconds_for_the_whole_config_extrapolated": cpu_s * T / sub,
                               "sample": f"the numpy reference layer (route, stable expert sort, three grouped fp32 GEMMs "
                                         f"per expert, weighted combine) on the first {sub} of {T} tokens, {nthreads} BLAS "
                                         f"threads, x{T // sub} extrapolation"}
    return res


def ctypes_void():
    import ctypes
    return ctypes.c_void_p()


def v_ref(v):
    import ctypes
    return ctypes.byref(v)


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
    nthreads = blas_threads()
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
            "blas_threads": nthreads,
            "sample": f"{reps} x full 8192^3 fp32 matmul of bf16-rounded operands (numpy, {nthreads} BLAS threads), "
                      f"{dt:.2f} s each", "seconds_per_step": dt}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import tessera_oracle as orc
    nthreads = blas_threads()
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
            "data": "synthetic (seeded N(0,1)/sqrt(K) operands)",
            "config": {"workload": WORKLOAD},
            "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port",
                             "blas_threads": nthreads,
                             "sample": f"each step = the full 8192^3 product: the reference's tessera.ops.gemm "
                                       f"(np.matmul) on fp32 arrays holding bf16 values, {nthreads} BLAS threads on "
                                       f"{os.cpu_count()} host cores"},
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
    elif name == "gemm_allgather":
        # the per-rank shape of the 4-GPU column-parallel GEMM with all four copies of Y on this GPU
        n, world = 8192, 4
        a, b = dev_normal((n, n), 1 / np.sqrt(n)), dev_normal((n, n), 1 / np.sqrt(n))
        ys = [DeviceArray.zeros((n, n), bfloat16) for _ in range(world)]
        ptrs = (ctypes.c_void_p * world)(*[y.ptr for y in ys])
        fn = lambda: _lib.call("tessera_sm100_gemm_allgather_device", a.ptr, b.ptr, ptrs, world, 1, n, n, n,
                               _lib.BF16, _lib.BF16, None)
    elif name == "mma_rate":
        # issue rate of tcgen05.mma on resident operands (no kernel of the hot path; prints a table)
        print("tcgen05.mma kind::f16 bf16, K 16, M 128 per CTA, 4000 MMAs per issuing CTA, all SMs at once")
        for pair, N, mn in ((0, 256, 1), (0, 128, 1), (0, 64, 1), (1, 256, 1), (1, 128, 1), (0, 256, 0), (0, 128, 0),
                            (1, 256, 0), (1, 128, 0)):
            cyc = ctypes.c_double(0)
            _lib.call("tessera_sm100_probe_mma_rate", pair, N, mn, 1000, ctypes.byref(cyc))
            print(f"  {'cta_group::2 M256' if pair else 'cta_group::1 M128'} N{N:3d} B {'MN' if mn else 'K '}-major: "
                  f"{cyc.value:6.1f} cycles per MMA (arithmetic at 4096 FMA/clk/SM: {128 * N * 16 / 4096:5.1f})")
        device.check_device_error("mma_rate")
        return
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
    ap.add_argument("--workload", default="all", choices=["all", "gemm", "gemm_batched", "attn_prefill", "attn_backward", "attn_decode",
                                                          "attn_decode_paged", "attn_decode_int8", "moe", "moe_fp8"])
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
    for name, fn in (("gemm_batched", bench_gemm_batched), ("attn_prefill", bench_attn_prefill),
                     ("attn_backward", bench_attn_backward), ("attn_decode", bench_attn_decode),
                     ("attn_decode_paged", bench_attn_decode_paged),
                     ("attn_decode_int8", bench_attn_decode_int8), ("moe", bench_moe),
                     ("moe_fp8", bench_moe_fp8)):
        if args.workload not in ("all", name):
            continue
        try:
            extras[name] = fn(ranks, args, peaks, peak_kind)
        except Exception as exc:
            extras[name] = {"error": f"{type(exc).__name__}: {exc}"}
        # every rank takes part in every workload: if one failed, say so on all of them
        errors = [e for e in ranks.gather(extras[name].get("error")) if e]
        if errors and "error" not in extras[name]:
            extras[name] = {"error": f"another rank failed: {errors[0]}"}
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

    # Parity gate: a wrong result makes the run fail, whatever the throughput.
    parity = {"tp_gemm" if ranks.world > 1 else "gemm": g["check_max_rel_err"]}
    failures = []
    if not (g["check_max_rel_err"] < PARITY_TOL):
        failures.append(f"gemm: max rel err {g['check_max_rel_err']:.3g} on some rank (per rank {g['check_per_rank']})")
    e2e_err = (g["e2e"] or {}).get("check_max_rel_err")
    if e2e_err is not None and not (e2e_err < PARITY_TOL):
        failures.append(f"gemm e2e: max rel err {e2e_err:.3g}")
    for name, key in (("gemm_batched", "gemm_batched"), ("attn_prefill", "attn_prefill"), ("attn_decode", "attn_decode"),
                      ("moe", "ep_moe" if ranks.world > 1 else "moe")):
        w = extras.get(name) or {}
        if "error" in w:
            failures.append(f"{name}: {w['error']}")
        par = w.get("parity")
        if par:
            parity[key] = par["max_rel_err"]
            if not (par["max_rel_err"] < par.get("tolerance", PARITY_TOL)):
                failures.append(f"{name}: max rel err {par['max_rel_err']:.3g}")
            if par.get("routing_bit_exact") is False:
                failures.append(f"{name}: routing differs from the reference router")
            if "routing_bit_exact" in par:
                parity[key + "_routing_bit_exact"] = par["routing_bit_exact"]
    if ranks.rank == 0:
        W = ranks.world
        roof = g["roofline"]
        roof["parity"] = parity
        roof["configs"] = {}
        for cfg, name in (("cfg1_batched_f16_gemm", "gemm_batched"), ("cfg3_causal_prefill", "attn_prefill"),
                          ("cfg4_gqa_decode", "attn_decode"), ("cfg5_moe_layer", "moe")):
            w = extras.get(name) or {}
            if "value" in w:
                entry = {"value": w["value"], "unit": w["unit"], "ms_per_step": w["ms_per_step"],
                         "frac": (w.get("roofline") or {}).get("frac"), "bound": (w.get("roofline") or {}).get("bound")}
                if "cpu_baseline" in w:
                    entry["cpu_value"] = w["cpu_baseline"]["value"]
                    entry["cpu_cores"] = w["cpu_baseline"]["cores"]
                roof["configs"][cfg] = entry
        line = {
            "metric": "bf16 GEMM TFLOP/s (M=N=K=8192)", "value": g["value"], "unit": "TFLOP/s",
            "n_gpus": W, "steps": args.steps, "warmup": args.warmup, "ms_per_step": g["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (seeded N(0,1)/sqrt(K) operands)",
            "config": {"workload": WORKLOAD,
                       "parallelism": "single GPU" if W == 1 else (
                           f"column-parallel tp{W}: W split on N, all-gather of Y fused into the GEMM "
                           f"epilogue (TMA stores into every rank's Y over NVLink)" if g["tp_mode"] == "fused"
                           else f"column-parallel tp{W}: W split on N, NCCL all-gather of Y + strided copies "
                                f"into row-major Y [{g['tp_mode']}]"),
                       "l2": "L2 flushed (256 MiB write) before every timed step, outside the event bracket",
                       "timing": "CUDA events per step on the launching stream, max over ranks, mean of steps"},
            "roofline": roof, "e2e": g["e2e"], "gpu_launches": g["gpu_launches"],
            "clocks": clocks, "check_max_rel_err": g["check_max_rel_err"], "parity_failures": failures,
            "workloads": extras,
        }
        if cpu:
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)
    ranks.close()
    if failures:
        sys.stderr.write("parity check failed: " + "; ".join(failures) + "\n")
        sys.exit(3)


if __name__ == "__main__":
    main()
