"""World-size-2 and -4 CPU runs (torch.distributed, gloo) of the multi-GPU host logic: the
expert-parallel planning/sequencing of tessera_b200.parallel with a numpy compute backend, and
the column-parallel GEMM partition. The same classes run on GPUs with NCCL and the CUDA kernels.
Equivalence bar: distributed == single device (tests/unit/test_megamoe_distributed.py:34-42)."""
import multiprocessing as mp
import os
import socket

import numpy as np
import pytest

from oracle import tessera_oracle as orc
from tessera_b200 import parallel


class _NumpyBackend:
    def __init__(self, wg, wu, wd):
        self.wg, self.wu, self.wd = wg, wu, wd

    def route(self, logits, top_k, normalize):
        r = orc.route_tokens(logits, top_k, normalize)
        return r.assignment.astype(np.int32), r.weights

    def gather_rows(self, rows, index):
        return np.asarray(rows)[np.asarray(index, np.int64)]

    def expert_ffn(self, rows, group_offsets):
        return orc.moe_swiglu_block(rows, self.wg, self.wu, self.wd, np.diff(group_offsets))

    def combine(self, rows, slot_of, weights, num_tokens):
        out = np.zeros((num_tokens, rows.shape[1]), np.float32)
        for j in range(slot_of.shape[1]):
            s = slot_of[:, j]
            ok = s >= 0
            out[ok] += weights[ok, j, None] * rows[s[ok]]
        return out


class _GlooTransport:
    def __init__(self, dist):
        self.dist, self.rank, self.world = dist, dist.get_rank(), dist.get_world_size()

    def all_gather_small(self, arr):
        out = [None] * self.world
        self.dist.all_gather_object(out, np.asarray(arr))
        return np.stack(out)

    def exchange_rows(self, rows, send_counts, recv_counts):
        chunks = np.split(np.asarray(rows), np.cumsum(send_counts)[:-1])
        everyone = [None] * self.world
        self.dist.all_gather_object(everyone, chunks)
        mine = [everyone[src][self.rank] for src in range(self.world)]
        assert [len(m) for m in mine] == [int(c) for c in recv_counts]
        return np.concatenate(mine, axis=0)


def _worker(rank, world, port, q):
    try:
        import torch.distributed as dist
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
        rng = np.random.default_rng(77)                     # identical on every rank
        T, H, F, E, k = 64, 16, 24, 8, 2
        x = orc.round_to_storage(rng.standard_normal((T, H)), "bf16")
        logits = rng.standard_normal((T, E)).astype(np.float32)
        wg = orc.round_to_storage(rng.standard_normal((E, H, F)) / 4, "bf16")
        wu = orc.round_to_storage(rng.standard_normal((E, H, F)) / 4, "bf16")
        wd = orc.round_to_storage(rng.standard_normal((E, F, H)) / 5, "bf16")
        Tl, Ep = T // world, E // world
        sl = slice(rank * Tl, (rank + 1) * Tl)
        es = slice(rank * Ep, (rank + 1) * Ep)
        moe = parallel.ExpertParallelMoE(E, k, _GlooTransport(dist), _NumpyBackend(wg[es], wu[es], wd[es]))
        y_local = moe.forward(x[sl], logits[sl])
        ref = orc.moe_layer_from_logits(x, logits, wg, wu, wd, k)[0]
        err_moe = float(np.abs(y_local - ref[sl]).max())
        # column-parallel GEMM: Y = all_gather(A @ W_r, axis=1)
        A = rng.standard_normal((12, 20)).astype(np.float32)
        W = rng.standard_normal((20, 16)).astype(np.float32)
        c0, nb = parallel.tp_column_range(16, world, rank)
        parts = [None] * world
        dist.all_gather_object(parts, A @ W[:, c0:c0 + nb])
        err_tp = float(np.abs(np.concatenate(parts, axis=1) - A @ W).max())
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, err_moe, err_tp, None))
    except Exception as exc:  # surfaced by the parent
        q.put((rank, None, None, repr(exc)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_and_tensor_parallel_equal_single_device(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, err_moe, err_tp, exc in results:
        assert exc is None, f"rank {rank}: {exc}"
        assert err_moe < 1e-4 and err_tp < 1e-5


def test_plans_are_consistent():
    rng = np.random.default_rng(3)
    E, world, k, Tl = 8, 4, 2, 50
    plans, counts = [], []
    assigns = []
    for r in range(world):
        a = orc.route_tokens(rng.standard_normal((Tl, E)).astype(np.float32), k).assignment
        a[rng.integers(0, Tl, 5), rng.integers(0, k, 5)] = -1          # some dropped slots
        assigns.append(a)
        p = parallel.ep_plan(a, E, world, r)
        plans.append(p)
        counts.append(p.send_expert_counts)
        assert p.send_counts.sum() == (a >= 0).sum()
        kept = p.slot_of_assignment >= 0
        np.testing.assert_array_equal(kept, a >= 0)
        # sent rows are ordered by expert, token-major inside an expert
        e_sent = a.reshape(-1)[np.argsort(np.where(kept.reshape(-1), p.slot_of_assignment.reshape(-1), 1 << 30))][:kept.sum()]
        assert np.all(np.diff(e_sent) >= 0)
    allc = np.stack(counts)
    for r in range(world):
        rp = parallel.ep_recv_plan(allc, r)
        assert rp.recv_counts.sum() == rp.group_offsets[-1]
        np.testing.assert_array_equal(np.sort(rp.to_grouped), np.arange(rp.group_offsets[-1]))
        np.testing.assert_array_equal(rp.to_grouped[rp.from_grouped], np.arange(rp.group_offsets[-1]))
        np.testing.assert_array_equal(rp.recv_counts, [plans[s].send_counts[r] for s in range(world)])
    with pytest.raises(ValueError):
        parallel.ep_plan(assigns[0], 7, world, 0)
    with pytest.raises(ValueError):
        parallel.tp_column_range(10, 4, 0)
