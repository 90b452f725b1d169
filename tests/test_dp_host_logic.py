"""CPU-only, world_size 2 over gloo: the host side of the data-parallel step.

The collective is injected (gloo stands where NCCL or the peer-memory kernel stands on GPUs); what is under test is the
library's bucket plan (wb_dp_plan_buckets), the shard arithmetic of the sharded optimizer (sum, Adam on this rank's
1/world of each bucket, gather of the parameters) against all-reduce + full Adam, and the host watchdog loop
(wb_watchdog_wait) with a rank that does not join a collective."""
import os
import socket
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # spawned ranks re-import this file

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from weta_b200.backend import load_library
from weta_b200.trainer import plan_buckets, watchdog_wait

# per-layer arena ranges, last layer first, every tensor padded to 32 elements like the trainer's arena
RANGES = [(0, 32), (32, 512), (544, 96), (640, 416)]


def test_bucket_plan_merges_adjacent_ranges():
    lib = load_library()
    assert plan_buckets(lib, [(0, 10), (10, 30), (40, 70), (110, 5), (115, 0), (200, 10)], 100) == [(0, 110), (110, 5), (200, 10)]
    assert plan_buckets(lib, RANGES, 256) == [(0, 544), (544, 512)]
    assert plan_buckets(lib, RANGES, 1) == [(0, 32), (32, 512), (544, 96), (640, 416)]
    assert plan_buckets(lib, [], 100) == []


def _adam(theta, g, m, v, t, lr=1e-3, b1=0.9, b2=0.999, eps=1e-8):
    f = np.float32
    m[:] = m * f(b1) + g * f(1 - b1)
    v[:] = v * f(b2) + (g * g) * f(1 - b2)
    den = np.sqrt(v) * f(1.0 / np.sqrt(1 - b2 ** t)) + f(eps)
    theta[:] = theta - (m / den) * f(lr / (1 - b1 ** t))


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lib = load_library()
    n = RANGES[-1][0] + RANGES[-1][1]
    buckets = plan_buckets(lib, RANGES, 256)
    rng = np.random.default_rng(100 + rank)
    theta0 = np.random.default_rng(7).standard_normal(n).astype(np.float32)  # same replica on every rank
    ok = True
    # reference: all-reduce the whole arena, Adam over everything on every rank
    th_a, m_a, v_a = theta0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
    # sharded: per bucket, sum, Adam on this rank's shard only, gather the parameters
    th_s, m_s, v_s = theta0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
    for t in (1, 2, 3):
        g_local = rng.standard_normal(n).astype(np.float32)
        total = torch.from_numpy(g_local.copy())
        dist.all_reduce(total, op=dist.ReduceOp.SUM)
        g_avg = total.numpy() * np.float32(1.0 / world)
        _adam(th_a, g_avg, m_a, v_a, t)
        for off, ln in buckets:
            assert ln % (4 * world) == 0 and off % 4 == 0
            shard = ln // world
            lo = off + rank * shard
            summed = torch.from_numpy(g_local[off:off + ln].copy())
            dist.all_reduce(summed, op=dist.ReduceOp.SUM)  # stands for the reduce-scatter: only [lo, lo + shard) is used
            g = summed.numpy()[rank * shard:(rank + 1) * shard] * np.float32(1.0 / world)
            _adam(th_s[lo:lo + shard], g, m_s[lo:lo + shard], v_s[lo:lo + shard], t)
            parts = [torch.zeros(shard) for _ in range(world)]
            dist.all_gather(parts, torch.from_numpy(th_s[lo:lo + shard].copy()))
            th_s[off:off + ln] = torch.cat(parts).numpy()
        ok = ok and np.array_equal(th_s, th_a)
    lo_hi = [(off + rank * (ln // world), off + (rank + 1) * (ln // world)) for off, ln in buckets]
    own = np.concatenate([np.arange(a, b) for a, b in lo_hi])
    ok = ok and np.array_equal(m_s[own], m_a[own]) and np.array_equal(v_s[own], v_a[own])
    out[rank] = bool(ok)
    dist.barrier()
    dist.destroy_process_group()


def _spawn(target, world=2, timeout=120):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Manager().dict()
    procs = [ctx.Process(target=target, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
        assert p.exitcode == 0
    return out


def test_sharded_optimizer_equals_all_reduce_then_adam():
    out = _spawn(_worker)
    assert out[0] and out[1]


def _watchdog_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lib = load_library()
    buf = torch.ones(1024)
    if rank == 1:
        time.sleep(3.0)  # this rank joins the collective far too late
        dist.all_reduce(buf)
        out[rank] = True
    else:
        work = dist.all_reduce(buf, async_op=True)
        t0 = time.time()
        status = watchdog_wait(lib, lambda: 0 if work.is_completed() else 1, timeout_ms=1000, interval_us=2000)
        waited = time.time() - t0
        message = lib.wb_last_error().decode()
        work.wait()  # the late rank arrives; both leave together
        out[rank] = status == 6 and 0.9 < waited < 2.5 and "1000 ms" in message  # WB_ERR_TIMEOUT, not a hang
        # and a collective every rank joins finishes inside the limit
    buf2 = torch.ones(8)
    work2 = dist.all_reduce(buf2, async_op=True)
    status2 = watchdog_wait(lib, lambda: 0 if work2.is_completed() else 1, timeout_ms=5000, interval_us=500)
    out[rank] = out[rank] and status2 == 0 and float(buf2[0]) == world
    dist.barrier()
    dist.destroy_process_group()


def test_watchdog_reports_a_rank_that_never_joins_instead_of_hanging():
    out = _spawn(_watchdog_worker)
    assert out[0] and out[1]
