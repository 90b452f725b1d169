"""The data-parallel step (include/weta_b200.h, wb_dp_*) on GPUs.

One-GPU cases: the bucketed per-bucket-Adam order against forward_backward + adam_step (bit for bit), the
peer-memory kernel against sum-then-Adam on local stand-ins for the replicas, the bounded device-side wait.
Two-GPU cases (skipped with fewer devices) run each rank as a child process: every exchange mode against the oracle
doing the ranks' shards one after the other and averaging the gradients (the reference has no multi-GPU path; its
step test is crates/weta/tests/cuda_parity.rs:230-273), and a rank that stops stepping."""
import ctypes
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from oracle.mirror import nn
from oracle.mirror.autograd import Var
from oracle.mirror.models import build_cnn, synthetic_batch
from oracle.mirror.tensor import Tensor
from weta_b200 import core
from weta_b200.backend import device_count
from weta_b200.core import DType, manual_seed
from weta_b200.trainer import DataParallelTrainer, FusedTrainer, _declare, _declare_dp, cnn_specs
from weta_b200.workloads import CnnConfig

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
FP32, TF32 = 2, 1


def _steps(gpu, use_dp, cfg, batch, steps, bucket_elems=1 << 10):
    manual_seed(11)
    tr = FusedTrainer(gpu, cnn_specs(cfg), batch, (cfg.in_ch, cfg.hw, cfg.hw), lr=1e-3, matmul_mode=FP32)
    tr.init_from_global_rng()
    dp = DataParallelTrainer(tr, 0, 1, None, bucket_elems=bucket_elems) if use_dp else None
    rng = np.random.default_rng(3)
    losses = []
    for _ in range(steps):
        tr.stage(rng.random((batch, cfg.in_ch, cfg.hw, cfg.hw)).astype(np.float32), rng.integers(0, 10, batch))
        if dp:
            dp.step()
            dp.wait()
        else:
            tr.forward_backward()
            tr.adam_step()
        losses.append(tr.loss())
    params = np.concatenate([tr.get_param(i) for i in range(len(tr.ranges))])
    buckets = list(dp.buckets) if dp else []
    if dp:
        dp.close()
    tr.close()
    return losses, params, buckets


def test_per_bucket_adam_equals_adam_after_backward_bit_for_bit(gpu):
    """One rank, buckets forced small: each bucket's Adam runs on the side stream as soon as backward has finished the
    bucket, the next step waits for the last one; losses and parameters equal the plain order exactly."""
    cfg = CnnConfig("tiny", 3, 8, 8, 16, 32)
    plain = _steps(gpu, False, cfg, 16, 4)
    bucketed = _steps(gpu, True, cfg, 16, 4)
    assert len(bucketed[2]) >= 3, bucketed[2]
    assert bucketed[0] == plain[0]
    assert np.array_equal(bucketed[1], plain[1])


@pytest.mark.parametrize("world", [2, 4, 8])
def test_reduce_adam_broadcast_equals_sum_then_adam(gpu, world):
    """The peer-mode kernel with `world` local buffers standing for as many replicas (each world size takes a different
    unrolling of the kernel): shard r of the range is owned by "rank" r.  Afterwards every parameter buffer holds what
    wb_adam_step gives on the gradient sum scaled by 1/world.  The shard length is not a multiple of the threads per
    round, so the last round of every variant is a partial one."""
    lib = gpu.lib
    _declare(lib)
    _declare_dp(lib)
    n = world * (1024 * 300 + 64)
    rng = np.random.default_rng(9)
    theta0 = rng.standard_normal(n).astype(np.float32)
    grads = [rng.standard_normal(n).astype(np.float32) * s for s in (1.0, 0.5, 2.0, 1e-3, 3.0, 0.25, 1e2, 1.5)[:world]]
    gsum = grads[0].copy()
    for g in grads[1:]:
        gsum = gsum + g  # index order, f32
    P = ctypes.c_void_p
    want_t, want_g = Tensor.from_numpy(theta0, gpu), Tensor.from_numpy(gsum, gpu)
    want_m, want_v = Tensor.from_numpy(np.zeros(n, np.float32), gpu), Tensor.from_numpy(np.zeros(n, np.float32), gpu)
    thetas = [Tensor.from_numpy(theta0, gpu) for _ in range(world)]
    gts = [Tensor.from_numpy(g, gpu) for g in grads]
    ms = [Tensor.from_numpy(np.zeros(n, np.float32), gpu) for _ in range(world)]
    vs = [Tensor.from_numpy(np.zeros(n, np.float32), gpu) for _ in range(world)]
    gp = (P * world)(*[t.storage.ptr for t in gts])
    tp = (P * world)(*[t.storage.ptr for t in thetas])
    shard = n // world
    assert shard % 4 == 0
    for t in (1, 2):
        gpu.check(lib.wb_adam_step(gpu.handle, P(want_t.storage.ptr), P(want_g.storage.ptr), P(want_m.storage.ptr), P(want_v.storage.ptr), n, t,
                                   1e-3, 0.9, 0.999, 1e-8, 0.0, 0, 1.0 / world))
        for r in range(world):
            gpu.check(lib.wb_reduce_adam_broadcast(gpu.handle, gp, tp, world, r, r * shard, shard, P(ms[r].storage.ptr), P(vs[r].storage.ptr), t,
                                                   1e-3, 0.9, 0.999, 1e-8, 0.0, 0, 1.0 / world))
        for r in range(world):
            assert np.array_equal(thetas[r].numpy(), want_t.numpy()), (t, r)
            lo, hi = r * shard, (r + 1) * shard
            assert np.array_equal(ms[r].numpy()[lo:hi], want_m.numpy()[lo:hi]) and np.array_equal(vs[r].numpy()[lo:hi], want_v.numpy()[lo:hi])
    # misaligned or ragged ranges are refused, not mis-read
    assert lib.wb_reduce_adam_broadcast(gpu.handle, gp, tp, world, 0, 2, 8, P(ms[0].storage.ptr), P(vs[0].storage.ptr), 1, 1e-3, 0.9, 0.999, 1e-8, 0.0,
                                        0, 1.0) == 1


def test_bounded_device_wait_runs_out_and_leaves_the_context_usable(gpu):
    """A wait on a flag that nothing sets: the kernel gives up after the limit and reports through its status word
    (WB_ERR_TIMEOUT); the same wait with the flag already set passes; ordinary work runs afterwards."""
    import time

    lib = gpu.lib
    _declare_dp(lib)
    t0 = time.time()
    assert lib.wb_dp_selftest_wait(gpu.handle, 300, 0) == 6
    assert 0.25 < time.time() - t0 < 3.0
    assert b"ran out" in lib.wb_last_error()
    assert lib.wb_dp_selftest_wait(gpu.handle, 300, 1) == 0
    x = Tensor.from_numpy(np.arange(16, dtype=np.float32), gpu)
    assert np.array_equal(x.add(x).numpy(), 2 * np.arange(16, dtype=np.float32))


def _run_ranks(scenario, world, tmp_path, extra_env=None, timeout=900):
    env = dict(os.environ)
    env.update({"NCCL_NVLS_ENABLE": "0", "WETA_B200_DP_TIMEOUT_MS": "20000"})
    env.update(extra_env or {})
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "dp_worker.py"), scenario, str(r), str(world), str(tmp_path)], env=env,
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()
            o, _ = p.communicate()
        outs.append(o)
    for r, p in enumerate(procs):
        assert p.returncode == 0, f"rank {r} exited with {p.returncode}:\n{outs[r][-3000:]}"
    return [json.load(open(os.path.join(tmp_path, f"rank{r}.json"))) for r in range(world)]


def _oracle_data_parallel(oracle, cfg, per_rank, world, steps):
    """What N ranks compute, on the CPU: every rank's shard through the same replica one after the other, gradients
    summed in rank order and scaled by 1/N, one Adam step.  All ranks draw the same dropout seeds (one host seed), so the
    generator is rewound for each shard.  Rank 0's BatchNorm buffers are the ones kept."""
    ref = build_cnn(cfg, oracle, 42)
    opt = nn.Adam(ref.parameters(), 1e-3)
    losses = [[] for _ in range(world)]
    for step in range(steps):
        state = core.global_rng().state
        saved = [(b, b.numpy().copy()) for _, b in ref.buffers()]
        total = None
        for rank in reversed(range(world)):  # rank 0 last: its running statistics stay
            core.global_rng().state = state
            if rank == 0:
                for b, v in saved:
                    b.assign(Tensor.from_numpy(v, oracle))
            x, y = synthetic_batch(cfg, per_rank, step, rank, oracle)
            loss = nn.cross_entropy(ref(Var(x)), y)
            opt.zero_grad()
            loss.backward()
            losses[rank].append(loss.item())
            g = [p.grad.numpy().copy() for p in ref.parameters()]
            total = g if total is None else [a + b for a, b in zip(g, total)]  # (g0 + g1): rank order for two ranks
        for p, g in zip(ref.parameters(), total):
            p.grad = Tensor.from_numpy(g * np.float32(1.0 / world), oracle)
        opt.step()
    return ref, losses


def _adam_params_close(name, got, want, steps, lr, frac_allowed):
    d = np.abs(got.astype(np.float64) - want.astype(np.float64))
    assert d.max() <= 2 * steps * lr * 1.01, f"{name}: max |diff| {d.max()}"
    frac = float((d > 1e-5 + 1e-4 * np.abs(want)).mean())
    assert frac < frac_allowed, f"{name}: {frac:.2%} of elements differ by more than 1e-5"


@pytest.mark.skipif(device_count() < 2, reason="needs two GPUs")
def test_two_ranks_match_the_oracle_in_every_exchange_mode(oracle, tmp_path, report):
    from dp_worker import CFG, PER_RANK_BATCH, STEPS

    infos = _run_ranks("parity", 2, tmp_path)
    # which mode actually ran (PEER needs the ranks to map each other's memory; it may have fallen back to SHARDED)
    modes = {tag: infos[0][tag]["mode"] for tag in infos[0]}
    report("two-rank data-parallel modes", modes=modes, losses={tag: [infos[r][tag]["losses"] for r in range(2)] for tag in infos[0]})
    assert modes["allreduce_fp32"] == 1 and modes["sharded_fp32"] == 2
    assert all(infos[r][tag]["buckets"] >= 3 for r in range(2) for tag in infos[0])
    load = lambda r, tag: np.load(os.path.join(tmp_path, f"rank{r}_{tag}.npz"))
    for mm in ("fp32", "tf32"):
        base = load(0, f"allreduce_{mm}")["params"]
        for tag in (f"allreduce_{mm}", f"sharded_{mm}", f"peer_{mm}"):
            # both ranks hold the same parameters, and with two ranks (a two-term sum is order-free) all modes agree exactly
            assert np.array_equal(load(0, tag)["params"], load(1, tag)["params"]), tag
            assert np.array_equal(load(0, tag)["params"], base), tag
            assert infos[0][tag]["losses"] == infos[0][f"allreduce_{mm}"]["losses"], tag
    # against the oracle (FP32 contractions on both sides)
    ref, losses = _oracle_data_parallel(oracle, CFG, PER_RANK_BATCH, 2, STEPS)
    for r in range(2):
        for a, b in zip(infos[r]["allreduce_fp32"]["losses"], losses[r]):
            assert abs(a - b) < 2e-4, (r, infos[r]["allreduce_fp32"]["losses"], losses[r])
    got = load(0, "allreduce_fp32")["params"]
    off = 0
    for n, p in ref.named_parameters():
        want = p.numpy().reshape(-1)
        mine = got[off:off + want.size]
        off += want.size
        if n in ("0.bias", "4.bias"):  # conv bias before BatchNorm: zero true gradient, Adam steps on rounding noise
            assert np.abs(mine - want).max() <= 2 * STEPS * 1e-3 * 1.01
        else:
            _adam_params_close(n, mine, want, STEPS, 1e-3, 2e-2)
    bufs = dict(ref.buffers())
    assert np.allclose(load(0, "allreduce_fp32")["running_var"], bufs["5.running_var"].numpy(), rtol=1e-3, atol=1e-5)


@pytest.mark.skipif(device_count() < 2, reason="needs two GPUs")
def test_a_rank_that_stops_stepping_gives_a_timeout_not_a_hang(tmp_path, report):
    infos = _run_ranks("timeout", 2, tmp_path, {"WETA_B200_DP_TIMEOUT_MS": "1000"}, timeout=300)
    report("two-rank timeout", rank0=infos[0])
    if infos[0]["mode"] != 3:
        pytest.skip("the ranks could not map each other's memory; the peer-memory mode did not run")
    assert infos[0]["status"] == 6, infos[0]  # WB_ERR_TIMEOUT
    assert "gave up waiting for rank 1" in infos[0]["message"]
    assert infos[0]["seconds"] < 30 and infos[0]["probe_ok"]
    assert infos[1]["waited_for_rank0"]
