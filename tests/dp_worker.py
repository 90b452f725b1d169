"""One rank of the multi-GPU data-parallel tests (run as a child process by tests/test_gpu_dp.py).

    python dp_worker.py <scenario> <rank> <world> <exchange dir>

The rendezvous id travels through a file in the exchange directory.  Every rank runs all of its steps and leaves
only between steps, with none of its kernels in flight; nothing here faults or hangs a GPU: the `timeout` scenario
makes a bounded device-side wait run out (a flag that no rank sets) and checks the status it reports."""
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import numpy as np

from weta_b200 import core
from weta_b200.backend import B200Backend, BackendError
from weta_b200.core import DType, Layout, manual_seed
from weta_b200.trainer import DP_MODE_NAMES, DataParallelTrainer, FusedTrainer, cnn_specs, make_dp_id
from weta_b200.workloads import CnnConfig, synthetic_batch_device

CFG = CnnConfig("cnn-dp-test", 3, 16, 128, 32, 64)
PER_RANK_BATCH = 16
STEPS = 3


def exchange_id(be, rank, path):
    if rank == 0:
        blob = make_dp_id(be.lib)
        with open(path + ".tmp", "wb") as f:
            f.write(blob)
        os.replace(path + ".tmp", path)
        return blob
    for _ in range(600):
        if os.path.exists(path):
            return open(path, "rb").read()
        time.sleep(0.05)
    raise RuntimeError("rank 0 never published the rendezvous id")


def stage(tr, be, step, rank):
    x, y = synthetic_batch_device(CFG, PER_RANK_BATCH, step, rank, be)
    n_in = PER_RANK_BATCH * CFG.in_ch * CFG.hw * CFG.hw
    hx = be.to_host(x, Layout.contiguous([n_in]), DType.F32)
    hy = be.to_host(y, Layout.contiguous([PER_RANK_BATCH]), DType.I64)
    tr.stage(hx, hy)


def run_mode(be, rank, world, xdir, mode, matmul_mode, tag):
    manual_seed(42)  # one model seed shared by all ranks
    tr = FusedTrainer(be, cnn_specs(CFG), PER_RANK_BATCH, (CFG.in_ch, CFG.hw, CFG.hw), lr=1e-3, matmul_mode=matmul_mode)
    tr.init_from_global_rng()
    dp = DataParallelTrainer(tr, rank, world, exchange_id(be, rank, os.path.join(xdir, f"id_{tag}")), mode=mode, bucket_elems=1 << 14)
    losses = []
    for step in range(STEPS):
        stage(tr, be, step, rank)
        dp.step()
        dp.wait(20000)
        losses.append(tr.loss())
    params = np.concatenate([tr.get_param(i) for i in range(len(tr.ranges))])
    rm, rv = tr.bn_buffers(1)
    used = dp.mode
    n_buckets = len(dp.buckets)
    be.gemm_check()
    dp.close()
    tr.close()
    return {"mode": used, "buckets": n_buckets, "losses": losses}, params, rm, rv


def scenario_parity(be, rank, world, xdir):
    out = {}
    for mode in (1, 2, 3):
        for matmul_mode, mm in ((2, "fp32"), (1, "tf32")):
            tag = f"{DP_MODE_NAMES[mode]}_{mm}"
            info, params, rm, rv = run_mode(be, rank, world, xdir, mode, matmul_mode, tag)
            out[tag] = info
            np.savez(os.path.join(xdir, f"rank{rank}_{tag}.npz"), params=params, running_mean=rm, running_var=rv)
    json.dump(out, open(os.path.join(xdir, f"rank{rank}.json"), "w"))


def scenario_timeout(be, rank, world, xdir):
    """Both ranks take two steps together; then rank 1 stops stepping (it stays alive, idle, until rank 0 is done).  Rank
    0's third step finds no `gradients-ready` flag from rank 1: its bounded wait gives up after the limit set in
    WETA_B200_DP_TIMEOUT_MS, the step's kernels all return, and wb_dp_wait reports WB_ERR_TIMEOUT."""
    manual_seed(42)
    tr = FusedTrainer(be, cnn_specs(CFG), PER_RANK_BATCH, (CFG.in_ch, CFG.hw, CFG.hw), lr=1e-3, matmul_mode=2)
    tr.init_from_global_rng()
    dp = DataParallelTrainer(tr, rank, world, exchange_id(be, rank, os.path.join(xdir, "id_timeout")), mode=3, bucket_elems=1 << 14)
    result = {"mode": dp.mode}
    for step in range(2):
        stage(tr, be, step, rank)
        dp.step()
        dp.wait(20000)
    done_flag = os.path.join(xdir, "rank0_done")
    if rank == 0:
        stage(tr, be, 2, rank)
        t0 = time.time()
        status, message = 0, ""
        try:
            dp.step()
            dp.wait(0)
        except BackendError as e:
            status, message = e.status, str(e)
        result.update(status=status, message=message, seconds=time.time() - t0)
        # the context is still usable: an ordinary operation runs and returns the right answer
        probe = be.from_host(np.arange(8, dtype=np.float32))
        result["probe_ok"] = bool(np.array_equal(be.to_host(probe, Layout.contiguous([8]), DType.F32), np.arange(8, dtype=np.float32)))
        open(done_flag, "w").write("done")
    else:
        for _ in range(1200):
            if os.path.exists(done_flag):
                break
            time.sleep(0.05)
        result["waited_for_rank0"] = os.path.exists(done_flag)
    json.dump(result, open(os.path.join(xdir, f"rank{rank}.json"), "w"))
    dp.close()
    tr.close()


def main():
    scenario, rank, world, xdir = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), sys.argv[4]
    be = B200Backend(rank)
    {"parity": scenario_parity, "timeout": scenario_timeout}[scenario](be, rank, world, xdir)
    be.close()


if __name__ == "__main__":
    main()
