"""Benchmark of the hot path: CNN train samples/s on 1/2/4/8 B200, plus the roofline of its dominant kernel.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference --steps 2 --warmup 1      # the CPU path, on the host cores

Workload: the data-parallel wide CNN (conv 3->128 + BN + ReLU + pool, conv 128->256 + BN + ReLU + pool,
dropout, fc 16384->1024, ReLU, dropout, fc 1024->10; 17.1 M parameters), synthetic 3x32x32 images in
[0,1) and uniform labels standing in for CIFAR-10 (no dataset is available offline), global batch 4096
split evenly over the ranks, f32 storage with TF32 tensor-core contractions, Adam lr 1e-3, one model
seed shared by all ranks.  A step is forward + cross-entropy + backward + gradient all-reduce + Adam.

One JSON line is printed by rank 0.  `value` times the step with inputs already resident in HBM;
`e2e` times the same step through the host-facing C-ABI calls (wb_dp_submit / wb_dp_step_submitted) with pinned host
buffers: upload of the batch and read-back of the loss inside the timed region.  Each timed pass of K steps is repeated
(--repeats, default 5); `value` and `e2e` are the medians, the spread and the SM clock of each leg are on the line.
Multi-GPU plumbing (rendezvous, barrier, max over ranks) is torch.distributed over gloo; the gradient exchange itself
is the library's (NCCL or its peer-memory kernel, include/weta_b200.h wb_dp_*).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

GLOBAL_BATCH = 4096
METRIC = "cnn_train_samples_per_s"


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([f.strip() for f in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        mhz, mx, reasons = [], None, set()
        for s in self.samples:
            if len(s) < 6:
                continue
            try:
                mhz.append(float(s[0]))
                mx = float(s[1])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(mhz)}


WORKLOAD = "data-parallel wide CNN train step (conv3-128, conv128-256, fc16384-1024-10; BN, ReLU, maxpool, dropout 0.25)"


def cpu_reference_run(steps: int, warmup: int, sample_batch: int):
    """The reference's CPU path (the oracle restating weta-cpu, driven op by op like the reference's
    own autograd would) on a bounded sample of the workload, with every host thread."""
    from oracle.cpu_backend import OracleBackend
    from oracle.mirror import nn
    from oracle.mirror.models import build_cnn, primitive_train_step, synthetic_batch
    from weta_b200.workloads import WIDE_CNN

    be = OracleBackend()
    be.set_num_threads(os.cpu_count() or 1)  # a launcher may have exported OMP_NUM_THREADS=1 for its ranks
    model = build_cnn(WIDE_CNN, be, 42)
    opt = nn.Adam(model.parameters(), 1e-3)
    batches = [synthetic_batch(WIDE_CNN, sample_batch, s, 0, be) for s in range(2)]
    for s in range(warmup):
        primitive_train_step(model, opt, *batches[s % 2])
    t0 = time.perf_counter()
    for s in range(steps):
        primitive_train_step(model, opt, *batches[s % 2])
    dt = time.perf_counter() - t0
    return {"value": sample_batch * steps / dt, "unit": "samples/s", "cores": be.num_threads(), "kind": "port",
            "sample": f"{steps} step(s) of the same wide CNN at batch {sample_batch} (of 4096), primitive-call stream on the C++ "
                      f"restatement of weta-cpu, OpenMP over {be.num_threads()} threads", "ms_per_step": dt / steps * 1e3}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = max(1, min(args.steps, 3)), max(1, min(args.warmup, 1))
    r = cpu_reference_run(steps, warmup, args.cpu_batch)
    line = {"impl": "reference", "metric": METRIC, "value": r["value"], "unit": "samples/s", "n_gpus": args.gpus, "steps": steps, "warmup": warmup,
            "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "global_batch": args.global_batch, "image": "3x32x32", "optimizer": "Adam lr 1e-3",
                       "sample": f"each step is one optimizer step on a {args.cpu_batch}-sample batch of this workload (a bounded sample: a full "
                                 f"{args.global_batch}-sample step takes minutes on the host cores); samples/s is what is compared"},
            "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": r["value"], "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def load_traffic():
    """DRAM bytes per launch (ncu dram__bytes_read.sum + dram__bytes_write.sum) of the trainer's ops at batch 512: lines
    "label bytes" in the capture summary kept beside the other profiler summaries."""
    path = os.path.join(ROOT, "profiles", "dram_traffic_trainer_batch512.txt")
    out = {}
    if os.path.exists(path):
        for line in open(path):
            parts = line.split()
            if len(parts) == 2 and not line.startswith("#"):
                out[parts[0]] = float(parts[1])
    return out


def median(xs):
    xs = sorted(xs)
    return xs[len(xs) // 2] if len(xs) % 2 else 0.5 * (xs[len(xs) // 2 - 1] + xs[len(xs) // 2])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--repeats", type=int, default=5, help="timed passes of --steps steps each; the line reports their median")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--cpu-batch", type=int, default=32, help="sample batch of the CPU baseline")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--global-batch", type=int, default=GLOBAL_BATCH)
    ap.add_argument("--dp-mode", default="auto", choices=["auto", "allreduce", "sharded", "peer"], help="gradient exchange of the data-parallel step")
    ap.add_argument("--bucket-elems", type=int, default=1 << 20)
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)

    import ctypes

    import torch
    import torch.distributed as dist

    from weta_b200.backend import B200Backend
    from weta_b200.core import DType, Layout, manual_seed
    from weta_b200.trainer import DP_MODE_NAMES, DataParallelTrainer, FusedTrainer, cnn_specs, make_dp_id
    from weta_b200.workloads import WIDE_CNN, synthetic_batch_device

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}"
    assert args.warmup >= 3, "at least 3 warm-up steps"
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("gloo")  # host-side plumbing only: rendezvous id, barriers, max over ranks
    cfg = WIDE_CNN
    gb = args.global_batch
    assert gb % world == 0
    batch = gb // world

    # The compute stream outranks the library's side streams (exchange, optimizer, upload), which are created at the
    # lowest priority: when both have blocks ready the step's own kernels are scheduled first.
    stream = torch.cuda.Stream(priority=-1)
    be = B200Backend(local, stream=stream.cuda_stream)
    manual_seed(42)  # one model seed shared by all ranks
    tr = FusedTrainer(be, cnn_specs(cfg), batch, (cfg.in_ch, cfg.hw, cfg.hw), lr=1e-3, matmul_mode=1)
    tr.init_from_global_rng()
    dp_id = None
    if world > 1:
        box = [make_dp_id(be.lib) if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        dp_id = box[0]
    mode = {"auto": 0, "allreduce": 1, "sharded": 2, "peer": 3}[args.dp_mode]
    dp = DataParallelTrainer(tr, rank, world, dp_id, mode=mode, bucket_elems=args.bucket_elems)

    # Synthetic batches: drawn on the device from the counter RNG, then copied to pinned host memory for
    # the end-to-end leg.  Two distinct batches alternate.
    n_in = batch * cfg.in_ch * cfg.hw * cfg.hw
    dev_batches, host_batches = [], []
    for s in range(2):
        x, y = synthetic_batch_device(cfg, batch, s, rank, be)
        dev_batches.append((x, y))
        hx = torch.empty(n_in, dtype=torch.float32, pin_memory=True)
        hy = torch.empty(batch, dtype=torch.int64, pin_memory=True)
        hx.copy_(torch.from_numpy(be.to_host(x, Layout.contiguous([n_in]), DType.F32)))
        hy.copy_(torch.from_numpy(be.to_host(y, Layout.contiguous([batch]), DType.I64)))
        host_batches.append((hx, hy))

    def stage_from_device(i):
        # the batch is already in HBM: the step reads it where it lies (two batches alternate)
        x, y = dev_batches[i % 2]
        be.check(be.lib.wb_trainer_set_input(tr.handle, ctypes.c_void_p(x.ptr), ctypes.c_void_p(y.ptr)))

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        """K steps bracketed by barrier + synchronize, timed with CUDA events on the compute stream; max over ranks."""
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(steps):
            fn(i)
        e1.record(stream)
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    def resident_step(i):
        stage_from_device(i)
        dp.step()

    losses = []
    pending = [0]

    # End to end: every step's batch is copied from pinned host memory inside the timed region; the copy of batch
    # i + 1 is in flight while step i computes (two device slots), and every step ends with the loss read-back.
    def e2e_step(i):
        if pending[0] == 0:
            dp.submit(host_batches[i % 2][0].data_ptr(), host_batches[i % 2][1].data_ptr())
            pending[0] += 1
        dp.submit(host_batches[(i + 1) % 2][0].data_ptr(), host_batches[(i + 1) % 2][1].data_ptr())
        losses.append(dp.step_submitted())

    def drain_e2e():
        while pending[0] > 0:  # a pass leaves one batch submitted ahead; step on it so the slots start empty again
            dp.step_submitted()
            pending[0] -= 1

    # ---- warm-up ------------------------------------------------------------------------------
    for i in range(args.warmup):
        resident_step(i)
    dp.wait()
    be.gemm_check()

    # ---- value: inputs resident in HBM ----------------------------------------------------------
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = be.launch_count()
    value_passes = [timed(resident_step, args.steps) for _ in range(args.repeats)]
    launches = (be.launch_count() - launches0) // args.repeats
    clocks = sampler.stop() if rank == 0 else None
    total_ms = median(value_passes)
    value = gb * args.steps / (total_ms / 1e3)

    # ---- roofline pass: the same K steps with an event pair around every trainer op ---------------
    # (the ~90 extra event records per step open small gaps between kernels, so `value` comes from the passes above)
    tr.set_timing(True)
    dp.set_timing(True)
    tr.timing_report()
    timed_ops_ms = timed(resident_step, args.steps)
    op_times = tr.timing_report()
    bucket_calls, bucket_ms = dp.timing_report()
    tr.set_timing(False)
    dp.set_timing(False)

    # ---- e2e: through the host-facing calls -------------------------------------------------------
    be.check(be.lib.wb_trainer_set_input(tr.handle, None, None))
    e2e_step(0)
    pending[0] = 1
    e2e_step(1)
    sampler2 = ClockSampler(local)
    if rank == 0:
        sampler2.start()
    e2e_passes = []
    for _ in range(args.repeats):
        e2e_passes.append(timed(e2e_step, args.steps))
    e2e_clocks = sampler2.stop() if rank == 0 else None
    drain_e2e()
    e2e_ms = median(e2e_passes)
    e2e_value = gb * args.steps / (e2e_ms / 1e3)
    dp.wait()
    be.gemm_check()
    dp_mode_used = DP_MODE_NAMES.get(dp.mode, str(dp.mode)) if world > 1 else "none (one rank)"

    if rank != 0:
        dp.close()
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel --------------------------------------------------------
    peaks = load_peaks()
    hw1, hw2 = cfg.hw * cfg.hw, (cfg.hw // 2) ** 2
    fc_in = cfg.c2 * (hw2 // 4)
    act1, act2 = 4.0 * batch * cfg.c1 * hw1, 4.0 * batch * cfg.c2 * hw2      # bytes of each conv output
    in1, in2 = 4.0 * batch * cfg.in_ch * hw1, 4.0 * batch * cfg.c1 * hw2     # bytes of each conv input
    work = {  # per launch, per rank: ("tensor", algorithmic 2*M*N*K flops) or ("hbm", algorithmic bytes moved)
        # conv1 contracts over 27 values per output: its two GEMMs are bound by writing / reading the 128-channel
        # activation (act1) plus the 27-row im2col matrix (9 x the input), not by the tensor cores
        # conv1's weight gradient is fused with the block's BatchNorm+ReLU+pool backward: it reads the activation, the
        # pooled gradient and the im2col matrix and writes nothing of that size
        "L0.conv_fwd_gemm": ("hbm", act1 + 9.0 * in1), "L0.conv_wgrad_gemm": ("hbm", act1 * 1.25 + 9.0 * in1),
        "L1.conv_fwd_gemm": ("tensor", 2.0 * batch * cfg.c2 * cfg.c1 * 9 * hw2), "L1.conv_wgrad_gemm": ("tensor", 2.0 * batch * cfg.c2 * cfg.c1 * 9 * hw2),
        "L1.conv_dgrad_gemm": ("tensor", 2.0 * batch * cfg.c2 * cfg.c1 * 9 * hw2),
        "L3.linear_fwd_gemm": ("tensor", 2.0 * batch * cfg.hidden * fc_in), "L3.linear_wgrad_gemm": ("tensor", 2.0 * batch * cfg.hidden * fc_in),
        "L3.linear_dgrad_gemm": ("tensor", 2.0 * batch * cfg.hidden * fc_in),
        "L5.linear_fwd_gemm": ("tensor", 2.0 * batch * cfg.classes * cfg.hidden), "L5.linear_wgrad_gemm": ("tensor", 2.0 * batch * cfg.classes * cfg.hidden),
        "L5.linear_dgrad_gemm": ("tensor", 2.0 * batch * cfg.classes * cfg.hidden),
        "L0.im2col": ("hbm", in1 * 10), "L1.im2col": ("hbm", in2 * 10), "L1.col2im": ("hbm", in2 * 10),
        # BN+ReLU+pool forward: the statistics come from the convolution's epilogue, so x is read once and x/4 written;
        # block 0 also writes the two column-shifted copies of its output that block 1's implicit GEMM reads.
        # Backward: the sums pass reads the pooled output and the pooled gradient (x/4 each), the dx pass reads x and
        # dy/4 and writes dx (no shifted copies of dx: block 1's input gradient applies the horizontal moves to its result).
        "L0.bn_relu_pool_fwd": ("hbm", act1 * 1.75), "L1.bn_relu_pool_fwd": ("hbm", act2 * 1.25),
        # (block 0: only the sums pass is left under this label; its dx pass lives in L0.conv_wgrad_gemm)
        "L0.bn_relu_pool_bwd": ("hbm", act1 * 0.5), "L1.bn_relu_pool_bwd": ("hbm", act2 * 2.75),
        "L2.dropout_fwd": ("hbm", 8.0 * batch * fc_in), "L2.dropout_bwd": ("hbm", 8.0 * batch * fc_in),
        "L4.dropout_fwd": ("hbm", 8.0 * batch * cfg.hidden), "L4.dropout_bwd": ("hbm", 12.0 * batch * cfg.hidden),
        "L6.adam": ("hbm", 28.0 * tr.arena_len),
    }
    # DRAM bytes per launch from the ncu capture at batch 512 (a full-size step is too large to capture); every one of
    # these ops streams its tensors once per image, so the traffic is scaled by batch / 512.
    ncu_traffic_batch512 = load_traffic()
    shares = {k: round(v[1] / timed_ops_ms, 4) for k, v in sorted(op_times.items(), key=lambda kv: -kv[1][1])}
    top_name, (top_calls, top_ms) = max(op_times.items(), key=lambda kv: kv[1][1])
    tf32_peak = peaks["bf16_tflops_sustained"] / 2.0
    per_op = {}
    for k, (calls, ms) in op_times.items():
        if k in work:
            kind, amount = work[k]
            rate = amount / (ms / calls * 1e-3)
            per_op[k] = {"bound": kind, "achieved": rate / (1e12 if kind == "tensor" else 1e9), "unit": "TFLOP/s" if kind == "tensor" else "GB/s",
                         "frac": rate / (tf32_peak * 1e12 if kind == "tensor" else peaks["hbm_gbs"] * 1e9), "avg_ms": ms / calls}
    if top_name in per_op:
        o = per_op[top_name]
        roofline = {"kernel": top_name, "bound": o["bound"], "achieved": o["achieved"], "peak": tf32_peak if o["bound"] == "tensor" else peaks["hbm_gbs"],
                    "unit": o["unit"], "frac": o["frac"],
                    "traffic": ncu_traffic_batch512[top_name] * batch / 512.0 if top_name in ncu_traffic_batch512 else None,
                    "traffic_note": "bytes per launch: ncu dram read+write at batch 512, scaled by batch/512",
                    "algorithmic": work[top_name][1], "avg_ms_per_launch": o["avg_ms"], "launches": top_calls,
                    "peak_note": (f"{peaks['source']} sustained bf16 cuBLAS rate / 2 (TF32 issues at half the bf16 rate)" if o["bound"] == "tensor"
                                  else f"{peaks['source']} copy bandwidth")}
    else:
        roofline = {"kernel": top_name, "bound": "hbm", "achieved": None, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": None, "traffic": None,
                    "avg_ms_per_launch": top_ms / top_calls, "launches": top_calls}
    gemm_ms = sum(v[1] for k, v in op_times.items() if k in work and work[k][0] == "tensor")
    gemm_flops = sum(work[k][1] * v[0] for k, v in op_times.items() if k in work and work[k][0] == "tensor")
    roofline["all_contractions_tflops"] = gemm_flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else None
    roofline["per_op"] = {k: {"bound": v["bound"], "achieved": round(v["achieved"], 1), "frac": round(v["frac"], 3), "ms": round(v["avg_ms"], 4)}
                          for k, v in per_op.items()}
    roofline["side_stream_ms_per_step"] = round(bucket_ms / max(args.steps, 1), 4)  # exchange + optimizer of all buckets (overlaps backward)

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        r = cpu_reference_run(2, 1, args.cpu_batch)
        cpu = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")}

    def with_product(c, ms_per_step):
        c = dict(c or {})
        c["ms_per_step_x_sm_mhz"] = round(ms_per_step * c["sm_mhz"], 1) if c.get("sm_mhz") else None
        return c

    line = {
        "metric": METRIC, "value": value, "unit": "samples/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32 (TF32 contractions)",
        "data": "synthetic",
        "config": {"workload": WORKLOAD,
                   "global_batch": gb, "per_gpu_batch": batch, "image": "3x32x32", "params": cfg.num_params(), "optimizer": "Adam lr 1e-3",
                   "parallelism": f"dp{world}", "gradient_exchange": dp_mode_used, "buckets": len(dp.buckets),
                   "l2": "per-step working set is several GB, far larger than the 126 MB L2; two batches alternate",
                   "step": "upload/stage + forward + cross-entropy + backward + gradient exchange + Adam",
                   "timing": f"value / e2e: median of {args.repeats} passes of K steps each, every pass bracketed by barrier + synchronize and timed "
                             "with CUDA events on the compute stream, max over ranks; roofline / op_time_shares: the same K steps timed once more with "
                             "an event pair around every op; e2e: batch i+1 uploaded from pinned memory while step i runs, loss read back every step"},
        "repeats": {"passes": args.repeats, "value_ms_per_step": [round(p / args.steps, 4) for p in value_passes],
                    "value_min_max": [gb * args.steps / (max(value_passes) / 1e3), gb * args.steps / (min(value_passes) / 1e3)],
                    "e2e_ms_per_step": [round(p / args.steps, 4) for p in e2e_passes],
                    "e2e_min_max": [gb * args.steps / (max(e2e_passes) / 1e3), gb * args.steps / (min(e2e_passes) / 1e3)]},
        "e2e": {"value": e2e_value, "unit": "samples/s", "ms_per_step": e2e_ms / args.steps, "h2d_bytes_per_step": n_in * 4 + batch * 8,
                "d2h_bytes_per_step": 4, "last_loss": losses[-1], "clocks": with_product(e2e_clocks, e2e_ms / args.steps)},
        "gpu_launches": int(launches), "clocks": with_product(clocks, total_ms / args.steps), "roofline": roofline, "op_time_shares": shares,
        "train_tflops": cfg.train_flops_per_sample() * value / 1e12,
    }
    if cpu is not None:
        line["cpu_baseline"] = cpu
    print(json.dumps(line), flush=True)
    dp.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
