"""A small, self-contained run of the fused training step, sized for profiler captures.

    python -m weta_b200.profile_case --batch 512 --steps 2

Runs the wide CNN step at a reduced batch (activations of a few hundred MB: larger than the L2 so DRAM
counters mean something, small enough that a multi-pass capture ends by itself).  Used as the target
command of the ncu captures summarised under profiles/.
"""
import argparse

import numpy as np

from .backend import B200Backend
from .core import manual_seed
from .trainer import FusedTrainer, cnn_specs
from .workloads import WIDE_CNN, synthetic_batch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=512)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--mode", type=int, default=1, help="0 = 3xTF32, 1 = TF32, 2 = FP32")
    args = ap.parse_args()
    be = B200Backend(0)
    cfg = WIDE_CNN
    manual_seed(42)
    tr = FusedTrainer(be, cnn_specs(cfg), args.batch, (cfg.in_ch, cfg.hw, cfg.hw), matmul_mode=args.mode)
    tr.init_from_global_rng()
    x, y = synthetic_batch(cfg, args.batch, 0, 0, be)
    tr.stage(x.numpy(), y.numpy())
    for _ in range(args.steps):
        tr.forward_backward()
        tr.adam_step()
    print("loss", tr.loss(), "launches", be.launch_count())
    be.gemm_check()
    tr.close()


if __name__ == "__main__":
    main()
