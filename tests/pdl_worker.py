"""One run of the fused trainer for tests/test_gpu_fused.py::test_programmatic_dependent_launch_changes_no_result
(a child process, because the library reads WETA_B200_NO_PDL once per process).

    python pdl_worker.py <mlp|cnn|wide>

Prints one JSON line: the losses of six steps and a SHA-256 of every parameter after them."""
import hashlib
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import numpy as np

from weta_b200.backend import B200Backend
from weta_b200.core import manual_seed
from weta_b200.trainer import FusedTrainer, cnn_specs, mlp_specs
from weta_b200.workloads import MNIST_CNN, CnnConfig

TF32 = 1


def main():
    model = sys.argv[1]
    if model == "mlp":
        specs, batch, shape = mlp_specs(), 128, (784, 1, 1)
    elif model == "cnn":
        specs, batch, shape = cnn_specs(MNIST_CNN), 64, (1, 28, 28)
    else:  # the benchmark's layer shapes at a small batch: implicit convolutions, the fused first-block backward
        specs, batch, shape = cnn_specs(CnnConfig("wide-small", 3, 32, 128, 256, 1024)), 32, (3, 32, 32)
    gpu = B200Backend(0)
    rng = np.random.default_rng(5)
    manual_seed(21)
    tr = FusedTrainer(gpu, specs, batch, shape, lr=1e-3, matmul_mode=TF32)
    tr.init_from_global_rng()
    losses = []
    for _ in range(6):
        tr.stage(rng.random((batch,) + shape, dtype=np.float32), rng.integers(0, 10, batch).astype(np.int64))
        tr.step()
        losses.append(tr.loss())
    gpu.gemm_check()
    h = hashlib.sha256()
    for i in range(len(tr.ranges)):
        h.update(np.ascontiguousarray(tr.get_param(i)).tobytes())
    tr.close()
    print(json.dumps({"losses": losses, "params": h.hexdigest()}))


if __name__ == "__main__":
    main()
