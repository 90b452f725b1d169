"""The fused training step: Python handle on `WbTrainer` (include/weta_b200.h) and its data-parallel wrapper.

`FusedTrainer` runs the step of crates/weta/examples/mnist_cnn.rs:63-73 (forward, cross-entropy,
backward, Adam) as a fixed sequence of fused kernels.  The reference draws one RNG seed per
parameter tensor at construction and one per dropout call in forward order
(crates/weta-tensor/src/random.rs:95-98); this class draws the same seeds from the same host
generator, so a fused run and a primitive-mode run started from `manual_seed(s)` see identical
initial weights and identical dropout masks.
"""
from __future__ import annotations

import ctypes
from typing import Callable, List, Optional, Sequence, Tuple

import numpy as np

from .backend import B200Backend
from .core import global_rng
from .workloads import CnnConfig

CONV, LINEAR, DROPOUT = 0, 1, 2


class WbLayerSpec(ctypes.Structure):
    _fields_ = [("kind", ctypes.c_int32), ("a", ctypes.c_int32), ("b", ctypes.c_int32), ("c", ctypes.c_int32),
                ("p", ctypes.c_double)]


class WbAdamConfig(ctypes.Structure):
    _fields_ = [("lr", ctypes.c_double), ("beta1", ctypes.c_double), ("beta2", ctypes.c_double), ("eps", ctypes.c_double),
                ("weight_decay", ctypes.c_double), ("decoupled", ctypes.c_int32)]


BUCKET_CB = ctypes.CFUNCTYPE(None, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64)

_declared = False


def _declare(lib):
    global _declared
    if _declared:
        return
    P, PP = ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p)
    i32, i64, f64 = ctypes.c_int, ctypes.c_int64, ctypes.c_double
    U64P = ctypes.POINTER(ctypes.c_uint64)
    sig = {
        "wb_trainer_create": ([P, ctypes.POINTER(WbLayerSpec), i32, i64, i64, i64, i64, ctypes.POINTER(WbAdamConfig), i32, PP], i32),
        "wb_trainer_destroy": ([P], i32),
        "wb_trainer_init": ([P, U64P, i32], i32),
        "wb_trainer_arena_len": ([P], i64),
        "wb_trainer_params": ([P], P), "wb_trainer_grads": ([P], P), "wb_trainer_exp_avg": ([P], P),
        "wb_trainer_exp_avg_sq": ([P], P), "wb_trainer_input": ([P], P), "wb_trainer_labels": ([P], P),
        "wb_trainer_loss_ptr": ([P], P),
        "wb_trainer_num_tensors": ([P], i32),
        "wb_trainer_tensor_range": ([P, i32, ctypes.POINTER(i64), ctypes.POINTER(i64)], i32),
        "wb_trainer_bn_buffers": ([P, i32, PP, PP, ctypes.POINTER(i64)], i32),
        "wb_trainer_set_bucket_callback": ([P, BUCKET_CB, P], i32),
        "wb_trainer_forward_backward": ([P, U64P, i32], i32),
        "wb_trainer_adam_step": ([P, f64], i32),
        "wb_trainer_step_host": ([P, P, P, U64P, i32, ctypes.POINTER(ctypes.c_float)], i32),
        "wb_trainer_use_graph": ([P, i32], i32),
        "wb_trainer_step": ([P, U64P, i32], i32),
        "wb_trainer_read_loss": ([P, ctypes.POINTER(ctypes.c_float)], i32),
        "wb_trainer_set_timing": ([P, i32], i32),
        "wb_trainer_timing_report": ([P], ctypes.c_char_p),
        "wb_dropout_fwd": ([P, P, P, i64, f64, ctypes.c_uint64], i32),
        "wb_dropout_relu_bwd": ([P, P, P, P, i64, f64, ctypes.c_uint64], i32),
        "wb_dropout_mask": ([P, P, i64, f64, ctypes.c_uint64], i32),
        "wb_softmax_ce": ([P, P, P, i64, i64, P, P, P, P, f64], i32),
        "wb_bn2d_stats": ([P, P, i64, i64, i64, f64, f64, P, P, P, P], i32),
        "wb_bn2d_apply": ([P, P, i64, i64, i64, P, P, P, P, i32, P], i32),
        "wb_bn2d_fwd": ([P, P, i64, i64, i64, P, P, P, P, f64, f64, P, P, P], i32),
        "wb_bn2d_bwd": ([P, P, P, i64, i64, i64, P, P, P, P, P, P], i32),
        "wb_bn_relu_pool_fwd": ([P, P, i64, i64, i64, i64, P, P, P, P, f64, f64, P, P, P], i32),
        "wb_bn_relu_pool_bwd": ([P, P, P, i64, i64, i64, i64, P, P, P, P, P, P, P, P], i32),
        "wb_adam_step": ([P, P, P, P, P, i64, i64, f64, f64, f64, f64, f64, i32, f64], i32),
        "wb_trainer_set_input": ([P, P, P], i32),
        "wb_trainer_begin_step": ([P], i64),
        "wb_trainer_adam_range": ([P, P, i64, i64, i64, f64], i32),
        "wb_linear_fwd": ([P, P, P, P, i64, i64, i64, i32, P], i32),
        "wb_linear_bwd": ([P, P, P, P, i64, i64, i64, P, P, P], i32),
        "wb_maxpool2d_fwd": ([P, P, i64, i64, i64, i64, i64, P], i32),
        "wb_maxpool2d_bwd": ([P, P, P, i64, i64, i64, i64, i64, P], i32),
        "wb_relu_bwd": ([P, P, P, P, i64], i32),
        "wb_conv3x3_fwd": ([P, P, P, P, i64, i64, i64, i64, i64, P], i32),
        "wb_conv3x3_bwd": ([P, P, P, P, i64, i64, i64, i64, i64, P, P], i32),
    }
    for name, (args, res) in sig.items():
        fn = getattr(lib, name)
        fn.argtypes, fn.restype = args, res
    _declared = True


def mlp_specs(sizes: Sequence[int] = (784, 512, 256, 10), dropout_p: float = 0.1) -> List[Tuple]:
    """784-512-256-10 with ReLU + Dropout after each hidden layer (crates/weta/examples/mnist_mlp.rs:14-33)."""
    specs: List[Tuple] = []
    for i in range(len(sizes) - 2):
        specs += [(LINEAR, sizes[i], sizes[i + 1], 1, 0.0), (DROPOUT, 0, 0, 0, dropout_p)]
    specs.append((LINEAR, sizes[-2], sizes[-1], 0, 0.0))
    return specs


def cnn_specs(cfg: CnnConfig) -> List[Tuple]:
    """crates/weta/examples/mnist_cnn.rs:16-32 at the widths of `cfg`."""
    flat = cfg.c2 * (cfg.hw // 4) ** 2
    return [(CONV, cfg.in_ch, cfg.c1, 0, 0.0), (CONV, cfg.c1, cfg.c2, 0, 0.0), (DROPOUT, 0, 0, 0, cfg.dropout),
            (LINEAR, flat, cfg.hidden, 1, 0.0), (DROPOUT, 0, 0, 0, cfg.dropout), (LINEAR, cfg.hidden, cfg.classes, 0, 0.0)]


class FusedTrainer:
    def __init__(self, backend: B200Backend, specs: Sequence[Tuple], batch: int, in_shape: Tuple[int, int, int], lr: float = 1e-3,
                 betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0, decoupled: bool = False, matmul_mode: int = 1):
        self.be = backend
        self.lib = backend.lib
        _declare(self.lib)
        self.batch = batch
        self.in_shape = in_shape
        self.specs = list(specs)
        arr = (WbLayerSpec * len(specs))(*[WbLayerSpec(*s) for s in specs])
        adam = WbAdamConfig(lr, betas[0], betas[1], eps, weight_decay, int(decoupled))
        out = ctypes.c_void_p()
        backend.check(self.lib.wb_trainer_create(backend.handle, arr, len(specs), batch, *in_shape, ctypes.byref(adam), matmul_mode,
                                                 ctypes.byref(out)))
        self.handle = out.value
        # F::dropout draws a seed only when it needs a mask (crates/weta-nn/src/functional.rs:66-71)
        self.n_dropout = sum(1 for s in specs if s[0] == DROPOUT and 0.0 < s[4] < 1.0)
        self.n_seeded = 2 * sum(1 for s in specs if s[0] in (CONV, LINEAR))
        self.arena_len = self.lib.wb_trainer_arena_len(self.handle)
        self._cb = None
        self.ranges = []
        for i in range(self.lib.wb_trainer_num_tensors(self.handle)):
            off, ln = ctypes.c_int64(), ctypes.c_int64()
            backend.check(self.lib.wb_trainer_tensor_range(self.handle, i, ctypes.byref(off), ctypes.byref(ln)))
            self.ranges.append((off.value, ln.value))

    def close(self):
        if self.handle:
            self.lib.wb_trainer_destroy(self.handle)
            self.handle = None

    # -- parameters -------------------------------------------------------------------------
    def init_from_global_rng(self):
        """Draws one seed per weight / bias tensor from the host generator, in creation order."""
        seeds = (ctypes.c_uint64 * self.n_seeded)(*[global_rng().next_u64() for _ in range(self.n_seeded)])
        self.be.check(self.lib.wb_trainer_init(self.handle, seeds, self.n_seeded))

    def _download(self, base_ptr: int, off: int, n: int) -> np.ndarray:
        out = np.empty(n, dtype=np.float32)
        self.be.check(self.lib.wb_download_async(self.be.handle, ctypes.c_void_p(base_ptr + 4 * off), out.ctypes.data, 4 * n))
        self.be.synchronize()
        return out

    def _upload(self, base_ptr: int, off: int, arr: np.ndarray):
        arr = np.ascontiguousarray(arr, dtype=np.float32)
        self.be.check(self.lib.wb_upload_async(self.be.handle, arr.ctypes.data, ctypes.c_void_p(base_ptr + 4 * off), 4 * arr.size))
        self.be.synchronize()

    def params_ptr(self) -> int: return self.lib.wb_trainer_params(self.handle)
    def grads_ptr(self) -> int: return self.lib.wb_trainer_grads(self.handle)
    def input_ptr(self) -> int: return self.lib.wb_trainer_input(self.handle)
    def labels_ptr(self) -> int: return self.lib.wb_trainer_labels(self.handle)

    def get_param(self, i: int) -> np.ndarray:
        off, n = self.ranges[i]
        return self._download(self.params_ptr(), off, n)

    def get_grad(self, i: int) -> np.ndarray:
        off, n = self.ranges[i]
        return self._download(self.grads_ptr(), off, n)

    def set_param(self, i: int, arr: np.ndarray):
        off, n = self.ranges[i]
        assert arr.size == n
        self._upload(self.params_ptr(), off, arr.reshape(-1))

    def bn_buffers(self, conv_index: int) -> Tuple[np.ndarray, np.ndarray]:
        rm, rv, ch = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_int64()
        self.be.check(self.lib.wb_trainer_bn_buffers(self.handle, conv_index, ctypes.byref(rm), ctypes.byref(rv), ctypes.byref(ch)))
        return self._download(rm.value, 0, ch.value), self._download(rv.value, 0, ch.value)

    # -- stepping ---------------------------------------------------------------------------
    def draw_dropout_seeds(self):
        return (ctypes.c_uint64 * max(self.n_dropout, 1))(*[global_rng().next_u64() for _ in range(self.n_dropout)])

    def stage(self, x: np.ndarray, y: np.ndarray):
        """Copies a host batch into the staged device buffers (synchronous; for tests)."""
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
        y = np.ascontiguousarray(y, dtype=np.int64).reshape(-1)
        self.be.check(self.lib.wb_upload_async(self.be.handle, x.ctypes.data, ctypes.c_void_p(self.input_ptr()), 4 * x.size))
        self.be.check(self.lib.wb_upload_async(self.be.handle, y.ctypes.data, ctypes.c_void_p(self.labels_ptr()), 8 * y.size))
        self.be.synchronize()

    def forward_backward(self, seeds=None):
        seeds = self.draw_dropout_seeds() if seeds is None else seeds
        self.be.check(self.lib.wb_trainer_forward_backward(self.handle, seeds, self.n_dropout))

    def use_graph(self, on: bool = True):
        """`step` and `step_host` replay the whole step from a CUDA graph captured once (one launch per step)."""
        self.be.check(self.lib.wb_trainer_use_graph(self.handle, int(on)))

    def step(self, seeds=None):
        """forward_backward followed by adam_step(1.0), as one call (a graph replay after `use_graph`)."""
        seeds = self.draw_dropout_seeds() if seeds is None else seeds
        self.be.check(self.lib.wb_trainer_step(self.handle, seeds, self.n_dropout))

    def adam_step(self, grad_scale: float = 1.0):
        self.be.check(self.lib.wb_trainer_adam_step(self.handle, grad_scale))

    def loss(self) -> float:
        out = ctypes.c_float()
        self.be.check(self.lib.wb_trainer_read_loss(self.handle, ctypes.byref(out)))
        return out.value

    def step_host(self, x_ptr: int, y_ptr: int, seeds=None) -> float:
        """One whole step from (pinned) host buffers: upload, forward/backward/Adam, loss download, wait."""
        seeds = self.draw_dropout_seeds() if seeds is None else seeds
        out = ctypes.c_float()
        self.be.check(self.lib.wb_trainer_step_host(self.handle, ctypes.c_void_p(x_ptr), ctypes.c_void_p(y_ptr), seeds, self.n_dropout,
                                                    ctypes.byref(out)))
        return out.value

    def set_timing(self, on: bool):
        self.be.check(self.lib.wb_trainer_set_timing(self.handle, int(on)))

    def timing_report(self) -> dict:
        """{label: (calls, total_ms)} of the ops timed since the last report; waits for the stream."""
        out = {}
        for line in self.lib.wb_trainer_timing_report(self.handle).decode().splitlines():
            label, calls, ms = line.split()
            out[label] = (int(calls), float(ms))
        return out

    def set_bucket_callback(self, fn: Optional[Callable[[int, int], None]]):
        """fn(device_pointer, n_floats) fires during backward whenever one layer's gradients are final (the library's
        "quiet point" notifications, which carry no range, are not forwarded)."""
        if fn is None:
            self._cb = BUCKET_CB(0)
        else:
            self._cb = BUCKET_CB(lambda user, ptr, n: fn(ptr, n) if n > 0 else None)
        self.be.check(self.lib.wb_trainer_set_bucket_callback(self.handle, self._cb, None))


class WbDpId(ctypes.Structure):
    _fields_ = [("bytes", ctypes.c_uint8 * 128)]


POLL_FN = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p)
DP_AUTO, DP_ALLREDUCE, DP_SHARDED, DP_PEER = 0, 1, 2, 3
DP_MODE_NAMES = {1: "allreduce", 2: "sharded", 3: "peer"}


def _declare_dp(lib):
    if getattr(lib, "_wb_dp_declared", False):
        return
    P, PP = ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p)
    i32, i64, f64 = ctypes.c_int, ctypes.c_int64, ctypes.c_double
    I64P, U64P = ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_uint64)
    sig = {
        "wb_dp_unique_id": ([ctypes.POINTER(WbDpId)], i32),
        "wb_dp_create": ([P, ctypes.POINTER(WbDpId), i32, i32, i32, i64, PP], i32),
        "wb_dp_destroy": ([P], i32),
        "wb_dp_mode": ([P], i32), "wb_dp_world": ([P], i32), "wb_dp_num_buckets": ([P], i32),
        "wb_dp_bucket": ([P, i32, I64P, I64P], i32),
        "wb_dp_step": ([P, U64P, i32], i32),
        "wb_dp_submit": ([P, P, P], i32),
        "wb_dp_step_submitted": ([P, U64P, i32, ctypes.POINTER(ctypes.c_float)], i32),
        "wb_dp_wait": ([P, i32], i32),
        "wb_dp_set_timing": ([P, i32], i32),
        "wb_dp_timing_report": ([P], ctypes.c_char_p),
        "wb_dp_plan_buckets": ([I64P, I64P, i32, i64, I64P, I64P, i32], i32),
        "wb_watchdog_wait": ([POLL_FN, P, i32, i32], i32),
        "wb_reduce_adam_broadcast": ([P, PP, PP, i32, i32, i64, i64, P, P, i64, f64, f64, f64, f64, f64, i32, f64], i32),
        "wb_dp_selftest_wait": ([P, i32, i32], i32),
    }
    for name, (args, res) in sig.items():
        fn = getattr(lib, name)
        fn.argtypes, fn.restype = args, res
    lib._wb_dp_declared = True


def plan_buckets(lib, ranges: Sequence[Tuple[int, int]], min_elems: int) -> List[Tuple[int, int]]:
    """How per-layer arena ranges (offset, length), in arena order, merge into exchange buckets (wb_dp_plan_buckets)."""
    _declare_dp(lib)
    n = len(ranges)
    off = (ctypes.c_int64 * max(n, 1))(*[r[0] for r in ranges])
    ln = (ctypes.c_int64 * max(n, 1))(*[r[1] for r in ranges])
    bo, bl = (ctypes.c_int64 * max(n, 1))(), (ctypes.c_int64 * max(n, 1))()
    nb = lib.wb_dp_plan_buckets(off, ln, n, min_elems, bo, bl, max(n, 1))
    if nb < 0:
        raise ValueError("wb_dp_plan_buckets: bad arguments")
    return [(bo[i], bl[i]) for i in range(nb)]


def watchdog_wait(lib, poll: Callable[[], int], timeout_ms: int, interval_us: int = 1000) -> int:
    """Runs the library's host watchdog loop over `poll()` (0 = finished, 1 = still running, other = failed)."""
    _declare_dp(lib)
    cb = POLL_FN(lambda user: int(poll()))
    return lib.wb_watchdog_wait(cb, None, timeout_ms, interval_us)


def make_dp_id(lib) -> bytes:
    """The 128-byte rendezvous id rank 0 creates and hands to the other ranks over any host channel."""
    _declare_dp(lib)
    out = WbDpId()
    st = lib.wb_dp_unique_id(ctypes.byref(out))
    if st != 0:
        raise RuntimeError(f"wb_dp_unique_id: status {st}: {lib.wb_last_error().decode()}")
    return ctypes.string_at(ctypes.addressof(out), 128)


class DataParallelTrainer:
    """Handle on `WbDp` (include/weta_b200.h): the data-parallel form of the fused step.

    One process per GPU, every rank a full replica, the batch sharded.  The reference has no multi-GPU path; this adds
    the one exchange a data-parallel step needs.  Streams, the NCCL communicator, the bucket plan, the peer-memory
    kernel and the double-buffered upload all live behind the C ABI; this class only forwards calls.
    BatchNorm statistics stay per rank, as they would in the reference (it has no SyncBN).
    """

    def __init__(self, trainer: FusedTrainer, rank: int = 0, world_size: int = 1, dp_id: Optional[bytes] = None, mode: int = DP_AUTO,
                 bucket_elems: int = 1 << 20):
        self.tr = trainer
        self.lib = trainer.lib
        _declare_dp(self.lib)
        self.world, self.rank = world_size, rank
        idp = None
        if world_size > 1:
            assert dp_id is not None and len(dp_id) == 128, "more than one rank needs the 128-byte id made by rank 0"
            idv = WbDpId()
            ctypes.memmove(ctypes.addressof(idv), dp_id, 128)
            idp = ctypes.byref(idv)
        out = ctypes.c_void_p()
        trainer.be.check(self.lib.wb_dp_create(trainer.handle, idp, rank, world_size, mode, bucket_elems, ctypes.byref(out)))
        self.handle = out.value
        self.mode = self.lib.wb_dp_mode(self.handle)
        self.buckets = []
        for i in range(self.lib.wb_dp_num_buckets(self.handle)):
            off, ln = ctypes.c_int64(), ctypes.c_int64()
            trainer.be.check(self.lib.wb_dp_bucket(self.handle, i, ctypes.byref(off), ctypes.byref(ln)))
            self.buckets.append((off.value, ln.value))

    def close(self):
        if self.handle:
            self.lib.wb_dp_destroy(self.handle)
            self.handle = None

    def step(self, seeds=None):
        """forward, backward with overlapped exchange and per-bucket Adam on the staged batch; asynchronous."""
        tr = self.tr
        seeds = tr.draw_dropout_seeds() if seeds is None else seeds
        tr.be.check(self.lib.wb_dp_step(self.handle, seeds, tr.n_dropout))

    def submit(self, x_ptr: int, y_ptr: int):
        """Queues the upload of one batch from pinned host memory into the next device slot."""
        self.tr.be.check(self.lib.wb_dp_submit(self.handle, ctypes.c_void_p(x_ptr), ctypes.c_void_p(y_ptr)))

    def step_submitted(self, seeds=None, read_loss: bool = True) -> Optional[float]:
        """One step on the oldest submitted batch; returns its loss (a device-to-host read that waits for the step)."""
        tr = self.tr
        seeds = tr.draw_dropout_seeds() if seeds is None else seeds
        out = ctypes.c_float()
        tr.be.check(self.lib.wb_dp_step_submitted(self.handle, seeds, tr.n_dropout, ctypes.byref(out) if read_loss else None))
        return out.value if read_loss else None

    def wait(self, timeout_ms: int = 0):
        self.tr.be.check(self.lib.wb_dp_wait(self.handle, timeout_ms))

    def set_timing(self, on: bool):
        self.tr.be.check(self.lib.wb_dp_set_timing(self.handle, int(on)))

    def timing_report(self) -> Tuple[int, float]:
        _, calls, ms = self.lib.wb_dp_timing_report(self.handle).decode().split()
        return int(calls), float(ms)
