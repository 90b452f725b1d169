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
        self.n_dropout = sum(1 for s in specs if s[0] == DROPOUT)
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
        """fn(device_pointer, n_floats) fires during backward whenever one layer's gradients are final."""
        if fn is None:
            self._cb = BUCKET_CB(0)
        else:
            self._cb = BUCKET_CB(lambda user, ptr, n: fn(ptr, n))
        self.be.check(self.lib.wb_trainer_set_bucket_callback(self.handle, self._cb, None))


class GradBucketer:
    """Turns the trainer's per-layer "gradients final" notifications into a few large all-reduces.

    Ranges arrive front to back over one flat arena (last layer first).  Adjacent ranges are merged
    until `min_elems` have accumulated, then `reduce_fn(start, length)` is called for the merged
    range; `flush()` sends whatever is left.  Pure host logic: the collective itself is injected.
    """

    def __init__(self, reduce_fn: Callable[[int, int], None], min_elems: int = 1 << 20):
        self.reduce_fn = reduce_fn
        self.min_elems = min_elems
        self.start: Optional[int] = None
        self.length = 0
        self.issued: List[Tuple[int, int]] = []

    def add(self, start: int, length: int):
        if length <= 0:
            return
        if self.start is None:
            self.start, self.length = start, length
        elif start == self.start + self.length:
            self.length += length
        else:  # not adjacent: send what we have and start over
            self.flush()
            self.start, self.length = start, length
        if self.length >= self.min_elems:
            self.flush()

    def flush(self):
        if self.start is not None and self.length > 0:
            self.reduce_fn(self.start, self.length)
            self.issued.append((self.start, self.length))
        self.start, self.length = None, 0


class _DevicePtr:
    """Exposes a raw device range to torch through __cuda_array_interface__ (no copy)."""

    def __init__(self, ptr: int, n: int, typestr: str = "<f4"):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (ptr, False), "version": 3, "strides": None}


class DataParallelTrainer:
    """Data-parallel wrapper: one process per GPU, every rank a full replica, the batch sharded.

    The reference has no multi-GPU path; this adds the one exchange a data-parallel step needs.
    Gradients are summed with NCCL (`torch.distributed`) on a side stream as soon as a bucket of the
    arena is final, and that bucket's Adam update (with 1/world) follows on a third stream, both while
    backward continues on the compute stream; the next step waits for the last update.
    BatchNorm statistics stay per rank, as they would in the reference (it has no SyncBN).
    """

    def __init__(self, trainer: FusedTrainer, compute_stream, world_size: int, bucket_elems: int = 1 << 20):
        import torch
        import torch.distributed as dist

        self.torch, self.dist = torch, dist
        self.tr = trainer
        self.world = world_size
        self.stream = compute_stream
        self.comm_stream = torch.cuda.Stream() if world_size > 1 else None
        self.adam_stream = torch.cuda.Stream() if world_size > 1 else None
        # a second handle on the same device whose kernels go to the optimizer stream
        self.adam_backend = B200Backend(trainer.be.ordinal, self.adam_stream.cuda_stream) if world_size > 1 else None
        self.step_t = 0
        self.covered = 0
        self.works = []
        self.grad_view = torch.as_tensor(_DevicePtr(trainer.grads_ptr(), trainer.arena_len), device=f"cuda:{trainer.be.ordinal}")
        self.bucketer = GradBucketer(self._all_reduce_range, bucket_elems)
        base = trainer.grads_ptr()
        if world_size > 1:
            trainer.set_bucket_callback(lambda ptr, n: self.bucketer.add((ptr - base) // 4, n))

    def _all_reduce_range(self, start: int, length: int):
        torch = self.torch
        ev = torch.cuda.Event()
        ev.record(self.stream)                   # everything queued so far, i.e. this bucket's gradients
        self.comm_stream.wait_event(ev)
        with torch.cuda.stream(self.comm_stream):
            work = self.dist.all_reduce(self.grad_view[start:start + length], op=self.dist.ReduceOp.SUM, async_op=True)
        with torch.cuda.stream(self.adam_stream):
            work.wait()  # orders the optimizer stream after this bucket's sum
            tr = self.tr
            tr.be.check(tr.lib.wb_trainer_adam_range(tr.handle, self.adam_backend.handle, start, length, self.step_t, 1.0 / self.world))
        self.works.append(work)
        self.covered += length

    def forward_backward_step(self, seeds=None):
        """forward, backward with overlapped all-reduce and per-bucket Adam.  Inputs must already be staged."""
        if self.world == 1:
            self.tr.forward_backward(seeds)
            self.tr.adam_step(1.0)
            return
        self.step_t = self.tr.lib.wb_trainer_begin_step(self.tr.handle)
        self.covered = 0
        self.tr.forward_backward(seeds)
        self.bucketer.flush()
        if self.covered != self.tr.arena_len:
            raise RuntimeError(f"gradient buckets covered {self.covered} of {self.tr.arena_len} arena elements")
        self.works.clear()
        self.stream.wait_stream(self.adam_stream)  # the next step reads the updated parameters

    def step_host(self, x_pinned, y_pinned, seeds=None) -> float:
        """One step from pinned host tensors: upload, forward/backward (+ all-reduce), Adam, loss read-back."""
        tr, be = self.tr, self.tr.be
        be.check(be.lib.wb_upload_async(be.handle, x_pinned.data_ptr(), ctypes.c_void_p(tr.input_ptr()), x_pinned.numel() * 4))
        be.check(be.lib.wb_upload_async(be.handle, y_pinned.data_ptr(), ctypes.c_void_p(tr.labels_ptr()), y_pinned.numel() * 8))
        self.forward_backward_step(seeds)
        return tr.loss()


class PrefetchingStepper:
    """Feeds host batches to a DataParallelTrainer with the upload of batch i+1 overlapped with step i.

    Two device slots; `submit` enqueues the host-to-device copy of one pinned batch on a copy stream, `step` runs one
    training step on the oldest submitted batch and returns its loss (a device-to-host read that waits for the
    step).  The copy into a slot waits for the step that last read it; the step waits for its slot's copy.
    """

    def __init__(self, dp: DataParallelTrainer):
        import torch

        self.torch, self.dp = torch, dp
        tr = dp.tr
        dev = f"cuda:{tr.be.ordinal}"
        n_in = tr.batch * int(np.prod(tr.in_shape))
        self.slots = [(torch.empty(n_in, dtype=torch.float32, device=dev), torch.empty(tr.batch, dtype=torch.int64, device=dev)) for _ in range(2)]
        self.copy_stream = torch.cuda.Stream()
        self.ready = [torch.cuda.Event() for _ in range(2)]
        self.consumed = [torch.cuda.Event() for _ in range(2)]
        for ev in self.consumed:
            ev.record(dp.stream)
        self.submitted = 0
        self.stepped = 0

    def submit(self, x_pinned, y_pinned):
        if self.submitted - self.stepped >= 2:
            raise RuntimeError("both slots hold batches that have not been stepped yet")
        slot = self.submitted % 2
        with self.torch.cuda.stream(self.copy_stream):
            self.copy_stream.wait_event(self.consumed[slot])
            self.slots[slot][0].copy_(x_pinned, non_blocking=True)
            self.slots[slot][1].copy_(y_pinned, non_blocking=True)
            self.ready[slot].record(self.copy_stream)
        self.submitted += 1

    def step(self, seeds=None) -> float:
        if self.stepped >= self.submitted:
            raise RuntimeError("no submitted batch to step on")
        slot = self.stepped % 2
        tr = self.dp.tr
        self.dp.stream.wait_event(self.ready[slot])
        x, y = self.slots[slot]
        tr.be.check(tr.lib.wb_trainer_set_input(tr.handle, ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(y.data_ptr())))
        self.dp.forward_backward_step(seeds)
        self.consumed[slot].record(self.dp.stream)
        self.stepped += 1
        return tr.loss()

    def close(self):
        tr = self.dp.tr
        tr.be.check(tr.lib.wb_trainer_set_input(tr.handle, None, None))
