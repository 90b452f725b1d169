"""Per-kernel roofline sweep: the contraction microbenchmark and the memory-bound op sweep.

    python -m weta_b200.microbench [--out results.json] [--quick]

Times each op with CUDA events on the backend's stream (5 warm-ups, 20 timed launches queued behind a
millisecond of device-side delay so that the device, not the Python binding, sets the pace (the training
steps at the end are timed without it: their pace is the caller's); outputs
pre-allocated through the `*_into` entry points so no allocation is timed) and reports achieved
GB/s or TFLOP/s against the measured copy bandwidth / half the measured bf16 GEMM rate.  Inputs are
f32 N(0,1) from the counter RNG.  Tensors are larger than the 126 MB L2 where the workload allows;
the softmax-cross-entropy logits (33 MB) rotate through 8 buffers so each launch reads from HBM.
Algorithmic bytes: unary 8 B/elem, binary 12 B/elem, mul backward 20 B/elem (read g, a, b; write g*b, g*a: timed
as the two trait launches the reference issues, which move 24), ReLU backward 12 B/elem (the fused wb_relu_bwd), BN
fwd 12 / bwd 20 B/elem, softmax-CE fused fwd+bwd 8*N*C, dropout mask 4 B/elem, Adam 28 B/elem; contractions 2*M*N*K flop.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os

import numpy as np

from .backend import B200Backend, WbConvParams
from .core import BinaryOp, Distribution, DType, Im2ColParams, Layout, ReduceOp, UnaryOp
from .trainer import _declare


class Arr:
    """A device storage with a layout: just enough of a tensor to build the views the sweep needs."""

    def __init__(self, storage, layout, dtype=DType.F32):
        self.storage, self.layout, self.dtype = storage, layout, dtype

    @property
    def shape(self):
        return self.layout.shape

    def transpose(self, a, b):
        return Arr(self.storage, self.layout.transpose(a, b), self.dtype)

    def t(self):
        return self.transpose(0, 1)

    def reshape(self, shape):
        return Arr(self.storage, self.layout.reshape(shape), self.dtype)


def load_peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return p["hbm_gbs"], p["bf16_tflops"] / 2.0, "measured"
    return 6650.0, 795.0, "fallback"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    ap.add_argument("--quick", action="store_true", help="smaller shapes (for a profiler capture)")
    ap.add_argument("--once", action="store_true", help="launch every op once instead of timing loops (for a profiler capture)")
    args = ap.parse_args()
    import torch

    be = B200Backend(0)
    lib = be.lib
    _declare(lib)
    hbm_peak, tf32_peak, src = load_peaks()
    stream = torch.cuda.ExternalStream(be.stream())
    results = {}

    def timeit(fn, iters=20, warm=5, paced=True):
        if args.once:
            iters, warm = 1, 0
        for _ in range(warm):
            fn()
        be.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if paced and not args.once:
            # About a millisecond of device-side delay ahead of the loop: its launches are queued by the time the first
            # of them starts, so a kernel shorter than one call through the Python binding is still timed at the
            # device's pace, not the binding's.
            with torch.cuda.stream(stream):
                torch.cuda._sleep(2_000_000)
        e0.record(stream)
        for i in range(iters):
            fn()
        e1.record(stream)
        e1.synchronize()
        return e0.elapsed_time(e1) / iters

    def rec(name, ms, bytes_=None, flops=None, note=""):
        r = {"ms": round(ms, 4)}
        if bytes_ is not None:
            r.update(gbs=round(bytes_ / ms / 1e6, 1), frac=round(bytes_ / ms / 1e6 / hbm_peak, 3), bound="hbm")
        if flops is not None:
            r.update(tflops=round(flops / ms / 1e9, 1), frac=round(flops / ms / 1e9 / tf32_peak, 3), bound="tensor")
        if note:
            r["note"] = note
        results[name] = r
        print(name, r, flush=True)

    def randn(shape, seed):
        l = Layout.contiguous(shape)
        return Arr(be.random(l.numel(), DType.F32, Distribution.normal(0.0, 1.0), seed), l)

    def filled(shape, value):
        l = Layout.contiguous(shape)
        z = be.zeros(l.numel(), DType.F32)
        return Arr(z if value == 0.0 else be.unary(UnaryOp.AFFINE, 1.0, value, z, l, DType.F32), l)

    def view(t):
        return ctypes.byref(t.layout.view(t.storage.ptr, t.dtype))

    # ---- memory-bound sweep on [256, 64, 56, 56] -------------------------------------------------
    shape = [64, 64, 56, 56] if args.quick else [256, 64, 56, 56]
    E = int(np.prod(shape))
    x, y, g = randn(shape, 1), randn(shape, 2), randn(shape, 3)
    P = lambda s: ctypes.c_void_p(s.ptr)
    out = be.alloc(E, DType.F32)
    out2 = be.alloc(E, DType.F32)
    o, o2 = ctypes.c_void_p(out.ptr), ctypes.c_void_p(out2.ptr)
    H = be.handle
    for lname, fx, fy, fg in (("contiguous", x, y, g), ("transposed(1,3)", x.transpose(1, 3), y.transpose(1, 3), g.transpose(1, 3)),
                               ("transposed(0,1)", x.transpose(0, 1), y.transpose(0, 1), g.transpose(0, 1))):
        rec(f"add fwd {lname}", timeit(lambda: be.check(lib.wb_binary_into(H, BinaryOp.ADD, view(fx), view(fy), o))), 12 * E)
        rec(f"mul fwd {lname}", timeit(lambda: be.check(lib.wb_binary_into(H, BinaryOp.MUL, view(fx), view(fy), o))), 12 * E)

        def mul_bwd():  # BinaryBw Mul: both g*b and g*a (crates/weta-autograd/src/ops.rs:199)
            be.check(lib.wb_binary_into(H, BinaryOp.MUL, view(fg), view(fy), o))
            be.check(lib.wb_binary_into(H, BinaryOp.MUL, view(fg), view(fx), o2))

        rec(f"mul bwd {lname}", timeit(mul_bwd), 20 * E, note="two trait launches (g*b, g*a) moving 24 B/elem; rate counted on the algorithmic 20")
        rec(f"relu fwd {lname}", timeit(lambda: be.check(lib.wb_unary_into(H, UnaryOp.RELU, 0.0, 0.0, view(fx), o))), 8 * E)

        def relu_bwd_chain():  # UnaryBw Relu as the reference issues it: step(x), then g * step (ops.rs:85)
            be.check(lib.wb_unary_into(H, UnaryOp.STEP, 0.0, 0.0, view(fx), o))
            s = Arr(out, Layout.contiguous(fx.shape))
            be.check(lib.wb_binary_into(H, BinaryOp.MUL, view(fg), view(s), o2))

        rec(f"relu bwd {lname}, trait chain", timeit(relu_bwd_chain), 12 * E,
            note="two trait launches (step(x), g*step) moving 20 B/elem; rate counted on the algorithmic 12")
        if lname == "contiguous":
            rec("relu bwd contiguous, fused wb_relu_bwd", timeit(lambda: be.check(lib.wb_relu_bwd(H, P(g.storage), P(x.storage), o, E))), 12 * E)

    # BatchNorm2d fwd + bwd, statistics over N*H*W per channel
    n, c, hw = shape[0], shape[1], shape[2] * shape[3]
    gamma, beta = randn([c], 4), randn([c], 5)
    rm = filled([c], 0.0)
    rv = filled([c], 1.0)
    sm, sr, dg, db = (be.alloc(c, DType.F32) for _ in range(4))
    rec("batchnorm2d fwd", timeit(lambda: be.check(lib.wb_bn2d_fwd(H, P(x.storage), n, c, hw, P(gamma.storage), P(beta.storage), P(rm.storage),
                                                                    P(rv.storage), 0.1, 1e-5, o, P(sm), P(sr)))), 12 * E)
    rec("batchnorm2d bwd", timeit(lambda: be.check(lib.wb_bn2d_bwd(H, P(x.storage), P(g.storage), n, c, hw, P(gamma.storage), P(sm), P(sr), o,
                                                                    P(dg), P(db)))), 20 * E)
    def mean_chain():  # mean over (0, 2, 3): one Backend::reduce per axis, highest first, then affine (tensor.rs:496-530)
        s3 = be.reduce(ReduceOp.SUM, x.storage, x.layout, DType.F32, 3)
        s2 = be.reduce(ReduceOp.SUM, s3, Layout.contiguous(shape[:3]), DType.F32, 2)
        s0 = be.reduce(ReduceOp.SUM, s2, Layout.contiguous(shape[:2]), DType.F32, 0)
        return be.unary(UnaryOp.AFFINE, 1.0 / (n * hw), 0.0, s0, Layout.contiguous([c]), DType.F32)

    rec("batchnorm mean, primitive chain (3 reduces + affine)", timeit(mean_chain), 4 * E,
        note="Backend::reduce called once per axis, as weta-tensor does")

    # softmax cross-entropy [8192, 1000], 8 rotating logits buffers (33 MB each)
    rows, cols = (2048, 1000) if args.quick else (8192, 1000)
    logits = [randn([rows, cols], 10 + i) for i in range(8)]
    lf = be.random(rows, DType.F64, Distribution.uniform(0.0, float(cols)), 99)
    labels = Arr(be.cast(lf, Layout.contiguous([rows]), DType.F64, DType.I64), Layout.contiguous([rows]), DType.I64)
    dz = be.alloc(rows * cols, DType.F32)
    loss = be.alloc(1, DType.F32)
    k = [0]

    def ce():
        k[0] += 1
        be.check(lib.wb_softmax_ce(H, P(logits[k[0] % 8].storage), P(labels.storage), rows, cols, None, P(dz), None, P(loss), 1.0))

    rec("softmax-cross-entropy fwd+bwd fused", timeit(ce), 8 * rows * cols, note="reads logits, writes dlogits and the mean loss")

    # dropout mask fill and Adam
    nmask = 1 << (26 if args.quick else 28)
    mask = be.alloc(nmask, DType.F32)
    rec("dropout mask fill p=0.1 seed 42", timeit(lambda: be.check(lib.wb_dropout_mask(H, P(mask), nmask, 0.1, 42)), iters=10), 4 * nmask)
    rec("uniform fill (Backend::random)", timeit(lambda: be.check(lib.wb_random_into(H, nmask, 0, 0, 0.0, 1.0, 42, P(mask))), iters=10), 4 * nmask)
    rec("normal fill (Backend::random)", timeit(lambda: be.check(lib.wb_random_into(H, nmask // 4, 0, 1, 0.0, 1.0, 42, P(mask))), iters=10), nmask)
    na = 25_000_000 if args.quick else 100_000_000
    th, gr = randn([na], 20), randn([na], 21)
    m1, v1 = filled([na], 0.0), filled([na], 0.0)
    step = [0]

    def adam():
        step[0] += 1
        be.check(lib.wb_adam_step(H, P(th.storage), P(gr.storage), P(m1.storage), P(v1.storage), na, step[0], 1e-3, 0.9, 0.999, 1e-8, 0.0, 0, 1.0))

    rec("adam step", timeit(adam, iters=10), 28 * na)

    # ---- contraction microbenchmark: forward plus both gradients ---------------------------------
    for mode, mname in ((1, "tf32"), (0, "3xtf32")):
        be.set_matmul_mode(mode)
        for nsz in ((512,) if args.quick else (512, 4096)):
            a, b, gg = randn([nsz, nsz], 1), randn([nsz, nsz], 2), randn([nsz, nsz], 3)
            oo = be.alloc(nsz * nsz, DType.F32)
            fl = 2.0 * nsz ** 3
            for label, (p, q) in (("fwd A.B", (a, b)), ("dA = G.B^T", (gg, b.t())), ("dB = A^T.G", (a.t(), gg))):
                pl, ql = p.layout.unsqueeze(0), q.layout.unsqueeze(0)
                pv, qv = pl.view(p.storage.ptr, 0), ql.view(q.storage.ptr, 0)
                ms = timeit(lambda: be.check(lib.wb_matmul_into(H, ctypes.byref(pv), ctypes.byref(qv), P(oo))))
                rec(f"matmul {nsz}^3 {label} {mname}", ms, flops=fl)
        # conv2d [64,32,14,14] * [64,32,3,3], stride 1, pad 1, with bias: im2col + W.cols + bias, then dW, dX
        xc, wc, bc = randn([64, 32, 14, 14], 1), randn([64, 32, 3, 3], 2), randn([64], 3)
        gc = randn([64, 64, 14, 14], 4)
        p3 = Im2ColParams((3, 3), (1, 1), (1, 1), (1, 1))
        fl = 2.0 * 64 * 64 * 288 * 196

        F = DType.F32
        w2 = Layout.contiguous([64, 288])
        cols_l, y_l = Layout.contiguous([64, 288, 196]), Layout.contiguous([64, 64, 196])

        def conv_fwd():  # F::conv2d_ext (functional.rs:84-106): im2col, W[O,K] broadcast over the batch, + bias[O,1]
            cols = be.im2col(xc.storage, xc.layout, F, p3)
            yv = be.matmul(wc.storage, w2.unsqueeze(0).broadcast_to([64, 64, 288]), cols, cols_l, F)
            return be.binary(BinaryOp.ADD, yv, y_l, bc.storage, Layout([1, 64, 1], [0, 1, 0]).broadcast_to([64, 64, 196]), F)

        def conv_bwd():  # MatmulBw + sum over the batch, Im2ColBw, bias sums (ops.rs:821-827, 865-868, 46-58)
            cols = be.im2col(xc.storage, xc.layout, F, p3)
            dwb = be.matmul(gc.storage, y_l, cols, cols_l.transpose(1, 2), F)
            dw = be.reduce(ReduceOp.SUM, dwb, Layout.contiguous([64, 64, 288]), F, 0)
            dcols = be.matmul(wc.storage, w2.transpose(0, 1).unsqueeze(0).broadcast_to([64, 288, 64]), gc.storage, y_l, F)
            dx = be.col2im(dcols, cols_l, F, p3, (32, 14, 14))
            db2 = be.reduce(ReduceOp.SUM, gc.storage, y_l, F, 2)
            dbias = be.reduce(ReduceOp.SUM, db2, Layout.contiguous([64, 64]), F, 0)
            return dw, dx, dbias

        rec(f"conv2d fwd (im2col + matmul + bias) {mname}", timeit(conv_fwd), flops=fl, note="trait-call sequence of F::conv2d")
        rec(f"conv2d dX+dW+db {mname}", timeit(conv_bwd), flops=2 * fl, note="trait-call sequence of its backward")
    be.set_matmul_mode(0)
    be.gemm_check()

    # ---- comparator, not weta: cuBLAS TF32 through torch.matmul on the same shapes ------------------
    torch.backends.cuda.matmul.allow_tf32 = True
    for nsz in ((512,) if args.quick else (512, 4096)):
        ta = torch.randn(nsz, nsz, device="cuda")
        tb = torch.randn(nsz, nsz, device="cuda")
        with torch.cuda.stream(stream):
            ms = timeit(lambda: torch.matmul(ta, tb))
        rec(f"comparator (not weta): cuBLAS TF32 torch.matmul {nsz}^3", ms, flops=2.0 * nsz ** 3)

    # ---- whole training steps of the two small named models (host batch in, loss out) ------------
    from .core import manual_seed
    from .trainer import FusedTrainer, cnn_specs, mlp_specs
    from .workloads import MNIST_CNN, synthetic_batch_device

    def host_batch(cfg_or_none, batch, feat):
        if cfg_or_none is not None:
            xs, ys = synthetic_batch_device(cfg_or_none, batch, 0, 0, be)
        else:  # config-1 inputs: pixels k/255 with k uniform in 0..255, labels uniform in 0..9
            pf = be.random(batch * feat, DType.F64, Distribution.uniform(0.0, 256.0), 10_000)
            pi = be.cast(pf, Layout.contiguous([batch * feat]), DType.F64, DType.I64)
            xs = be.unary(UnaryOp.AFFINE, 1.0 / 255.0, 0.0, be.cast(pi, Layout.contiguous([batch * feat]), DType.I64, DType.F32),
                          Layout.contiguous([batch * feat]), DType.F32)
            ys = be.cast(be.random(batch, DType.F64, Distribution.uniform(0.0, 10.0), 20_000), Layout.contiguous([batch]), DType.F64, DType.I64)
        return (be.to_host(xs, Layout.contiguous([batch * feat]), DType.F32), be.to_host(ys, Layout.contiguous([batch]), DType.I64))

    def step_rate(name, specs, batch, in_shape, xy, mode):
        manual_seed(42)
        tr = FusedTrainer(be, specs, batch, in_shape, lr=1e-3, matmul_mode=mode)
        tr.init_from_global_rng()
        x = np.ascontiguousarray(xy[0], dtype=np.float32)
        y = np.ascontiguousarray(xy[1], dtype=np.int64)
        ms = timeit(lambda: tr.step_host(x.ctypes.data, y.ctypes.data), iters=50, warm=10, paced=False)
        results[name] = {"ms": round(ms, 4), "samples_per_s": round(batch / ms * 1e3, 1), "batch": batch}
        print(name, results[name], flush=True)
        # the same call with the step replayed from a CUDA graph (host batch in, loss out, every step)
        tr.use_graph(True)
        ms = timeit(lambda: tr.step_host(x.ctypes.data, y.ctypes.data), iters=50, warm=10, paced=False)
        results[name + ", graph"] = {"ms": round(ms, 4), "samples_per_s": round(batch / ms * 1e3, 1), "batch": batch}
        print(name + ", graph", results[name + ", graph"], flush=True)
        tr.close()

    for mode, mname in ((0, "3xtf32"), (1, "tf32")):
        step_rate(f"mlp 784-512-256-10 train step, batch 128, {mname}", mlp_specs(), 128, (784, 1, 1), host_batch(None, 128, 784), mode)
        step_rate(f"cnn-mnist-422k train step, batch 64, {mname}", cnn_specs(MNIST_CNN), 64, (1, 28, 28), host_batch(MNIST_CNN, 64, 784), mode)
    results["_peaks"] = {"hbm_gbs": hbm_peak, "tf32_tflops": tf32_peak, "source": src}
    if args.out:
        os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
        json.dump(results, open(args.out, "w"), indent=1)


if __name__ == "__main__":
    main()
