"""Per-kernel roofline sweep: the contraction microbenchmark and the memory-bound op sweep.

    python -m weta_b200.microbench [--out results.json] [--quick]

Times each op with CUDA events on the backend's stream (5 warm-ups, 20 timed launches, outputs
pre-allocated through the `*_into` entry points so no allocation is timed) and reports achieved
GB/s or TFLOP/s against the measured copy bandwidth / half the measured bf16 GEMM rate.  Inputs are
f32 N(0,1) from the counter RNG.  Tensors are larger than the 126 MB L2 where the workload allows;
the softmax-cross-entropy logits (33 MB) rotate through 8 buffers so each launch reads from HBM.
Algorithmic bytes: unary 8 B/elem, binary 12 B/elem, BN fwd 12 / bwd 20 B/elem, softmax-CE fused
fwd+bwd 8*N*C, dropout mask 4 B/elem, Adam 28 B/elem; contractions 2*M*N*K flop.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os

import numpy as np

from .backend import B200Backend, WbConvParams
from .core import BinaryOp, Distribution, DType, Im2ColParams, UnaryOp
from .tensor import Tensor
from .trainer import _declare


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

    def timeit(fn, iters=20, warm=5):
        if args.once:
            iters, warm = 1, 0
        for _ in range(warm):
            fn()
        be.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
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
        return Tensor.random_seeded(shape, Distribution.normal(0.0, 1.0), DType.F32, be, seed)

    def view(t):
        return ctypes.byref(t.layout.view(t.storage.ptr, t.dtype))

    # ---- memory-bound sweep on [256, 64, 56, 56] -------------------------------------------------
    shape = [64, 64, 56, 56] if args.quick else [256, 64, 56, 56]
    E = int(np.prod(shape))
    x, y, g = randn(shape, 1), randn(shape, 2), randn(shape, 3)
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

        rec(f"mul bwd {lname}", timeit(mul_bwd), 24 * E, note="two launches: g*b and g*a, 12 B/elem each")
        rec(f"relu fwd {lname}", timeit(lambda: be.check(lib.wb_unary_into(H, UnaryOp.RELU, 0.0, 0.0, view(fx), o))), 8 * E)

        def relu_bwd():  # UnaryBw Relu: g * step(x) (ops.rs:85)
            be.check(lib.wb_unary_into(H, UnaryOp.STEP, 0.0, 0.0, view(fx), o))
            s = Tensor(out, fx.layout.__class__.contiguous(fx.shape), DType.F32, be)
            be.check(lib.wb_binary_into(H, BinaryOp.MUL, view(fg), view(s), o2))

        rec(f"relu bwd {lname}", timeit(relu_bwd), 20 * E, note="two launches: step(x) 8 B/elem, g*step 12 B/elem")

    # BatchNorm2d fwd + bwd, statistics over N*H*W per channel
    n, c, hw = shape[0], shape[1], shape[2] * shape[3]
    gamma, beta = randn([c], 4), randn([c], 5)
    rm = Tensor.zeros([c], DType.F32, be)
    rv = Tensor.ones([c], DType.F32, be)
    sm, sr, dg, db = (be.alloc(c, DType.F32) for _ in range(4))
    P = lambda s: ctypes.c_void_p(s.ptr)
    rec("batchnorm2d fwd", timeit(lambda: be.check(lib.wb_bn2d_fwd(H, P(x.storage), n, c, hw, P(gamma.storage), P(beta.storage), P(rm.storage),
                                                                    P(rv.storage), 0.1, 1e-5, o, P(sm), P(sr)))), 12 * E)
    rec("batchnorm2d bwd", timeit(lambda: be.check(lib.wb_bn2d_bwd(H, P(x.storage), P(g.storage), n, c, hw, P(gamma.storage), P(sm), P(sr), o,
                                                                    P(dg), P(db)))), 20 * E)
    rec("batchnorm mean, primitive chain (3 reduces + affine)", timeit(lambda: x.mean_dims([0, 2, 3])), 4 * E,
        note="Backend::reduce called once per axis, as weta-tensor does")

    # softmax cross-entropy [8192, 1000], 8 rotating logits buffers (33 MB each)
    rows, cols = (2048, 1000) if args.quick else (8192, 1000)
    logits = [randn([rows, cols], 10 + i) for i in range(8)]
    labels = Tensor.random_seeded([rows], Distribution.uniform(0.0, float(cols)), DType.I64, be, 99)
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
    m1, v1 = Tensor.zeros([na], DType.F32, be), Tensor.zeros([na], DType.F32, be)
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

        def conv_fwd():
            return xc.conv2d(wc, bc, 1, 1)

        def conv_bwd():
            cols = xc.im2col(p3)
            g3 = gc.reshape([64, 64, 196])
            dw = g3.matmul(cols.transpose(1, 2)).sum_dims([0])
            dx = wc.reshape([64, 288]).t().matmul(g3).col2im(p3, (32, 14, 14))
            dbias = g3.sum_dims([2]).sum_dims([0])
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
    from .workloads import MNIST_CNN, mlp_batch, synthetic_batch

    def step_rate(name, specs, batch, in_shape, xy, mode):
        manual_seed(42)
        tr = FusedTrainer(be, specs, batch, in_shape, lr=1e-3, matmul_mode=mode)
        tr.init_from_global_rng()
        x = np.ascontiguousarray(xy[0].numpy(), dtype=np.float32)
        y = np.ascontiguousarray(xy[1].numpy(), dtype=np.int64)
        ms = timeit(lambda: tr.step_host(x.ctypes.data, y.ctypes.data), iters=50, warm=10)
        results[name] = {"ms": round(ms, 4), "samples_per_s": round(batch / ms * 1e3, 1), "batch": batch}
        print(name, results[name], flush=True)
        tr.close()

    for mode, mname in ((0, "3xtf32"), (1, "tf32")):
        step_rate(f"mlp 784-512-256-10 train step, batch 128, {mname}", mlp_specs(), 128, (784, 1, 1), mlp_batch(128, 0, be), mode)
        step_rate(f"cnn-mnist-422k train step, batch 64, {mname}", cnn_specs(MNIST_CNN), 64, (1, 28, 28), synthetic_batch(MNIST_CNN, 64, 0, 0, be), mode)
    results["_peaks"] = {"hbm_gbs": hbm_peak, "tf32_tflops": tf32_peak, "source": src}
    if args.out:
        os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
        json.dump(results, open(args.out, "w"), indent=1)


if __name__ == "__main__":
    main()
