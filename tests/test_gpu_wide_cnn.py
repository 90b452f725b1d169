"""The workload the benchmark times, against the oracle: the wide CNN (3 -> 128 -> 256 channels on 32x32, fc 16384 ->
1024 -> 10) through the fused TF32 step with the implicit-GEMM second convolution and BatchNorm statistics from the
GEMM epilogue, compared with the oracle running the reference's primitive-call step (crates/weta/examples/
mnist_cnn.rs:63-73) with its contraction operands read as TF32.  The model to follow is the reference's own step
test, crates/weta/tests/cuda_parity.rs:230-273."""
import numpy as np
import pytest

from oracle.mirror import nn
from oracle.mirror.models import build_cnn, primitive_train_step, synthetic_batch
from oracle.mirror.tensor import Tensor
from test_gpu_fused import TF32, _check_cnn
from weta_b200 import core
from weta_b200.core import manual_seed
from weta_b200.trainer import DROPOUT, FusedTrainer, cnn_specs
from weta_b200.workloads import WIDE_CNN, CnnConfig

pytestmark = pytest.mark.gpu


def test_wide_cnn_fused_tf32_step_matches_the_oracle(tf32_oracle, gpu, report):
    """Batch 32 (the oracle needs about a second per step), two Adam steps.  First loss to 5e-5 (measured 5e-7).  Every
    gradient's 2-norm to 3e-2 (measured 1.0e-2..1.4e-2; a plain-f32 oracle sits at 2.5e-2..4.8e-2 from the same run): at
    this batch the model amplifies perturbations ~1e4-fold in its first layers (see _check_cnn), and each contraction by
    itself is pinned to 2e-5 by the next test.  The second loss is checked to 1 % only: Adam's first update moves each
    of fc1's 16.8 M weights by lr in the direction of its gradient's sign, so the loss on the next batch jumps to ~40
    and the entries whose gradient is rounding noise around zero go either way."""
    _check_cnn(tf32_oracle, gpu, WIDE_CNN, 32, TF32, grad_norm_tol=3e-2, tf32_operands=True, steps=2, loss_tol=1e-2, report=report,
               name="cnn-wide-17M batch 32")


def test_wide_cnn_fp32_step_matches_the_plain_oracle(oracle, gpu, report):
    """The same model and batch with FP32 contractions against the plain restatement of weta-cpu: every gradient to 1e-5 in
    the 2-norm except the first block's (conv weight, BatchNorm weight / bias), whose conditioning leaves 1e-3..3e-3."""
    _check_cnn_fp32_wide(oracle, gpu, report)


def _check_cnn_fp32_wide(oracle, gpu, report):
    cfg, batch = WIDE_CNN, 32
    ref = build_cnn(cfg, oracle, 42)
    opt = nn.Adam(ref.parameters(), 1e-3)
    manual_seed(42)
    tr = FusedTrainer(gpu, cnn_specs(cfg), batch, (cfg.in_ch, cfg.hw, cfg.hw), lr=1e-3, matmul_mode=2)
    tr.init_from_global_rng()
    state = core.global_rng().state
    x, y = synthetic_batch(cfg, batch, 0, 0, oracle)
    want_loss = primitive_train_step(ref, opt, x, y)
    core.global_rng().state = state
    tr.stage(x.numpy(), y.numpy())
    tr.forward_backward()
    errs = {}
    for i, (n, p) in enumerate(ref.named_parameters()):
        g = p.grad.numpy().reshape(-1)
        errs[n] = float(np.linalg.norm(tr.get_grad(i) - g) / max(np.linalg.norm(g), 1e-30))
    report("wide CNN FP32 vs plain oracle, batch 32", loss=(tr.loss(), want_loss), grad_norm_err=errs)
    assert abs(tr.loss() - want_loss) < 5e-6
    for n, e in errs.items():
        if n in ("0.bias", "4.bias"):
            continue  # zero true gradient
        assert e < (1e-2 if n in ("0.weight", "1.weight", "1.bias") else 1e-5), (n, e)
    tr.close()


def test_wide_cnn_contractions_match_the_oracle_on_tf32_operands(tf32_oracle, gpu, report):
    """Every tensor-core contraction of the wide CNN by itself, at the model's shapes and batch 32, N(0,1) operands, TF32
    mode: the second convolution through the implicit GEMM (forward, input gradient, weight gradient), fc1 (forward,
    both gradients) and the first convolution's weight gradient through the trait chain, each against the oracle
    contracting the same operands truncated to TF32 with a double accumulator.  Largest error over an output <= 5e-5 of
    the output's rms (measured 1e-6..3.5e-5).  The first convolution's forward product through Backend::matmul has
    rows of 27 floats, which TMA cannot read (pitch not a multiple of 16 bytes): it runs on the CUDA cores in FP32 and
    is compared with the plain oracle instead."""
    from test_gpu_fullsize import P, randn
    from weta_b200.core import DType, Layout
    from weta_b200.trainer import _declare
    from oracle.mirror.autograd import Var

    lib, H = gpu.lib, gpu.handle
    _declare(lib)
    gpu.set_matmul_mode(TF32)
    errs = {}

    def rel(got, want):
        return float(np.abs(got.astype(np.float64) - want).max() / np.sqrt((want.astype(np.float64) ** 2).mean()))

    def fetch(storage, shape):
        return gpu.to_host(storage, Layout.contiguous(shape), DType.F32).reshape(shape)

    try:
        # conv2: [32,128,16,16] * [256,128,3,3] + bias
        n, c, h, w, o = 32, 128, 16, 16, 256
        xo, wo, bo, go = randn([n, c, h, w], 1, tf32_oracle), randn([o, c, 3, 3], 2, tf32_oracle), randn([o], 3, tf32_oracle), randn([n, o, h, w], 4, tf32_oracle)
        xv, wv, bv = Var(xo, requires_grad=True), Var(wo, requires_grad=True), Var(bo, requires_grad=True)
        yv = nn.conv2d(xv, wv, bv, stride=(1, 1), padding=(1, 1))
        yv.mul(Var(go)).sum().backward()
        xg, wg, bg, gg = randn([n, c, h, w], 1, gpu), randn([o, c, 3, 3], 2, gpu), randn([o], 3, gpu), randn([n, o, h, w], 4, gpu)
        ys, dxs, dws = gpu.alloc(n * o * h * w, DType.F32), gpu.alloc(n * c * h * w, DType.F32), gpu.alloc(o * c * 9, DType.F32)
        gpu.check(lib.wb_conv3x3_fwd(H, P(xg.storage.ptr), P(wg.storage.ptr), P(bg.storage.ptr), n, c, h, w, o, P(ys.ptr)))
        gpu.check(lib.wb_conv3x3_bwd(H, P(xg.storage.ptr), P(wg.storage.ptr), P(gg.storage.ptr), n, c, h, w, o, P(dxs.ptr), P(dws.ptr)))
        errs["conv2 y"] = rel(fetch(ys, [n, o, h, w]), yv.numpy())
        errs["conv2 dx"] = rel(fetch(dxs, [n, c, h, w]), xv.grad.numpy())
        errs["conv2 dw"] = rel(fetch(dws, [o, c, 3, 3]), wv.grad.numpy())
        # fc1: [32,16384] x [1024,16384]^T + bias, ReLU off
        n, fin, fout = 32, 16384, 1024
        xo, wo, bo, go = randn([n, fin], 5, tf32_oracle), randn([fout, fin], 6, tf32_oracle), randn([fout], 7, tf32_oracle), randn([n, fout], 8, tf32_oracle)
        xv, wv, bv = Var(xo, requires_grad=True), Var(wo, requires_grad=True), Var(bo, requires_grad=True)
        yv = nn.linear(xv, wv, bv)
        yv.mul(Var(go)).sum().backward()
        xg, wg, bg, gg = randn([n, fin], 5, gpu), randn([fout, fin], 6, gpu), randn([fout], 7, gpu), randn([n, fout], 8, gpu)
        ys, dxs, dws, dbs = gpu.alloc(n * fout, DType.F32), gpu.alloc(n * fin, DType.F32), gpu.alloc(fout * fin, DType.F32), gpu.alloc(fout, DType.F32)
        gpu.check(lib.wb_linear_fwd(H, P(xg.storage.ptr), P(wg.storage.ptr), P(bg.storage.ptr), n, fin, fout, 0, P(ys.ptr)))
        gpu.check(lib.wb_linear_bwd(H, P(xg.storage.ptr), P(wg.storage.ptr), P(gg.storage.ptr), n, fin, fout, P(dxs.ptr), P(dws.ptr), P(dbs.ptr)))
        errs["fc1 y"] = rel(fetch(ys, [n, fout]), yv.numpy())
        errs["fc1 dx"] = rel(fetch(dxs, [n, fin]), xv.grad.numpy())
        errs["fc1 dw"] = rel(fetch(dws, [fout, fin]), wv.grad.numpy())
        errs["fc1 db"] = rel(fetch(dbs, [fout]), bv.grad.numpy())
        # conv1: [32,3,32,32] * [128,3,3,3] + bias through the trait chain (im2col, matmul, add) on both sides
        out = {}
        for name, be in (("cpu", tf32_oracle), ("gpu", gpu)):
            xv = Var(randn([32, 3, 32, 32], 9, be))
            wv, bv = Var(randn([128, 3, 3, 3], 10, be), requires_grad=True), Var(randn([128], 11, be), requires_grad=True)
            yv = nn.conv2d(xv, wv, bv, stride=(1, 1), padding=(1, 1))
            yv.mul(Var(randn([32, 128, 32, 32], 12, be))).sum().backward()
            out[name] = (yv.numpy(), wv.grad.numpy())
        errs["conv1 dw"] = rel(out["gpu"][1], out["cpu"][1])
        tf32_oracle.set_matmul_test_mode(0, True)  # plain operands for the product that runs in FP32 on the GPU
        y_plain = nn.conv2d(Var(randn([32, 3, 32, 32], 9, tf32_oracle)), Var(randn([128, 3, 3, 3], 10, tf32_oracle)), Var(randn([128], 11, tf32_oracle)),
                            stride=(1, 1), padding=(1, 1)).numpy()
        errs["conv1 y (FP32 path)"] = rel(out["gpu"][0], y_plain)
        gpu.gemm_check()
    finally:
        gpu.set_matmul_mode(0)
    report("wide CNN contractions, TF32 mode vs oracle on TF32 operands", max_err_over_rms=errs)
    for k, e in errs.items():
        assert e <= 5e-5, (k, e)



def test_batch_norm_statistics_survive_channel_means_far_above_the_spread(tf32_oracle, gpu, report):
    """Convolution biases of 30 and 1000 against activations of spread ~0.3: the GEMM epilogue accumulates its sums
    about the bias, and channels whose sums still cancel are recomputed from the activation, so the fused step's
    gradients keep matching the oracle's two-pass statistics (crates/weta-nn/src/functional.rs:144-180)."""
    cfg = CnnConfig("cnn-implicit", 3, 16, 128, 32, 64)
    batch = 16
    ref = build_cnn(cfg, tf32_oracle, 42)
    manual_seed(42)
    tr = FusedTrainer(gpu, cnn_specs(cfg), batch, (cfg.in_ch, cfg.hw, cfg.hw), lr=1e-3, matmul_mode=TF32)
    tr.init_from_global_rng()
    names = [n for n, _ in ref.named_parameters()]
    rng = np.random.default_rng(3)
    for conv_bias, scale in (("0.bias", 30.0), ("4.bias", 1000.0)):
        i = names.index(conv_bias)
        p = ref.parameters()[i]
        vals = (scale * (1.0 + 0.1 * rng.standard_normal(p.numpy().size))).astype(np.float32)
        p.data.assign(Tensor.from_numpy(vals.reshape(p.numpy().shape), tf32_oracle))
        tr.set_param(i, vals)
    # The first convolution sees all-positive pixels: shift its weights so its raw output also has a large mean.
    i = names.index("0.weight")
    w = ref.parameters()[i].numpy() + np.float32(0.5)
    ref.parameters()[i].data.assign(Tensor.from_numpy(w, tf32_oracle))
    tr.set_param(i, w)
    opt = nn.Adam(ref.parameters(), 1e-3)
    state = core.global_rng().state
    x, y = synthetic_batch(cfg, batch, 0, 0, tf32_oracle)
    want_loss = primitive_train_step(ref, opt, x, y)
    want = [p.grad.numpy().reshape(-1) for p in ref.parameters()]
    core.global_rng().state = state
    tr.stage(x.numpy(), y.numpy())
    tr.forward_backward()
    errs = {}
    for k, g in enumerate(want):
        if names[k] in ("0.bias", "4.bias"):
            continue
        errs[names[k]] = float(np.linalg.norm(tr.get_grad(k) - g) / max(np.linalg.norm(g), 1e-20))
    report("BN statistics with large channel means", loss=(tr.loss(), want_loss), grad_norm_err=errs)
    # With |mean| / spread up to ~3000 the f32 activations themselves carry ~1e-4 of the spread as rounding noise,
    # which BatchNorm's 1 / std amplifies on both sides alike: 2e-2 on gradient 2-norms, 1e-3 on the loss.
    assert abs(tr.loss() - want_loss) < 1e-3, (tr.loss(), want_loss)
    for n, e in errs.items():
        assert e < 2e-2, (n, e)
    bufs = dict(ref.buffers())
    for k, idx in ((0, "1"), (1, "5")):
        rm, rv = tr.bn_buffers(k)
        assert np.allclose(rm, bufs[f"{idx}.running_mean"].numpy(), rtol=1e-5, atol=1e-5)
        assert np.allclose(rv, bufs[f"{idx}.running_var"].numpy(), rtol=2e-3, atol=1e-6)
    gpu.gemm_check()
    tr.close()


def test_dropout_with_p_zero_draws_no_seed(oracle, gpu):
    """F::dropout returns before Tensor::rand when p = 0 (crates/weta-nn/src/functional.rs:66-71), so such a layer must
    leave the host generator where it was: the fused trainer and the primitive step then keep seeing the same seeds."""
    cfg = CnnConfig("tiny-p0", 3, 8, 8, 16, 32, dropout=0.0)
    ref = build_cnn(cfg, oracle, 7)
    opt = nn.Adam(ref.parameters(), 1e-3)
    manual_seed(7)
    tr = FusedTrainer(gpu, cnn_specs(cfg), 8, (3, 8, 8), lr=1e-3, matmul_mode=2)
    tr.init_from_global_rng()
    assert tr.n_dropout == 0 and sum(1 for s in tr.specs if s[0] == DROPOUT) == 2
    state = core.global_rng().state
    losses = []
    for step in range(2):
        x, y = synthetic_batch(cfg, 8, step, 0, oracle)
        losses.append(primitive_train_step(ref, opt, x, y))
    assert core.global_rng().state == state, "the primitive step drew a seed for a p = 0 dropout"
    for step in range(2):
        x, y = synthetic_batch(cfg, 8, step, 0, oracle)
        tr.stage(x.numpy(), y.numpy())
        tr.forward_backward()
        tr.adam_step()
        assert abs(tr.loss() - losses[step]) < 2e-4
    assert core.global_rng().state == state, "the fused trainer drew a seed for a p = 0 dropout"
    tr.close()


def test_batch_norm_backward_sums_with_unusable_gamma(oracle, gpu, report):
    """The backward sums of BatchNorm -> ReLU -> pool normally come from the pooled tensors (xhat at a window's winner is
    (y - beta) / gamma); channels whose gamma is zero, tiny, or far below |beta| must be summed from the activation
    instead.  Both kinds of channel in one layer, FP32 contractions, against the oracle's autograd chain."""
    cfg = CnnConfig("cnn-implicit", 3, 16, 128, 32, 64)
    batch = 16
    ref = build_cnn(cfg, oracle, 42)
    manual_seed(42)
    tr = FusedTrainer(gpu, cnn_specs(cfg), batch, (cfg.in_ch, cfg.hw, cfg.hw), lr=1e-3, matmul_mode=2)
    tr.init_from_global_rng()
    names = [n for n, _ in ref.named_parameters()]
    rng = np.random.default_rng(8)
    for bn in ("1", "5"):
        gi, bi = names.index(f"{bn}.weight"), names.index(f"{bn}.bias")
        c = ref.parameters()[gi].numpy().size
        gamma = (1.0 + 0.2 * rng.standard_normal(c)).astype(np.float32)
        beta = (0.3 * rng.standard_normal(c)).astype(np.float32)
        gamma[0::4] = 0.0          # no slope at all
        gamma[1::4] = 1e-8         # tiny
        beta[2::4] = 100.0         # |beta| far above 64 |gamma|
        for i, v in ((gi, gamma), (bi, beta)):
            ref.parameters()[i].data.assign(Tensor.from_numpy(v, oracle))
            tr.set_param(i, v)
    opt = nn.Adam(ref.parameters(), 1e-3)
    state = core.global_rng().state
    x, y = synthetic_batch(cfg, batch, 0, 0, oracle)
    want_loss = primitive_train_step(ref, opt, x, y)
    core.global_rng().state = state
    tr.stage(x.numpy(), y.numpy())
    tr.forward_backward()
    errs = {}
    for k, (n, p) in enumerate(ref.named_parameters()):
        if n in ("0.bias", "4.bias"):
            continue
        g = p.grad.numpy().reshape(-1)
        errs[n] = float(np.abs(tr.get_grad(k) - g).max() / max(np.abs(g).max(), 1e-20))
    report("BN backward sums with unusable gamma", loss=(tr.loss(), want_loss), grad_max_err=errs)
    assert abs(tr.loss() - want_loss) < 2e-4
    for n, e in errs.items():
        assert e < 2e-3, (n, e)
    tr.close()


@pytest.mark.parametrize("batch", [48, 512])
def test_first_block_backward_fused_with_its_weight_gradient(gpu, report, batch):
    """The first block's BatchNorm+ReLU+pool backward and the convolution's weight gradient as one kernel (the output
    gradient never reaches memory) against the same trainer with the two stand-alone ops: the dconv values are computed
    with the same arithmetic and reach the tensor core as the same TF32 operands, so only the order of the f32
    accumulation differs.  Every other gradient is bit-identical."""
    import os

    cfg = WIDE_CNN  # 48 images x 16 row pairs = 768 steps over 148 CTAs: unequal ranges, some of five steps, some of six; 512: the 8-GPU rank
    rng = np.random.default_rng(3)
    x = rng.random((batch, cfg.in_ch, cfg.hw, cfg.hw), dtype=np.float32)
    y = rng.integers(0, cfg.classes, batch).astype(np.int64)
    gamma = (1.0 + 0.3 * rng.standard_normal(cfg.c1)).astype(np.float32)
    beta = (0.2 * rng.standard_normal(cfg.c1)).astype(np.float32)
    grads = {}
    for fused in (False, True):
        os.environ["WETA_B200_NO_FUSED_CONV1_BWD"] = "0" if fused else "1"
        try:
            manual_seed(11)
            tr = FusedTrainer(gpu, cnn_specs(cfg), batch, (cfg.in_ch, cfg.hw, cfg.hw), lr=1e-3, matmul_mode=TF32)
            tr.init_from_global_rng()
            # BatchNorm parameters away from their initial 1 / 0, so every term of dx is exercised
            tr.set_param(2, gamma)
            tr.set_param(3, beta)
            tr.stage(x, y)
            manual_seed(5)
            tr.forward_backward()
            gpu.gemm_check()
            grads[fused] = [tr.get_grad(i) for i in range(len(tr.ranges))]
            loss = tr.loss()
            grads[("loss", fused)] = loss
            tr.close()
        finally:
            os.environ.pop("WETA_B200_NO_FUSED_CONV1_BWD", None)
    assert grads[("loss", True)] == grads[("loss", False)]
    a, b = grads[False], grads[True]
    dw_err = float(np.linalg.norm(a[0] - b[0]) / np.linalg.norm(a[0]))
    # the bias gradient of a convolution followed by BatchNorm is rounding noise around zero: compare on the scale of
    # the sum of |dconv| it is the residue of, which the weight gradient's magnitude stands for
    db_err = float(np.abs(a[1] - b[1]).max() / max(float(np.abs(a[0]).max()), 1e-30))
    report(f"first-block fused backward, batch {batch}", dw_rel_l2=dw_err, dbias_abs_over_dw_max=db_err)
    # 1.7e-6 at batch 48, 1.4e-5 at batch 512 (measured): the two paths split the contraction over images and pixels into
    # different partial sums, and the tensor core adds into its f32 accumulator with truncation (about 2^-24 of the
    # running sum per product), so the difference grows with the length of the contraction
    assert dw_err < (5e-6 if batch <= 64 else 5e-5), dw_err
    assert db_err < 1e-4, db_err
    for i in range(2, len(a)):
        assert np.array_equal(a[i], b[i]), i
