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
    """Batch 32 (the oracle needs about a second per step), two Adam steps: first loss to 2e-4, every gradient's
    2-norm to 1e-3.  The second loss is checked to 1 % only: Adam's first update moves each of fc1's 16.8 M weights
    by lr in the direction of its gradient's sign, so the loss on the next batch jumps to ~40 and the entries whose
    gradient is rounding noise around zero go either way."""
    _check_cnn(tf32_oracle, gpu, WIDE_CNN, 32, TF32, tf32_operands=True, steps=2, loss_tol=1e-2, report=report, name="cnn-wide-17M batch 32")


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
