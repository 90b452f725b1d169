"""Training-step parity in primitive mode: the same primitive-call stream on the CUDA backend and on
the CPU oracle (crates/weta/tests/cuda_parity.rs:230-273, and the MLP / CNN configs)."""
import numpy as np
import pytest

from oracle.mirror import nn
from oracle.mirror.autograd import Var
from weta_b200.core import Distribution, DType, manual_seed
from oracle.mirror.tensor import Tensor, allclose
from weta_b200.workloads import MNIST_CNN
from oracle.mirror.models import build_cnn, mlp_batch, primitive_train_step, synthetic_batch

pytestmark = pytest.mark.gpu


def test_training_step_matches_cpu(oracle, gpu):  # cuda_parity.rs:230-273
    def make(be):
        manual_seed(3)
        return nn.Sequential(nn.Conv2d(1, 4, 3, be, padding=1), nn.BatchNorm2d(4, be), nn.ReLU(), nn.MaxPool2d(2),
                             nn.Flatten(), nn.Linear(4 * 4 * 4, 10, be))

    cpu, dev = make(oracle), make(gpu)
    for (n, a), (_, b) in zip(cpu.state_dict().items(), dev.state_dict().items()):
        assert np.array_equal(a.numpy(), b.numpy()), f"initial {n} differs"
    x = Tensor.random_seeded([8, 1, 8, 8], Distribution.normal(0.0, 1.0), DType.F32, oracle, 11)
    y = Tensor.random_seeded([8], Distribution.uniform(0.0, 10.0), DType.I64, oracle, 12)
    # SGD, not Adam: the conv bias feeds BatchNorm, its true gradient is ~0 (cuda_parity.rs:251-253)
    o1 = nn.SGD(cpu.parameters(), 0.1, momentum=0.9)
    o2 = nn.SGD(dev.parameters(), 0.1, momentum=0.9)
    for _ in range(3):
        l1 = nn.cross_entropy(cpu(Var(x)), y)
        o1.zero_grad(); l1.backward(); o1.step()
        l2 = nn.cross_entropy(dev(Var(x.to_backend(gpu))), y.to_backend(gpu))
        o2.zero_grad(); l2.backward(); o2.step()
        assert abs(l1.item() - l2.item()) < 1e-4
        for p, q in zip(cpu.parameters(), dev.parameters()):
            assert allclose(q.grad.numpy(), p.grad.numpy(), 1e-3, 1e-3)
    for (n, a), (_, b) in zip(cpu.state_dict().items(), dev.state_dict().items()):
        assert allclose(b.numpy(), a.numpy(), 1e-3, 1e-3), n


def _adam_params_close(name, dev, cpu, steps, lr):
    d = np.abs(dev.astype(np.float64) - cpu.astype(np.float64))
    # Hard bound: Adam moves a parameter by at most ~lr per step, so two runs can differ by 2*steps*lr.
    assert d.max() <= 2 * steps * lr * 1.01, f"{name}: max |diff| {d.max()}"
    # Typical: rounding-level agreement; only parameters whose true gradient is ~0 may flip direction.
    frac = float((d > 1e-5 + 1e-4 * np.abs(cpu)).mean())
    assert frac < 2e-3, f"{name}: {frac:.2%} of elements differ by more than 1e-5"


def test_mlp_ten_adam_steps(oracle, gpu):
    """784-512-256-10, ReLU + Dropout(0.1), batch 128, Adam lr 1e-3, seed 42: loss every step,
    gradients at steps 0 and 9, parameters after 10 steps."""
    models, opts = [], []
    for be in (oracle, gpu):
        manual_seed(42)
        m = nn.mlp(be, 0.1)
        models.append(m)
        opts.append(nn.Adam(m.parameters(), 1e-3))
    # Both runs draw dropout seeds from the global generator: replay it per backend.
    from weta_b200 import core
    losses = [[], []]
    grads = [{}, {}]
    for i, be in enumerate((oracle, gpu)):
        core._global_rng = core.Pcg(4242)
        for step in range(10):
            x, y = mlp_batch(128, step, be)
            losses[i].append(primitive_train_step(models[i], opts[i], x, y))
            if step in (0, 9):
                grads[i][step] = [p.grad.numpy() for p in models[i].parameters()]
    for a, b in zip(*losses):
        assert abs(a - b) < 1e-4, (losses[0], losses[1])
    for step in (0, 9):
        for gc, gg in zip(grads[0][step], grads[1][step]):
            assert np.abs(gg - gc).max() <= 1e-3 * max(np.abs(gc).max(), 1e-6)
    for (n, pc), (_, pg) in zip(models[0].named_parameters(), models[1].named_parameters()):
        _adam_params_close(n, pg.numpy(), pc.numpy(), 10, 1e-3)


def test_cnn_three_adam_steps(oracle, gpu):
    """The 422k-parameter conv-BN CNN, batch 64, Adam lr 1e-3: loss, gradients and state after 3 steps."""
    from weta_b200 import core
    runs = []
    for be in (oracle, gpu):
        model = build_cnn(MNIST_CNN, be, 42)
        opt = nn.Adam(model.parameters(), 1e-3)
        core._global_rng = core.Pcg(777)
        losses = []
        for step in range(3):
            x, y = synthetic_batch(MNIST_CNN, 64, step, 0, be)
            losses.append(primitive_train_step(model, opt, x, y))
        runs.append((model, losses, [p.grad.numpy() for p in model.parameters()]))
    (mc, lc, gc), (mg, lg, gg) = runs
    for a, b in zip(lc, lg):
        assert abs(a - b) < 2e-4, (lc, lg)
    for (n, _), a, b in zip(mc.named_parameters(), gc, gg):
        if n in ("0.bias", "4.bias"):
            continue  # conv bias before BatchNorm: true gradient is zero, what is left is rounding noise
        assert np.abs(b - a).max() <= 2e-3 * max(np.abs(a).max(), 1e-6), n
    for (n, pc), (_, pg) in zip(mc.named_parameters(), mg.named_parameters()):
        if n in ("0.bias", "4.bias"):
            assert np.abs(pg.numpy() - pc.numpy()).max() <= 2 * 3 * 1e-3 * 1.01
        else:
            _adam_params_close(n, pg.numpy(), pc.numpy(), 3, 1e-3)
    for (n, bc), (_, bg) in zip(mc.buffers(), mg.buffers()):
        # The running mean sits downstream of the noise-driven conv bias (it shifts with it one for one),
        # so it inherits that bound scaled by the momentum; the variance does not depend on the bias.
        tol = (0.0, 3 * 1e-3) if n.endswith("running_mean") else (1e-4, 1e-5)
        assert allclose(bg.numpy(), bc.numpy(), *tol), n


def test_gradcheck_on_the_gpu(gpu):  # cuda_parity.rs:214-228
    """f64 central differences through conv2d -> relu -> max_pool2d -> softmax on the CUDA backend (every primitive in
    f64: im2col, the CUDA-core matmul, reductions, element-wise ops), eps 1e-5, tolerance 1e-6 like the reference."""
    from oracle.mirror.gradcheck import gradcheck

    manual_seed(5)
    leaf = lambda s: Var(Tensor.randn(s, DType.F64, gpu), requires_grad=True)
    x, w, b = leaf([2, 2, 5, 5]), leaf([3, 2, 3, 3]), leaf([3])
    f = lambda t: nn.max_pool2d(nn.conv2d(t[0], t[1], t[2], stride=(1, 1), padding=(1, 1)).relu(), 2, 2).softmax(1)
    assert gradcheck(f, [x, w, b]) is None
