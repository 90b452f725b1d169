"""Pins the CPU oracle to the reference's PyTorch fixture (f64, 1e-9), test for test with
crates/weta/tests/reference.rs."""
import numpy as np
import pytest

from oracle.mirror import nn
from oracle.mirror.autograd import Var
from oracle.mirror.tensor import Tensor


def close(name, got, want):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{name}: shape {got.shape} vs {want.shape}"
    bad = np.abs(got - want) > 1e-9 + 1e-9 * np.abs(want)
    assert not bad.any(), f"{name}: max err {np.abs(got - want).max()}"


def leaf(be, g, name):
    return Var(Tensor.from_numpy(g[name], be), requires_grad=True)


def test_mlp_with_label_smoothing(oracle, golden):  # reference.rs:31-43
    g = golden
    x, w1, b1, w2, b2 = (leaf(oracle, g, f"mlp.{n}") for n in ("x", "w1", "b1", "w2", "b2"))
    logits = nn.linear(nn.relu(nn.linear(x, w1, b1)), w2, b2)
    loss = logits.cross_entropy(Tensor.from_numpy(g["mlp.y"], oracle), "mean", 0.1)
    loss.backward()
    close("logits", logits.numpy(), g["mlp.logits"])
    close("loss", loss.numpy(), g["mlp.loss"])
    for n, t in (("x", x), ("w1", w1), ("b1", b1), ("w2", w2), ("b2", b2)):
        close(n, t.grad.numpy(), g[f"mlp.grad.{n}"])


def test_cnn_with_batch_norm(oracle, golden):  # reference.rs:45-63
    g, be = golden, oracle
    x, w, b, gamma, beta = (leaf(be, g, f"cnn.{n}") for n in ("x", "w", "b", "gamma", "beta"))
    rm = Tensor.from_numpy(np.zeros(3), be)
    rv = Tensor.from_numpy(np.ones(3), be)
    h = nn.conv2d(x, w, b, (1, 1), (1, 1))
    h = nn.batch_norm(h, rm, rv, gamma, beta, True, 0.1, 1e-5)
    h = nn.max_pool2d(nn.relu(h), 2, 2)
    loss = nn.mse_loss(h, Var(Tensor.from_numpy(g["cnn.target"], be)))
    loss.backward()
    close("out", h.numpy(), g["cnn.out"])
    close("loss", loss.numpy(), g["cnn.loss"])
    close("running_mean", rm.numpy(), g["cnn.running_mean"])
    close("running_var", rv.numpy(), g["cnn.running_var"])
    for n, t in (("x", x), ("w", w), ("b", b), ("gamma", gamma), ("beta", beta)):
        close(n, t.grad.numpy(), g[f"cnn.grad.{n}"])


def test_strided_conv_and_padded_avg_pool(oracle, golden):  # reference.rs:65-74
    g, be = golden, oracle
    x, w = leaf(be, g, "conv2.x"), leaf(be, g, "conv2.w")
    h = nn.avg_pool2d(nn.conv2d(x, w, None, (2, 2), (0, 0)), 2, 2, 1)
    close("out", h.numpy(), g["conv2.out"])
    h.mul(Var(Tensor.from_numpy(g["conv2.g"], be))).sum().backward()
    close("grad x", x.grad.numpy(), g["conv2.grad.x"])
    close("grad w", w.grad.numpy(), g["conv2.grad.w"])


@pytest.mark.parametrize("name,f", [
    ("softmax", lambda t: t.softmax(1)),
    ("log_softmax", lambda t: t.log_softmax(1)),
    ("gelu", nn.gelu),
    ("gelu_tanh", nn.gelu_tanh),
    ("silu", nn.silu),
    ("layer_norm", lambda t: nn.layer_norm(t, 1, None, None, 1e-5)),
    ("logsumexp", lambda t: t.logsumexp(1, False)),
])
def test_functions_forward_and_backward(oracle, golden, name, f):  # reference.rs:76-96
    g, be = golden, oracle
    z = leaf(be, g, "fn.z")
    r = f(z)
    close(name, r.numpy(), g[f"fn.{name}.out"])
    r.mul(Var(Tensor.from_numpy(g[f"fn.{name}.g"], be))).sum().backward()
    close(name + " grad", z.grad.numpy(), g[f"fn.{name}.grad"])


@pytest.mark.parametrize("name,make", [
    ("sgd", lambda ps: nn.SGD(ps, 0.1, momentum=0.9, nesterov=True, weight_decay=0.01)),
    ("adam", lambda ps: nn.Adam(ps, 0.01, betas=(0.8, 0.99), weight_decay=0.1)),
    ("adamw", lambda ps: nn.AdamW(ps, 0.01, weight_decay=0.1)),
])
def test_optimisers_match_pytorch(oracle, golden, name, make):  # reference.rs:98-114
    g, be = golden, oracle
    p = Var(Tensor.from_numpy(g["opt.p0"].copy(), be), requires_grad=True)
    opt = make([p])
    for i in range(3):
        p.grad = Tensor.from_numpy(g[f"opt.grad{i}"], be)
        opt.step()
    close(name, p.numpy(), g[f"opt.{name}"])
