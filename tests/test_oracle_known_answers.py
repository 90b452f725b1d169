"""Pins the CPU oracle to the literal answers in the reference's own unit tests."""
import numpy as np

from weta_b200.core import (DType, Distribution, Im2ColParams, Layout, Pcg, broadcast_shapes, resolve_shape,
                            splitmix64)
from oracle.mirror.tensor import Tensor
from oracle.mirror.autograd import Var
from oracle.mirror import nn


def T(be, a, dtype=np.float32):
    return Tensor.from_numpy(np.asarray(a, dtype=dtype), be)


def test_matmul_with_transposed_input(oracle):  # crates/weta-cpu/src/lib.rs:577-585
    a = T(oracle, [[[1, 2, 3], [4, 5, 6]]])
    b = T(oracle, [[[1, 0, 1], [0, 1, 1]]]).transpose(1, 2)
    assert a.matmul(b).numpy().reshape(-1).tolist() == [4, 5, 10, 11]


def test_reduce_over_middle_axis(oracle):  # crates/weta-cpu/src/lib.rs:588-595
    x = T(oracle, np.arange(24).reshape(2, 3, 4), np.float64)
    assert x.sum_dims([1]).numpy().reshape(-1).tolist() == [12, 15, 18, 21, 48, 51, 54, 57]
    assert x.argmax(2).numpy().reshape(-1).tolist() == [3] * 6


def test_im2col_then_col2im_counts_overlaps(oracle):  # crates/weta-cpu/src/lib.rs:598-607
    x = T(oracle, np.ones((1, 1, 3, 3)))
    p = Im2ColParams((2, 2))
    cols = x.im2col(p)
    assert cols.shape == (1, 4, 4)
    assert cols.col2im(p, (1, 3, 3)).numpy().reshape(-1).tolist() == [1, 2, 1, 2, 4, 2, 1, 2, 1]


def test_layout_offsets_and_broadcasting():  # crates/weta-core/src/layout.rs:265-302
    l = Layout.contiguous([2, 3, 4])
    assert l.strides == (12, 4, 1) and l.is_contiguous()
    t = l.transpose(1, 2)
    assert t.shape == (2, 4, 3) and not t.is_contiguous()
    assert Layout.contiguous([2, 3]).transpose(0, 1).offsets().tolist() == [0, 3, 1, 4, 2, 5]
    assert Layout.contiguous([3, 4]).narrow(1, 1, 2).offsets().tolist() == [1, 2, 5, 6, 9, 10]
    assert broadcast_shapes([64, 1], [10]) == [64, 10]
    assert broadcast_shapes([2, 1, 3], [4, 1]) == [2, 4, 3]
    b = Layout.contiguous([3]).broadcast_to([2, 3])
    assert b.strides == (0, 1) and b.offsets().tolist() == [0, 1, 2, 0, 1, 2]
    assert resolve_shape(12, [-1, 4]) == [3, 4]


def test_tensor_unit_answers(oracle):  # crates/weta-tensor/src/lib.rs:32-92
    a = T(oracle, [[1, 2, 3], [4, 5, 6]])
    assert a.add(T(oracle, [10, 20, 30])).numpy().tolist() == [[11, 22, 33], [14, 25, 36]]
    b = T(oracle, [[1, 2], [3, 4], [5, 6]])
    assert a.matmul(b).numpy().reshape(-1).tolist() == [22, 28, 49, 64]
    assert a.matmul(a.t()).numpy().reshape(-1).tolist() == [14, 32, 32, 77]
    x = T(oracle, np.ones((1, 1, 3, 3)))
    w = T(oracle, np.ones((1, 1, 2, 2)))
    assert x.conv2d(w, None, 1, 0).numpy().reshape(-1).tolist() == [4, 4, 4, 4]
    m = T(oracle, [[[[1, 7, 2, 4], [3, 0, 1, 1], [9, 2, 6, 5], [1, 1, 0, 3]]]])
    assert m.max_pool2d(2, 2).numpy().reshape(-1).tolist() == [7, 4, 9, 6]


def test_adam_first_step_matches_pytorch(oracle):  # crates/weta-optim/src/lib.rs:313-321
    p = Var(T(oracle, [1.0, -2.0]), requires_grad=True)
    opt = nn.Adam([p], 0.01)
    p.mul(Var(T(oracle, [3.0, -0.5]))).sum().backward()
    opt.step()
    v = p.numpy()
    assert abs(v[0] - 0.99) < 1e-6 and abs(v[1] + 1.99) < 1e-6


def test_dropout_values(oracle):  # crates/weta/tests/nn.rs:109-113: p = 0.5 gives only 0 or 2
    x = Var(Tensor.ones([1000], DType.F32, oracle))
    y = nn.dropout(x, 0.5, True).numpy()
    assert set(np.unique(y).tolist()) <= {0.0, 2.0}
    assert 350 < (y == 0).sum() < 650


def test_rng_is_the_documented_algorithm(oracle):
    # splitmix64 finaliser: the C++ oracle and the independent Python statement agree.
    for seed, i in [(0, 0), (42, 7), (2**64 - 1, 2**40), (67280421310721, 123456789)]:
        assert oracle.lib.wo_splitmix64(seed, i) == splitmix64(seed, i)
    # repeatability and moments (crates/weta-tensor/src/random.rs:152-180)
    n = Tensor.random_seeded([40000], Distribution.normal(2.0, 3.0), DType.F64, oracle, 5).numpy()
    assert abs(n.mean() - 2.0) < 0.05 and abs(n.std() - 3.0) < 0.05
    u = Tensor.random_seeded([40000], Distribution.uniform(-1.0, 1.0), DType.F32, oracle, 6).numpy()
    assert (u >= -1).all() and (u < 1).all() and abs(u.mean()) < 0.02
    u64 = Tensor.random_seeded([16], Distribution.uniform(0.0, 1.0), DType.F64, oracle, 9).numpy()
    want = [(splitmix64(9, i) >> 11) * 2.0**-53 for i in range(16)]
    assert u64.tolist() == want
    r = Pcg(3)
    xs = np.array([r.uniform() for _ in range(20000)])
    assert abs(xs.mean() - 0.5) < 0.01


def test_integer_semantics(oracle):  # crates/weta-cpu/src/lib.rs:190-241, :552-565
    x, y = T(oracle, [7, -7, 3, -7], np.int64), T(oracle, [2, 2, 3, -2], np.int64)
    assert x.div(y).numpy().tolist() == [3, -4, 1, 4]  # Euclidean division
    assert T(oracle, [-3, 0, 4, 7], np.int64).affine(2.0, 1.0).numpy().tolist() == [-5, 1, 9, 15]
    f = T(oracle, [1.9, -1.9, np.nan, 1e30, -1e30], np.float64).to_dtype(DType.I64).numpy().tolist()
    assert f == [1, -1, 0, 2**63 - 1, -2**63]
    nanmax = T(oracle, [[1.0, np.nan, 3.0]]).max_dims([1]).numpy()
    assert np.isnan(nanmax).all()  # NaN anywhere wins a reduction (dtype.rs:136-149)
    ties = T(oracle, [[2.0, 5.0, 5.0, 1.0]]).argmax(1).numpy().tolist()
    assert ties == [1]


def test_gradcheck_of_a_conv_relu_pool_softmax_chain(oracle):
    """crates/weta-autograd/tests/gradcheck.rs style: f64 central differences, eps 1e-5, tolerance 1e-6, on the chain the
    reference also checks on its GPU backend (crates/weta/tests/cuda_parity.rs:214-228); a wrong backward rule is caught."""
    from oracle.mirror.gradcheck import gradcheck
    from weta_b200.core import manual_seed

    manual_seed(5)
    leaf = lambda s: Var(Tensor.randn(s, DType.F64, oracle), requires_grad=True)
    x, w, b = leaf([2, 2, 5, 5]), leaf([3, 2, 3, 3]), leaf([3])
    f = lambda t: nn.max_pool2d(nn.conv2d(t[0], t[1], t[2], stride=(1, 1), padding=(1, 1)).relu(), 2, 2).softmax(1)
    assert gradcheck(f, [x, w, b]) is None
    wrong = lambda t: t[0].mul(t[0]).detach().mul(t[0])  # d/dx (x^2 x) reported as x^2: must be flagged
    assert gradcheck(wrong, [leaf([3])]) is not None
