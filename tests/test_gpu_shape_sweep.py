"""Exhaustive small shapes: every shape with dims 1..7 in up to three dimensions, under every view the layout type can
express (contiguous, each transposition, a broadcast operand, a slice with an offset, a stepped view), for unary,
binary, reduce, copy and cast.  Integer-valued data, so every comparison with the CPU oracle is exact.  This is the
index-arithmetic net a memory checker would otherwise provide: a wrong bound or stride shows as a wrong element."""
import itertools

import numpy as np
import pytest

from oracle.mirror.tensor import Tensor
from weta_b200.core import BinaryOp as B, DType, UnaryOp as U

pytestmark = pytest.mark.gpu
DIMS = range(1, 8)


def _views(t: Tensor):
    """(name, view) pairs over one tensor; every view keeps at least one element."""
    out = [("contiguous", t)]
    nd = t.ndim
    for a, b in itertools.combinations(range(nd), 2):
        out.append((f"transpose({a},{b})", t.transpose(a, b)))
    for d in range(nd):
        if t.shape[d] >= 3:
            out.append((f"narrow({d})", t.narrow(d, 1, t.shape[d] - 2)))
            out.append((f"step({d})", t.step_by(d, 2)))
    return out


def _pairs(oracle, gpu, arr):
    return Tensor.from_numpy(arr, oracle), Tensor.from_numpy(arr, gpu)


def _shapes():
    for nd in (1, 2, 3):
        yield from itertools.product(DIMS, repeat=nd)


def _eq(name, c: Tensor, g: Tensor):
    cn, gn = c.numpy(), g.numpy()
    assert cn.shape == gn.shape and np.array_equal(cn, gn), name


@pytest.mark.parametrize("dt", [np.float32, np.int64])
def test_unary_binary_copy_over_every_small_shape(oracle, gpu, dt):
    rng = np.random.default_rng(5)
    checked = 0
    for shape in _shapes():
        a = rng.integers(-9, 10, shape).astype(dt)
        b = rng.integers(-9, 10, shape).astype(dt)
        ac, ag = _pairs(oracle, gpu, a)
        bc, bg = _pairs(oracle, gpu, b)
        for (name, vc), (_, vg), (_, wc), (_, wg) in zip(_views(ac), _views(ag), _views(bc), _views(bg)):
            tag = f"{shape} {name}"
            _eq(f"relu {tag}", vc.relu(), vg.relu())
            _eq(f"affine {tag}", vc.affine(2.0, -1.0), vg.affine(2.0, -1.0))
            _eq(f"add {tag}", vc.add(wc), vg.add(wg))
            _eq(f"mul {tag}", vc.mul(wc), vg.mul(wg))
            _eq(f"contiguous {tag}", vc.contiguous(), vg.contiguous())
            _eq(f"cast {tag}", vc.to_dtype(DType.F64), vg.to_dtype(DType.F64))
            # a broadcast operand: the view's last dimension alone, stride 0 everywhere else
            if vc.ndim >= 2:
                rc = vc.narrow(0, 0, 1) if vc.ndim == 2 else vc.narrow(0, 0, 1).narrow(1, 0, 1)
                rg = vg.narrow(0, 0, 1) if vg.ndim == 2 else vg.narrow(0, 0, 1).narrow(1, 0, 1)
                _eq(f"broadcast sub {tag}", vc.sub(rc.broadcast_to(vc.shape)), vg.sub(rg.broadcast_to(vg.shape)))
            # assignment into a strided destination (Backend::copy_strided)
            dc, dg = Tensor.zeros(list(shape), DType.of(a), oracle), Tensor.zeros(list(shape), DType.of(a), gpu)
            dst_c, dst_g = dict(_views(dc))[name], dict(_views(dg))[name]
            dst_c.assign(wc)
            dst_g.assign(wg)
            _eq(f"assign {tag}", dc, dg)
            checked += 1
    assert checked > 1500


def test_reduce_over_every_small_shape(oracle, gpu):
    rng = np.random.default_rng(6)
    checked = 0
    for shape in _shapes():
        a = rng.integers(-9, 10, shape).astype(np.float32)
        ac, ag = _pairs(oracle, gpu, a)
        for (name, vc), (_, vg) in zip(_views(ac), _views(ag)):
            for d in range(vc.ndim):
                tag = f"{shape} {name} axis {d}"
                _eq(f"sum {tag}", vc.sum_dims([d]), vg.sum_dims([d]))
                _eq(f"max {tag}", vc.max_dims([d]), vg.max_dims([d]))
                _eq(f"argmax {tag}", vc.argmax(d), vg.argmax(d))
                _eq(f"argmin {tag}", vc.argmin(d), vg.argmin(d))
                checked += 1
    assert checked > 3000
