"""Differential test of the lazy front end: seeded random expression trees (elementwise functors, scalar
operands, broadcasts, slices with steps, transposes, reductions with and without keepdims, softmax-like
normalisations, reuse of sub-expressions) evaluated by the GPU back end and by numpy on the same inputs.
fp32 elementwise results to 2e-5 relative (the special-function-unit exp / sigmoid are good to 5.5e-6 per
application and trees nest a few of them), reductions within 1e-5 of sum |x|."""
import numpy as np
import pytest

from dali_b200.array import Array, DTYPE_FLOAT, lazy_stats, op

pytestmark = pytest.mark.gpu


class Gen:
    def __init__(self, seed):
        self.rng = np.random.default_rng(seed)
        self.leaves = []

    def leaf(self, shape):
        x = (self.rng.standard_normal(shape) * 0.8).astype(np.float32)
        return Array(x), x.astype(np.float64)

    def scalar(self):
        v = float(np.float32(self.rng.uniform(-1.5, 1.5)))
        return Array(v, DTYPE_FLOAT), v

    def unary(self, a, n):
        k = self.rng.integers(0, 7)
        if k == 0: return op.tanh(a), np.tanh(n)
        if k == 1: return op.sigmoid(a), 1.0 / (1.0 + np.exp(-n))
        if k == 2: return op.exp(op.tanh(a)), np.exp(np.tanh(n))
        if k == 3: return op.square(a), n * n
        if k == 4: return op.abs(a), np.abs(n)
        if k == 5: return op.relu(a), np.maximum(n, 0.0)
        return -a, -n

    def binary(self, a, n, b, m):
        k = self.rng.integers(0, 4)
        if k == 0: return a + b, n + m
        if k == 1: return a - b, n - m
        if k == 2: return a * b, n * m
        return a / (op.abs(b) + Array(1.0, DTYPE_FLOAT)), n / (np.abs(m) + 1.0)

    def view(self, a, n):
        k = self.rng.integers(0, 4)
        if n.ndim == 2 and k == 0:
            return a.transpose(), n.T
        if n.ndim >= 1 and k == 1 and n.shape[0] >= 4:
            s = slice(int(self.rng.integers(0, 2)), n.shape[0], int(self.rng.integers(1, 3)))
            return a[s], n[s]
        if n.ndim == 2 and k == 2 and n.shape[1] >= 4:
            lo = int(self.rng.integers(0, n.shape[1] // 2))
            return a[:, lo:lo + n.shape[1] // 2], n[:, lo:lo + n.shape[1] // 2]
        return a, n

    def reduce(self, a, n):
        if n.ndim == 0:
            return a, n
        k = self.rng.integers(0, 3)
        axis = int(self.rng.integers(0, n.ndim))
        keep = bool(self.rng.integers(0, 2))
        if k == 0: return op.sum(a, [axis], keep), n.sum(axis=axis, keepdims=keep)
        if k == 1: return op.max(a, [axis], keep), n.max(axis=axis, keepdims=keep)
        return op.mean(a, [axis], keep), n.mean(axis=axis, keepdims=keep)

    def tree(self, shape, depth):
        if depth == 0 or self.rng.random() < 0.15:
            return self.leaf(shape)
        k = self.rng.integers(0, 10)
        if k < 3:
            return self.unary(*self.tree(shape, depth - 1))
        if k < 6:
            a, n = self.tree(shape, depth - 1)
            pick = self.rng.integers(0, 4)
            if pick == 0:
                b, m = self.scalar()
            elif pick == 1 and len(shape) == 2:
                b, m = self.leaf((1, shape[1]))                     # a row broadcast over the rows
                b, m = b.broadcast_to_shape(shape), np.broadcast_to(m, shape)
            elif pick == 2:
                b, m = a, n                                          # a shared sub-expression
            else:
                b, m = self.tree(shape, depth - 1)
            return self.binary(a, n, b, m)
        if k < 8 and len(shape) == 2:
            # normalisation: x - reduce(x, keepdims) broadcast back, the softmax pattern
            a, n = self.tree(shape, depth - 1)
            axis = int(self.rng.integers(0, 2))
            r, rn = op.max(a, [axis], True), n.max(axis=axis, keepdims=True)
            e, en = op.exp(a - r), np.exp(n - rn)
            return e / op.sum(e, [axis], True), en / en.sum(axis=axis, keepdims=True)
        a, n = self.tree(shape, depth - 1)
        return a, n


def check(got, want, what):
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    scale = max(1.0, float(np.abs(want).max()) if want.size else 1.0)
    err = float(np.abs(got.astype(np.float64) - want).max()) if want.size else 0.0
    assert err <= 4e-5 * scale, (what, err, scale)


@pytest.mark.parametrize("seed", range(40))
def test_random_trees_against_numpy(seed):
    g = Gen(seed)
    shape = [(7, 33), (64, 128), (5, 1024), (130, 9), (257,), (31, 32)][seed % 6]
    a, n = g.tree(shape, depth=4)
    check(a.numpy(), n, "tree")
    # a view of the lazy result, then a reduction of it: two more kernels over the same graph
    v, vn = g.view(a, n)
    check(v.numpy(), vn, "view")
    r, rn = g.reduce(v, vn)
    check(r.numpy(), rn, "reduce")


@pytest.mark.parametrize("seed", range(12))
def test_random_trees_before_evaluation(seed):
    """The same, but views and reductions are stacked on the tree while it is still lazy, so that they must fuse
    (or be split into temporaries) correctly instead of reading an evaluated buffer."""
    g = Gen(1000 + seed)
    shape = [(16, 48), (9, 256), (128, 20)][seed % 3]
    a, n = g.tree(shape, depth=3)
    v, vn = g.view(a, n)
    r, rn = g.reduce(v, vn)
    w, wn = g.unary(r, rn)
    check(w.numpy(), wn, "stacked")
    check(a.numpy(), n, "root after its consumers")
