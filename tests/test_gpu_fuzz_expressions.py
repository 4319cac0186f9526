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


@pytest.mark.parametrize("seed", range(16))
def test_random_index_work_is_bit_exact(seed):
    """argmax / argmin (first occurrence on ties), gather, gather_from_rows, scatter-add through a gathered view,
    integer running sums and one_hot on random int32 data: every answer equal to numpy's, bit for bit."""
    from dali_b200.array import DTYPE_INT32
    rng = np.random.default_rng(5000 + seed)
    rows, cols = int(rng.integers(1, 70)), int(rng.integers(1, 300))
    x = rng.integers(-5, 6, (rows, cols)).astype(np.int32)             # many ties
    a = Array(x)
    np.testing.assert_array_equal(op.argmax(a, 1).numpy(), x.argmax(1))
    np.testing.assert_array_equal(op.argmin(a, 0).numpy(), x.argmin(0))
    assert int(op.argmax(a).numpy()) == int(x.argmax())
    np.testing.assert_array_equal(op.max(a, [0]).numpy(), x.max(0))
    np.testing.assert_array_equal(op.sum(a, [1]).numpy(), x.sum(1, dtype=np.int32))
    np.testing.assert_array_equal(op.cumsum(a).numpy(), np.cumsum(x, axis=1, dtype=np.int32))
    idx = rng.integers(0, rows, (int(rng.integers(1, 50)),)).astype(np.int32)
    np.testing.assert_array_equal(op.gather(a, Array(idx)).numpy(), x[idx])
    np.testing.assert_array_equal(op.gather(a + 1, Array(idx)).numpy(), (x + 1)[idx])       # lazy source
    ridx = rng.integers(0, cols, (rows,)).astype(np.int32)
    np.testing.assert_array_equal(op.gather_from_rows(a, Array(ridx)).numpy(), x[np.arange(rows), ridx])
    dest_np = rng.integers(-3, 4, (rows, cols)).astype(np.int32)
    dest = Array(dest_np.copy())
    g = dest[Array(idx)]
    g += Array(x[idx])
    g.eval()
    want = dest_np.copy()
    np.add.at(want, idx, x[idx])
    np.testing.assert_array_equal(dest.numpy(), want)
    depth = int(rng.integers(1, 12))
    k = rng.integers(0, depth, (rows,)).astype(np.int32)
    oh = op.one_hot(Array(k), depth, Array(3, DTYPE_INT32), Array(-1, DTYPE_INT32)).numpy()
    np.testing.assert_array_equal(oh, np.where(np.arange(depth)[None, :] == k[:, None], 3, -1))


@pytest.mark.parametrize("seed", range(16))
def test_random_products_with_epilogues(seed):
    """dot inside elementwise trees at random (often ragged) shapes: tensor-core path with the tree as epilogue where
    the layout allows it, the general kernel otherwise; sums of two products; products of transposed views.
    Against fp64 numpy within 1e-5 of |A|.|B| (plus the functors' 2e-5)."""
    rng = np.random.default_rng(7000 + seed)
    m, k, n = (int(rng.integers(1, 40)) * int(rng.choice([1, 4, 8])) for _ in range(3))
    A = (rng.standard_normal((m, k)) * 0.5).astype(np.float32)
    B = (rng.standard_normal((k, n)) * 0.5).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    res = rng.standard_normal((m, n)).astype(np.float32)
    a, b = Array(A), Array(B)
    A64, B64 = A.astype(np.float64), B.astype(np.float64)
    bound = np.abs(A64) @ np.abs(B64)
    tol = 1e-5 * bound + 2e-5

    def close(got, want):
        assert got.shape == want.shape
        assert np.all(np.abs(got - want) <= tol + 2e-5 * np.abs(want)), float(np.max(np.abs(got - want)))

    close(op.dot(a, b).numpy(), A64 @ B64)
    close((op.dot(a, b) + Array(bias)[None, :]).numpy(), A64 @ B64 + bias)
    close((Array(res) - op.dot(a, b) * Array(0.5, DTYPE_FLOAT)).numpy(), res - 0.5 * (A64 @ B64))
    d = Array(res.copy())
    d += op.dot(a, b)
    close(d.numpy(), res + A64 @ B64)
    close(op.dot(Array(np.ascontiguousarray(A.T)).transpose(), b).numpy(), A64 @ B64)        # transposed view as operand
    k2 = int(rng.integers(1, 30)) * 4
    A2 = (rng.standard_normal((m, k2)) * 0.5).astype(np.float32)
    B2 = (rng.standard_normal((k2, n)) * 0.5).astype(np.float32)
    two = op.tanh(op.dot(a, b) + op.dot(Array(A2), Array(B2)) + Array(bias)[None, :]).numpy()
    want = np.tanh(A64 @ B64 + A2.astype(np.float64) @ B2.astype(np.float64) + bias)
    bound2 = bound + np.abs(A2).astype(np.float64) @ np.abs(B2).astype(np.float64)
    assert np.all(np.abs(two - want) <= 1e-5 * bound2 + 4e-5)
