"""arange / eye / diag / one_hot / outer (lazy index expressions) and the running
reductions, on the GPU through the Array front end and the C ABI, against the
reference's outputs (tests/golden) and the CPU oracle.  Integer and index work
bit-exact; floating running sums within 1e-5 of sum |x| (a parallel scan adds in
another order than the reference's left-to-right loop)."""
import numpy as np
import pytest
import torch

import dali_oracle as oracle
from dali_b200.array import Array, DTYPE_DOUBLE, DTYPE_FLOAT, DTYPE_INT32, last_ir, lazy_stats, op

pytestmark = pytest.mark.gpu


def test_arange_against_the_reference(golden):
    np.testing.assert_array_equal(op.arange(2, 17, 3).numpy(), golden["arange/i32_2_17_3"])
    np.testing.assert_array_equal(op.arange(24).numpy(), golden["arange/i32_24"])
    np.testing.assert_array_equal(op.arange(10, -5, -4).numpy(), golden["arange/i32_neg"])
    got = op.arange(Array(0.5, DTYPE_FLOAT), Array(3.2, DTYPE_FLOAT), Array(0.25, DTYPE_FLOAT)).numpy()
    assert got.dtype == np.float32
    np.testing.assert_array_equal(got, oracle.arange(0.5, 3.2, 0.25, np.float32))
    # tests.cpp:166-214: x (op)= arange(6).reshape({3, 2}) on an int array
    x = Array(np.full((3, 2), 10, np.int32))
    x += op.arange(6).reshape((3, 2))
    np.testing.assert_array_equal(x.numpy(), 10 + np.arange(6).reshape(3, 2))
    x *= op.arange(6).reshape((3, 2))
    np.testing.assert_array_equal(x.numpy(), (10 + np.arange(6).reshape(3, 2)) * np.arange(6).reshape(3, 2))
    # slices, transposes and broadcasts of an arange stay index arithmetic
    a = op.arange(24).reshape((2, 3, 4))
    ref = np.arange(24, dtype=np.int32).reshape(2, 3, 4)
    np.testing.assert_array_equal(a[:, 1, ::2].numpy(), ref[:, 1, ::2])
    np.testing.assert_array_equal(a.transpose().numpy(), ref.transpose())
    np.testing.assert_array_equal(a[1][::-1].numpy(), ref[1][::-1])
    big = op.arange(1 << 22)                                                  # vectorised path, many CTAs
    got = big.numpy()
    np.testing.assert_array_equal(got, np.arange(1 << 22, dtype=np.int32))
    assert int(op.sum(op.arange(1000)).numpy()) == 499500                     # fused straight into a reduction


def test_diag_and_eye(golden):
    for key, d, dt, (r, c) in (("diag/f64_5_4x5", 5.0, DTYPE_DOUBLE, (4, 5)), ("diag/f32_1_6x3", 1.0, DTYPE_FLOAT, (6, 3)),
                               ("diag/i32_7_3x3", 7, DTYPE_INT32, (3, 3))):
        got = op.diag(Array(d, dt), r, c).numpy()
        assert got.dtype == golden[key].dtype
        np.testing.assert_array_equal(got, golden[key])
    np.testing.assert_array_equal(op.eye(4, 5).numpy(), np.eye(4, 5, dtype=np.float32))
    v = np.arange(1, 6, dtype=np.float32)
    for r, c in ((3, 5), (5, 3), (5, 5), (4, 4)):
        np.testing.assert_array_equal(op.diag(Array(v), r, c).numpy(), oracle.diag(v, r, c))
    vn = np.array([np.inf, np.nan, 2.0], np.float32)                          # a select, not a multiplication by 0
    got = op.diag(Array(vn), 3, 3).numpy()
    assert got[0, 0] == np.inf and np.isnan(got[1, 1]) and got[2, 2] == 2.0 and np.all(got[~np.eye(3, dtype=bool)] == 0)
    # tests.cpp:245-277: assign into an int matrix, then subtract another diagonal
    m = Array.empty((4, 5), DTYPE_INT32)
    m.assign(op.diag(Array(5.0, DTYPE_DOUBLE), 4, 5))
    np.testing.assert_array_equal(m.numpy(), np.eye(4, 5, dtype=np.int32) * 5)
    m -= op.diag(Array(1.0, DTYPE_DOUBLE), 4, 5)
    np.testing.assert_array_equal(m.numpy(), np.eye(4, 5, dtype=np.int32) * 4)


def test_one_hot_and_outer(golden):
    got = op.one_hot(Array(golden["one_hot/idx"]), 7, 112.2, 42.0).numpy()     # tests.cpp:1000-1012
    assert got.dtype == np.float64
    np.testing.assert_array_equal(got, golden["one_hot/out"])
    rng = np.random.default_rng(3)
    idx = rng.integers(0, 50, (64, 33)).astype(np.int32)
    got = op.one_hot(Array(idx), 50, Array(1.0, DTYPE_FLOAT), Array(0.0, DTYPE_FLOAT)).numpy()
    np.testing.assert_array_equal(got, oracle.one_hot(idx, 50, 1.0, 0.0, np.float32))
    assert got.sum() == idx.size
    np.testing.assert_array_equal(op.outer(Array(golden["outer/a"]), Array(golden["outer/b"])).numpy(), golden["outer/out"])
    # tests.cpp:968-983: chainable operands, one of them a reduction
    x, y = op.arange(3), op.arange(4)
    got = op.outer(op.tanh(x.astype(DTYPE_FLOAT) - 3.0), op.tanh(y.astype(DTYPE_FLOAT) - 2.0)).numpy()
    want = np.outer(np.tanh(np.arange(3.0) - 3.0), np.tanh(np.arange(4.0) - 2.0))
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-6)
    y16 = op.arange(16).reshape((4, 4))
    got = op.outer(op.arange(3), op.sum(y16, [0])).numpy()
    np.testing.assert_array_equal(got, np.outer(np.arange(3), np.arange(16).reshape(4, 4).sum(0)))


@pytest.mark.parametrize("inclusive", [True, False])
def test_running_reductions_against_the_reference(golden, inclusive):
    for dt in ("i32", "f32"):
        x = golden["scan/" + dt]
        for kind, fn in (("sum", op.cumsum), ("prod", op.cumprod)):
            want = golden["scan/%s/%s/%d" % (dt, kind, int(inclusive))]
            got = fn(Array(x), inclusive).numpy()
            assert got.shape == want.shape and got.dtype == want.dtype
            if dt == "i32":
                np.testing.assert_array_equal(got, want)
            else:
                np.testing.assert_allclose(got, want, rtol=1e-5)
    a = op.arange(0, 20)                                                      # tests.cpp:1737-1771
    np.testing.assert_array_equal(op.cumsum(a, inclusive).numpy(), oracle.scan("sum", np.arange(20, dtype=np.int32), inclusive))
    np.testing.assert_array_equal(op.cumsum(a.reshape((2, 10)), inclusive).numpy(),
                                  oracle.scan("sum", np.arange(20, dtype=np.int32).reshape(2, 10), inclusive))
    p = op.arange(1, 21)
    np.testing.assert_array_equal(op.cumprod(p, inclusive).numpy(), oracle.scan("prod", np.arange(1, 21, dtype=np.int32), inclusive))


@pytest.mark.parametrize("shape", [(1, 1), (7, 3), (300, 9), (64, 20), (5, 128), (33, 70), (5, 300), (3, 1025), (1000, 37),
                                   (700, 20000), (3, 1 << 16), (2, 100003), (1, 1 << 22)])
def test_scan_shapes_through_the_c_abi(lib, shape):
    """Rows owned by 1 .. 32 lanes, by a CTA, or cut into pieces over many CTAs (few, very long rows); ragged
    tiles; exact integer-valued floats so that any lost or doubled element shows; running max / min bit-exact on
    random data."""
    rows, cols = shape
    rng = np.random.default_rng(rows * 7 + cols)
    x = rng.integers(-3, 4, shape).astype(np.float32)                          # partial sums stay exact in fp32
    xd = torch.from_numpy(x).cuda()
    for inclusive in (1, 0):
        out = torch.full((rows, cols + (0 if inclusive else 1)), -77.0, device="cuda")
        lib.scan(0, 0, inclusive, rows, cols, xd, out)
        np.testing.assert_array_equal(out.cpu().numpy(), oracle.scan("sum", x, bool(inclusive)))
    r = rng.standard_normal(shape)
    rd = torch.from_numpy(r).cuda()
    for opcode, kind in ((2, "max"), (3, "min")):
        out = torch.empty((rows, cols), dtype=torch.float64, device="cuda")
        lib.scan(1, opcode, 1, rows, cols, rd, out)
        np.testing.assert_array_equal(out.cpu().numpy(), oracle.scan(kind, r, True))
    xi = rng.integers(-1000, 1000, shape).astype(np.int32)
    out = torch.empty((rows, cols), dtype=torch.int32, device="cuda")
    lib.scan(2, 0, 1, rows, cols, torch.from_numpy(xi).cuda(), out)
    np.testing.assert_array_equal(out.cpu().numpy(), oracle.scan("sum", xi, True))


def test_float_cumsum_error_bound():
    rng = np.random.default_rng(11)
    x = rng.standard_normal((4, 50000)).astype(np.float32)
    got = op.cumsum(Array(x)).numpy()
    want = np.cumsum(x.astype(np.float64), axis=1)
    bound = 1e-5 * np.cumsum(np.abs(x).astype(np.float64), axis=1)
    assert np.all(np.abs(got - want) <= bound)
    ref = oracle.scan("sum", x, True)                    # the reference's own left-to-right fp32 order, same bound
    assert np.all(np.abs(ref - want) <= bound)


# ---- op::concatenate / hstack / vstack (dali/array/op/concatenate.cpp:10-73; tests.cpp ConcatenateTests) ----
def test_concatenate_along_every_axis_with_lazy_and_broadcast_pieces():
    rng = np.random.default_rng(11)
    a_np = rng.standard_normal((3, 4, 5)).astype(np.float32)
    b_np = rng.standard_normal((3, 2, 5)).astype(np.float32)
    c_np = rng.standard_normal((3, 1, 5)).astype(np.float32)
    a, b, c = Array(a_np), Array(b_np), Array(c_np)
    got = op.concatenate([a, op.tanh(b), c], 1)
    np.testing.assert_allclose(got.numpy(), np.concatenate([a_np, np.tanh(b_np), c_np], 1), rtol=1e-5, atol=1e-6)
    for axis in (0, 2, -1):
        np.testing.assert_array_equal(op.concatenate([a, a], axis).numpy(), np.concatenate([a_np, a_np], axis))
    m_np = rng.standard_normal((6, 7)).astype(np.float32)
    m = Array(m_np)
    np.testing.assert_array_equal(op.hstack([m, m[:, 0:3]]).numpy(), np.hstack([m_np, m_np[:, 0:3]]))
    np.testing.assert_array_equal(op.vstack([m, m[::-1]]).numpy(), np.vstack([m_np, m_np[::-1]]))
    # a dim of size 1 outside the axis broadcasts to the common shape
    row = Array(m_np[0:1])
    np.testing.assert_array_equal(op.hstack([m, row]).numpy(), np.hstack([m_np, np.broadcast_to(m_np[0:1], (6, 7))]))
    ints = Array(np.arange(6, dtype=np.int32))
    np.testing.assert_array_equal(op.concatenate([ints, ints + 6]).numpy(), np.arange(12, dtype=np.int32))
    with pytest.raises(RuntimeError):
        op.concatenate([a, m], 0)
    with pytest.raises(RuntimeError):
        op.concatenate([a, a], 3)
    with pytest.raises(RuntimeError):
        op.concatenate([], 0)
