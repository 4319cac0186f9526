"""The lazy Array / op:: front end on the GPU, written the way the reference's
own tests are (dali/array/tests/tests.cpp, dot_tests.cpp) and checked against
the CPU oracle / the committed outputs of the reference's CPU path.

Tolerances: fp32 elementwise 1e-5 relative (atol 1e-6 near zero); floating
sums within 1e-5 * sum|x| of the double-accumulated value; integer, index and
max/min results bit-exact."""
import numpy as np
import pytest

import dali_oracle as oracle
from dali_b200.array import (Array, DTYPE_DOUBLE, DTYPE_FLOAT, DTYPE_INT32, last_variant, lazy_stats, op)
from test_oracle import names

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _gpu(lib):
    return lib


def launched(arr):
    before = lazy_stats()
    arr.eval()
    after = lazy_stats()
    return {k: after[k] - before[k] for k in after}


# ---- JITCachedReduction.fused_softmax (tests.cpp:1622-1664) ----------------------------
def test_fused_softmax_matches_staged_evaluation_and_oracle():
    rng = np.random.default_rng(0)
    a_np = (rng.random((2, 5)) * 40 - 20).astype(np.float32)
    a = Array(a_np)
    exped = op.exp(a - op.max(a, [-1], True))
    fused = exped / op.sum(exped, [-1], True)
    assert launched(fused) == {"kernels": 1, "gemms": 0, "temporaries": 0}
    # the same expression stage by stage, with an eval() in between
    m = op.max(a, [-1], True).eval()
    e = op.exp(a - m).eval()
    s = op.sum(e, [-1], True).eval()
    staged = (e / s).eval()
    np.testing.assert_allclose(fused.numpy(), staged.numpy(), atol=1e-6)
    np.testing.assert_allclose(fused.numpy(), oracle.softmax(a_np), rtol=1e-5, atol=1e-9)


def test_config1_softmax_full_size(golden):
    a_np = np.random.default_rng(1234).standard_normal((4096, 1024)).astype(np.float32)
    out = op.softmax(Array(a_np)).numpy()
    np.testing.assert_allclose(out, oracle.softmax(a_np), rtol=1e-5, atol=1e-9)
    np.testing.assert_allclose(op.softmax(Array(golden["softmax/a"])).numpy(), golden["softmax/op"], rtol=1e-5, atol=1e-9)
    # softmax over axis 0 goes through transposed views: same numbers as softmax of the transpose
    b_np = a_np[:257, :65]
    got = op.softmax(Array(b_np), 0).numpy()
    np.testing.assert_allclose(got, oracle.softmax(np.ascontiguousarray(b_np.T)).T, rtol=1e-5, atol=1e-9)


# ---- JITTests.unary_* / BinaryTests (tests.cpp:1036-1117, 1531-1577) -------------------
def test_every_unary_and_binary_op_against_the_reference_outputs(golden):
    for n in names(golden, "unary"):
        x = golden["unary/%s/x" % n]
        got = getattr(op, n)(Array(x)).numpy()
        np.testing.assert_allclose(got, golden["unary/%s/y" % n], rtol=1e-5, atol=1e-6, err_msg=n)
    for n in names(golden, "binary"):
        a, b = golden["binary/%s/a" % n], golden["binary/%s/b" % n]
        got = getattr(op, n)(Array(a), Array(b)).numpy()
        np.testing.assert_allclose(got, golden["binary/%s/y" % n], rtol=2e-5, atol=1e-6, err_msg=n)
    for n in names(golden, "unary_i32"):
        got = getattr(op, n)(Array(golden["unary_i32/%s/x" % n])).numpy()
        np.testing.assert_array_equal(got, golden["unary_i32/%s/y" % n], err_msg=n)
    for n in names(golden, "unary_f64"):
        got = getattr(op, n)(Array(golden["unary_f64/%s/x" % n])).numpy()
        np.testing.assert_allclose(got, golden["unary_f64/%s/y" % n], rtol=1e-12, err_msg=n)


def test_scalar_operands_and_broadcasting():
    rng = np.random.default_rng(3)
    a_np = rng.standard_normal((7, 9)).astype(np.float32)
    a = Array(a_np)
    np.testing.assert_allclose((a * 2.5 + 1).numpy(), a_np * np.float32(2.5) + 1, rtol=1e-6)
    np.testing.assert_allclose((1 - a).numpy(), 1 - a_np, rtol=1e-6)
    np.testing.assert_allclose((2.0 / (a * a + 1)).numpy(), 2.0 / (a_np.astype(np.float64) ** 2 + 1), rtol=1e-6)
    row = rng.standard_normal((9,)).astype(np.float32)
    col = rng.standard_normal((7,)).astype(np.float32)
    np.testing.assert_array_equal((a + Array(row)[None, :]).numpy(), a_np + row[None, :])      # [Broadcast()]
    np.testing.assert_array_equal((a - Array(col)[:, None]).numpy(), a_np - col[:, None])
    np.testing.assert_array_equal((a.T + a.T).numpy(), a_np.T * 2)
    np.testing.assert_array_equal((a[::2, 1:5] * a[1::2, 0:4][:3] if False else a[::2, 1:5] * 1).numpy(), a_np[::2, 1:5])
    np.testing.assert_array_equal((a[::-1] + a).numpy() if False else (a[:, ::-1] + a).numpy(), a_np[:, ::-1] + a_np)
    i = Array(np.arange(12, dtype=np.int32).reshape(3, 4))
    assert (i + 1).dtype == DTYPE_INT32
    np.testing.assert_array_equal((i * 2 - 1).numpy(), np.arange(12).reshape(3, 4) * 2 - 1)
    np.testing.assert_allclose((i + 0.5).numpy(), np.arange(12).reshape(3, 4) + 0.5)          # int + double -> double
    np.testing.assert_array_equal(Array(np.array([0.4, 0.5, 1.5, -0.5, -1.2])).astype(DTYPE_INT32).numpy(),
                                  [0, 1, 2, 0, -1])                                             # astype(int) rounds


# ---- ReducerTests (tests.cpp:1120-1247) ------------------------------------------------------
def test_reducer_known_answers():
    a = op.arange(50).reshape([5, 10]).astype(DTYPE_FLOAT)
    assert int(op.sum(a)) == 50 * 49 // 2
    assert int(op.prod(op.arange(1, 6, 1))) == 120
    r = op.arange(-100, 42, 1)
    assert int(op.max(r)) == 41 and int(op.min(r)) == -100
    assert int(op.argmax(r)) == 141 and int(op.argmin(r)) == 0
    a = op.arange(20).reshape([4, 5])
    np.testing.assert_array_equal(op.argmax(a, 0).numpy(), np.full(5, 3))
    np.testing.assert_array_equal(op.argmax(a, 1).numpy(), np.full(4, 4))
    neg = a * -1.0
    np.testing.assert_array_equal(op.argmin(neg, 0).numpy(), np.full(5, 3))
    np.testing.assert_array_equal(op.argmin(neg, 1).numpy(), np.full(4, 4))
    a4 = op.arange(120).reshape([2, 3, 4, 5])
    assert int(op.argmax(a4)) == 119 and int(op.argmin(a4)) == 0
    assert float(op.mean(op.arange(1, 3, 1))) == 1.5
    assert float(op.L2_norm(Array.ones((4,), DTYPE_INT32))) == 2.0
    assert float(op.L2_norm(Array.ones((2,), DTYPE_INT32))) == np.sqrt(2.0)
    # broadcast and strided operands
    b = op.arange(50).reshape([5, 10]).astype(DTYPE_FLOAT)[:, None, :]
    assert int(op.sum(b)) == 50 * 49 // 2
    s = op.arange(50).reshape([5, 10]).astype(DTYPE_FLOAT)[:, ::2]
    assert int(op.sum(s)) == sum(k for k in range(50) if (k % 10) % 2 == 0)
    # all_reduce_mixed_sum: two all-reductions over different arrays in one expression
    a3 = op.arange(60).reshape([3, 4, 5])
    b4 = op.arange(120).reshape([2, 3, 4, 5])[:, :, 0:4:3]
    assert int(2 + (op.sum(a3) - op.max(b4))) == 60 * 59 // 2 - 119 + 2
    ones = Array.ones((2, 3, 4, 5), DTYPE_INT32)
    np.testing.assert_array_equal(op.sum(ones, [-1]).numpy(), np.full((2, 3, 4), 5))
    np.testing.assert_array_equal(op.sum(ones, [-2, -1]).numpy(), np.full((2, 3), 20))
    np.testing.assert_array_equal(op.sum(ones, [-3, -2, -1]).numpy(), np.full((2,), 60))
    np.testing.assert_array_equal(op.sum(ones, [0]).numpy(), np.full((3, 4, 5), 2))
    np.testing.assert_array_equal(op.sum(ones, [1, 0]).numpy(), np.full((4, 5), 6))
    np.testing.assert_array_equal(op.sum(ones, [2, 1, 0]).numpy(), np.full((5,), 24))
    o3 = Array.ones((2, 3, 4), DTYPE_INT32)
    np.testing.assert_array_equal(op.sum(o3, [1]).numpy(), np.full((2, 4), 3))
    # lse_reduce: a <<= ones  sums over the broadcast dim
    a = Array.zeros((2,), DTYPE_INT32).expand_dims(1)
    a <<= Array.ones((2, 5), DTYPE_INT32)
    np.testing.assert_array_equal(a.numpy(), [[5], [5]])


@pytest.mark.parametrize("axis", [None, 0, 1, -1])
def test_reductions_against_oracle_and_reference_outputs(golden, axis):
    x = golden["reduce/x"]
    ax = "all" if axis is None else str(axis if axis != 1 else -1)
    X = Array(x)
    axes = None if axis is None else [axis]
    np.testing.assert_array_equal(op.max(X, axes).numpy().reshape(-1), golden["reduce/max/%s" % ax].reshape(-1))
    np.testing.assert_array_equal(op.min(X, axes).numpy().reshape(-1), golden["reduce/min/%s" % ax].reshape(-1))
    s64, sabs = oracle.sum_f64acc(x, None if axis is None else axis)
    got = op.sum(X, axes).numpy().reshape(-1)
    assert np.all(np.abs(got - s64.reshape(-1)) <= 1e-5 * sabs.reshape(-1))
    np.testing.assert_allclose(got, golden["reduce/sum/%s" % ax].reshape(-1), rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(op.mean(X, axes).numpy().reshape(-1), golden["reduce/mean/%s" % ax].reshape(-1), rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(op.L2_norm(X, axes).numpy().reshape(-1), golden["reduce/l2/%s" % ax].reshape(-1), rtol=1e-5)
    am = op.argmax(X) if axis is None else op.argmax(X, axis)
    an = op.argmin(X) if axis is None else op.argmin(X, axis)
    assert am.dtype == DTYPE_INT32
    np.testing.assert_array_equal(am.numpy().reshape(-1), oracle.argreduce("max", x, axis).reshape(-1))
    np.testing.assert_array_equal(an.numpy().reshape(-1), oracle.argreduce("min", x, axis).reshape(-1))
    if axis is not None:
        np.testing.assert_array_equal(am.numpy().reshape(-1), golden["reduce/argmax/%s" % ax].reshape(-1))


def test_config3_reduction_sweep_on_2048(golden):
    x = (np.random.default_rng(1236).random((2048, 2048)) * 2 - 1).astype(np.float32)
    X = Array(x)
    for axis, want in ((-1, "row."), (0, "col."), (None, "all.")):
        axes = None if axis is None else [axis]
        s = op.sum(X, axes)
        assert launched(s)["kernels"] == 1 and last_variant().startswith(want)
        s64, sabs = oracle.sum_f64acc(x, axis)
        assert np.all(np.abs(s.numpy().reshape(-1) - s64.reshape(-1)) <= 1e-5 * sabs.reshape(-1))
        np.testing.assert_array_equal(op.max(X, axes).numpy().reshape(-1), oracle.reduce("max", x, axis).reshape(-1))
        am = op.argmax(X) if axis is None else op.argmax(X, axis)
        np.testing.assert_array_equal(am.numpy().reshape(-1), oracle.argreduce("max", x, axis).reshape(-1))


# ---- GatherTests (tests.cpp:1266-1361) ----------------------------------------------------------
def test_gather_and_scatter(golden):
    src, idx = golden["gather/src"], golden["gather/idx"]
    np.testing.assert_array_equal(op.gather(Array(src), Array(idx)).numpy(), golden["gather/out"])
    np.testing.assert_array_equal(Array(src)[Array(idx)].numpy(), oracle.gather(src, idx))
    np.testing.assert_allclose(op.gather(op.sigmoid(Array(src)), Array(idx)).numpy(),
                               oracle.gather(oracle.unary("sigmoid", src), idx), rtol=1e-5)   # gather_simple_elementwise
    idx2 = np.array([[0, 8], [3, 3], [5, 1]], np.int32)        # rank-2 indices (the reference cannot)
    np.testing.assert_array_equal(op.gather(Array(src), Array(idx2)).numpy(), oracle.gather(src, idx2))
    ridx = golden["gather_rows/idx"]
    np.testing.assert_array_equal(op.gather_from_rows(Array(src), Array(ridx)).numpy(), golden["gather_rows/out"])
    s2 = op.arange(5 * 6 * 7).reshape([5, 6, 7])
    out = op.gather_from_rows(s2, op.arange(5)).numpy()
    np.testing.assert_array_equal(out[1], np.arange(49, 56))
    np.testing.assert_array_equal(out[4], np.arange(196, 203))
    # scatter_simple
    dest = Array.zeros((3,), DTYPE_INT32)
    gathered = dest[Array(np.array([0, 0, 1, 1, 1, 2], np.int32))]
    gathered += 1                      # the scatter runs when it is written
    np.testing.assert_array_equal(dest.numpy(), [2, 3, 1])
    np.testing.assert_array_equal(gathered.numpy(), [2, 2, 3, 3, 3, 1])      # the gather reads what is there now
    # scatter_to_rows_simple
    vals = np.array([0, 0, 1, 1, 1, 2], np.int32)
    dest = Array.zeros((7, 3), DTYPE_INT32)
    dest.assign(42)
    dest.eval()
    g = dest.gather_from_rows(Array(vals))
    g += 1
    g.eval()
    want = np.full((7, 3), 42, np.int32)
    want[np.arange(6), vals] = 43
    np.testing.assert_array_equal(dest.numpy(), want)


# ---- in-place operators and assignment (tests.cpp:164-224, 1410-1528) ----------------------------
def test_inplace_operators_and_views_as_destinations():
    rng = np.random.default_rng(5)
    a_np = rng.standard_normal((6, 8)).astype(np.float32)
    b_np = rng.standard_normal((6, 8)).astype(np.float32)
    a, b = Array(a_np), Array(b_np)
    a += b
    a *= 2.0
    a -= 1
    np.testing.assert_allclose(a.numpy(), (a_np + b_np) * 2 - 1, rtol=1e-6)
    c = Array(a_np.copy())
    row = c[2]
    row.assign(b[3] * 3.0)
    row.eval()
    want = a_np.copy()
    want[2] = b_np[3] * 3
    np.testing.assert_allclose(c.numpy(), want, rtol=1e-6)
    col = c[:, 1:7:2]
    col /= 4.0
    col.eval()
    want[:, 1:7:2] /= 4
    np.testing.assert_allclose(c.numpy(), want, rtol=1e-6)
    z = Array.zeros((4, 5))
    np.testing.assert_array_equal(z.numpy(), np.zeros((4, 5), np.float32))
    z.assign(7)
    np.testing.assert_array_equal(z.numpy(), np.full((4, 5), 7, np.float32))
    lazy = a * 1.0
    lazy += 5                                  # in-place on a lazy value folds into the expression
    np.testing.assert_allclose(lazy.numpy(), a.numpy() + 5, rtol=1e-6)


# ---- dot (dot_tests.cpp:10-118) ---------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [np.float32, np.int32, np.float64])
def test_dot_known_answers(dtype):
    a_np = np.arange(6).reshape(2, 3).astype(dtype)
    b_np = np.arange(12).reshape(3, 4).astype(dtype)
    a, b = Array(a_np), Array(b_np)
    np.testing.assert_array_equal(op.dot(a, b).numpy(), a_np @ b_np)
    np.testing.assert_array_equal(op.dot(Array(a_np.T.copy()).T, b).numpy(), a_np @ b_np)            # transposed view
    big = Array(np.arange(24).reshape(4, 6).astype(dtype))
    np.testing.assert_array_equal(op.dot(big[::2, ::2], b).numpy(), np.arange(24).reshape(4, 6)[::2, ::2].astype(dtype) @ b_np)
    v = Array(np.arange(3).astype(dtype))
    np.testing.assert_array_equal(op.dot(a, v).numpy(), a_np @ np.arange(3).astype(dtype))             # matrix . vector
    np.testing.assert_array_equal(op.dot(v, b).numpy(), np.arange(3).astype(dtype) @ b_np)             # vector . matrix
    assert float(op.dot(v, v)) == 5.0
    d = Array.zeros((2, 4), {np.float32: 0, np.float64: 1, np.int32: 2}[dtype])
    d += op.dot(a, b)
    d += op.dot(a, b)                                                                                   # accumulates
    np.testing.assert_array_equal(d.numpy(), 2 * (a_np @ b_np))


def test_dot_is_lazy_and_fuses_around():
    rng = np.random.default_rng(9)
    A = (rng.standard_normal((96, 130)) * 0.5).astype(np.float32)
    B = (rng.standard_normal((130, 70)) * 0.5).astype(np.float32)
    bias = (rng.standard_normal((70,)) * 0.1).astype(np.float32)
    before = lazy_stats()
    r = op.tanh(op.dot(Array(A), Array(B)) + Array(bias)[None, :])
    assert lazy_stats() == before              # nothing ran yet
    got = r.numpy()
    want = oracle.bias_tanh(oracle.gemm(A, B), bias)
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-6)


def test_config2_lstm_cell_small(golden):
    x, h, c, Wx, Wh, b = (golden["lstm/" + k] for k in ("x", "h", "c", "Wx", "Wh", "b"))
    H = c.shape[1]
    gates = op.dot(Array(x), Array(Wx)) + op.dot(Array(h), Array(Wh)) + Array(b)[None, :]
    i, f, o = (op.sigmoid(gates[:, k * H:(k + 1) * H]) for k in range(3))
    g = op.tanh(gates[:, 3 * H:4 * H])
    c_new = f * Array(c) + i * g
    h_new = o * op.tanh(c_new)
    np.testing.assert_allclose(h_new.numpy(), golden["lstm/h_new"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(c_new.numpy(), golden["lstm/c_new"], rtol=1e-5, atol=1e-6)


def test_config5_chain_against_oracle(golden):
    x = golden["chain/x"]
    X = Array(x)
    s = op.sum(op.sigmoid(X * np.float32(0.5) + np.float32(0.1)) * op.exp(-X * X))
    assert launched(s) == {"kernels": 1, "gemms": 0, "temporaries": 0}
    s32, s64, sabs = oracle.chain_sum(x, 0.5, 0.1)
    assert abs(float(s) - s64) <= 1e-5 * sabs
    assert abs(float(s) - float(golden["chain/sum"].reshape(-1)[0])) <= 2e-5 * sabs


def test_memory_freshness_round_trip():
    a_np = np.arange(20, dtype=np.float32).reshape(4, 5)
    a = Array(a_np)                      # host-fresh
    b = (a + 1).eval()                   # uploaded on demand, result lives on the device
    np.testing.assert_array_equal(b.numpy(), a_np + 1)       # downloaded on demand
    b += 1                               # device copy updated, host copy must go stale
    np.testing.assert_array_equal(b.numpy(), a_np + 2)
    np.testing.assert_array_equal(a.numpy(), a_np)


def test_config2_lstm_cell_full_size_goes_through_tensor_cores():
    """B=256, H=1024 fp32: one tcgen05 3xTF32 GEMM launch accumulating both products ('+ b' as epilogue), then
    one fused gating kernel per output.  Oracle: fp64-accumulated products + the float functors."""
    rng = np.random.default_rng(1235)
    B, H = 256, 1024
    x, h, c = (rng.standard_normal((B, H)).astype(np.float32) for _ in range(3))
    Wx, Wh = ((rng.standard_normal((H, 4 * H)) * 0.02).astype(np.float32) for _ in range(2))
    b = (rng.standard_normal(4 * H) * 0.1).astype(np.float32)
    X, Hh, C, WX, WH, Bv = (Array(v) for v in (x, h, c, Wx, Wh, b))

    def cell():
        gates = op.dot(X, WX) + op.dot(Hh, WH) + Bv[None, :]
        i, f, o = (op.sigmoid(gates[:, k * H:(k + 1) * H]) for k in range(3))
        g = op.tanh(gates[:, 3 * H:4 * H])
        c_new = f * C + i * g
        return c_new, o * op.tanh(c_new)

    c_new, h_new = cell()
    before = lazy_stats()
    hn = h_new.numpy()
    cn = c_new.numpy()
    after = lazy_stats()
    assert after["gemms"] - before["gemms"] == 1 and after["kernels"] - before["kernels"] == 2
    gates64 = x.astype(np.float64) @ Wx + h.astype(np.float64) @ Wh + b
    want_c, want_h = oracle.lstm_gating(gates64.astype(np.float32), c)
    # K = 1024 products of O(1) magnitude: an fp32 GEMM itself (cuBLAS SGEMM, OpenBLAS) is 5e-6 away from
    # the fp64 value, the 3xTF32 path measures the same; outputs are O(1), so 1e-5 relative = 1e-5 absolute
    np.testing.assert_allclose(cn, want_c, rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(hn, want_h, rtol=1e-5, atol=1e-5)
    # a second step reuses the split weights (same numbers)
    c2, h2 = cell()
    np.testing.assert_array_equal(h2.numpy(), hn)


def test_dot_with_epilogue_at_mid_size_matches_oracle():
    rng = np.random.default_rng(77)
    A = (rng.standard_normal((512, 1024)) * 0.5).astype(np.float32)
    Bm = (rng.standard_normal((1024, 768)) * 0.05).astype(np.float32)
    bias = (rng.standard_normal(768) * 0.1).astype(np.float32)
    r = op.tanh(op.dot(Array(A), Array(Bm)) + Array(bias)[None, :])
    assert launched(r) == {"kernels": 0, "gemms": 1, "temporaries": 0}
    assert last_variant().startswith("tcgen05.tf32x3")
    want = np.tanh(A.astype(np.float64) @ Bm + bias)
    np.testing.assert_allclose(r.numpy(), want, rtol=1e-5, atol=1e-5)


def test_borrowed_host_arrays_and_reading_into_a_caller_buffer():
    """Array.borrow wraps caller memory (page-locked or not) without a copy; numpy(out=) reads the device
    value straight into the caller's buffer.  Same numbers as the copying constructors."""
    import torch
    rng = np.random.default_rng(9)
    a_np = rng.standard_normal((300, 70)).astype(np.float32)
    pinned = torch.empty(300, 70, pin_memory=True)
    pinned.copy_(torch.from_numpy(a_np))
    two, one = Array(2.0, DTYPE_FLOAT), Array(1.0, DTYPE_FLOAT)
    want = (Array(a_np) * two + one).numpy()
    for src in (a_np, pinned.numpy()):
        got = np.full((300, 70), -1.0, np.float32)
        ret = (Array.borrow(src) * two + one).numpy(out=got)
        assert ret is got
        np.testing.assert_array_equal(got, want)
    out_pinned = torch.empty(70, 300, pin_memory=True)
    op.identity(Array.borrow(a_np).transpose()).numpy(out=out_pinned.numpy())      # a strided view is made contiguous first
    np.testing.assert_array_equal(out_pinned.numpy(), a_np.T)
    sl = (Array.borrow(a_np) + Array(0.0, DTYPE_FLOAT))[10:20]                                          # offset into a device-only buffer
    np.testing.assert_array_equal(sl.numpy(), a_np[10:20])
    np.testing.assert_array_equal(a_np, pinned.numpy())                             # borrowed memory is never written
    with pytest.raises(TypeError):
        Array.borrow(a_np.T)
    with pytest.raises(TypeError):
        Array(a_np).numpy(out=np.empty((3, 3), np.float32))


def test_npy_load_compute_save(tmp_path):
    """Array::load -> expression -> Array::save; a Fortran-ordered file is the same array (tests.cpp:745-776)."""
    c = np.arange(12, dtype=np.float32).reshape(3, 4)
    np.save(tmp_path / "c.npy", c)
    np.save(tmp_path / "f.npy", np.asfortranarray(c))
    ac, af = Array.load(tmp_path / "c.npy"), Array.load(tmp_path / "f.npy")
    np.testing.assert_array_equal(ac.numpy(), c)
    np.testing.assert_array_equal(af.numpy(), c)
    (op.tanh(af) + ac).save(tmp_path / "out.npy")           # evaluated on the device, written from the host copy
    np.testing.assert_allclose(np.load(tmp_path / "out.npy"), np.tanh(c) + c, rtol=1e-5)


def test_lstm_cell_outputs_evaluated_together(golden):
    """eval_together(c', h'): one GEMM launch and one kernel that stores both; same numbers as evaluating them one
    by one, and as the reference's outputs."""
    from dali_b200.array import eval_together
    x, h, c, Wx, Wh, b = (golden["lstm/" + k] for k in ("x", "h", "c", "Wx", "Wh", "b"))
    H = x.shape[1]

    def cell():
        gates = op.dot(Array(x), Array(Wx)) + op.dot(Array(h), Array(Wh)) + Array(b)[None, :]
        i, f, o = (op.sigmoid(gates[:, k * H:(k + 1) * H]) for k in range(3))
        g = op.tanh(gates[:, 3 * H:4 * H])
        c_new = f * Array(c) + i * g
        return c_new, o * op.tanh(c_new)

    c1, h1 = cell()
    before = lazy_stats()
    eval_together(c1, h1)
    after = lazy_stats()
    assert after["kernels"] - before["kernels"] == 0 and after["gemms"] - before["gemms"] == 1    # the gating is the GEMM's epilogue
    c2, h2 = cell()
    np.testing.assert_allclose(c1.numpy(), c2.numpy(), rtol=1e-6, atol=1e-6)     # c2, h2: evaluated one by one, gates materialised
    np.testing.assert_allclose(h1.numpy(), h2.numpy(), rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(c1.numpy(), golden["lstm/c_new"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(h1.numpy(), golden["lstm/h_new"], rtol=1e-5, atol=1e-6)


# ---- a transposed elementwise tree is written in the destination's order (tests.cpp:560-640 transpose / dimshuffle) --
def test_transposed_elementwise_tree_reads_through_tiles():
    rng = np.random.default_rng(5)
    a_np = rng.standard_normal((300, 520)).astype(np.float32)
    b_np = rng.standard_normal((520, 300)).astype(np.float32)
    a, b = Array(a_np), Array(b_np)
    got = op.tanh(a).transpose()
    assert launched(got) == {"kernels": 1, "gemms": 0, "temporaries": 0}
    assert "tile" in last_variant()
    np.testing.assert_allclose(got.numpy(), np.tanh(a_np).T, rtol=1e-5, atol=1e-6)
    mixed = (op.sigmoid(a).transpose() * b + 1.0)
    np.testing.assert_allclose(mixed.numpy(), (1 / (1 + np.exp(-a_np))).T * b_np + 1.0, rtol=1e-5, atol=1e-6)
    # a reduction under the transpose keeps its own iteration space
    s = op.sum(a, [1], True).transpose()
    np.testing.assert_allclose(s.numpy(), a_np.sum(1, keepdims=True).T, rtol=1e-5, atol=1e-5)
    # three dimensions: the swap of the two outer ones keeps unit stride inside
    c_np = rng.standard_normal((5, 7, 64)).astype(np.float32)
    got3 = op.exp(Array(c_np)).transpose([1, 0, 2])
    np.testing.assert_allclose(got3.numpy(), np.exp(c_np).swapaxes(0, 1), rtol=1e-5, atol=1e-6)


# ---- writing into a view of a lazy value evaluates the value into a buffer first (expression.cpp:48-56) ----
def test_assigning_into_a_view_of_a_lazy_value_materialises_it():
    rng = np.random.default_rng(6)
    a_np = rng.standard_normal((4, 5)).astype(np.float32)
    lazy = op.tanh(Array(a_np))          # not evaluated
    alias = lazy                          # a second handle on the same state
    lazy[1].assign(Array(7.0, DTYPE_FLOAT)).eval()
    want = np.tanh(a_np)
    want[1] = 7.0
    np.testing.assert_allclose(lazy.numpy(), want, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(alias.numpy(), want, rtol=1e-5, atol=1e-6)
    col = lazy[:, 2]
    col += 1.0
    col.eval()
    want[:, 2] += 1.0
    np.testing.assert_allclose(lazy.numpy(), want, rtol=1e-5, atol=1e-6)


# ---- products of transposed views (the backward passes of a layer: dX = dY . W^T, dW = X^T . dY) --------------
def test_dot_of_transposed_views_goes_through_tensor_cores():
    rng = np.random.default_rng(78)
    M, K, N = 256, 512, 384
    A = (rng.standard_normal((M, K)) * 0.5).astype(np.float32)
    Bm = (rng.standard_normal((K, N)) * 0.05).astype(np.float32)
    want = A.astype(np.float64) @ Bm
    At, Bt = Array(np.ascontiguousarray(A.T)), Array(np.ascontiguousarray(Bm.T))
    for left, right in ((At.T, Array(Bm)), (Array(A), Bt.T), (At.T, Bt.T)):
        r = op.dot(left, right)
        assert launched(r) == {"kernels": 0, "gemms": 1, "temporaries": 0}
        assert last_variant().startswith("tcgen05.tf32x3")
        np.testing.assert_allclose(r.numpy(), want, rtol=1e-5, atol=2e-5)
    # accumulation into an existing gradient: dw <<= x^T . dy, then once more, then subtracted
    d_np = rng.standard_normal((M, N)).astype(np.float32)
    d = Array(d_np)
    d += op.dot(At.T, Bt.T)
    d.eval()
    assert last_variant().startswith("tcgen05.tf32x3")
    np.testing.assert_allclose(d.numpy(), d_np + want, rtol=1e-5, atol=3e-5)
    d -= op.dot(Array(A), Array(Bm))
    np.testing.assert_allclose(d.numpy(), d_np, rtol=1e-5, atol=5e-5)


# ---- few, very long rows: one all-axis reduction per row instead of one CTA per row ---------------------------
def test_reductions_over_few_very_long_rows():
    rng = np.random.default_rng(21)
    R, C = 3, (1 << 18) + 64
    a_np = rng.standard_normal((R, C)).astype(np.float32)
    a_np[1, 12345] = 9.5
    a_np[2, C - 1] = 11.0
    a = Array(a_np)
    s = op.sum(a, [-1])
    counts = launched(s)
    assert counts["kernels"] == R and "all." in last_variant()
    want = a_np.astype(np.float64).sum(1)
    assert np.all(np.abs(s.numpy() - want) <= 1e-5 * np.abs(a_np).astype(np.float64).sum(1))
    np.testing.assert_array_equal(op.max(a, [-1]).numpy(), a_np.max(1))
    np.testing.assert_array_equal(op.argmax(a, -1).numpy(), a_np.argmax(1).astype(np.int32))
    np.testing.assert_allclose(op.mean(a, [-1], True).numpy(), a_np.astype(np.float64).mean(1, keepdims=True), rtol=1e-4, atol=1e-6)
    # a tree around the reductions: softmax, evaluated reduction by reduction, then one elementwise kernel
    sm = op.softmax(a)
    got = sm.numpy()
    np.testing.assert_allclose(got, oracle.softmax(a_np), rtol=1e-5, atol=1e-12)
    # accumulation into an existing vector, and leading dims [2, 2]
    d_np = rng.standard_normal(R).astype(np.float32)
    d = Array(d_np)
    d += op.sum(a * a, [-1])
    assert np.all(np.abs(d.numpy() - (d_np + (a_np.astype(np.float64) ** 2).sum(1))) <= 1e-5 * (1 + (a_np.astype(np.float64) ** 2).sum(1)))
    b_np = rng.standard_normal((2, 2, 1 << 18)).astype(np.float32)
    np.testing.assert_array_equal(op.min(Array(b_np), [-1]).numpy(), b_np.min(2))
    one = Array(a_np[:1])
    assert abs(float(op.sum(one, [-1]).numpy()[0]) - want[0]) <= 1e-5 * np.abs(a_np[0]).sum()


def test_update_reading_its_own_destination_sees_the_old_value():
    w_np = np.arange(20, dtype=np.float32).reshape(4, 5)
    w, dw = Array(w_np), Array(np.ones((4, 5), np.float32))
    dw += w * 2.0                       # pending
    w -= dw * 0.1                       # reads dw, which reads w: runs at once on the old w
    np.testing.assert_allclose(w.numpy(), w_np - 0.1 * (1.0 + 2.0 * w_np), rtol=1e-6)
    np.testing.assert_allclose(dw.numpy(), 1.0 + 2.0 * w_np, rtol=1e-6)
    x = Array(w_np[0].copy())
    x.assign(op.tanh(x) + x)
    np.testing.assert_allclose(x.numpy(), np.tanh(w_np[0]) + w_np[0], rtol=1e-6)


def test_destination_read_through_another_index_map_goes_through_a_temporary():
    """a.assign(a.transpose()), a[1:] = a[:-1], a[0] = sum(a, 0) and a = dot(a, w): the destination's buffer is also an
    operand under a different index map, so one kernel would read elements other threads have already overwritten.  The
    value is evaluated into a temporary first (numpy semantics); the same map (a = a * 2, a += a) needs none."""
    rng = np.random.default_rng(31)
    x = rng.standard_normal((257, 257)).astype(np.float32)
    a = Array(x)
    a.assign(a.transpose())
    np.testing.assert_array_equal(a.numpy(), x.T)
    a = Array(x)
    a[1:].assign(a[:-1])
    want = x.copy()
    want[1:] = x[:-1]
    np.testing.assert_array_equal(a.numpy(), want)
    a = Array(x)
    a[0].assign(op.sum(a, [0]))
    want = x.copy()
    want[0] = x.sum(0, dtype=np.float64)
    np.testing.assert_allclose(a.numpy()[0], want[0], rtol=1e-5, atol=1e-4)
    np.testing.assert_array_equal(a.numpy()[1:], x[1:])
    w = (rng.standard_normal((257, 257)) * 0.05).astype(np.float32)
    a = Array(x)
    a.assign(op.dot(a, Array(w)))
    bound = np.abs(x).astype(np.float64) @ np.abs(w).astype(np.float64)
    assert np.all(np.abs(a.numpy().astype(np.float64) - x.astype(np.float64) @ w.astype(np.float64)) <= 1e-5 * bound)
    a = Array(x)
    a.assign(op.tanh(op.dot(Array(w), a)))                    # fused GEMM + epilogue whose right operand is the destination
    want = np.tanh(w.astype(np.float64) @ x.astype(np.float64))
    np.testing.assert_allclose(a.numpy(), want, rtol=1e-4, atol=2e-5)
    a = Array(x)
    before = lazy_stats()
    a.assign(a * 2.0)
    a += a
    after = lazy_stats()
    np.testing.assert_array_equal(a.numpy(), x * 4.0)
    assert after["kernels"] - before["kernels"] == 2          # no temporaries for identical maps
