"""Pins the CPU oracle (oracle/dali_oracle.c) against
  * outputs of the reference's own CPU path, committed as
    tests/golden/reference_cpu.npz by tests/golden/make_golden.py, and
  * the known-answer cases of the reference's own test-suite
    (dali/array/tests/tests.cpp:1120-1361, dot_tests.cpp:10-67).
CPU only."""
import numpy as np
import pytest

import dali_oracle as oracle

# op:: name (dali/array/op/unary.cpp, binary.cpp) -> functor name (dali/array/functor.h)
FUNCTOR = {"sqrt": "sqrt_f", "eltinv": "inv", "pow": "power", "maximum": "max_scalar", "minimum": "min_scalar",
           "isnan": "isnotanumber", "isinf": "isinfinity"}


def names(golden, prefix):
    return sorted({k.split("/")[1] for k in golden.files if k.startswith(prefix + "/")})


def test_unary_bit_exact(golden):
    for n in names(golden, "unary"):
        x, y = golden["unary/%s/x" % n], golden["unary/%s/y" % n]
        got = oracle.unary(FUNCTOR.get(n, n), x)
        np.testing.assert_array_equal(got, y, err_msg=n)


def test_unary_int_and_double(golden):
    for pre in ("unary_i32", "unary_f64"):
        for n in names(golden, pre):
            x, y = golden["%s/%s/x" % (pre, n)], golden["%s/%s/y" % (pre, n)]
            got = oracle.unary(FUNCTOR.get(n, n), x)
            assert got.dtype == y.dtype
            np.testing.assert_array_equal(got, y, err_msg=pre + n)


def test_binary_bit_exact(golden):
    for n in names(golden, "binary"):
        a, b, y = (golden["binary/%s/%s" % (n, k)] for k in "aby")
        got = oracle.binary(FUNCTOR.get(n, n), a, b)
        np.testing.assert_array_equal(got, y, err_msg=n)


@pytest.mark.parametrize("ax", ["-1", "0", "all"])
def test_float_reductions(golden, ax):
    x = golden["reduce/x"]
    axis = None if ax == "all" else int(ax)
    for opn in ("sum", "prod", "max", "min"):
        want = golden["reduce/%s/%s" % (opn, ax)]
        got = oracle.reduce(opn, x, axis)
        np.testing.assert_array_equal(got.reshape(want.shape), want, err_msg=opn)
    n = x.size if axis is None else x.shape[axis]
    mean = oracle.binary("eltdiv", oracle.reduce("sum", x, axis), np.float32(n))
    np.testing.assert_array_equal(mean.reshape(-1), golden["reduce/mean/%s" % ax].reshape(-1))
    l2 = oracle.unary("sqrt_f", oracle.reduce("sum", oracle.unary("square", x), axis))
    np.testing.assert_array_equal(l2.reshape(-1), golden["reduce/l2/%s" % ax].reshape(-1))
    # double-accumulated sum is within 1e-5 * sum|x| of the reference's own fp32 fold
    s64, sabs = oracle.sum_f64acc(x, axis)
    assert np.all(np.abs(s64.reshape(-1) - golden["reduce/sum/%s" % ax].reshape(-1)) <= 1e-5 * sabs.reshape(-1))


@pytest.mark.parametrize("ax", ["-1", "0"])
def test_float_axis_argreduce(golden, ax):
    x = golden["reduce/x"]
    for opn, kind in (("argmax", "max"), ("argmin", "min")):
        want = golden["reduce/%s/%s" % (opn, ax)]
        assert want.dtype == np.int32
        np.testing.assert_array_equal(oracle.argreduce(kind, x, int(ax)), want)


def test_all_axis_argreduce_reference_returns_float(golden):
    """The reference types the all-axis argmax of a float array as float
    (dali/array/op/reducer_operation.cpp:681-684); the value still is the first
    occurrence.  The oracle (and the library) return it as int32."""
    x = golden["reduce/x"]
    for opn, kind in (("argmax", "max"), ("argmin", "min")):
        want = golden["reduce/%s/all" % opn]
        assert want.dtype == np.float32
        got = oracle.argreduce(kind, x, None)
        assert got.dtype == np.int32
        assert int(got) == int(want.reshape(-1)[0])


@pytest.mark.parametrize("ax", ["-1", "0", "1", "all"])
def test_int_reductions(golden, ax):
    x = golden["reduce_i32/x"]
    axis = None if ax == "all" else int(ax)
    for opn in ("sum", "max", "min"):
        np.testing.assert_array_equal(oracle.reduce(opn, x, axis).reshape(-1),
                                      golden["reduce_i32/%s/%s" % (opn, ax)].reshape(-1))
    if ax in ("-1", "0"):
        x2 = golden["reduce_i32_2d/x"]
        for opn, kind in (("argmax", "max"), ("argmin", "min")):
            np.testing.assert_array_equal(oracle.argreduce(kind, x2, axis),
                                          golden["reduce_i32_2d/%s/%s" % (opn, ax)])


def test_softmax(golden):
    a = golden["softmax/a"]
    np.testing.assert_array_equal(oracle.softmax(a), golden["softmax/op"])
    np.testing.assert_array_equal(oracle.softmax(a), golden["softmax/naive"])
    np.testing.assert_array_equal(oracle.softmax(golden["softmax2/a"]), golden["softmax2/naive"])


def test_gather(golden):
    src, idx = golden["gather/src"], golden["gather/idx"]
    np.testing.assert_array_equal(oracle.gather(src, idx), golden["gather/out"])
    np.testing.assert_array_equal(oracle.gather(golden["gather/src2d"], idx), golden["gather/out2d"])
    np.testing.assert_array_equal(oracle.gather_from_rows(src, golden["gather_rows/idx"]), golden["gather_rows/out"])
    got = oracle.scatter_add(np.zeros(3, np.int32), golden["scatter/idx"], np.ones(6, np.int32))
    np.testing.assert_array_equal(got, golden["scatter/out"])
    np.testing.assert_array_equal(got, [2, 3, 1])          # tests.cpp:1318-1331


def test_dot_and_fused_configs(golden):
    A, B, bias = golden["dot/A"], golden["dot/B"], golden["dot/bias"]
    # CBLAS is third-party and unpinned: agree to fp32 rounding of a K=20 dot product
    np.testing.assert_allclose(oracle.gemm(A, B), golden["dot/out"], rtol=1e-5, atol=1e-6)
    np.testing.assert_array_equal(oracle.bias_tanh(golden["dot/out"], bias), golden["dot/gemm_tanh"])
    cn, hn = oracle.lstm_cell(*(golden["lstm/" + k] for k in ("x", "h", "c", "Wx", "Wh", "b")))
    np.testing.assert_allclose(cn, golden["lstm/c_new"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(hn, golden["lstm/h_new"], rtol=1e-5, atol=1e-6)
    s32, s64, sabs = oracle.chain_sum(golden["chain/x"], 0.5, 0.1)
    assert np.float32(s32) == golden["chain/sum"].reshape(-1)[0]
    assert abs(s64 - s32) <= 1e-5 * sabs


# ---- known answers of the reference's own suite --------------------------------------
def test_known_answers_reducers():
    a = np.arange(50, dtype=np.float32).reshape(5, 10)
    assert int(oracle.reduce("sum", a)) == 50 * 49 // 2                      # tests.cpp:1120-1126
    assert int(oracle.reduce("prod", np.arange(1, 6, dtype=np.int32))) == 120  # :1128-1132
    r = np.arange(-100, 42, dtype=np.int32)
    assert int(oracle.reduce("max", r)) == 41 and int(oracle.reduce("min", r)) == -100   # :1134-1139
    assert int(oracle.argreduce("max", r)) == 141 and int(oracle.argreduce("min", r)) == 0  # :1141-1146
    a = np.arange(20, dtype=np.int32).reshape(4, 5)
    np.testing.assert_array_equal(oracle.argreduce("max", a, 0), np.full(5, 3))   # :1148-1157
    np.testing.assert_array_equal(oracle.argreduce("max", a, 1), np.full(4, 4))
    np.testing.assert_array_equal(oracle.argreduce("min", -a, 0), np.full(5, 3))
    np.testing.assert_array_equal(oracle.argreduce("min", -a, 1), np.full(4, 4))
    a4 = np.arange(120, dtype=np.int32).reshape(2, 3, 4, 5)
    assert int(oracle.argreduce("max", a4)) == 119 and int(oracle.argreduce("min", a4)) == 0   # :1159-1164
    ones = np.ones((2, 3, 4, 5), np.int32)
    np.testing.assert_array_equal(oracle.reduce("sum", ones, -1), np.full((2, 3, 4), 5))      # :1215-1221
    np.testing.assert_array_equal(oracle.reduce("sum", ones, 0), np.full((3, 4, 5), 2))       # :1223-1229
    s = np.arange(50, dtype=np.float32).reshape(5, 10)[:, ::2]                                # :1188-1202
    assert int(oracle.reduce("sum", np.ascontiguousarray(s))) == sum(k for k in range(50) if (k % 10) % 2 == 0)


def test_known_answers_gather_and_dot():
    src = np.arange(5 * 6 * 7, dtype=np.int32).reshape(5, 6, 7)
    out = oracle.gather_from_rows(src, np.arange(5, dtype=np.int32))          # tests.cpp:1296-1315
    np.testing.assert_array_equal(out[1], np.arange(49, 56))
    np.testing.assert_array_equal(out[4], np.arange(196, 203))
    a = np.arange(6, dtype=np.int32).reshape(2, 3)
    b = np.arange(12, dtype=np.int32).reshape(3, 4)
    np.testing.assert_array_equal(oracle.gemm(a, b), a @ b)                    # dot_tests.cpp:37-67
    np.testing.assert_array_equal(oracle.gemm(a.astype(np.float32), b.astype(np.float32)), (a @ b).astype(np.float32))


def test_arange_diag_one_hot_outer_pinned_by_the_reference(golden):
    """The restated index ops against what the reference's own kernels wrote, bit for bit."""
    np.testing.assert_array_equal(oracle.arange(2, 17, 3), golden["arange/i32_2_17_3"])
    np.testing.assert_array_equal(oracle.arange(0, 24, 1), golden["arange/i32_24"])
    np.testing.assert_array_equal(oracle.arange(10, -5, -4), golden["arange/i32_neg"])
    for key, d, (r, c) in (("diag/f64_5_4x5", np.float64(5.0), (4, 5)), ("diag/f32_1_6x3", np.float32(1.0), (6, 3)),
                           ("diag/i32_7_3x3", np.int32(7), (3, 3))):
        want = golden[key]
        got = oracle.diag(d, r, c)
        assert got.dtype == want.dtype
        np.testing.assert_array_equal(got, want)
    # vector diagonal: the reference throws on it; known answer from its kernel text (eye.cpp:37)
    np.testing.assert_array_equal(oracle.diag(np.arange(1, 6, dtype=np.float32), 3, 5),
                                  np.eye(3, 5, dtype=np.float32) * np.arange(1, 6, dtype=np.float32))
    want = golden["one_hot/out"]
    got = oracle.one_hot(golden["one_hot/idx"], 7, 112.2, 42.0, np.float64)
    assert got.dtype == want.dtype
    np.testing.assert_array_equal(got, want)                                   # tests.cpp:1000-1012
    np.testing.assert_array_equal(oracle.outer(golden["outer/a"], golden["outer/b"]), golden["outer/out"])


def test_running_reductions_pinned_by_the_reference(golden):
    for dt in ("i32", "f32"):
        x = golden["scan/" + dt]
        for kind in ("sum", "prod"):
            for inc in (1, 0):
                want = golden["scan/%s/%s/%d" % (dt, kind, inc)]
                got = oracle.scan(kind, x, bool(inc))
                assert got.shape == want.shape and got.dtype == want.dtype
                np.testing.assert_array_equal(got, want)
    np.testing.assert_array_equal(oracle.scan("sum", np.arange(20, dtype=np.int32), False), golden["scan/1d/sum/0"])
    # known answers of tests.cpp:1737-1771: cumsum of arange(0, 20), cumprod of arange(1, 21) (int32 wraps like the reference's)
    a = np.arange(20, dtype=np.int32)
    np.testing.assert_array_equal(oracle.scan("sum", a), np.cumsum(a, dtype=np.int32))
    np.testing.assert_array_equal(oracle.scan("sum", a.reshape(2, 10), False)[:, 1:], np.cumsum(a.reshape(2, 10), axis=1, dtype=np.int32))
    p = np.arange(1, 13, dtype=np.int32)
    np.testing.assert_array_equal(oracle.scan("prod", p), np.cumprod(p, dtype=np.int32))
    f = np.array([[3.0, -1.0, 7.0, 2.0]], np.float32)
    np.testing.assert_array_equal(oracle.scan("max", f), [[3, 3, 7, 7]])
    np.testing.assert_array_equal(oracle.scan("min", f, False), [[np.finfo(np.float32).max, 3, -1, -1, -1]])


def test_known_answer_vectors_of_the_random_generator():
    """Philox4x32-10 (Salmon et al., SC'11): the known-answer vectors published with the algorithm pin the
    restatement that the GPU stream is compared with."""
    h = lambda v: [int(w) for w in v]
    assert h(oracle.philox4x32_10((0, 0, 0, 0), (0, 0))) == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    assert h(oracle.philox4x32_10((0xffffffff,) * 4, (0xffffffff,) * 2)) == [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
    pi_digits = oracle.philox4x32_10((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0))
    assert h(pi_digits) == [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]
    u = oracle.rng_uniform(1 << 16, 99)
    assert u.dtype == np.float32 and u.min() >= 0.0 and u.max() < 1.0 and abs(u.mean() - 0.5) < 0.01
