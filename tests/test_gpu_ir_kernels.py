"""Parity of the generated sm_100a kernels with the CPU oracle, driven through
the C ABI (dalib200_compile / dalib200_launch) with hand-built IR.

Tolerances (fp32): elementwise outputs 1e-5 relative (atol 1e-6 where values
approach zero); floating sums |gpu - double-accumulated| <= 1e-5 * sum|x|;
max / min / argmax / argmin / integer work bit-exact."""
import numpy as np
import pytest
import torch

import dali_oracle as oracle
from dali_b200.ir import IRBuilder, chain_sum_ir, lstm_gating_ir, reduce_ir, softmax_ir

pytestmark = pytest.mark.gpu


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def host(t):
    torch.cuda.synchronize()
    return t.cpu().numpy()


@pytest.mark.parametrize("shape", [(2, 5), (7, 33), (5, 64), (64, 1000), (33, 1001), (4096, 1024), (3, 40000),
                                   (1, 4096), (300, 7)])
def test_softmax(lib, shape):
    rng = np.random.default_rng(1234)
    a = rng.standard_normal(shape).astype(np.float32)
    if shape == (7, 33):
        a = (rng.random(shape) * 40 - 20).astype(np.float32)     # range of the reference's own test
    h = lib.compile(softmax_ir())
    d_a, d_out = dev(a), torch.empty(shape, dtype=torch.float32, device="cuda")
    lib.launch(h, shape, [d_out, d_a])
    got = host(d_out)
    want = oracle.softmax(a)
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-9)
    np.testing.assert_allclose(got.sum(-1), 1.0, rtol=1e-5)


def test_softmax_in_place_and_row_stride(lib):
    rng = np.random.default_rng(7)
    big = rng.standard_normal((50, 96)).astype(np.float32)
    h = lib.compile(softmax_ir())
    d = dev(big)
    # view big[:, 32:64]: row stride 96, offset 32; written in place
    lib.launch(h, (50, 32), [d, d], strides=[[96, 1], [96, 1]], offsets=[32, 32])
    got = host(d)
    want = big.copy()
    want[:, 32:64] = oracle.softmax(np.ascontiguousarray(big[:, 32:64]))
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-9)


REDUCE_SHAPES = [(13, 37), (4, 5), (300, 257), (64, 4096), (2048, 2048), (5, 100000), (3000, 3)]


@pytest.mark.parametrize("shape", REDUCE_SHAPES)
@pytest.mark.parametrize("layout", ["row", "col", "all"])
def test_float_reductions(lib, shape, layout):
    rng = np.random.default_rng(99)
    x = (rng.random(shape) * 2 - 1).astype(np.float32)
    x[shape[0] // 2, shape[1] // 3] = x[shape[0] // 2, (2 * shape[1]) // 3] = 0.99999994   # ties
    x[0, 0] = x[shape[0] - 1, shape[1] - 1] = -0.99999994
    d_x = dev(x)
    rows, cols = shape
    for kind in ("sum", "max", "min", "prod"):
        for arg in (False, True):
            if arg and kind in ("sum", "prod"):
                continue
            xin, d_in = x, d_x
            if kind == "prod":
                # factors whose product is exact in fp32 in any order (powers of two and three 3s),
                # so a dropped or doubled element cannot hide behind rounding
                xin = np.ones(shape, np.float32).ravel()
                pos = rng.permutation(xin.size)[:min(123, xin.size)]
                xin[pos[:60]] = 2.0
                xin[pos[60:120]] = 0.5
                xin[pos[120:]] = 3.0
                xin = xin.reshape(shape)
                d_in = dev(xin)
            if kind == "sum" and arg is False:
                # integer-valued floats: every partial sum is exact, so the result is order-independent
                xi = rng.integers(-3, 4, shape).astype(np.float32)
                hs = lib.compile(reduce_ir("sum", "f32", 2, 2 if layout == "all" else 1, False))
                n_o = {"row": rows, "col": cols, "all": 1}[layout]
                o2 = torch.full((n_o,), -7.0, device="cuda")
                if layout == "col":
                    lib.launch(hs, (cols, rows), [o2, dev(xi)], strides=[None, [1, cols]])
                else:
                    lib.launch(hs, (rows, cols), [o2, dev(xi)])
                ax = {"row": 1, "col": 0, "all": None}[layout]
                np.testing.assert_array_equal(host(o2), xi.astype(np.float64).sum(axis=ax).reshape(-1))
            if layout == "row":
                space, strides, axis, n_out = (rows, cols), None, 1, rows
            elif layout == "col":      # axis 0 == last-axis reduce of the transposed view
                space, strides, axis, n_out = (cols, rows), [None, [1, cols]], 0, cols
            else:
                space, strides, axis, n_out = (rows, cols), None, None, 1
            h = lib.compile(reduce_ir(kind, "f32", 2, 2 if layout == "all" else 1, arg))
            out = torch.full((n_out,), -7, dtype=torch.int32 if arg else torch.float32, device="cuda")
            lib.launch(h, space, [out, d_in], strides=strides)
            got = host(out)
            tag = "%s %s arg=%s %s [%s]" % (layout, kind, arg, shape, lib.last_variant())
            if arg:
                np.testing.assert_array_equal(got, oracle.argreduce(kind, xin, axis).reshape(-1), err_msg=tag)
            elif kind in ("max", "min"):
                np.testing.assert_array_equal(got, oracle.reduce(kind, xin, axis).reshape(-1), err_msg=tag)
            elif kind == "sum":
                s64, sabs = oracle.sum_f64acc(xin, axis)
                assert np.all(np.abs(got - s64.reshape(-1)) <= 1e-5 * sabs.reshape(-1)), tag
            else:
                ref = np.prod(xin.astype(np.float64), axis=axis).reshape(-1)
                np.testing.assert_array_equal(got, ref, err_msg=tag)


@pytest.mark.parametrize("layout", ["row", "col", "all"])
def test_int_reductions_bit_exact(lib, layout):
    rng = np.random.default_rng(5)
    x = rng.integers(-1000, 1000, (257, 129)).astype(np.int32)
    d_x = dev(x)
    rows, cols = x.shape
    for kind in ("sum", "max", "min"):
        for arg in (False, True):
            if arg and kind == "sum":
                continue
            if layout == "row":
                space, strides, axis, n_out = (rows, cols), None, 1, rows
            elif layout == "col":
                space, strides, axis, n_out = (cols, rows), [None, [1, cols]], 0, cols
            else:
                space, strides, axis, n_out = (rows, cols), None, None, 1
            h = lib.compile(reduce_ir(kind, "i32", 2, 2 if layout == "all" else 1, arg))
            out = torch.zeros((n_out,), dtype=torch.int32, device="cuda")
            lib.launch(h, space, [out, d_x], strides=strides)
            want = (oracle.argreduce if arg else oracle.reduce)(kind, x, axis).reshape(-1)
            np.testing.assert_array_equal(host(out), want, err_msg="%s %s %s" % (layout, kind, arg))


def test_strided_and_broadcast_all_reduce(lib):
    """ReducerTests.all_reduce_sum_with_strides / _with_broadcast (tests.cpp:1180-1213)."""
    a = np.arange(50, dtype=np.float32).reshape(5, 10)
    d_a = dev(a)
    h = lib.compile(reduce_ir("sum", "f32", 2, 2))
    out = torch.zeros(1, device="cuda")
    lib.launch(h, (5, 5), [out, d_a], strides=[None, [10, 2]])
    assert int(host(out)[0]) == sum(k for k in range(50) if (k % 10) % 2 == 0)
    h3 = lib.compile(reduce_ir("sum", "f32", 3, 3))
    lib.launch(h3, (5, 1, 10), [out, d_a], strides=[None, [10, 0, 1]])
    assert int(host(out)[0]) == 50 * 49 // 2
    # middle-axis reduce of a rank-3 array: reduce dim 1 of [6, 5, 4] -> space [6, 4, 5]
    x = np.random.default_rng(3).integers(-9, 9, (6, 5, 4)).astype(np.int32)
    hm = lib.compile(reduce_ir("sum", "i32", 3, 1))
    o = torch.zeros((6, 4), dtype=torch.int32, device="cuda")
    lib.launch(hm, (6, 4, 5), [o, dev(x)], strides=[None, [20, 1, 4]])
    np.testing.assert_array_equal(host(o), x.sum(1))


@pytest.mark.parametrize("n", [1, 4099, 1 << 20, (1 << 22) + 3])
def test_chain_sum(lib, n):
    x = np.random.default_rng(11).standard_normal(n).astype(np.float32)
    h = lib.compile(chain_sum_ir())
    out = torch.zeros(1, device="cuda")
    lib.launch(h, (n,), [out, dev(x)], scalars=[np.float32(0.5), np.float32(0.1)])
    s32, s64, sabs = oracle.chain_sum(x, 0.5, 0.1)
    got = float(host(out)[0])
    assert abs(got - s64) <= 1e-5 * sabs, (got, s64, s32, lib.last_variant())
    # twice in a row through the same scratch: the ticket counter must have reset itself
    lib.launch(h, (n,), [out, dev(x)], scalars=[np.float32(0.5), np.float32(0.1)])
    assert abs(float(host(out)[0]) - s64) <= 1e-5 * sabs


def test_lstm_gating_on_column_slices(lib):
    rng = np.random.default_rng(21)
    B, H = 37, 96
    gates = rng.standard_normal((B, 4 * H)).astype(np.float32)
    c = rng.standard_normal((B, H)).astype(np.float32)
    h = lib.compile(lstm_gating_ir())
    d_g, d_c = dev(gates), dev(c)
    cn = torch.empty((B, H), device="cuda")
    hn = torch.empty((B, H), device="cuda")
    gs = [4 * H, 1]
    lib.launch(h, (B, H), [cn, hn, d_g, d_g, d_g, d_g, d_c], strides=[None, None, gs, gs, gs, gs, None],
               offsets=[0, 0, 0, H, 2 * H, 3 * H, 0])
    assert lib.last_variant().startswith("map") and ".v4." in lib.last_variant()
    want_c, want_h = oracle.lstm_gating(gates, c)
    np.testing.assert_allclose(host(cn), want_c, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(host(hn), want_h, rtol=1e-5, atol=1e-6)


def binary_map_ir(name, dtype="f32", op="assign"):
    b = IRBuilder(2, 0)
    out, l, r = b.arg(dtype), b.arg(dtype), b.arg(dtype)
    b.st(out, b.op(name, b.ld(l), b.ld(r)), op)
    return b.text()


def test_map_broadcast_transpose_inplace(lib):
    rng = np.random.default_rng(8)
    R, C = 70, 52
    a = rng.standard_normal((R, C)).astype(np.float32)
    row = rng.standard_normal((C,)).astype(np.float32)
    col = rng.standard_normal((R,)).astype(np.float32)
    at = np.ascontiguousarray(a.T)
    h = lib.compile(binary_map_ir("add"))
    out = torch.empty((R, C), device="cuda")
    lib.launch(h, (R, C), [out, dev(a), dev(row)], strides=[None, None, [0, 1]])       # [R,C] + [1,C]
    np.testing.assert_array_equal(host(out), a + row[None, :])
    lib.launch(h, (R, C), [out, dev(a), dev(col)], strides=[None, None, [1, 0]])       # [R,C] + [R,1]
    np.testing.assert_array_equal(host(out), a + col[:, None])
    lib.launch(h, (R, C), [out, dev(at), dev(a)], strides=[None, [1, R], None])        # a.T.T + a
    np.testing.assert_array_equal(host(out), a + a)
    hsub = lib.compile(binary_map_ir("eltmul", op="sub"))                                # out -= l * r
    base = rng.standard_normal((R, C)).astype(np.float32)
    d_out = dev(base)
    lib.launch(hsub, (R, C), [d_out, dev(a), dev(a)])
    np.testing.assert_allclose(host(d_out), base - a * a, rtol=1e-6, atol=1e-6)
    # negative step view: out = a[::-1] + a  (offset R-1 rows, row stride -C)
    lib.launch(h, (R, C), [out, dev(a), dev(a)], strides=[None, [-C, 1], None], offsets=[0, (R - 1) * C, 0])
    np.testing.assert_array_equal(host(out), a[::-1] + a)


def test_unary_and_binary_functors_against_oracle(lib, golden):
    """Every functor, on the inputs of the committed reference fixtures."""
    from test_oracle import FUNCTOR, names
    for n in names(golden, "unary"):
        x = golden["unary/%s/x" % n]
        b = IRBuilder(2, 0)
        o, i = b.arg("f32"), b.arg("f32")
        b.st(o, b.op(FUNCTOR.get(n, n), b.ld(i)))
        out = torch.empty(x.shape, device="cuda")
        lib.launch(lib.compile(b.text()), x.shape, [out, dev(x)])
        np.testing.assert_allclose(host(out), golden["unary/%s/y" % n], rtol=1e-5, atol=1e-6, err_msg=n)
    for n in names(golden, "binary"):
        a, bb = golden["binary/%s/a" % n], golden["binary/%s/b" % n]
        out = torch.empty(a.shape, device="cuda")
        lib.launch(lib.compile(binary_map_ir(FUNCTOR.get(n, n))), a.shape, [out, dev(a), dev(bb)])
        np.testing.assert_allclose(host(out), golden["binary/%s/y" % n], rtol=2e-5, atol=1e-6, err_msg=n)
    for pre, dt, tdt in (("unary_i32", "i32", torch.int32), ("unary_f64", "f64", torch.float64)):
        for n in names(golden, pre):
            x = golden["%s/%s/x" % (pre, n)]
            b = IRBuilder(2, 0)
            o, i = b.arg(dt), b.arg(dt)
            b.st(o, b.op(FUNCTOR.get(n, n), b.ld(i)))
            out = torch.empty(x.shape, dtype=tdt, device="cuda")
            lib.launch(lib.compile(b.text()), x.shape, [out, dev(x)])
            want = golden["%s/%s/y" % (pre, n)]
            if dt == "i32":
                np.testing.assert_array_equal(host(out), want, err_msg=pre + n)
            else:
                np.testing.assert_allclose(host(out), want, rtol=1e-12, atol=1e-14, err_msg=pre + n)


def test_gather_and_scatter(lib, golden):
    src, idx = golden["gather/src"], golden["gather/idx"]          # [9, 6, 3], [5]
    # out[i, j, k] = src[idx[i], j, k]: space [5, 18]; index arg broadcast along the inner dim
    b = IRBuilder(2, 0)
    o, s, ix = b.arg("f32"), b.arg("f32"), b.arg("i32")
    b.st(o, b.ldx(s, b.ld(ix)))
    h = lib.compile(b.text())
    out = torch.empty((5, 18), device="cuda")
    lib.launch(h, (5, 18), [out, dev(src), dev(idx)], strides=[None, [0, 1, 18], [1, 0]])
    np.testing.assert_array_equal(host(out).reshape(5, 6, 3), golden["gather/out"])
    # gather_from_rows: out[i, k] = src[i, idx[i], k]: space [9, 3]
    ridx = golden["gather_rows/idx"]
    out = torch.empty((9, 3), device="cuda")
    lib.launch(h, (9, 3), [out, dev(src), dev(ridx)], strides=[None, [18, 1, 3], [1, 0]])
    np.testing.assert_array_equal(host(out), golden["gather_rows/out"])
    # scatter-add: dest[idx[i]] += 1  (tests.cpp:1318-1331)
    b = IRBuilder(1, 0)
    d, ix = b.arg("i32"), b.arg("i32")
    b.stx(d, b.ld(ix), b.const("i32", "1"), "add")
    dest = torch.zeros(3, dtype=torch.int32, device="cuda")
    sidx = golden["scatter/idx"]
    lib.launch(lib.compile(b.text()), (6,), [dest, dev(sidx)], strides=[[0, 1], None])
    np.testing.assert_array_equal(host(dest), [2, 3, 1])
    # float scatter-add of rows with repeated indices against the serial oracle
    rng = np.random.default_rng(4)
    idx = rng.integers(0, 11, (500,)).astype(np.int32)
    upd = rng.integers(-3, 4, (500, 8)).astype(np.float32)          # small integers: order-independent sums
    b = IRBuilder(2, 0)
    d, ix, u = b.arg("f32"), b.arg("i32"), b.arg("f32")
    b.stx(d, b.ld(ix), b.ld(u), "add")
    dest = torch.zeros((11, 8), device="cuda")
    lib.launch(lib.compile(b.text()), (500, 8), [dest, dev(idx), dev(upd)], strides=[[0, 1, 8], [1, 0], None])
    np.testing.assert_array_equal(host(dest), oracle.scatter_add(np.zeros((11, 8), np.float32), idx, upd))


def test_mean_and_l2_fused_post_ops(lib):
    """mean = sum / n and L2 = sqrt(sum(x*x)) as one kernel each (row-level functors after the fold)."""
    x = np.random.default_rng(2).standard_normal((100, 300)).astype(np.float32)
    d_x = dev(x)
    for layout in ("row", "col", "all"):
        b = IRBuilder(2, 2 if layout == "all" else 1)
        o, a = b.arg("f32", "R"), b.arg("f32")
        n = x.size if layout == "all" else (x.shape[1] if layout == "row" else x.shape[0])
        s = b.red("sum", b.op("square", b.ld(a)))
        b.st(o, b.op("sqrt_f", b.op("eltdiv", s, b.const("f32", str(n)))))
        if layout == "row":
            space, strides, axis, n_out = x.shape, None, 1, x.shape[0]
        elif layout == "col":
            space, strides, axis, n_out = x.shape[::-1], [None, [1, x.shape[1]]], 0, x.shape[1]
        else:
            space, strides, axis, n_out = x.shape, None, None, 1
        out = torch.zeros(n_out, device="cuda")
        lib.launch(lib.compile(b.text()), space, [out, d_x], strides=strides)
        want = np.sqrt((x.astype(np.float64) ** 2).sum(axis=axis) / n).reshape(-1)
        np.testing.assert_allclose(host(out), want, rtol=1e-5, err_msg=layout)


def test_launch_host_round_trip(lib):
    a = np.random.default_rng(6).standard_normal((33, 65)).astype(np.float32)
    out = np.zeros_like(a)
    lib.launch_host(lib.compile(softmax_ir()), a.shape, [out, a])
    np.testing.assert_allclose(out, oracle.softmax(a), rtol=1e-5, atol=1e-9)


def test_errors_are_statuses_not_crashes(lib):
    from dali_b200 import DaliB200Error
    with pytest.raises(DaliB200Error):
        lib.compile("dali-ir 1\nspace 2 0\narg 0 f32 E\nv0 f32 op nosuchfunctor v0\nend\n")
    h = lib.compile(softmax_ir())
    with pytest.raises(DaliB200Error):
        lib.launch(h, (4, 4, 4), [0, 0])           # wrong rank
    with pytest.raises(DaliB200Error):
        lib.launch(0xdeadbeef, (4, 4), [0, 0])     # unknown hash


@pytest.mark.parametrize("shape", [(32, 32), (33, 65), (100, 257), (1024, 512), (36, 132), (64, 200), (5, 4000), (4000, 7)])
def test_map_with_transposed_operands_uses_shared_memory_tiles(lib, shape):
    """out = tanh(a^T) + b + bias[col] with a stored column-major: the transposed operand goes through 4 x 4 register
    blocks (extents multiples of 4: 128-bit accesses on both sides) or 32 x 32 shared-memory tiles (ragged extents);
    same numbers as numpy.  Below 32 rows or columns the plain strided kernel takes over."""
    R, C = shape
    rng = np.random.default_rng(R * 31 + C)
    at = rng.standard_normal((C, R)).astype(np.float32)        # a^T in memory: a[r, c] = at[c, r]
    b = rng.standard_normal((R, C)).astype(np.float32)
    bias = rng.standard_normal(C).astype(np.float32)
    e = IRBuilder(2, 0)
    O, A, B, Bi = e.arg("f32"), e.arg("f32"), e.arg("f32"), e.arg("f32")
    e.st(O, e.op("add", e.op("add", e.op("tanh", e.ld(A)), e.ld(B)), e.ld(Bi)))
    h = lib.compile(e.text())
    out = torch.full((R, C), -7.0, device="cuda")
    lib.launch(h, (R, C), [out, dev(at), dev(b), dev(bias)], strides=[None, [1, R], None, [0, 1]])
    torch.cuda.synchronize()
    assert (".tile" in lib.last_variant()) == (R >= 32 and C >= 32)
    assert (".tile4" in lib.last_variant()) == (R >= 32 and C >= 32 and R % 4 == 0 and C % 4 == 0)
    np.testing.assert_allclose(out.cpu().numpy(), np.tanh(at.T) + b + bias, rtol=1e-5, atol=1e-6)
    # two transposed operands and an in-place destination
    e2 = IRBuilder(2, 0)
    D, A2, B2 = e2.arg("f32"), e2.arg("f32"), e2.arg("f32")
    e2.st(D, e2.op("eltmul", e2.ld(A2), e2.ld(B2)), "add")
    h2 = lib.compile(e2.text())
    bt = rng.standard_normal((C, R)).astype(np.float32)
    d = dev(b.copy())
    lib.launch(h2, (R, C), [d, dev(at), dev(bt)], strides=[None, [1, R], [1, R]])
    torch.cuda.synchronize()
    np.testing.assert_allclose(d.cpu().numpy(), b + at.T * bt.T, rtol=1e-6, atol=1e-6)


def test_rows_staged_through_shared_memory_by_bulk_copies(lib, monkeypatch):
    """The row skeleton's opt-in `stage` variant (DALI_B200_ROW_STAGE = ring depth): one warp per row, rows copied into
    a per-warp ring in shared memory by cp.async.bulk ahead of the rows being worked on.  Same results as the plain
    variant: a softmax (rows of 1000 and 512 elements, a ragged number of rows) and a two-operand normalisation."""
    import dali_oracle as oracle
    from dali_b200.ir import softmax_ir
    monkeypatch.setenv("DALI_B200_ROW_STAGE", "3")
    rng = np.random.default_rng(17)
    for rows, cols in ((4099, 1000), (3000, 512)):
        a = rng.standard_normal((rows, cols)).astype(np.float32)
        out = torch.empty((rows, cols), device="cuda")
        lib.launch(lib.compile(softmax_ir()), (rows, cols), [out, dev(a)])
        assert ".stage3" in lib.last_variant(), lib.last_variant()
        np.testing.assert_allclose(host(out), oracle.softmax(a), rtol=1e-5, atol=1e-9)
    b = IRBuilder(2, 1)
    o, x, y = b.arg("f32"), b.arg("f32"), b.arg("f32")
    s = b.op("add", b.ld(x), b.ld(y))
    b.st(o, b.op("eltdiv", s, b.red("sum", s)))
    xs, ys = (rng.random((2600, 640)).astype(np.float32) + 0.5 for _ in range(2))
    out = torch.empty((2600, 640), device="cuda")
    lib.launch(lib.compile(b.text()), (2600, 640), [out, dev(xs), dev(ys)])
    assert ".stage" in lib.last_variant(), lib.last_variant()
    want = (xs + ys) / (xs + ys).astype(np.float64).sum(1, keepdims=True)
    np.testing.assert_allclose(host(out), want, rtol=1e-5)
    # a view whose rows do not start on 16-byte boundaries falls back to the plain variant
    a = rng.standard_normal((2400, 516)).astype(np.float32)
    d = dev(a)
    out = torch.empty((2400, 512), device="cuda")
    lib.launch(lib.compile(softmax_ir()), (2400, 512), [out, d], strides=[None, [516, 1]], offsets=[0, 1])
    assert ".stage" not in lib.last_variant()
    np.testing.assert_allclose(host(out), oracle.softmax(np.ascontiguousarray(a[:, 1:513])), rtol=1e-5, atol=1e-9)


@pytest.mark.parametrize("shape", [(20, 200000), (9, 300001), (150, 65536), (3, 1 << 20)])
def test_few_long_rows_shared_by_a_thread_block_cluster(lib, shape):
    """Rows too long for one CTA's registers and too few to fill the machine one CTA each: the row skeleton's `cluster`
    variant gives every row to a thread-block cluster, each CTA a slice of the columns, partial results exchanged through
    distributed shared memory and folded in rank order.  Softmax, sum, max and argmax (first occurrence across the
    CTAs' slices) against the oracle; rows whose length is not a multiple of the cluster's slices."""
    import dali_oracle as oracle
    from dali_b200.ir import softmax_ir
    rows, cols = shape
    rng = np.random.default_rng(rows + cols)
    a = rng.standard_normal((rows, cols)).astype(np.float32)
    a[0, cols - 7] = a[0, 11] = 9.5                       # a tie between the first and the last slice
    d = dev(a)
    out = torch.empty((rows, cols), device="cuda")
    lib.launch(lib.compile(softmax_ir()), (rows, cols), [out, d])
    assert ".cl" in lib.last_variant(), lib.last_variant()
    # (held to the fp64 softmax: the reference's own sequential fp32 sum over rows this long is 1e-4 off)
    e = np.exp(a.astype(np.float64) - a.max(1, keepdims=True))
    np.testing.assert_allclose(host(out), e / e.sum(1, keepdims=True), rtol=1e-5, atol=1e-12)
    for kind in ("sum", "max"):
        o = torch.empty(rows, device="cuda")
        lib.launch(lib.compile(reduce_ir(kind, "f32", 2, 1)), (rows, cols), [o, d])
        assert ".cl" in lib.last_variant(), lib.last_variant()
        if kind == "max":
            np.testing.assert_array_equal(host(o), a.max(1))
        else:
            want, bound = oracle.sum_f64acc(a, 1)
            assert np.all(np.abs(host(o) - want) <= 1e-5 * bound)
    o = torch.empty(rows, device="cuda", dtype=torch.int32)
    lib.launch(lib.compile(reduce_ir("max", "f32", 2, 1, True)), (rows, cols), [o, d])
    got = host(o)
    np.testing.assert_array_equal(got, oracle.argreduce("max", a, 1))
    assert got[0] == 11


@pytest.mark.parametrize("kind", ["max", "min"])
@pytest.mark.parametrize("shape", [(300, 200), (2048, 1536)])
def test_value_and_position_pairs_in_one_kernel(lib, kind, shape):
    """arg_pair_ir: the extreme value and its first position (+ an offset) from one kernel -- what a rank computes of a sharded
    argmax / argmin before the ranks' pairs are combined.  Over the last axis (row skeleton), over axis 0 (column skeleton,
    where the extreme is read off the arg-reduction's running pair) and over all axes; integer-valued inputs with many ties."""
    from dali_b200.ir import arg_pair_ir
    R, C = shape
    g = torch.Generator(device="cuda")
    g.manual_seed(R + C)
    x = torch.randint(-5, 6, (R, C), generator=g, device="cuda").float()
    xn = x.cpu().numpy()
    off = np.int32(1000)
    pick, argpick = (np.max, np.argmax) if kind == "max" else (np.min, np.argmin)
    h = lib.compile(arg_pair_ir(kind, "f32", 2, 1))
    vals, pos = torch.empty(R, device="cuda"), torch.empty(R, dtype=torch.int32, device="cuda")
    lib.launch(h, (R, C), [vals, pos, x], scalars=[off])
    assert lib.last_variant().startswith("row.")
    np.testing.assert_array_equal(vals.cpu().numpy(), pick(xn, axis=1))
    np.testing.assert_array_equal(pos.cpu().numpy(), argpick(xn, axis=1) + 1000)
    vals, pos = torch.empty(C, device="cuda"), torch.empty(C, dtype=torch.int32, device="cuda")
    lib.launch(h, (C, R), [vals, pos, x], strides=[None, None, [1, C]], scalars=[off])
    assert lib.last_variant().startswith("col.")
    np.testing.assert_array_equal(vals.cpu().numpy(), pick(xn, axis=0))
    np.testing.assert_array_equal(pos.cpu().numpy(), argpick(xn, axis=0) + 1000)
    h2 = lib.compile(arg_pair_ir(kind, "f32", 2, 2))
    vals, pos = torch.empty(1, device="cuda"), torch.empty(1, dtype=torch.int32, device="cuda")
    lib.launch(h2, (R, C), [vals, pos, x], scalars=[off])
    assert lib.last_variant().startswith("all.")
    assert float(vals) == float(pick(xn)) and int(pos) == int(argpick(xn)) + 1000
