"""Host logic of the lazy Array / op:: front end, without a GPU: shapes and
view algebra, error behaviour (the reference's tests expect std::runtime_error,
which arrives here as DaliB200Error), and -- in dry-run mode, where kernels are
lowered and NVRTC-compiled but nothing is launched -- what fuses into what."""
import numpy as np
import pytest

import dali_b200
from dali_b200 import DaliB200Error
from dali_b200.array import (Array, DTYPE_DOUBLE, DTYPE_FLOAT, DTYPE_INT32, last_ir, last_variant, lazy_stats, op,
                             set_dry_run)


@pytest.fixture(autouse=True, scope="module")
def dry(tmp_path_factory):
    dali_b200.load_library().cache_set_dir(str(tmp_path_factory.mktemp("dali_cache")))
    set_dry_run(True)
    yield
    set_dry_run(False)


def launched(arr):
    before = lazy_stats()
    arr.eval()
    after = lazy_stats()
    return {k: after[k] - before[k] for k in after}


def test_shapes_and_views():
    a = Array(np.zeros((3, 4, 5), np.float32))
    assert a.shape == (3, 4, 5) and a.ndim == 3 and a.dtype == DTYPE_FLOAT
    assert a[1].shape == (4, 5)
    assert a[:, 1:3].shape == (3, 2, 5)
    assert a[:, ::2, 4].shape == (3, 2)
    assert a[None].shape == (1, 3, 4, 5)
    assert a.T.shape == (5, 4, 3)
    assert a.transpose([1, 0, 2]).shape == (4, 3, 5)
    assert a.reshape([12, 5]).shape == (12, 5)
    assert a.reshape([-1]).shape == (60,)
    assert a.expand_dims(1).squeeze(1).shape == (3, 4, 5)
    assert a[:, 0:1].broadcast_to_shape([3, 7, 5]).shape == (3, 7, 5)
    # views of lazy nodes keep being lazy
    e = op.exp(a)
    assert e[1].shape == (4, 5) and not e.is_buffer()
    assert op.sum(a, [1], True).shape == (3, 1, 5)
    assert op.sum(a, [0, 2]).shape == (4,)
    assert op.argmax(a, 1).shape == (3, 5) and op.argmax(a, 1).dtype == DTYPE_INT32
    assert op.sum(a).shape == () and op.argmax(a).dtype == DTYPE_INT32


def test_type_promotion():
    f = Array(np.zeros((2, 2), np.float32))
    d = Array(np.zeros((2, 2), np.float64))
    i = Array(np.zeros((2, 2), np.int32))
    assert (f + d).dtype == DTYPE_DOUBLE and (f + i).dtype == DTYPE_FLOAT and (d + i).dtype == DTYPE_DOUBLE
    assert (i + i).dtype == DTYPE_INT32 and (i * 2).dtype == DTYPE_INT32 and (i * 2.0).dtype == DTYPE_DOUBLE
    assert op.mean(i).dtype == DTYPE_DOUBLE          # reducers.cpp: mean of ints is a double
    assert f.astype(DTYPE_INT32).dtype == DTYPE_INT32


def test_errors_like_the_reference():
    a = Array(np.zeros((3, 4), np.float32))
    b = Array(np.zeros((3, 5), np.float32))
    v = Array(np.zeros((4,), np.float32))
    with pytest.raises(DaliB200Error):      # incompatible shapes
        (a + b).eval()
    with pytest.raises(DaliB200Error):      # rank mismatch (tests.cpp:613)
        a + v
    with pytest.raises(DaliB200Error):      # reduction axis out of range
        op.sum(a, [2])
    with pytest.raises(DaliB200Error):      # duplicate axes
        op.sum(a, [0, 0])
    with pytest.raises(DaliB200Error):      # slice out of range (python slices clamp, Slice(2, 9) does not)
        Array._new(dali_b200.load_library().c.dali_array_slice, a._h, 1, 2, 9, 1)
    with pytest.raises(DaliB200Error):      # index out of range
        a[3]
    with pytest.raises(DaliB200Error):      # reshape changes element count (tests.cpp:438-440)
        a.reshape([5, 5])
    with pytest.raises(DaliB200Error):      # gather needs int32 indices
        op.gather(a, Array(np.zeros((2,), np.float32)))
    with pytest.raises(DaliB200Error):      # dot shapes (dot_tests.cpp:213-216)
        op.dot(a, b)
    with pytest.raises(DaliB200Error):      # unknown functor name through the binding
        op._unary("nosuchop", a)


def test_softmax_is_one_kernel_without_temporaries():
    a = Array(np.zeros((4096, 1024), np.float32))
    exped = op.exp(a - op.max(a, [-1], True))
    s = exped / op.sum(exped, [-1], True)
    assert "View(max(Buffer))" in s.expression_name()
    assert launched(s) == {"kernels": 1, "gemms": 0, "temporaries": 0}
    ir = last_ir()
    assert ir.count(" ld ") == 1 and ir.count("red max") == 1 and ir.count("red sum") == 1 and ir.count("op exp") == 1
    assert last_variant().startswith("row.") and ".v4." in last_variant()
    assert s.is_buffer()                       # evaluated once, remembered
    assert launched(s) == {"kernels": 0, "gemms": 0, "temporaries": 0}
    # the library composition lowers to the very same program
    s2 = op.softmax(Array(np.zeros((4096, 1024), np.float32)))
    s2.eval()
    assert last_ir() == ir


def test_reduction_skeletons_from_the_front_end():
    x = Array(np.zeros((2048, 2048), np.float32))
    for fn, want in ((lambda: op.sum(x, [-1]), "row."), (lambda: op.sum(x, [0]), "col."), (lambda: op.sum(x), "all."),
                     (lambda: op.max(x, [0], True), "col."), (lambda: op.argmax(x, 0), "col."),
                     (lambda: op.argmax(x, -1), "row."), (lambda: op.argmin(x), "all."),
                     (lambda: op.mean(x, [0]), "col."), (lambda: op.L2_norm(x, [-1]), "row.")):
        assert launched(fn()) == {"kernels": 1, "gemms": 0, "temporaries": 0}
        assert last_variant().startswith(want), (want, last_variant())


def test_chain_fuses_into_the_all_reduce():
    v = Array(np.zeros((1 << 20,), np.float32))
    s = op.sum(op.sigmoid(v * np.float32(0.5) + np.float32(0.1)) * op.exp(-v * v))
    assert launched(s) == {"kernels": 1, "gemms": 0, "temporaries": 0}
    ir = last_ir()
    assert "scalar 0 f32" in ir and "scalar 1 f32" in ir and " ld " in ir and ir.count(" ld ") == 1
    assert last_variant().startswith("all.")
    # other scalar values reuse the same program (values are run-time arguments)
    s2 = op.sum(op.sigmoid(v * np.float32(0.25) + np.float32(0.7)) * op.exp(-v * v))
    s2.eval()
    assert last_ir() == ir


def test_unfusable_subtrees_become_temporaries():
    x = Array(np.zeros((64, 64), np.float32))
    assert launched(x - op.mean(x)) == {"kernels": 2, "gemms": 0, "temporaries": 1}      # all-reduce inside a map
    assert launched(x / op.sum(x, [0], True)) == {"kernels": 2, "gemms": 0, "temporaries": 1}   # reduce over a leading dim
    y = op.sum(x, [-1], True) * op.max(x, [-1], True) + x                               # two row reductions: one kernel
    assert launched(y) == {"kernels": 1, "gemms": 0, "temporaries": 0}
    # an elementwise tree around a product is the epilogue of ONE tensor-core GEMM: no separate kernel
    w = Array(np.zeros((64, 32), np.float32))
    assert launched(op.tanh(op.dot(x, w) + Array(np.zeros((32,), np.float32))[None])) == {"kernels": 0, "gemms": 1, "temporaries": 0}
    assert "acc" in last_ir() and "op tanh" in last_ir() and last_variant().startswith("tcgen05")
    # layouts TMA cannot address (k = 62) go to the CUDA-core GEMM plus one fused elementwise kernel
    x62 = Array(np.zeros((64, 62), np.float32))
    w62 = Array(np.zeros((62, 32), np.float32))
    assert launched(op.tanh(op.dot(x62, w62) + 1.0)) == {"kernels": 1, "gemms": 1, "temporaries": 1}


def test_lstm_cell_lowering():
    """gates = dot(x,Wx) + dot(h,Wh) + b is evaluated once (one GEMM launch accumulating both products, "+ b" as its
    epilogue) because it is used through four column slices; each output is then one map kernel."""
    B, H = 32, 64
    x, h, c = (Array(np.zeros((B, H), np.float32)) for _ in range(3))
    Wx, Wh = (Array(np.zeros((H, 4 * H), np.float32)) for _ in range(2))
    b = Array(np.zeros((4 * H,), np.float32))
    gates = op.dot(x, Wx) + op.dot(h, Wh) + b[None, :]
    i, f, o = (op.sigmoid(gates[:, k * H:(k + 1) * H]) for k in range(3))
    g = op.tanh(gates[:, 3 * H:4 * H])
    c_new = f * c + i * g
    h_new = o * op.tanh(c_new)
    assert launched(h_new) == {"kernels": 1, "gemms": 1, "temporaries": 1}
    assert launched(c_new) == {"kernels": 1, "gemms": 0, "temporaries": 0}


def test_lstm_cell_outputs_together_are_one_gemm_and_one_kernel():
    from dali_b200.array import eval_together
    B, H = 32, 64
    x, h, c = (Array(np.zeros((B, H), np.float32)) for _ in range(3))
    Wx, Wh = (Array(np.zeros((H, 4 * H), np.float32)) for _ in range(2))
    b = Array(np.zeros((4 * H,), np.float32))
    gates = op.dot(x, Wx) + op.dot(h, Wh) + b[None, :]
    i, f, o = (op.sigmoid(gates[:, k * H:(k + 1) * H]) for k in range(3))
    g = op.tanh(gates[:, 3 * H:4 * H])
    c_new = f * c + i * g
    h_new = o * op.tanh(c_new)
    before = lazy_stats()
    eval_together(c_new, h_new)
    after = lazy_stats()
    # the whole cell is ONE GEMM launch: the gating is its epilogue over the four column blocks of the product
    assert {k: after[k] - before[k] for k in after} == {"kernels": 0, "gemms": 1, "temporaries": 0}
    assert c_new.is_buffer() and h_new.is_buffer()
    ir = last_ir()
    assert ir.count("st ") == 2 and ir.count("op tanh") == 2                   # c' computed once, both stored
    assert all(t in ir for t in (" acc\n", " acc 1\n", " acc 2\n", " acc 3\n"))
    assert ir.count(" ld ") == 5 and ".sl4" in last_variant() or "tf32x3" in last_variant()   # four bias blocks + c
    # evaluated one at a time (the reference's way) the gates are materialised once and sliced
    c2 = f * c + i * g
    assert launched(c2) == {"kernels": 1, "gemms": 1, "temporaries": 1}
    # what cannot share a kernel is evaluated one by one
    s, m = op.sum(x, [-1]), x * 2.0
    before = lazy_stats()
    eval_together(s, m)
    assert lazy_stats()["kernels"] - before["kernels"] == 2


def test_lstm_gating_on_slices_is_one_map_kernel():
    H = 128
    g = Array(np.zeros((16, 4 * H), np.float32))
    c = Array(np.zeros((16, H), np.float32))
    i, f, o = (op.sigmoid(g[:, k * H:(k + 1) * H]) for k in range(3))
    gg = op.tanh(g[:, 3 * H:4 * H])
    cn = f * c + i * gg
    hn = o * op.tanh(cn)
    assert launched(hn) == {"kernels": 1, "gemms": 0, "temporaries": 0}
    assert last_variant().startswith("map.o1.i1.v4.")
    assert last_ir().count(" ld ") == 5       # four gate slices + c, each read once


def test_inplace_and_scatter_lowering():
    a = Array(np.zeros((8, 8), np.float32))
    b = Array(np.zeros((8, 8), np.float32))
    # an update of a place runs when it is written (the arrays it reads may change afterwards), as one kernel
    before = lazy_stats()
    a += b * 2.0
    assert {k: lazy_stats()[k] - before[k] for k in before} == {"kernels": 1, "gemms": 0, "temporaries": 0}
    assert launched(a) == {"kernels": 0, "gemms": 0, "temporaries": 0}
    assert "st 1 add" in last_ir() or "st 0 add" in last_ir()
    dest = Array.zeros((3,), DTYPE_INT32)
    idx = Array(np.array([0, 0, 1, 1, 1, 2], np.int32))
    gathered = dest[idx]
    before = lazy_stats()
    gathered += 1
    assert {k: lazy_stats()[k] - before[k] for k in before} == {"kernels": 1, "gemms": 0, "temporaries": 0}
    assert "stx" in last_ir() and " add " in last_ir()
    lse = Array.zeros((2, 1), DTYPE_INT32)
    lse <<= Array.ones((2, 5), DTYPE_INT32)
    assert "red sum" in last_ir()
    # a lazy value is not a place: the operator is folded into its expression and nothing runs
    lazy = op.tanh(a)
    before = lazy_stats()
    lazy += b
    assert lazy_stats() == before
    assert launched(lazy) == {"kernels": 1, "gemms": 0, "temporaries": 0}


def test_index_ops_are_lazy_and_fuse_into_one_kernel():
    """arange / eye / one_hot / outer are affine index expressions or views: no memory, no kernel of their own."""
    x = Array(np.zeros((3, 2), np.float32))
    r = x + op.arange(6).reshape((3, 2)).astype(DTYPE_FLOAT)
    assert launched(r) == {"kernels": 1, "gemms": 0, "temporaries": 0}
    assert " iota" in last_ir() and last_ir().count("arg ") == 3
    idx = Array(np.zeros((2, 3), np.int32))
    oh = op.one_hot(idx, 7, 112.2, 42.0)
    assert oh.shape == (2, 3, 7) and oh.dtype == DTYPE_DOUBLE
    assert launched(oh) == {"kernels": 1, "gemms": 0, "temporaries": 0}
    e = op.eye(4, 5)
    assert e.shape == (4, 5) and launched(e) == {"kernels": 1, "gemms": 0, "temporaries": 0}
    assert last_ir().count(" iota") == 2 and "where_nonzero" in last_ir()
    a, b = Array(np.zeros(3, np.float32)), Array(np.zeros(4, np.float32))
    o = op.outer(op.tanh(a - 3.0), op.tanh(b - 2.0))          # tests.cpp:968-974: chainable
    assert o.shape == (3, 4) and launched(o) == {"kernels": 1, "gemms": 0, "temporaries": 0}
    s = op.arange(24).reshape((2, 3, 4))[:, 1, ::2]            # slicing an arange stays an index expression
    assert s.shape == (2, 2) and launched(s) == {"kernels": 1, "gemms": 0, "temporaries": 0}
    with pytest.raises(RuntimeError):
        op.one_hot(Array(np.zeros(3, np.float32)), 4, 1.0, 0.0)
    with pytest.raises(RuntimeError):
        op.diag(Array(np.zeros(2, np.float32)), 3, 4)


def test_running_reduction_lowering():
    x = Array(np.zeros((4, 10), np.float32))
    c = op.cumsum(op.tanh(x))
    assert c.shape == (4, 10)
    assert launched(c) == {"kernels": 2, "gemms": 0, "temporaries": 0}      # fused producer, then the scan kernel
    assert last_variant() == "scan.inclusive_scan_sum"
    assert op.cumprod(x, inclusive=False).shape == (4, 11)
    y = op.cumsum(x) * 2.0                                                   # never fused with its consumer (scan.cpp:37-39)
    assert launched(y) == {"kernels": 2, "gemms": 0, "temporaries": 1}


def test_random_operators_fuse_into_their_consumer():
    """op::uniform / normal / bernoulli are functions of (element index, seed): a dropout mask is generated
    inside the kernel that applies it."""
    from dali_b200.array import set_seed
    set_seed(5)
    x = Array(np.zeros((64, 32), np.float32))
    y = x * op.bernoulli_normalized(Array(0.5, DTYPE_FLOAT), (64, 32))
    assert launched(y) == {"kernels": 1, "gemms": 0, "temporaries": 0}
    ir = last_ir()
    assert "rng_uniform" in ir and " iota" in ir and ir.count("arg ") == 3      # out, x, the index
    n = op.normal(0.0, 2.0, (5, 7))
    assert n.shape == (5, 7) and n.dtype == DTYPE_DOUBLE
    assert launched(n) == {"kernels": 1, "gemms": 0, "temporaries": 0} and "rng_normal" in last_ir()
    u = op.uniform(Array(0, DTYPE_INT32), Array(6, DTYPE_INT32), (2, 3))         # tests.cpp:1001: uniform(0, 6, {2, 3})
    assert u.dtype == DTYPE_INT32 and launched(u)["kernels"] == 1
    with pytest.raises(RuntimeError):
        op.uniform(Array(np.zeros(2, np.float32)), 1.0, (3,))


def test_npy_files_round_trip_with_numpy(tmp_path):
    """Array::load / Array::save against numpy's own reader and writer (reference tests: tests.cpp:745-776)."""
    set_dry_run(False)
    try:
        rng = np.random.default_rng(2)
        for arr in (np.arange(12, dtype=np.int32).reshape(3, 4), rng.standard_normal((2, 3, 5)).astype(np.float32),
                    rng.standard_normal(7), np.arange(5, dtype=np.float32)):
            p = tmp_path / "a.npy"
            np.save(p, arr)
            a = Array.load(p)
            assert a.shape == arr.shape and a.dtype == {np.dtype(np.int32): DTYPE_INT32, np.dtype(np.float32): DTYPE_FLOAT,
                                                          np.dtype(np.float64): DTYPE_DOUBLE}[arr.dtype]
            q = tmp_path / "b.npy"
            a.save(q)                                                          # host-fresh buffer: no device involved
            back = np.load(q)
            assert back.dtype == arr.dtype and not np.isfortran(back)
            np.testing.assert_array_equal(back, arr)
        # a Fortran-ordered file is the same array (tests.cpp:745-760: arange12.npy vs arange12.fortran.npy)
        f = np.asfortranarray(np.arange(12, dtype=np.float64).reshape(3, 4))
        np.save(tmp_path / "f.npy", f)
        af = Array.load(tmp_path / "f.npy")
        assert af.shape == (3, 4)
        with pytest.raises(RuntimeError):
            Array.load(tmp_path / "missing.npy")
        np.save(tmp_path / "i8.npy", np.arange(3, dtype=np.int64))
        with pytest.raises(RuntimeError):
            Array.load(tmp_path / "i8.npy")
    finally:
        set_dry_run(True)


def test_two_equal_subtrees_keep_their_own_temporaries():
    """all_close(softmax(a), softmax(a)): four temporaries (two row maxima, two row sums) feed one all-axis kernel.
    Nodes replaced by their evaluated buffers during lowering must not lend their addresses to later ones."""
    a = Array(np.zeros((5, 10), np.float32))

    def softmax():
        e = op.exp(a - op.max(a, [-1], True))
        return e / op.sum(e, [-1], True)

    # (built in one expression: a large value that a second handle also names would be evaluated on its own first)
    p = op.prod(op.lessthanequal(op.abs(op.subtract(softmax(), softmax())), Array(1e-6, DTYPE_DOUBLE)))
    assert launched(p) == {"kernels": 5, "gemms": 0, "temporaries": 4}
    ir = last_ir()
    assert ir.count("arg ") == 6 and ir.count(" ld ") == 5          # a, 2 maxima, 2 sums read; one result written


def test_prefix_slice_of_a_lazy_value_is_not_a_pure_reindexing():
    """b[:, 0:4] of a lazy [130, 9] value starts at 0 with step 1 but is narrower: it must be lowered as a slice,
    not peeled off the root like a transpose."""
    a = Array(np.zeros((130, 9), np.float32))
    w = op.tanh(a)[:, 0:4]
    assert w.shape == (130, 4)
    assert launched(w) == {"kernels": 1, "gemms": 0, "temporaries": 0}
    t = op.tanh(a).transpose()                      # a real permutation still is peeled: one kernel, transposed store
    assert launched(t) == {"kernels": 1, "gemms": 0, "temporaries": 0}


def test_an_update_that_reads_the_array_it_updates_runs_at_once():
    """w -= 0.1 * dw while dw += 2 * w is still pending: handles share their state, so a pending update of w
    installed in w's state would be read back by dw's pending value (a cycle; the reference's solvers build exactly
    this, dali/tensor/solver.cpp + op/solver_updates/sgd.cpp).  Such an update runs immediately instead."""
    w = Array(np.ones((4, 5), np.float32))
    dw = Array(np.zeros((4, 5), np.float32))
    dw += w * 2.0
    before = lazy_stats()
    w -= dw * 0.1                       # reads dw, whose pending value reads w
    ran = {k: lazy_stats()[k] - before[k] for k in before}
    assert ran["kernels"] >= 1          # not left pending
    assert launched(w) == {"kernels": 0, "gemms": 0, "temporaries": 0}
    x = Array(np.ones((3,), np.float32))
    x.assign(op.tanh(x) + x)            # x = f(x)
    assert launched(x) == {"kernels": 0, "gemms": 0, "temporaries": 0}


def test_large_shared_lazy_values_are_evaluated_once():
    """State carried from step to step as a lazy expression of its own previous value (the m and v of the reference's
    Adam, never evaluated by the caller) must not make every step's program longer than the last one's: a value that
    another handle names and whose tree has grown past a couple of dozen nodes is evaluated in place."""
    g = Array(np.ones((8, 8), np.float32))
    w = Array(np.ones((8, 8), np.float32))
    m = Array(np.zeros((8, 8), np.float32))
    sizes = []
    for step in range(12):
        m = m * 0.9 + g * 0.1 + op.square(g) * 0.01          # rebinding: m is a lazy tree over the previous m
        w -= m * 0.5
        w.eval()
        sizes.append(len(last_ir().splitlines()))
    assert max(sizes) < 80 and max(sizes[6:]) <= max(sizes[:6])   # bounded, not growing with the step count


def test_every_computation_opens_one_trace_scope():
    """dali/array/tests/dot_tests.cpp:17-35 counts the scopes a ScopeObserver sees to show that a product is one
    computation; the same count here, through the C binding of the observer (lowering only, nothing is launched)."""
    from dali_b200.array import scope_trace
    a, b = Array(np.ones((2, 3), np.float32)), Array(np.ones((3, 4), np.float32))
    with scope_trace() as t:
        c = op.dot(a, b)
        assert t.names == []
    with scope_trace() as t:
        c.eval()
    assert t.names == ["MatMul(Buffer, Buffer)"]
    x = Array(np.ones((8, 16), np.float32))
    with scope_trace() as t:
        op.softmax(x).eval()
    assert [n for n in t.names if n != "get_function"] == [
        "eltdiv(exp(subtract(Buffer, View(max(Buffer)))), View(sum(exp(subtract(Buffer, View(max(Buffer)))))))"]
    assert t.names.count("get_function") == 1
    # a reduction that cannot share the root's kernel is a computation of its own
    with scope_trace() as t:
        (x / op.sum(x)).eval()
    assert len([n for n in t.names if n != "get_function"]) == 2
    with scope_trace() as t:
        x.eval()                      # a buffer: nothing to do
    assert t.names == []


def test_shard_marks_travel_with_values_and_guard_the_axis():
    x = Array(np.zeros((64, 32), np.float32))
    x.set_shard(0, 64, 128)
    assert x.shard == (0, 64, 128)
    assert (x * 2.0 + 1.0).shard == (0, 64, 128)
    assert x.T.shard == (1, 64, 128) and x[:, 3:9].shard == (0, 64, 128) and x[None].shard == (1, 64, 128)
    assert x.reshape([64, 4, 8]).shard == (0, 64, 128) and x.reshape([-1]).shard == (0, 64 * 32, 128 * 32)
    assert op.sum(x, [1]).shard == (0, 64, 128) and op.sum(x, [0]).shard[0] == -1 and op.sum(x).shard[0] == -1
    assert op.softmax(x, -1).shard == (0, 64, 128)
    w = Array(np.zeros((32, 16), np.float32))
    assert op.dot(x, w).shard == (0, 64, 128)
    assert op.dot(w.T, x.T).shard == (1, 64, 128)
    assert op.dot(x.T, x).shard[0] == -1                       # contracts the sharded dimension: every rank gets the whole product
    for bad in (lambda: x[3], lambda: x[2:10], lambda: x[::2], lambda: op.gather(x, Array(np.zeros(4, np.int32))),
                lambda: op.dot(x.T, w[:, :16].T[:, :64] if False else Array(np.zeros((64, 8), np.float32))),
                lambda: x.reshape([32, 64]), lambda: op.cumsum(x.T)):
        with pytest.raises(DaliB200Error):
            bad()
    y = Array(np.zeros((64, 32), np.float32))
    y.set_shard(0, 0, 128)
    with pytest.raises(DaliB200Error, match="sharded differently"):
        x + y
    with pytest.raises(DaliB200Error):
        x.set_shard(0, 100, 128)                                # rows [100, 164) do not lie inside [0, 128)
    x.set_shard(-1, 0, 0)
    assert x.shard[0] == -1 and x[3].shape == (32,)


def test_overlapping_source_and_destination_lower_through_a_temporary():
    """The destination's buffer read through another index map (transpose in place, a shifted slice, a reduction of the array
    into one of its own rows, a product into one of its operands) takes one more launch for the temporary; identical maps
    (a = f(a), a += a) do not."""
    def ran(statement):
        before = lazy_stats()
        statement()
        after = lazy_stats()
        return {k: after[k] - before[k] for k in before}
    a = Array(np.zeros((64, 64), np.float32))
    assert ran(lambda: a.assign(a.transpose()))["kernels"] == 2
    assert ran(lambda: a[1:].assign(a[:-1]))["kernels"] == 2
    assert ran(lambda: a[0].assign(op.sum(a, [0])))["kernels"] == 2
    w = Array(np.zeros((64, 64), np.float32))
    r = ran(lambda: a.assign(op.dot(a, w)))
    assert r["gemms"] == 1 and r["kernels"] == 1              # product into a temporary, then the copy
    assert ran(lambda: a.assign(a * 2.0))["kernels"] == 1
    assert ran(lambda: a.__iadd__(a))["kernels"] == 1
    b = Array(np.zeros((128, 64), np.float32))
    assert ran(lambda: b[:64].assign(b[64:]))["kernels"] == 1   # disjoint halves of one buffer
