"""op::uniform / normal / bernoulli on the GPU.  The reference's own CPU (mt19937) and GPU (thrust)
streams differ from each other (dali/array/op/random.cu.cpp:59-88 vs 153-232), so there is no
reference stream to match: the checks are bit-exactness against the CPU restatement of the
counter-based generator (oracle/dali_oracle.py, pinned by the published Philox4x32-10 known-answer
vectors), determinism under set_seed, ranges and moments."""
import numpy as np
import pytest

import dali_oracle as oracle
from dali_b200.array import Array, DTYPE_DOUBLE, DTYPE_FLOAT, DTYPE_INT32, lazy_stats, op, set_seed

pytestmark = pytest.mark.gpu


def test_uniform_stream_is_the_restated_philox():
    # the index part of the contract, seed fixed through the low-level IR
    import torch
    import dali_b200
    from dali_b200.ir import IRBuilder
    L = dali_b200.load_library()
    L.init()
    for dt, npdt, tdt in (("f32", np.float32, torch.float32), ("f64", np.float64, torch.float64)):
        for fn, ref in (("rng_uniform", oracle.rng_uniform), ("rng_normal", oracle.rng_normal)):
            b = IRBuilder(1, 0)
            out = b.arg(dt)
            idx = b.arg("i32", iota=True)
            seed = b.scalar("i32")
            b.st(out, b.op(fn, b.ld(idx), b.sc(seed), dtype=dt))
            h = L.compile(b.text())
            n = 100003
            o = torch.empty(n, dtype=tdt, device="cuda")
            L.launch(h, (n,), [o, 0], scalars=[np.int32(123456789)], strides=[None, [1]])
            torch.cuda.synchronize()
            got, want = o.cpu().numpy(), ref(n, 123456789, npdt)
            if fn == "rng_uniform":
                np.testing.assert_array_equal(got, want)
            else:
                np.testing.assert_allclose(got, want, rtol=2e-5 if dt == "f32" else 1e-12, atol=2e-6 if dt == "f32" else 1e-14)


def test_determinism_and_independence():
    set_seed(42)
    a = op.uniform(Array(0.0, DTYPE_FLOAT), Array(1.0, DTYPE_FLOAT), (257, 33))
    b = op.uniform(Array(0.0, DTYPE_FLOAT), Array(1.0, DTYPE_FLOAT), (257, 33))
    av, bv = a.numpy(), b.numpy()
    assert not np.array_equal(av, bv)                    # two nodes, two seeds
    np.testing.assert_array_equal(a.numpy(), av)         # one node, one stream, however often it is evaluated
    set_seed(42)
    a2 = op.uniform(Array(0.0, DTYPE_FLOAT), Array(1.0, DTYPE_FLOAT), (257, 33))
    np.testing.assert_array_equal(a2.numpy(), av)
    # the same numbers whatever the shape they are laid out in (the stream is indexed by element)
    set_seed(42)
    flat = op.uniform(Array(0.0, DTYPE_FLOAT), Array(1.0, DTYPE_FLOAT), (257 * 33,))
    np.testing.assert_array_equal(flat.numpy(), av.ravel())


def test_ranges_and_moments():
    set_seed(7)
    n = (1024, 1024)
    u = op.uniform(Array(-2.0, DTYPE_FLOAT), Array(3.0, DTYPE_FLOAT), n).numpy()
    assert u.dtype == np.float32 and u.min() >= -2.0 and u.max() < 3.0
    assert abs(u.mean() - 0.5) < 0.01 and abs(u.var() - 25.0 / 12.0) < 0.02
    g = op.normal(Array(1.0, DTYPE_FLOAT), Array(2.0, DTYPE_FLOAT), n).numpy()
    assert abs(g.mean() - 1.0) < 0.01 and abs(g.std() - 2.0) < 0.01
    assert abs(np.mean(((g - 1.0) / 2.0) ** 4) - 3.0) < 0.05                  # kurtosis of a normal
    gd = op.normal(0.0, 1.0, (512, 512)).numpy()
    assert gd.dtype == np.float64 and abs(gd.mean()) < 0.01 and abs(gd.std() - 1.0) < 0.01
    k = op.uniform(Array(0, DTYPE_INT32), Array(6, DTYPE_INT32), n).numpy()      # inclusive, tests.cpp:1001
    assert k.dtype == np.int32 and k.min() == 0 and k.max() == 6
    counts = np.bincount(k.ravel(), minlength=7) / k.size
    assert np.all(np.abs(counts - 1.0 / 7.0) < 0.002)
    m = op.bernoulli(Array(0.3, DTYPE_FLOAT), n).numpy()
    assert set(np.unique(m)) == {0.0, 1.0} and abs(m.mean() - 0.3) < 0.003
    mn = op.bernoulli_normalized(Array(0.25, DTYPE_FLOAT), n).numpy()
    assert set(np.unique(mn)) == {0.0, 4.0} and abs(mn.mean() - 1.0) < 0.01


def test_dropout_is_one_kernel():
    set_seed(3)
    x_np = np.random.default_rng(0).standard_normal((300, 70)).astype(np.float32)
    mask = op.bernoulli_normalized(Array(0.5, DTYPE_FLOAT), (300, 70))
    y = Array(x_np) * mask
    before = lazy_stats()
    yv = y.numpy()
    after = lazy_stats()
    assert after["kernels"] - before["kernels"] == 1 and after["temporaries"] == before["temporaries"]
    mv = mask.numpy()
    np.testing.assert_array_equal(yv, x_np * mv)         # the mask the product saw is the mask the node yields
