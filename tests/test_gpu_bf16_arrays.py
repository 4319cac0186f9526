"""bf16 as a storage dtype of the Array front end (not in the reference, whose dtypes are float, double and int32:
dali/array/dtype.h:6-10).  Benchmark configuration 4 written as the reference would write it,
op::tanh(op::dot(A, B) + bias), on bf16 Arrays: the oracle is the reference's fp32 product on the bf16-rounded inputs
(tolerance 1e-2, bf16 outputs at bf16 rounding).  Everything else computed on a bf16 Array is computed on its float
values, exactly."""
import numpy as np
import pytest

import dali_oracle as oracle
from dali_b200.array import (Array, DTYPE_BF16, DTYPE_FLOAT, from_bf16_bits, last_ir, last_variant, lazy_stats, op, to_bf16_bits)

pytestmark = pytest.mark.gpu


def rounded(x):
    return from_bf16_bits(to_bf16_bits(x))


def test_rounding_matches_the_host_conversion_bit_for_bit(lib):
    rng = np.random.default_rng(0)
    x = rng.standard_normal(100000).astype(np.float32) * 100
    x[:8] = [np.nan, np.inf, -np.inf, 0.0, -0.0, 1.00390625, 1.01171875, 3.3895314e38]     # two exact halfway cases
    a = Array(x)
    got = a.astype(DTYPE_BF16).numpy()
    assert got.dtype == np.uint16
    want = to_bf16_bits(x)
    assert np.array_equal(got[1:], want[1:]) and (got[0] & 0x7F80) == 0x7F80 and (got[0] & 0x7F) != 0       # NaN stays NaN
    back = Array(got, dtype=DTYPE_BF16).astype(DTYPE_FLOAT).numpy()
    np.testing.assert_array_equal(back[1:], from_bf16_bits(want)[1:])


def test_config_4_expression_on_bf16_arrays(lib):
    rng = np.random.default_rng(4)
    m, k, n = 256, 512, 384
    a = rounded((rng.standard_normal((m, k)) * 0.02).astype(np.float32))
    b = rounded((rng.standard_normal((k, n)) * 0.02).astype(np.float32))
    bias = (rng.standard_normal(n) * 0.1).astype(np.float32)
    A, B, bias_a = Array(a, dtype=DTYPE_BF16), Array(b, dtype=DTYPE_BF16), Array(bias)
    assert A.dtype == DTYPE_BF16 and op.dot(A, B).dtype == DTYPE_FLOAT
    before = lazy_stats()
    y = op.tanh(op.dot(A, B) + bias_a[None, :])
    out32 = y.numpy()
    after = lazy_stats()
    assert after["gemms"] - before["gemms"] == 1 and after["kernels"] == before["kernels"]       # ONE launch: GEMM + epilogue
    assert last_variant().startswith("tcgen05.bf16"), last_variant()
    want = np.tanh(oracle.gemm(a, b) + bias)                                 # fp32 sgemm restated, bf16-rounded inputs
    np.testing.assert_allclose(out32, want, rtol=1e-2, atol=1e-4)
    exact = np.tanh(a.astype(np.float64) @ b.astype(np.float64) + bias)
    np.testing.assert_allclose(out32, exact, rtol=1e-5, atol=1e-6)           # (fp32 accumulation of exact products)
    out16 = op.tanh(op.dot(A, B) + bias_a[None, :]).astype(DTYPE_BF16)
    bits = out16.numpy()
    assert out16.dtype == DTYPE_BF16 and bits.dtype == np.uint16 and "bf16_round" in last_ir()
    np.testing.assert_allclose(from_bf16_bits(bits), exact, rtol=2.0 ** -8, atol=1e-6)
    # assignment into a bf16 destination rounds the same way
    dest = Array.zeros((m, n), DTYPE_BF16)
    dest.assign(op.tanh(op.dot(A, B) + bias_a[None, :]))
    np.testing.assert_array_equal(dest.numpy(), bits)
    # += into a float destination
    acc = Array(np.ones((m, n), np.float32))
    acc += op.dot(A, B)
    np.testing.assert_allclose(acc.numpy(), 1.0 + a.astype(np.float64) @ b.astype(np.float64), rtol=1e-5, atol=1e-6)


def test_everything_else_computes_on_the_float_values(lib):
    rng = np.random.default_rng(9)
    x = rounded(rng.standard_normal((300, 200)).astype(np.float32))
    X = Array(x, dtype=DTYPE_BF16)
    assert X.T.dtype == DTYPE_BF16 and X[3:9].dtype == DTYPE_BF16 and (X * 2.0).dtype != DTYPE_BF16
    np.testing.assert_array_equal(op.exp(X).numpy(), op.exp(Array(x)).numpy())
    np.testing.assert_array_equal((X.T + 1.0).numpy(), (x.T.astype(np.float64) + 1.0))
    np.testing.assert_array_equal(op.max(X, [0]).numpy(), x.max(0))
    np.testing.assert_array_equal(op.argmax(X, 1).numpy(), oracle.argreduce("max", x, 1))
    s = op.sum(X).numpy()
    assert abs(float(s) - x.astype(np.float64).sum()) <= 1e-5 * np.abs(x).sum()
    np.testing.assert_allclose(op.softmax(X, -1).numpy(), oracle.softmax(x), rtol=1e-5, atol=1e-9)
    idx = rng.integers(0, 300, 50).astype(np.int32)
    g = op.gather(X, Array(idx))
    assert g.dtype == DTYPE_FLOAT
    np.testing.assert_array_equal(g.numpy(), x[idx])
    np.testing.assert_array_equal(op.cumsum(X[:4]).numpy(), op.cumsum(Array(x[:4])).numpy())
    assert float(X[5][7].astype(DTYPE_FLOAT).numpy()) == x[5, 7]
    # a strided bf16 destination
    d = Array.zeros((300, 400), DTYPE_BF16)
    d[:, ::2].assign(Array(x) * 3.0)
    got = from_bf16_bits(d.numpy())
    np.testing.assert_array_equal(got[:, ::2], rounded(x * np.float32(3.0)))
    assert not got[:, 1::2].any()


def test_bf16_arrays_and_npy_files(lib, tmp_path):
    x = rounded(np.random.default_rng(2).standard_normal((17, 5)).astype(np.float32))
    X = Array(x, dtype=DTYPE_BF16)
    X.save(tmp_path / "x.npy")
    np.testing.assert_array_equal(np.load(tmp_path / "x.npy"), x)            # written as the float32 values it holds
    back = Array.load(tmp_path / "x.npy").astype(DTYPE_BF16)
    np.testing.assert_array_equal(back.numpy(), to_bf16_bits(x))


def test_bf16_products_that_the_tensor_core_path_cannot_take_are_refused(lib):
    from dali_b200 import DaliB200Error
    a = Array(np.ones((64, 64), np.float32), dtype=DTYPE_BF16)
    with pytest.raises(DaliB200Error, match="tensor cores only"):
        op.dot(a.T, a).numpy()                                               # a transposed view of a bf16 matrix
