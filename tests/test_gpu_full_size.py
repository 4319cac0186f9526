"""The benchmark configurations at full size through size-independent properties, through the C ABI: exact inputs (integer-valued
floats, whose partial sums are exact in fp32 whatever the order), a checksum of checksums, and
sortedness of arg-reduction answers.  Small-size parity with the oracle is in the other GPU tests."""
import numpy as np
import pytest
import torch

from dali_b200.ir import chain_sum_ir, reduce_ir, softmax_ir

pytestmark = pytest.mark.gpu
N = 8192


@pytest.fixture(scope="module")
def x8192():
    g = torch.Generator(device="cuda")
    g.manual_seed(1236)
    return torch.randint(-3, 4, (N, N), generator=g, device="cuda").float()      # sums stay exact in fp32


def test_config3_reductions_at_full_size(lib, x8192):
    """fp32 [8192,8192]: sum / max / argmax over axis -1, axis 0 (the strided case) and all, exact."""
    x = x8192
    for kind in ("sum", "max"):
        h_row = lib.compile(reduce_ir(kind, "f32", 2, 1))
        out = torch.empty(N, device="cuda")
        lib.launch(h_row, (N, N), [out, x])
        want = x.sum(1) if kind == "sum" else x.max(1).values
        assert torch.equal(out, want)
        lib.launch(h_row, (N, N), [out, x], strides=[None, [1, N]])              # axis 0 = last axis of the transposed view
        want = x.sum(0) if kind == "sum" else x.max(0).values
        assert torch.equal(out, want)
        h_all = lib.compile(reduce_ir(kind, "f32", 2, 2))
        one = torch.empty(1, device="cuda")
        lib.launch(h_all, (N, N), [one, x])
        assert float(one) == float(x.sum(dtype=torch.float64) if kind == "sum" else x.max())
    h_arg = lib.compile(reduce_ir("max", "f32", 2, 1, arg=True))
    idx = torch.empty(N, dtype=torch.int32, device="cuda")
    lib.launch(h_arg, (N, N), [idx, x])
    # first occurrence of the row maximum: nothing before it reaches the maximum
    rows = torch.arange(N, device="cuda")
    mx = x.max(1).values
    assert torch.equal(x[rows, idx.long()], mx)
    first = (x == mx[:, None]).float().argmax(1)
    assert torch.equal(idx.long(), first)
    lib.launch(h_arg, (N, N), [idx, x], strides=[None, [1, N]])
    first0 = (x == x.max(0).values[None, :]).float().argmax(0)
    assert torch.equal(idx.long(), first0)


def test_config1_softmax_rows_sum_to_one_and_keep_order(lib):
    a = torch.randn(4096, 1024, device="cuda")
    out = torch.empty_like(a)
    lib.launch(lib.compile(softmax_ir()), (4096, 1024), [out, a])
    assert torch.allclose(out.sum(1, dtype=torch.float64), torch.ones(4096, dtype=torch.float64, device="cuda"), atol=1e-5)
    assert torch.equal(out.argmax(1), a.argmax(1)) and bool((out > 0).all())
    # shifting a row by a constant does not change its softmax (to rounding)
    out2 = torch.empty_like(a)
    lib.launch(lib.compile(softmax_ir()), (4096, 1024), [out2, a + 3.0])
    assert torch.allclose(out, out2, rtol=2e-5, atol=1e-9)


def test_config5_chain_sum_is_the_sum_of_its_parts(lib):
    """2^31 elements in one launch (64-bit sizes) against the sum of eight 2^28 launches."""
    n = 1 << 31
    x = torch.randn(n, device="cuda")
    h = lib.compile(chain_sum_ir())
    w, b = np.float32(0.5), np.float32(0.1)
    whole = torch.zeros(1, device="cuda")
    lib.launch(h, (n,), [whole, x], scalars=[w, b])
    parts = torch.zeros(8, device="cuda")
    step = n // 8
    for k in range(8):
        lib.launch(h, (step,), [parts[k:k + 1], x[k * step:(k + 1) * step]], scalars=[w, b])
    torch.cuda.synchronize()
    total = float(parts.double().sum())
    # every term is positive and below 1: sum |y| = the sum itself
    assert abs(float(whole) - total) <= 1e-5 * total
    # a length that ends inside a chunk: the launch runs unchecked full chunks and one checked, partial chunk
    m = n - 3 * 4096 - 8
    head, tail = torch.zeros(1, device="cuda"), torch.zeros(1, device="cuda")
    lib.launch(h, (m,), [head, x[:m]], scalars=[w, b])
    assert ".nc" in lib.last_variant()
    lib.launch(h, (n - m,), [tail, x[m:]], scalars=[w, b])
    torch.cuda.synchronize()
    assert abs(float(whole) - (float(head) + float(tail))) <= 1e-5 * total
    ref = float((torch.sigmoid(x[:1 << 24].double() * 0.5 + 0.1) * torch.exp(-x[:1 << 24].double() ** 2)).sum())
    chunk = torch.zeros(1, device="cuda")
    lib.launch(h, (1 << 24,), [chunk, x[:1 << 24]], scalars=[w, b])
    assert abs(float(chunk) - ref) <= 1e-5 * ref


def test_config3_nine_reductions_on_uniform_8192_through_arrays():
    """sum / max / argmax over axis -1, axis 0 and all axes of fp32 [8192,8192] ~ U(-1,1), evaluated through the Array front end,
    against the oracle: sums within 1e-5 * sum|x| of the double-accumulated sum, max exactly, argmax bit-exact."""
    import dali_oracle as oracle
    from dali_b200.array import Array, op, last_variant
    x = (np.random.default_rng(1236).random((N, N)) * 2 - 1).astype(np.float32)
    X = Array(x)
    for axis, skeleton in ((-1, "row."), (0, "col."), (None, "all.")):
        axes = None if axis is None else [axis]
        got = op.sum(X, axes).numpy().reshape(-1)
        assert last_variant().startswith(skeleton)
        s64, sabs = oracle.sum_f64acc(x, axis)
        assert np.all(np.abs(got - s64.reshape(-1)) <= 1e-5 * sabs.reshape(-1))
        np.testing.assert_array_equal(op.max(X, axes).numpy().reshape(-1), oracle.reduce("max", x, axis).reshape(-1))
        am = op.argmax(X) if axis is None else op.argmax(X, axis)
        np.testing.assert_array_equal(am.numpy().reshape(-1), oracle.argreduce("max", x, axis).reshape(-1))
