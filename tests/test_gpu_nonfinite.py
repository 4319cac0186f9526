"""NaN and infinities through the fast paths: the fp32 sigmoid (its clamp must not swallow a NaN: the reference's
1 / (1 + exp(-a)), dali/array/functor.h:157-162, propagates it), the LSTM gating fused as a GEMM epilogue, and the
3xTF32 product with an infinite operand (the reference's sgemm returns +-inf there)."""
import numpy as np
import pytest
import torch

from dali_b200.ir import IRBuilder, gemm_store_ir, lstm_cell_epilogue_ir

pytestmark = pytest.mark.gpu


def test_sigmoid_keeps_nan_and_saturates_at_infinity(lib):
    x = torch.tensor([float("nan"), float("inf"), float("-inf"), 0.0, 200.0, -200.0, 1.5] * 64, device="cuda")
    for name, scalars in (("sigmoid", None), ("steep_sigmoid", [np.float32(2.0)])):
        b = IRBuilder(1, 0)
        o, a = b.arg("f32"), b.arg("f32")
        v = b.ld(a)
        b.st(o, b.op(name, v, b.sc(b.scalar("f32"))) if scalars else b.op(name, v))
        out = torch.zeros_like(x)
        lib.launch(lib.compile(b.text()), (x.numel(),), [out, x], scalars=scalars)
        torch.cuda.synchronize()
        got = out.cpu().numpy()[:7]
        g = 2.0 if scalars else 1.0
        assert np.isnan(got[0]), (name, got)
        assert got[1] == 1.0 and abs(got[2]) < 1e-37 and got[3] == 0.5 and got[4] == 1.0 and abs(got[5]) < 1e-37
        assert abs(got[6] - 1.0 / (1.0 + np.exp(-g * 1.5))) < 1e-6
    # any_isnan over the result sees it
    from dali_b200.array import Array, op
    y = op.sigmoid(Array(x.cpu().numpy()))
    assert bool(op.any_isnan(y).numpy())


def test_nan_reaches_the_outputs_of_the_fused_lstm_epilogue(lib):
    B, H = 64, 128
    rng = np.random.default_rng(0)
    x, h, c = (rng.standard_normal((B, H)).astype(np.float32) for _ in range(3))
    Wx, Wh = ((rng.standard_normal((H, 4 * H)) * 0.05).astype(np.float32) for _ in range(2))
    b = np.zeros(4 * H, np.float32)
    b[5] = np.nan                   # input gate of unit 5, every row
    b[2 * H + 9] = np.nan           # output gate of unit 9: only h' is affected
    d = [torch.from_numpy(v).cuda() for v in (x, Wx, h, Wh)]
    bd, cd = torch.from_numpy(b).cuda(), torch.from_numpy(c).cuda()
    c_new, h_new = torch.zeros(B, H, device="cuda"), torch.zeros(B, H, device="cuda")
    row = [0, 1]
    lib.gemm_fused_sum(0, B, H, [(H, d[0], H, d[1], 4 * H), (H, d[2], H, d[3], 4 * H)], lib.compile(lstm_cell_epilogue_ir()),
                       [c_new, h_new, bd, bd, bd, bd, cd], strides=[None, None, row, row, row, row, None],
                       offsets=[0, 0, 0, H, 2 * H, 3 * H, 0])
    torch.cuda.synchronize()
    assert lib.gemm_error_flag() == 0
    cn, hn = c_new.cpu().numpy(), h_new.cpu().numpy()
    assert np.isnan(cn[:, 5]).all() and np.isnan(hn[:, 5]).all()
    assert np.isfinite(cn[:, 9]).all() and np.isnan(hn[:, 9]).all()
    mask = np.ones(H, bool)
    mask[[5, 9]] = False
    assert np.isfinite(cn[:, mask]).all() and np.isfinite(hn[:, mask]).all()


def test_tf32x3_product_with_an_infinite_operand(lib):
    """An infinite element of A makes its row of the product +-inf (sign of the matching B element), as sgemm does --
    not NaN: the low part of the split of an infinity is zero, not inf - inf.  (B here has no element whose low part is
    zero; inf times such an element is still inf . 0 = NaN in the correction product.)"""
    m, n, k = 128, 128, 64
    rng = np.random.default_rng(1)
    a = rng.standard_normal((m, k)).astype(np.float32)
    bm = (rng.standard_normal((k, n)) + 3.0).astype(np.float32)
    bm = (bm.view(np.uint32) | 1).view(np.float32)                  # no element is exactly representable in TF32
    a[3, 7] = np.inf
    a[40, 0] = -np.inf
    out = torch.zeros(m, n, device="cuda")
    lib.gemm_fused(0, m, n, k, torch.from_numpy(a).cuda(), k, torch.from_numpy(bm).cuda(), n, lib.compile(gemm_store_ir("f32")), [out])
    torch.cuda.synchronize()
    assert lib.gemm_error_flag() == 0 and lib.last_gemm_kernel().startswith("tcgen05.tf32x3")
    got = out.cpu().numpy()
    with np.errstate(invalid="ignore", over="ignore"):
        want = a.astype(np.float64) @ bm.astype(np.float64)
    assert np.array_equal(np.isinf(got), np.isinf(want)) and not np.isnan(got).any()
    assert np.array_equal(np.sign(got[np.isinf(got)]), np.sign(want[np.isinf(want)]))
    fin = np.isfinite(want)
    bound = np.abs(np.where(np.isfinite(a), a, 0)).astype(np.float64) @ np.abs(bm).astype(np.float64)
    assert np.all(np.abs(got[fin] - want[fin]) <= 1e-5 * bound[fin])
