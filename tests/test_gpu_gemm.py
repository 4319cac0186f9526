"""dalib200_gemm (CUDA-core kernel for any layout) and dalib200_gemm_fused
(tcgen05 / TMEM kernel with the spliced epilogue) against the CPU oracle.

Tolerances: fp32 products |gpu - fp64| <= 1e-5 * (|A| . |B|) elementwise (the
3xTF32 split measures ~2e-6); bf16 inputs are exact in fp32 products, so the
fp32-accumulated result is compared at 1e-5 * (|A| . |B|) too, and bf16 outputs
at bf16 rounding (2^-8 relative); int32 bit-exact."""
import numpy as np
import pytest
import torch

import dali_oracle as oracle
from dali_b200.ir import IRBuilder, gemm_bias_tanh_ir, gemm_store_ir, lstm_cell_epilogue_ir

pytestmark = pytest.mark.gpu


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def host(t):
    torch.cuda.synchronize()
    return t.float().cpu().numpy() if t.dtype == torch.bfloat16 else t.cpu().numpy()


def to_bf16(x):
    """fp32 -> nearest-even bf16, returned as fp32 values and as a torch bf16 tensor."""
    t = torch.from_numpy(x).bfloat16()
    return t.float().numpy(), t.cuda()


@pytest.mark.parametrize("dtype", [np.float32, np.float64, np.int32])
def test_simt_gemm_layouts_and_accumulate(lib, dtype):
    rng = np.random.default_rng(0)
    m, n, k = 37, 29, 53
    if dtype == np.int32:
        a, b = rng.integers(-9, 9, (m, k)).astype(dtype), rng.integers(-9, 9, (k, n)).astype(dtype)
    else:
        a, b = rng.standard_normal((m, k)).astype(dtype), rng.standard_normal((k, n)).astype(dtype)
    code = {np.float32: 0, np.float64: 1, np.int32: 2}[dtype]
    want = a.astype(np.float64) @ b.astype(np.float64)
    tol = dict(rtol=0, atol=0) if dtype == np.int32 else dict(rtol=1e-5 if dtype == np.float32 else 1e-12, atol=1e-5 if dtype == np.float32 else 1e-12)
    c = torch.zeros((m, n), dtype=torch.from_numpy(a).dtype, device="cuda")
    lib.gemm(code, m, n, k, dev(a), (k, 1), dev(b), (n, 1), c, (n, 1))
    np.testing.assert_allclose(host(c), want, **tol)
    at, bt = np.ascontiguousarray(a.T), np.ascontiguousarray(b.T)          # transposed views
    lib.gemm(code, m, n, k, dev(at), (1, m), dev(bt), (1, k), c, (n, 1))
    np.testing.assert_allclose(host(c), want, **tol)
    big = np.zeros((2 * m, 3 * k), dtype)                                   # strided view
    big[::2, ::3] = a
    lib.gemm(code, m, n, k, dev(big), (2 * 3 * k, 3), dev(b), (n, 1), c, (n, 1))
    np.testing.assert_allclose(host(c), want, **tol)
    lib.gemm(code, m, n, k, dev(a), (k, 1), dev(b), (n, 1), c, (n, 1), alpha=-1.0, beta=1.0)   # c -= a.b
    np.testing.assert_allclose(host(c), np.zeros((m, n)), atol=1e-4)
    ct = torch.zeros((n, m), dtype=c.dtype, device="cuda")                  # transposed destination
    lib.gemm(code, m, n, k, dev(a), (k, 1), dev(b), (n, 1), ct, (1, m))
    np.testing.assert_allclose(host(ct).T, want, **tol)
    assert lib.last_gemm_kernel() == "simt"


@pytest.mark.parametrize("shape", [(128, 64, 64), (128, 256, 512), (200, 328, 136), (256, 4096, 1024), (1024, 1024, 2048)])
def test_tcgen05_fp32_product_matches_fp64_oracle(lib, shape):
    m, n, k = shape
    rng = np.random.default_rng(m + n + k)
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
    out = torch.full((m, n), -7.0, device="cuda")
    lib.gemm_fused(0, m, n, k, dev(a), k, dev(b), n, lib.compile(gemm_store_ir("f32")), [out])
    got = host(out)
    assert lib.gemm_error_flag() == 0
    assert lib.last_gemm_kernel().startswith("tcgen05.tf32x3")
    want = a.astype(np.float64) @ b.astype(np.float64)
    bound = np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64)
    assert np.all(np.abs(got - want) <= 1e-5 * bound), float(np.max(np.abs(got - want) / bound))
    if m * n * k <= 128 * 256 * 512:
        np.testing.assert_allclose(got, oracle.gemm(a, b), rtol=1e-5, atol=1e-5 * float(bound.max()))


def test_tcgen05_presplit_weights_and_accumulating_epilogue(lib):
    """x.Wx then += h.Wh with weights split once (the LSTM pattern)."""
    rng = np.random.default_rng(5)
    B, H = 64, 256
    x, h = (rng.standard_normal((B, H)).astype(np.float32) for _ in range(2))
    Wx, Wh = ((rng.standard_normal((H, 4 * H)) * 0.02).astype(np.float32) for _ in range(2))
    d = {k: dev(v) for k, v in dict(x=x, h=h, Wx=Wx, Wh=Wh).items()}
    parts = {}
    for name, rows, cols, tr in (("x", B, H, False), ("h", B, H, False), ("Wx", H, 4 * H, True), ("Wh", H, 4 * H, True)):
        hi, lo = torch.empty(rows * cols, device="cuda"), torch.empty(rows * cols, device="cuda")
        lib.gemm_split_tf32(d[name], rows, cols, cols, hi, lo, transpose=tr)
        parts[name] = (hi, lo)
    hi, lo = (host(t) for t in parts["Wx"])
    np.testing.assert_array_equal((hi + lo).reshape(4 * H, H), Wx.T)                    # the split is exact
    assert np.all((hi.view(np.uint32) & 0x1FFF) == 0)
    gates = torch.zeros((B, 4 * H), device="cuda")
    lib.gemm_fused(0, B, 4 * H, H, parts["x"][0], H, parts["Wx"][0], H, lib.compile(gemm_store_ir("f32")), [gates],
                   a_lo=parts["x"][1], b_lo=parts["Wx"][1])
    lib.gemm_fused(0, B, 4 * H, H, parts["h"][0], H, parts["Wh"][0], H, lib.compile(gemm_store_ir("f32", "add")), [gates],
                   a_lo=parts["h"][1], b_lo=parts["Wh"][1])
    got = host(gates)
    assert lib.gemm_error_flag() == 0
    want = x.astype(np.float64) @ Wx + h.astype(np.float64) @ Wh
    bound = np.abs(x).astype(np.float64) @ np.abs(Wx) + np.abs(h).astype(np.float64) @ np.abs(Wh)
    assert np.all(np.abs(got - want) <= 1e-5 * bound)


@pytest.mark.parametrize("shape", [(64, 1024, 256, 256), (200, 328, 136, 72), (256, 4096, 1024, 1024), (128, 128, 32, 480)])
def test_two_products_in_one_accumulator(lib, shape):
    """acc = x.Wx + h.Wh in one launch (different K per pair allowed), '+ b' as epilogue; against fp64 and
    against the two-launch form of the same sum."""
    m, n, k1, k2 = shape
    rng = np.random.default_rng(sum(shape))
    x, h = rng.standard_normal((m, k1)).astype(np.float32), rng.standard_normal((m, k2)).astype(np.float32)
    Wx, Wh = (rng.standard_normal((k1, n)) * 0.02).astype(np.float32), (rng.standard_normal((k2, n)) * 0.02).astype(np.float32)
    b = rng.standard_normal(n).astype(np.float32)
    e = IRBuilder(2, 0)
    o, bias = e.arg("f32"), e.arg("f32")
    e.st(o, e.op("add", e.acc(), e.ld(bias)))
    out = torch.full((m, n), -7.0, device="cuda")
    d = [dev(v) for v in (x, Wx, h, Wh)]
    lib.gemm_fused_sum(0, m, n, [(k1, d[0], k1, d[1], n), (k2, d[2], k2, d[3], n)], lib.compile(e.text()), [out, dev(b)],
                       strides=[None, [0, 1]])
    got = host(out)
    assert lib.gemm_error_flag() == 0
    assert lib.last_gemm_kernel().startswith("tcgen05.tf32x3") and lib.last_gemm_kernel().endswith("x2")
    want = x.astype(np.float64) @ Wx + h.astype(np.float64) @ Wh + b
    bound = np.abs(x).astype(np.float64) @ np.abs(Wx) + np.abs(h).astype(np.float64) @ np.abs(Wh) + np.abs(b)
    assert np.all(np.abs(got - want) <= 1e-5 * bound), float(np.max(np.abs(got - want) / bound))
    two = torch.zeros((m, n), device="cuda")
    lib.gemm_fused(0, m, n, k1, d[0], k1, d[1], n, lib.compile(gemm_store_ir("f32")), [two])
    e2 = IRBuilder(2, 0)
    o2, first, bias2 = e2.arg("f32"), e2.arg("f32"), e2.arg("f32")
    e2.st(o2, e2.op("add", e2.op("add", e2.acc(), e2.ld(first)), e2.ld(bias2)))
    lib.gemm_fused(0, m, n, k2, d[2], k2, d[3], n, lib.compile(e2.text()), [two, two, dev(b)], strides=[None, None, [0, 1]])
    np.testing.assert_allclose(got, host(two), rtol=1e-5, atol=1e-5 * float(bound.max()))


@pytest.mark.parametrize("ksplit", ["1", "0", "pairs"])
@pytest.mark.parametrize("shape", [(64, 128), (256, 1024), (200, 72), (130, 40), (384, 2048)])
def test_lstm_gating_as_the_epilogue_of_the_gate_products(lib, shape, ksplit, monkeypatch):
    """The four gate slices of x.Wx + h.Wh meet in the epilogue (acc 0..3): c' and h' come out of the GEMM
    kernel, the [B,4H] gates matrix is never written.  Against the oracle's gating on fp64-accumulated gates;
    ragged B and H (H not a multiple of the units a tile covers).  ksplit = 1: a cluster of two CTAs per tile, one
    operand pair each, partial sums exchanged through distributed shared memory; 0: one CTA accumulates both pairs."""
    # "pairs": the K split over cta_group::2 pairs (clusters of four CTAs on tiles of 256 rows), an opt-in variant
    pairs = ksplit == "pairs"
    if pairs:
        ksplit = "1"
        monkeypatch.setenv("DALI_B200_GEMM_KPAIR", "1")
    monkeypatch.setenv("DALI_B200_GEMM_KSPLIT", ksplit)
    B, H = shape
    rng = np.random.default_rng(B + H)
    x, h, c = (rng.standard_normal((B, H)).astype(np.float32) for _ in range(3))
    Wx, Wh = ((rng.standard_normal((H, 4 * H)) * 0.05).astype(np.float32) for _ in range(2))
    b = (rng.standard_normal(4 * H) * 0.1).astype(np.float32)
    c_new, h_new = torch.full((B, H), -7.0, device="cuda"), torch.full((B, H), -7.0, device="cuda")
    bd, d = dev(b), [dev(v) for v in (x, Wx, h, Wh)]
    row = [0, 1]
    lib.gemm_fused_sum(0, B, H, [(H, d[0], H, d[1], 4 * H), (H, d[2], H, d[3], 4 * H)], lib.compile(lstm_cell_epilogue_ir()),
                       [c_new, h_new, bd, bd, bd, bd, dev(c)], strides=[None, None, row, row, row, row, None],
                       offsets=[0, 0, 0, H, 2 * H, 3 * H, 0])
    got_c, got_h = host(c_new), host(h_new)
    assert lib.gemm_error_flag() == 0
    assert ".sl4" in lib.last_gemm_kernel() and lib.last_gemm_kernel().count(".ksplit") == int(ksplit)
    assert lib.last_gemm_kernel().count(".kpair") == int(pairs and B > 128)
    gates = (x.astype(np.float64) @ Wx + h.astype(np.float64) @ Wh + b).astype(np.float32)
    want_c, want_h = oracle.lstm_gating(gates, c)
    # the gates carry the product's error, bounded by 1e-5 * (|x|.|Wx| + |h|.|Wh|) (measured: 40 times smaller); the
    # gating has slope <= ~1.25 in every gate for |c| <= 5, so outputs are held to 2.5e-7 of that sum (1.3e-5 at
    # B=256, H=1024) -- far below what a misplaced slice or a lost partial sum would cause (O(0.1))
    bound = float((np.abs(x).astype(np.float64) @ np.abs(Wx) + np.abs(h).astype(np.float64) @ np.abs(Wh)).max())
    np.testing.assert_allclose(got_c, want_c, rtol=1e-5, atol=2.5e-7 * bound + 1e-6)
    np.testing.assert_allclose(got_h, want_h, rtol=1e-5, atol=2.5e-7 * bound + 1e-6)


def test_lstm_epilogue_leaves_the_next_hidden_state_split(lib):
    """lstm_cell_epilogue_ir(split_h=True): the epilogue also stores the two TF32 parts of h' (hi = the top 19 bits, lo = h' - hi,
    exact).  Two steps of a recurrence in which the second step's h operand is what the first one's epilogue left, against the
    oracle's gating of fp64 gate products."""
    B, H = 256, 1024
    rng = np.random.default_rng(5)
    xs = [rng.standard_normal((B, H)).astype(np.float32) for _ in range(2)]
    h, c = (rng.standard_normal((B, H)).astype(np.float32) for _ in range(2))
    Wx, Wh = ((rng.standard_normal((H, 4 * H)) * 0.02).astype(np.float32) for _ in range(2))
    b = (rng.standard_normal(4 * H) * 0.1).astype(np.float32)
    bd = dev(b)
    W = []
    for w in (Wx, Wh):
        hi, lo = torch.empty(4 * H * H, device="cuda"), torch.empty(4 * H * H, device="cuda")
        lib.gemm_split_tf32(dev(w), H, 4 * H, 4 * H, hi, lo, transpose=True)
        W.append((hi, lo))
    xp = [torch.empty(B * H, device="cuda") for _ in range(2)]
    hp = [[torch.empty(B * H, device="cuda") for _ in range(2)] for _ in range(2)]
    cs = [dev(c), torch.empty((B, H), device="cuda")]
    hs = [torch.empty((B, H), device="cuda") for _ in range(2)]
    lib.gemm_split_tf32(dev(h), B, H, H, *hp[0])
    prog = lib.compile(lstm_cell_epilogue_ir(split_h=True))
    row = [0, 1]
    for i in range(2):
        p, q = i % 2, 1 - i % 2
        lib.gemm_split_tf32(dev(xs[i]), B, H, H, *xp)
        lib.gemm_fused_sum(0, B, H, [(H, xp[0], H, W[0][0], H, xp[1], W[0][1]), (H, hp[p][0], H, W[1][0], H, hp[p][1], W[1][1])], prog,
                           [cs[q], hs[q], bd, bd, bd, bd, cs[p], hp[q][0], hp[q][1]],
                           strides=[None, None, row, row, row, row, None, None, None], offsets=[0, 0, 0, H, 2 * H, 3 * H, 0, 0, 0])
        assert lib.gemm_error_flag() == 0
        gates = (xs[i].astype(np.float64) @ Wx + h.astype(np.float64) @ Wh + b).astype(np.float32)
        c, h = oracle.lstm_gating(gates, c)
        np.testing.assert_allclose(host(cs[q]), c, rtol=1e-5, atol=1e-5 * (i + 1))
        np.testing.assert_allclose(host(hs[q]), h, rtol=1e-5, atol=1e-5 * (i + 1))
        hi, lo = host(hp[q][0]).reshape(B, H), host(hp[q][1]).reshape(B, H)
        np.testing.assert_array_equal(hi + lo, host(hs[q]))
        assert not np.any(hi.view(np.uint32) & 0x1fff)


def test_two_bf16_products_in_one_accumulator(lib):
    m, n, k1, k2 = 256, 512, 192, 320
    rng = np.random.default_rng(77)
    (x, xd), (h, hd) = to_bf16(rng.standard_normal((m, k1)).astype(np.float32)), to_bf16(rng.standard_normal((m, k2)).astype(np.float32))
    (Wx, Wxd), (Wh, Whd) = (to_bf16((rng.standard_normal((k, n)) * 0.05).astype(np.float32)) for k in (k1, k2))
    out = torch.zeros((m, n), device="cuda")
    lib.gemm_fused_sum(3, m, n, [(k1, xd, k1, Wxd, n), (k2, hd, k2, Whd, n)], lib.compile(gemm_store_ir("f32")), [out])
    got = host(out)
    assert lib.gemm_error_flag() == 0
    want = x.astype(np.float64) @ Wx + h.astype(np.float64) @ Wh
    bound = np.abs(x).astype(np.float64) @ np.abs(Wx) + np.abs(h).astype(np.float64) @ np.abs(Wh)
    assert np.all(np.abs(got - want) <= 1e-5 * bound)


@pytest.mark.parametrize("shape", [(128, 64, 64), (200, 328, 136), (512, 2048, 1024), (2048, 2048, 512)])
def test_tcgen05_bf16_product_and_fused_bias_tanh(lib, shape):
    m, n, k = shape
    rng = np.random.default_rng(k)
    a32, a16 = to_bf16((rng.standard_normal((m, k)) * 0.5).astype(np.float32))
    b32, b16 = to_bf16((rng.standard_normal((k, n)) * 0.5).astype(np.float32))
    bias = (rng.standard_normal(n) * 0.1).astype(np.float32)
    want = a32.astype(np.float64) @ b32.astype(np.float64)
    bound = np.abs(a32).astype(np.float64) @ np.abs(b32).astype(np.float64)
    out = torch.full((m, n), -7.0, device="cuda")
    lib.gemm_fused(3, m, n, k, a16, k, b16, n, lib.compile(gemm_store_ir("f32")), [out])
    got = host(out)
    assert lib.gemm_error_flag() == 0 and lib.last_gemm_kernel().startswith("tcgen05.bf16")
    assert np.all(np.abs(got - want) <= 1e-5 * bound)
    # config-4 epilogue: tanh(product + bias) stored as bf16; the reference's fp32 path on the same
    # bf16-rounded inputs is the yardstick, at bf16 output rounding (1e-2 relative allowed, 2^-8 measured)
    out16 = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    lib.gemm_fused(3, m, n, k, a16, k, b16, n, lib.compile(gemm_bias_tanh_ir("bf16")), [out16, dev(bias)],
                   strides=[None, [0, 1]])
    ref = oracle.bias_tanh(want.astype(np.float32), bias)
    np.testing.assert_allclose(host(out16), ref, rtol=1e-2, atol=4e-3)
    out32 = torch.zeros((m, n), device="cuda")
    lib.gemm_fused(3, m, n, k, a16, k, b16, n, lib.compile(gemm_bias_tanh_ir("f32")), [out32, dev(bias)],
                   strides=[None, [0, 1]])
    np.testing.assert_allclose(host(out32), ref, rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("shape", [(256, 256, 64), (200, 328, 136), (1024, 768, 1024), (2048, 2048, 512)])
def test_cta_pair_bf16_product(lib, shape, monkeypatch):
    """Two CTAs per 256 x 256 tile (tcgen05 cta_group::2), forced on for shapes the heuristic would leave to the
    single-CTA kernel, ragged edges included; same bound as the single-CTA path, and bit-identical to it where
    the accumulation order is the same (one K sweep per output)."""
    m, n, k = shape
    rng = np.random.default_rng(m * 3 + n * 5 + k)
    a, ad = to_bf16(rng.standard_normal((m, k)).astype(np.float32))
    b, bd = to_bf16((rng.standard_normal((k, n)) * 0.05).astype(np.float32))
    out = {}
    for mode in ("1", "0"):
        monkeypatch.setenv("DALI_B200_GEMM_PAIR", mode)
        o = torch.full((m, n), -7.0, device="cuda")
        lib.gemm_fused(3, m, n, k, ad, k, bd, n, lib.compile(gemm_store_ir("f32")), [o])
        out[mode] = host(o)
        assert lib.gemm_error_flag() == 0
        assert lib.last_gemm_kernel().endswith(".pair") == (mode == "1")
    want = a.astype(np.float64) @ b.astype(np.float64)
    bound = np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64)
    assert np.all(np.abs(out["1"] - want) <= 1e-5 * bound)
    np.testing.assert_array_equal(out["1"], out["0"])


def test_epilogue_with_strided_destination_scalars_and_residual(lib):
    """out[:, ::2] = relu(acc * s + residual): column-strided store, runtime scalar, second operand."""
    rng = np.random.default_rng(11)
    m, n, k = 256, 192, 128
    a32, a16 = to_bf16(rng.standard_normal((m, k)).astype(np.float32))
    b32, b16 = to_bf16(rng.standard_normal((k, n)).astype(np.float32))
    res = rng.standard_normal((m, n)).astype(np.float32)
    b = IRBuilder(2, 0)
    o, r = b.arg("f32"), b.arg("f32")
    s = b.scalar("f32")
    b.st(o, b.op("relu", b.op("add", b.op("eltmul", b.acc(), b.sc(s)), b.ld(r))))
    out = torch.full((m, 2 * n), -1.0, device="cuda")
    lib.gemm_fused(3, m, n, k, a16, k, b16, n, lib.compile(b.text()), [out, dev(res)], strides=[[2 * n, 2], None],
                   scalars=[np.float32(0.25)])
    got = host(out)
    assert lib.gemm_error_flag() == 0
    want = np.maximum((a32.astype(np.float64) @ b32) * 0.25 + res, 0)
    np.testing.assert_allclose(got[:, ::2], want, rtol=1e-5, atol=1e-4)
    assert np.all(got[:, 1::2] == -1.0)


@pytest.mark.parametrize("pair", ["1", "0"])
def test_full_size_product_whole_output(lib, pair, monkeypatch):
    """Config-4 size, CTA-pair and single-CTA kernels: the WHOLE [8192,8192] output against tanh(A . B + bias) computed in
    fp32 on the device (torch as the checker; a tile the persistent scheduler mis-assigned would show), and six probe rows
    against the fp64 product."""
    monkeypatch.setenv("DALI_B200_GEMM_PAIR", pair)
    n = 8192
    g = torch.Generator(device="cuda").manual_seed(1237)
    A = (torch.randn(n, n, device="cuda", generator=g) * 0.02).bfloat16()
    B = (torch.randn(n, n, device="cuda", generator=g) * 0.02).bfloat16()
    bias = torch.randn(n, device="cuda", generator=g) * 0.1
    out = torch.zeros((n, n), dtype=torch.bfloat16, device="cuda")
    lib.gemm_fused(3, n, n, n, A, n, B, n, lib.compile(gemm_bias_tanh_ir("bf16")), [out, bias], strides=[None, [0, 1]])
    torch.cuda.synchronize()
    assert lib.gemm_error_flag() == 0
    assert lib.last_gemm_kernel().endswith(".pair") == (pair == "1")
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        want_all = torch.tanh(A.float() @ B.float() + bias)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    assert bool(((out.float() - want_all).abs() <= 1e-2 * want_all.abs() + 4e-3).all())
    del want_all
    rows = [0, 1, 127, 128, 4095, 8191]
    a = A[rows].float().cpu().numpy().astype(np.float64)
    want = np.tanh(a @ B.float().cpu().numpy().astype(np.float64) + bias.cpu().numpy())
    np.testing.assert_allclose(out[rows].float().cpu().numpy(), want, rtol=1e-2, atol=4e-3)


def test_unsupported_layouts_are_refused_not_faked(lib):
    from dali_b200 import DaliB200Error
    x = torch.zeros(64 * 64 + 1, device="cuda")
    with pytest.raises(DaliB200Error) as e:     # base pointer 4 bytes off a 16-byte boundary
        lib.gemm_fused(0, 64, 64, 64, x[1:], 64, x, 64, lib.compile(gemm_store_ir("f32")), [x])
    assert e.value.status == -6
    with pytest.raises(DaliB200Error):          # epilogue program without 'acc'
        b = IRBuilder(2, 0)
        o, i = b.arg("f32"), b.arg("f32")
        b.st(o, b.ld(i))
        lib.gemm_fused(0, 64, 64, 64, x, 64, x, 64, lib.compile(b.text()), [x, x])
