"""Generates tests/golden/reference_cpu.npz by running the REFERENCE's own CPU
path (oracle/_ref/ref_driver, built by oracle/build_ref.sh from the reference
checkout) on small seeded inputs.  Run in a container that has the reference
checkout; the fixture it writes is committed so that the oracle can be pinned
where the checkout is absent.

    python tests/golden/make_golden.py
"""
import os
import subprocess
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
DRIVER = os.path.join(ROOT, "oracle", "_ref", "ref_driver")
CACHE = os.path.join(ROOT, "oracle", "_ref", "cache")
OUT = os.path.join(ROOT, "tests", "golden", "reference_cpu.npz")

UNARY = {  # name in the reference's op:: namespace -> input domain
    "identity": "any", "sqrt": "pos", "square": "any", "abs": "any", "sigmoid": "any", "dsigmoid": "unit",
    "tanh": "any", "dtanh": "unit", "relu": "any", "relu_backward": "any", "eltinv": "pos", "exp": "any",
    "log": "pos", "log_or_zero": "any", "sign": "any", "softplus": "wide", "softplus_backward": "wide",
    "cube": "any", "rsqrt": "pos", "isnan": "any", "isinf": "any", "inverse_tanh": "unit",
}
BINARY = {
    "add": "any", "subtract": "any", "eltmul": "any", "eltdiv": "pos", "equals": "ints", "pow": "pos",
    "steep_sigmoid": "any", "steep_sigmoid_backward": "any", "clipped_relu": "pos2", "clipped_relu_backward": "pos2",
    "prelu": "any", "prelu_backward_weights": "any", "prelu_backward_inputs": "any", "lessthanequal": "ints",
    "greaterthanequal": "ints", "maximum": "any", "minimum": "any", "clip": "pos2",
    "binary_cross_entropy": "prob", "binary_cross_entropy_grad": "prob",
}


def domain(rng, kind, shape, second=False):
    if kind == "any":
        return rng.standard_normal(shape).astype(np.float32)
    if kind == "pos":
        return (rng.random(shape) * 3 + 0.1).astype(np.float32)
    if kind == "pos2":
        return (rng.random(shape) * 2 + 0.05).astype(np.float32) if second else (rng.standard_normal(shape) * 2).astype(np.float32)
    if kind == "unit":
        return (rng.random(shape) * 1.8 - 0.9).astype(np.float32)
    if kind == "wide":
        return (rng.standard_normal(shape) * 12).astype(np.float32)
    if kind == "ints":
        return rng.integers(-2, 3, shape).astype(np.float32)
    if kind == "prob":
        return (rng.random(shape) * 0.9 + 0.05).astype(np.float32)
    raise KeyError(kind)


def run(case, inputs, n_out=1, extra=()):
    """inputs: list of arrays or strings (verbatim args, in order); returns output arrays."""
    with tempfile.TemporaryDirectory() as tmp:
        args = []
        k = 0
        for x in inputs:
            if isinstance(x, np.ndarray):
                path = os.path.join(tmp, "in%d.npy" % k)
                np.save(path, x)
                args.append(path)
                k += 1
            else:
                args.append(str(x))
        outs = [os.path.join(tmp, "out%d.npy" % i) for i in range(n_out)]
        cmd = [DRIVER, CACHE, case] + args + outs + [str(e) for e in extra]
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
        if r.returncode != 0:
            raise RuntimeError("ref_driver failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout, r.stderr))
        return [np.load(o) for o in outs]


def main():
    if not os.path.exists(DRIVER):
        sys.exit("oracle/_ref/ref_driver is missing: run `make -C oracle ref` where the reference checkout exists")
    rng = np.random.default_rng(20240607)
    g = {}
    shape = (3, 17)
    for name, dom in UNARY.items():
        x = domain(rng, dom, shape)
        if name in ("isnan", "isinf"):
            x[0, 1] = np.nan
            x[1, 2] = np.inf
            x[2, 3] = -np.inf
        g["unary/%s/x" % name] = x
        g["unary/%s/y" % name] = run("unary", [name, x])[0]
    for name, dom in BINARY.items():
        a = domain(rng, dom, shape)
        b = domain(rng, dom, shape, second=True)
        g["binary/%s/a" % name] = a
        g["binary/%s/b" % name] = b
        g["binary/%s/y" % name] = run("binary", [name, a, b])[0]
    # int32 and float64 instantiations of a few functors
    xi = rng.integers(-4, 5, shape).astype(np.int32)
    for name in ("square", "abs", "relu", "sign", "cube", "tanh", "sigmoid"):
        g["unary_i32/%s/x" % name] = xi
        g["unary_i32/%s/y" % name] = run("unary", [name, xi])[0]
    xd = rng.standard_normal(shape)
    for name in ("exp", "tanh", "sigmoid", "softplus", "square"):
        g["unary_f64/%s/x" % name] = xd
        g["unary_f64/%s/y" % name] = run("unary", [name, xd])[0]
    # reductions
    x = (rng.random((13, 37)) * 2 - 1).astype(np.float32)
    x[4, 9] = x[4, 20] = 0.99999   # ties: first occurrence must win
    x[:, 5] = x[2, 5]
    g["reduce/x"] = x
    for opn in ("sum", "prod", "max", "min", "mean", "l2", "argmax", "argmin"):
        for ax in ("-1", "0", "all"):
            g["reduce/%s/%s" % (opn, ax)] = run("reduce", [opn, ax, x])[0]
    xi = rng.integers(-50, 50, (6, 5, 4)).astype(np.int32)
    g["reduce_i32/x"] = xi
    for opn in ("sum", "max", "min"):
        for ax in ("-1", "0", "1", "all"):
            g["reduce_i32/%s/%s" % (opn, ax)] = run("reduce", [opn, ax, xi])[0]
    # argmax/argmin along an axis are pinned on rank-2 input only: on rank-3 input the
    # reference's ArgumentAxisReduce node is copied during rank collapse, loses its type
    # (it has no copy() override) and returns the extreme VALUE instead of its index
    xi2 = rng.integers(-50, 50, (7, 11)).astype(np.int32)
    g["reduce_i32_2d/x"] = xi2
    for opn in ("argmax", "argmin"):
        for ax in ("-1", "0"):
            g["reduce_i32_2d/%s/%s" % (opn, ax)] = run("reduce", [opn, ax, xi2])[0]
    # softmax: library composition and the spelled-out expression, incl. the reference test's range
    a = (rng.random((7, 33)) * 40 - 20).astype(np.float32)
    g["softmax/a"] = a
    g["softmax/op"] = run("softmax", [a])[0]
    g["softmax/naive"] = run("softmax_naive", [a])[0]
    a2 = rng.standard_normal((5, 64)).astype(np.float32)
    g["softmax2/a"] = a2
    g["softmax2/naive"] = run("softmax_naive", [a2])[0]
    # gather / gather_from_rows / scatter
    src = rng.standard_normal((9, 6, 3)).astype(np.float32)
    idx = rng.integers(0, 9, (5,)).astype(np.int32)
    g["gather/src"] = src
    g["gather/idx"] = idx
    g["gather/out"] = run("gather", [src, idx])[0]
    # (rank-2 index arrays make the reference's JIT throw "min computation rank lower than
    # its ndim", so only rank-1 indices can be pinned against it)
    src2d = np.ascontiguousarray(src[:, :, 0])
    g["gather/src2d"] = src2d
    g["gather/out2d"] = run("gather", [src2d, idx])[0]
    rows_idx = rng.integers(0, 6, (9,)).astype(np.int32)
    g["gather_rows/idx"] = rows_idx
    g["gather_rows/out"] = run("gather_rows", [src, rows_idx])[0]
    dest = np.zeros((3,), np.int32)
    sidx = np.array([0, 0, 1, 1, 1, 2], np.int32)
    g["scatter/idx"] = sidx
    g["scatter/out"] = run("scatter_add", [dest, sidx])[0]
    # dot, gemm + epilogue, LSTM cell, chain
    A = (rng.standard_normal((12, 20)) * 0.5).astype(np.float32)
    B = (rng.standard_normal((20, 16)) * 0.5).astype(np.float32)
    bias = (rng.standard_normal((16,)) * 0.1).astype(np.float32)
    g["dot/A"], g["dot/B"], g["dot/bias"] = A, B, bias
    g["dot/out"] = run("dot", [A, B])[0]
    g["dot/gemm_tanh"] = run("gemm_tanh", [A, B, bias])[0]
    Bn, H = 6, 8
    xs = rng.standard_normal((Bn, H)).astype(np.float32)
    hs = rng.standard_normal((Bn, H)).astype(np.float32)
    cs = rng.standard_normal((Bn, H)).astype(np.float32)
    Wx = (rng.standard_normal((H, 4 * H)) * 0.3).astype(np.float32)
    Wh = (rng.standard_normal((H, 4 * H)) * 0.3).astype(np.float32)
    b = (rng.standard_normal((4 * H,)) * 0.1).astype(np.float32)
    g["lstm/x"], g["lstm/h"], g["lstm/c"], g["lstm/Wx"], g["lstm/Wh"], g["lstm/b"] = xs, hs, cs, Wx, Wh, b
    cn, hn = run("lstm", [xs, hs, cs, Wx, Wh, b.reshape(1, -1)], n_out=2)
    g["lstm/c_new"], g["lstm/h_new"] = cn, hn
    xc = rng.standard_normal((4099,)).astype(np.float32)
    g["chain/x"] = xc
    g["chain/sum"] = run("chain", [xc, "0.5", "0.1"])[0]
    # ---- arange / diag / one_hot / outer / running reductions (appended: earlier draws are unchanged)
    g["arange/i32_2_17_3"] = run("arange", ["i32", 2, 17, 3])[0]
    g["arange/i32_24"] = run("arange", ["i32", 0, 24, 1])[0]
    g["arange/i32_neg"] = run("arange", ["i32", 10, -5, -4])[0]
    # (a float arange does not compile in the reference: op::ceil names a functor, "ceiling", that
    # dali/array/functor.h does not define; and diag of a vector throws "cast a non-jit expression
    # (Buffer) into a JITNode": only the scalar diagonal can be pinned against it)
    g["diag/f64_5_4x5"] = run("diag_scalar", ["f64", 5.0, 4, 5])[0]
    g["diag/f32_1_6x3"] = run("diag_scalar", ["f32", 1.0, 6, 3])[0]
    g["diag/i32_7_3x3"] = run("diag_scalar", ["i32", 7, 3, 3])[0]
    oh_idx = rng.integers(0, 7, (2, 3)).astype(np.int32)
    g["one_hot/idx"] = oh_idx
    g["one_hot/out"] = run("one_hot", [oh_idx, 7, 112.2, 42.0])[0]
    oa = rng.standard_normal((5,)).astype(np.float32)
    ob = rng.standard_normal((2, 4)).astype(np.float32)
    g["outer/a"], g["outer/b"] = oa, ob
    g["outer/out"] = run("outer", [oa, ob])[0]
    si = rng.integers(-9, 10, (4, 23)).astype(np.int32)
    sf = (rng.random((3, 41)) + 0.5).astype(np.float32)
    g["scan/i32"], g["scan/f32"] = si, sf
    for kind in ("sum", "prod"):
        for inc in (1, 0):
            g["scan/i32/%s/%d" % (kind, inc)] = run("scan", [kind, inc, si])[0]
            g["scan/f32/%s/%d" % (kind, inc)] = run("scan", [kind, inc, sf])[0]
    g["scan/1d/sum/0"] = run("scan", ["sum", 0, np.arange(20, dtype=np.int32)])[0]
    np.savez_compressed(OUT, **g)
    print("wrote %s: %d arrays, %d bytes" % (OUT, len(g), os.path.getsize(OUT)))


if __name__ == "__main__":
    main()
