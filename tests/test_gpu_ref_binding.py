"""The reference-side binding (oracle/ref_binding/): the reference's OWN expression graph -- its Array / op:: front end, its
canonical() and jit_merge, compiled from its sources into oracle/_ref/libdali_ref_bound.so with the binding spliced into
jit.cpp and cpu_gemm.cpp -- evaluated by libdali_b200.so on the GPU, against the same cases evaluated by the unmodified
reference on the CPU (oracle/_ref/ref_driver).  Each case must have gone through the binding with nothing left to the
reference's own JIT."""
import os
import re
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref")
PLAIN, BOUND, CACHE = os.path.join(REF, "ref_driver"), os.path.join(REF, "ref_driver_bound"), os.path.join(REF, "cache")

needs_drivers = pytest.mark.skipif(not (os.path.exists(PLAIN) and os.path.exists(BOUND)),
                                   reason="oracle/_ref/ref_driver(_bound) not built (no reference checkout at build time)")


def run(driver, case, tmp, env=None):
    e = dict(os.environ)
    e.update(env or {})
    r = subprocess.run([driver, CACHE] + case, cwd=tmp, capture_output=True, text=True, env=e, timeout=900)
    assert r.returncode == 0, r.stdout + r.stderr
    m = re.search(r"BINDING launched=(\d+) fell_back=(\d+) gemms=(\d+)", r.stdout)
    return tuple(int(g) for g in m.groups()) if m else None, r.stderr


def inputs(tmp):
    rng = np.random.default_rng(99)
    np.save(os.path.join(tmp, "a.npy"), rng.standard_normal((192, 320)).astype(np.float32))
    np.save(os.path.join(tmp, "u.npy"), (rng.random((96, 200)) * 2 - 1).astype(np.float32))
    np.save(os.path.join(tmp, "x.npy"), rng.standard_normal(1 << 16).astype(np.float32))
    np.save(os.path.join(tmp, "b.npy"), (rng.standard_normal((320, 64)) * 0.1).astype(np.float32))
    np.save(os.path.join(tmp, "src.npy"), rng.standard_normal((500, 48)).astype(np.float32))
    np.save(os.path.join(tmp, "idx.npy"), rng.integers(0, 500, (300,)).astype(np.int32))
    np.save(os.path.join(tmp, "idxr.npy"), rng.integers(0, 48, (500,)).astype(np.int32))
    np.save(os.path.join(tmp, "v.npy"), rng.standard_normal(130).astype(np.float32))
    np.save(os.path.join(tmp, "w.npy"), rng.standard_normal(70).astype(np.float32))


CASES = [(["softmax_naive", "a.npy"], "close"), (["softmax", "a.npy"], "close"), (["chain", "x.npy", "0.5", "0.1"], "close"),
         (["unary", "tanh", "a.npy"], "close"), (["unary", "sigmoid", "a.npy"], "close"), (["binary", "eltmul", "a.npy", "a.npy"], "close"),
         (["dot", "a.npy", "b.npy"], "close"), (["gather", "src.npy", "idx.npy"], "exact"),
         (["gather_rows", "src.npy", "idxr.npy"], "exact"), (["outer", "v.npy", "w.npy"], "exact"),
         (["one_hot", "idx.npy", "500", "2.5", "-0.5"], "exact")]
for _op in ("sum", "max", "argmax", "min", "argmin", "mean", "l2"):
    for _ax in ("-1", "0", "all"):
        CASES.append((["reduce", _op, _ax, "u.npy"], "exact" if _op in ("max", "min", "argmax", "argmin") else "close"))


@needs_drivers
@pytest.mark.gpu
@pytest.mark.parametrize("case,how", CASES, ids=[" ".join(c[:3]) for c, _ in CASES])
def test_reference_graph_runs_on_the_gpu_through_the_binding(case, how, tmp_path):
    tmp = str(tmp_path)
    inputs(tmp)
    _, _ = run(PLAIN, case + ["want.npy"], tmp)
    stats, err = run(BOUND, case + ["got.npy"], tmp, {"DALI_B200_BINDING_VERBOSE": "1"})
    launched, fell_back, gemms = stats
    assert fell_back == 0, err
    assert (gemms == 1) if case[0] == "dot" else (launched >= 1), err
    want, got = np.load(os.path.join(tmp, "want.npy")), np.load(os.path.join(tmp, "got.npy"))
    assert want.shape == got.shape and want.dtype == got.dtype
    if how == "exact":
        np.testing.assert_array_equal(got, want)
    elif case[0] == "dot":
        a, b = np.load(os.path.join(tmp, "a.npy")), np.load(os.path.join(tmp, "b.npy"))
        bound = np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64)
        assert np.all(np.abs(got.astype(np.float64) - a.astype(np.float64) @ b.astype(np.float64)) <= 1e-5 * bound)
        assert np.all(np.abs(got.astype(np.float64) - want) <= 2e-5 * bound)
    else:
        # sums carry the rounding of two different summation orders: 1e-5 of the sum of magnitudes that went into an output
        atol = 1e-6
        if case[0] == "chain":
            atol += 1e-5 * float(np.abs(want).sum())
        elif case[0] == "reduce":
            u = np.abs(np.load(os.path.join(tmp, "u.npy"))).astype(np.float64)
            mags = u.sum() if case[2] == "all" else u.sum(axis=int(case[2])).max()
            atol += 1e-5 * float(mags if case[1] != "l2" else np.sqrt((u * u).sum()))
        np.testing.assert_allclose(got, want, rtol=1e-5, atol=atol)


@needs_drivers
def test_binding_translates_the_reference_graph_without_a_gpu(tmp_path):
    """DALI_B200_BINDING_DRYRUN: every JITRunner of the case is translated to dali-ir and accepted by dalib200_compile (parse +
    validation); the computation itself then runs on the reference's CPU path."""
    tmp = str(tmp_path)
    inputs(tmp)
    for case, _ in CASES:
        if case[0] == "dot":
            continue
        stats, err = run(BOUND, case + ["out.npy"], tmp, {"DALI_B200_BINDING_DRYRUN": "1", "DALI_B200_BINDING_VERBOSE": "1"})
        assert stats is not None and stats[0] >= 1, (case, err)
        assert "left to the reference" not in err and "program refused" not in err, (case, err)


@needs_drivers
@pytest.mark.gpu
def test_reference_lstm_cell_and_gemm_epilogue_through_the_binding(tmp_path):
    """Benchmark configurations 2 and 4 as the reference's driver writes them (fp32): the products go to dalib200_gemm, the
    gating / bias + tanh expressions over (sliced views of) the product to generated kernels."""
    tmp = str(tmp_path)
    rng = np.random.default_rng(7)
    B, H = 64, 128
    for k in ("x", "h", "c"):
        np.save(os.path.join(tmp, k + ".npy"), rng.standard_normal((B, H)).astype(np.float32))
    for k in ("Wx", "Wh"):
        np.save(os.path.join(tmp, k + ".npy"), (rng.standard_normal((H, 4 * H)) * 0.05).astype(np.float32))
    np.save(os.path.join(tmp, "b.npy"), (rng.standard_normal((1, 4 * H)) * 0.1).astype(np.float32))
    np.save(os.path.join(tmp, "bias.npy"), (rng.standard_normal(4 * H) * 0.1).astype(np.float32))
    files = ["x.npy", "h.npy", "c.npy", "Wx.npy", "Wh.npy", "b.npy"]
    run(PLAIN, ["lstm"] + files + ["c_want.npy", "h_want.npy"], tmp)
    stats, err = run(BOUND, ["lstm"] + files + ["c_got.npy", "h_got.npy"], tmp, {"DALI_B200_BINDING_VERBOSE": "1"})
    assert stats[1] == 0 and stats[2] >= 2 and stats[0] >= 1, err
    for k in ("c", "h"):
        np.testing.assert_allclose(np.load(os.path.join(tmp, k + "_got.npy")), np.load(os.path.join(tmp, k + "_want.npy")), rtol=1e-5, atol=2e-5)
    run(PLAIN, ["gemm_tanh", "x.npy", "Wx.npy", "bias.npy", "want.npy"], tmp)
    stats, err = run(BOUND, ["gemm_tanh", "x.npy", "Wx.npy", "bias.npy", "got.npy"], tmp, {"DALI_B200_BINDING_VERBOSE": "1"})
    assert stats[1] == 0 and stats[2] == 1 and stats[0] >= 1, err
    np.testing.assert_allclose(np.load(os.path.join(tmp, "got.npy")), np.load(os.path.join(tmp, "want.npy")), rtol=1e-5, atol=2e-5)
