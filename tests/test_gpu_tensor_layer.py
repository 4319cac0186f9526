"""The caller of the hot path: the reference's own autodiff layer (class Tensor, graph::backward,
tensor_ops) built UNCHANGED from the reference checkout against this back end's Array headers
(oracle/tensor_layer/build_tensor_layer.sh -> oracle/_ref/), driven by tests/cpp/tensor_layer_smoke.cpp:
analytic gradients from the reference's tape against central finite differences in double precision
(tolerances per case in the program, the reference's own: 1e-5 .. 1e-2), an LSTM cell forward and backward
at [256, 1024], a least-squares fit by gradient descent, the reference's six solvers, .npy round trip.

The binaries are made where the reference checkout is present; a machine without them skips."""
import json
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "oracle", "_ref", "tensor_layer_smoke")


def test_reference_tensor_layer_runs_on_this_back_end(tmp_path):
    if not os.path.exists(EXE):
        pytest.skip("oracle/_ref/tensor_layer_smoke was not built (needs the reference checkout at build time)")
    r = subprocess.run([EXE, str(tmp_path)], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-4000:] + r.stderr[-2000:]
    summary = json.loads(r.stdout.strip().splitlines()[-1])
    assert summary["failures"] == 0 and summary["checks"] >= 100
