"""dalib200_sum_f32_noalloc: the all-axis sum for callers that cannot allocate
device memory at call time (a latency-critical host thread that must not take
allocator locks, an embedding under a memory budget fixed at load time).  Its exchange space is a fixed array in
the library image instead of the growable arena of dalib200_launch.

Checked through the C ABI against the regular entry point (the generated
all-axis reduction kernel) on the same device data, twice in a row -- the
second call runs on whatever the first left in the shared array.  Tolerance as
for every floating sum here: |a - b| <= 1e-5 * sum|x| (the two kernels fold in
different orders)."""
import ctypes

import numpy as np
import pytest
import torch

from dali_b200.ir import reduce_ir

pytestmark = pytest.mark.gpu


def noalloc_sum(lib, x, out, n=None):
    fn = lib.c.dalib200_sum_f32_noalloc
    fn.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]
    return fn(0, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), ctypes.c_void_p(x.data_ptr()),
              x.numel() if n is None else n, ctypes.c_void_p(out.data_ptr()))


@pytest.mark.parametrize("n", [1, 1000, 4097, (1 << 22) + 5, 1 << 26])
def test_matches_the_regular_all_axis_sum_twice_in_a_row(lib, n):
    torch.manual_seed(n)
    h = lib.compile(reduce_ir("sum", "f32", 1, 1))
    for call in range(2):
        x = torch.rand(n, device="cuda") * 2 - 1 + call
        want = torch.zeros(1, device="cuda")
        got = torch.full((1,), -123.0, device="cuda")
        lib.launch(h, (n,), [want, x], stream=torch.cuda.current_stream().cuda_stream)
        assert noalloc_sum(lib, x, got) == 0, lib.last_error()
        torch.cuda.synchronize()
        bound = 1e-5 * float(x.abs().sum(dtype=torch.float64))
        assert abs(float(got) - float(want)) <= bound, (call, float(got), float(want))
        assert abs(float(got) - float(x.sum(dtype=torch.float64))) <= bound


def test_exact_on_integer_valued_input_and_unaligned_pointer(lib):
    x = torch.randint(-3, 4, (1 << 20,), device="cuda").float()
    out = torch.zeros(1, device="cuda")
    for view in (x, x[1:], x[3:1000]):          # x[1:] starts 4 bytes off a 16-byte boundary
        assert noalloc_sum(lib, view, out) == 0, lib.last_error()
        torch.cuda.synchronize()
        assert float(out) == float(view.sum(dtype=torch.float64))


def test_rejects_sizes_beyond_the_fixed_maximum(lib):
    x = torch.zeros(16, device="cuda")
    out = torch.zeros(1, device="cuda")
    rc = noalloc_sum(lib, x, out, n=(1 << 31) + 1)      # size check happens before anything is read
    assert rc == -7
    assert "exceed the fixed maximum" in lib.last_error()
    assert noalloc_sum(lib, x, out, n=-1) == -1
