"""CPU-side checks of the C-ABI library: it loads, exports every symbol the
header declares, parses / rejects IR, picks the expected kernel skeleton for
a layout and gets every generated kernel through NVRTC for sm_100a (no GPU
needed for any of it)."""
import os
import re

import numpy as np
import pytest

import dali_b200
from dali_b200 import DaliB200Error
from dali_b200.ir import IRBuilder, chain_sum_ir, lstm_gating_ir, reduce_ir, softmax_ir

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L(tmp_path_factory):
    lib = dali_b200.load_library()
    lib.cache_set_dir(str(tmp_path_factory.mktemp("dali_cache")))
    return lib


def test_library_exports_every_declared_symbol(L):
    names = set()
    for fn in os.listdir(os.path.join(ROOT, "include")):
        text = open(os.path.join(ROOT, "include", fn)).read()
        names |= set(re.findall(r"\b(dalib200_[a-z0-9_]+)\s*\(", text))
    assert len(names) >= 20
    for n in sorted(names):
        assert hasattr(L.c, n), "symbol %s declared in include/ but not exported" % n
    assert L.abi_version() == 1


def test_no_device_is_an_error_not_a_fallback(L):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(DaliB200Error) as e:
        L.init(0)
    assert e.value.status == -2
    h = L.compile(softmax_ir())
    with pytest.raises(DaliB200Error) as e:
        L.launch(h, (4, 4), [4096, 8192])
    assert e.value.status == -2


def test_ir_validation(L):
    bad = [
        "",                                                   # empty
        "dali-ir 2\nspace 1 0\nend\n",                        # version
        "dali-ir 1\nspace 1 0\narg 0 f32 E\nend\n",           # stores nothing
        "dali-ir 1\nspace 1 0\narg 0 f32 E\nv0 f32 ld 0\nv1 f32 red sum v0\nst 0 assign v1\nend\n",   # red without nreduce
        "dali-ir 1\nspace 1 0\narg 0 f32 E\narg 1 i32 E\nv0 i32 ld 1\nst 0 assign v0\nend\n",         # type mismatch
        "dali-ir 1\nspace 2 1\narg 0 f32 R\narg 1 f32 E\nv0 f32 ld 1\nst 0 assign v0\nend\n",         # E value into R arg
        "dali-ir 1\nspace 1 0\narg 0 f32 E\nv0 f32 ld 0\nv2 f32 op exp v0\nst 0 assign v2\nend\n",    # sparse numbering
        "dali-ir 1\nspace 9 0\narg 0 f32 E\nv0 f32 ld 0\nst 0 assign v0\nend\n",                      # rank
    ]
    for text in bad:
        with pytest.raises(DaliB200Error):
            L.compile(text)
    h = L.compile(softmax_ir())
    assert L.is_loaded(h) and not L.is_loaded(h + 1)
    assert L.compile(softmax_ir(), h) == h                    # same text: no-op
    with pytest.raises(DaliB200Error):                        # other text under the same hash
        L.compile(chain_sum_ir(), h)


def variant_of(L, ir, space, n, strides=None, pointers=None, offsets=None):
    h = L.compile(ir)
    size = L.precompile(h, space, n, strides=strides, pointers=pointers, offsets=offsets)
    assert size > 1000
    return L.last_variant()


def test_skeleton_choice_and_nvrtc(L):
    v = variant_of(L, softmax_ir(), (4096, 1024), 2)
    assert v.startswith("row.") and ".v4." in v and ".T64.p4." in v            # two warps per row, row kept in registers
    assert variant_of(L, softmax_ir(), (33, 1001), 2).startswith("row.o1.i1.v1.")
    assert ".p0." in variant_of(L, softmax_ir(), (3, 40000), 2)                # streaming fallback
    assert variant_of(L, softmax_ir(), (300, 7), 2).startswith("row.")
    # misaligned base pointer -> scalar path
    assert ".v1." in variant_of(L, softmax_ir(), (64, 64), 2, pointers=[4096, 4100])
    v = variant_of(L, chain_sum_ir(), (1 << 31,), 2)
    assert v.startswith("all.") and ".v4." in v and "C=2147483648" in v
    for kind, arg in (("sum", False), ("max", False), ("max", True), ("min", True), ("prod", False)):
        assert variant_of(L, reduce_ir(kind, "f32", 2, 1, arg), (8192, 8192), 2).startswith("row.")
        v = variant_of(L, reduce_ir(kind, "f32", 2, 1, arg), (8192, 8192), 2, strides=[None, [1, 8192]])
        assert v.startswith("col.") and ".v4." in v
        assert variant_of(L, reduce_ir(kind, "f32", 2, 2, arg), (8192, 8192), 2).startswith("all.")
        assert variant_of(L, reduce_ir(kind, "i32", 2, 1, arg), (257, 129), 2, strides=[None, [1, 257]]).startswith("col.")
        assert variant_of(L, reduce_ir(kind, "f64", 2, 1, arg), (64, 64), 2).startswith("row.")
    # non-collapsible inner dims: strided all-reduce keeps two inner dims
    v = variant_of(L, reduce_ir("sum", "f32", 2, 2), (5, 5), 2, strides=[None, [10, 3]])
    assert v.startswith("all.o0.i2.")
    v = variant_of(L, reduce_ir("sum", "i32", 3, 1), (6, 4, 5), 2, strides=[None, [20, 1, 4]])
    assert v.startswith("row.o2.i1.") or v.startswith("col.")
    gs = [4096, 1]
    v = variant_of(L, lstm_gating_ir(), (256, 1024), 7, strides=[None, None, gs, gs, gs, gs, None],
                   offsets=[0, 0, 0, 1024, 2048, 3072, 0])
    assert v.startswith("map.o1.i1.v4.")


def test_every_functor_compiles_for_every_dtype(L):
    from test_oracle import FUNCTOR
    import sys
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    from make_golden import BINARY, UNARY
    for dt in ("f32", "f64", "i32"):
        b = IRBuilder(1, 0)
        o, i, j = b.arg(dt), b.arg(dt), b.arg(dt)
        acc = b.ld(i)
        other = b.ld(j)
        for n in list(UNARY) + ["negate", "safe_entropy_log", "negative_log"]:
            acc = b.op("add", acc, b.op(FUNCTOR.get(n, n), other))
        for n in list(BINARY) + ["fill", "div_grad", "threshold"]:
            acc = b.op("add", acc, b.op(FUNCTOR.get(n, n), other, acc))
        if dt != "i32":
            acc = b.op("add", acc, b.cast(dt, b.op("round", other, dtype="i32")))
            acc = b.op("add", acc, b.cast(dt, b.op("ceiling", other, dtype="i32")))
        b.st(o, acc)
        assert variant_of(L, b.text(), (1000,), 3).startswith("map.")


def test_disk_cache_and_recompile_counters(L, tmp_path):
    L.cache_set_dir(str(tmp_path))
    ir = reduce_ir("sum", "f32", 2, 1) + "# cache test\n"
    h = L.compile(ir)
    before = L.cache_stats()
    L.precompile(h, (128, 128), 2)
    mid = L.cache_stats()
    assert mid["compilations"] == before["compilations"] + 1
    files = os.listdir(str(tmp_path))
    assert any(f.endswith(".cubin") for f in files) and any(f.endswith(".cu") for f in files)
    L.precompile(h, (128, 128), 2)                       # memory hit
    assert L.cache_stats()["compilations"] == mid["compilations"]
    L.cache_clear(False)                                  # drop memory, keep files
    L.precompile(h, (128, 128), 2)
    after = L.cache_stats()
    assert after["compilations"] == mid["compilations"] and after["disk_hits"] == mid["disk_hits"] + 1
    # a truncated image on disk is rebuilt, not loaded
    cub = [f for f in os.listdir(str(tmp_path)) if f.endswith(".cubin")][0]
    with open(os.path.join(str(tmp_path), cub), "wb") as f:
        f.write(b"\x7fELF")
    L.cache_clear(False)
    L.precompile(h, (128, 128), 2)
    assert L.cache_stats()["compilations"] == after["compilations"] + 1


def test_transposed_operands_pick_a_tiled_map_variant(L):
    """A read-only operand whose unit stride runs along the outer dim: 4 x 4 register blocks when everything is
    16-byte aligned, shared-memory tiles when the extents are ragged, the plain strided kernel for thin shapes.
    Planning compiles the variant with NVRTC, so this also checks that each one builds."""
    from dali_b200.ir import IRBuilder
    e = IRBuilder(2, 0)
    O, A, B = e.arg("f32"), e.arg("f32"), e.arg("f32")
    e.st(O, e.op("add", e.op("tanh", e.ld(A)), e.ld(B)))
    ir = e.text()
    assert ".tile4" in variant_of(L, ir, (1024, 512), 3, strides=[None, [1, 1024], None])
    assert ".tile32" in variant_of(L, ir, (100, 257), 3, strides=[None, [1, 100], None])
    assert ".tile32" in variant_of(L, ir, (1024, 512), 3, strides=[None, [1, 1024], None], pointers=[4096, 8196, 12288])
    assert ".tile" not in variant_of(L, ir, (5, 4000), 3, strides=[None, [1, 5], None])
    e = IRBuilder(2, 0)
    O, A = e.arg("f64"), e.arg("f64")
    e.st(O, e.ld(A))
    assert ".tile32" in variant_of(L, e.text(), (64, 64), 2, strides=[None, [1, 64]])


def test_all_axis_grid_follows_the_work_per_cta(L):
    """The all-axis skeleton runs in whole waves of 148 x 8 CTAs, about 8 chunks of 4096 elements to a CTA, at most 16
    waves; full chunks skip their bounds checks (.nc) only where a CTA runs 16 or more of them."""
    import re

    def grid(v):
        return int(re.search(r"grid=(\d+)x1", v).group(1))
    v = variant_of(L, chain_sum_ir(), (1 << 20,), 2)
    assert grid(v) == 256 and ".nc" not in v                  # 256 chunks: one CTA each, far less than a wave
    v = variant_of(L, reduce_ir("sum", "f32", 2, 2), (8192, 8192), 2)
    assert grid(v) == 2 * 1184 and ".nc" not in v             # 2^26 elements: two waves
    v = variant_of(L, chain_sum_ir(), (1 << 28,), 2)
    assert grid(v) == 7 * 1184 and ".nc" not in v
    v = variant_of(L, chain_sum_ir(), (1 << 31,), 2)
    assert grid(v) == 16 * 1184 and v.split(" ")[0].endswith(".nc")


def test_pair_programs_read_the_extreme_off_the_arg_reduction(L, tmp_path):
    """arg_pair_ir (max and argmax of one operand): in the column and all-axis skeletons the element loop accumulates the
    arg-reduction only; the max is copied from its running pair after the loop."""
    from dali_b200.ir import arg_pair_ir
    old_dir = L.cache_get_dir()
    L.cache_set_dir(str(tmp_path))
    try:
        N = 1024
        h = L.compile(arg_pair_ir("max", "f32", 2, 1) + "# pair test\n")
        L.precompile(h, (N, N), 3, strides=[None, None, [1, N]])
        assert L.last_variant().startswith("col.")
        src = "".join(open(str(p)).read() for p in tmp_path.glob("*.cu"))
        body = src[src.index("dali_kernel"):]
        assert re.search(r"acc\d+\[j\] = acc\d+\[j\]\.v;", body)
        assert "RMax::apply(acc" not in body.split("fold")[0].split("__syncthreads")[0]
    finally:
        L.cache_set_dir(old_dir)
