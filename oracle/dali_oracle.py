"""TEST INFRASTRUCTURE ONLY: numpy-facing wrapper of oracle/dali_oracle.c.

Imported by tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs,
never by the dali_b200 package.  Builds libdali_oracle.so with gcc on first use.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libdali_oracle.so")
_lib = None

_DT = {np.dtype(np.float32): 0, np.dtype(np.float64): 1, np.dtype(np.int32): 2}
_SUF = {0: "f32", 1: "f64", 2: "i32"}
_KIND = {"sum": 0, "prod": 1, "max": 2, "min": 3}


def build():
    src = os.path.join(_HERE, "dali_oracle.c")
    if not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "libdali_oracle.so"], stdout=subprocess.DEVNULL)
    return _SO


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
    return _lib


def _p(a):
    return ctypes.c_void_p(a.ctypes.data)


def _i64(v):
    return ctypes.c_int64(int(v))


def unary(name, x):
    x = np.ascontiguousarray(x)
    y = np.empty_like(x)
    rc = lib().oracle_unary(name.encode(), _DT[x.dtype], _p(x), _p(y), _i64(x.size))
    if rc != 0:
        raise KeyError(name)
    return y


def binary(name, a, b):
    """b may be a 0-d / 1-element array (scalar operand) or have a's shape."""
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b, dtype=a.dtype)
    stride = 0 if b.size == 1 else 1
    if stride:
        assert b.shape == a.shape
    y = np.empty_like(a)
    rc = lib().oracle_binary(name.encode(), _DT[a.dtype], _p(a), _p(b), _i64(stride), _p(y), _i64(a.size))
    if rc != 0:
        raise KeyError(name)
    return y


def round_to_int(x):
    x = np.ascontiguousarray(x)
    y = np.empty(x.shape, np.int32)
    fn = lib().oracle_round_f32_i32 if x.dtype == np.float32 else lib().oracle_round_f64_i32
    fn(_p(x), _p(y), _i64(x.size))
    return y


def _as_rows(x, axis):
    """View of x as [rows, cols] (element strides) with `axis` (or all) reduced."""
    x = np.ascontiguousarray(x)
    if axis is None:
        return x, 1, x.size, x.size, 1, ()
    axis = axis % x.ndim
    moved = np.ascontiguousarray(np.moveaxis(x, axis, -1))
    cols = moved.shape[-1]
    rows = moved.size // cols
    return moved, rows, cols, cols, 1, moved.shape[:-1]


def reduce(kind, x, axis=None):
    """Sequential left-to-right fold in x's own dtype (the reference's CPU loop)."""
    m, rows, cols, rs, cs, oshape = _as_rows(x, axis)
    out = np.empty(rows, m.dtype)
    fn = getattr(lib(), "oracle_reduce_" + _SUF[_DT[m.dtype]])
    fn(_KIND[kind], _p(m), _i64(rows), _i64(cols), _i64(rs), _i64(cs), _p(out))
    return out.reshape(oshape)


def argreduce(kind, x, axis=None):
    m, rows, cols, rs, cs, oshape = _as_rows(x, axis)
    out = np.empty(rows, np.int32)
    fn = getattr(lib(), "oracle_argreduce_" + _SUF[_DT[m.dtype]])
    fn(_KIND[kind], _p(m), _i64(rows), _i64(cols), _i64(rs), _i64(cs), _p(out))
    return out.reshape(oshape)


def sum_f64acc(x, axis=None):
    """(double-accumulated sum, sum of |x|) of a float32 array along axis."""
    m, rows, cols, rs, cs, oshape = _as_rows(x.astype(np.float32, copy=False), axis)
    out = np.empty(rows, np.float64)
    out_abs = np.empty(rows, np.float64)
    lib().oracle_sum_f64acc_f32(_p(m), _i64(rows), _i64(cols), _i64(rs), _i64(cs), _p(out), _p(out_abs))
    return out.reshape(oshape), out_abs.reshape(oshape)


def softmax(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    cols = a.shape[-1]
    out = np.empty_like(a)
    lib().oracle_softmax_f32(_p(a), _i64(a.size // cols), _i64(cols), _p(out))
    return out


def gather(src, idx):
    src = np.ascontiguousarray(src)
    idx = np.ascontiguousarray(idx, dtype=np.int32)
    row_len = int(np.prod(src.shape[1:], dtype=np.int64))
    out = np.empty(idx.shape + src.shape[1:], src.dtype)
    lib().oracle_gather(_p(src), _p(idx), _i64(idx.size), _i64(row_len), src.itemsize, _p(out))
    return out


def gather_from_rows(src, idx):
    src = np.ascontiguousarray(src)
    idx = np.ascontiguousarray(idx, dtype=np.int32)
    inner = int(np.prod(src.shape[2:], dtype=np.int64))
    out = np.empty((src.shape[0],) + src.shape[2:], src.dtype)
    lib().oracle_gather_from_rows(_p(src), _p(idx), _i64(src.shape[0]), _i64(src.shape[1]), _i64(inner),
                                  src.itemsize, _p(out))
    return out


def scatter_add(dest, idx, upd):
    dest = np.array(dest, copy=True, order="C")
    idx = np.ascontiguousarray(idx, dtype=np.int32)
    upd = np.ascontiguousarray(np.broadcast_to(upd, idx.shape + dest.shape[1:]), dtype=dest.dtype)
    row_len = int(np.prod(dest.shape[1:], dtype=np.int64))
    fn = lib().oracle_scatter_add_f32 if dest.dtype == np.float32 else lib().oracle_scatter_add_i32
    fn(_p(dest), _p(idx), _p(upd), _i64(idx.size), _i64(row_len))
    return dest


def gemm(a, b):
    """Row-major a @ b with a double accumulator (float32) or exact (int32)."""
    if a.dtype == np.int32:
        a = np.ascontiguousarray(a)
        b = np.ascontiguousarray(b)
        c = np.empty((a.shape[0], b.shape[1]), np.int32)
        lib().oracle_gemm_i32(_p(a), _p(b), _p(c), _i64(a.shape[0]), _i64(b.shape[1]), _i64(a.shape[1]))
        return c
    a = np.asarray(a, dtype=np.float32)
    b = np.asarray(b, dtype=np.float32)
    c = np.empty((a.shape[0], b.shape[1]), np.float32)
    es = a.itemsize
    lib().oracle_gemm_f32(_p(a), _i64(a.strides[0] // es), _i64(a.strides[1] // es), _p(b), _i64(b.strides[0] // es),
                          _i64(b.strides[1] // es), _p(c), _i64(a.shape[0]), _i64(b.shape[1]), _i64(a.shape[1]))
    return c


def lstm_gating(gates, c):
    gates = np.ascontiguousarray(gates, dtype=np.float32)
    c = np.ascontiguousarray(c, dtype=np.float32)
    B, H = c.shape
    cn = np.empty_like(c)
    hn = np.empty_like(c)
    lib().oracle_lstm_gating_f32(_p(gates), _p(c), _i64(B), _i64(H), _p(cn), _p(hn))
    return cn, hn


def lstm_cell(x, h, c, Wx, Wh, b):
    gates = gemm(x, Wx) + gemm(h, Wh)          # float32 adds, as the reference's fused add kernel
    gates = (gates + np.asarray(b, np.float32).reshape(1, -1)).astype(np.float32)
    return lstm_gating(gates, c)


def chain_sum(x, w, b):
    """(reference-order fp32 sum, double-accumulated sum, sum |y|) of sigmoid(x*w+b)*exp(-x*x)."""
    x = np.ascontiguousarray(x, dtype=np.float32).ravel()
    s32 = ctypes.c_float()
    s64 = ctypes.c_double()
    sabs = ctypes.c_double()
    lib().oracle_chain_sum_f32(_p(x), _i64(x.size), ctypes.c_float(w), ctypes.c_float(b), ctypes.byref(s32),
                               ctypes.byref(s64), ctypes.byref(sabs))
    return s32.value, s64.value, sabs.value


def bias_tanh(x, bias):
    x = np.ascontiguousarray(x, dtype=np.float32)
    bias = np.ascontiguousarray(bias, dtype=np.float32)
    out = np.empty_like(x)
    lib().oracle_bias_tanh_f32(_p(x), _p(bias), _i64(x.shape[0]), _i64(x.shape[1]), _p(out))
    return out


_SCAN_OPS = {"sum": 0, "prod": 1, "max": 2, "min": 3}


def scan(kind, x, inclusive=True):
    """Running reduction over the last axis, in the reference's left-to-right order (op/scan.cpp:47-77)."""
    x = np.ascontiguousarray(x)
    cols = x.shape[-1]
    rows = x.size // cols if cols else 0
    out = np.empty(x.shape[:-1] + (cols + (0 if inclusive else 1),), x.dtype)
    rc = lib().oracle_scan(_SCAN_OPS[kind], _DT[x.dtype], int(bool(inclusive)), _i64(rows), _i64(cols), _p(x), _p(out))
    if rc != 0:
        raise KeyError((kind, x.dtype))
    return out


def one_hot(indices, depth, on_value, off_value, dtype=np.float64):
    """out[..., d] = on * (idx == d) + (1 - (idx == d)) * off in on_value's type (op/one_hot.cpp:41-46)."""
    idx = np.ascontiguousarray(indices, dtype=np.int32)
    out = np.empty(idx.shape + (depth,), dtype)
    rc = lib().oracle_one_hot(_p(idx), _i64(idx.size), int(depth), _DT[np.dtype(dtype)], ctypes.c_double(on_value),
                              ctypes.c_double(off_value), _p(out))
    if rc != 0:
        raise KeyError(dtype)
    return out


def diag(d, rows, cols):
    """value[i, j] = i == j ? d[j] : 0 with d a scalar or a vector (op/eye.cpp:33-38)."""
    scalar = np.ndim(d) == 0
    d = np.ascontiguousarray(d)          # a scalar becomes shape (1,)
    out = np.empty((rows, cols), d.dtype)
    rc = lib().oracle_diag(_DT[d.dtype], _p(d), _i64(0 if scalar else d.shape[0]), _i64(rows), _i64(cols), _p(out))
    if rc != 0:
        raise KeyError(d.dtype)
    return out


def arange(start, stop, step, dtype=np.int32):
    """start + i * step for i < size, in start's type (op/arange.cpp:41).  size = (int)ceil((stop - start) / step)
    evaluated in the operands' common type (arange.cpp:63): for three ints the division TRUNCATES, so
    arange(10, -5, -4) has 3 elements and arange(0, 10, 3) has 3, one fewer than numpy's."""
    if all(isinstance(v, (int, np.integer)) for v in (start, stop, step)):
        n = int((int(stop) - int(start)) / int(step))          # C integer division truncates toward zero
    else:
        n = int(np.ceil((float(stop) - float(start)) / float(step)))
    t = np.dtype(dtype).type
    return (t(start) + np.arange(n).astype(dtype) * t(step)).astype(dtype)


def outer(a, b):
    """left[i] * right[j] over the ravelled operands (op/outer.cpp:21, :43-47)."""
    a, b = np.ravel(a), np.ravel(b)
    t = np.result_type(a.dtype, b.dtype)
    return a.astype(t)[:, None] * b.astype(t)[None, :]


# ---- counter-based random numbers ------------------------------------------------------
# The reference draws from std::mt19937 on the CPU and from thrust's generators on the GPU
# (dali/array/op/random.cu.cpp:59-88, 153-232): its two streams differ from each other, so no
# stream of its own can be pinned.  The B200 back end uses Philox4x32-10 (Salmon, Moraes, Dror,
# Shaw: "Parallel random numbers: as easy as 1, 2, 3", SC'11) with counter = (element index, 0,
# 0, 0) and key = (seed, 0); this is its plain restatement.
_PHILOX_M0, _PHILOX_M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
_PHILOX_W0, _PHILOX_W1 = 0x9E3779B9, 0xBB67AE85


def philox4x32_10(counter, key):
    """counter: 4 arrays (or ints) of uint32 words, key: 2 words -> 4 uint32 arrays."""
    c = [np.asarray(w, dtype=np.uint64) & np.uint64(0xFFFFFFFF) for w in counter]
    k0, k1 = int(key[0]) & 0xFFFFFFFF, int(key[1]) & 0xFFFFFFFF
    mask = np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0 = _PHILOX_M0 * c[0]
        p1 = _PHILOX_M1 * c[2]
        hi0, lo0 = p0 >> np.uint64(32), p0 & mask
        hi1, lo1 = p1 >> np.uint64(32), p1 & mask
        c = [hi1 ^ c[1] ^ np.uint64(k0), lo1, hi0 ^ c[3] ^ np.uint64(k1), lo0]
        k0 = (k0 + _PHILOX_W0) & 0xFFFFFFFF
        k1 = (k1 + _PHILOX_W1) & 0xFFFFFFFF
    return [w.astype(np.uint32) for w in c]


def _philox_words(n, seed, per_element):
    """The words element i < n reads: fp32 uniforms take one word (block i >> 2, word i & 3), fp64 uniforms and fp32
    normals two (block i >> 1, words 2 (i & 1), 2 (i & 1) + 1), fp64 normals the whole block i."""
    i = np.arange(n, dtype=np.uint64)
    shift = {1: 2, 2: 1, 4: 0}[per_element]
    x = philox4x32_10((i >> np.uint64(shift), 0, 0, 0), (seed, 0))
    words = np.stack(x, axis=1)                                   # [n, 4]
    first = ((i & np.uint64((1 << shift) - 1)) * np.uint64(per_element)).astype(np.int64)
    return [words[np.arange(n), first + k] for k in range(per_element)]


def rng_uniform(n, seed, dtype=np.float32):
    """u[i] in [0, 1) for element index i < n."""
    if np.dtype(dtype) == np.float32:
        (w,) = _philox_words(n, seed, 1)
        return ((w >> np.uint32(8)).astype(np.float32) * np.float32(1.0 / 16777216.0)).astype(np.float32)
    w0, w1 = _philox_words(n, seed, 2)
    hi, lo = (w0 >> np.uint32(5)).astype(np.float64), (w1 >> np.uint32(6)).astype(np.float64)
    return (hi * 67108864.0 + lo) * (1.0 / 9007199254740992.0)


def rng_normal(n, seed, dtype=np.float32):
    """Box-Muller on two uniforms of the same Philox block: sqrt(-2 ln u1) cos(2 pi u2), u1 in (0, 1]."""
    if np.dtype(dtype) == np.float32:
        w0, w1 = _philox_words(n, seed, 2)
        u1 = ((w0 >> np.uint32(8)).astype(np.float64) + 1.0) / 16777216.0
        u2 = (w1 >> np.uint32(8)).astype(np.float64) / 16777216.0
    else:
        x = _philox_words(n, seed, 4)
        u1 = ((x[0] >> np.uint32(5)).astype(np.float64) * 67108864.0 + (x[1] >> np.uint32(6)).astype(np.float64) + 1.0) / 9007199254740992.0
        u2 = ((x[2] >> np.uint32(5)).astype(np.float64) * 67108864.0 + (x[3] >> np.uint32(6)).astype(np.float64)) / 9007199254740992.0
    return (np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)).astype(dtype)
