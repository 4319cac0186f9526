"""Python face of the C++ Array / op:: front end (include/dali_b200_array.h).

Harness only: every object here is a handle to a C++ `Array`; expressions are
built, fused, compiled, cached and run inside libdali_b200.so exactly as for a
C++ caller.  Lets tests and benchmarks be written the way the reference's own
tests are:

    from dali_b200.array import Array, op
    a = Array(np_a)
    s = op.exp(a - op.max(a, [-1], True)) / op.sum(exped, [-1], True)
    s.numpy()
"""
import ctypes

import numpy as np

from .capi import load_library

DTYPE_FLOAT, DTYPE_DOUBLE, DTYPE_INT32, DTYPE_BF16 = 0, 1, 2, 3
_NP2D = {np.dtype(np.float32): 0, np.dtype(np.float64): 1, np.dtype(np.int32): 2}
_D2NP = {0: np.float32, 1: np.float64, 2: np.int32, 3: np.uint16}      # bf16 travels as its 16-bit patterns (numpy has no bf16)


def to_bf16_bits(x):
    """float32 array -> uint16 bf16 bit patterns, round to nearest even (NaN stays NaN)."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return np.where(np.isnan(x), np.uint16(0x7FC0), r).astype(np.uint16)


def from_bf16_bits(b):
    """uint16 bf16 bit patterns -> the float32 values they stand for."""
    return (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)
_H = ctypes.c_void_p
_lib = None


def _c():
    global _lib
    if _lib is None:
        L = load_library()
        c = L.c
        c.dali_array_expression_name.restype = ctypes.c_size_t
        c.dali_lazy_last_ir.restype = ctypes.c_size_t
        c.dali_lazy_last_variant.restype = ctypes.c_size_t
        c.dali_array_free.argtypes = [_H]
        c.dali_array_ndim.argtypes = [_H]
        c.dali_array_dtype.argtypes = [_H]
        c.dali_array_is_buffer.argtypes = [_H]
        c.dali_array_scalar.argtypes = [ctypes.c_double, ctypes.c_int, ctypes.POINTER(_H)]
        c.dali_array_set_shard.argtypes = [_H, ctypes.c_int, ctypes.c_int64, ctypes.c_int64]
        c.dali_array_get_shard.argtypes = [_H, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_int64)]
        c.dali_lazy_collectives.restype = ctypes.c_size_t
        c.dali_lazy_collectives.argtypes = [ctypes.POINTER(ctypes.c_int64), ctypes.c_char_p, ctypes.c_size_t]
        _lib = L
    return _lib


def _check(rc):
    _c().check(rc)


def _shape_arg(shape):
    return (ctypes.c_int64 * max(len(shape), 1))(*[int(s) for s in shape])


class Array:
    """Handle to a lazy C++ Array."""
    __array_priority__ = 1000

    def __init__(self, value=None, dtype=None, _handle=None):
        self._h = None
        if _handle is not None:
            self._h = _handle
            return
        L = _c()
        h = _H()
        if isinstance(value, Array):
            raise TypeError("copy an Array with op.identity(a)")
        if np.isscalar(value):
            if dtype is None:
                dtype = DTYPE_INT32 if isinstance(value, (int, np.integer)) else DTYPE_DOUBLE if isinstance(value, float) else DTYPE_FLOAT
            _check(L.c.dali_array_scalar(float(value), int(dtype), ctypes.byref(h)))
        else:
            if dtype == DTYPE_BF16 and np.asarray(value).dtype != np.uint16:
                value = to_bf16_bits(np.asarray(value, np.float32))           # floats are rounded to bf16
            arr = np.ascontiguousarray(value, dtype=_D2NP[dtype] if dtype is not None else None)
            if arr.dtype not in _NP2D and dtype != DTYPE_BF16:
                arr = arr.astype(np.float32 if arr.dtype.kind == "f" else np.int32)
            code = DTYPE_BF16 if dtype == DTYPE_BF16 else _NP2D[arr.dtype]
            _check(L.c.dali_array_from_host(ctypes.c_void_p(arr.ctypes.data), _shape_arg(arr.shape), arr.ndim,
                                            code, ctypes.byref(h)))
        self._h = h

    def __del__(self):
        if self._h is not None and _lib is not None:
            _lib.c.dali_array_free(self._h)
            self._h = None

    # ---- construction -----------------------------------------------------------------
    @staticmethod
    def _new(fn, *args):
        h = _H()
        _check(fn(*args, ctypes.byref(h)))
        return Array(_handle=h)

    @staticmethod
    def zeros(shape, dtype=DTYPE_FLOAT):
        return Array._new(_c().c.dali_array_zeros, _shape_arg(shape), len(shape), int(dtype))

    @staticmethod
    def empty(shape, dtype=DTYPE_FLOAT):
        return Array._new(_c().c.dali_array_empty, _shape_arg(shape), len(shape), int(dtype))

    @staticmethod
    def ones(shape, dtype=DTYPE_FLOAT):
        out = Array.empty(shape, dtype)
        out.assign(Array(1, dtype))
        return out

    @staticmethod
    def borrow(array, dtype=None):
        """Wraps a C-contiguous numpy array WITHOUT copying it (page-locked memory then reaches the GPU by DMA);
        the caller keeps it alive and unchanged until the expressions reading it have been evaluated.
        dtype=DTYPE_BF16: a uint16 array of bf16 bit patterns."""
        bf16 = dtype == DTYPE_BF16 and isinstance(array, np.ndarray) and array.dtype == np.uint16
        if not (isinstance(array, np.ndarray) and array.flags.c_contiguous and (array.dtype in _NP2D or bf16)):
            raise TypeError("Array.borrow needs a C-contiguous float32 / float64 / int32 (or, as bf16, uint16) numpy array")
        out = Array._new(_c().c.dali_array_borrow_host, ctypes.c_void_p(array.ctypes.data), _shape_arg(array.shape),
                         array.ndim, DTYPE_BF16 if bf16 else _NP2D[array.dtype])
        out._keep = array
        return out

    @staticmethod
    def load(path):
        """Array::load: a .npy file (float32 / float64 / int32, C or Fortran order)."""
        return Array._new(_c().c.dali_array_load, str(path).encode())

    def save(self, path):
        """Array::save: evaluates and writes a C-ordered .npy file."""
        _check(_c().c.dali_array_save(str(path).encode(), self._h))

    @staticmethod
    def from_device(ptr, shape, dtype=DTYPE_FLOAT, gpu=0):
        """Wraps device memory owned by the caller (e.g. a torch CUDA tensor's data_ptr())."""
        return Array._new(_c().c.dali_array_from_device, ctypes.c_void_p(int(ptr)), _shape_arg(shape), len(shape),
                          int(dtype), int(gpu))

    # ---- sharding over the ranks of the communicator (dali_b200.comm) ---------------------------------------
    @staticmethod
    def scatter_rows(array):
        """Keeps this rank's rows of a (global) numpy array and marks them as a shard along axis 0."""
        arr = np.ascontiguousarray(array)
        if arr.dtype not in _NP2D:
            arr = arr.astype(np.float32 if arr.dtype.kind == "f" else np.int32)
        return Array._new(_c().c.dali_array_scatter_rows, ctypes.c_void_p(arr.ctypes.data), _shape_arg(arr.shape), arr.ndim,
                          _NP2D[arr.dtype])

    def set_shard(self, axis, lo, total):
        """Declares this array to be indices [lo, lo + extent) of `total` along `axis` of a logical array spread over the ranks."""
        _check(_c().c.dali_array_set_shard(self._h, int(axis), ctypes.c_int64(lo), ctypes.c_int64(total)))
        return self

    @property
    def shard(self):
        """(axis, lo, total); axis < 0: not sharded."""
        axis, lo, total = ctypes.c_int(-1), ctypes.c_int64(0), ctypes.c_int64(0)
        _check(_c().c.dali_array_get_shard(self._h, ctypes.byref(axis), ctypes.byref(lo), ctypes.byref(total)))
        return axis.value, lo.value, total.value

    # ---- inspection ---------------------------------------------------------------------
    @property
    def ndim(self):
        return _c().c.dali_array_ndim(self._h)

    @property
    def dtype(self):
        return _c().c.dali_array_dtype(self._h)

    @property
    def shape(self):
        n = self.ndim
        s = (ctypes.c_int64 * max(n, 1))()
        _check(_c().c.dali_array_shape(self._h, s))
        return tuple(int(s[i]) for i in range(n))

    def is_buffer(self):
        return bool(_c().c.dali_array_is_buffer(self._h))

    def expression_name(self):
        buf = ctypes.create_string_buffer(1 << 16)
        _c().c.dali_array_expression_name(self._h, buf, len(buf))
        return buf.value.decode()

    # ---- evaluation ---------------------------------------------------------------------
    def eval(self, wait=True):
        _check(_c().c.dali_array_eval(self._h, int(wait)))
        return self

    def numpy(self, out=None):
        """Evaluates and returns the value as a numpy array (written into `out` when given)."""
        if out is None:
            out = np.empty(self.shape, _D2NP[self.dtype])
        elif not (out.flags.c_contiguous and out.shape == self.shape and out.dtype == _D2NP[self.dtype]):
            raise TypeError("numpy(out=...): out must be C-contiguous with the Array's shape and dtype")
        _check(_c().c.dali_array_to_host(self._h, ctypes.c_void_p(out.ctypes.data), out.nbytes))
        return out

    def item(self):
        v = ctypes.c_double()
        _check(_c().c.dali_array_item(self._h, ctypes.byref(v)))
        return v.value

    def __float__(self):
        return self.item()

    def __int__(self):
        return int(self.item())

    def device_ptr(self, gpu=0):
        p = ctypes.c_void_p()
        _check(_c().c.dali_array_device_ptr(self._h, gpu, ctypes.byref(p)))
        return p.value

    # ---- views --------------------------------------------------------------------------
    def pluck_axis(self, axis, idx):
        c = _c().c
        if isinstance(idx, slice):
            n = self.shape[axis]
            start, stop, step = idx.indices(n)
            if step < 0:   # python [hi:lo:-s] -> Slice(lo + 1, hi + 1, -s), which walks that range backwards
                start, stop = stop + 1, start + 1
            return Array._new(c.dali_array_slice, self._h, axis, start, stop, step)
        return Array._new(c.dali_array_index, self._h, axis, int(idx))

    def __getitem__(self, key):
        if isinstance(key, Array):
            return op.gather(self, key)
        if not isinstance(key, tuple):
            key = (key,)
        out, axis = self, 0
        for k in key:
            if k is None:
                out = out.expand_dims(axis)
                axis += 1
            elif isinstance(k, slice):
                if k != slice(None):
                    out = out.pluck_axis(axis, k)
                axis += 1
            else:
                out = out.pluck_axis(axis, k)
        return out

    def expand_dims(self, axis):
        return Array._new(_c().c.dali_array_expand_dims, self._h, axis)

    def squeeze(self, axis):
        return Array._new(_c().c.dali_array_squeeze, self._h, axis)

    def transpose(self, axes=None):
        axes = list(axes or [])
        arr = (ctypes.c_int * max(len(axes), 1))(*axes)
        return Array._new(_c().c.dali_array_transpose, self._h, arr, len(axes))

    @property
    def T(self):
        return self.transpose()

    def broadcast_to_shape(self, shape):
        return Array._new(_c().c.dali_array_broadcast_to, self._h, _shape_arg(shape), len(shape))

    def reshape(self, shape):
        return Array._new(_c().c.dali_array_reshape, self._h, _shape_arg(shape), len(shape))

    def astype(self, dtype):
        return Array._new(_c().c.dali_array_astype, self._h, int(dtype))

    # ---- assignment -----------------------------------------------------------------------
    def assign(self, other):
        return self._inplace(0, other)

    def _inplace(self, code, other):
        value = _wrap(other)          # keep the temporary alive across the call
        _check(_c().c.dali_array_assign(self._h, code, value._h))
        return self

    def __iadd__(self, o): return self._inplace(1, o)
    def __isub__(self, o): return self._inplace(2, o)
    def __imul__(self, o): return self._inplace(3, o)
    def __itruediv__(self, o): return self._inplace(4, o)
    def __ilshift__(self, o): return self._inplace(5, o)

    # ---- arithmetic ------------------------------------------------------------------------
    def __add__(self, o): return op.add(self, o)
    def __radd__(self, o): return op.add(o, self)
    def __sub__(self, o): return op.subtract(self, o)
    def __rsub__(self, o): return op.subtract(o, self)
    def __mul__(self, o): return op.eltmul(self, o)
    def __rmul__(self, o): return op.eltmul(o, self)
    def __truediv__(self, o): return op.eltdiv(self, o)
    def __rtruediv__(self, o): return op.eltdiv(o, self)
    def __neg__(self): return op._unary("negate", self)

    def sum(self, axes=None, keepdims=False): return op.sum(self, axes, keepdims)
    def max(self, axes=None, keepdims=False): return op.max(self, axes, keepdims)
    def min(self, axes=None, keepdims=False): return op.min(self, axes, keepdims)
    def mean(self, axes=None, keepdims=False): return op.mean(self, axes, keepdims)
    def exp(self): return op.exp(self)
    def dot(self, o): return op.dot(self, o)
    def gather_from_rows(self, idx): return op.gather_from_rows(self, idx)


def _wrap(x):
    if isinstance(x, Array):
        return x
    if isinstance(x, (np.floating,)):
        return Array(float(x), DTYPE_FLOAT if x.dtype == np.float32 else DTYPE_DOUBLE)
    if np.isscalar(x):
        return Array(x)
    return Array(np.asarray(x))


class _Op:
    """namespace op:: of the reference (dali/array/op.h)."""

    def _unary(self, name, a):
        a = _wrap(a)
        return Array._new(_c().c.dali_op_unary, name.encode(), a._h)

    def _binary(self, name, a, b):
        a, b = _wrap(a), _wrap(b)
        return Array._new(_c().c.dali_op_binary, name.encode(), a._h, b._h)

    def _reduce(self, name, a, axes, keepdims):
        if axes is None:
            return Array._new(_c().c.dali_op_reduce, name.encode(), a._h, None, -1, int(keepdims))
        axes = [int(x) for x in axes]
        arr = (ctypes.c_int * max(len(axes), 1))(*axes)
        return Array._new(_c().c.dali_op_reduce, name.encode(), a._h, arr, len(axes), int(keepdims))

    def sum(self, a, axes=None, keepdims=False): return self._reduce("sum", a, axes, keepdims)
    def prod(self, a, axes=None, keepdims=False): return self._reduce("prod", a, axes, keepdims)
    def max(self, a, axes=None, keepdims=False): return self._reduce("max", a, axes, keepdims)
    def min(self, a, axes=None, keepdims=False): return self._reduce("min", a, axes, keepdims)
    def mean(self, a, axes=None, keepdims=False): return self._reduce("mean", a, axes, keepdims)
    def L2_norm(self, a, axes=None, keepdims=False): return self._reduce("L2_norm", a, axes, keepdims)

    def argmax(self, a, axis=None):
        return Array._new(_c().c.dali_op_argreduce, b"argmax", a._h, int(axis or 0), int(axis is None))

    def argmin(self, a, axis=None):
        return Array._new(_c().c.dali_op_argreduce, b"argmin", a._h, int(axis or 0), int(axis is None))

    def gather(self, source, indices):
        indices = _wrap(indices)
        return Array._new(_c().c.dali_op_gather, source._h, indices._h)

    def gather_from_rows(self, source, indices):
        indices = _wrap(indices)
        return Array._new(_c().c.dali_op_gather_from_rows, source._h, indices._h)

    def softmax(self, logits, axis=-1):
        return Array._new(_c().c.dali_op_softmax, logits._h, int(axis))

    def dot(self, a, b):
        return Array._new(_c().c.dali_op_dot, a._h, b._h)

    def arange(self, start, stop=None, step=1):
        """Lazy: ints give an int32 index expression, anything else op::arange(Array, Array, Array)."""
        if stop is None:
            start, stop = 0, start
        if all(isinstance(v, (int, np.integer)) for v in (start, stop, step)):
            return Array._new(_c().c.dali_array_arange, int(start), int(stop), int(step))
        a, b, c = _wrap(start), _wrap(stop), _wrap(step)
        return Array._new(_c().c.dali_op_arange, a._h, b._h, c._h)

    def diag(self, d, rows=None, cols=None):
        d = _wrap(d)
        if rows is None:
            rows = d.shape[0]
        return Array._new(_c().c.dali_op_diag, d._h, int(rows), int(rows if cols is None else cols))

    def eye(self, rows, cols=None):
        return self.diag(Array(1.0, DTYPE_FLOAT), rows, cols)

    def one_hot(self, indices, depth, on_value, off_value):
        on, off = _wrap(on_value), _wrap(off_value)
        return Array._new(_c().c.dali_op_one_hot, indices._h, int(depth), on._h, off._h)

    def outer(self, a, b):
        return Array._new(_c().c.dali_op_outer, a._h, b._h)

    def concatenate(self, arrays, axis=0):
        arrays = [_wrap(a) for a in arrays]
        hs = (_H * len(arrays))(*[a._h.value for a in arrays])
        return Array._new(_c().c.dali_op_concatenate, hs, len(arrays), int(axis))

    def hstack(self, arrays):
        return self.concatenate(arrays, -1)

    def vstack(self, arrays):
        return self.concatenate(arrays, 0)

    def _random(self, kind, a, b, shape):
        a, b = _wrap(a), _wrap(b)
        return Array._new(_c().c.dali_op_random, kind.encode(), a._h, b._h, _shape_arg(shape), len(shape))

    def uniform(self, low, high, shape):
        return self._random("uniform", low, high, shape)

    def normal(self, loc, scale, shape):
        return self._random("normal", loc, scale, shape)

    def bernoulli(self, prob, shape):
        return self._random("bernoulli", prob, prob, shape)

    def bernoulli_normalized(self, prob, shape):
        return self._random("bernoulli_normalized", prob, prob, shape)

    def axis_scan(self, a, reducer, inclusive=True):
        return Array._new(_c().c.dali_op_scan, a._h, reducer.encode(), int(bool(inclusive)))

    def cumsum(self, a, inclusive=True):
        return self.axis_scan(a, "sum", inclusive)

    def cumprod(self, a, inclusive=True):
        return self.axis_scan(a, "prod", inclusive)

    def astype(self, a, dtype):
        return a.astype(dtype)

    def any_isnan(self, a, axes=None, keepdims=False):
        """op::any_isnan (dali/array/op/reducers.cpp:66-75): max over isnan."""
        return self.max(self.isnan(a), axes, keepdims)

    def any_isinf(self, a, axes=None, keepdims=False):
        return self.max(self.isinf(a), axes, keepdims)

    def __getattr__(self, name):
        unary = {"identity", "sqrt", "square", "abs", "sigmoid", "dsigmoid", "tanh", "dtanh", "relu", "relu_backward",
                 "eltinv", "exp", "log", "log_or_zero", "sign", "softplus", "softplus_backward", "cube", "rsqrt",
                 "isnan", "isinf", "inverse_tanh", "round", "ceil"}
        binary = {"add", "subtract", "eltmul", "eltdiv", "equals", "pow", "steep_sigmoid", "steep_sigmoid_backward",
                  "clipped_relu", "clipped_relu_backward", "prelu", "prelu_backward_weights", "prelu_backward_inputs",
                  "lessthanequal", "greaterthanequal", "maximum", "minimum", "clip", "binary_cross_entropy",
                  "binary_cross_entropy_grad", "all_equals"}
        if name in unary:
            return lambda a: self._unary(name, a)
        if name in binary:
            return lambda a, b: self._binary(name, a, b)
        raise AttributeError(name)


op = _Op()


def lazy_stats():
    """(kernels, gemms, temporaries) launched by this thread's evaluations so far."""
    s = (ctypes.c_int64 * 3)()
    _c().c.dali_lazy_stats(s)
    return {"kernels": int(s[0]), "gemms": int(s[1]), "temporaries": int(s[2])}


def collectives():
    """(number of cross-rank combines issued by this thread's evaluations, description of the last one)."""
    n = ctypes.c_int64(0)
    buf = ctypes.create_string_buffer(1 << 12)
    _c().c.dali_lazy_collectives(ctypes.byref(n), buf, len(buf))
    return int(n.value), buf.value.decode()


class scope_trace:
    """with scope_trace() as t: ...; t.names lists the trace scopes left inside the block, in order (Scope / ScopeObserver
    of dali/utils/scope.h: one per computation, named after the evaluated expression, plus "get_function")."""

    def __enter__(self):
        _c().c.dali_scope_trace_start()
        self.names = []
        return self

    def __exit__(self, *exc):
        _c().c.dali_scope_trace_stop.restype = ctypes.c_size_t
        buf = ctypes.create_string_buffer(1 << 20)
        _c().c.dali_scope_trace_stop(buf, len(buf))
        self.names = [n for n in buf.value.decode().split("\n") if n]
        return False


def set_dry_run(on):
    """Lower and compile only (no device work, results undefined): inspect fusion without a GPU."""
    _c().c.dali_lazy_set_dry_run(int(bool(on)))


def eval_together(*arrays, wait=True):
    """Evaluates several lazy arrays of one shape in one kernel where their trees allow it (not in the reference)."""
    hs = (_H * len(arrays))(*[a._h.value for a in arrays])
    _check(_c().c.dali_array_eval_together(hs, len(arrays), int(wait)))


def set_seed(seed):
    """utils::random::set_seed: the seeds of the random operators built from now on."""
    _check(_c().c.dali_random_set_seed(int(seed)))


def set_default_device(gpu):
    """memory::default_preferred_device = Device::gpu(gpu) (one process per GPU sets its own)."""
    _check(_c().c.dali_set_default_device(int(gpu)))


def last_ir():
    buf = ctypes.create_string_buffer(1 << 16)
    _c().c.dali_lazy_last_ir(buf, len(buf))
    return buf.value.decode()


def last_variant():
    buf = ctypes.create_string_buffer(1 << 12)
    _c().c.dali_lazy_last_variant(buf, len(buf))
    return buf.value.decode()
