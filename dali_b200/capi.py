"""ctypes binding of include/dali_b200.h -- test / benchmark plumbing only.

Nothing here computes: every call goes into libdali_b200.so, and loading fails
loudly when the library has not been built.
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libdali_b200.so")

F32, F64, I32, BF16 = 0, 1, 2, 3
_NP_DTYPE = {F32: np.float32, F64: np.float64, I32: np.int32}

c_i64p = ctypes.POINTER(ctypes.c_int64)


class DaliB200Error(RuntimeError):
    def __init__(self, status, message):
        super().__init__("dali_b200 status %d: %s" % (status, message))
        self.status = status


def _i64_array(values):
    return (ctypes.c_int64 * len(values))(*[int(v) for v in values])


class Library:
    """Thin wrapper: one method per C entry point, errors raised as exceptions."""

    def __init__(self, path=LIB_PATH):
        if not os.path.exists(path):
            raise ImportError("libdali_b200.so is not built (%s); run __graft_entry__.build()" % path)
        self.path = path
        self.c = ctypes.CDLL(path)
        c = self.c
        c.dalib200_last_error.restype = ctypes.c_size_t
        c.dalib200_last_error.argtypes = [ctypes.c_char_p, ctypes.c_size_t]
        c.dalib200_last_variant.restype = ctypes.c_size_t
        c.dalib200_last_variant.argtypes = [ctypes.c_char_p, ctypes.c_size_t]
        c.dalib200_cache_get_dir.restype = ctypes.c_size_t
        c.dalib200_cache_get_dir.argtypes = [ctypes.c_char_p, ctypes.c_size_t]
        c.dalib200_compile.argtypes = [ctypes.c_uint64, ctypes.c_char_p, ctypes.c_size_t]
        c.dalib200_is_loaded.argtypes = [ctypes.c_uint64]
        c.dalib200_precompile.argtypes = [ctypes.c_uint64, c_i64p, ctypes.c_int, ctypes.POINTER(ctypes.c_void_p),
                                          c_i64p, ctypes.POINTER(c_i64p), ctypes.c_int,
                                          ctypes.POINTER(ctypes.c_size_t)]
        c.dalib200_launch.argtypes = [ctypes.c_uint64, ctypes.c_int, ctypes.c_void_p, c_i64p, ctypes.c_int,
                                      ctypes.POINTER(ctypes.c_void_p), c_i64p, ctypes.POINTER(c_i64p), ctypes.c_int,
                                      ctypes.POINTER(ctypes.c_void_p), ctypes.c_int]
        c.dalib200_launch_host.argtypes = [ctypes.c_uint64, ctypes.c_int, c_i64p, ctypes.c_int,
                                           ctypes.POINTER(ctypes.c_void_p), c_i64p, c_i64p, ctypes.POINTER(c_i64p),
                                           ctypes.c_int, ctypes.POINTER(ctypes.c_void_p), ctypes.c_int]
        c.dalib200_alloc.argtypes = [ctypes.c_int, ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p)]
        c.dalib200_free.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t]
        for name in ("dalib200_memcpy_h2d", "dalib200_memcpy_d2h", "dalib200_memcpy_d2d"):
            getattr(c, name).argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t,
                                         ctypes.c_void_p]
        c.dalib200_memset.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t, ctypes.c_void_p]
        c.dalib200_sync.argtypes = [ctypes.c_int, ctypes.c_void_p]
        c.dalib200_gemm.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int] + [ctypes.c_int64] * 3 + \
            [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64] * 3 + [ctypes.c_double, ctypes.c_double]
        c.dalib200_gemm_fused.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_int64,
                                          ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64,
                                          ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint64,
                                          ctypes.POINTER(ctypes.c_void_p), c_i64p, ctypes.POINTER(c_i64p), ctypes.c_int,
                                          ctypes.POINTER(ctypes.c_void_p), ctypes.c_int]
        vpp = ctypes.POINTER(ctypes.c_void_p)
        c.dalib200_gemm_fused_sum.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int64,
                                              ctypes.c_int64, c_i64p, vpp, c_i64p, vpp, c_i64p, vpp, vpp, ctypes.c_uint64,
                                              vpp, c_i64p, ctypes.POINTER(c_i64p), ctypes.c_int, vpp, ctypes.c_int]
        c.dalib200_gemm_split_tf32.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                               ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_void_p,
                                               ctypes.c_void_p]
        c.dalib200_scan.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int64,
                                    ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64]
        c.dalib200_gemm_split_tf32_pair.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p] + \
            [ctypes.c_int64] * 4 + [ctypes.c_void_p] * 4
        c.dalib200_gemm_error_flag.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_int)]
        c.dalib200_last_gemm_kernel.restype = ctypes.c_size_t
        c.dalib200_last_gemm_kernel.argtypes = [ctypes.c_char_p, ctypes.c_size_t]
        c.dalib200_cache_set_dir.argtypes = [ctypes.c_char_p]
        c.dalib200_cache_stats.argtypes = [ctypes.POINTER(ctypes.c_uint64)]
        # ranks and collectives
        self.HOST_ALLREDUCE = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_int)
        self.HOST_ALLGATHER = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64)
        c.dalib200_comm_unique_id.argtypes = [ctypes.c_void_p]
        c.dalib200_comm_init_rank.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        c.dalib200_comm_init_host.argtypes = [ctypes.c_int, ctypes.c_int, self.HOST_ALLREDUCE, self.HOST_ALLGATHER, ctypes.c_void_p]
        c.dalib200_comm_transport.restype = ctypes.c_size_t
        c.dalib200_comm_transport.argtypes = [ctypes.c_char_p, ctypes.c_size_t]
        c.dalib200_comm_error_flag.argtypes = [ctypes.POINTER(ctypes.c_int)]
        c.dalib200_shard_range.argtypes = [ctypes.c_int64, ctypes.c_int, ctypes.c_int, c_i64p, c_i64p]
        c.dalib200_allreduce.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_int]
        c.dalib200_arg_allreduce.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                             ctypes.c_int, ctypes.c_int]
        c.dalib200_peer_emulate.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                            ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p), ctypes.c_int64,
                                            ctypes.c_int, ctypes.POINTER(ctypes.c_int)]
        self._host_callbacks = None
        self._next_hash = 0x0da11b200

    # -- errors ---------------------------------------------------------------
    def last_error(self):
        buf = ctypes.create_string_buffer(1 << 16)
        self.c.dalib200_last_error(buf, len(buf))
        return buf.value.decode(errors="replace")

    def last_variant(self):
        buf = ctypes.create_string_buffer(1 << 12)
        self.c.dalib200_last_variant(buf, len(buf))
        return buf.value.decode()

    def check(self, status):
        if status != 0:
            raise DaliB200Error(status, self.last_error())

    # -- lifecycle ------------------------------------------------------------
    def abi_version(self):
        return self.c.dalib200_abi_version()

    def init(self, n_gpus=0):
        self.check(self.c.dalib200_init(n_gpus))

    def device_count(self):
        return self.c.dalib200_device_count()

    def cache_set_dir(self, path):
        self.check(self.c.dalib200_cache_set_dir(path.encode()))

    def cache_get_dir(self):
        buf = ctypes.create_string_buffer(4096)
        self.c.dalib200_cache_get_dir(buf, len(buf))
        return buf.value.decode()

    def cache_clear(self, remove_files=False):
        self.check(self.c.dalib200_cache_clear(int(remove_files)))

    def cache_stats(self):
        s = (ctypes.c_uint64 * 5)()
        self.check(self.c.dalib200_cache_stats(s))
        return dict(zip(("programs", "kernels", "compilations", "disk_hits", "launches"), [int(x) for x in s]))

    # -- compile / launch -----------------------------------------------------
    def compile(self, ir, hash_=None):
        """Registers `ir`; returns the hash it is registered under."""
        if hash_ is None:
            h = 1469598103934665603
            for ch in ir.encode():
                h = ((h ^ ch) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
            hash_ = h
        data = ir.encode()
        self.check(self.c.dalib200_compile(ctypes.c_uint64(hash_), data, len(data)))
        return hash_

    def is_loaded(self, hash_):
        return bool(self.c.dalib200_is_loaded(ctypes.c_uint64(hash_)))

    @staticmethod
    def _strides_arg(strides, n):
        keep = []
        if strides is None:
            return None, keep
        arr = (c_i64p * n)()
        for i, s in enumerate(strides):
            if s is None:
                arr[i] = None
            else:
                a = _i64_array(s)
                keep.append(a)
                arr[i] = ctypes.cast(a, c_i64p)
        return arr, keep

    def precompile(self, hash_, space, n_arrays, strides=None, pointers=None, offsets=None):
        ptrs = (ctypes.c_void_p * n_arrays)(*[(pointers[i] if pointers else 4096) for i in range(n_arrays)])
        offs = _i64_array(offsets if offsets else [0] * n_arrays)
        st, keep = self._strides_arg(strides, n_arrays)
        size = ctypes.c_size_t(0)
        self.check(self.c.dalib200_precompile(ctypes.c_uint64(hash_), _i64_array(space), len(space), ptrs, offs, st,
                                              n_arrays, ctypes.byref(size)))
        return size.value

    @staticmethod
    def _scalars_arg(scalars):
        keep = [np.ascontiguousarray(s) for s in (scalars or [])]
        arr = (ctypes.c_void_p * max(len(keep), 1))(*[k.ctypes.data for k in keep])
        return arr, keep

    def launch(self, hash_, space, arrays, strides=None, offsets=None, scalars=None, device=0, stream=None):
        """arrays: device pointers (ints) or objects with data_ptr() (torch CUDA tensors)."""
        n = len(arrays)
        ptrs = (ctypes.c_void_p * n)(*[(a.data_ptr() if hasattr(a, "data_ptr") else int(a)) for a in arrays])
        offs = _i64_array(offsets if offsets else [0] * n)
        st, keep = self._strides_arg(strides, n)
        sc, keep2 = self._scalars_arg(scalars)
        self.check(self.c.dalib200_launch(ctypes.c_uint64(hash_), device, ctypes.c_void_p(stream or 0),
                                          _i64_array(space), len(space), ptrs, offs, st, n, sc,
                                          len(scalars or [])))

    def launch_host(self, hash_, space, arrays, strides=None, offsets=None, scalars=None, device=0):
        """arrays: numpy arrays (whole buffers, C-contiguous); written ones are updated in place."""
        n = len(arrays)
        for a in arrays:
            assert a.flags["C_CONTIGUOUS"]
        ptrs = (ctypes.c_void_p * n)(*[a.ctypes.data for a in arrays])
        ext = _i64_array([a.size for a in arrays])
        offs = _i64_array(offsets if offsets else [0] * n)
        st, keep = self._strides_arg(strides, n)
        sc, keep2 = self._scalars_arg(scalars)
        self.check(self.c.dalib200_launch_host(ctypes.c_uint64(hash_), device, _i64_array(space), len(space), ptrs,
                                               ext, offs, st, n, sc, len(scalars or [])))

    # -- GEMM -----------------------------------------------------------------
    @staticmethod
    def _ptr(x):
        return ctypes.c_void_p(x.data_ptr() if hasattr(x, "data_ptr") else int(x))

    def gemm(self, dtype, m, n, k, a, a_strides, b, b_strides, c, c_strides, alpha=1.0, beta=0.0, device=0, stream=None):
        self.check(self.c.dalib200_gemm(device, ctypes.c_void_p(stream or 0), dtype, m, n, k, self._ptr(a), a_strides[0],
                                        a_strides[1], self._ptr(b), b_strides[0], b_strides[1], self._ptr(c), c_strides[0],
                                        c_strides[1], alpha, beta))

    def gemm_fused(self, ab_dtype, m, n, k, a, lda, b, ldb, epilogue_hash, arrays, strides=None, offsets=None, scalars=None,
                   a_lo=None, b_lo=None, device=0, stream=None):
        """acc = A[m,k] . B[k,n] on the tensor cores, then the registered epilogue program over [m,n]."""
        na = len(arrays)
        ptrs = (ctypes.c_void_p * na)(*[(x.data_ptr() if hasattr(x, "data_ptr") else int(x)) for x in arrays])
        offs = _i64_array(offsets if offsets else [0] * na)
        st, keep = self._strides_arg(strides, na)
        sc, keep2 = self._scalars_arg(scalars)
        self.check(self.c.dalib200_gemm_fused(device, ctypes.c_void_p(stream or 0), ab_dtype, m, n, k, self._ptr(a), lda,
                                              self._ptr(b), ldb, self._ptr(a_lo) if a_lo is not None else None,
                                              self._ptr(b_lo) if b_lo is not None else None, ctypes.c_uint64(epilogue_hash),
                                              ptrs, offs, st, na, sc, len(scalars or [])))

    def gemm_fused_sum(self, ab_dtype, m, n, pairs, epilogue_hash, arrays, strides=None, offsets=None, scalars=None,
                       device=0, stream=None):
        """acc = sum over pairs of A_p[m,k_p] . B_p[k_p,n] in one launch, then the epilogue program.  Each pair is
        (k, a, lda, b, ldb) or, with the TF32 split parts of fp32 operands, (k, a_hi, lda, b_hi, ldb, a_lo, b_lo)."""
        na, npairs = len(arrays), len(pairs)
        ptrs = (ctypes.c_void_p * na)(*[(x.data_ptr() if hasattr(x, "data_ptr") else int(x)) for x in arrays])
        offs = _i64_array(offsets if offsets else [0] * na)
        st, keep = self._strides_arg(strides, na)
        sc, keep2 = self._scalars_arg(scalars)

        def col(j):
            return (ctypes.c_void_p * npairs)(*[self._ptr(p[j]).value for p in pairs])
        with_lo = all(len(p) == 7 for p in pairs)
        self.check(self.c.dalib200_gemm_fused_sum(device, ctypes.c_void_p(stream or 0), ab_dtype, npairs, m, n,
                                                  _i64_array([p[0] for p in pairs]), col(1), _i64_array([p[2] for p in pairs]),
                                                  col(3), _i64_array([p[4] for p in pairs]), col(5) if with_lo else None,
                                                  col(6) if with_lo else None, ctypes.c_uint64(epilogue_hash), ptrs, offs, st,
                                                  na, sc, len(scalars or [])))

    def gemm_split_tf32(self, x, rows, cols, ld, hi, lo, transpose=False, device=0, stream=None):
        self.check(self.c.dalib200_gemm_split_tf32(device, ctypes.c_void_p(stream or 0), self._ptr(x), rows, cols, ld,
                                                   int(transpose), self._ptr(hi), self._ptr(lo)))

    def scan(self, dtype, op, inclusive, rows, cols, x, out, in_row_stride=None, out_row_stride=None, device=0, stream=None):
        """Running reduction (op 0 sum, 1 prod, 2 max, 3 min) along the rows of a [rows, cols] matrix."""
        self.check(self.c.dalib200_scan(device, ctypes.c_void_p(stream or 0), dtype, op, int(bool(inclusive)), rows, cols,
                                        self._ptr(x), cols if in_row_stride is None else in_row_stride, self._ptr(out),
                                        (cols + (0 if inclusive else 1)) if out_row_stride is None else out_row_stride))

    def gemm_split_tf32_pair(self, x0, x1, rows, cols, ld0, ld1, hi0, lo0, hi1, lo1, device=0, stream=None):
        self.check(self.c.dalib200_gemm_split_tf32_pair(device, ctypes.c_void_p(stream or 0), self._ptr(x0), self._ptr(x1), rows,
                                                        cols, ld0, ld1, self._ptr(hi0), self._ptr(lo0), self._ptr(hi1),
                                                        self._ptr(lo1)))

    def gemm_error_flag(self, device=0):
        f = ctypes.c_int(0)
        self.check(self.c.dalib200_gemm_error_flag(device, ctypes.byref(f)))
        return f.value

    def last_gemm_kernel(self):
        buf = ctypes.create_string_buffer(512)
        self.c.dalib200_last_gemm_kernel(buf, len(buf))
        return buf.value.decode()

    # -- ranks and collectives ---------------------------------------------------
    OPS = {"sum": 0, "prod": 1, "max": 2, "min": 3}

    def comm_unique_id(self):
        buf = ctypes.create_string_buffer(128)
        self.check(self.c.dalib200_comm_unique_id(buf))
        return buf.raw

    def comm_init_rank(self, device, world, rank, unique_id=None):
        self.check(self.c.dalib200_comm_init_rank(device, world, rank, unique_id))

    def comm_init_host(self, world, rank, allreduce, allgather):
        """allreduce(buf_address, n, dtype, op) / allgather(send_address, recv_address, nbytes): Python callables on host
        memory addresses; they return nothing and raise on failure."""
        def ar(ctx, buf, n, dtype, op):
            try:
                allreduce(buf, n, dtype, op)
                return 0
            except Exception:       # the C side reports the failure as a status
                return 1

        def ag(ctx, send, recv, nbytes):
            try:
                allgather(send, recv, nbytes)
                return 0
            except Exception:
                return 1
        self._host_callbacks = (self.HOST_ALLREDUCE(ar), self.HOST_ALLGATHER(ag))      # kept alive for the C side
        self.check(self.c.dalib200_comm_init_host(world, rank, self._host_callbacks[0], self._host_callbacks[1], None))

    def comm_destroy(self):
        self.check(self.c.dalib200_comm_destroy())
        self._host_callbacks = None

    def comm_world(self):
        return self.c.dalib200_comm_world()

    def comm_rank(self):
        return self.c.dalib200_comm_rank()

    def comm_transport(self):
        buf = ctypes.create_string_buffer(512)
        self.c.dalib200_comm_transport(buf, len(buf))
        return buf.value.decode()

    def comm_error_flag(self):
        f = ctypes.c_int(0)
        self.check(self.c.dalib200_comm_error_flag(ctypes.byref(f)))
        return f.value

    def shard_range(self, n, rank, world):
        lo, hi = ctypes.c_int64(0), ctypes.c_int64(0)
        self.check(self.c.dalib200_shard_range(n, rank, world, ctypes.byref(lo), ctypes.byref(hi)))
        return lo.value, hi.value

    @staticmethod
    def _buf(x):
        if isinstance(x, np.ndarray):
            return ctypes.c_void_p(x.ctypes.data)
        return ctypes.c_void_p(x.data_ptr() if hasattr(x, "data_ptr") else int(x))

    def allreduce(self, buf, n, dtype, op, device=0, stream=None):
        """buf: torch CUDA tensor / device address, or (device = -1, host transport) a numpy array."""
        self.check(self.c.dalib200_allreduce(device, ctypes.c_void_p(stream or 0), self._buf(buf), n, dtype, self.OPS.get(op, op)))

    def arg_allreduce(self, values, indices, n, dtype, op, device=0, stream=None):
        self.check(self.c.dalib200_arg_allreduce(device, ctypes.c_void_p(stream or 0), self._buf(values), self._buf(indices), n,
                                                 dtype, self.OPS.get(op, op)))

    def peer_emulate(self, bufs, n, dtype, op, indices=None, repeats=1, device=0, stream=None):
        """The peer-exchange protocol with len(bufs) virtual ranks in one kernel on one GPU; returns the error flag."""
        world = len(bufs)
        pb = (ctypes.c_void_p * world)(*[self._buf(b).value for b in bufs])
        pi = (ctypes.c_void_p * world)(*[self._buf(i).value for i in indices]) if indices is not None else None
        flag = ctypes.c_int(0)
        self.check(self.c.dalib200_peer_emulate(device, ctypes.c_void_p(stream or 0), world, dtype, self.OPS.get(op, op),
                                                int(indices is not None), pb, pi, n, repeats, ctypes.byref(flag)))
        return flag.value

    # -- memory ---------------------------------------------------------------
    def alloc(self, nbytes, device=0):
        p = ctypes.c_void_p()
        self.check(self.c.dalib200_alloc(device, nbytes, ctypes.byref(p)))
        return p.value

    def free(self, ptr, nbytes, device=0):
        self.check(self.c.dalib200_free(device, ctypes.c_void_p(ptr), nbytes))

    def h2d(self, dst, src_np, device=0, stream=None):
        self.check(self.c.dalib200_memcpy_h2d(device, ctypes.c_void_p(dst), src_np.ctypes.data, src_np.nbytes,
                                              ctypes.c_void_p(stream or 0)))

    def d2h(self, dst_np, src, device=0, stream=None):
        self.check(self.c.dalib200_memcpy_d2h(device, dst_np.ctypes.data, ctypes.c_void_p(src), dst_np.nbytes,
                                              ctypes.c_void_p(stream or 0)))

    def sync(self, device=0, stream=None):
        self.check(self.c.dalib200_sync(device, ctypes.c_void_p(stream or 0)))


_LIB = None


def load_library():
    global _LIB
    if _LIB is None:
        _LIB = Library()
    return _LIB
