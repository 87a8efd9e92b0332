"""numpy front-end of the CPU oracle (TEST INFRASTRUCTURE ONLY).

Loads oracle/_build/libsmore_oracle.so (the plain-C restatement in
smore_oracle.c) and, when present, oracle/_ref/libsmore_ref_host.so (the
reference's own functor header compiled as host C++).  Only tests, the smoke
check and the CPU-baseline legs of the benchmark may import this module; the
product package never does.
"""
import ctypes
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

DIST_IDS = {"box_out": 0, "box_in": 1, "rotate": 2, "l1": 3, "l2": 4, "complex": 5, "distmult": 6}
OPT_IDS = {"sgd": 0, "adam": 1, "adagrad": 2}
TWO_PART_ROWS = {"rotate", "complex"}           # entity row = [part0 | part1], each `dim` long
TWO_PART_QUERY = {"box_out", "box_in", "rotate", "complex"}

_f32p = ctypes.POINTER(ctypes.c_float)
_f64p = ctypes.POINTER(ctypes.c_double)
_i64p = ctypes.POINTER(ctypes.c_int64)
_i32p = ctypes.POINTER(ctypes.c_int32)
_sz = ctypes.c_size_t


def _ptr(a, typ):
    if a is None:
        return ctypes.cast(None, typ)
    return a.ctypes.data_as(typ)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class _Lib:
    def __init__(self, path, prefix, with_optimizer):
        self.path = path
        self.lib = ctypes.CDLL(path)
        fwd = getattr(self.lib, prefix + "dist_forward")
        fwd.restype = ctypes.c_int
        fwd.argtypes = [ctypes.c_int, _f32p, _f32p, _f32p, _f32p] + [_sz] * 7
        bwd = getattr(self.lib, prefix + "dist_backward")
        bwd.restype = ctypes.c_int
        bwd.argtypes = [ctypes.c_int] + [_f32p] * 7 + [_sz] * 7
        self._fwd, self._bwd = fwd, bwd
        if with_optimizer:
            L = self.lib
            L.oracle_dist_forward_f64acc.restype = ctypes.c_int
            L.oracle_dist_forward_f64acc.argtypes = [ctypes.c_int, _f32p, _f32p, _f32p, _f64p] + [_sz] * 7
            L.oracle_unique_rows.restype = ctypes.c_int64
            L.oracle_unique_rows.argtypes = [_i64p, _sz, _i64p, _i32p, _i32p]
            L.oracle_scatter_sum_rows.restype = ctypes.c_int
            L.oracle_scatter_sum_rows.argtypes = [_f32p, _i32p, _sz, _sz, _f32p, _sz]
            L.oracle_sparse_update_rows.restype = ctypes.c_int
            L.oracle_sparse_update_rows.argtypes = [ctypes.c_int, _f32p, _f32p, _f32p, _i64p, _f32p, _sz, _sz,
                                                    ctypes.c_double, ctypes.c_double, ctypes.c_double,
                                                    ctypes.c_double, ctypes.c_int64, ctypes.c_int]
            L.oracle_gather_rows.restype = ctypes.c_int
            L.oracle_gather_rows.argtypes = [_f32p, _i64p, _sz, _sz, _f32p]
            L.oracle_num_threads.restype = ctypes.c_int

    # entity [be, ne, mul*dim]; first/second [bc, nc, dim]
    def dist_forward(self, name, entity, first, second=None):
        entity, first = _f32(entity), _f32(first)
        second = None if second is None else _f32(second)
        be, ne, _ = entity.shape
        bc, nc, dim = first.shape
        bsize, num = max(be, bc), max(ne, nc)
        dst = np.empty((bsize, num), dtype=np.float32)
        rc = self._fwd(DIST_IDS[name], _ptr(entity, _f32p), _ptr(first, _f32p), _ptr(second, _f32p),
                       _ptr(dst, _f32p), bsize, num, be, ne, bc, nc, dim)
        if rc != 0:
            raise RuntimeError("oracle forward failed: %d" % rc)
        return dst

    def dist_backward(self, name, gout, entity, first, second=None):
        gout, entity, first = _f32(gout), _f32(entity), _f32(first)
        second = None if second is None else _f32(second)
        be, ne, _ = entity.shape
        bc, nc, dim = first.shape
        bsize, num = gout.shape
        g_ent = np.full(entity.shape, np.nan, dtype=np.float32)
        g_first = np.full(first.shape, np.nan, dtype=np.float32)
        g_second = None if second is None else np.full(first.shape, np.nan, dtype=np.float32)
        rc = self._bwd(DIST_IDS[name], _ptr(gout, _f32p), _ptr(entity, _f32p), _ptr(first, _f32p),
                       _ptr(second, _f32p), _ptr(g_ent, _f32p), _ptr(g_first, _f32p), _ptr(g_second, _f32p),
                       bsize, num, be, ne, bc, nc, dim)
        if rc != 0:
            raise RuntimeError("oracle backward failed: %d" % rc)
        return g_ent, g_first, g_second


class Oracle(_Lib):
    def __init__(self):
        path = os.path.join(HERE, "_build", "libsmore_oracle.so")
        if not os.path.exists(path):
            raise FileNotFoundError(path + " missing: run `python oracle/build.py`")
        super().__init__(path, "oracle_", True)

    def num_threads(self):
        return int(self.lib.oracle_num_threads())

    def dist_forward_f64acc(self, name, entity, first, second=None):
        entity, first = _f32(entity), _f32(first)
        second = None if second is None else _f32(second)
        be, ne, _ = entity.shape
        bc, nc, dim = first.shape
        bsize, num = max(be, bc), max(ne, nc)
        dst = np.empty((bsize, num), dtype=np.float64)
        self.lib.oracle_dist_forward_f64acc(DIST_IDS[name], _ptr(entity, _f32p), _ptr(first, _f32p),
                                            _ptr(second, _f32p), _ptr(dst, _f64p), bsize, num, be, ne, bc, nc,
                                            dim)
        return dst

    def unique_rows(self, idx):
        idx = np.ascontiguousarray(idx, dtype=np.int64).reshape(-1)
        n = idx.shape[0]
        uniq = np.empty(n, dtype=np.int64)
        inverse = np.empty(n, dtype=np.int32)
        counts = np.empty(n, dtype=np.int32)
        nu = self.lib.oracle_unique_rows(_ptr(idx, _i64p), n, _ptr(uniq, _i64p), _ptr(inverse, _i32p),
                                         _ptr(counts, _i32p))
        if nu < 0:
            raise MemoryError
        return uniq[:nu].copy(), inverse, counts[:nu].copy()

    def scatter_sum_rows(self, grad, inverse, n_unique):
        grad = _f32(grad)
        inverse = np.ascontiguousarray(inverse, dtype=np.int32)
        n, width = grad.shape
        merged = np.empty((n_unique, width), dtype=np.float32)
        self.lib.oracle_scatter_sum_rows(_ptr(grad, _f32p), _ptr(inverse, _i32p), n, width, _ptr(merged, _f32p),
                                         n_unique)
        return merged

    def sparse_update_rows(self, opt, table, m, v, uniq, grad, lr, step, squeeze, beta1=0.9, beta2=0.999,
                           eps=1e-8):
        """In-place on table / m / v (float32, C-contiguous)."""
        for a in (table, m, v):
            assert a is None or (a.dtype == np.float32 and a.flags.c_contiguous)
        uniq = np.ascontiguousarray(uniq, dtype=np.int64)
        grad = _f32(grad)
        n_unique, width = grad.shape
        self.lib.oracle_sparse_update_rows(OPT_IDS[opt], _ptr(table, _f32p), _ptr(m, _f32p), _ptr(v, _f32p),
                                           _ptr(uniq, _i64p), _ptr(grad, _f32p), n_unique, width, lr, beta1,
                                           beta2, eps, step, int(bool(squeeze)))

    def gather_rows(self, table, idx):
        table = _f32(table)
        idx = np.ascontiguousarray(idx, dtype=np.int64).reshape(-1)
        out = np.empty((idx.shape[0], table.shape[1]), dtype=np.float32)
        self.lib.oracle_gather_rows(_ptr(table, _f32p), _ptr(idx, _i64p), idx.shape[0], table.shape[1],
                                    _ptr(out, _f32p))
        return out


class ReferenceHost(_Lib):
    """The reference's functor header compiled for the host (oracle/_ref)."""

    def __init__(self):
        path = os.path.join(HERE, "_ref", "libsmore_ref_host.so")
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        super().__init__(path, "ref_host_", False)


def reference_host_available():
    return os.path.exists(os.path.join(HERE, "_ref", "libsmore_ref_host.so"))


def reference_cuda_path():
    p = os.path.join(HERE, "_ref", "libsmore_ref_cuda.so")
    return p if os.path.exists(p) else None
