"""ctypes front end of ``libfg_oracle.so`` (the C restatement in fg_oracle.c).

TEST INFRASTRUCTURE: the checker for the CUDA path and the timed CPU baseline,
never a code path of the product.  The C file's header states what it follows
in the reference and how its parity is pinned.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libfg_oracle.so")
_lib = None

_i32p = ctypes.POINTER(ctypes.c_int32)
_f32p = ctypes.POINTER(ctypes.c_float)
_f64p = ctypes.POINTER(ctypes.c_double)


def build(force=False):
    """Compile fg_oracle.c with the flags in the Makefile (gcc, OpenMP)."""
    src = os.path.join(_HERE, "fg_oracle.c")
    if (not force and os.path.exists(_LIB_PATH)
            and os.path.getmtime(_LIB_PATH) >= os.path.getmtime(src)):
        return _LIB_PATH
    subprocess.run(["make", "-C", _HERE, "-B", "libfg_oracle.so"], check=True,
                   capture_output=True)
    return _LIB_PATH


def _load():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        lib = ctypes.CDLL(_LIB_PATH)
        lib.fg_oracle_max_threads.restype = ctypes.c_int
        lib.fg_oracle_set_threads.argtypes = [ctypes.c_int]
        lib.fg_oracle_spmm_csr_f32.argtypes = [
            ctypes.c_int64, ctypes.c_int64, ctypes.c_int32, _i32p, _i32p, _f32p, _f32p, _f32p,
            ctypes.c_int32, _f32p]
        lib.fg_oracle_spmm_csr_f64.argtypes = [
            ctypes.c_int64, ctypes.c_int32, _i32p, _i32p, _f32p, _f32p, _f64p]
        lib.fg_oracle_sddmm_coo_f32.argtypes = [
            ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int32, ctypes.c_int32,
            _i32p, _i32p, _f32p, _f32p, _f32p, ctypes.c_int32, ctypes.c_int32, _f32p]
        lib.fg_oracle_sddmm_coo_f64.argtypes = [
            ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, _i32p, _i32p, _f32p, _f32p, _f64p]
        _lib = lib
    return _lib


def _c(a, dtype):
    a = np.ascontiguousarray(a, dtype=dtype)
    return a


def _p(a, ptype):
    return a.ctypes.data_as(ptype)


def max_threads():
    return int(_load().fg_oracle_max_threads())


def set_threads(n):
    _load().fg_oracle_set_threads(int(n))


def spmm_csr_f32(indptr, indices, vals, x, n_cols=None, num_feat_partitions=1, out=None,
                 work=None):
    """Y = A @ X in the reference's x86 loop order (vanilla_spmm.py:43-60, 73-78)."""
    lib = _load()
    indptr, indices = _c(indptr, np.int32), _c(indices, np.int32)
    vals, x = _c(vals, np.float32), _c(x, np.float32)
    n_rows = indptr.shape[0] - 1
    n_cols = x.shape[0] if n_cols is None else n_cols
    assert x.shape[0] == n_cols
    f = x.shape[1]
    y = np.empty((n_rows, f), np.float32) if out is None else out
    if work is None:
        work = np.empty((n_rows + n_cols) * f, np.float32)
    rc = lib.fg_oracle_spmm_csr_f32(n_rows, n_cols, f, _p(indptr, _i32p), _p(indices, _i32p),
                                    _p(vals, _f32p), _p(x, _f32p), _p(y, _f32p),
                                    int(num_feat_partitions), _p(work, _f32p))
    if rc != 0:
        raise ValueError("fg_oracle_spmm_csr_f32: bad argument")
    return y


def spmm_csr_f64(indptr, indices, vals, x):
    lib = _load()
    indptr, indices = _c(indptr, np.int32), _c(indices, np.int32)
    vals, x = _c(vals, np.float32), _c(x, np.float32)
    n_rows = indptr.shape[0] - 1
    y = np.empty((n_rows, x.shape[1]), np.float64)
    lib.fg_oracle_spmm_csr_f64(n_rows, x.shape[1], _p(indptr, _i32p), _p(indices, _i32p),
                               _p(vals, _f32p), _p(x, _f32p), _p(y, _f64p))
    return y


def sddmm_coo_f32(row, col, src, dst, num_heads=1, num_feat_partitions=1, parallel=False,
                  out=None):
    """out[e,h] = sum_d src[col[e],h,d] * dst[row[e],h,d]  (vanilla_sddmm.py:43-62, 66-74).

    Returns shape (nnz,) for one head, (nnz, H) otherwise.
    """
    lib = _load()
    row, col = _c(row, np.int32), _c(col, np.int32)
    src, dst = _c(src, np.float32), _c(dst, np.float32)
    nnz = row.shape[0]
    n_cols, f = src.shape[0], int(np.prod(src.shape[1:]))
    n_rows = dst.shape[0]
    assert int(np.prod(dst.shape[1:])) == f
    res = np.empty((nnz, num_heads), np.float32) if out is None else out
    work = None
    if num_feat_partitions > 1:
        work = np.empty((n_rows + n_cols) * f, np.float32)
    rc = lib.fg_oracle_sddmm_coo_f32(nnz, n_rows, n_cols, f, int(num_heads), _p(row, _i32p),
                                     _p(col, _i32p), _p(src, _f32p), _p(dst, _f32p),
                                     _p(res, _f32p), int(num_feat_partitions), int(bool(parallel)),
                                     _p(work, _f32p) if work is not None else None)
    if rc != 0:
        raise ValueError("fg_oracle_sddmm_coo_f32: bad argument")
    return res.reshape(nnz) if num_heads == 1 and out is None else res


def sddmm_coo_f64(row, col, src, dst, num_heads=1):
    lib = _load()
    row, col = _c(row, np.int32), _c(col, np.int32)
    src, dst = _c(src, np.float32), _c(dst, np.float32)
    nnz = row.shape[0]
    f = int(np.prod(src.shape[1:]))
    res = np.empty((nnz, num_heads), np.float64)
    rc = lib.fg_oracle_sddmm_coo_f64(nnz, f, int(num_heads), _p(row, _i32p), _p(col, _i32p),
                                     _p(src, _f32p), _p(dst, _f32p), _p(res, _f64p))
    if rc != 0:
        raise ValueError("fg_oracle_sddmm_coo_f64: bad argument")
    return res.reshape(nnz) if num_heads == 1 else res


MSG_OPS = ("mul", "add", "sub", "div", "copy_lhs", "copy_rhs")
REDUCE_OPS = ("sum", "max", "min")


def gspmm_csr_f32(indptr, indices, vals, x, msg_op="mul", reduce_op="sum"):
    """Generalised SpMM: Y[r, f] = reduce over the row's nonzeros, in CSR order, of
    msg(X[indices[e], f], vals[e]) (the operator table is in fg_oracle.c)."""
    lib = _load()
    lib.fg_oracle_gspmm_csr_f32.argtypes = [
        ctypes.c_int64, ctypes.c_int32, _i32p, _i32p, _f32p, _f32p, _f32p, ctypes.c_int32,
        ctypes.c_int32]
    indptr, indices = _c(indptr, np.int32), _c(indices, np.int32)
    vals, x = _c(vals, np.float32), _c(x, np.float32)
    n_rows = indptr.shape[0] - 1
    y = np.empty((n_rows, x.shape[1]), np.float32)
    rc = lib.fg_oracle_gspmm_csr_f32(n_rows, x.shape[1], _p(indptr, _i32p), _p(indices, _i32p),
                                     _p(vals, _f32p), _p(x, _f32p), _p(y, _f32p),
                                     MSG_OPS.index(msg_op), REDUCE_OPS.index(reduce_op))
    if rc != 0:
        raise ValueError("fg_oracle_gspmm_csr_f32: bad argument")
    return y


def gsddmm_coo_f32(row, col, src, dst, num_heads=1, msg_op="mul", reduce_op="sum"):
    """Generalised SDDMM: out[e, h] = reduce over d ascending of
    msg(src[col[e], h, d], dst[row[e], h, d])."""
    lib = _load()
    lib.fg_oracle_gsddmm_coo_f32.argtypes = [
        ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, _i32p, _i32p, _f32p, _f32p, _f32p,
        ctypes.c_int32, ctypes.c_int32]
    row, col = _c(row, np.int32), _c(col, np.int32)
    src, dst = _c(src, np.float32), _c(dst, np.float32)
    nnz, f = row.shape[0], int(np.prod(src.shape[1:]))
    res = np.empty((nnz, num_heads), np.float32)
    rc = lib.fg_oracle_gsddmm_coo_f32(nnz, f, int(num_heads), _p(row, _i32p), _p(col, _i32p),
                                      _p(src, _f32p), _p(dst, _f32p), _p(res, _f32p),
                                      MSG_OPS.index(msg_op), REDUCE_OPS.index(reduce_op))
    if rc != 0:
        raise ValueError("fg_oracle_gsddmm_coo_f32: bad argument")
    return res.reshape(nnz) if num_heads == 1 else res


def spmm_dds_f32(s1_pos, s1_idx, vals, x, n_rows, num_col_partitions):
    """Y = A @ X over the DDS form (vanilla_spmm.py:149-246): per column block a partial sum
    in stored order, then the blocks' partial sums added in ascending block order."""
    lib = _load()
    lib.fg_oracle_spmm_dds_f32.argtypes = [
        ctypes.c_int64, ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, _i32p, _i32p, _f32p,
        _f32p, _f32p]
    s1_pos, s1_idx = _c(s1_pos, np.int32), _c(s1_idx, np.int32)
    vals, x = _c(vals, np.float32), _c(x, np.float32)
    y = np.empty((n_rows, x.shape[1]), np.float32)
    rc = lib.fg_oracle_spmm_dds_f32(n_rows, x.shape[0], x.shape[1], int(num_col_partitions),
                                    _p(s1_pos, _i32p), _p(s1_idx, _i32p), _p(vals, _f32p),
                                    _p(x, _f32p), _p(y, _f32p))
    if rc != 0:
        raise ValueError("fg_oracle_spmm_dds_f32: bad argument")
    return y
