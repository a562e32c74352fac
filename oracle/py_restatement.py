"""Pure-Python restatement of the same loops, for tiny cases only.

TEST INFRASTRUCTURE.  A second, independent spelling of the summation order
documented in fg_oracle.c (np.float32 scalars, one operation at a time) that
the tests use to check the C oracle bit for bit.
"""
import numpy as np


def spmm_csr(indptr, indices, vals, x):
    """vanilla_spmm.py:46-56 with the loop order of :73 -- e ascending per row."""
    n_rows, f = len(indptr) - 1, x.shape[1]
    y = np.zeros((n_rows, f), np.float32)
    for r in range(n_rows):
        for e in range(indptr[r], indptr[r + 1]):
            v = np.float32(vals[e])
            for k in range(f):
                prod = np.float32(v * np.float32(x[indices[e], k]))
                y[r, k] = np.float32(y[r, k] + prod)
    return y


def sddmm_coo(row, col, src, dst, num_heads=1):
    """vanilla_sddmm.py:43-47 -- k ascending per edge (per head)."""
    nnz, f = len(row), src.shape[1]
    d = f // num_heads
    out = np.zeros((nnz, num_heads), np.float32)
    for e in range(nnz):
        for h in range(num_heads):
            acc = np.float32(0.0)
            for k in range(h * d, (h + 1) * d):
                prod = np.float32(np.float32(src[col[e], k]) * np.float32(dst[row[e], k]))
                acc = np.float32(acc + prod)
            out[e, h] = acc
    return out.reshape(nnz) if num_heads == 1 else out


_F32_MAX = np.finfo(np.float32).max


def _msg(op, lhs, rhs):
    with np.errstate(all="ignore"):
        return {"mul": lambda: np.float32(lhs * rhs), "add": lambda: np.float32(lhs + rhs),
                "sub": lambda: np.float32(lhs - rhs), "div": lambda: np.float32(lhs / rhs),
                "copy_lhs": lambda: lhs, "copy_rhs": lambda: rhs}[op]()


def _reduce(op, acc, m):
    if op == "sum":
        return np.float32(acc + m)
    if op == "max":
        return m if m > acc else acc
    return m if m < acc else acc


def _identity(op):
    return np.float32({"sum": 0.0, "max": -_F32_MAX, "min": _F32_MAX}[op])


def gspmm_csr(indptr, indices, vals, x, msg_op, reduce_op):
    """The generalised SpMM of fg_oracle.c, one scalar operation at a time."""
    n_rows, f = len(indptr) - 1, x.shape[1]
    y = np.full((n_rows, f), _identity(reduce_op), np.float32)
    for r in range(n_rows):
        for e in range(indptr[r], indptr[r + 1]):
            for k in range(f):
                m = _msg(msg_op, np.float32(x[indices[e], k]), np.float32(vals[e]))
                y[r, k] = _reduce(reduce_op, y[r, k], m)
    return y


def gsddmm_coo(row, col, src, dst, num_heads, msg_op, reduce_op):
    nnz, f = len(row), src.shape[1]
    d = f // num_heads
    out = np.zeros((nnz, num_heads), np.float32)
    for e in range(nnz):
        for h in range(num_heads):
            acc = _identity(reduce_op)
            for k in range(h * d, (h + 1) * d):
                acc = _reduce(reduce_op, acc, _msg(msg_op, np.float32(src[col[e], k]),
                                                   np.float32(dst[row[e], k])))
            out[e, h] = acc
    return out.reshape(nnz) if num_heads == 1 else out


def spmm_dds(s1_pos, s1_idx, vals, x, n_rows, num_col_partitions):
    """vanilla_spmm.py:201-218: a partial sum per (column block, row), then the blocks'
    partial sums added in ascending block order, both from an accumulator of 0."""
    n_cols, f = x.shape
    width = -(-n_cols // num_col_partitions)
    y = np.zeros((n_rows, f), np.float32)
    for r in range(n_rows):
        for k in range(f):
            total = np.float32(0.0)
            for p in range(num_col_partitions):
                acc = np.float32(0.0)
                for e in range(s1_pos[p * (n_rows + 1) + r], s1_pos[p * (n_rows + 1) + r + 1]):
                    prod = np.float32(np.float32(vals[e]) * np.float32(x[s1_idx[e] + p * width, k]))
                    acc = np.float32(acc + prod)
                total = np.float32(total + acc)
            y[r, k] = total
    return y
