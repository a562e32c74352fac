"""Small seeded input builders shared by the tests."""
import numpy as np
import scipy.sparse as sp


def random_csr(n_rows, n_cols, density, seed, empty_rows=(), dense_rows=()):
    rs = np.random.RandomState(seed)
    a = sp.random(n_rows, n_cols, density=density, format="lil", random_state=rs,
                  dtype=np.float32)
    for r in dense_rows:
        a[r, :] = rs.random_sample(n_cols).astype(np.float32) + 0.5
    for r in empty_rows:
        a[r, :] = 0
    a = a.tocsr().astype(np.float32)
    a.eliminate_zeros()
    a.sort_indices()
    return a


def features(shape, seed):
    return np.random.default_rng(seed).standard_normal(shape, dtype=np.float32)


def bits(a):
    """float32 results as int32 bit patterns, so that comparisons are bit-exact.  NaNs are
    mapped to one pattern: the payload of a propagated NaN differs between x86 (keeps the
    operand's) and the GPU (canonical NaN) and carries no information."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    out = a.view(np.int32).copy()
    out[np.isnan(a)] = 0x7FC00000
    return out


def row_classes(spmm_module):
    """(giant, heavy, light) row counts of a built SpMM module's plan."""
    import re
    text = spmm_module.describe()
    return tuple(int(re.search(r"%s: (\d+) rows" % k, text).group(1))
                 for k in ("giant", "heavy", "light"))
