"""Randomised parity sweep: many small random matrices, shapes, feature lengths and row-class
thresholds per test, every result bit-equal to the CPU oracle.  Seeds are fixed, so a failure
names its case."""
import numpy as np
import pytest
import scipy.sparse as sp

from featgraph_b200 import nd, te
from featgraph_b200.module import PartitionedSDDMMcuda, VanillaSDDMMcuda, VanillaSpMMcuda
from helpers import bits, features

pytestmark = pytest.mark.gpu

FEAT_LENS = [1, 2, 5, 8, 16, 31, 32, 48, 64, 65, 96, 128, 160, 192, 256]


def _random_matrix(rs):
    """A random CSR matrix with a skewed degree distribution: some empty rows, a few rows
    far longer than the rest, unsorted column order and duplicates now and then."""
    n_rows, n_cols = int(rs.randint(1, 260)), int(rs.randint(1, 260))
    base = rs.randint(0, max(2, n_cols // 4), size=n_rows)
    base[rs.random_sample(n_rows) < 0.15] = 0
    for _ in range(int(rs.randint(0, 4))):                       # long rows
        base[rs.randint(n_rows)] = int(rs.randint(n_cols, 6 * n_cols + 2))
    rows, cols = [], []
    for r, d in enumerate(base):
        d = int(d)
        if d <= n_cols and rs.random_sample() < 0.7:
            c = np.sort(rs.choice(n_cols, d, replace=False))      # canonical row
        else:
            c = rs.randint(0, n_cols, size=d)                     # unsorted, with duplicates
        rows.append(np.full(d, r, np.int32))
        cols.append(c.astype(np.int32))
    row = np.concatenate(rows) if rows else np.zeros(0, np.int32)
    col = np.concatenate(cols) if cols else np.zeros(0, np.int32)
    val = (rs.random_sample(len(row)) * 2 - 1).astype(np.float32)
    indptr = np.concatenate([[0], np.cumsum(base)]).astype(np.int32)
    csr = sp.csr_matrix((val, col, indptr), shape=(n_rows, n_cols))   # stored order is kept
    return csr, row, col


@pytest.mark.parametrize("block", range(4))
def test_random_spmm_cases(oracle, block):
    for seed in range(block * 12, block * 12 + 12):
        rs = np.random.RandomState(1000 + seed)
        csr, _, _ = _random_matrix(rs)
        f = FEAT_LENS[rs.randint(len(FEAT_LENS))]
        thr = [0, 0, 1, 4, 8, 64][rs.randint(6)]
        x = features((csr.shape[1], f), seed=seed)
        m = VanillaSpMMcuda(csr)
        m.build([te.placeholder(x.shape)], {}, {"heavy_row_threshold": thr} if thr else {})
        y = m.run([nd.array(x, m.ctx)]).asnumpy()
        want = oracle.spmm_csr_f32(csr.indptr, csr.indices, csr.data, x, n_cols=csr.shape[1])
        assert m.device_status() == 0
        assert np.array_equal(bits(want), bits(y)), \
            "seed %d shape %r nnz %d feat_len %d threshold %d" % (seed, csr.shape, csr.nnz, f, thr)


@pytest.mark.parametrize("block", range(4))
def test_random_sddmm_cases(oracle, block):
    for seed in range(block * 12, block * 12 + 12):
        rs = np.random.RandomState(2000 + seed)
        csr, row, col = _random_matrix(rs)
        if len(row) == 0:
            continue
        heads, dim = [(1, 1), (1, 7), (1, 32), (1, 64), (1, 100), (2, 16), (4, 16), (4, 8),
                      (8, 4), (2, 32), (3, 64), (5, 3), (1, 256)][rs.randint(13)]
        shape = (heads, dim) if heads > 1 else (dim,)
        src = features((csr.shape[1],) + shape, seed=seed)
        dst = features((csr.shape[0],) + shape, seed=seed + 500)
        coo = sp.coo_matrix((np.zeros(len(row), np.float32), (row, col)), shape=csr.shape)
        parts = (int(rs.randint(1, 4)), int(rs.randint(1, 4)))
        # the reference's partitioning utility goes through tocsr(), which merges duplicate
        # edges (and their ids): blocking is only defined for duplicate-free edge lists
        no_dups = len(np.unique(row.astype(np.int64) * csr.shape[1] + col)) == len(row)
        blocked = parts != (1, 1) and no_dups and rs.random_sample() < 0.7
        m = PartitionedSDDMMcuda(coo, *parts) if blocked else VanillaSDDMMcuda(coo)
        m.build([te.placeholder(src.shape), te.placeholder(dst.shape)], {},
                {"num_cuda_blocks": min(64, len(row))})
        out = m.run([nd.array(src, m.ctx), nd.array(dst, m.ctx)]).asnumpy()
        if blocked:
            out = out[m.edge_mapping]
        want = oracle.sddmm_coo_f32(row, col, src, dst, num_heads=heads)
        assert np.array_equal(bits(want.reshape(out.shape)), bits(out)), \
            "seed %d shape %r nnz %d feat %r blocked %r" % (seed, csr.shape, len(row), shape,
                                                           parts if blocked else None)
