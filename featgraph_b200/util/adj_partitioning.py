"""Host-side adjacency re-orderings with the semantics of
python/featgraph/util/adj_partitioning.py, written as single vectorised passes
(one stable sort) instead of one scipy slice per partition.
"""
import numpy as np


def _ceil_div(a, b):
    return (a + b - 1) // b


def util_convert_csr_to_dds(adj_scipy_csr, num_col_partitions):
    """CSR -> dense-dense-sparse: split the columns into ``num_col_partitions`` equal
    blocks of ceil(num_cols / P) (the last one takes the remainder) and store the blocks
    one after the other, each in CSR order with block-local column indices.

    Same result as util_convert_csr_to_dds (adj_partitioning.py:7-57).

    Returns
    -------
    s1_pos : (P * (num_rows + 1),) row pointers of every block, offset into the arrays below
    s1_idx : (nnz,) block-local column indices
    vals   : (nnz,) values
    with the dtypes of the input's indptr / indices / data.
    """
    num_rows, num_cols = adj_scipy_csr.shape
    indptr, indices, data = adj_scipy_csr.indptr, adj_scipy_csr.indices, adj_scipy_csr.data
    P = int(num_col_partitions)
    width = max(_ceil_div(num_cols, P), 1)
    nnz = indices.shape[0]

    block = (indices // width).astype(np.int64)           # column block of every entry
    rows = np.repeat(np.arange(num_rows, dtype=np.int64), np.diff(indptr))
    order = np.argsort(block, kind="stable")              # CSR order survives inside a block

    s1_idx = (indices[order] - (block[order] * width).astype(indices.dtype)).astype(indices.dtype)
    vals = data[order]

    counts = np.bincount(block * num_rows + rows, minlength=P * num_rows).reshape(P, num_rows)
    block_start = np.concatenate(([0], np.cumsum(counts.sum(axis=1))[:-1]))
    s1_pos = np.zeros((P, num_rows + 1), dtype=np.int64)
    np.cumsum(counts, axis=1, out=s1_pos[:, 1:])
    s1_pos += block_start[:, None]
    assert s1_idx.shape[0] == nnz and vals.shape[0] == nnz
    return s1_pos.reshape(-1).astype(indptr.dtype), s1_idx, vals


def util_partition_adj_coo_2d(adj_scipy_coo, num_row_partitions, num_col_partitions):
    """2-D blocking of a COO edge list: edges are regrouped block by block (row blocks
    outer, column blocks inner, block sizes ceil(n / parts)), row-major inside a block.

    Same result as util_partition_adj_coo_2d (adj_partitioning.py:60-128), including its
    two side effects: the argument's ``data`` is overwritten with the edge ids 1..nnz
    (:92), and the trip through CSR (:95) merges duplicate (row, col) entries, summing
    their ids and leaving the tail of the returned arrays zero.

    Returns (edge_id_list, row_indices, col_indices) after partitioning, each of length nnz.
    """
    num_rows, num_cols = adj_scipy_coo.shape
    row_in, col_in = adj_scipy_coo.row, adj_scipy_coo.col
    nnz = row_in.shape[0]
    assert col_in.shape[0] == nnz, \
        "length of adj_row_indices and that of adj_col_indices do not match"
    adj_scipy_coo.data = np.arange(1, 1 + nnz, dtype="int32")

    csr = adj_scipy_coo.tocsr()
    rows = np.repeat(np.arange(num_rows, dtype=np.int64), np.diff(csr.indptr))
    cols = csr.indices.astype(np.int64)
    rows_per = max(_ceil_div(num_rows, int(num_row_partitions)), 1)
    cols_per = max(_ceil_div(num_cols, int(num_col_partitions)), 1)
    block = (rows // rows_per) * int(num_col_partitions) + cols // cols_per
    order = np.argsort(block, kind="stable")              # csr is row-major already

    m = order.shape[0]
    edge_ids = np.zeros(nnz, dtype=adj_scipy_coo.data.dtype)
    row_out = np.zeros(nnz, dtype=row_in.dtype)
    col_out = np.zeros(nnz, dtype=col_in.dtype)
    edge_ids[:m] = csr.data[order]
    row_out[:m] = rows[order]
    col_out[:m] = cols[order]
    return edge_ids, row_out, col_out
