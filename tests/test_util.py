"""Known-answer tests of the partitioning utilities: the vectors of the reference's
tests/test_util.py and fixtures produced by running the reference's own functions."""
import numpy as np
import scipy.sparse as sp

from featgraph_b200.util import util_convert_csr_to_dds, util_partition_adj_coo_2d


def _sample():
    row = np.array([0, 0, 0, 0, 1, 1, 2, 3, 4])
    col = np.array([0, 1, 2, 3, 0, 2, 1, 3, 2])
    ids = np.arange(1, 10)
    m = sp.coo_matrix((ids, (row, col)), shape=(5, 5), dtype="int32")
    dense = np.array([[1, 2, 3, 4, 0], [5, 0, 6, 0, 0], [0, 7, 0, 0, 0], [0, 0, 0, 8, 0],
                      [0, 0, 9, 0, 0]])
    np.testing.assert_array_equal(dense, m.toarray())
    return m


def test_util_convert_csr_to_dds():
    # expected vectors: tests/test_util.py:22-24
    s1_pos, s1_idx, vals = util_convert_csr_to_dds(_sample().tocsr(), 2)
    np.testing.assert_array_equal(vals, [1, 2, 3, 5, 6, 7, 9, 4, 8])
    np.testing.assert_array_equal(s1_idx, [0, 1, 2, 0, 2, 1, 2, 0, 0])
    np.testing.assert_array_equal(s1_pos, [0, 3, 5, 6, 6, 7, 7, 8, 8, 8, 9, 9])


def test_util_partition_adj_coo_2d():
    # expected vector: tests/test_util.py:43
    m = _sample()
    ids, rows, cols = util_partition_adj_coo_2d(m, 2, 2)
    np.testing.assert_array_equal(ids, [1, 2, 3, 5, 6, 7, 4, 9, 8])
    np.testing.assert_array_equal(m.data, np.arange(1, 10))      # the documented side effect
    np.testing.assert_array_equal(rows[np.argsort(ids)], m.row)
    np.testing.assert_array_equal(cols[np.argsort(ids)], m.col)


def _golden_adj(golden):
    return sp.csr_matrix((golden["spmm_data"], golden["spmm_indices"], golden["spmm_indptr"]),
                         shape=(127, 255))


def test_dds_matches_reference_outputs(golden):
    adj = _golden_adj(golden)
    for tag, parts in (("p2", 2), ("p4", 4), ("p7", 7)):
        pos, idx, vals = util_convert_csr_to_dds(adj, parts)
        for name, got in (("pos", pos), ("idx", idx), ("vals", vals)):
            want = golden["dds_%s_%s" % (tag, name)]
            assert got.dtype == want.dtype
            np.testing.assert_array_equal(got, want)


def test_partition_2d_matches_reference_outputs(golden):
    adj = _golden_adj(golden)
    for tag, (rp, cp) in (("2x2", (2, 2)), ("4x4", (4, 4)), ("3x5", (3, 5))):
        ids, rows, cols = util_partition_adj_coo_2d(adj.tocoo(), rp, cp)
        for name, got in (("ids", ids), ("rows", rows), ("cols", cols)):
            want = golden["p2d_%s_%s" % (tag, name)]
            assert got.dtype == want.dtype
            np.testing.assert_array_equal(got, want)


def test_more_partitions_than_columns():
    m = _sample().tocsr().astype("float32")
    pos, idx, vals = util_convert_csr_to_dds(m, 8)
    assert pos.shape == (8 * 6,) and idx.shape == (9,) and vals.shape == (9,)
    assert pos[-1] == 9
