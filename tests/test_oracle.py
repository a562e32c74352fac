"""Pins the CPU oracle: against the fixtures that hold the reference tests' own expected
values, against scipy/numpy at the reference's tolerance, and bit for bit against an
independent pure-Python spelling of the same loop order."""
import numpy as np
import pytest

from helpers import bits, features, random_csr
from oracle import py_restatement


def test_spmm_oracle_matches_reference_test_oracle(golden, oracle):
    # tests/test_module_spmm.py:29-30 -- scipy dot, rtol = atol = 1e-4
    y = oracle.spmm_csr_f32(golden["spmm_indptr"], golden["spmm_indices"], golden["spmm_data"],
                            golden["spmm_x"])
    np.testing.assert_allclose(golden["spmm_y_scipy"], y, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("parts", [1, 4])
def test_spmm_oracle_feature_partitions_do_not_change_bits(golden, oracle, parts):
    # the x86 cases (128, 1, 1) and (128, 1, 4) of tests/test_module_spmm.py:32-34
    base = oracle.spmm_csr_f32(golden["spmm_indptr"], golden["spmm_indices"],
                               golden["spmm_data"], golden["spmm_x"])
    y = oracle.spmm_csr_f32(golden["spmm_indptr"], golden["spmm_indices"], golden["spmm_data"],
                            golden["spmm_x"], num_feat_partitions=parts)
    assert np.array_equal(bits(base), bits(y))


def test_sddmm_oracle_matches_reference_test_oracle(golden, oracle):
    # tests/test_module_sddmm.py:34-37
    out = oracle.sddmm_coo_f32(golden["sddmm_row"], golden["sddmm_col"], golden["sddmm_src"],
                               golden["sddmm_dst"])
    np.testing.assert_allclose(golden["sddmm_out_numpy"], out, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("parts,parallel", [(1, True), (4, False), (4, True)])
def test_sddmm_oracle_variants_do_not_change_bits(golden, oracle, parts, parallel):
    base = oracle.sddmm_coo_f32(golden["sddmm_row"], golden["sddmm_col"], golden["sddmm_src"],
                                golden["sddmm_dst"])
    out = oracle.sddmm_coo_f32(golden["sddmm_row"], golden["sddmm_col"], golden["sddmm_src"],
                               golden["sddmm_dst"], num_feat_partitions=parts, parallel=parallel)
    assert np.array_equal(bits(base), bits(out))


def test_spmm_oracle_bit_equal_to_python_loops(oracle):
    a = random_csr(13, 17, 0.3, seed=3, empty_rows=(2,), dense_rows=(5,))
    x = features((17, 6), seed=4)
    ref = py_restatement.spmm_csr(a.indptr, a.indices, a.data, x)
    got = oracle.spmm_csr_f32(a.indptr, a.indices, a.data, x)
    assert np.array_equal(bits(ref), bits(got))
    assert not got[2].any()          # empty row -> zeros


@pytest.mark.parametrize("heads", [1, 2, 4])
def test_sddmm_oracle_bit_equal_to_python_loops(oracle, heads):
    a = random_csr(11, 9, 0.4, seed=5).tocoo()
    src, dst = features((9, 8), seed=6), features((11, 8), seed=7)
    ref = py_restatement.sddmm_coo(a.row, a.col, src, dst, heads)
    got = oracle.sddmm_coo_f32(a.row, a.col, src, dst, num_heads=heads)
    assert ref.shape == got.shape
    assert np.array_equal(bits(ref), bits(got))


def test_multihead_oracle_is_per_head_single_head(oracle):
    a = random_csr(40, 30, 0.2, seed=8).tocoo()
    src, dst = features((30, 4, 16), seed=9), features((40, 4, 16), seed=10)
    multi = oracle.sddmm_coo_f32(a.row, a.col, src, dst, num_heads=4)
    for h in range(4):
        single = oracle.sddmm_coo_f32(a.row, a.col, np.ascontiguousarray(src[:, h]),
                                      np.ascontiguousarray(dst[:, h]))
        assert np.array_equal(bits(multi[:, h]), bits(single))


def test_oracle_close_to_fp64_truth(oracle):
    a = random_csr(64, 80, 0.25, seed=11)
    x = features((80, 32), seed=12)
    y32 = oracle.spmm_csr_f32(a.indptr, a.indices, a.data, x)
    y64 = oracle.spmm_csr_f64(a.indptr, a.indices, a.data, x)
    np.testing.assert_allclose(y32, y64, rtol=1e-5, atol=1e-5)
    c = a.tocoo()
    src, dst = features((80, 32), seed=13), features((64, 32), seed=14)
    o32 = oracle.sddmm_coo_f32(c.row, c.col, src, dst)
    o64 = oracle.sddmm_coo_f64(c.row, c.col, src, dst)
    np.testing.assert_allclose(o32, o64, rtol=1e-5, atol=1e-5)


def test_oracle_empty_inputs(oracle):
    x = features((5, 4), seed=1)
    y = oracle.spmm_csr_f32(np.zeros(4, np.int32), np.zeros(0, np.int32), np.zeros(0, np.float32), x)
    assert y.shape == (3, 4) and not y.any()
    out = oracle.sddmm_coo_f32(np.zeros(0, np.int32), np.zeros(0, np.int32), x, x)
    assert out.shape == (0,)


@pytest.mark.parametrize("msg_op", ["mul", "add", "sub", "div", "copy_lhs", "copy_rhs"])
@pytest.mark.parametrize("reduce_op", ["sum", "max", "min"])
def test_generalised_oracle_equals_its_python_restatement(oracle, msg_op, reduce_op):
    # the generalised operators are defined by the oracle itself (the reference ships only
    # multiply / sum); the C code is checked against a scalar-by-scalar Python spelling
    from oracle import py_restatement
    from helpers import features, random_csr
    adj = random_csr(23, 19, 0.3, seed=3, empty_rows=(0, 7))
    x = features((19, 8), seed=4)
    x[3, 2] = 0.0
    want = py_restatement.gspmm_csr(adj.indptr, adj.indices, adj.data, x, msg_op, reduce_op)
    got = oracle.gspmm_csr_f32(adj.indptr, adj.indices, adj.data, x, msg_op, reduce_op)
    assert np.array_equal(want.view(np.int32), got.view(np.int32))
    ident = {"sum": 0.0, "max": -np.finfo(np.float32).max, "min": np.finfo(np.float32).max}
    assert (got[0] == np.float32(ident[reduce_op])).all()          # empty row = the identity
    coo = adj.tocoo()
    dst = features((23, 8), seed=5)
    want = py_restatement.gsddmm_coo(coo.row, coo.col, x, dst, 2, msg_op, reduce_op)
    got = oracle.gsddmm_coo_f32(coo.row, coo.col, x, dst, 2, msg_op, reduce_op)
    assert np.array_equal(want.view(np.int32), got.view(np.int32))


def test_generalised_oracle_with_mul_sum_is_the_reference_kernel(oracle):
    from helpers import features, random_csr
    adj = random_csr(40, 30, 0.2, seed=6)
    x, dst = features((30, 16), seed=7), features((40, 16), seed=8)
    a = oracle.spmm_csr_f32(adj.indptr, adj.indices, adj.data, x)
    b = oracle.gspmm_csr_f32(adj.indptr, adj.indices, adj.data, x, "mul", "sum")
    assert np.array_equal(a.view(np.int32), b.view(np.int32))
    coo = adj.tocoo()
    a = oracle.sddmm_coo_f32(coo.row, coo.col, x, dst, num_heads=4)
    b = oracle.gsddmm_coo_f32(coo.row, coo.col, x, dst, 4, "mul", "sum")
    assert np.array_equal(a.view(np.int32), b.view(np.int32))


@pytest.mark.parametrize("parts", [1, 2, 4, 7])
def test_dds_oracle(oracle, parts):
    # the reference's x86 test runs the DDS op with 4 column partitions and compares with
    # scipy at 1e-4 (tests/test_module_spmm.py:12-34); the C restatement is also checked bit
    # for bit against the scalar Python spelling, and with one partition against the CSR op
    from featgraph_b200.util import util_convert_csr_to_dds
    adj = random_csr(127, 255, 0.1, seed=30 + parts, empty_rows=(0, 126))
    x = features((255, 24), seed=31)
    pos, idx, vals = util_convert_csr_to_dds(adj, parts)
    y = oracle.spmm_dds_f32(pos, idx, vals, x, 127, parts)
    np.testing.assert_allclose(adj.dot(x), y, rtol=1e-4, atol=1e-4)
    want = py_restatement.spmm_dds(pos, idx, vals, x, 127, parts)
    assert np.array_equal(want.view(np.int32), y.view(np.int32))
    if parts == 1:
        csr = oracle.spmm_csr_f32(adj.indptr, adj.indices, adj.data, x)
        assert np.array_equal(bits(csr + np.float32(0.0)), bits(y))     # 0 + sum: -0 becomes +0
