"""SpMM over the DDS form (1-D source-vertex partitioning) on the GPU against the CPU
restatement of vanilla_spmm_dds_x86 (python/featgraph/op/vanilla_spmm.py:149-246): a
partial sum per column block in stored order, the blocks added in ascending order.  The
bar is bit-equality with that order; the reference's own bar for this op (rtol = atol =
1e-4 against scipy, tests/test_module_spmm.py:12-34) is asserted as well."""
import numpy as np
import pytest
import scipy.sparse as sp

from featgraph_b200 import graphs, nd, te
from featgraph_b200.module import VanillaSpMMcuda
from featgraph_b200.util import util_convert_csr_to_dds
from helpers import bits, features, random_csr

pytestmark = pytest.mark.gpu


def run_dds(adj, x, parts):
    m = VanillaSpMMcuda(adj, num_col_partitions=parts)
    m.build([te.placeholder(x.shape)], {}, {})
    return m, m.run([nd.array(x, m.ctx)]).asnumpy()


def oracle_dds(oracle, adj, x, parts):
    pos, idx, vals = util_convert_csr_to_dds(adj, parts)
    return oracle.spmm_dds_f32(pos, idx, vals, x, adj.shape[0], parts)


def test_reference_x86_case_on_the_gpu(golden, oracle):
    # tests/test_module_spmm.py:12-34: 127 x 255, density 0.1, feat_len 128, 4 column
    # partitions (its feature partitioning only re-lays the arrays out)
    adj = sp.csr_matrix((golden["spmm_data"], golden["spmm_indices"], golden["spmm_indptr"]),
                        shape=(127, 255))
    x = golden["spmm_x"]
    m, y = run_dds(adj, x, 4)
    np.testing.assert_allclose(golden["spmm_y_scipy"], y, rtol=1e-4, atol=1e-4)
    assert np.array_equal(bits(oracle_dds(oracle, adj, x, 4)), bits(y))
    assert m.device_status() == 0
    assert "4 column blocks" in m.lower_to_ir([te.placeholder(x.shape)], {}, {})


@pytest.mark.parametrize("parts", [2, 3, 8, 300])
@pytest.mark.parametrize("feat_len", [1, 32, 64, 100, 256])
def test_partitions_and_feature_lengths(oracle, parts, feat_len):
    # 257 columns: a ragged last block for every partition count; 300 partitions leave
    # blocks of one column and empty ones at the end
    adj = random_csr(300, 257, 0.08, seed=feat_len, empty_rows=(0, 17, 299), dense_rows=(5, 200))
    x = features((257, feat_len), seed=100 + feat_len)
    m, y = run_dds(adj, x, parts)
    assert np.array_equal(bits(oracle_dds(oracle, adj, x, parts)), bits(y))
    np.testing.assert_allclose(adj.dot(x), y, rtol=1e-4, atol=1e-4)
    assert not y[[0, 17, 299]].any()
    assert m.device_status() == 0


def test_long_rows_take_the_heavy_and_giant_kernels_in_every_block(oracle):
    # a power-law graph whose longest rows pass the class boundaries inside each block
    adj = graphs.powerlaw_graph(20000, 1_500_000, seed=5).to_scipy()
    x = features((20000, 64), seed=6)
    m, y = run_dds(adj, x, 2)
    assert np.array_equal(bits(oracle_dds(oracle, adj, x, 2)), bits(y))
    assert m.num_launches() >= 4
    assert m.device_status() == 0


def test_second_call_does_not_add_to_the_first(oracle):
    adj = random_csr(200, 300, 0.05, seed=9)
    x = features((300, 64), seed=10)
    m, y1 = run_dds(adj, x, 4)
    y2 = m.run([nd.array(x, m.ctx)]).asnumpy()
    assert np.array_equal(bits(y1), bits(y2))


def test_one_partition_is_the_csr_op(oracle):
    adj = random_csr(200, 300, 0.05, seed=11)
    x = features((300, 64), seed=12)
    m = VanillaSpMMcuda(adj, num_col_partitions=1)
    m.build([te.placeholder(x.shape)], {}, {})
    y = m.run([nd.array(x, m.ctx)]).asnumpy()
    want = oracle.spmm_csr_f32(adj.indptr, adj.indices, adj.data, x, n_cols=300)
    assert np.array_equal(bits(want), bits(y))


def test_unsupported_combinations_raise():
    adj = random_csr(50, 60, 0.1, seed=13)
    m = VanillaSpMMcuda(adj, num_col_partitions=2)
    with pytest.raises(TypeError):
        m.build([te.placeholder((60, 32))], {"msg_op": "add"}, {})
    m.build([te.placeholder((60, 32))], {}, {})
    with pytest.raises(NotImplementedError):
        m.set_poll_limit(3)
