"""Generalised SpMM / SDDMM (a message operator and a reducer in place of multiply and sum)
against the CPU oracle's twins, bit for bit.  The reference ships only multiply / sum
(python/featgraph/op/vanilla_spmm.py:53, 121; vanilla_sddmm.py:47), so the other operator
pairs are pinned by the oracle's own definition; every kernel class is driven: light,
heavy and giant rows (tiny thresholds), the generic kernel (odd feature length), the tile
and the generic SDDMM kernels, one head and several."""
import numpy as np
import pytest
import scipy.sparse as sp

from featgraph_b200 import nd, te
from featgraph_b200.module import VanillaSDDMMcuda, VanillaSpMMcuda
from helpers import bits, features, random_csr, row_classes

pytestmark = pytest.mark.gpu

MSG = ["mul", "add", "sub", "div", "copy_lhs", "copy_rhs"]
RED = ["sum", "max", "min"]


def _matrix():
    adj = random_csr(260, 700, 0.03, seed=61, empty_rows=(0, 100)).tolil()
    rs = np.random.RandomState(62)
    adj[7, :] = rs.random_sample(700).astype(np.float32) + 0.5        # giant with threshold 8
    adj[90, :300] = rs.random_sample(300).astype(np.float32) + 0.5
    adj[91, 5:40] = rs.random_sample(35).astype(np.float32) + 0.5
    return adj.tocsr().astype(np.float32)


@pytest.mark.parametrize("reduce_op", RED)
@pytest.mark.parametrize("msg_op", MSG)
def test_spmm_operator_pairs(oracle, msg_op, reduce_op):
    adj = _matrix()
    for feat_len, threshold in ((64, 8), (32, 0), (33, 0)):
        x = features((700, feat_len), seed=63)
        x[5, 3] = 0.0                                                # a division by zero
        m = VanillaSpMMcuda(adj)
        m.build([te.placeholder(x.shape)], {"msg_op": msg_op, "reduce_op": reduce_op},
                {"heavy_row_threshold": threshold})
        if feat_len == 64:
            assert all(n > 0 for n in row_classes(m))                # all three row classes
        y = m.run([nd.array(x, m.ctx)]).asnumpy()
        want = oracle.gspmm_csr_f32(adj.indptr, adj.indices, adj.data, x, msg_op, reduce_op)
        assert np.array_equal(bits(want), bits(y)), (feat_len, threshold)
        assert m.device_status() == 0


@pytest.mark.parametrize("reduce_op", RED)
@pytest.mark.parametrize("msg_op", MSG)
def test_sddmm_operator_pairs(oracle, msg_op, reduce_op):
    coo = random_csr(170, 140, 0.1, seed=64).tocoo()
    for shape in ((64,), (4, 16), (8, 8), (2, 64), (100,)):
        heads = shape[0] if len(shape) == 2 else 1
        src, dst = features((140,) + shape, seed=65), features((170,) + shape, seed=66)
        dst[3] = 0.0
        m = VanillaSDDMMcuda(coo)
        m.build([te.placeholder(src.shape), te.placeholder(dst.shape)],
                {"msg_op": msg_op, "reduce_op": reduce_op}, {"num_cuda_blocks": 64})
        out = m.run([nd.array(src, m.ctx), nd.array(dst, m.ctx)]).asnumpy()
        want = oracle.gsddmm_coo_f32(coo.row, coo.col, src, dst, heads, msg_op, reduce_op)
        assert np.array_equal(bits(want.reshape(out.shape)), bits(out)), shape


def test_unknown_operators_are_refused():
    adj = random_csr(20, 30, 0.2, seed=67)
    m = VanillaSpMMcuda(adj)
    with pytest.raises(ValueError, match="msg_op"):
        m.build([te.placeholder((30, 32))], {"msg_op": "pow"}, {})
    with pytest.raises(ValueError, match="reduce_op"):
        m.build([te.placeholder((30, 32))], {"reduce_op": "prod"}, {})
    from featgraph_b200 import _lib
    lib = _lib.load()
    assert lib.fg_sddmm_coo_f32_general(None, None, None, None, None, 0, 4, 4, 32, 1, 6, 0, 0,
                                        None) == 1
    assert lib.fg_sddmm_coo_f32_general(None, None, None, None, None, 0, 4, 4, 32, 1, 0, 3, 0,
                                        None) == 1


def test_the_default_pair_through_the_general_entry_point(oracle):
    import ctypes
    import torch
    from featgraph_b200 import _lib
    adj = _matrix()
    x = features((700, 64), seed=68)
    m = VanillaSpMMcuda(adj)
    m.build([te.placeholder(x.shape)], {}, {"heavy_row_threshold": 8})
    want = m.run([nd.array(x, m.ctx)]).asnumpy()
    y = torch.full((260, 64), float("nan"), device="cuda")
    xd = torch.from_numpy(x).cuda()
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    _lib.check(_lib.load().fg_spmm_csr_f32_general(
        m._plan, vp(m._adj_indptr_tvm.torch), vp(m._adj_indices_tvm.torch),
        vp(m._adj_vals_tvm.torch), vp(xd), vp(y), 0, 0,
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    torch.cuda.synchronize()
    assert np.array_equal(bits(want), bits(y.cpu().numpy()))
    assert np.array_equal(bits(oracle.spmm_csr_f32(adj.indptr, adj.indices, adj.data, x)),
                          bits(want))
