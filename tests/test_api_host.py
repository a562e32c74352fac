"""Host-side behaviour of the module / op layers that needs no GPU: names, argument
checks, the reference's assertions, and loud failure where there is no device."""
import numpy as np
import pytest
import scipy.sparse as sp
import torch

import featgraph_b200 as fg
from featgraph_b200 import nd, te
from featgraph_b200 import op as ops
from featgraph_b200.module import (VanillaSDDMMcuda, VanillaSDDMMx86, VanillaSpMMcuda,
                                   VanillaSpMMx86)
from helpers import random_csr


def test_import_surface_matches_reference_names():
    fg.install_as_featgraph()
    from featgraph.module import VanillaSpMMx86 as a, VanillaSpMMcuda as b  # noqa: F401
    from featgraph.module import VanillaSDDMMx86 as c, VanillaSDDMMcuda as d  # noqa: F401
    from featgraph.util import util_convert_csr_to_dds, util_partition_adj_coo_2d  # noqa: F401
    import featgraph.op as o
    for name in ("vanilla_sddmm", "schedule_vanilla_sddmm_x86",
                 "schedule_vanilla_sddmm_cuda_tree_reduce",
                 "schedule_vanilla_sddmm_cuda_single_thread_reduce", "vanilla_spmm_csr_x86",
                 "schedule_vanilla_spmm_csr_x86", "vanilla_spmm_dds_x86",
                 "schedule_vanilla_spmm_dds_x86", "vanilla_spmm_csr_cuda",
                 "schedule_vanilla_spmm_csr_cuda"):
        assert callable(getattr(o, name))


def test_placeholder_and_ndarray_on_cpu():
    p = te.placeholder((255, 128))
    assert p.shape == (255, 128) and p.dtype == "float32"
    a = nd.array(np.arange(6, dtype=np.float32).reshape(2, 3), fg.cpu(0))
    assert a.shape == (2, 3) and a.dtype == "float32" and a.ctx == fg.cpu(0)
    np.testing.assert_array_equal(a.asnumpy(), np.arange(6, dtype=np.float32).reshape(2, 3))
    assert fg.get_const_tuple(p.shape) == (255, 128)
    assert repr(fg.gpu(0)) == "gpu(0)"


def test_spmm_op_specs_and_hints():
    out = ops.vanilla_spmm_csr_cuda(te.placeholder((255, 128)), te.placeholder((128,), "int32"),
                                    te.placeholder((3238,), "int32"), te.placeholder((3238,)))
    assert out.shape == (127, 128) and out.kind == "spmm_csr"
    s = ops.schedule_vanilla_spmm_csr_cuda(out)
    assert s.hints == {"num_cuda_blocks": 127, "num_threads_per_cuda_block": 128}
    s = ops.schedule_vanilla_spmm_csr_cuda(out, num_threads_per_cuda_block=32)
    assert s.hints["num_threads_per_cuda_block"] == 32
    with pytest.raises(AssertionError):
        ops.vanilla_spmm_csr_cuda(te.placeholder((255, 128)), te.placeholder((128,), "int32"),
                                  te.placeholder((10,), "int32"), te.placeholder((11,)))


def test_sddmm_op_specs_and_reference_assertions():
    row, col = te.placeholder((3238,), "int32"), te.placeholder((3238,), "int32")
    out = ops.vanilla_sddmm(te.placeholder((255, 128)), te.placeholder((127, 128)), row, col)
    assert out.shape == (3238,) and out.attrs["num_heads"] == 1
    ops.schedule_vanilla_sddmm_cuda_tree_reduce(out, num_cuda_blocks=256)
    ops.schedule_vanilla_sddmm_cuda_single_thread_reduce(out)
    with pytest.raises(AssertionError, match="num_cuda_blocks must be smaller"):
        ops.schedule_vanilla_sddmm_cuda_tree_reduce(out, num_cuda_blocks=4000)
    with pytest.raises(AssertionError, match="feat dimension tiling"):
        ops.schedule_vanilla_sddmm_cuda_tree_reduce(out, num_feat_partitions=4)
    with pytest.raises(AssertionError, match="dimension mismatch"):
        ops.vanilla_sddmm(te.placeholder((255, 128)), te.placeholder((127, 64)), row, col)
    mh = ops.vanilla_sddmm(te.placeholder((255, 4, 16)), te.placeholder((127, 4, 16)), row, col)
    assert mh.shape == (3238, 4) and mh.attrs == {"feat_len": 64, "num_heads": 4,
                                                  "num_feat_partitions": 1,
                                                  "msg_op": "mul", "reduce_op": "sum"}
    gen = ops.vanilla_sddmm(te.placeholder((255, 64)), te.placeholder((127, 64)), row, col,
                            msg_op="sub", reduce_op="max")
    assert (gen.attrs["msg_op"], gen.attrs["reduce_op"]) == ("sub", "max")
    with pytest.raises(ValueError, match="msg_op"):
        ops.vanilla_sddmm(te.placeholder((255, 64)), te.placeholder((127, 64)), row, col,
                          msg_op="pow")
    mh2 = ops.vanilla_sddmm(te.placeholder((255, 64)), te.placeholder((127, 64)), row, col,
                            num_heads=8)
    assert mh2.shape == (3238, 8)
    with pytest.raises(ValueError):
        ops.vanilla_sddmm(te.placeholder((255, 64)), te.placeholder((127, 64)), row, col,
                          num_heads=5)


def test_x86_names_exist_but_have_no_code_path():
    adj = random_csr(127, 255, 0.1, seed=1)
    m = VanillaSpMMx86(adj, num_col_partitions=4)        # DDS preprocessing still runs
    assert m.target == "llvm" and m._adj_s1_pos.shape == (4 * 128,)
    with pytest.raises(NotImplementedError):
        m.build([te.placeholder((255, 128))], {"num_feat_partitions": 1}, {})
    with pytest.raises(AssertionError):
        VanillaSpMMx86(adj, num_col_partitions=0)
    s = VanillaSDDMMx86(adj.tocoo(), 4, 4)
    coo = adj.tocoo()
    # edge_mapping undoes the 2-D blocking: permuted[edge_mapping] is in the caller's order
    assert np.array_equal(s._adj_row_indices[s.edge_mapping], coo.row)
    assert np.array_equal(s._adj_col_indices[s.edge_mapping], coo.col)
    with pytest.raises(NotImplementedError):
        s.build([te.placeholder((255, 128)), te.placeholder((127, 128))],
                {"num_feat_partitions": 4}, {"num_feat_partitions": 4})
    with pytest.raises(AssertionError, match="no graph partitioning"):
        VanillaSDDMMx86(adj.tocoo()).edge_mapping
    with pytest.raises(NotImplementedError):
        ops.vanilla_spmm_csr_x86(None, None, None, None)


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU failure mode")
def test_cuda_classes_fail_loudly_without_a_gpu():
    adj = random_csr(16, 16, 0.2, seed=2)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        VanillaSpMMcuda(adj)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        VanillaSDDMMcuda(adj)
    from featgraph_b200.module import PartitionedSDDMMcuda
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        PartitionedSDDMMcuda(adj, num_col_partitions=2)


def test_float64_adjacency_is_rejected_not_cast(monkeypatch):
    adj = sp.random(8, 8, density=0.5, format="csr", dtype=np.float64, random_state=0)
    with pytest.raises(TypeError, match="float32"):
        VanillaSpMMx86(adj)


def test_single_row_tile_share_of_an_edge_list():
    # the statistic the cuda module uses to choose the row-register SDDMM kernel: the share
    # of 32-edge tiles whose edges all have one row index (host side, so it runs here)
    import scipy.sparse as sp
    from featgraph_b200.module import VanillaSDDMMx86
    rows = np.repeat(np.arange(10, dtype=np.int32), 320)           # 10 rows of 320 edges
    cols = np.tile(np.arange(320, dtype=np.int32), 10)
    coo = sp.coo_matrix((np.ones(3200, np.float32), (rows, cols)), shape=(10, 320))
    assert VanillaSDDMMx86(coo)._single_row_tile_share() == 1.0
    short = sp.coo_matrix((np.ones(3200, np.float32),
                           (np.arange(3200, dtype=np.int32) // 4, cols)), shape=(800, 320))
    assert VanillaSDDMMx86(short)._single_row_tile_share() == 0.0
    order = np.random.RandomState(0).permutation(3200)             # unsorted: the general test
    shuffled = sp.coo_matrix((np.ones(3200, np.float32), (rows[order], cols[order])),
                             shape=(10, 320))
    assert VanillaSDDMMx86(shuffled)._single_row_tile_share() < 0.05
    tiny = sp.coo_matrix((np.ones(5, np.float32), (np.zeros(5, np.int32), np.arange(5, dtype=np.int32))),
                         shape=(1, 5))
    assert VanillaSDDMMx86(tiny)._single_row_tile_share() == 0.0   # no whole tile
