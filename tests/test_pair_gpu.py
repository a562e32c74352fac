"""An SpMM and an SDDMM that do not depend on each other, chained into one stream by
programmatic dependent launches (fg_next_launch_options), and the options one by one: the
SpMM cut into its giant rows and the rest, an SDDMM with a bounded grid.  Each result must
equal what the plain calls give and the oracle, bit for bit, however the kernels overlap."""
import ctypes

import numpy as np
import pytest
import scipy.sparse as sp
import torch

from featgraph_b200 import _lib, graphs, nd, te
from featgraph_b200.distributed import OverlappedPair, ShardedSDDMM, ShardedSpMM
from featgraph_b200.module import VanillaSDDMMcuda, VanillaSpMMcuda
from helpers import bits, features, random_csr, row_classes

pytestmark = pytest.mark.gpu


def test_pair_on_one_gpu_equals_the_plain_calls(oracle):
    g = graphs.powerlaw_graph(n=30000, nnz_target=5000000, device="cuda")
    adj = g.to_scipy()
    dev = torch.device("cuda", 0)
    x = graphs.normal_features(g.n_cols, 64, graphs.FEAT_SEED, dev)
    y2 = graphs.normal_features(g.n_cols, 64, graphs.FEAT2_SEED, dev)
    spmm = ShardedSpMM(adj, 64, dev)
    sddmm = ShardedSDDMM(g.coo_rows(), g.indices, g.n_rows, g.n_cols, 64, dev)
    assert all(n > 0 for n in row_classes(spmm.module))    # giant rows exist: all phases run
    want_y = oracle.spmm_csr_f32(adj.indptr, adj.indices, adj.data, x.cpu().numpy())
    want_o = oracle.sddmm_coo_f32(g.coo_rows().cpu().numpy(), g.indices.cpu().numpy(),
                                  y2.cpu().numpy(), x.cpu().numpy(), parallel=True)
    # "chain": the SpMM, then the SDDMM behind it; "split": the SpMM's long rows, the SDDMM,
    # the SpMM's light rows
    for order in ("chain", "split"):
        pair = OverlappedPair(spmm, sddmm, order=order)
        assert pair.chained
        for _ in range(3):                                 # overlapping changes nothing
            spmm.out.fill_(float("nan"))
            sddmm.out.fill_(float("nan"))
            y, out = pair.run(x, y2, x)
        torch.cuda.synchronize()
        assert np.array_equal(bits(want_y), bits(y.cpu().numpy())), order
        assert np.array_equal(bits(want_o), bits(out.cpu().numpy())), order
        assert spmm.device_status() == 0


def test_spmm_in_two_phases_and_bounded_sddmm_grids(oracle):
    adj = random_csr(96, 3000, 0.02, seed=77, empty_rows=(1,)).tolil()
    rs = np.random.RandomState(78)
    adj[3, :] = rs.random_sample(3000).astype(np.float32) + 0.5
    adj[40, :2500] = rs.random_sample(2500).astype(np.float32) + 0.5
    adj = adj.tocsr().astype(np.float32)
    giant = np.diff(adj.indptr) > 128
    for feat_len, threshold in ((64, 8), (33, 0)):          # row classes / the generic kernel
        x = features((3000, feat_len), seed=79)
        want = bits(oracle.spmm_csr_f32(adj.indptr, adj.indices, adj.data, x))
        m = VanillaSpMMcuda(adj)
        m.build([te.placeholder(x.shape)], {}, {"heavy_row_threshold": threshold})
        xd = nd.array(x, m.ctx)
        m.out_tvm.torch.fill_(float("nan"))
        y = m.run([xd], launch_flags=_lib.SPMM_GIANT_ROWS_ONLY).asnumpy()
        if feat_len == 64:
            assert np.array_equal(want[giant], bits(y)[giant]) and np.isnan(y[~giant]).all()
        else:
            assert np.isnan(y).all()                         # the generic kernel has no classes
        y = m.run([xd], launch_flags=_lib.SPMM_SKIP_GIANT_ROWS | _lib.LAUNCH_PROGRAMMATIC).asnumpy()
        assert np.array_equal(want, bits(y))
        # the same cut one class further down: giant and heavy rows, then the light rows
        long_rows = np.diff(adj.indptr) > max(threshold, 1) if feat_len == 64 else giant & False
        m.out_tvm.torch.fill_(float("nan"))
        y = m.run([xd], launch_flags=_lib.SPMM_LONG_ROWS_ONLY).asnumpy()
        assert np.array_equal(want[long_rows], bits(y)[long_rows]) and np.isnan(y[~long_rows]).all()
        y = m.run([xd], launch_flags=_lib.SPMM_SKIP_LONG_ROWS | _lib.LAUNCH_PROGRAMMATIC).asnumpy()
        assert np.array_equal(want, bits(y))
    coo = random_csr(700, 600, 0.05, seed=80).tocoo()
    src, dst = features((600, 4, 16), seed=81), features((700, 4, 16), seed=82)
    want = oracle.sddmm_coo_f32(coo.row, coo.col, src, dst, num_heads=4)
    s = VanillaSDDMMcuda(coo)
    s.build([te.placeholder(src.shape), te.placeholder(dst.shape)], {}, {"num_cuda_blocks": 64})
    for max_ctas in (1, 3, 7, 1000):
        s.out_tvm.torch.fill_(float("nan"))
        out = s.run([nd.array(src, s.ctx), nd.array(dst, s.ctx)],
                    launch_flags=_lib.LAUNCH_PROGRAMMATIC, max_ctas=max_ctas).asnumpy()
        assert np.array_equal(bits(want), bits(out)), max_ctas
    lib = _lib.load()
    assert lib.fg_next_launch_options(1 << 20, 0) == 1 and lib.fg_next_launch_options(6, 0) == 1
    assert lib.fg_next_launch_options(16 | 32, 0) == 1 and lib.fg_next_launch_options(2 | 32, 0) == 1
    assert lib.fg_next_launch_options(0, -1) == 1
    assert lib.fg_next_launch_options(1, 5) == 0 and lib.fg_next_launch_options(0, 0) == 0
