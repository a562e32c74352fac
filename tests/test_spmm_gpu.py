"""Parity of the CUDA SpMM path (module API -> C ABI -> sm_100a kernels) with the CPU
oracle.  The kernels keep the oracle's summation order, so the bar is bit-equality; the
reference's own bar (rtol = atol = 1e-4 against scipy) is asserted as well."""
import ctypes

import numpy as np
import pytest
import scipy.sparse as sp
import torch

import featgraph_b200 as fg
from featgraph_b200 import _lib, graphs, nd, te
from featgraph_b200.module import VanillaSpMMcuda
from helpers import bits, features, random_csr, row_classes

pytestmark = pytest.mark.gpu


def run_spmm(adj, x, schedule_args=None):
    m = VanillaSpMMcuda(adj)
    m.build([te.placeholder(x.shape)], {}, dict(schedule_args or {}))
    out = m.run([nd.array(x, m.ctx)])
    return m, out.asnumpy()


def oracle_spmm(oracle, adj, x):
    return oracle.spmm_csr_f32(adj.indptr, adj.indices, adj.data, x, n_cols=adj.shape[1])


@pytest.mark.parametrize("threads", [32, 128, None])
def test_reference_cuda_cases(golden, oracle, threads):
    # tests/test_module_spmm.py:37-59: 127 x 255, density 0.1, feat_len 128
    adj = sp.csr_matrix((golden["spmm_data"], golden["spmm_indices"], golden["spmm_indptr"]),
                        shape=(127, 255))
    x = golden["spmm_x"]
    _, y = run_spmm(adj, x, {"num_threads_per_cuda_block": threads})
    np.testing.assert_allclose(golden["spmm_y_scipy"], y, rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(adj.dot(x), y, rtol=1e-4, atol=1e-4)
    assert np.array_equal(bits(oracle_spmm(oracle, adj, x)), bits(y))


@pytest.mark.parametrize("feat_len", [1, 3, 32, 33, 64, 96, 100, 128, 256, 512])
@pytest.mark.parametrize("threshold", [0, 8])
def test_feature_lengths_and_both_row_paths(oracle, feat_len, threshold):
    adj = random_csr(300, 257, 0.08, seed=feat_len, empty_rows=(0, 17, 299), dense_rows=(5, 200))
    x = features((257, feat_len), seed=100 + feat_len)
    m, y = run_spmm(adj, x, {"heavy_row_threshold": threshold})
    assert np.array_equal(bits(oracle_spmm(oracle, adj, x)), bits(y))
    assert not y[[0, 17, 299]].any()
    assert m.device_status() == 0
    if feat_len % 32 == 0 and threshold == 8:
        # the giant, heavy and light kernels, once per residency slab of the features
        slab = 128 if feat_len % 128 == 0 else 64 if feat_len % 64 == 0 else 32
        assert all(n > 0 for n in row_classes(m))
        assert m.num_launches() == 3 * (feat_len // slab)


@pytest.mark.parametrize("feat_len", [32, 64, 128])
def test_giant_rows_wrap_the_stage_ring(oracle, feat_len):
    # rows of 3000 / 2500 / 1900 nonzeros with a tiny threshold take the multi-warp giant
    # kernel and go round its 32-block ring several times; ragged last blocks included
    adj = random_csr(96, 3000, 0.02, seed=77, empty_rows=(1,)).tolil()
    rs = np.random.RandomState(78)
    adj[3, :] = rs.random_sample(3000).astype(np.float32) + 0.5
    adj[40, :2500] = rs.random_sample(2500).astype(np.float32) + 0.5
    adj[41, 1100:] = rs.random_sample(1900).astype(np.float32) + 0.5
    adj = adj.tocsr().astype(np.float32)
    x = features((3000, feat_len), seed=79)
    m, y = run_spmm(adj, x, {"heavy_row_threshold": 8})
    text = m.lower_to_ir([te.placeholder(x.shape)], {}, {"heavy_row_threshold": 8})
    assert "giant: 0 rows" not in text and all(n > 0 for n in row_classes(m))
    assert m.device_status() == 0
    assert np.array_equal(bits(oracle_spmm(oracle, adj, x)), bits(y))


def test_weighted_values_are_not_fused(oracle):
    # U(0,1) values: a fused multiply-add would differ from the oracle in the last bit
    adj = random_csr(500, 400, 0.2, seed=42)
    x = features((400, 64), seed=43)
    for thr in (0, 16):
        _, y = run_spmm(adj, x, {"heavy_row_threshold": thr})
        assert np.array_equal(bits(oracle_spmm(oracle, adj, x)), bits(y))


def test_unsorted_and_duplicate_entries_keep_csr_order(oracle):
    rs = np.random.RandomState(5)
    n_rows, n_cols, per_row = 64, 50, 40
    indices = rs.randint(0, n_cols, size=n_rows * per_row).astype(np.int32)   # unsorted, repeats
    indptr = (np.arange(n_rows + 1) * per_row).astype(np.int32)
    data = rs.random_sample(n_rows * per_row).astype(np.float32)
    adj = sp.csr_matrix((data, indices, indptr), shape=(n_rows, n_cols))
    assert not adj.has_canonical_format
    x = features((n_cols, 64), seed=6)
    for thr in (0, 8):
        m = VanillaSpMMcuda(adj)
        assert np.array_equal(m._adj_indices, indices)       # structure is taken bit-exactly
        m.build([te.placeholder(x.shape)], {}, {"heavy_row_threshold": thr})
        y = m.run([nd.array(x, m.ctx)]).asnumpy()
        assert np.array_equal(bits(oracle.spmm_csr_f32(indptr, indices, data, x)), bits(y))


def test_degenerate_shapes(oracle):
    x = features((7, 32), seed=1)
    _, y = run_spmm(sp.csr_matrix((5, 7), dtype=np.float32), x)          # nnz == 0
    assert y.shape == (5, 32) and not y.any()
    one = sp.csr_matrix(np.ones((1, 7), np.float32))                     # one dense row
    _, y = run_spmm(one, x)
    assert np.array_equal(bits(oracle_spmm(oracle, one, x)), bits(y))
    _, y = run_spmm(sp.csr_matrix((0, 7), dtype=np.float32), x)          # no rows
    assert y.shape == (0, 32)


def test_non_finite_features_stay_in_their_rows(oracle):
    # column 0 is referenced by no edge: an Inf there must not leak through padded lanes
    adj = random_csr(200, 100, 0.3, seed=9).tolil()
    adj[:, 0] = 0
    adj = adj.tocsr().astype(np.float32)
    adj.eliminate_zeros()
    x = features((100, 64), seed=10)
    x[0] = np.inf
    x[7, 3] = np.nan
    for thr in (0, 8):
        _, y = run_spmm(adj, x, {"heavy_row_threshold": thr})
        assert np.array_equal(bits(oracle_spmm(oracle, adj, x)), bits(y))
        assert np.isfinite(np.delete(y, 3, axis=1)).all()


def test_run_returns_the_same_buffer_and_overwrites_it(oracle):
    adj = random_csr(100, 100, 0.1, seed=11, empty_rows=(3,))
    x1, x2 = features((100, 64), seed=12), features((100, 64), seed=13)
    m = VanillaSpMMcuda(adj)
    m.build([te.placeholder((100, 64))], {}, {})
    assert not m.out_tvm.asnumpy().any()                 # zero-filled at build
    o1 = m.run([nd.array(x1, m.ctx)])
    m.out_tvm.torch.fill_(float("nan"))
    o2 = m.run([nd.array(x2, m.ctx)])
    assert o1 is o2 is m.out_tvm
    assert np.array_equal(bits(oracle_spmm(oracle, adj, x2)), bits(o2.asnumpy()))


def test_inputs_are_checked():
    adj = random_csr(20, 30, 0.2, seed=14)
    m = VanillaSpMMcuda(adj)
    with pytest.raises(RuntimeError, match="build"):
        m.run([nd.array(features((30, 32), 1), m.ctx)])
    with pytest.raises(ValueError, match="columns"):
        m.build([te.placeholder((31, 32))], {}, {})
    m.build([te.placeholder((30, 32))], {}, {})
    with pytest.raises(ValueError, match="shape"):
        m.run([nd.array(features((30, 64), 1), m.ctx)])
    with pytest.raises(TypeError, match="dtype"):
        m.run([nd.array(np.zeros((30, 32), np.float64), m.ctx)])
    with pytest.raises(ValueError, match="lives on"):
        m.run([nd.array(features((30, 32), 1), fg.cpu(0))])
    with pytest.raises(ValueError, match="contiguous"):
        m.run([torch.zeros(32, 30, device="cuda").t()])
    y = m.run([features((30, 32), 2)])                   # numpy input is copied to the device
    assert y.shape == (20, 32)


def test_lower_to_ir_and_timing():
    g = graphs.powerlaw_graph(n=4000, nnz_target=400000, device="cuda")
    adj = g.to_scipy()
    m = VanillaSpMMcuda(adj)
    text = m.lower_to_ir([te.placeholder((4000, 64))], {}, {"num_cuda_blocks": 64})
    assert "spmm_light_kernel" in text and "heavy" in text and "num_cuda_blocks" in text
    m.build([te.placeholder((4000, 64))], {}, {})
    t = m.measure_average_time([nd.array(features((4000, 64), 3), m.ctx)], 5)
    assert 0 < t < 1.0


def test_config1_regular_graph(oracle):
    g = graphs.regular_graph(device="cuda")              # 65 536 x 65 536, 16 per row
    adj = g.to_scipy()
    assert adj.nnz == 1048576 and adj.has_sorted_indices
    x = graphs.normal_features(65536, 64, graphs.FEAT_SEED, "cuda").cpu().numpy()
    _, y = run_spmm(adj, x)
    assert np.array_equal(bits(oracle_spmm(oracle, adj, x)), bits(y))


@pytest.mark.parametrize("feat_len", [32, 64, 128, 256])
def test_powerlaw_medium(oracle, feat_len):
    g = graphs.powerlaw_graph(n=20000, nnz_target=3000000, device="cuda")
    adj = g.to_scipy()
    assert np.diff(adj.indptr).max() > 2048              # the default heavy path is exercised
    x = graphs.normal_features(20000, feat_len, graphs.FEAT_SEED, "cuda").cpu().numpy()
    m, y = run_spmm(adj, x)
    # light + heavy, and the giant class where the plan's time model makes the longest rows giant
    giant, heavy, light = row_classes(m)
    assert heavy > 0 and light > 0
    assert m.device_status() == 0          # no bounded wait in the giant kernel gave up
    assert np.array_equal(bits(oracle_spmm(oracle, adj, x)), bits(y))


@pytest.mark.parametrize("feat_len", [64, 96])
def test_rmat_graph_with_uniform_values(oracle, feat_len):
    # R-MAT (a, b, c, d) = (0.57, 0.19, 0.19, 0.05) with U(0,1) values: another degree
    # profile than Chung-Lu, and values for which a fused multiply-add would show
    g = graphs.rmat_graph(scale=17, edge_draws=1 << 21, device="cuda")
    adj = g.to_scipy()
    assert adj.nnz > 1500000 and 0 < adj.data.min() and adj.data.max() < 1
    x = graphs.normal_features(g.n_cols, feat_len, graphs.FEAT_SEED, "cuda").cpu().numpy()
    for thr in (0, 64):                    # the plan's own classes, and all three forced
        m, y = run_spmm(adj, x, {"heavy_row_threshold": thr})
        assert m.device_status() == 0
        assert np.array_equal(bits(oracle_spmm(oracle, adj, x)), bits(y))


def test_giant_kernel_gives_up_without_hanging(oracle):
    # Every wait inside the giant-row kernel is a bounded poll.  With the limit set to zero
    # the consumer warp cannot wait for its producers at all: the kernel must return, report
    # through the status word and leave NaN -- never stale values -- in the rows it gave up;
    # the next call, with the default limit, is right again and the status is clean.
    adj = random_csr(96, 3000, 0.02, seed=77, empty_rows=(1,)).tolil()
    rs = np.random.RandomState(78)
    adj[3, :] = rs.random_sample(3000).astype(np.float32) + 0.5
    adj[40, :2500] = rs.random_sample(2500).astype(np.float32) + 0.5
    adj = adj.tocsr().astype(np.float32)
    x = features((3000, 64), seed=79)
    m = VanillaSpMMcuda(adj)
    m.build([te.placeholder(x.shape)], {}, {"heavy_row_threshold": 8})
    assert "giant: 0 rows" not in m.lower_to_ir([te.placeholder(x.shape)], {},
                                                 {"heavy_row_threshold": 8})
    xd = nd.array(x, m.ctx)
    want = bits(oracle_spmm(oracle, adj, x))
    assert np.array_equal(want, bits(m.run([xd]).asnumpy())) and m.device_status() == 0
    m.set_poll_limit(0)
    y = m.run([xd]).asnumpy()              # returns: nothing spins
    with pytest.raises(_lib.FeatGraphError, match="gave up"):
        m.device_status()
    assert np.isnan(y[3]).all() and np.isnan(y[40]).all()          # the giant rows
    others = np.diff(adj.indptr) <= 128    # light and heavy rows: not the giant kernel's
    assert others.sum() == 94 and np.array_equal(want[others], bits(y)[others])
    assert m.device_status() == 0          # reported once, then cleared
    m.set_poll_limit(-1)
    assert np.array_equal(want, bits(m.run([xd]).asnumpy())) and m.device_status() == 0


def test_host_buffer_entry_point(oracle):
    adj = random_csr(300, 200, 0.1, seed=21)
    x = features((200, 64), seed=22)
    m = VanillaSpMMcuda(adj)
    m.build([te.placeholder((200, 64))], {}, {})
    y = np.empty((300, 64), np.float32)
    xs = torch.empty(200, 64, device="cuda")
    ys = torch.empty(300, 64, device="cuda")
    lib = _lib.load()
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    _lib.check(lib.fg_spmm_csr_f32_host(
        m._plan, vp(m._adj_indptr_tvm.torch), vp(m._adj_indices_tvm.torch),
        vp(m._adj_vals_tvm.torch), x.ctypes.data_as(ctypes.c_void_p),
        y.ctypes.data_as(ctypes.c_void_p), vp(xs), vp(ys),
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    assert np.array_equal(bits(oracle_spmm(oracle, adj, x)), bits(y))


# ---- full size: 232 965 vertices, ~114.6 M edges ------------------------------------------

@pytest.fixture(scope="module")
def full_graph():
    g = graphs.powerlaw_graph(device="cuda")
    assert abs(g.nnz - graphs.REDDIT_NUM_EDGES) < 0.01 * graphs.REDDIT_NUM_EDGES
    return g


@pytest.fixture(scope="module")
def full_module(full_graph):
    g = full_graph
    m = VanillaSpMMcuda(g.to_scipy())
    m.build([te.placeholder((g.n_cols, 64))], {}, {})
    return m


def test_full_size_structure_properties(full_graph, full_module):
    g, m = full_graph, full_module
    deg = (g.indptr[1:] - g.indptr[:-1]).to(torch.float32)
    # all-ones features and unit values: every output is the row's degree, exactly
    y = m.run([torch.ones(g.n_cols, 64, device="cuda")]).torch
    assert torch.equal(y, deg[:, None].expand(-1, 64))
    # indicator features: Y[r, f] counts the neighbours whose id is congruent to f mod 64
    ind = torch.zeros(g.n_cols, 64, device="cuda")
    ind[torch.arange(g.n_cols, device="cuda"), torch.arange(g.n_cols, device="cuda") % 64] = 1
    y = m.run([ind]).torch
    rows = g.coo_rows().to(torch.int64)
    want = torch.bincount(rows * 64 + (g.indices.to(torch.int64) % 64),
                          minlength=g.n_rows * 64).reshape(g.n_rows, 64).to(torch.float32)
    assert torch.equal(y, want)


@pytest.mark.parametrize("feat_len", [64, 128, 256])
def test_full_size_sampled_rows_against_oracle(full_graph, full_module, oracle, feat_len):
    # feat_len 128 and 256 get another plan on this graph than on any small one (two
    # 64-float slabs of X per L2 residency, another light / heavy boundary)
    g = full_graph
    if feat_len == 64:
        m = full_module
    else:
        m = VanillaSpMMcuda(g.to_scipy())
        m.build([te.placeholder((g.n_cols, feat_len))], {}, {})
    x = graphs.normal_features(g.n_cols, feat_len, graphs.FEAT_SEED, "cuda")
    y1 = m.run([x]).torch.clone()
    y2 = m.run([x]).torch
    assert torch.equal(y1.view(torch.int32), y2.view(torch.int32))     # run-to-run identical
    indptr = g.indptr.cpu().numpy()
    deg = np.diff(indptr)
    rng = np.random.default_rng(0)
    picks = np.unique(np.concatenate([np.argsort(deg)[-24:], rng.integers(0, g.n_rows, 3000)]))
    sub_ptr = np.concatenate(([0], np.cumsum(deg[picks]))).astype(np.int32)
    sel = np.concatenate([np.arange(indptr[r], indptr[r + 1]) for r in picks])
    sel_t = torch.from_numpy(sel).cuda()
    sub_idx = g.indices[sel_t].cpu().numpy()
    sub_val = g.vals[sel_t].cpu().numpy()
    want = oracle.spmm_csr_f32(sub_ptr, sub_idx, sub_val, x.cpu().numpy(), n_cols=g.n_cols)
    got = y1[torch.from_numpy(picks).cuda()].cpu().numpy()
    assert m.device_status() == 0
    assert np.array_equal(bits(want), bits(got))


@pytest.mark.parametrize("feat_len", [32, 64])
def test_giant_rows_of_every_tail_length(oracle, feat_len):
    # the giant kernel works in blocks of 32 nonzeros, groups of 8 blocks and a ring of 4
    # groups: rows that end anywhere within a block, a group and a round of the ring, from
    # shorter than the consumer's three-block read-ahead to many rounds
    degs = [129, 130, 159, 160, 161, 191, 192, 193, 255, 256, 257, 288, 320, 479, 480, 511, 512,
            513, 544, 767, 768, 769, 1023, 1024, 1025, 1056, 1279, 1280, 1281, 2047, 2048, 2049,
            2303, 2304, 2560, 3071, 3072, 4095, 4096, 4097, 5000, 6143, 6144, 6145]
    n_cols = 6200
    rs = np.random.RandomState(5)
    indptr = np.concatenate([[0], np.cumsum(degs)]).astype(np.int32)
    cols = np.concatenate([np.sort(rs.choice(n_cols, d, replace=False)) for d in degs])
    vals = (rs.random_sample(len(cols)) + 0.5).astype(np.float32)
    adj = sp.csr_matrix((vals, cols.astype(np.int32), indptr), shape=(len(degs), n_cols))
    x = features((n_cols, feat_len), seed=6)
    m, y = run_spmm(adj, x, {"heavy_row_threshold": 8})
    text = m.lower_to_ir([te.placeholder(x.shape)], {}, {"heavy_row_threshold": 8})
    assert "giant: %d rows" % len(degs) in text, text
    assert m.device_status() == 0
    assert np.array_equal(bits(oracle_spmm(oracle, adj, x)), bits(y))


@pytest.mark.parametrize("threshold", [0, 8])
def test_extra_outputs_receive_the_same_rows(oracle, threshold):
    # fg_spmm_csr_f32_multi: every row is stored to each listed buffer (in a multi-GPU run
    # the extra ones are peers' memory); here two more local buffers stand in for them
    adj = random_csr(300, 200, 0.08, seed=21)
    dense = np.zeros(200, bool)
    dense[::3] = True                                   # a few rows of every class
    adj = sp.vstack([adj, sp.csr_matrix(np.tile(dense, (2, 1)).astype(np.float32))]).tocsr()
    x = features((200, 96), seed=22)
    m = VanillaSpMMcuda(adj)
    m.build([te.placeholder(x.shape)], {}, {"heavy_row_threshold": threshold})
    extra = [torch.full((adj.shape[0], 96), float("nan"), device="cuda") for _ in range(2)]
    m.set_extra_outputs([e.data_ptr() for e in extra])
    y = m.run([nd.array(x, m.ctx)]).asnumpy()
    torch.cuda.synchronize()
    want = bits(oracle_spmm(oracle, adj, x))
    assert np.array_equal(want, bits(y))
    for e in extra:
        assert np.array_equal(want, bits(e.cpu().numpy()))
    with pytest.raises(_lib.FeatGraphError):
        m.set_extra_outputs([extra[0].data_ptr()] * 8)  # 1 + 8 outputs: over the limit
        m.run([nd.array(x, m.ctx)])
