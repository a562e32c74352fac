"""Parity of the CUDA SDDMM path (single- and multi-head) with the CPU oracle: bit-equal,
plus the reference's own check against numpy at rtol = atol = 1e-4."""
import ctypes

import numpy as np
import pytest
import scipy.sparse as sp
import torch

import featgraph_b200 as fg
from featgraph_b200 import _lib, graphs, nd, te
from featgraph_b200.module import VanillaSDDMMcuda
from helpers import bits, features, random_csr

pytestmark = pytest.mark.gpu


def run_sddmm(adj, src, dst, compute_args=None, schedule_args=None):
    m = VanillaSDDMMcuda(adj)
    if schedule_args is None:            # the reference requires num_cuda_blocks <= nnz
        schedule_args = {"num_cuda_blocks": min(8192, adj.nnz)}
    m.build([te.placeholder(src.shape), te.placeholder(dst.shape)], dict(compute_args or {}),
            dict(schedule_args))
    out = m.run([nd.array(src, m.ctx), nd.array(dst, m.ctx)])
    return m, out.asnumpy()


@pytest.mark.parametrize("blocks", [32, 256])
def test_reference_cuda_cases(golden, oracle, blocks):
    # tests/test_module_sddmm.py:45-70: 127 x 255, density 0.1, feat_len 128; the adjacency
    # is cast to int32 there (values become 0 and are never read)
    coo = sp.coo_matrix((np.zeros(len(golden["sddmm_row"]), np.int32),
                         (golden["sddmm_row"], golden["sddmm_col"])), shape=(127, 255))
    src, dst = golden["sddmm_src"], golden["sddmm_dst"]
    _, out = run_sddmm(coo, src, dst, {}, {"num_cuda_blocks": blocks})
    np.testing.assert_allclose(golden["sddmm_out_numpy"], out, rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose((src[coo.col] * dst[coo.row]).sum(axis=-1), out, rtol=1e-4,
                               atol=1e-4)
    assert np.array_equal(bits(oracle.sddmm_coo_f32(coo.row, coo.col, src, dst)), bits(out))


def test_reference_assertions_survive():
    coo = random_csr(20, 30, 0.2, seed=1).tocoo()
    m = VanillaSDDMMcuda(coo)
    with pytest.raises(AssertionError, match="num_cuda_blocks must be smaller"):
        m.build([te.placeholder((30, 32)), te.placeholder((20, 32))], {},
                {"num_cuda_blocks": coo.nnz + 1})
    with pytest.raises(AssertionError, match="no graph partitioning on cuda"):
        m.edge_mapping


@pytest.mark.parametrize("feat_len", [1, 3, 16, 32, 33, 64, 96, 100, 128, 256, 512])
def test_feature_lengths(oracle, feat_len):
    coo = random_csr(150, 130, 0.1, seed=feat_len).tocoo()
    src, dst = features((130, feat_len), seed=1), features((150, feat_len), seed=2)
    _, out = run_sddmm(coo, src, dst)
    assert out.shape == (coo.nnz,)
    assert np.array_equal(bits(oracle.sddmm_coo_f32(coo.row, coo.col, src, dst)), bits(out))


def test_edge_order_is_preserved(oracle):
    coo = random_csr(90, 70, 0.15, seed=3).tocoo()
    perm = np.random.default_rng(4).permutation(coo.nnz)
    shuffled = sp.coo_matrix((coo.data[perm], (coo.row[perm], coo.col[perm])), shape=coo.shape)
    src, dst = features((70, 64), seed=5), features((90, 64), seed=6)
    m, out = run_sddmm(shuffled, src, dst)
    assert np.array_equal(m._adj_row_indices, coo.row[perm])
    assert np.array_equal(bits(oracle.sddmm_coo_f32(coo.row[perm], coo.col[perm], src, dst)),
                          bits(out))
    # duplicate edges are separate outputs
    dup = sp.coo_matrix((np.ones(4, np.float32), ([1, 1, 1, 2], [3, 3, 3, 0])), shape=(90, 70))
    _, out = run_sddmm(dup, src, dst)
    assert out.shape == (4,) and out[0] == out[1] == out[2]


def test_csr_input_is_converted_row_major(oracle):
    csr = random_csr(60, 80, 0.1, seed=7)
    coo = csr.tocoo()
    src, dst = features((80, 32), seed=8), features((60, 32), seed=9)
    _, out = run_sddmm(csr, src, dst)
    assert np.array_equal(bits(oracle.sddmm_coo_f32(coo.row, coo.col, src, dst)), bits(out))


@pytest.mark.parametrize("heads,dim", [(4, 16), (8, 32), (16, 64), (2, 8), (8, 4), (2, 128),
                                       (3, 5), (1, 64), (5, 32)])
def test_multi_head(oracle, heads, dim):
    coo = random_csr(120, 110, 0.1, seed=heads * 100 + dim).tocoo()
    src = features((110, heads, dim), seed=10)
    dst = features((120, heads, dim), seed=11)
    want = oracle.sddmm_coo_f32(coo.row, coo.col, src, dst, num_heads=heads)
    want = want.reshape(coo.nnz, heads)
    _, out = run_sddmm(coo, src, dst)                                   # 3-D placeholders
    assert out.shape == (coo.nnz, heads)
    assert np.array_equal(bits(want), bits(out))
    _, out2 = run_sddmm(coo, src.reshape(110, -1), dst.reshape(120, -1),
                        {"num_heads": heads})                           # 2-D + num_heads
    assert np.array_equal(bits(want), bits(out2.reshape(coo.nnz, heads)))


def test_degenerate_shapes():
    src, dst = features((7, 32), seed=1), features((5, 32), seed=2)
    m = VanillaSDDMMcuda(sp.coo_matrix((5, 7), dtype=np.float32))       # nnz == 0
    m.build([te.placeholder((7, 32)), te.placeholder((5, 32))], {}, {"num_cuda_blocks": 0})
    assert m.run([nd.array(src, m.ctx), nd.array(dst, m.ctx)]).asnumpy().shape == (0,)


def test_run_returns_the_same_buffer_and_overwrites_it(oracle):
    coo = random_csr(100, 100, 0.1, seed=11).tocoo()
    src, dst = features((100, 64), seed=12), features((100, 64), seed=13)
    m = VanillaSDDMMcuda(coo)
    m.build([te.placeholder((100, 64)), te.placeholder((100, 64))], {}, {"num_cuda_blocks": 64})
    assert not m.out_tvm.asnumpy().any()
    o1 = m.run([nd.array(src, m.ctx), nd.array(dst, m.ctx)])
    m.out_tvm.torch.fill_(float("nan"))
    o2 = m.run([nd.array(src, m.ctx), nd.array(dst, m.ctx)])
    assert o1 is o2 is m.out_tvm
    assert np.array_equal(bits(oracle.sddmm_coo_f32(coo.row, coo.col, src, dst)),
                          bits(o2.asnumpy()))
    t = m.measure_average_time([nd.array(src, m.ctx), nd.array(dst, m.ctx)], 5)
    assert 0 < t < 1.0
    assert "sddmm_tile_kernel" in m.lower_to_ir(
        [te.placeholder((100, 64)), te.placeholder((100, 64))], {}, {"num_cuda_blocks": 64})


def test_inputs_are_checked():
    coo = random_csr(20, 30, 0.2, seed=14).tocoo()
    m = VanillaSDDMMcuda(coo)
    with pytest.raises(ValueError, match="indexed by col"):
        m.build([te.placeholder((20, 32)), te.placeholder((20, 32))], {}, {"num_cuda_blocks": 8})
    m.build([te.placeholder((30, 32)), te.placeholder((20, 32))], {}, {"num_cuda_blocks": 8})
    good_s, good_d = features((30, 32), 1), features((20, 32), 2)
    with pytest.raises(ValueError, match="shape"):
        m.run([nd.array(good_d, m.ctx), nd.array(good_s, m.ctx)])        # swapped operands
    with pytest.raises(ValueError, match="two input"):
        m.run([nd.array(good_s, m.ctx)])
    with pytest.raises(ValueError, match="lives on"):
        m.run([nd.array(good_s, fg.cpu(0)), nd.array(good_d, m.ctx)])


def test_host_buffer_entry_point(oracle):
    coo = random_csr(300, 200, 0.1, seed=21).tocoo()
    src, dst = features((200, 64), seed=22), features((300, 64), seed=23)
    m = VanillaSDDMMcuda(coo)
    out = np.empty(coo.nnz, np.float32)
    ss, ds = torch.empty(200, 64, device="cuda"), torch.empty(300, 64, device="cuda")
    os_ = torch.empty(coo.nnz, device="cuda")
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    hp = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    _lib.check(_lib.load().fg_sddmm_coo_f32_host(
        vp(m._adj_row_indices_tvm.torch), vp(m._adj_col_indices_tvm.torch), hp(src), hp(dst),
        hp(out), vp(ss), vp(ds), vp(os_), coo.nnz, 300, 200, 64, 1, 0,
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    assert np.array_equal(bits(oracle.sddmm_coo_f32(coo.row, coo.col, src, dst)), bits(out))


def test_powerlaw_medium(oracle):
    g = graphs.powerlaw_graph(n=20000, nnz_target=3000000, device="cuda")
    coo = g.to_scipy().tocoo()
    src = graphs.normal_features(20000, 64, graphs.FEAT2_SEED, "cuda").cpu().numpy()
    dst = graphs.normal_features(20000, 64, graphs.FEAT_SEED, "cuda").cpu().numpy()
    _, out = run_sddmm(coo, src, dst)
    assert np.array_equal(bits(oracle.sddmm_coo_f32(coo.row, coo.col, src, dst, parallel=True)),
                          bits(out))


@pytest.mark.parametrize("shape", [(64,), (8, 8)])
def test_rmat_graph(oracle, shape):
    # R-MAT (a, b, c, d) = (0.57, 0.19, 0.19, 0.05): another degree profile than Chung-Lu,
    # many very short rows (tiles with more runs of equal rows than the stage has slots)
    g = graphs.rmat_graph(scale=17, edge_draws=1 << 21, device="cuda")
    coo = g.to_scipy().tocoo()
    heads = shape[0] if len(shape) == 2 else 1
    src = graphs.normal_features(g.n_cols, shape, graphs.FEAT2_SEED, "cuda").cpu().numpy()
    dst = graphs.normal_features(g.n_rows, shape, graphs.FEAT_SEED, "cuda").cpu().numpy()
    _, out = run_sddmm(coo, src, dst)
    want = oracle.sddmm_coo_f32(coo.row, coo.col, src, dst, num_heads=heads, parallel=True)
    assert np.array_equal(bits(want.reshape(out.shape)), bits(out))


# ---- full size ------------------------------------------------------------------------------

@pytest.fixture(scope="module")
def full():
    g = graphs.powerlaw_graph(device="cuda")
    m = VanillaSDDMMcuda(sp.coo_matrix((g.n_rows, g.n_cols), dtype=np.float32))
    # install the device-resident edge list directly (the scipy route would round-trip
    # 0.9 GB through the host for nothing)
    rows = g.coo_rows()
    m._adj_row_indices = np.empty(g.nnz, np.int8)        # only .shape[0] is used after init
    m._adj_col_indices = m._adj_row_indices
    m._adj_row_indices_placeholder = te.placeholder((g.nnz,), "int32")
    m._adj_col_indices_placeholder = te.placeholder((g.nnz,), "int32")
    m._adj_row_indices_tvm = nd.NDArray(rows, m.ctx)
    m._adj_col_indices_tvm = nd.NDArray(g.indices, m.ctx)
    return g, m


def test_full_size_properties(full):
    g, m = full
    m.build([te.placeholder((g.n_cols, 64)), te.placeholder((g.n_rows, 64))], {}, {})
    ones = torch.ones(g.n_cols, 64, device="cuda")
    out = m.run([ones, ones]).torch
    assert torch.equal(out, torch.full_like(out, 64.0))
    # the host-buffer entry point cuts a list this long into pieces and overlaps the download
    ones_host = torch.ones(g.n_cols, 64).pin_memory()
    out_host = torch.zeros(g.nnz).pin_memory()
    m.out_tvm.torch.zero_()
    m.run_host(ones_host, ones_host, out_host)
    assert torch.equal(out_host, torch.full_like(out_host, 64.0))
    ar = torch.arange(g.n_cols, device="cuda")
    ind = torch.zeros(g.n_cols, 64, device="cuda")
    ind[ar, ar % 64] = 1
    out = m.run([ind, ind]).torch
    want = ((g.indices % 64) == (m._adj_row_indices_tvm.torch % 64)).to(torch.float32)
    assert torch.equal(out, want)


@pytest.mark.parametrize("heads,dim", [(1, 64), (4, 16), (1, 128), (8, 32)])
def test_full_size_sampled_edges_against_oracle(full, oracle, heads, dim):
    g, m = full
    shape = (g.n_cols, dim) if heads == 1 else (g.n_cols, heads, dim)
    m.build([te.placeholder(shape), te.placeholder(shape)], {}, {})
    src = graphs.normal_features(g.n_cols, shape[1:], graphs.FEAT2_SEED, "cuda")
    dst = graphs.normal_features(g.n_rows, shape[1:], graphs.FEAT_SEED, "cuda")
    out1 = m.run([src, dst]).torch.clone()
    out2 = m.run([src, dst]).torch
    assert torch.equal(out1.view(torch.int32), out2.view(torch.int32))
    rng = np.random.default_rng(1)
    starts = np.concatenate(([0, g.nnz - 50000], rng.integers(0, g.nnz - 50000, 6)))
    sel = torch.from_numpy(np.concatenate([np.arange(s, s + 50000) for s in starts])).cuda()
    r = m._adj_row_indices_tvm.torch[sel].cpu().numpy()
    c = g.indices[sel].cpu().numpy()
    want = oracle.sddmm_coo_f32(r, c, src.cpu().numpy(), dst.cpu().numpy(), num_heads=heads,
                                parallel=True)
    assert np.array_equal(bits(want), bits(out1[sel].cpu().numpy()))


@pytest.mark.parametrize("shape", [(64,), (4, 16), (100,)])
def test_extra_outputs_receive_the_same_results(oracle, shape):
    # fg_sddmm_coo_f32_multi: tile kernel (64; 4 x 16) and generic kernel (100)
    coo = random_csr(170, 140, 0.1, seed=31).tocoo()
    src, dst = features((140,) + shape, seed=32), features((170,) + shape, seed=33)
    m = VanillaSDDMMcuda(coo)
    m.build([te.placeholder(src.shape), te.placeholder(dst.shape)], {}, {"num_cuda_blocks": 64})
    heads = shape[0] if len(shape) == 2 else 1
    extra = [torch.full((coo.nnz * heads,), float("nan"), device="cuda") for _ in range(3)]
    m.set_extra_outputs([e.data_ptr() for e in extra])
    out = m.run([nd.array(src, m.ctx), nd.array(dst, m.ctx)]).asnumpy()
    torch.cuda.synchronize()
    want = bits(oracle.sddmm_coo_f32(coo.row, coo.col, src, dst, num_heads=heads))
    assert np.array_equal(want.reshape(-1), bits(out).reshape(-1))
    for e in extra:
        assert np.array_equal(want.reshape(-1), bits(e.cpu().numpy()))


@pytest.mark.parametrize("parts", [(1, 4), (3, 1), (2, 5)])
@pytest.mark.parametrize("shape", [(64,), (4, 16)])
def test_partitioned_edges_and_edge_mapping(oracle, parts, shape):
    # the reference's 2-D blocking (x86 only there) on the GPU: the output is in blocked
    # order and edge_mapping takes it back to the caller's order, bit for bit
    from featgraph_b200.module import PartitionedSDDMMcuda
    coo = random_csr(230, 190, 0.08, seed=41).tocoo()
    src, dst = features((190,) + shape, seed=42), features((230,) + shape, seed=43)
    heads = shape[0] if len(shape) == 2 else 1
    m = PartitionedSDDMMcuda(coo, num_row_partitions=parts[0], num_col_partitions=parts[1])
    m.build([te.placeholder(src.shape), te.placeholder(dst.shape)], {}, {"num_cuda_blocks": 64})
    out = m.run([nd.array(src, m.ctx), nd.array(dst, m.ctx)]).asnumpy()
    want = oracle.sddmm_coo_f32(coo.row, coo.col, src, dst, num_heads=heads)
    assert np.array_equal(bits(want.reshape(out.shape)), bits(out[m.edge_mapping]))
    # blocked order: row partition major, column partition minor (adj_partitioning.py:60-128)
    rp = m._adj_row_indices // -(-230 // parts[0])
    cp = m._adj_col_indices // -(-190 // parts[1])
    key = rp.astype(np.int64) * parts[1] + cp
    assert np.all(np.diff(key) >= 0)
    dup = sp.coo_matrix((np.ones(3, np.float32), ([1, 1, 2], [3, 3, 0])), shape=(230, 190))
    with pytest.raises(ValueError, match="duplicate-free"):
        PartitionedSDDMMcuda(dup, num_col_partitions=2)


def test_multi_head_results_reach_an_unaligned_output(oracle):
    # with H a multiple of four a lane stores its heads four at a time (16 bytes); an output
    # that is not 16-byte aligned must take the 4-byte stores instead
    import ctypes
    coo = random_csr(170, 140, 0.1, seed=71).tocoo()
    src, dst = features((140, 8, 8), seed=72), features((170, 8, 8), seed=73)
    want = oracle.sddmm_coo_f32(coo.row, coo.col, src, dst, num_heads=8)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    r, c, s, d = dev(coo.row), dev(coo.col), dev(src), dev(dst)
    buf = torch.full((coo.nnz * 8 + 1,), float("nan"), device="cuda")
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    for off in (0, 1):
        out = buf[off:off + coo.nnz * 8]
        assert out.data_ptr() % 16 == 4 * off
        _lib.check(_lib.load().fg_sddmm_coo_f32(vp(r), vp(c), vp(s), vp(d), vp(out), coo.nnz, 170,
                                                140, 64, 8, 0, None))
        torch.cuda.synchronize()
        assert np.array_equal(bits(want).reshape(-1), bits(out.cpu().numpy()))


@pytest.mark.parametrize("shape", [(32,), (64,), (256,), (4, 8), (8, 16), (2, 32), (2, 64)])
def test_tma_staging_is_bit_identical(oracle, shape):
    # the same tiles with the gathers handed to the tensor memory accelerator (tile::gather4
    # copies, 128-byte swizzle, mbarriers): every head size the tile kernel has, row-sorted
    # edges (staged dst runs) and a shuffled list (direct dst reads), ragged last tile
    from featgraph_b200 import _lib
    adj = random_csr(500, 400, 0.06, seed=91, dense_rows=(7, 300)).tocoo()
    for shuffle in (False, True):
        row, col = adj.row.astype(np.int32), adj.col.astype(np.int32)
        if shuffle:
            order = np.random.RandomState(92).permutation(row.shape[0])
            row, col = row[order], col[order]
        coo = sp.coo_matrix((np.ones(row.shape[0], np.float32), (row, col)), shape=adj.shape)
        src = features((400,) + shape, seed=93)
        dst = features((500,) + shape, seed=94)
        m = VanillaSDDMMcuda(coo)
        m.build([te.placeholder(src.shape), te.placeholder(dst.shape)], {}, {})
        plain = m.run([nd.array(src, m.ctx), nd.array(dst, m.ctx)]).asnumpy().copy()
        m.out_tvm.torch.zero_()
        y = m.run([nd.array(src, m.ctx), nd.array(dst, m.ctx)],
                  launch_flags=_lib.SDDMM_TMA_STAGING).asnumpy()
        assert m.device_status() == 0
        assert np.array_equal(bits(plain), bits(y))
        heads = shape[0] if len(shape) == 2 else 1
        want = oracle.sddmm_coo_f32(row, col, src.reshape(400, -1), dst.reshape(500, -1), heads)
        assert np.array_equal(bits(want.reshape(y.shape)), bits(y))


def test_tma_staging_refuses_what_it_does_not_cover():
    from featgraph_b200 import _lib
    adj = random_csr(50, 60, 0.1, seed=95).tocoo()
    src, dst = features((60, 48), seed=96), features((50, 48), seed=97)
    m = VanillaSDDMMcuda(adj)
    m.build([te.placeholder(src.shape), te.placeholder(dst.shape)], {}, {"num_cuda_blocks": 64})
    with pytest.raises(_lib.FeatGraphError):        # feat_len 48 runs the generic kernel
        m.run([nd.array(src, m.ctx), nd.array(dst, m.ctx)], launch_flags=_lib.SDDMM_TMA_STAGING)


@pytest.mark.parametrize("feat_len", [32, 64, 256])
@pytest.mark.parametrize("ops", [("mul", "sum"), ("sub", "max")])
def test_row_register_kernel_is_bit_identical(oracle, feat_len, ops):
    # the kernel that keeps the dst operand in registers, forced by its launch flag: long rows
    # (tiles inside one run of equal rows), short rows (every tile crosses row boundaries, dst
    # read from global memory), a shuffled list, a ragged last tile and a last group of tiles
    # that is not whole
    long_rows = random_csr(40, 3000, 0.5, seed=101, empty_rows=(3,)).tocoo()
    short_rows = random_csr(3000, 500, 0.01, seed=102).tocoo()
    for adj, shuffle in ((long_rows, False), (short_rows, False), (long_rows, True)):
        row, col = adj.row.astype(np.int32), adj.col.astype(np.int32)
        if shuffle:
            order = np.random.RandomState(103).permutation(row.shape[0])
            row, col = row[order], col[order]
        coo = sp.coo_matrix((np.ones(row.shape[0], np.float32), (row, col)), shape=adj.shape)
        src = features((adj.shape[1], feat_len), seed=104)
        dst = features((adj.shape[0], feat_len), seed=105)
        m = VanillaSDDMMcuda(coo)
        m.build([te.placeholder(src.shape), te.placeholder(dst.shape)],
                {"msg_op": ops[0], "reduce_op": ops[1]}, {})
        chosen = bool(m.default_launch_flags & _lib.SDDMM_ROW_REGISTERS)
        assert chosen == (adj is long_rows and not shuffle)     # the module's own choice
        for force in (0, _lib.SDDMM_ROW_REGISTERS):
            m.default_launch_flags = force
            m.out_tvm.torch.fill_(float("nan"))
            y = m.run([nd.array(src, m.ctx), nd.array(dst, m.ctx)]).asnumpy()
            want = oracle.gsddmm_coo_f32(row, col, src, dst, 1, ops[0], ops[1])
            assert np.array_equal(bits(want.reshape(y.shape)), bits(y)), (force, shuffle)


def test_row_register_hint_is_ignored_where_it_does_not_apply(oracle):
    adj = random_csr(60, 70, 0.2, seed=106).tocoo()
    for shape in ((48,), (4, 16)):                    # generic kernel; several heads
        src, dst = features((70,) + shape, seed=107), features((60,) + shape, seed=108)
        m = VanillaSDDMMcuda(adj)
        m.build([te.placeholder(src.shape), te.placeholder(dst.shape)], {}, {"num_cuda_blocks": 64})
        assert not m.default_launch_flags & _lib.SDDMM_ROW_REGISTERS
        y = m.run([nd.array(src, m.ctx), nd.array(dst, m.ctx)],
                  launch_flags=_lib.SDDMM_ROW_REGISTERS).asnumpy()
        heads = shape[0] if len(shape) == 2 else 1
        want = oracle.sddmm_coo_f32(adj.row, adj.col, src.reshape(70, -1), dst.reshape(60, -1), heads)
        assert np.array_equal(bits(want.reshape(y.shape)), bits(y))
