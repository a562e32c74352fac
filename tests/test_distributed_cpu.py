"""Host-side logic of the multi-GPU path on CPU ranks (gloo, world size 2 and 3): shard
bounds, sub-matrix extraction, in-place local compute and reassembly by all-gather.  The
rank-local operator is swapped for the CPU oracle here -- the device kernels themselves
are covered by the gpu-marked tests."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import bits, features, random_csr


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, heads):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from featgraph_b200.distributed import ShardedSDDMM, ShardedSpMM, shard_edges
        from oracle import fg_oracle

        class OracleSpMM(ShardedSpMM):
            def make_local(self, local_csr, schedule_args):
                view = self._views[self.rank]

                def f(x):
                    view.copy_(torch.from_numpy(fg_oracle.spmm_csr_f32(
                        local_csr.indptr, local_csr.indices, local_csr.data, x.numpy(),
                        n_cols=self.n_cols)))
                return f

        class OracleSDDMM(ShardedSDDMM):
            def make_local(self, row_local, col_local):
                n_local = self.edge_hi - self.edge_lo
                slot = self._slot[:n_local * self.num_heads]

                def f(src, dst):
                    slot.copy_(torch.from_numpy(fg_oracle.sddmm_coo_f32(
                        row_local, col_local, src.numpy(), dst.numpy(),
                        num_heads=self.num_heads).reshape(-1)))
                return f

        adj = random_csr(97, 61, 0.15, seed=5, empty_rows=(0, 96), dense_rows=(40,))
        x = features((61, 32), seed=6)
        op = OracleSpMM(adj, 32, "cpu")
        assert op.bounds[0] == 0 and op.bounds[-1] == 97 and len(op.bounds) == world + 1
        y = op.run(torch.from_numpy(x)).numpy()
        want = fg_oracle.spmm_csr_f32(adj.indptr, adj.indices, adj.data, x, n_cols=61)
        assert np.array_equal(bits(want), bits(y)), "rank %d: SpMM reassembly differs" % rank

        coo = adj.tocoo()
        shape = (heads, 8) if heads > 1 else (32,)
        src, dst = features((61,) + shape, seed=7), features((97,) + shape, seed=8)
        sd = OracleSDDMM(coo.row, coo.col, 97, 61, shape, "cpu")
        out = sd.run(torch.from_numpy(src), torch.from_numpy(dst)).numpy()
        want = fg_oracle.sddmm_coo_f32(coo.row, coo.col, src, dst, num_heads=heads)
        assert out.shape == want.shape
        assert np.array_equal(bits(want), bits(out)), "rank %d: SDDMM reassembly differs" % rank

        # end to end from host buffers: every rank uploads 1/world of the replicated inputs
        # and the blocks are exchanged with one all-gather; each rank "downloads" its block
        y_host = torch.zeros(97, 32)
        op.run_host(torch.from_numpy(x), y_host)
        want = fg_oracle.spmm_csr_f32(adj.indptr, adj.indices, adj.data, x, n_cols=61)
        assert np.array_equal(bits(want[op.row_lo:op.row_hi]),
                              bits(y_host[op.row_lo:op.row_hi].numpy()))
        o_host = torch.zeros(out.shape)
        sd.run_host(torch.from_numpy(src), torch.from_numpy(dst), o_host)
        want = fg_oracle.sddmm_coo_f32(coo.row, coo.col, src, dst, num_heads=heads)
        assert np.array_equal(bits(want.reshape(out.shape)[sd.edge_lo:sd.edge_hi]),
                              bits(o_host[sd.edge_lo:sd.edge_hi].numpy()))
        assert list(sd.bounds) == list(shard_edges(coo.nnz, world))

        # more ranks than edges / rows: empty shards must not break the collectives
        tiny = random_csr(2, 5, 0.5, seed=9)
        op = OracleSpMM(tiny, 4, "cpu")
        xt = features((5, 4), seed=10)
        want = fg_oracle.spmm_csr_f32(tiny.indptr, tiny.indices, tiny.data, xt, n_cols=5)
        assert np.array_equal(bits(want), bits(op.run(torch.from_numpy(xt)).numpy()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,heads", [(2, 1), (3, 4)])
def test_sharded_ops_reassemble_the_full_result(world, heads):
    mp.spawn(_worker, args=(world, _free_port(), heads), nprocs=world, join=True)


def test_single_process_bounds():
    from featgraph_b200.distributed import shard_edges, shard_rows_by_nnz
    adj = random_csr(500, 300, 0.05, seed=1, dense_rows=(10, 250))
    for world in (1, 2, 4, 8):
        b = shard_rows_by_nnz(adj.indptr, world)
        assert b[0] == 0 and b[-1] == 500 and (np.diff(b) >= 0).all()
        per = np.diff(adj.indptr[b])
        assert per.sum() == adj.nnz and per.max() - adj.nnz / world <= 300
        e = shard_edges(adj.nnz, world)
        assert e[0] == 0 and e[-1] == adj.nnz and (np.diff(e) >= 0).all()
        assert (e[:-1] % 32 == 0).all() and np.diff(e).max() < adj.nnz / world + 32


def _leaving_worker(rank, world, port, result):
    """Rank 1 raises between two steps; rank 0's next exchange must end with an error within
    the process group's timeout instead of blocking."""
    import datetime
    import time
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=8))
    from featgraph_b200.distributed import ShardedSpMM
    from oracle import fg_oracle

    class OracleSpMM(ShardedSpMM):
        def make_local(self, local_csr, schedule_args):
            view = self._views[self.rank]

            def f(x):
                view.copy_(torch.from_numpy(fg_oracle.spmm_csr_f32(
                    local_csr.indptr, local_csr.indices, local_csr.data, x.numpy(),
                    n_cols=self.n_cols)))
            return f

    adj = random_csr(40, 30, 0.2, seed=3)
    x = torch.from_numpy(features((30, 8), seed=4))
    op = OracleSpMM(adj, 8, "cpu")
    op.run(x)                                   # step 1: both ranks
    if rank == 1:
        os._exit(0)                             # leaves between steps, nothing in flight
    t = time.time()
    try:
        op.run(x)                               # step 2: the peer is gone
        result.put("no error")
    except Exception as exc:                    # noqa: BLE001 - any error is the point
        result.put("error after %.1f s: %s" % (time.time() - t, type(exc).__name__))


def test_a_rank_that_leaves_between_steps_gives_an_error_not_a_hang():
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    procs = [ctx.Process(target=_leaving_worker, args=(r, 2, _free_port_once(), result))
             for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=90)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.kill()
    assert not alive, "a rank blocked"
    assert result.get(timeout=5).startswith("error")


_PORT = []


def _free_port_once():
    if not _PORT:
        _PORT.append(_free_port())
    return _PORT[0]
