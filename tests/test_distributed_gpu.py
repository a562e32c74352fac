"""Multi-GPU path on real devices: one process per GPU over NCCL, SpMM sharded by
nnz-balanced row blocks and SDDMM by edge ranges, outputs all-gathered; every rank must hold
the full result, bit-equal to the CPU oracle.  Each world size is skipped when fewer GPUs are visible."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from helpers import bits

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from featgraph_b200 import graphs
        from featgraph_b200.distributed import OverlappedPair, ShardedSDDMM, ShardedSpMM
        from oracle import fg_oracle

        g = graphs.powerlaw_graph(n=30000, nnz_target=4000000, device=dev)
        adj = g.to_scipy()
        x = graphs.normal_features(g.n_cols, 64, graphs.FEAT_SEED, dev)
        y2 = graphs.normal_features(g.n_cols, 64, graphs.FEAT2_SEED, dev)
        # every rank generated the same graph
        probe = torch.tensor([g.nnz, int(g.indices[::997].sum())], device=dev)
        gathered = [torch.zeros_like(probe) for _ in range(world)]
        dist.all_gather(gathered, probe)
        assert all(torch.equal(t, probe) for t in gathered)

        want_y = fg_oracle.spmm_csr_f32(adj.indptr, adj.indices, adj.data, x.cpu().numpy())
        rows = g.coo_rows()
        want_sd = {heads: fg_oracle.sddmm_coo_f32(rows.cpu().numpy(), g.indices.cpu().numpy(),
                                                  y2.cpu().numpy(), x.cpu().numpy(),
                                                  num_heads=heads, parallel=True)
                   for heads in (1, 4)}
        modes = set()
        # fused: the kernels deliver their results to every peer's output themselves (plain
        # peer stores, or one multicast store through the NVLink switch); else NCCL gathers
        for fused, spmm_mode in ((True, "store"), (True, "mcast"), (False, "auto")):
            spmm = ShardedSpMM(adj, 64, dev, fused_gather=fused, peer_mode=spmm_mode)
            modes.add(spmm.gather_mode)
            for _ in range(2):                   # the second call overwrites the first's result
                y = spmm.run(x)
            torch.cuda.synchronize(dev)
            dist.barrier()
            assert np.array_equal(bits(want_y), bits(y.cpu().numpy())), \
                "rank %d SpMM (%s)" % (rank, spmm.gather_mode)
            assert spmm.device_status() == 0
            per_rank = np.diff(adj.indptr[spmm.bounds])
            assert per_rank.max() - per_rank.min() <= np.diff(adj.indptr).max()
            # peers get the results from the SDDMM kernel's own stores (unicast or multicast),
            # or from the copy kernel that pushes finished pieces while the next piece computes
            for shape, heads, peer_mode in (((64,), 1, "store"), ((64,), 1, "push"),
                                            ((64,), 1, "mcast"), ((4, 16), 4, "mcast"),
                                            ((4, 16), 4, "push"), ((4, 16), 4, "auto")):
                sd = ShardedSDDMM(rows, g.indices, g.n_rows, g.n_cols, shape, dev,
                                  fused_gather=fused, peer_mode=peer_mode)
                modes.add(sd.gather_mode)
                for _ in range(2):
                    out = sd.run(y2.view((-1,) + shape), x.view((-1,) + shape))
                torch.cuda.synchronize(dev)
                dist.barrier()
                assert np.array_equal(bits(want_sd[heads].reshape(out.shape)),
                                      bits(out.cpu().numpy())), \
                    "rank %d SDDMM %r (%s)" % (rank, shape, sd.gather_mode)
                assert sd.device_status() == 0
            # the two operators side by side in one chain of programmatic launches, one
            # barrier pair around both
            out.zero_()
            y.zero_()
            pair = OverlappedPair(spmm, sd)
            for _ in range(2):
                y, out = pair.run(x, y2.view(-1, 4, 16), x.view(-1, 4, 16))
            torch.cuda.synchronize(dev)
            dist.barrier()
            assert np.array_equal(bits(want_y), bits(y.cpu().numpy()))
            assert np.array_equal(bits(want_sd[4]), bits(out.cpu().numpy()))
            # end to end from host buffers: 1/world of the inputs per rank over PCIe
            y_host = torch.zeros(g.n_rows, 64).pin_memory()
            o_host = torch.zeros(g.nnz, 4).pin_memory()
            spmm.run_host(x.cpu().pin_memory(), y_host)
            sd.run_host(y2.view(-1, 4, 16).cpu().pin_memory(), x.view(-1, 4, 16).cpu().pin_memory(),
                        o_host)
            assert np.array_equal(bits(want_y[spmm.row_lo:spmm.row_hi]),
                                  bits(y_host[spmm.row_lo:spmm.row_hi].numpy()))
            assert np.array_equal(bits(want_sd[4][sd.edge_lo:sd.edge_hi]),
                                  bits(o_host[sd.edge_lo:sd.edge_hi].numpy()))
            assert spmm.device_status() == 0 and sd.device_status() == 0
            del spmm, sd, pair
        assert "nccl" in modes and "peer_store" in modes
        if rank == 0:
            print("gather modes exercised on %d GPUs: %s" % (world, sorted(modes)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_ops_on_several_gpus(world):
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    mp.spawn(_worker, args=(world, _free_port()), nprocs=world, join=True)
