"""Multi-GPU path on real devices: one process per GPU over NCCL, SpMM sharded by
nnz-balanced row blocks and SDDMM by edge ranges, outputs all-gathered; every rank must hold
the full result, bit-equal to the CPU oracle.  Skipped when fewer than two GPUs are visible."""
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
        from featgraph_b200.distributed import ShardedSDDMM, ShardedSpMM
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
        modes = set()
        # fused: kernels store into every peer's output (symmetric memory); else NCCL gathers
        for fused in (True, False):
            spmm = ShardedSpMM(adj, 64, dev, fused_gather=fused)
            modes.add(spmm.gather_mode)
            for _ in range(2):                   # the second call overwrites the first's result
                y = spmm.run(x)
            torch.cuda.synchronize(dev)
            dist.barrier()
            assert np.array_equal(bits(want_y), bits(y.cpu().numpy())), \
                "rank %d SpMM (%s)" % (rank, spmm.gather_mode)
            assert spmm.module.device_status() == 0
            per_rank = np.diff(adj.indptr[spmm.bounds])
            assert per_rank.max() - per_rank.min() <= np.diff(adj.indptr).max()
            # peers get the results from the SDDMM kernel's own stores, or from the copy
            # kernel that pushes finished pieces while the next piece computes
            for shape, heads, peer_mode in (((64,), 1, "store"), ((64,), 1, "push"),
                                            ((4, 16), 4, "push"), ((4, 16), 4, "auto")):
                sd = ShardedSDDMM(rows, g.indices, g.n_rows, g.n_cols, shape, dev,
                                  fused_gather=fused, peer_mode=peer_mode)
                for _ in range(2):
                    out = sd.run(y2.view((-1,) + shape), x.view((-1,) + shape))
                torch.cuda.synchronize(dev)
                dist.barrier()
                want = fg_oracle.sddmm_coo_f32(rows.cpu().numpy(), g.indices.cpu().numpy(),
                                               y2.cpu().numpy(), x.cpu().numpy(),
                                               num_heads=heads, parallel=True)
                assert np.array_equal(bits(want.reshape(out.shape)), bits(out.cpu().numpy())), \
                    "rank %d SDDMM %r (%s)" % (rank, shape, sd.gather_mode)
            del spmm, sd
        assert "nccl" in modes
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
def test_sharded_ops_on_two_gpus():
    mp.spawn(_worker, args=(2, _free_port()), nprocs=2, join=True)
