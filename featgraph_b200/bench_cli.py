"""Command-line benchmark with the flags of the reference's scripts
(benchmark/bench_vanilla_spmm.py:71-84, bench_vanilla_sddmm.py:77-90):

    python -m featgraph_b200.bench_cli --kernel spmm  --dataset reddit_csr_float32.npz --feat-len 64 --target cuda
    python -m featgraph_b200.bench_cli --kernel sddmm --synthetic powerlaw --feat-len 128
    python -m featgraph_b200.bench_cli --kernel sddmm --synthetic powerlaw --heads 8 --head-dim 32
    torchrun --nproc-per-node 8 -m featgraph_b200.bench_cli --kernel spmm --synthetic rmat --feat-len 64

``--dataset`` is a scipy ``save_npz`` file (CSR for SpMM, COO for SDDMM), as the reference's
download script writes them; ``--synthetic`` generates one of the seeded graphs of
``featgraph_b200.graphs`` on the GPU instead.  The reference's scripts sweep TVM schedule
parameters and print the mean of 5 runs; the kernels here have no such parameters, so one
JSON line per feature length is printed: mean milliseconds over ``--num-runs`` launches
(kernel only, inputs resident, as ``measure_average_time``), GFLOP/s and algorithmic GB/s.
Under torchrun the graph is sharded over the ranks and the all-gather is inside the time.
The features are seeded N(0,1) arrays (``graphs.normal_features`` with FEAT_SEED for the
array indexed by column, FEAT2_SEED for the one indexed by row); ``--dump-output FILE``
saves the last feature length's result as a ``.npy`` file so that it can be checked.
"""
import argparse
import json
import os

import numpy as np
import torch

from . import _lib, graphs
from .distributed import ShardedSDDMM, ShardedSpMM

NOMINAL_HBM_GBS = 8000.0


def _load_graph(args, device):
    if args.dataset:
        import scipy.sparse as sp
        m = sp.load_npz(args.dataset)
        csr = m.tocsr().astype(np.float32)
        csr.sort_indices()
        g = graphs.CSRGraph(csr.shape[0], csr.shape[1],
                            torch.from_numpy(csr.indptr.astype(np.int32)).to(device),
                            torch.from_numpy(csr.indices.astype(np.int32)).to(device),
                            torch.from_numpy(csr.data).to(device))
        if args.kernel == "sddmm":
            # the edge list exactly as stored (a COO file keeps its order, as the
            # reference's SDDMM module does: python/featgraph/module/sddmm.py:28-31, 51-52)
            coo = m if m.format == "coo" else m.tocoo()
            g.edge_list = (torch.from_numpy(coo.row.astype(np.int32)).to(device),
                           torch.from_numpy(coo.col.astype(np.int32)).to(device))
        return g, "file:" + args.dataset
    if args.synthetic == "powerlaw":
        g = graphs.powerlaw_graph(n=args.vertices or graphs.REDDIT_NUM_VERTICES,
                                  nnz_target=args.edges or graphs.REDDIT_NUM_EDGES, device=device)
    elif args.synthetic == "rmat":
        g = graphs.rmat_graph(scale=args.scale, edge_draws=args.edges or (1 << (args.scale + 4)),
                              device=device)
    else:
        g = graphs.regular_graph(n=args.vertices or 65536, device=device)
    return g, "synthetic:" + args.synthetic


class _PartitionedSpMM(object):
    """The DDS form of the SpMM (VanillaSpMMcuda with num_col_partitions > 1) behind the
    few names the timing loop uses."""
    gather_mode = "none"

    def __init__(self, adj, feat_len, device_id, parts):
        from . import te
        from .module import VanillaSpMMcuda
        self.module = VanillaSpMMcuda(adj, device_id=device_id, num_col_partitions=parts)
        self.module.build([te.placeholder((adj.shape[1], feat_len))], {}, {})
        self.out = None

    def run(self, x):
        self.out = self.module.run([x]).torch
        return self.out

    def device_status(self):
        return self.module.device_status()


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--kernel", choices=["spmm", "sddmm"], default="spmm")
    ap.add_argument("--dataset", type=str, default=None,
                    help="adjacency matrix stored as a scipy npz file")
    ap.add_argument("--synthetic", choices=["powerlaw", "rmat", "regular"], default="powerlaw")
    ap.add_argument("--feat-len", type=str, default="128",
                    help="feature length, or a comma-separated list")
    ap.add_argument("--heads", type=int, default=1, help="SDDMM heads (feat-len = heads x head-dim)")
    ap.add_argument("--head-dim", type=int, default=0)
    ap.add_argument("--target", choices=["cuda", "x86"], default="cuda")
    ap.add_argument("--num-runs", type=int, default=20)
    ap.add_argument("--vertices", type=int, default=0)
    ap.add_argument("--edges", type=int, default=0)
    ap.add_argument("--scale", type=int, default=24, help="R-MAT scale (2**scale vertices)")
    ap.add_argument("--row-partitions", type=int, default=1,
                    help="SDDMM: the reference's 2-D edge blocking (VanillaSDDMMx86's arguments)")
    ap.add_argument("--col-partitions", type=int, default=1,
                    help="SpMM (one GPU): the reference's 1-D source-vertex partitioning, "
                         "VanillaSpMMx86's num_col_partitions; SDDMM: see --row-partitions")
    ap.add_argument("--sddmm-tma", action="store_true",
                    help="SDDMM: stage the tiles with TMA tile::gather4 copies "
                         "(FG_SDDMM_TMA_STAGING) instead of cp.async")
    ap.add_argument("--sweep", action="store_true",
                    help="run the whole configured sweep in one process: SpMM and SDDMM at feat-len "
                         "32 ... 512, then multi-head SDDMM (4,16), (8,32), (16,64)")
    ap.add_argument("--peer-mode", choices=["auto", "store", "mcast", "push"], default="auto",
                    help="multi-GPU: how results reach the peers (featgraph_b200.distributed)")
    ap.add_argument("--dump-output", type=str, default=None,
                    help="save the (last) result array to this .npy file (rank 0)")
    args = ap.parse_args(argv)
    if args.target != "cuda":
        raise SystemExit("this backend ships the cuda target only (no x86 code path)")

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":    # its banner goes to stdout
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=device)

    g, source = _load_graph(args, device)
    n = g.n_rows
    records = []
    # the cases of this run: (kernel, feat_len, heads)
    if args.sweep:
        cases = [("spmm", f, 1) for f in (32, 64, 128, 256, 512)]
        cases += [("sddmm", f, 1) for f in (32, 64, 128, 256, 512)]
        cases += [("sddmm", h * d, h) for h, d in ((4, 16), (8, 32), (16, 64))]
    elif args.heads > 1:
        cases = [(args.kernel, args.heads * (args.head_dim or 16), args.heads)]
    else:
        cases = [(args.kernel, int(f), 1) for f in args.feat_len.split(",")]
    kernels = set(k for k, _, _ in cases)
    adj = g.to_scipy() if "spmm" in kernels else None
    rows = g.coo_rows() if "sddmm" in kernels else None
    cols = g.indices
    nnz_sd = g.nnz
    if "sddmm" in kernels and hasattr(g, "edge_list"):
        rows, cols = g.edge_list
        nnz_sd = int(rows.shape[0])
    if "sddmm" in kernels and (args.row_partitions > 1 or args.col_partitions > 1):
        # the blocked edge order of util_partition_adj_coo_2d (row partition major, column
        # partition minor, row-major inside a block), computed on the device
        rows_per = max(-(-g.n_rows // args.row_partitions), 1)
        cols_per = max(-(-g.n_cols // args.col_partitions), 1)
        key = (rows // rows_per).to(torch.int64) * args.col_partitions + (cols // cols_per)
        order = torch.argsort(key, stable=True)
        rows, cols = rows[order].contiguous(), cols[order].contiguous()
        del key, order

    for kernel, f, heads in cases:
        shape = (heads, f // heads) if heads > 1 else (f,)
        x = graphs.normal_features(g.n_cols, shape, graphs.FEAT_SEED, device)
        if kernel == "spmm":
            nnz = g.nnz
            if args.col_partitions > 1:
                if world > 1:
                    raise SystemExit("--col-partitions with --kernel spmm runs on one GPU")
                op = _PartitionedSpMM(adj, f, local, args.col_partitions)
            else:
                op = ShardedSpMM(adj, f, device, peer_mode=args.peer_mode)
            call = lambda: op.run(x)                       # noqa: E731
            alg = 4 * (n + 1) + 8 * nnz + 4 * nnz * f + 4 * n * f
        else:
            nnz = nnz_sd
            y2 = graphs.normal_features(g.n_rows, shape, graphs.FEAT2_SEED, device)
            op = ShardedSDDMM(rows, cols, n, g.n_cols, shape, device, peer_mode=args.peer_mode)
            if args.sddmm_tma:
                op.module.default_launch_flags = _lib.SDDMM_TMA_STAGING
            call = lambda: op.run(x, y2)                   # noqa: E731
            alg = 8 * nnz + 8 * nnz * f + 4 * nnz * heads
        for _ in range(3):
            call()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(args.num_runs):
            call()
        t1.record()
        torch.cuda.synchronize(device)
        op.device_status()                # raises if a bounded device-side wait gave up
        ms = torch.tensor([t0.elapsed_time(t1) / args.num_runs], device=device,
                          dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        ms = float(ms)
        if rank == 0:
            if args.dump_output:
                np.save(args.dump_output, op.out.cpu().numpy())
            records.append({
                "kernel": kernel, "graph": source, "rows": n, "nnz": nnz, "feat_len": f,
                "heads": heads, "n_gpus": world, "num_runs": args.num_runs,
                "gather": op.gather_mode,
                "partitions": [args.row_partitions, args.col_partitions],
                "ms": round(ms, 4), "gflops": round(2.0 * nnz * f / ms / 1e6, 1),
                "alg_gbs": round(alg / ms / 1e6, 1),
                "frac_of_8TBs": round(alg / ms / 1e6 / NOMINAL_HBM_GBS, 4),
                "degree": g.degree_stats()})
            print(json.dumps(records[-1]), flush=True)
        del op, x, call
        if kernel == "sddmm":
            del y2
        torch.cuda.empty_cache()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return records


if __name__ == "__main__":
    main()
