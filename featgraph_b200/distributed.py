"""One-process-per-GPU sharding of SpMM and SDDMM over ``torch.distributed``.

The reference is single-device (python/featgraph/module/spmm.py:218, sddmm.py:185); this
is the multi-GPU extension: SpMM is split into contiguous destination-row blocks that
hold about nnz / world nonzeros each, SDDMM into equal contiguous edge ranges.  The
dense features are replicated on every rank; each rank computes its block straight into
its slice of a full-size output, and every rank ends up with the whole result (what a
following GNN layer needs).  On GPUs the full-size outputs live in symmetric memory and
the kernels store each finished row / edge result into every peer's copy themselves
(plain stores over NVLink, bracketed by two device-side barriers per call); where that
cannot be set up the slices are exchanged with NCCL collectives instead.

The classes take an already initialised process group (NCCL on GPUs).  ``make_local``
is the only place that touches a device kernel, so host-side logic (bounds, sub-matrix
extraction, reassembly) can be exercised on CPU ranks with another local operator.
"""
import ctypes

import numpy as np
import scipy.sparse as sp
import torch
import torch.distributed as dist

from . import _lib
from .runtime import NDArray, Placeholder


def shard_rows_by_nnz(indptr, world):
    """world + 1 row bounds with about nnz / world nonzeros per block (C ABI, host)."""
    indptr = np.ascontiguousarray(indptr, dtype=np.int32)
    bounds = (ctypes.c_int64 * (world + 1))()
    _lib.check(_lib.load().fg_shard_rows_by_nnz(indptr.ctypes.data_as(_lib.c_i32p),
                                                indptr.shape[0] - 1, world, bounds))
    return np.array(bounds[:], dtype=np.int64)


def shard_edges(nnz, world):
    bounds = (ctypes.c_int64 * (world + 1))()
    _lib.check(_lib.load().fg_shard_edges(int(nnz), world, bounds))
    return np.array(bounds[:], dtype=np.int64)


def _symmetric_buffer(numel, device, group, world):
    """A float32 buffer of ``numel`` elements that every rank of the group can address
    directly (torch symmetric memory over NVLink), or None if that cannot be set up on
    every rank.  Returns (tensor, handle)."""
    ok, buf, hdl = 1, None, None
    try:
        import torch.distributed._symmetric_memory as symm_mem
        pg = group if group is not None else dist.group.WORLD
        buf = symm_mem.empty(max(int(numel), 1), dtype=torch.float32, device=device)
        hdl = symm_mem.rendezvous(buf, pg)
        if len(hdl.buffer_ptrs) != world:
            ok = 0
    except Exception:                      # no peer access / API missing: use NCCL instead
        ok = 0
    flag = torch.tensor([ok], device=device, dtype=torch.int32)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    if int(flag) == 0:
        return None, None
    return buf, hdl


def _group_info(group):
    if group is None and not dist.is_initialized():
        return 0, 1
    return dist.get_rank(group), dist.get_world_size(group)


class ShardedSpMM(object):
    """Row-block sharded CSR SpMM.

    adj_scipy_csr : the FULL matrix (every rank passes the same one)
    feat_len      : feature length F
    device        : torch device of this rank
    """

    def __init__(self, adj_scipy_csr, feat_len, device, group=None, schedule_args=None,
                 fused_gather=True):
        self.group = group
        self.rank, self.world = _group_info(group)
        self.device = torch.device(device)
        self._symm = None
        self.n_rows, self.n_cols = adj_scipy_csr.shape
        self.feat_len = int(feat_len)
        self.bounds = shard_rows_by_nnz(adj_scipy_csr.indptr, self.world)
        lo, hi = int(self.bounds[self.rank]), int(self.bounds[self.rank + 1])
        self.row_lo, self.row_hi = lo, hi
        ptr = adj_scipy_csr.indptr
        e0, e1 = int(ptr[lo]), int(ptr[hi])
        local = sp.csr_matrix((adj_scipy_csr.data[e0:e1], adj_scipy_csr.indices[e0:e1],
                               (ptr[lo:hi + 1] - ptr[lo]).astype(ptr.dtype)),
                              shape=(hi - lo, self.n_cols))
        self.local_nnz = e1 - e0
        self.out = None
        if fused_gather and self.world > 1 and self.device.type == "cuda":
            # the kernels store every finished row into all peers' outputs themselves
            buf, hdl = _symmetric_buffer(self.n_rows * self.feat_len, self.device, group,
                                         self.world)
            if buf is not None:
                self.out = buf[:self.n_rows * self.feat_len].view(self.n_rows, self.feat_len)
                self.out.zero_()
                self._symm = hdl
        if self.out is None:
            self.out = torch.zeros(self.n_rows, self.feat_len, dtype=torch.float32,
                                   device=self.device)
        self._views = [self.out[int(self.bounds[k]):int(self.bounds[k + 1])]
                       for k in range(self.world)]
        self._local = self.make_local(local, dict(schedule_args or {}))
        if self._symm is not None:
            off = self.row_lo * self.feat_len * 4
            self.module.set_extra_outputs([int(p) + off for r, p in
                                           enumerate(self._symm.buffer_ptrs) if r != self.rank])
            self._symm.barrier()

    def make_local(self, local_csr, schedule_args):
        """Build the rank-local operator: ``f(x) -> None`` writing rows [row_lo, row_hi)."""
        from .module import VanillaSpMMcuda
        m = VanillaSpMMcuda(local_csr, device_id=self.device.index or 0)
        m.build([Placeholder((self.n_cols, self.feat_len))], {}, schedule_args)
        m.out_tvm = NDArray(self._views[self.rank], m.ctx)     # compute in place in the slice
        self.module = m
        return lambda x: m.run([x])

    @property
    def gather_mode(self):
        """'peer_stores' (kernels write into every rank's output), 'nccl', or 'none'."""
        return "none" if self.world == 1 else ("peer_stores" if self._symm is not None else "nccl")

    def compute_local(self, x):
        if self._symm is not None:
            # peers store into this rank's output: they may start only when this rank's
            # stream has passed everything that read the previous result
            self._symm.barrier()
        self._local(x)

    def gather(self):
        """Uneven all-gather of the row blocks: one broadcast per owner -- or, with the
        fused path, just the barrier after which every rank's stores have landed."""
        if self.world == 1:
            return
        if self._symm is not None:
            self._symm.barrier()
            return
        for k in range(self.world):
            if self._views[k].numel():
                dist.broadcast(self._views[k], src=dist.get_global_rank(self.group, k)
                               if self.group is not None else k, group=self.group)

    def run(self, x):
        """x: replicated (n_cols, F) features on this rank's device.  Returns the full
        (n_rows, F) result, identical on every rank."""
        self.compute_local(x)
        self.gather()
        return self.out

    def run_host(self, x_host, y_host):
        """End to end from pinned HOST buffers: upload the replicated features, compute this
        rank's row block, all-gather, download this rank's block into ``y_host`` (the ranks'
        blocks together are the whole result).  Synchronises the stream."""
        if self.world == 1:
            return self.module.run_host(x_host, y_host)
        if getattr(self, "_x_stage", None) is None:
            self._x_stage = torch.empty(self.n_cols, self.feat_len, dtype=torch.float32,
                                        device=self.device)
        self._x_stage.copy_(x_host, non_blocking=True)
        self.run(self._x_stage)
        y_host[self.row_lo:self.row_hi].copy_(self._views[self.rank], non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        return y_host

    def num_launches(self):
        return self.module.num_launches() if hasattr(self, "module") else 0


class ShardedSDDMM(object):
    """Edge-range sharded COO SDDMM (single- or multi-head).

    row, col : the FULL edge list (numpy int32 or torch tensors); every rank passes the same
    """

    def __init__(self, row, col, n_rows, n_cols, feat_shape, device, group=None,
                 fused_gather=True, peer_mode="auto"):
        """peer_mode (fused path only): 'store' -- the SDDMM kernel stores each result into
        every peer's output itself; 'push' -- a copy kernel pushes finished pieces to the
        peers while the next piece computes; 'auto' -- 'store' (measured faster on 2 and on
        8 GPUs once every rank's slice starts on a 128-byte boundary)."""
        self.group = group
        self.rank, self.world = _group_info(group)
        self.device = torch.device(device)
        self._symm = None
        self.n_rows, self.n_cols = int(n_rows), int(n_cols)
        self.feat_shape = (feat_shape,) if isinstance(feat_shape, int) else tuple(feat_shape)
        self.num_heads = self.feat_shape[0] if len(self.feat_shape) == 2 else 1
        self.nnz = int(row.shape[0])
        # equal chunks (the last one padded) so that one all-gather assembles the output
        # (a multiple of 32 edges: every rank's slice then starts on a 128-byte boundary, so a
        # warp's 32 results are one aligned line in the peers' memory -- unaligned slices made
        # the in-kernel peer stores 1.7 times slower on 8 GPUs)
        self.chunk = ((self.nnz + self.world - 1) // self.world + 31) // 32 * 32 if self.nnz else 0
        lo = min(self.rank * self.chunk, self.nnz)
        hi = min(lo + self.chunk, self.nnz)
        self.edge_lo, self.edge_hi = lo, hi
        self._padded = None
        if fused_gather and self.world > 1 and self.device.type == "cuda":
            buf, hdl = _symmetric_buffer(self.world * self.chunk * self.num_heads, self.device,
                                         group, self.world)
            if buf is not None:
                self._padded = buf[:self.world * self.chunk * self.num_heads]
                self._padded.zero_()
                self._symm = hdl
        if self._padded is None:
            self._padded = torch.zeros(self.world * self.chunk * self.num_heads,
                                       dtype=torch.float32, device=self.device)
        out_shape = (self.nnz, self.num_heads) if len(self.feat_shape) == 2 else (self.nnz,)
        self.out = self._padded[:self.nnz * self.num_heads].view(out_shape)
        self._slot = self._padded[self.rank * self.chunk * self.num_heads:
                                  (self.rank + 1) * self.chunk * self.num_heads]
        self._local = self.make_local(row[lo:hi], col[lo:hi])
        if self._symm is not None:
            off = self.rank * self.chunk * self.num_heads * 4
            self.peer_mode = "store" if peer_mode == "auto" else peer_mode
            self.module.set_extra_outputs([int(p) + off for r, p in
                                           enumerate(self._symm.buffer_ptrs) if r != self.rank],
                                          push=self.peer_mode == "push")
            self._symm.barrier()

    def make_local(self, row_local, col_local):
        from .module import VanillaSDDMMcuda
        to_np = lambda a: a.cpu().numpy() if isinstance(a, torch.Tensor) else np.asarray(a)
        coo = sp.coo_matrix((np.zeros(row_local.shape[0], np.float32),
                             (to_np(row_local), to_np(col_local))),
                            shape=(self.n_rows, self.n_cols))
        m = VanillaSDDMMcuda(coo, device_id=self.device.index or 0)
        m.build([Placeholder((self.n_cols,) + self.feat_shape),
                 Placeholder((self.n_rows,) + self.feat_shape)], {},
                {"num_cuda_blocks": min(8192, coo.nnz)})
        n_local = self.edge_hi - self.edge_lo
        shape = (n_local, self.num_heads) if len(self.feat_shape) == 2 else (n_local,)
        m.out_tvm = NDArray(self._slot[:n_local * self.num_heads].view(shape), m.ctx)
        self.module = m
        return lambda src, dst: m.run([src, dst])

    @property
    def gather_mode(self):
        if self.world == 1:
            return "none"
        return ("peer_" + self.peer_mode) if self._symm is not None else "nccl"

    def compute_local(self, src, dst):
        if self._symm is not None:
            self._symm.barrier()   # as in ShardedSpMM.compute_local
        if self.edge_hi > self.edge_lo:
            self._local(src, dst)

    def gather(self):
        if self.world > 1 and self.chunk:
            if self._symm is not None:
                self._symm.barrier()      # every rank's stores into this buffer have landed
            else:
                dist.all_gather_into_tensor(self._padded, self._slot, group=self.group)

    def run(self, src, dst):
        """src (n_cols, ...) is indexed by col, dst (n_rows, ...) by row, both replicated.
        Returns the full output in the given edge order, identical on every rank."""
        self.compute_local(src, dst)
        self.gather()
        return self.out

    def run_host(self, src_host, dst_host, out_host):
        """End to end from pinned HOST buffers; each rank downloads its own edge range."""
        if self.world == 1:
            return self.module.run_host(src_host, dst_host, out_host)
        if getattr(self, "_stage", None) is None:
            self._stage = (torch.empty((self.n_cols,) + self.feat_shape, dtype=torch.float32,
                                       device=self.device),
                           torch.empty((self.n_rows,) + self.feat_shape, dtype=torch.float32,
                                       device=self.device))
        self._stage[0].copy_(src_host, non_blocking=True)
        self._stage[1].copy_(dst_host, non_blocking=True)
        self.run(self._stage[0], self._stage[1])
        out_host[self.edge_lo:self.edge_hi].copy_(self.out[self.edge_lo:self.edge_hi],
                                                  non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        return out_host

    def num_launches(self):
        return self.module.num_launches() if hasattr(self, "module") else 0
