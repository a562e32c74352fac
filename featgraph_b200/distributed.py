"""One-process-per-GPU sharding of SpMM and SDDMM over ``torch.distributed``.

The reference is single-device (python/featgraph/module/spmm.py:218, sddmm.py:185); this
is the multi-GPU extension: SpMM is split into contiguous destination-row blocks that
hold about nnz / world nonzeros each, SDDMM into equal contiguous edge ranges.  The
dense features are replicated on every rank; each rank computes its block straight into
its slice of a full-size output, and every rank ends up with the whole result (what a
following GNN layer needs).  On GPUs the full-size outputs live in symmetric memory and
the kernels deliver each finished row / edge result to every peer's copy themselves --
plain stores over NVLink to each peer ('store'), or one store through the NVLink
switch's multicast address ('mcast') -- bracketed by two device-side barriers per call
whose waits are bounded (``PeerSync``); where that cannot be set up the slices are
exchanged with NCCL collectives instead.

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
    """world + 1 edge bounds: equal ranges of a multiple of 32 edges (C ABI, host)."""
    bounds = (ctypes.c_int64 * (world + 1))()
    _lib.check(_lib.load().fg_shard_edges(int(nnz), world, bounds))
    return np.array(bounds[:], dtype=np.int64)


def _all_agree(ok, device, group):
    flag = torch.tensor([1 if ok else 0], device=device, dtype=torch.int32)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    return int(flag) == 1


def _symmetric_buffer(numel, device, group, world, dtype=torch.float32):
    """A buffer of ``numel`` elements that every rank of the group can address directly
    (torch symmetric memory over NVLink), or None if that cannot be set up on every rank.
    Returns (tensor, handle)."""
    ok, buf, hdl = True, None, None
    try:
        import torch.distributed._symmetric_memory as symm_mem
        pg = group if group is not None else dist.group.WORLD
        buf = symm_mem.empty(max(int(numel), 1), dtype=dtype, device=device)
        hdl = symm_mem.rendezvous(buf, pg)
        ok = len(hdl.buffer_ptrs) == world
    except Exception:                      # no peer access / API missing: use NCCL instead
        ok = False
    if not _all_agree(ok, device, group):
        return None, None
    return buf, hdl


def _multicast_base(hdl, device, group):
    """The handle's multicast address (one address that the NVLink switch maps onto every
    rank's copy of the buffer), or 0 unless every rank has one."""
    try:
        ptr = int(hdl.multicast_ptr)
    except Exception:
        ptr = 0
    return ptr if _all_agree(ptr != 0, device, group) else 0


def _group_info(group):
    if group is None and not dist.is_initialized():
        return 0, 1
    return dist.get_rank(group), dist.get_world_size(group)


class PeerBarrierTimeout(RuntimeError):
    """A device-side barrier gave up waiting for a peer."""


class PeerSync(object):
    """Device-side barrier between the ranks' GPUs with bounded waits (fg_peer_barrier).

    Each rank holds ``world`` 32-bit counters in symmetric memory; barrier number k writes k
    into this rank's slot on every peer and waits until all of its own slots hold k.  A wait
    polls ``max_polls`` times at most (default: a few seconds) -- a rank that raised between
    two steps therefore cannot leave the others' GPUs spinning: their barrier kernel writes
    a status word and returns, and ``check()`` raises ``PeerBarrierTimeout`` on the host.
    """

    _cache = {}

    @classmethod
    def get(cls, device, group=None):
        """The group's PeerSync on this device (made once), or None if symmetric memory
        cannot be set up.  Collective: every rank of the group must call it."""
        key = (str(device), id(group) if group is not None else 0)
        if key not in cls._cache:
            cls._cache[key] = cls._make(torch.device(device), group)
        return cls._cache[key]

    @classmethod
    def _make(cls, device, group):
        rank, world = _group_info(group)
        buf, hdl = _symmetric_buffer(64, device, group, world, dtype=torch.int32)
        if buf is None:
            return None
        buf.zero_()
        torch.cuda.synchronize(device)
        dist.barrier(group=group)           # nobody signals before everybody's flags are zero
        torch.cuda.synchronize(device)
        self = cls()
        self.device, self.group, self.rank, self.world = device, group, rank, world
        self._buf, self._hdl = buf, hdl
        self._flags = (ctypes.c_void_p * world)(*[int(p) for p in hdl.buffer_ptrs])
        self._status = torch.zeros(1, dtype=torch.int32, device=device)
        self.epoch = 0
        self.max_polls = -1
        return self

    def barrier(self):
        """Enqueue one barrier on the current stream (asynchronous)."""
        self.epoch = (self.epoch + 1) & 0xFFFFFFFF
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        _lib.check(_lib.load().fg_peer_barrier(
            self._flags, self.rank, self.world, self.epoch,
            ctypes.c_void_p(self._status.data_ptr()), self.max_polls, self.device.index or 0,
            stream))

    def check(self):
        """Synchronise and raise if any barrier since the last check gave up."""
        code = int(self._status.item())
        if code:
            self._status.zero_()
            raise PeerBarrierTimeout("rank %d: a device-side barrier gave up waiting for rank %d"
                                     % (self.rank, code - 1))
        return 0


def _pick_peer_mode(peer_mode, mcast_base):
    """'store' | 'mcast' | 'push' from the caller's wish and what the hardware offers."""
    if peer_mode == "auto":
        return "store"
    if peer_mode == "mcast" and not mcast_base:
        return "store"
    return peer_mode


class _Sharded(object):
    """What the two sharded operators share: the replicated-feature upload of run_host."""

    def _feature_stage(self, name, n, tail):
        """(padded, per): a (world * ceil(n / world), *tail) device buffer whose first n rows
        are the replicated array, and the rows per rank."""
        cache = self.__dict__.setdefault("_stages", {})
        if name not in cache:
            per = -(-n // self.world)
            padded = torch.empty((self.world * per,) + tuple(tail), dtype=torch.float32,
                                 device=self.device)
            cache[name] = (padded, per)
        return cache[name]

    def _upload_replicated(self, name, host):
        """Each rank copies 1/world of ``host`` (pinned, identical on every rank) over PCIe and
        the blocks are exchanged over NVLink (one in-place NCCL all-gather), so a replicated
        array costs every host link 1/world of its bytes.  Returns the device array."""
        n = host.shape[0]
        padded, per = self._feature_stage(name, n, host.shape[1:])
        lo, hi = min(self.rank * per, n), min((self.rank + 1) * per, n)
        slot = padded[self.rank * per:(self.rank + 1) * per]
        if hi > lo:
            slot[:hi - lo].copy_(host[lo:hi], non_blocking=True)
        dist.all_gather_into_tensor(padded.view(-1), slot.reshape(-1), group=self.group)
        return padded[:n]


class ShardedSpMM(_Sharded):
    """Row-block sharded CSR SpMM.

    adj_scipy_csr : the FULL matrix (every rank passes the same one)
    feat_len      : feature length F
    device        : torch device of this rank
    peer_mode     : fused path only -- 'store': the kernels store every finished row into each
                    peer's output; 'mcast': one store per row through the NVLink switch's
                    multicast address; 'auto': 'store'
    """

    def __init__(self, adj_scipy_csr, feat_len, device, group=None, schedule_args=None,
                 fused_gather=True, peer_mode="auto"):
        self.group = group
        self.rank, self.world = _group_info(group)
        self.device = torch.device(device)
        self._symm = self._sync = None
        self.peer_mode = "none"
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
            self._sync = PeerSync.get(self.device, group)
            buf, hdl = (None, None) if self._sync is None else _symmetric_buffer(
                self.n_rows * self.feat_len, self.device, group, self.world)
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
            mcast = _multicast_base(self._symm, self.device, group) if peer_mode == "mcast" else 0
            self.peer_mode = _pick_peer_mode(peer_mode, mcast)
            if self.peer_mode == "mcast":
                self.module.set_multicast_output(mcast + off)
            else:
                self.peer_mode = "store"
                self.module.set_extra_outputs([int(p) + off for r, p in
                                               enumerate(self._symm.buffer_ptrs)
                                               if r != self.rank])
            self._sync.barrier()

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
        """'peer_store' / 'peer_mcast' (kernels write into every rank's output), 'nccl', or
        'none'."""
        if self.world == 1:
            return "none"
        return ("peer_" + self.peer_mode) if self._symm is not None else "nccl"

    def launch_local(self, x):
        """This rank's kernels only (no barrier, no exchange)."""
        self._local(x)

    def compute_local(self, x):
        if self._symm is not None:
            # peers store into this rank's output: they may start only when this rank's
            # stream has passed everything that read the previous result
            self._sync.barrier()
        self._local(x)

    def gather(self):
        """Uneven all-gather of the row blocks: one broadcast per owner -- or, with the
        fused path, just the barrier after which every rank's stores have landed."""
        if self.world == 1:
            return
        if self._symm is not None:
            self._sync.barrier()
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
        """End to end from pinned HOST buffers: each rank uploads 1/world of the features and
        the ranks exchange them over NVLink, compute their row blocks, all-gather, and
        download their own block into ``y_host`` (the ranks' blocks together are the whole
        result).  Synchronises the stream."""
        if self.world == 1:
            return self.module.run_host(x_host, y_host)
        self.run(self._upload_replicated("x", x_host))
        y_host[self.row_lo:self.row_hi].copy_(self._views[self.rank], non_blocking=True)
        if self.device.type == "cuda":
            torch.cuda.current_stream(self.device).synchronize()
        return y_host

    def device_status(self):
        """Synchronise; raises if a bounded device-side wait (giant-row kernel, barrier) gave
        up since the last check."""
        code = self.module.device_status() if hasattr(self, "module") else 0
        if self._sync is not None:
            self._sync.check()
        return code

    def num_launches(self):
        return self.module.num_launches() if hasattr(self, "module") else 0


class ShardedSDDMM(_Sharded):
    """Edge-range sharded COO SDDMM (single- or multi-head).

    row, col : the FULL edge list (numpy int32 or torch tensors); every rank passes the same
    """

    def __init__(self, row, col, n_rows, n_cols, feat_shape, device, group=None,
                 fused_gather=True, peer_mode="auto"):
        """peer_mode (fused path only): 'store' -- the SDDMM kernel stores each result into
        every peer's output itself; 'mcast' -- one store per result through the NVLink
        switch's multicast address; 'push' -- a copy kernel pushes finished pieces to the
        peers while the next piece computes; 'auto' -- 'store'."""
        self.group = group
        self.rank, self.world = _group_info(group)
        self.device = torch.device(device)
        self._symm = self._sync = None
        self.peer_mode = "none"
        self.n_rows, self.n_cols = int(n_rows), int(n_cols)
        self.feat_shape = (feat_shape,) if isinstance(feat_shape, int) else tuple(feat_shape)
        self.num_heads = self.feat_shape[0] if len(self.feat_shape) == 2 else 1
        self.nnz = int(row.shape[0])
        # equal ranges (fg_shard_edges), so that one all-gather assembles the padded output;
        # a multiple of 32 edges each: every rank's slice then starts on a 128-byte boundary,
        # so a warp's 32 results are one aligned line in the peers' memory -- unaligned slices
        # made the in-kernel peer stores 1.7 times slower on 8 GPUs
        self.bounds = shard_edges(self.nnz, self.world)
        self.chunk = int(self.bounds[1])
        lo, hi = int(self.bounds[self.rank]), int(self.bounds[self.rank + 1])
        self.edge_lo, self.edge_hi = lo, hi
        self._padded = None
        if fused_gather and self.world > 1 and self.device.type == "cuda":
            self._sync = PeerSync.get(self.device, group)
            buf, hdl = (None, None) if self._sync is None else _symmetric_buffer(
                self.world * self.chunk * self.num_heads, self.device, group, self.world)
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
            mcast = _multicast_base(self._symm, self.device, group) if peer_mode == "mcast" else 0
            self.peer_mode = _pick_peer_mode(peer_mode, mcast)
            if self.peer_mode == "mcast":
                self.module.set_multicast_output(mcast + off)
            else:
                self.module.set_extra_outputs([int(p) + off for r, p in
                                               enumerate(self._symm.buffer_ptrs)
                                               if r != self.rank],
                                              push=self.peer_mode == "push")
            self._sync.barrier()

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

    def launch_local(self, src, dst):
        """This rank's kernel only (no barrier, no exchange)."""
        if self.edge_hi > self.edge_lo:
            self._local(src, dst)

    def compute_local(self, src, dst):
        if self._symm is not None:
            self._sync.barrier()   # as in ShardedSpMM.compute_local
        self.launch_local(src, dst)

    def gather(self):
        if self.world > 1 and self.chunk:
            if self._symm is not None:
                self._sync.barrier()      # every rank's stores into this buffer have landed
            else:
                dist.all_gather_into_tensor(self._padded, self._slot, group=self.group)

    def run(self, src, dst):
        """src (n_cols, ...) is indexed by col, dst (n_rows, ...) by row, both replicated.
        Returns the full output in the given edge order, identical on every rank."""
        self.compute_local(src, dst)
        self.gather()
        return self.out

    def run_host(self, src_host, dst_host, out_host):
        """End to end from pinned HOST buffers; each rank uploads 1/world of both feature
        arrays (exchanged over NVLink) and downloads its own edge range."""
        if self.world == 1:
            return self.module.run_host(src_host, dst_host, out_host)
        src = self._upload_replicated("src", src_host)
        dst = self._upload_replicated("dst", dst_host)
        self.run(src, dst)
        out_host[self.edge_lo:self.edge_hi].copy_(self.out[self.edge_lo:self.edge_hi],
                                                  non_blocking=True)
        if self.device.type == "cuda":
            torch.cuda.current_stream(self.device).synchronize()
        return out_host

    def device_status(self):
        """Raises if a bounded device-side wait gave up (peer barrier, TMA staging); else 0."""
        if self._sync is not None:
            self._sync.check()
        return self.module.device_status() if hasattr(self, "module") else 0

    def num_launches(self):
        return self.module.num_launches() if hasattr(self, "module") else 0


class OverlappedPair(object):
    """One SpMM and one SDDMM that do not depend on each other, run as one chain.

    On a shard the SpMM is bound by the dependent add chain of its longest row: a handful of
    whole-SM CTAs run for hundreds of microseconds after the rest of the SpMM is done, and
    the SMs idle.  Here the SDDMM is launched programmatically behind the SpMM in the SAME
    stream (fg_next_launch_options): it is dispatched as soon as the SpMM's last kernel is
    resident and fills the machine under the giant rows' tail; and the pair shares ONE
    barrier before and ONE after instead of two each.  Measured on 4 GPUs (feat_len 64, ms
    per step): one after the other 1.48, this chain 1.37.  What was tried and dropped: the
    SDDMM on a second stream beside the SpMM -- its CTAs take every SM first and the giant
    rows, which need a whole SM each, start when it has drained (1.46); the SDDMM between
    the SpMM's giant rows and its other rows (1.43); the same with the SDDMM's grid bounded
    so that both are resident at once (1.65 to 1.97: the SDDMM needs its full occupancy).
    """

    def __init__(self, spmm, sddmm, order="chain"):
        """order: "chain" -- the SpMM, then the SDDMM behind it; "split" -- the SpMM's long
        rows (giant and heavy: the dependent chains), the SDDMM, then the SpMM's light rows,
        so that the SDDMM's results start crossing NVLink at once."""
        assert order in ("chain", "split")
        self.order = order
        self.spmm, self.sddmm = spmm, sddmm
        self.device = spmm.device
        self.fused = spmm._symm is not None and sddmm._symm is not None
        self.chained = self.device.type == "cuda" and hasattr(spmm, "module") \
            and hasattr(sddmm, "module")

    def run(self, x, src, dst):
        """Returns (spmm.out, sddmm.out), whole and identical on every rank."""
        spmm, sddmm = self.spmm, self.sddmm
        if self.fused:
            spmm._sync.barrier()
        split = self.order == "split" and self.chained
        if split:
            spmm.module.run([x], launch_flags=_lib.SPMM_LONG_ROWS_ONLY)
        else:
            spmm.launch_local(x)
        if sddmm.edge_hi > sddmm.edge_lo:
            if self.chained:
                sddmm.module.run([src, dst], launch_flags=_lib.LAUNCH_PROGRAMMATIC)
            else:
                sddmm.launch_local(src, dst)
        if split:
            spmm.module.run([x], launch_flags=_lib.SPMM_SKIP_LONG_ROWS | _lib.LAUNCH_PROGRAMMATIC)
        if self.fused:
            spmm._sync.barrier()
        elif spmm.world > 1:
            spmm.gather()
            sddmm.gather()
        return spmm.out, sddmm.out
