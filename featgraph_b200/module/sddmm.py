"""SDDMM module classes with the interface of python/featgraph/module/sddmm.py.

Single-head use is unchanged from the reference; ``compute_args={'num_heads': H}`` (or
3-D placeholders (N, H, D)) selects the multi-head kernel, whose output is (nnz, H).
"""
import numpy as np
import torch

from .. import _lib
from ..op import vanilla_sddmm, schedule_vanilla_sddmm_cuda_tree_reduce
from ..op.spec import no_x86
from ..runtime import Placeholder, array, cpu, gpu, zeros
from ..util import util_partition_adj_coo_2d
from .base import as_device_tensor, current_stream_handle, ptr, time_launches


class SDDMMbase(object):
    """Base of the SDDMM-like kernels (counterpart of SDDMMbase, sddmm.py:11-165).

    Edges keep the order of the COO matrix given (sddmm.py:51-52); the adjacency values
    are never read.
    """

    def __init__(self, adj_scipy, num_row_partitions=1, num_col_partitions=1):
        coo = adj_scipy if adj_scipy.format == "coo" else adj_scipy.tocoo()
        self._num_rows, self._num_cols = int(coo.shape[0]), int(coo.shape[1])
        assert num_row_partitions >= 1, "num_row_partitions should be larger than or equal to 1"
        assert num_col_partitions >= 1, "num_col_partitions should be larger than or equal to 1"
        self._num_row_partitions = int(num_row_partitions)
        self._num_col_partitions = int(num_col_partitions)
        self._target = self._ctx = self._compute_func = self._schedule_func = None
        self._register()

        if self._num_row_partitions > 1 or self._num_col_partitions > 1:
            # 2-D blocking; output position i holds edge edge_id_list[i], so sorting the
            # ids gives the permutation back to the caller's order (sddmm.py:45-49).
            edge_ids, rows, cols = self._preprocess_adj(coo, self._num_row_partitions,
                                                        self._num_col_partitions)
            self._edge_mapping = np.argsort(edge_ids)
        else:
            rows, cols = coo.row, coo.col
        self._adj_row_indices = self._index_array(rows, "row indices")
        self._adj_col_indices = self._index_array(cols, "col indices")
        self._adj_row_indices_placeholder = Placeholder(self._adj_row_indices.shape, "int32",
                                                        "adj_row_indices_placeholder")
        self._adj_col_indices_placeholder = Placeholder(self._adj_col_indices.shape, "int32",
                                                        "adj_col_indices_placeholder")
        self._adj_row_indices_tvm = array(self._adj_row_indices, self._ctx)
        self._adj_col_indices_tvm = array(self._adj_col_indices, self._ctx)
        self._func = None
        self._spec = None
        self.out_tvm = None

    @staticmethod
    def _index_array(a, what):
        if a.dtype == np.int32:
            return np.ascontiguousarray(a)
        if a.size and (a.max() > np.iinfo(np.int32).max or a.min() < 0):
            raise ValueError("%s do not fit int32" % what)
        return np.ascontiguousarray(a.astype(np.int32))

    def _preprocess_adj(self, adj_scipy_coo, num_row_partitions=1, num_col_partitions=1):
        return util_partition_adj_coo_2d(adj_scipy_coo, num_row_partitions, num_col_partitions)

    def _register(self):
        raise NotImplementedError("Please register target, ctx, compute_func, and schedule_func.")

    def _specialise(self, input_placeholders, compute_args, schedule_args):
        if self._target != "cuda":
            raise no_x86(type(self).__name__ + ".build")
        out = self._compute_func(*input_placeholders, self._adj_row_indices_placeholder,
                                 self._adj_col_indices_placeholder, **compute_args)
        sched = self._schedule_func(out, **schedule_args)
        src, dst = input_placeholders[0], input_placeholders[1]
        if src.shape[0] != self._num_cols:
            raise ValueError("SrcFeat has %d rows, the adjacency has %d columns (SrcFeat is "
                             "indexed by col)" % (src.shape[0], self._num_cols))
        if dst.shape[0] != self._num_rows:
            raise ValueError("DstFeat has %d rows, the adjacency has %d rows (DstFeat is "
                             "indexed by row)" % (dst.shape[0], self._num_rows))
        if src.dtype != "float32" or dst.dtype != "float32":
            raise TypeError("only float32 features are supported")
        return out, sched

    def build(self, input_placeholders, compute_args, schedule_args):
        """Fix the static shapes and allocate the zero-filled output.

        input_placeholders : [SrcFeat (num_cols, F), DstFeat (num_rows, F)], or both 3-D
            (N, H, D) for the multi-head kernel
        compute_args : e.g. ``{'num_heads': H}``, ``{'msg_op': 'sub', 'reduce_op': 'max'}``
        schedule_args : e.g. ``{'num_cuda_blocks': n}`` (checked as in the reference, then
            a hint only)
        """
        out, sched = self._specialise(input_placeholders, compute_args, schedule_args)
        _lib.load()
        self._spec, self._func = out, sched
        self.out_tvm = zeros(out.shape, out.dtype, self._ctx)
        # one head over a list whose runs of 32 consecutive edges nearly all share a row:
        # the kernel that keeps the dst operand in registers (FG_SDDMM_ROW_REGISTERS)
        flags = getattr(self, "default_launch_flags", 0) & ~_lib.SDDMM_ROW_REGISTERS
        if out.attrs["num_heads"] == 1 and out.attrs["feat_len"] % 32 == 0 \
                and self._single_row_tile_share() >= 0.75:
            flags |= _lib.SDDMM_ROW_REGISTERS
        self.default_launch_flags = flags

    def _single_row_tile_share(self):
        """Share of the 32-edge tiles of the edge list whose edges all have one row index
        (computed once per module, on the host)."""
        if getattr(self, "_tile_share", None) is None:
            rows = self._adj_row_indices
            full = (rows.shape[0] // 32) * 32
            if rows.dtype != np.int32 or full == 0:
                self._tile_share = 0.0
            else:
                t = rows[:full].reshape(-1, 32)
                self._tile_share = float((t[:, 0] == t[:, 31]).mean()
                                         if bool((np.diff(rows) >= 0).all())
                                         else (t == t[:, :1]).all(axis=1).mean())
        return self._tile_share

    def lower_to_ir(self, input_placeholders, compute_args, schedule_args):
        """Debug text of the launch ``build`` would choose (sddmm.py:94-113)."""
        import ctypes
        out, sched = self._specialise(input_placeholders, compute_args, schedule_args)
        buf = ctypes.create_string_buffer(2048)
        _lib.check(_lib.load().fg_sddmm_describe(out.shape[0], out.attrs["feat_len"],
                                                 out.attrs["num_heads"], buf, len(buf)))
        text = buf.value.decode()
        if out.attrs["num_heads"] == 1 and out.attrs["feat_len"] % 32 == 0:
            share = self._single_row_tile_share()
            text += (" | %.0f %% of the 32-edge tiles lie inside one run of equal rows: %s"
                     % (100 * share, "sddmm_rowreg_kernel (dst operand in registers, "
                        "FG_SDDMM_ROW_REGISTERS) instead" if share >= 0.75 else "tile kernel kept"))
        return text + " | hints: %r" % (sched.hints,)

    def set_extra_outputs(self, device_pointers, push=False):
        """Also deliver every result to these device addresses (peer-mapped copies of this
        edge range's output on other GPUs, at most 7): the multi-GPU path's fused all-gather.
        push=False: the SDDMM kernel stores each result to all of them itself.  push=True:
        the edge range is computed in pieces and a copy kernel pushes piece k to the peers
        while piece k+1 computes.  Measured on 8 GPUs with 128-byte aligned slices: in-kernel
        stores 0.67 ms per SDDMM, push 1.01 ms; on 2 GPUs 1.49 against 1.78 ms."""
        self._extra_outputs = [int(p) for p in device_pointers]
        self._push_outputs = bool(push)
        self._mcast_output = None

    def set_multicast_output(self, mcast_pointer):
        """Deliver every result with ONE store to this address instead: the position of the
        edge range inside an NVLink-switch multicast mapping of the output, which the switch
        writes into every GPU's copy (this GPU's included).  None switches it off."""
        self._mcast_output = int(mcast_pointer) if mcast_pointer else None
        self._extra_outputs = None

    def _launch(self, src, dst, flags=0, max_ctas=0):
        """``flags`` / ``max_ctas``: fg_next_launch_options for this one call."""
        if flags or max_ctas:
            _lib.check(_lib.load().fg_next_launch_options(int(flags), int(max_ctas)))
        a = self._spec.attrs
        if (a["msg_op"], a["reduce_op"]) != ("mul", "sum"):
            if getattr(self, "_mcast_output", None) or getattr(self, "_extra_outputs", None):
                raise NotImplementedError("extra outputs are provided for the multiply / sum "
                                          "operator pair only")
            _lib.check(_lib.load().fg_sddmm_coo_f32_general(
                ptr(self._adj_row_indices_tvm.torch), ptr(self._adj_col_indices_tvm.torch),
                ptr(src), ptr(dst), ptr(self.out_tvm.torch), self._adj_row_indices.shape[0],
                self._num_rows, self._num_cols, a["feat_len"], a["num_heads"],
                _lib.MSG_OPS.index(a["msg_op"]), _lib.REDUCE_OPS.index(a["reduce_op"]),
                self._ctx.device_id, current_stream_handle(self._ctx)))
            return
        mcast = getattr(self, "_mcast_output", None)
        if mcast:
            import ctypes
            _lib.check(_lib.load().fg_sddmm_coo_f32_mcast(
                ptr(self._adj_row_indices_tvm.torch), ptr(self._adj_col_indices_tvm.torch),
                ptr(src), ptr(dst), ctypes.c_void_p(mcast), self._adj_row_indices.shape[0],
                self._num_rows, self._num_cols, a["feat_len"], a["num_heads"],
                self._ctx.device_id, current_stream_handle(self._ctx)))
            return
        extra = getattr(self, "_extra_outputs", None)
        if extra and getattr(self, "_push_outputs", False):
            import ctypes
            peers = (ctypes.c_void_p * len(extra))(*extra)
            _lib.check(_lib.load().fg_sddmm_coo_f32_push(
                ptr(self._adj_row_indices_tvm.torch), ptr(self._adj_col_indices_tvm.torch),
                ptr(src), ptr(dst), ptr(self.out_tvm.torch), peers, len(extra),
                self._adj_row_indices.shape[0], self._num_rows, self._num_cols, a["feat_len"],
                a["num_heads"], self._ctx.device_id, current_stream_handle(self._ctx)))
            return
        if extra:
            import ctypes
            outs = (ctypes.c_void_p * (1 + len(extra)))(self.out_tvm.torch.data_ptr(), *extra)
            _lib.check(_lib.load().fg_sddmm_coo_f32_multi(
                ptr(self._adj_row_indices_tvm.torch), ptr(self._adj_col_indices_tvm.torch),
                ptr(src), ptr(dst), outs, len(outs), self._adj_row_indices.shape[0],
                self._num_rows, self._num_cols, a["feat_len"], a["num_heads"],
                self._ctx.device_id, current_stream_handle(self._ctx)))
            return
        _lib.check(_lib.load().fg_sddmm_coo_f32(
            ptr(self._adj_row_indices_tvm.torch), ptr(self._adj_col_indices_tvm.torch),
            ptr(src), ptr(dst), ptr(self.out_tvm.torch), self._adj_row_indices.shape[0],
            self._num_rows, self._num_cols, a["feat_len"], a["num_heads"],
            self._ctx.device_id, current_stream_handle(self._ctx)))

    def _checked_inputs(self, input_tvm_ndarrays):
        if self._spec is None:
            raise RuntimeError("build() must be called before run()")
        if len(input_tvm_ndarrays) != 2:
            raise ValueError("SDDMM takes exactly two input arrays (SrcFeat, DstFeat)")
        sp, dp = self._spec.inputs[0], self._spec.inputs[1]
        src = as_device_tensor(input_tvm_ndarrays[0], self._ctx, sp.shape, sp.dtype, "SrcFeat")
        dst = as_device_tensor(input_tvm_ndarrays[1], self._ctx, dp.shape, dp.dtype, "DstFeat")
        return src, dst

    def run(self, input_tvm_ndarrays, launch_flags=0, max_ctas=0):
        """Launch with [SrcFeat (indexed by col), DstFeat (indexed by row)]; returns
        ``self.out_tvm``, the same array every call (sddmm.py:115-129).  ``launch_flags`` /
        ``max_ctas`` (additions): fg_next_launch_options for this call."""
        src, dst = self._checked_inputs(input_tvm_ndarrays)
        flags = launch_flags | getattr(self, "default_launch_flags", 0)
        if flags & _lib.SDDMM_TMA_STAGING:
            flags &= ~_lib.SDDMM_ROW_REGISTERS
        self._launch(src, dst, flags, max_ctas)
        return self.out_tvm

    def measure_average_time(self, input_tvm_ndarrays, num_runs):
        """Mean kernel time in seconds over ``num_runs`` launches (sddmm.py:131-150)."""
        src, dst = self._checked_inputs(input_tvm_ndarrays)
        flags = getattr(self, "default_launch_flags", 0)
        return time_launches(self._ctx, lambda: self._launch(src, dst, flags), num_runs)

    def run_host(self, src_host, dst_host, out_host):
        """End-to-end call on HOST buffers (ideally pinned): uploads both feature arrays,
        launches, downloads the result into ``out_host`` and synchronises; the edge lists
        stay on the device.  Goes through the C ABI's fg_sddmm_coo_f32_host."""
        if self._spec is None:
            raise RuntimeError("build() must be called before run_host()")
        sp_, dp_ = self._spec.inputs[0], self._spec.inputs[1]
        for a, shape, what in ((src_host, sp_.shape, "src_host"), (dst_host, dp_.shape, "dst_host"),
                               (out_host, self._spec.shape, "out_host")):
            if not (isinstance(a, torch.Tensor) and a.device.type == "cpu" and a.is_contiguous()
                    and a.dtype == torch.float32 and tuple(a.shape) == tuple(shape)):
                raise ValueError("%s must be a contiguous float32 CPU tensor of shape %r"
                                 % (what, tuple(shape)))
        dev = self._ctx.torch_device
        if getattr(self, "_stage", None) is None or tuple(self._stage[0].shape) != sp_.shape \
                or tuple(self._stage[1].shape) != dp_.shape:
            self._stage = (torch.empty(sp_.shape, dtype=torch.float32, device=dev),
                           torch.empty(dp_.shape, dtype=torch.float32, device=dev))
        a = self._spec.attrs
        if getattr(self, "default_launch_flags", 0):
            _lib.check(_lib.load().fg_next_launch_options(self.default_launch_flags, 0))
        _lib.check(_lib.load().fg_sddmm_coo_f32_host(
            ptr(self._adj_row_indices_tvm.torch), ptr(self._adj_col_indices_tvm.torch),
            ptr(src_host), ptr(dst_host), ptr(out_host), ptr(self._stage[0]),
            ptr(self._stage[1]), ptr(self.out_tvm.torch), self._adj_row_indices.shape[0],
            self._num_rows, self._num_cols, a["feat_len"], a["num_heads"],
            self._ctx.device_id, current_stream_handle(self._ctx)))
        return out_host

    def device_status(self):
        """Synchronise and return the status word of the kernel that stages its tiles with
        TMA copies (``launch_flags=_lib.SDDMM_TMA_STAGING``): 0 when every bounded wait
        completed; raises FeatGraphError otherwise (once: the word is then cleared)."""
        import ctypes
        status = ctypes.c_int32(0)
        _lib.check(_lib.load().fg_sddmm_status(self._ctx.device_id, ctypes.byref(status)))
        return int(status.value)

    def num_launches(self):
        if self._spec is None:
            return 0
        a = self._spec.attrs
        return int(_lib.load().fg_sddmm_num_launches(self._adj_row_indices.shape[0],
                                                     a["feat_len"], a["num_heads"]))

    _cuda_partitioning = False   # the reference's cuda class forces one partition

    @property
    def edge_mapping(self):
        assert self._target != "cuda" or self._cuda_partitioning, \
            "no graph partitioning on cuda, no edge_mapping"
        assert self._num_row_partitions > 1 or self._num_col_partitions > 1, \
            "no graph partitioning, no edge_mapping"
        return self._edge_mapping

    @property
    def ctx(self):
        return self._ctx

    @property
    def target(self):
        return self._target


class VanillaSDDMMcuda(SDDMMbase):
    """COO SDDMM on the GPU (counterpart of VanillaSDDMMcuda, sddmm.py:179-187);
    ``device_id`` as in VanillaSpMMcuda."""

    def __init__(self, adj_scipy, device_id=0):
        self._device_id = int(device_id)
        super(VanillaSDDMMcuda, self).__init__(adj_scipy, num_row_partitions=1,
                                               num_col_partitions=1)

    def _register(self):
        if not torch.cuda.is_available():
            raise RuntimeError("VanillaSDDMMcuda needs a CUDA device; there is no CPU fallback")
        _lib.load()
        self._target = "cuda"
        self._ctx = gpu(self._device_id)
        self._compute_func = vanilla_sddmm
        self._schedule_func = schedule_vanilla_sddmm_cuda_tree_reduce


class PartitionedSDDMMcuda(VanillaSDDMMcuda):
    """The reference's 2-D edge blocking (sddmm.py:45-49, adj_partitioning.py:60-128) on the
    GPU, where the reference's own cuda class forces a single partition (sddmm.py:180-181).

    The edges are reordered block by block (row partition major, column partition minor, the
    caller's order inside a block) exactly as ``VanillaSDDMMx86`` does, the same kernels run
    over the reordered list, and -- as there -- position i of the output holds the edge that
    ``edge_mapping`` maps back: ``out[edge_mapping]`` is in the caller's order.  Per-edge
    results do not depend on the order, so they are bit-identical to the unpartitioned ones.
    Column partitions confine a stretch of edges to a window of SrcFeat rows: when SrcFeat
    exceeds L2 (feat_len >= 256 on the 232 965-vertex graph) the window's rows are then
    gathered from L2 instead of DRAM.
    """
    _cuda_partitioning = True

    def __init__(self, adj_scipy, num_row_partitions=1, num_col_partitions=1, device_id=0):
        self._device_id = int(device_id)
        if num_row_partitions > 1 or num_col_partitions > 1:
            # the reference's utility converts through CSR, which merges duplicate edges
            # and adds up their ids (adj_partitioning.py:92-95): refuse instead
            coo = adj_scipy if adj_scipy.format == "coo" else adj_scipy.tocoo()
            key = coo.row.astype(np.int64) * int(coo.shape[1]) + coo.col
            if np.unique(key).shape[0] != key.shape[0]:
                raise ValueError("edge blocking needs a duplicate-free edge list")
        SDDMMbase.__init__(self, adj_scipy, num_row_partitions, num_col_partitions)


class VanillaSDDMMx86(SDDMMbase):
    """Name kept from the reference (sddmm.py:168-176).  The 2-D partitioning and
    ``edge_mapping`` work, but this backend has no x86 code path: ``build`` raises
    NotImplementedError."""

    def __init__(self, adj_scipy, num_row_partitions=1, num_col_partitions=1):
        super(VanillaSDDMMx86, self).__init__(adj_scipy, num_row_partitions, num_col_partitions)

    def _register(self):
        self._target = "llvm"
        self._ctx = cpu(0)
        self._compute_func = None
        self._schedule_func = None
