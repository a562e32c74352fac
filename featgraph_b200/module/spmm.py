"""SpMM module classes with the interface of python/featgraph/module/spmm.py.

``VanillaSpMMcuda(adj).build([SrcFeat], {}, {...}); out = m.run([x])`` works as it does
there; behind it the TVM-generated kernel is replaced by the sm_100a kernels of
csrc/spmm.cu, reached through the C ABI (include/featgraph_b200.h).
"""
import ctypes

import numpy as np
import torch

from .. import _lib
from ..op import vanilla_spmm_csr_cuda, schedule_vanilla_spmm_csr_cuda
from ..op.vanilla_spmm import vanilla_spmm_dds_cuda, schedule_vanilla_spmm_dds_cuda
from ..op.spec import no_x86
from ..runtime import Placeholder, NDArray, array, cpu, gpu, zeros
from ..util import util_convert_csr_to_dds
from .base import as_device_tensor, current_stream_handle, ptr, time_launches


class SpMMbase(object):
    """Base of the SpMM-like kernels (counterpart of SpMMbase, spmm.py:12-194).

    ``__init__`` normalises the adjacency to CSR and uploads it once; ``build`` fixes the
    feature shape, makes the launch plan and allocates the zero-filled output; ``run``
    launches and returns that same output array on every call.
    """

    def __init__(self, adj_scipy, num_col_partitions=1):
        csr = adj_scipy if adj_scipy.format == "csr" else adj_scipy.tocsr()
        self._num_rows, self._num_cols = int(csr.shape[0]), int(csr.shape[1])
        assert num_col_partitions >= 1, "num_col_partitions should be larger than or equal to 1"
        self._num_col_partitions = int(num_col_partitions)
        self._target = self._ctx = self._compute_func = self._schedule_func = None
        self._register()

        if self._num_col_partitions > 1:
            # 1-D source-vertex partitioning (x86 only in the reference, spmm.py:41-56).
            pos, idx, vals = self._preprocess_adj(csr, self._num_col_partitions)
            self._adj_s1_pos, self._adj_s1_idx, self._adj_vals = pos, idx, vals
            self._adj_d1_size = self._num_col_partitions
            self._adj_d2_size = self._num_rows + 1
            if self._target == "cuda":
                self._adj_s1_pos = self._index_array(pos, "s1_pos")
                self._adj_s1_idx = self._index_array(idx, "s1_idx")
                if vals.dtype != np.float32:
                    raise TypeError("adjacency values must be float32 (got %s); cast the matrix "
                                    "with .astype('float32') first" % vals.dtype)
                self._adj_s1_pos_placeholder = Placeholder(self._adj_s1_pos.shape, "int32",
                                                           "adj_s1_pos_placeholder")
                self._adj_s1_idx_placeholder = Placeholder(self._adj_s1_idx.shape, "int32",
                                                           "adj_s1_idx_placeholder")
                self._adj_vals_placeholder = Placeholder(vals.shape, "float32",
                                                         "adj_vals_placeholder")
                self._adj_s1_pos_tvm = array(self._adj_s1_pos, self._ctx)
                self._adj_s1_idx_tvm = array(self._adj_s1_idx, self._ctx)
                self._adj_vals_tvm = array(np.ascontiguousarray(vals), self._ctx)
        else:
            self._adj_indptr = self._index_array(csr.indptr, "indptr")
            self._adj_indices = self._index_array(csr.indices, "indices")
            self._adj_vals = csr.data
            if self._adj_vals.dtype != np.float32:
                raise TypeError("adjacency values must be float32 (got %s); cast the matrix "
                                "with .astype('float32') first" % self._adj_vals.dtype)
            self._adj_indptr_placeholder = Placeholder(self._adj_indptr.shape, "int32",
                                                       "adj_indptr_placeholder")
            self._adj_indices_placeholder = Placeholder(self._adj_indices.shape, "int32",
                                                        "adj_indices_placeholder")
            self._adj_vals_placeholder = Placeholder(self._adj_vals.shape, "float32",
                                                     "adj_vals_placeholder")
            # the one host -> device copy of the adjacency (spmm.py:67-69)
            self._adj_indptr_tvm = array(self._adj_indptr, self._ctx)
            self._adj_indices_tvm = array(self._adj_indices, self._ctx)
            self._adj_vals_tvm = array(self._adj_vals, self._ctx)
        self._func = None      # the launch plan, set by build()
        self._plan = None
        self._spec = None
        self.out_tvm = None

    @staticmethod
    def _index_array(a, what):
        """int32 view of a scipy index array; bit-exact or an error, never a lossy cast."""
        if a.dtype == np.int32:
            return np.ascontiguousarray(a)
        if a.size and (a.max() > np.iinfo(np.int32).max or a.min() < 0):
            raise ValueError("%s does not fit int32" % what)
        return np.ascontiguousarray(a.astype(np.int32))

    def _preprocess_adj(self, adj_scipy_csr, num_col_partitions=1):
        return util_convert_csr_to_dds(adj_scipy_csr, num_col_partitions)

    def _register(self):
        raise NotImplementedError("Please register target, ctx, compute_func, and schedule_func.")

    # -- build ---------------------------------------------------------------------------
    def _specialise(self, input_placeholders, compute_args, schedule_args):
        if self._target != "cuda":
            raise no_x86(type(self).__name__ + ".build")
        if self._num_col_partitions > 1:
            out = self._compute_func(*input_placeholders, self._adj_s1_pos_placeholder,
                                     self._adj_s1_idx_placeholder, self._adj_vals_placeholder,
                                     self._adj_d1_size, self._adj_d2_size, **compute_args)
        else:
            out = self._compute_func(*input_placeholders, self._adj_indptr_placeholder,
                                     self._adj_indices_placeholder, self._adj_vals_placeholder,
                                     **compute_args)
        sched = self._schedule_func(out, **schedule_args)
        src = input_placeholders[0]
        if src.shape[0] != self._num_cols:
            raise ValueError("SrcFeat has %d rows, the adjacency has %d columns"
                             % (src.shape[0], self._num_cols))
        if src.dtype != "float32":
            raise TypeError("only float32 features are supported, got %s" % src.dtype)
        return out, sched

    def build(self, input_placeholders, compute_args, schedule_args):
        """Fix the static shapes, plan the launch and allocate the output.

        input_placeholders : [SrcFeat], a placeholder of shape (num_cols, feat_len)
        compute_args : dict of keyword arguments of the compute function (none in the
            reference's cuda op; here optionally ``msg_op`` / ``reduce_op``, the generalised
            operators of ``vanilla_spmm_csr_cuda``)
        schedule_args : dict of keyword arguments of the schedule function, e.g.
            ``num_cuda_blocks`` / ``num_threads_per_cuda_block`` (accepted as hints), plus
            ``heavy_row_threshold`` (rows longer than this take the staged heavy-row kernel).
        """
        schedule_args = dict(schedule_args)
        threshold = int(schedule_args.pop("heavy_row_threshold", 0))
        out, sched = self._specialise(input_placeholders, compute_args, schedule_args)
        self._release_plan()
        self._plan, self._spec, self._func = self._make_plan(out, threshold), out, sched
        self.out_tvm = zeros(out.shape, out.dtype, self._ctx)

    def lower_to_ir(self, input_placeholders, compute_args, schedule_args):
        """Debug text of the plan ``build`` would make with the same arguments (the role
        of the lowered IR in the reference, spmm.py:113-140)."""
        schedule_args = dict(schedule_args)
        threshold = int(schedule_args.pop("heavy_row_threshold", 0))
        out, sched = self._specialise(input_placeholders, compute_args, schedule_args)
        lib = _lib.load()
        plan = self._make_plan(out, threshold)
        try:
            if self._num_col_partitions > 1:
                text = ("spmm_dds: %d column blocks of %d columns, one CSR plan each, %d kernel "
                        "launches per call" % (self._num_col_partitions,
                                               -(-self._num_cols // self._num_col_partitions),
                                               lib.fg_spmm_dds_plan_num_launches(plan)))
            else:
                buf = ctypes.create_string_buffer(2048)
                _lib.check(lib.fg_spmm_plan_describe(plan, buf, len(buf)))
                text = buf.value.decode()
        finally:
            self._destroy(plan)
        return text + " | hints: %r" % (sched.hints,)

    def _make_plan(self, out, threshold):
        lib = _lib.load()
        plan = ctypes.c_void_p()
        if self._num_col_partitions > 1:
            _lib.check(lib.fg_spmm_dds_plan_create(
                self._adj_s1_pos.ctypes.data_as(_lib.c_i32p), self._num_rows, self._num_cols,
                out.attrs["feat_len"], self._num_col_partitions, self._ctx.device_id,
                ctypes.byref(plan)))
        else:
            _lib.check(lib.fg_spmm_plan_create(
                self._adj_indptr.ctypes.data_as(_lib.c_i32p), self._num_rows, self._num_cols,
                out.attrs["feat_len"], self._ctx.device_id, threshold, ctypes.byref(plan)))
        return plan

    def _destroy(self, plan):
        lib = _lib.load()
        (lib.fg_spmm_dds_plan_destroy if self._num_col_partitions > 1
         else lib.fg_spmm_plan_destroy)(plan)

    # -- run -----------------------------------------------------------------------------
    def set_extra_outputs(self, device_pointers):
        """Also store every result row at these device addresses (peer-mapped copies of the
        output block on other GPUs, at most 7): the multi-GPU path's fused all-gather."""
        self._extra_outputs = [int(p) for p in device_pointers]
        self._mcast_output = None

    def set_multicast_output(self, mcast_pointer):
        """Store every result row ONCE to this address instead: the position of the row block
        inside an NVLink-switch multicast mapping of the output, which the switch writes into
        every GPU's copy (this GPU's included).  None switches it off."""
        self._mcast_output = int(mcast_pointer) if mcast_pointer else None
        self._extra_outputs = None

    def _launch(self, x, flags=0):
        """``flags``: fg_launch_flags for this one call (giant rows only / all but them /
        programmatic first kernel); see fg_next_launch_options."""
        if self._num_col_partitions > 1:
            if getattr(self, "_mcast_output", None) or getattr(self, "_extra_outputs", None):
                raise NotImplementedError("extra outputs are provided for the CSR form only")
            _lib.check(_lib.load().fg_spmm_dds_f32(
                self._plan, ptr(self._adj_s1_pos_tvm.torch), ptr(self._adj_s1_idx_tvm.torch),
                ptr(self._adj_vals_tvm.torch), ptr(x), ptr(self.out_tvm.torch),
                current_stream_handle(self._ctx)))
            return
        if flags:
            _lib.check(_lib.load().fg_next_launch_options(int(flags), 0))
        a = self._spec.attrs
        if (a["msg_op"], a["reduce_op"]) != ("mul", "sum"):
            if getattr(self, "_mcast_output", None) or getattr(self, "_extra_outputs", None):
                raise NotImplementedError("extra outputs are provided for the multiply / sum "
                                          "operator pair only")
            _lib.check(_lib.load().fg_spmm_csr_f32_general(
                self._plan, ptr(self._adj_indptr_tvm.torch), ptr(self._adj_indices_tvm.torch),
                ptr(self._adj_vals_tvm.torch), ptr(x), ptr(self.out_tvm.torch),
                _lib.MSG_OPS.index(a["msg_op"]), _lib.REDUCE_OPS.index(a["reduce_op"]),
                current_stream_handle(self._ctx)))
            return
        mcast = getattr(self, "_mcast_output", None)
        if mcast:
            _lib.check(_lib.load().fg_spmm_csr_f32_mcast(
                self._plan, ptr(self._adj_indptr_tvm.torch), ptr(self._adj_indices_tvm.torch),
                ptr(self._adj_vals_tvm.torch), ptr(x), ctypes.c_void_p(mcast),
                current_stream_handle(self._ctx)))
            return
        extra = getattr(self, "_extra_outputs", None)
        if extra:
            outs = (ctypes.c_void_p * (1 + len(extra)))(self.out_tvm.torch.data_ptr(), *extra)
            _lib.check(_lib.load().fg_spmm_csr_f32_multi(
                self._plan, ptr(self._adj_indptr_tvm.torch), ptr(self._adj_indices_tvm.torch),
                ptr(self._adj_vals_tvm.torch), ptr(x), outs, len(outs),
                current_stream_handle(self._ctx)))
            return
        _lib.check(_lib.load().fg_spmm_csr_f32(
            self._plan, ptr(self._adj_indptr_tvm.torch), ptr(self._adj_indices_tvm.torch),
            ptr(self._adj_vals_tvm.torch), ptr(x), ptr(self.out_tvm.torch),
            current_stream_handle(self._ctx)))

    def _checked_input(self, input_tvm_ndarrays):
        if self._plan is None:
            raise RuntimeError("build() must be called before run()")
        if len(input_tvm_ndarrays) != 1:
            raise ValueError("SpMM takes exactly one input array (SrcFeat)")
        src = self._spec.inputs[0]
        return as_device_tensor(input_tvm_ndarrays[0], self._ctx, src.shape, src.dtype, "SrcFeat")

    def run(self, input_tvm_ndarrays, launch_flags=0):
        """Launch on the current stream of the module's device; returns ``self.out_tvm``,
        the same array every call (spmm.py:142-161).  Asynchronous until it is read.
        ``launch_flags`` (an addition): fg_launch_flags, for callers that interleave the
        SpMM's phases with another kernel (featgraph_b200.distributed.OverlappedPair)."""
        x = self._checked_input(input_tvm_ndarrays)
        self._launch(x, launch_flags)
        return self.out_tvm

    def measure_average_time(self, input_tvm_ndarrays, num_runs):
        """Mean kernel time in seconds over ``num_runs`` launches (spmm.py:163-186)."""
        x = self._checked_input(input_tvm_ndarrays)
        return time_launches(self._ctx, lambda: self._launch(x), num_runs)

    def run_host(self, x_host, y_host):
        """End-to-end call on HOST buffers (ideally pinned): uploads ``x_host`` (num_cols, F),
        launches, downloads the result into ``y_host`` (num_rows, F) and synchronises.  The
        adjacency stays on the device, as after ``__init__`` in the reference.  Goes through
        the C ABI's fg_spmm_csr_f32_host with staging buffers owned by the module."""
        if self._plan is None:
            raise RuntimeError("build() must be called before run_host()")
        if self._num_col_partitions > 1:
            raise NotImplementedError("run_host is provided for the CSR form only")
        src = self._spec.inputs[0]
        for a, shape, what in ((x_host, src.shape, "x_host"), (y_host, self._spec.shape, "y_host")):
            if not (isinstance(a, torch.Tensor) and a.device.type == "cpu" and a.is_contiguous()
                    and a.dtype == torch.float32 and tuple(a.shape) == tuple(shape)):
                raise ValueError("%s must be a contiguous float32 CPU tensor of shape %r"
                                 % (what, tuple(shape)))
        if getattr(self, "_x_stage", None) is None or tuple(self._x_stage.shape) != src.shape:
            self._x_stage = torch.empty(src.shape, dtype=torch.float32,
                                        device=self._ctx.torch_device)
        _lib.check(_lib.load().fg_spmm_csr_f32_host(
            self._plan, ptr(self._adj_indptr_tvm.torch), ptr(self._adj_indices_tvm.torch),
            ptr(self._adj_vals_tvm.torch), ptr(x_host), ptr(y_host), ptr(self._x_stage),
            ptr(self.out_tvm.torch), current_stream_handle(self._ctx)))
        return y_host

    def set_poll_limit(self, polls):
        """Test hook: how often a wait inside the giant-row kernel polls before it gives up
        (negative: the default)."""
        if self._num_col_partitions > 1:
            raise NotImplementedError("the poll limit is a hook of the CSR form's plan")
        _lib.check(_lib.load().fg_spmm_plan_set_poll_limit(self._plan, int(polls)))

    def device_status(self):
        """Synchronise and return the status word of the plan's kernels: 0 when every
        bounded device-side wait completed; raises FeatGraphError otherwise (once: the
        word is cleared when it is reported)."""
        if self._plan is None:
            return 0
        status = ctypes.c_int32(0)
        lib = _lib.load()
        _lib.check((lib.fg_spmm_dds_plan_status if self._num_col_partitions > 1
                    else lib.fg_spmm_plan_status)(self._plan, ctypes.byref(status)))
        return int(status.value)

    def describe(self):
        """One line on the built plan: row classes, kernels and grids (the CSR form)."""
        if not self._plan or self._num_col_partitions > 1:
            return ""
        buf = ctypes.create_string_buffer(2048)
        _lib.check(_lib.load().fg_spmm_plan_describe(self._plan, buf, len(buf)))
        return buf.value.decode()

    def num_launches(self):
        """Kernels launched per ``run`` call."""
        if not self._plan:
            return 0
        lib = _lib.load()
        return int((lib.fg_spmm_dds_plan_num_launches if self._num_col_partitions > 1
                    else lib.fg_spmm_plan_num_launches)(self._plan))

    def _release_plan(self):
        if getattr(self, "_plan", None):
            self._destroy(self._plan)
            self._plan = None

    def __del__(self):
        try:
            self._release_plan()
        except Exception:
            pass

    @property
    def ctx(self):
        return self._ctx

    @property
    def target(self):
        return self._target


class VanillaSpMMcuda(SpMMbase):
    """CSR SpMM on the GPU (counterpart of VanillaSpMMcuda, spmm.py:212-220).

    ``device_id`` (default 0, the reference's ``tvm.gpu(0)``) selects the GPU; it exists
    for one-process-per-GPU runs.  ``num_col_partitions`` > 1 (the reference offers it on
    VanillaSpMMx86 only, spmm.py:197-209) selects the 1-D source-vertex partitioning: the
    adjacency is converted to the DDS form and the column blocks are summed one after the
    other, in the order of vanilla_spmm_dds_x86 (op/vanilla_spmm.py:149-220).
    """

    def __init__(self, adj_scipy, device_id=0, num_col_partitions=1):
        self._device_id = int(device_id)
        super(VanillaSpMMcuda, self).__init__(adj_scipy, num_col_partitions)

    def _register(self):
        if not torch.cuda.is_available():
            raise RuntimeError("VanillaSpMMcuda needs a CUDA device; there is no CPU fallback")
        _lib.load()
        self._target = "cuda"
        self._ctx = gpu(self._device_id)
        if self._num_col_partitions > 1:
            self._compute_func = vanilla_spmm_dds_cuda
            self._schedule_func = schedule_vanilla_spmm_dds_cuda
        else:
            self._compute_func = vanilla_spmm_csr_cuda
            self._schedule_func = schedule_vanilla_spmm_csr_cuda


class VanillaSpMMx86(SpMMbase):
    """Name kept from the reference (spmm.py:197-209).  The adjacency preprocessing
    (CSR / DDS) runs, but this backend has no x86 code path: ``build`` raises
    NotImplementedError."""

    def __init__(self, adj_scipy, num_col_partitions=1):
        super(VanillaSpMMx86, self).__init__(adj_scipy, num_col_partitions)

    def _register(self):
        self._target = "llvm"
        self._ctx = cpu(0)
        self._compute_func = None
        self._schedule_func = None
