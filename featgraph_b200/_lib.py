"""ctypes binding of csrc/libfeatgraph_b200.so (C ABI: include/featgraph_b200.h).

There is no fallback: if the CUDA library has not been built, loading raises.
"""
import ctypes
import os

from .build import LIB_PATH

_lib = None

c_i32p = ctypes.POINTER(ctypes.c_int32)
c_i64p = ctypes.POINTER(ctypes.c_int64)
c_void = ctypes.c_void_p


class FeatGraphError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, code, message):
        super().__init__("featgraph_b200 status %d: %s" % (code, message))
        self.code = code


#: every symbol include/featgraph_b200.h declares
EXPORTED_SYMBOLS = (
    "fg_last_error_string", "fg_version",
    "fg_spmm_plan_create", "fg_spmm_plan_destroy", "fg_spmm_plan_describe",
    "fg_spmm_plan_num_launches", "fg_spmm_plan_status", "fg_spmm_plan_set_poll_limit", "fg_spmm_csr_f32", "fg_spmm_csr_f32_host",
    "fg_spmm_csr_f32_noalloc", "fg_spmm_noalloc_max_rows", "fg_spmm_csr_f32_multi",
    "fg_sddmm_coo_f32_multi", "fg_sddmm_coo_f32_push",
    "fg_sddmm_coo_f32", "fg_sddmm_coo_f32_host", "fg_sddmm_num_launches", "fg_sddmm_describe",
    "fg_shard_rows_by_nnz", "fg_shard_edges",
    "fg_spmm_csr_f32_mcast", "fg_sddmm_coo_f32_mcast", "fg_peer_barrier", "fg_gather_probe",
    "fg_spmm_csr_f32_general", "fg_sddmm_coo_f32_general", "fg_next_launch_options",
    "fg_spmm_dds_plan_create", "fg_spmm_dds_plan_destroy", "fg_spmm_dds_plan_num_launches",
    "fg_spmm_dds_plan_status", "fg_spmm_dds_f32", "fg_sddmm_status",
)

LAUNCH_PROGRAMMATIC, SPMM_GIANT_ROWS_ONLY, SPMM_SKIP_GIANT_ROWS, SDDMM_TMA_STAGING = 1, 2, 4, 8  # fg_launch_flags
SPMM_LONG_ROWS_ONLY, SPMM_SKIP_LONG_ROWS, SDDMM_ROW_REGISTERS = 16, 32, 64
MSG_OPS = ("mul", "add", "sub", "div", "copy_lhs", "copy_rhs")    # enum fg_msg_op
REDUCE_OPS = ("sum", "max", "min")                                # enum fg_reduce_op


def load():
    """Load the shared library once and declare the argument types."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "featgraph_b200: %s is missing -- the CUDA extension has not been built "
            "(run `python -m featgraph_b200.build`); there is no CPU fallback" % LIB_PATH)
    lib = ctypes.CDLL(LIB_PATH)
    i32, i64 = ctypes.c_int32, ctypes.c_int64
    lib.fg_last_error_string.restype = ctypes.c_char_p
    lib.fg_version.restype = ctypes.c_char_p
    lib.fg_spmm_plan_create.argtypes = [c_i32p, i64, i64, i32, i32, i32, ctypes.POINTER(c_void)]
    lib.fg_spmm_plan_destroy.argtypes = [c_void]
    lib.fg_spmm_plan_describe.argtypes = [c_void, ctypes.c_char_p, i64]
    lib.fg_spmm_plan_num_launches.argtypes = [c_void]
    lib.fg_spmm_plan_status.argtypes = [c_void, c_i32p]
    lib.fg_spmm_plan_set_poll_limit.argtypes = [c_void, i64]
    lib.fg_next_launch_options.argtypes = [i32, i32]
    lib.fg_spmm_dds_plan_create.argtypes = [c_i32p, i64, i64, i32, i32, i32, ctypes.POINTER(c_void)]
    lib.fg_spmm_dds_plan_destroy.argtypes = [c_void]
    lib.fg_spmm_dds_plan_num_launches.argtypes = [c_void]
    lib.fg_spmm_dds_plan_status.argtypes = [c_void, c_i32p]
    lib.fg_spmm_dds_f32.argtypes = [c_void] * 7
    lib.fg_sddmm_status.argtypes = [i32, c_i32p]
    lib.fg_spmm_csr_f32.argtypes = [c_void] * 7
    lib.fg_spmm_csr_f32_host.argtypes = [c_void] * 9
    lib.fg_spmm_csr_f32_multi.argtypes = [c_void] * 5 + [ctypes.POINTER(c_void), i32, c_void]
    lib.fg_sddmm_coo_f32_multi.argtypes = [c_void] * 4 + [ctypes.POINTER(c_void), i32, i64, i64,
                                                          i64, i32, i32, i32, c_void]
    lib.fg_sddmm_coo_f32_push.argtypes = [c_void] * 5 + [ctypes.POINTER(c_void), i32, i64, i64,
                                                         i64, i32, i32, i32, c_void]
    lib.fg_spmm_csr_f32_noalloc.argtypes = [c_void] * 5 + [i64, i64, i32, i32, c_void]
    lib.fg_sddmm_coo_f32.argtypes = [c_void] * 5 + [i64, i64, i64, i32, i32, i32, c_void]
    lib.fg_sddmm_coo_f32_host.argtypes = [c_void] * 8 + [i64, i64, i64, i32, i32, i32, c_void]
    lib.fg_sddmm_num_launches.argtypes = [i64, i32, i32]
    lib.fg_sddmm_describe.argtypes = [i64, i32, i32, ctypes.c_char_p, i64]
    lib.fg_spmm_csr_f32_mcast.argtypes = [c_void] * 7
    lib.fg_sddmm_coo_f32_mcast.argtypes = [c_void] * 5 + [i64, i64, i64, i32, i32, i32, c_void]
    lib.fg_spmm_csr_f32_general.argtypes = [c_void] * 6 + [i32, i32, c_void]
    lib.fg_sddmm_coo_f32_general.argtypes = [c_void] * 5 + [i64, i64, i64, i32, i32, i32, i32, i32,
                                                            c_void]
    lib.fg_peer_barrier.argtypes = [ctypes.POINTER(c_void), i32, i32, ctypes.c_uint32, c_void,
                                    i64, i32, c_void]
    lib.fg_gather_probe.argtypes = [c_void, i64, i32, i64, i32, c_void, i32, c_void]
    lib.fg_shard_rows_by_nnz.argtypes = [c_i32p, i64, i32, c_i64p]
    lib.fg_shard_edges.argtypes = [i64, i32, c_i64p]
    _lib = lib
    return lib


def check(status):
    if status != 0:
        raise FeatGraphError(status, load().fg_last_error_string().decode())
