"""SpMM op layer: same names and arguments as python/featgraph/op/vanilla_spmm.py."""
from .spec import ComputeSpec, ScheduleSpec, no_x86


def _check_ops(msg_op, reduce_op):
    from .._lib import MSG_OPS, REDUCE_OPS
    if msg_op not in MSG_OPS:
        raise ValueError("msg_op must be one of %r, got %r" % (MSG_OPS, msg_op))
    if reduce_op not in REDUCE_OPS:
        raise ValueError("reduce_op must be one of %r, got %r" % (REDUCE_OPS, reduce_op))
    return {"msg_op": msg_op, "reduce_op": reduce_op}


def vanilla_spmm_csr_cuda(SrcFeat, Adj_indptr, Adj_indices, Adj_vals, msg_op="mul",
                          reduce_op="sum"):
    """Out[row, f] = sum over the row's nonzeros of Adj_vals[e] * SrcFeat[Adj_indices[e], f].

    Counterpart of vanilla_spmm_csr_cuda (python/featgraph/op/vanilla_spmm.py:83-125).

    Generalised form (no counterpart in the reference, which hard-codes multiply and sum,
    :121): ``Out[row, f] = reduce_op over the row's nonzeros, in CSR order, of
    msg_op(SrcFeat[Adj_indices[e], f], Adj_vals[e])`` with msg_op in mul / add / sub / div /
    copy_lhs / copy_rhs and reduce_op in sum / max / min (max and min start from the lowest /
    highest finite float, as TVM's te.max / te.min do).

    SrcFeat : placeholder, (num_src_vertices, feat_len)
    Adj_indptr : placeholder, (num_dst_vertices + 1,)
    Adj_indices, Adj_vals : placeholders, (nnz,)
    Returns the ComputeSpec of Out, (num_dst_vertices, feat_len).
    """
    assert Adj_indices.shape[0] == Adj_vals.shape[0]
    if len(SrcFeat.shape) != 2:
        raise ValueError("SrcFeat must be 2-D (num_src_vertices, feat_len), got %r"
                         % (SrcFeat.shape,))
    _, feat_len = SrcFeat.shape
    num_dst_vertices = Adj_indptr.shape[0] - 1
    return ComputeSpec("spmm_csr", (num_dst_vertices, feat_len), SrcFeat.dtype,
                       (SrcFeat, Adj_indptr, Adj_indices, Adj_vals),
                       dict(_check_ops(msg_op, reduce_op), feat_len=feat_len))


def schedule_vanilla_spmm_csr_cuda(Out, num_cuda_blocks=None, num_threads_per_cuda_block=None):
    """Counterpart of schedule_vanilla_spmm_csr_cuda (vanilla_spmm.py:128-146).

    The reference binds rows to blockIdx.x and features to threadIdx.x with these two
    knobs.  The kernels here pick their own launch shape from the degree distribution, so
    the knobs are checked and recorded as hints only; the result does not depend on them.
    """
    num_rows, feat_len = Out.shape
    if num_cuda_blocks is None:
        num_cuda_blocks = num_rows
    if num_threads_per_cuda_block is None:
        num_threads_per_cuda_block = feat_len
    if num_rows > 0 and (int(num_cuda_blocks) < 1 or int(num_threads_per_cuda_block) < 1):
        raise ValueError("num_cuda_blocks and num_threads_per_cuda_block must be positive")
    return ScheduleSpec(Out, "cuda", {"num_cuda_blocks": int(num_cuda_blocks),
                                      "num_threads_per_cuda_block": int(num_threads_per_cuda_block)})


def vanilla_spmm_csr_x86(SrcFeat, Adj_indptr, Adj_indices, Adj_vals, num_feat_partitions=1):
    """x86 op of the reference (vanilla_spmm.py:6-62); not provided by this backend."""
    raise no_x86("vanilla_spmm_csr_x86")


def schedule_vanilla_spmm_csr_x86(Out):
    raise no_x86("schedule_vanilla_spmm_csr_x86")


def vanilla_spmm_dds_cuda(SrcFeat, Adj_s1_pos, Adj_s1_idx, Adj_vals, d1_size, d2_size):
    """SpMM over the dense-dense-sparse form: the arguments of vanilla_spmm_dds_x86
    (python/featgraph/op/vanilla_spmm.py:149-220) without its feature partitioning, which
    only re-lays the arrays out.  The reference has this op for x86 only.

    Out[row, f] = ((0 + S_0) + S_1) + ... with S_p[row, f] the sum, in stored order, of
    Adj_vals[e] * SrcFeat[Adj_s1_idx[e] + p * ceil(num_src_vertices / d1_size), f] over the
    entries Adj_s1_pos[p * d2_size + row] <= e < Adj_s1_pos[p * d2_size + row + 1].

    SrcFeat : placeholder, (num_src_vertices, feat_len)
    Adj_s1_pos : placeholder, (d1_size * d2_size,)
    Adj_s1_idx, Adj_vals : placeholders, (nnz,)
    d1_size : number of source-vertex partitions; d2_size : num_dst_vertices + 1
    """
    assert Adj_s1_pos.shape[0] == d1_size * d2_size
    assert Adj_s1_idx.shape[0] == Adj_vals.shape[0]
    if len(SrcFeat.shape) != 2:
        raise ValueError("SrcFeat must be 2-D (num_src_vertices, feat_len), got %r"
                         % (SrcFeat.shape,))
    _, feat_len = SrcFeat.shape
    return ComputeSpec("spmm_dds", (d2_size - 1, feat_len), SrcFeat.dtype,
                       (SrcFeat, Adj_s1_pos, Adj_s1_idx, Adj_vals),
                       {"msg_op": "mul", "reduce_op": "sum", "feat_len": feat_len,
                        "num_col_partitions": int(d1_size)})


def schedule_vanilla_spmm_dds_cuda(Out):
    """Counterpart of schedule_vanilla_spmm_dds_x86 (vanilla_spmm.py:223-246) for the cuda
    target; like it, it takes no knobs."""
    return ScheduleSpec(Out, "cuda", {})


def vanilla_spmm_dds_x86(SrcFeat, Adj_s1_pos, Adj_s1_idx, Adj_vals, d1_size, d2_size,
                         num_feat_partitions=1):
    """x86 DDS op of the reference (vanilla_spmm.py:149-220); not provided by this backend."""
    raise no_x86("vanilla_spmm_dds_x86")


def schedule_vanilla_spmm_dds_x86(Out):
    raise no_x86("schedule_vanilla_spmm_dds_x86")
