"""SDDMM op layer: same names and arguments as python/featgraph/op/vanilla_sddmm.py."""
from .spec import ComputeSpec, ScheduleSpec, no_x86


def _flat_feat(shape):
    n = 1
    for s in shape[1:]:
        n *= s
    return n


def vanilla_sddmm(SrcFeat, DstFeat, Adj_row_indices, Adj_col_indices, num_feat_partitions=1,
                  num_heads=None, msg_op="mul", reduce_op="sum"):
    """Out[e] = sum_k SrcFeat[Adj_col_indices[e], k] * DstFeat[Adj_row_indices[e], k].

    Counterpart of vanilla_sddmm (python/featgraph/op/vanilla_sddmm.py:6-63).  SrcFeat is
    indexed by COL and DstFeat by ROW, as there (:47).

    Multi-head extension (no counterpart in the reference): with ``num_heads = H`` (or 3-D
    placeholders (N, H, D)) the feature axis is split into H heads of D and
    Out[e, h] = sum_d SrcFeat[col[e], h, d] * DstFeat[row[e], h, d], shape (nnz, H).

    Generalised form (no counterpart either; the reference hard-codes Src * Dst under a sum,
    :47): Out[e, h] = reduce_op over d ascending of msg_op(SrcFeat[col[e], h, d],
    DstFeat[row[e], h, d]), operators as in vanilla_spmm_csr_cuda.
    """
    from .vanilla_spmm import _check_ops
    ops = _check_ops(msg_op, reduce_op)
    feat_len = _flat_feat(SrcFeat.shape)
    assert _flat_feat(DstFeat.shape) == feat_len, "dimension mismatch"
    num_edges = Adj_row_indices.shape[0]
    assert Adj_col_indices.shape[0] == num_edges, "dimension mismatch"
    if len(SrcFeat.shape) == 3:
        assert len(DstFeat.shape) == 3 and DstFeat.shape[1] == SrcFeat.shape[1], \
            "dimension mismatch"
        assert num_heads in (None, SrcFeat.shape[1]), "num_heads contradicts the placeholders"
        num_heads = SrcFeat.shape[1]
    elif len(SrcFeat.shape) != 2 or len(DstFeat.shape) != 2:
        raise ValueError("feature placeholders must be 2-D (N, F) or 3-D (N, H, D)")
    multi = num_heads is not None and (num_heads != 1 or len(SrcFeat.shape) == 3)
    num_heads = 1 if num_heads is None else int(num_heads)
    if num_heads < 1 or feat_len % num_heads != 0:
        raise ValueError("feat_len %d is not a multiple of num_heads %d" % (feat_len, num_heads))
    oshape = (num_edges, num_heads) if multi else (num_edges,)
    return ComputeSpec("sddmm_coo", oshape, SrcFeat.dtype,
                       (SrcFeat, DstFeat, Adj_row_indices, Adj_col_indices),
                       dict(ops, feat_len=feat_len, num_heads=num_heads,
                            num_feat_partitions=int(num_feat_partitions)),
                       name="vanilla_sddmm")


def schedule_vanilla_sddmm_cuda_tree_reduce(Out, num_feat_partitions=1, num_cuda_blocks=8192):
    """Counterpart of schedule_vanilla_sddmm_cuda_tree_reduce (vanilla_sddmm.py:77-89).

    Keeps the reference's two assertions; ``num_cuda_blocks`` is a recorded hint.
    """
    assert num_feat_partitions == 1 and Out.attrs["num_feat_partitions"] == 1, \
        "cuda schedule for sddmm does not support feat dimension tiling, " \
        "which requires cross-cuda-block reduction and atomic operations."
    num_edges = Out.shape[0]
    assert num_cuda_blocks <= num_edges, "num_cuda_blocks must be smaller than num_edges, " \
                                         "which is {}.".format(num_edges)
    return ScheduleSpec(Out, "cuda", {"num_cuda_blocks": int(num_cuda_blocks),
                                      "reduce": "tree"})


def schedule_vanilla_sddmm_cuda_single_thread_reduce(Out, num_feat_partitions=1,
                                                     num_threads_per_cuda_block=32):
    """Counterpart of schedule_vanilla_sddmm_cuda_single_thread_reduce (vanilla_sddmm.py:92-100)."""
    assert num_feat_partitions == 1 and Out.attrs["num_feat_partitions"] == 1, \
        "cuda schedule for sddmm does not support feat dimension tiling, " \
        "which requires cross-cuda-block reduction and atomic operations."
    return ScheduleSpec(Out, "cuda",
                        {"num_threads_per_cuda_block": int(num_threads_per_cuda_block),
                         "reduce": "single_thread"})


def schedule_vanilla_sddmm_x86(Out, num_feat_partitions=1):
    """x86 schedule of the reference (vanilla_sddmm.py:66-74); not provided by this backend."""
    raise no_x86("schedule_vanilla_sddmm_x86")
