"""Regenerates tests/golden/reference_cases.npz.  Needs the reference checkout:

    python tests/golden/make_golden.py /path/to/FeatGraph

What can be imported from the reference without TVM -- ``featgraph.util`` -- is RUN here
to produce known-answer vectors for the two partitioning utilities.  The SpMM / SDDMM
kernels cannot run (TVM v0.7 is not installable), so their fixtures hold what the
reference's own tests compare against: ``adj.dot(x)`` (tests/test_module_spmm.py:29) and
``(src[col] * dst[row]).sum(-1)`` (tests/test_module_sddmm.py:34-36), on seeded inputs of
the shapes those tests use (127 x 255, density 0.1, feat_len 128).
"""
import os
import sys

import numpy as np
import scipy.sparse as sp


def main(ref_root):
    sys.path.insert(0, os.path.join(ref_root, "python"))
    from featgraph.util import util_convert_csr_to_dds, util_partition_adj_coo_2d

    out = {}
    rng = np.random.default_rng(12345)

    # --- kernels: the reference tests' shapes, seeded --------------------------------------
    adj = sp.random(127, 255, density=0.1, format="csr", random_state=np.random.RandomState(7),
                    dtype=np.float32)
    adj.sort_indices()
    x = rng.random((255, 128), dtype=np.float32)
    out["spmm_indptr"], out["spmm_indices"], out["spmm_data"] = adj.indptr, adj.indices, adj.data
    out["spmm_x"] = x
    out["spmm_y_scipy"] = adj.dot(x)

    coo = adj.tocoo()
    src = rng.random((255, 128), dtype=np.float32)
    dst = rng.random((127, 128), dtype=np.float32)
    out["sddmm_row"], out["sddmm_col"] = coo.row, coo.col
    out["sddmm_src"], out["sddmm_dst"] = src, dst
    out["sddmm_out_numpy"] = (src[coo.col] * dst[coo.row]).sum(axis=-1)

    # --- utilities: outputs of the reference's own functions --------------------------------
    for tag, parts in (("p2", 2), ("p4", 4), ("p7", 7)):
        pos, idx, vals = util_convert_csr_to_dds(adj, parts)
        out["dds_%s_pos" % tag], out["dds_%s_idx" % tag], out["dds_%s_vals" % tag] = pos, idx, vals
    for tag, (rp, cp) in (("2x2", (2, 2)), ("4x4", (4, 4)), ("3x5", (3, 5))):
        c = adj.tocoo()
        ids, rows, cols = util_partition_adj_coo_2d(c, rp, cp)
        out["p2d_%s_ids" % tag], out["p2d_%s_rows" % tag], out["p2d_%s_cols" % tag] = ids, rows, cols

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_cases.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py <path of a checkout of amazon-science/FeatGraph>")
    main(sys.argv[1])
