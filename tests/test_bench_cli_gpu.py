"""The command-line benchmark with the reference's flags (benchmark/bench_vanilla_spmm.py:71-84,
bench_vanilla_sddmm.py:77-90): ``--dataset <scipy npz> --feat-len F --target cuda``.  The
files are written as the reference's download script writes them
(benchmark/download_reddit_dataset.py:11-20): a canonical float32 CSR for SpMM, its COO
form for SDDMM.  The result the CLI computed is dumped and compared with the CPU oracle."""
import numpy as np
import pytest
import scipy.sparse as sp

from featgraph_b200 import bench_cli, graphs
from helpers import bits, random_csr

pytestmark = pytest.mark.gpu


def _files(tmp_path):
    csr = random_csr(700, 700, 0.05, seed=51, empty_rows=(0, 9), dense_rows=(33,))
    assert csr.has_canonical_format and csr.dtype == np.float32
    csr_path, coo_path = str(tmp_path / "adj_csr_float32.npz"), str(tmp_path / "adj_coo.npz")
    sp.save_npz(csr_path, csr)
    sp.save_npz(coo_path, csr.tocoo())
    return csr, csr_path, coo_path


def test_spmm_from_an_npz_file(tmp_path, oracle):
    csr, csr_path, _ = _files(tmp_path)
    dump = str(tmp_path / "y.npy")
    recs = bench_cli.main(["--kernel", "spmm", "--dataset", csr_path, "--feat-len", "64",
                           "--target", "cuda", "--num-runs", "3", "--dump-output", dump])
    assert len(recs) == 1 and recs[0]["nnz"] == csr.nnz and recs[0]["ms"] > 0
    assert recs[0]["graph"] == "file:" + csr_path and recs[0]["feat_len"] == 64
    x = graphs.normal_features(700, 64, graphs.FEAT_SEED, "cuda").cpu().numpy()
    want = oracle.spmm_csr_f32(csr.indptr, csr.indices, csr.data, x, n_cols=700)
    assert np.array_equal(bits(want), bits(np.load(dump)))


@pytest.mark.parametrize("heads", [1, 4])
def test_sddmm_from_an_npz_file_keeps_the_stored_edge_order(tmp_path, oracle, heads):
    csr, _, coo_path = _files(tmp_path)
    # a COO file whose edges are NOT in row-major order: the output follows the file
    coo = csr.tocoo()
    perm = np.random.default_rng(2).permutation(coo.nnz)
    shuffled = sp.coo_matrix((coo.data[perm], (coo.row[perm], coo.col[perm])), shape=coo.shape)
    sp.save_npz(coo_path, shuffled)
    dump = str(tmp_path / "out.npy")
    argv = ["--kernel", "sddmm", "--dataset", coo_path, "--target", "cuda", "--num-runs", "3",
            "--dump-output", dump]
    argv += ["--heads", "4", "--head-dim", "16"] if heads > 1 else ["--feat-len", "64"]
    recs = bench_cli.main(argv)
    assert recs[0]["nnz"] == coo.nnz and recs[0]["heads"] == heads
    shape = (4, 16) if heads > 1 else (64,)
    src = graphs.normal_features(700, shape, graphs.FEAT_SEED, "cuda").cpu().numpy()
    dst = graphs.normal_features(700, shape, graphs.FEAT2_SEED, "cuda").cpu().numpy()
    want = oracle.sddmm_coo_f32(shuffled.row, shuffled.col, src, dst, num_heads=heads)
    got = np.load(dump)
    assert np.array_equal(bits(want.reshape(got.shape)), bits(got))


def test_the_x86_target_is_refused():
    with pytest.raises(SystemExit, match="cuda target only"):
        bench_cli.main(["--kernel", "spmm", "--synthetic", "regular", "--target", "x86"])
