"""Seeded synthetic graphs and features for the benchmark and the full-size tests.

They stand in for the Reddit graph that the reference's benchmark scripts load
(benchmark/download_reddit_dataset.py:9-20): same vertex count, edge count and a
power-law degree profile, but generated, not the dataset.

Vertex weights come from numpy's Generator (bit-reproducible everywhere); the bulk edge
sampling uses torch's generator on the chosen device, so a graph is reproducible per
(seed, device type), not across CPU and GPU.
"""
import numpy as np
import torch

GRAPH_SEED = 20200
FEAT_SEED = 20201
FEAT2_SEED = 20202

REDDIT_NUM_VERTICES = 232965
REDDIT_NUM_EDGES = 114615892


class CSRGraph(object):
    """int32 CSR (sorted, duplicate-free) with float32 values, as torch tensors."""

    def __init__(self, n_rows, n_cols, indptr, indices, vals):
        self.n_rows, self.n_cols = int(n_rows), int(n_cols)
        self.indptr, self.indices, self.vals = indptr, indices, vals

    @property
    def nnz(self):
        return int(self.indices.shape[0])

    def coo_rows(self):
        """Row index of every nonzero in CSR order (int32) -- the row-major sorted COO."""
        deg = (self.indptr[1:] - self.indptr[:-1]).to(torch.int64)
        return torch.repeat_interleave(
            torch.arange(self.n_rows, dtype=torch.int32, device=self.indptr.device), deg)

    def degree_stats(self):
        deg = (self.indptr[1:] - self.indptr[:-1]).to(torch.float64)
        if deg.numel() == 0:
            return {"max": 0, "median": 0, "p99": 0, "mean": 0.0}
        return {"max": int(deg.max()), "median": int(deg.median()),
                "p99": int(torch.quantile(deg.cpu(), 0.99)), "mean": float(deg.mean())}

    def to_scipy(self):
        import scipy.sparse as sp
        return sp.csr_matrix((self.vals.cpu().numpy(), self.indices.cpu().numpy(),
                              self.indptr.cpu().numpy()), shape=(self.n_rows, self.n_cols))


def _csr_from_sorted_keys(keys, n_rows, n_cols, vals_mode, gen, device):
    rows = torch.div(keys, n_cols, rounding_mode="floor")
    cols = (keys - rows * n_cols).to(torch.int32)
    counts = torch.bincount(rows, minlength=n_rows)
    indptr = torch.zeros(n_rows + 1, dtype=torch.int64, device=device)
    torch.cumsum(counts, 0, out=indptr[1:])
    nnz = int(keys.shape[0])
    if vals_mode == "ones":
        vals = torch.ones(nnz, dtype=torch.float32, device=device)
    else:
        vals = torch.rand(nnz, dtype=torch.float32, device=device, generator=gen)
    return CSRGraph(n_rows, n_cols, indptr.to(torch.int32), cols, vals)


def _sample_categorical(cdf, count, gen, device):
    u = torch.rand(count, dtype=torch.float64, device=device, generator=gen)
    idx = torch.searchsorted(cdf, u, right=True)
    return idx.clamp_(max=cdf.shape[0] - 1)


def powerlaw_graph(n=REDDIT_NUM_VERTICES, nnz_target=REDDIT_NUM_EDGES, seed=GRAPH_SEED,
                   device="cpu", zipf_a=2.1, vals="ones", chunk=1 << 25):
    """Chung-Lu style directed graph with heavy-tailed expected degrees.

    Vertex weights w ~ Zipf(zipf_a); out- and in-weights are independent permutations of w.
    Edge (r, c) is present with probability 1 - exp(-lam * w_out[r] * w_in[c]) (so rows
    saturate at degree n instead of producing duplicates), realised by drawing
    M = lam * sum(w)^2 endpoint pairs proportionally to the weights and discarding
    repeats; lam is solved so that the expected edge count equals ``nnz_target``.
    Self-loops are kept, there are no duplicate edges, columns are sorted within a row.
    """
    rng = np.random.default_rng(seed)
    w = rng.zipf(zipf_a, n).astype(np.float64)
    w_out = w[rng.permutation(n)]
    w_in = w[rng.permutation(n)]
    nnz_target = min(int(nnz_target), n * n)

    # expected nnz as a function of lam, over the distinct weight values only
    ua, ca = np.unique(w_out, return_counts=True)
    ub, cb = np.unique(w_in, return_counts=True)
    pair_w = ua[:, None] * ub[None, :]
    pair_n = ca[:, None].astype(np.float64) * cb[None, :]

    def expected(lam):
        return float((pair_n * -np.expm1(-lam * pair_w)).sum())

    lo, hi = 1e-18, 1e3
    for _ in range(200):
        mid = (lo * hi) ** 0.5
        if expected(mid) < nnz_target:
            lo = mid
        else:
            hi = mid
    lam = hi
    draws = int(round(lam * w_out.sum() * w_in.sum()))

    dev = torch.device(device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(int(seed))
    cdf_out = torch.from_numpy(np.cumsum(w_out) / w_out.sum()).to(dev)
    cdf_in = torch.from_numpy(np.cumsum(w_in) / w_in.sum()).to(dev)
    parts = []
    left = draws
    while left > 0:
        m = min(left, chunk)
        r = _sample_categorical(cdf_out, m, gen, dev)
        c = _sample_categorical(cdf_in, m, gen, dev)
        parts.append(torch.unique(r * n + c))
        left -= m
    keys = torch.unique(torch.cat(parts)) if parts else torch.empty(0, dtype=torch.int64,
                                                                    device=dev)
    del parts
    return _csr_from_sorted_keys(keys, n, n, vals, gen, dev)


def regular_graph(n=65536, per_row=16, seed=GRAPH_SEED, device="cpu"):
    """Square matrix with exactly ``per_row`` distinct uniformly random columns in every row
    (sorted), values U(0,1): the CPU-runnable configuration."""
    dev = torch.device(device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(int(seed))
    per_row = min(per_row, n)
    cols = torch.randint(0, n, (n, per_row), dtype=torch.int64, device=dev, generator=gen)
    for _ in range(64):
        cols, _ = torch.sort(cols, dim=1)
        bad = (cols[:, 1:] == cols[:, :-1]).any(dim=1)
        n_bad = int(bad.sum())
        if n_bad == 0:
            break
        cols[bad] = torch.randint(0, n, (n_bad, per_row), dtype=torch.int64, device=dev,
                                  generator=gen)
    else:
        raise RuntimeError("could not draw distinct columns")
    indptr = (torch.arange(n + 1, dtype=torch.int64, device=dev) * per_row).to(torch.int32)
    vals = torch.rand(n * per_row, dtype=torch.float32, device=dev, generator=gen)
    return CSRGraph(n, n, indptr, cols.reshape(-1).to(torch.int32), vals)


def rmat_graph(scale=24, edge_draws=1 << 28, abcd=(0.57, 0.19, 0.19, 0.05), seed=GRAPH_SEED,
               device="cpu", vals="uniform", chunk=1 << 26):
    """R-MAT graph: 2**scale vertices, ``edge_draws`` recursive-quadrant draws with
    probabilities (a, b, c, d), duplicates removed, values U(0,1)."""
    dev = torch.device(device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(int(seed))
    a, b, c, _ = abcd
    n = 1 << scale
    parts = []
    left = int(edge_draws)
    while left > 0:
        m = min(left, chunk)
        r = torch.zeros(m, dtype=torch.int64, device=dev)
        col = torch.zeros(m, dtype=torch.int64, device=dev)
        for _ in range(scale):
            u = torch.rand(m, dtype=torch.float32, device=dev, generator=gen)
            down = u >= (a + b)                       # quadrants c, d: lower half
            right = ((u >= a) & (u < a + b)) | (u >= a + b + c)   # quadrants b, d
            r = r * 2 + down.to(torch.int64)
            col = col * 2 + right.to(torch.int64)
        parts.append(torch.unique(r * n + col))
        left -= m
    keys = torch.unique(torch.cat(parts))
    del parts
    return _csr_from_sorted_keys(keys, n, n, vals, gen, dev)


def normal_features(n, shape_tail, seed, device="cpu"):
    """(n, *shape_tail) float32 ~ N(0,1)."""
    dev = torch.device(device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(int(seed))
    tail = (shape_tail,) if isinstance(shape_tail, int) else tuple(shape_tail)
    return torch.randn((n,) + tail, dtype=torch.float32, device=dev, generator=gen)
