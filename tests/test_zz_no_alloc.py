"""The allocation-free SpMM entry point, fg_spmm_csr_f32_noalloc.

It exists for hosts that may not allocate device memory once they are running (a plug-in
in a server that owns the device pool, a loop where cudaMalloc is banned because it
synchronises the device).  Its row-order scratch is a fixed array inside the library, shared
by all calls and rebuilt by each, so the test makes two calls in a row, on different
matrices, and requires both to equal the plan-based fg_spmm_csr_f32 -- and the CPU oracle --
bit for bit.

The file is named so that pytest collects it last.
"""
import ctypes

import numpy as np
import pytest
import torch

from featgraph_b200 import _lib, graphs
from helpers import bits, features, random_csr


def _vp(t):
    return ctypes.c_void_p(t.data_ptr())


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _with_plan(lib, indptr_host, d_ptr, d_idx, d_val, x, n_rows, n_cols, feat_len, stream):
    y = torch.full((n_rows, feat_len), float("nan"), device="cuda")
    plan = ctypes.c_void_p()
    _lib.check(lib.fg_spmm_plan_create(indptr_host.ctypes.data_as(_lib.c_i32p), n_rows, n_cols,
                                       feat_len, 0, 0, ctypes.byref(plan)))
    try:
        _lib.check(lib.fg_spmm_csr_f32(plan, _vp(d_ptr), _vp(d_idx), _vp(d_val), _vp(x), _vp(y),
                                       stream))
        torch.cuda.synchronize()
    finally:
        lib.fg_spmm_plan_destroy(plan)
    return y


@pytest.mark.gpu
def test_noalloc_entry_point_equals_plan_entry_point_on_two_calls_in_a_row(oracle):
    lib = _lib.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    g = graphs.powerlaw_graph(n=20000, nnz_target=2000000, device="cuda")   # rows up to ~15 K long
    small = random_csr(300, 257, 0.08, seed=3, empty_rows=(0, 17, 299), dense_rows=(5, 200))
    cases = [
        (g.indptr.cpu().numpy(), g.indptr, g.indices, g.vals, g.n_rows, g.n_cols, 64),
        (small.indptr, _dev(small.indptr), _dev(small.indices), _dev(small.data), 300, 257, 96),
    ]
    for indptr_host, d_ptr, d_idx, d_val, n_rows, n_cols, feat_len in cases:
        x = _dev(features((n_cols, feat_len), seed=feat_len))
        want = _with_plan(lib, indptr_host, d_ptr, d_idx, d_val, x, n_rows, n_cols, feat_len,
                          stream)
        got = torch.full((n_rows, feat_len), float("nan"), device="cuda")
        _lib.check(lib.fg_spmm_csr_f32_noalloc(_vp(d_ptr), _vp(d_idx), _vp(d_val), _vp(x),
                                               _vp(got), n_rows, n_cols, feat_len, 0, stream))
        torch.cuda.synchronize()
        assert torch.equal(want.view(torch.int32), got.view(torch.int32))
        ref = oracle.spmm_csr_f32(indptr_host, d_idx.cpu().numpy(), d_val.cpu().numpy(),
                                  x.cpu().numpy(), n_cols=n_cols)
        assert np.array_equal(bits(ref), bits(got.cpu().numpy()))


@pytest.mark.gpu
def test_noalloc_entry_point_rejects_what_it_cannot_hold():
    lib = _lib.load()
    limit = lib.fg_spmm_noalloc_max_rows()
    assert limit == 1 << 20
    dummy = torch.zeros(64, device="cuda")
    args = [_vp(dummy)] * 5
    assert lib.fg_spmm_csr_f32_noalloc(*args, limit + 1, 10, 64, 0, None) == 3
    assert b"at most" in lib.fg_last_error_string()
    assert lib.fg_spmm_csr_f32_noalloc(*args, 10, 10, 48, 0, None) == 3
    assert b"multiple of 32" in lib.fg_last_error_string()
    assert lib.fg_spmm_csr_f32_noalloc(*args, 0, 10, 64, 0, None) == 0      # nothing to do
