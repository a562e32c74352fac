"""The C-ABI library loads and exports every symbol the header declares; the host-only
entry points and the argument checks are exercised (no device work)."""
import ctypes
import os
import re

import numpy as np
import pytest

from conftest import ROOT
from featgraph_b200 import _lib
from featgraph_b200.build import build_library


@pytest.fixture(scope="module")
def lib():
    build_library()
    return _lib.load()


def _header_functions():
    text = open(os.path.join(ROOT, "include", "featgraph_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fg_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    declared = _header_functions()
    assert len(declared) >= 14
    for name in declared:
        assert hasattr(lib, name), name
    assert sorted(_lib.EXPORTED_SYMBOLS) == declared


def test_version_and_error_string(lib):
    assert lib.fg_version().decode().count(".") == 2
    assert isinstance(lib.fg_last_error_string(), bytes)


def _bounds(world):
    return (ctypes.c_int64 * (world + 1))()


def test_shard_rows_by_nnz_balances_nonzeros(lib):
    rng = np.random.default_rng(0)
    deg = rng.zipf(1.8, 5000).clip(max=3000)
    indptr = np.concatenate(([0], np.cumsum(deg))).astype(np.int32)
    for world in (1, 2, 4, 8):
        b = _bounds(world)
        assert lib.fg_shard_rows_by_nnz(indptr.ctypes.data_as(_lib.c_i32p), 5000, world, b) == 0
        b = np.array(b[:])
        assert b[0] == 0 and b[-1] == 5000 and (np.diff(b) >= 0).all()
        share = np.diff(indptr[b])
        assert abs(share - indptr[-1] / world).max() <= deg.max()


def test_shard_rows_degenerate_cases(lib):
    b = _bounds(4)
    empty = np.zeros(1, np.int32)
    assert lib.fg_shard_rows_by_nnz(empty.ctypes.data_as(_lib.c_i32p), 0, 4, b) == 0
    assert list(b) == [0, 0, 0, 0, 0]
    one = np.array([0, 7], np.int32)      # a single row cannot be split
    assert lib.fg_shard_rows_by_nnz(one.ctypes.data_as(_lib.c_i32p), 1, 4, b) == 0
    assert b[0] == 0 and b[4] == 1 and sorted(b[:]) == list(b[:])
    assert lib.fg_shard_rows_by_nnz(one.ctypes.data_as(_lib.c_i32p), 1, 0, b) == 1
    assert b"world" in lib.fg_last_error_string()
    bad = np.array([0, 5, 3], np.int32)
    assert lib.fg_shard_rows_by_nnz(bad.ctypes.data_as(_lib.c_i32p), 2, 2, b) == 1


def test_shard_edges(lib):
    b = _bounds(8)
    assert lib.fg_shard_edges(114615892, 8, b) == 0
    b = np.array(b[:])
    assert b[0] == 0 and b[-1] == 114615892
    # equal ranges of a multiple of 32 edges; only the last one is short
    assert (b[:-1] % 32 == 0).all() and len(set(np.diff(b)[:-1])) == 1
    assert 0 < np.diff(b)[-1] <= np.diff(b)[0] < 114615892 / 8 + 32
    b = _bounds(4)
    assert lib.fg_shard_edges(40, 4, b) == 0 and list(b) == [0, 32, 40, 40, 40]
    assert lib.fg_shard_edges(0, 4, b) == 0 and list(b) == [0, 0, 0, 0, 0]
    assert lib.fg_shard_edges(-1, 8, _bounds(8)) == 1


def test_argument_errors_return_status_not_abort(lib):
    plan = ctypes.c_void_p()
    indptr = np.array([0, 2, 1], np.int32)
    rc = lib.fg_spmm_plan_create(indptr.ctypes.data_as(_lib.c_i32p), 2, 4, 64, 0, 0,
                                 ctypes.byref(plan))
    assert rc == 1 and b"decreases" in lib.fg_last_error_string()
    rc = lib.fg_spmm_plan_create(None, 2, 4, 64, 0, 0, ctypes.byref(plan))
    assert rc == 1
    rc = lib.fg_spmm_plan_create(indptr.ctypes.data_as(_lib.c_i32p), 2, 4, 0, 0, 0,
                                 ctypes.byref(plan))
    assert rc == 1
    assert lib.fg_spmm_csr_f32(None, None, None, None, None, None, None) == 1
    # feat_len not a multiple of num_heads
    assert lib.fg_sddmm_coo_f32(None, None, None, None, None, 10, 4, 4, 30, 4, 0, None) == 1
    # nnz == 0 is a no-op that needs no device
    assert lib.fg_sddmm_coo_f32(None, None, None, None, None, 0, 4, 4, 32, 1, 0, None) == 0
    buf = ctypes.create_string_buffer(512)
    assert lib.fg_sddmm_describe(1000, 64, 1, buf, 512) == 0 and b"sddmm_tile_kernel" in buf.value
    assert lib.fg_sddmm_describe(1000, 33, 1, buf, 512) == 0 and b"generic" in buf.value
    with pytest.raises(_lib.FeatGraphError):
        _lib.check(lib.fg_shard_edges(-5, 2, _bounds(2)))
