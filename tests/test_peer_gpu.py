"""The device-side barrier of the multi-GPU path (fg_peer_barrier) on ONE GPU: the flag
arrays of two "ranks" are two local buffers, so the kernel's arithmetic and -- the point --
its bounded wait can be checked without a second device.  The wait is made to run out by a
flag that nothing sets; the kernel must return and report through the status word."""
import ctypes

import pytest
import torch

from featgraph_b200 import _lib

pytestmark = pytest.mark.gpu


def _call(lib, flags, rank, world, epoch, status, max_polls):
    arr = (ctypes.c_void_p * world)(*[f.data_ptr() for f in flags])
    _lib.check(lib.fg_peer_barrier(arr, rank, world, epoch, ctypes.c_void_p(status.data_ptr()),
                                   max_polls, 0,
                                   ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))


def test_barrier_passes_when_every_rank_has_arrived():
    lib = _lib.load()
    flags = [torch.zeros(8, dtype=torch.int32, device="cuda") for _ in range(2)]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    # rank 1's announcements of epochs 1 and 2 are already in rank 0's array
    flags[0][1] = 2
    for epoch in (1, 2):
        _call(lib, flags, 0, 2, epoch, status, 1000)
        torch.cuda.synchronize()
        assert int(status) == 0
        assert flags[0][0] == epoch and flags[1][0] == epoch      # announced to both arrays
    # a wrapped counter still compares as "reached"
    flags[0][1] = 5
    _call(lib, flags, 0, 2, 0xFFFFFFFE, status, 1000)
    torch.cuda.synchronize()
    assert int(status) == 0


def test_barrier_wait_runs_out_and_reports():
    lib = _lib.load()
    flags = [torch.zeros(8, dtype=torch.int32, device="cuda") for _ in range(3)]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    flags[0][1] = 1                          # rank 1 has arrived, rank 2 never does
    _call(lib, flags, 0, 3, 1, status, 2000)
    torch.cuda.synchronize()                 # returns: the wait is bounded
    assert int(status) == 3                  # 1 + the rank that was waited for
    # the first code sticks, and the context is still usable
    _call(lib, flags, 0, 3, 2, status, 10)
    torch.cuda.synchronize()
    assert int(status) in (2, 3)
    assert float(torch.ones(4, device="cuda").sum()) == 4.0


def test_barrier_rejects_bad_arguments():
    lib = _lib.load()
    flags = [torch.zeros(8, dtype=torch.int32, device="cuda")]
    arr = (ctypes.c_void_p * 1)(flags[0].data_ptr())
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    sp = ctypes.c_void_p(status.data_ptr())
    assert lib.fg_peer_barrier(arr, 1, 1, 1, sp, 10, 0, None) == 1          # rank >= world
    assert lib.fg_peer_barrier(arr, 0, 9, 1, sp, 10, 0, None) == 1          # more than 8 ranks
    assert lib.fg_peer_barrier(None, 0, 1, 1, sp, 10, 0, None) == 1
    assert lib.fg_peer_barrier(arr, 0, 1, 1, None, 10, 0, None) == 1


def test_gather_probe_runs():
    lib = _lib.load()
    table = torch.randn(100000, 64, device="cuda")
    sink = torch.zeros(1, device="cuda")
    for row_floats in (32, 64, 128):
        _lib.check(lib.fg_gather_probe(ctypes.c_void_p(table.data_ptr()),
                                       100000 * 64 // row_floats, row_floats, 64, 148,
                                       ctypes.c_void_p(sink.data_ptr()), 0, None))
    torch.cuda.synchronize()
    assert float(sink) == 0.0
    assert lib.fg_gather_probe(ctypes.c_void_p(table.data_ptr()), 100, 48, 64, 8,
                               ctypes.c_void_p(sink.data_ptr()), 0, None) == 3
