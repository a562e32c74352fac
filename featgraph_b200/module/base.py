"""What the SpMM and SDDMM module classes share: input checking, launch-stream lookup
and CUDA-event timing."""
import ctypes

import numpy as np
import torch

from ..runtime import NDArray, array


def ptr(t):
    """Device (or host) address of a torch tensor as a ctypes void pointer."""
    return ctypes.c_void_p(t.data_ptr())


def current_stream_handle(ctx):
    return ctypes.c_void_p(torch.cuda.current_stream(ctx.torch_device).cuda_stream)


def as_device_tensor(x, ctx, shape, dtype, what):
    """Validate one run-time input against its placeholder and return the torch tensor.

    Accepts an NDArray, a torch tensor, or a numpy array (which is copied to ``ctx``).
    Raises TypeError / ValueError on a wrong dtype, shape, device or layout -- the role
    TVM's generated argument checks play in the reference.
    """
    if isinstance(x, NDArray):
        t = x.torch
    elif isinstance(x, torch.Tensor):
        t = x
    elif isinstance(x, np.ndarray):
        t = array(x, ctx).torch
    else:
        raise TypeError("%s: expected an NDArray, torch.Tensor or numpy array, got %r"
                        % (what, type(x)))
    if str(t.dtype).replace("torch.", "") != dtype:
        raise TypeError("%s: dtype %s does not match the placeholder's %s" % (what, t.dtype, dtype))
    if tuple(t.shape) != tuple(shape):
        raise ValueError("%s: shape %r does not match the placeholder's %r"
                         % (what, tuple(t.shape), tuple(shape)))
    if t.device != ctx.torch_device:
        raise ValueError("%s: array lives on %s, the module on %s" % (what, t.device,
                                                                      ctx.torch_device))
    if not t.is_contiguous():
        raise ValueError("%s: array must be C-contiguous" % what)
    return t


def time_launches(ctx, launch, num_runs):
    """Mean seconds per call of ``launch()`` over ``num_runs`` back-to-back calls, timed
    with CUDA events on the launching stream after one untimed call -- the figure the
    reference's time_evaluator reports (python/featgraph/module/spmm.py:179-186)."""
    num_runs = int(num_runs)
    if num_runs < 1:
        raise ValueError("num_runs must be at least 1")
    dev = ctx.torch_device
    launch()
    torch.cuda.synchronize(dev)
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    start.record(torch.cuda.current_stream(dev))
    for _ in range(num_runs):
        launch()
    stop.record(torch.cuda.current_stream(dev))
    stop.synchronize()
    return start.elapsed_time(stop) * 1e-3 / num_runs
