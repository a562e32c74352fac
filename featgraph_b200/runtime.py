"""Device contexts, device arrays and placeholders.

The reference passes TVM objects across its module boundary: ``te.placeholder`` to
``build`` and ``tvm.nd.array`` to ``run`` (python/featgraph/module/spmm.py:81-111,
142-161).  These are the stand-ins: a placeholder is a static (shape, dtype) pair, an
NDArray is a thin owner of a torch tensor on the context's device.
"""
import numpy as np
import torch


class Context(object):
    """A device, in the spirit of ``tvm.gpu(0)`` / ``tvm.cpu(0)``."""

    def __init__(self, device_type, device_id=0):
        if device_type not in ("cuda", "cpu"):
            raise ValueError("unknown device type %r" % (device_type,))
        self.device_type = device_type
        self.device_id = int(device_id)

    @property
    def torch_device(self):
        if self.device_type == "cpu":
            return torch.device("cpu")
        return torch.device("cuda", self.device_id)

    def sync(self):
        if self.device_type == "cuda":
            torch.cuda.synchronize(self.torch_device)

    def __eq__(self, other):
        return (isinstance(other, Context) and other.device_type == self.device_type
                and other.device_id == self.device_id)

    def __hash__(self):
        return hash((self.device_type, self.device_id))

    def __repr__(self):
        return "%s(%d)" % ("gpu" if self.device_type == "cuda" else "cpu", self.device_id)


def gpu(dev_id=0):
    return Context("cuda", dev_id)


def cpu(dev_id=0):
    return Context("cpu", dev_id)


class Placeholder(object):
    """Static description of a dense input: ``shape`` (tuple of int) and ``dtype`` (str)."""

    def __init__(self, shape, dtype="float32", name="placeholder"):
        self.shape = tuple(int(s) for s in shape)
        if any(s < 0 for s in self.shape):
            raise ValueError("negative extent in shape %r" % (shape,))
        self.dtype = str(dtype)
        self.name = name

    def __repr__(self):
        return "Placeholder(%s, shape=%r, dtype=%s)" % (self.name, self.shape, self.dtype)


def placeholder(shape, dtype="float32", name="placeholder"):
    return Placeholder(shape, dtype, name)


def get_const_tuple(shape):
    """Counterpart of ``tvm.topi.util.get_const_tuple`` for the shapes used here."""
    return tuple(int(s) for s in shape)


class NDArray(object):
    """A dense array resident on one context; owns (or views) a torch tensor."""

    def __init__(self, tensor, ctx=None):
        if not isinstance(tensor, torch.Tensor):
            raise TypeError("NDArray wraps a torch.Tensor, got %r" % type(tensor))
        self._t = tensor
        if ctx is None:
            ctx = gpu(tensor.device.index or 0) if tensor.is_cuda else cpu(0)
        self.ctx = ctx

    @property
    def torch(self):
        return self._t

    @property
    def shape(self):
        return tuple(self._t.shape)

    @property
    def dtype(self):
        return str(self._t.dtype).replace("torch.", "")

    def asnumpy(self):
        """Blocking copy to a new host array (synchronises the producing stream)."""
        return self._t.detach().cpu().numpy()

    def copyfrom(self, source):
        src = source.torch if isinstance(source, NDArray) else torch.as_tensor(np.asarray(source))
        if tuple(src.shape) != self.shape:
            raise ValueError("shape mismatch: %r vs %r" % (tuple(src.shape), self.shape))
        self._t.copy_(src)
        return self

    def __dlpack__(self, stream=None):
        return self._t.__dlpack__(stream=stream)

    def __dlpack_device__(self):
        return self._t.__dlpack_device__()

    def __repr__(self):
        return "NDArray(shape=%r, dtype=%s, ctx=%r)" % (self.shape, self.dtype, self.ctx)


def array(source, ctx=None):
    """Copy a numpy array (or torch tensor / NDArray) onto ``ctx``; like ``tvm.nd.array``."""
    ctx = cpu(0) if ctx is None else ctx
    if isinstance(source, NDArray):
        source = source.torch
    if isinstance(source, torch.Tensor):
        t = source.detach().to(ctx.torch_device, copy=True).contiguous()
    else:
        host = np.ascontiguousarray(source)
        t = torch.from_numpy(host).to(ctx.torch_device, copy=True)
    return NDArray(t, ctx)


def empty(shape, dtype="float32", ctx=None):
    ctx = cpu(0) if ctx is None else ctx
    return NDArray(torch.empty(tuple(shape), dtype=getattr(torch, dtype),
                               device=ctx.torch_device), ctx)


def zeros(shape, dtype="float32", ctx=None):
    ctx = cpu(0) if ctx is None else ctx
    return NDArray(torch.zeros(tuple(shape), dtype=getattr(torch, dtype),
                               device=ctx.torch_device), ctx)
