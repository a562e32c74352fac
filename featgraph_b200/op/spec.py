"""Descriptors passed between the op layer and the module layer.

The reference's op functions return a TVM tensor expression and its schedule functions
return a TVM schedule; the module layer hands both to ``tvm.build``
(python/featgraph/module/spmm.py:105-109).  Here an op function returns a ``ComputeSpec``
(what is computed, on which operands, with which static shapes) and a schedule function
returns a ``ScheduleSpec`` (the target and the caller's launch hints); the module layer
turns the pair into a launch plan of the hand-written kernels.
"""


class ComputeSpec(object):
    def __init__(self, kind, shape, dtype, inputs, attrs=None, name="Out"):
        self.kind = kind            # 'spmm_csr' | 'sddmm_coo'
        self.shape = tuple(int(s) for s in shape)
        self.dtype = dtype
        self.inputs = tuple(inputs)  # placeholders, in the reference's argument order
        self.attrs = dict(attrs or {})
        self.name = name

    def __repr__(self):
        return "ComputeSpec(%s, shape=%r, attrs=%r)" % (self.kind, self.shape, self.attrs)


class ScheduleSpec(object):
    def __init__(self, out, target, hints):
        self.out = out
        self.target = target        # 'cuda'
        self.hints = dict(hints)    # validated, recorded, not binding on the kernels

    def __repr__(self):
        return "ScheduleSpec(%s on %s, hints=%r)" % (self.out.kind, self.target, self.hints)


def no_x86(name):
    return NotImplementedError(
        "%s: this backend ships the cuda target only; it has no x86 code path "
        "(use the *cuda classes and schedules)" % name)
