"""featgraph_b200 -- FeatGraph's SpMM / SDDMM module API on hand-written sm_100a kernels.

    from featgraph_b200 import te, nd, gpu
    from featgraph_b200.module import VanillaSpMMcuda
    m = VanillaSpMMcuda(adj_scipy_csr)
    m.build([te.placeholder((num_cols, 64))], {}, {})
    y = m.run([nd.array(x_np, m.ctx)]).asnumpy()

``install_as_featgraph()`` makes the package importable under the reference's own name
(``from featgraph.module import VanillaSpMMcuda``).
"""
import sys

from . import nd, te  # noqa: F401
from .runtime import Context, NDArray, Placeholder, cpu, gpu, get_const_tuple  # noqa: F401

__version__ = "0.1.0"


def install_as_featgraph():
    """Alias this package and its module/op/util subpackages as ``featgraph``."""
    from . import module, op, util
    me = sys.modules[__name__]
    sys.modules.setdefault("featgraph", me)
    sys.modules.setdefault("featgraph.module", module)
    sys.modules.setdefault("featgraph.op", op)
    sys.modules.setdefault("featgraph.util", util)
    return me
