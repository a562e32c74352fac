"""Drop-in proof: the reference's OWN test scripts (tests/test_module_spmm.py and
tests/test_module_sddmm.py of a FeatGraph checkout), unmodified, run against this backend.

The scripts import ``tvm`` (``te.placeholder``, ``tvm.nd.array``,
``tvm.topi.util.get_const_tuple``) and ``featgraph.module``.  For the duration of the test
those names are bound to this package's stand-ins -- no line of the scripts is rewritten --
and their cuda test functions are called the way their ``__main__`` blocks call them.

The checkout is not part of this repository: point FEATGRAPH_REFERENCE_DIR at one to run
the test; without it the test is skipped (tests/test_spmm_gpu.py::test_reference_cuda_cases
and tests/test_sddmm_gpu.py hold the same cases re-typed, on seeded inputs).
"""
import os
import sys
import types

import pytest
import scipy.sparse

pytestmark = pytest.mark.gpu

REF = os.environ.get("FEATGRAPH_REFERENCE_DIR", "")


def _load_script(path):
    import featgraph_b200 as fg
    fg.install_as_featgraph()
    tvm = types.ModuleType("tvm")
    tvm.te, tvm.nd, tvm.gpu, tvm.cpu = fg.te, fg.nd, fg.gpu, fg.cpu
    topi = types.ModuleType("tvm.topi")
    util = types.ModuleType("tvm.topi.util")
    util.get_const_tuple = fg.get_const_tuple
    topi.util = util
    tvm.topi = topi
    shims = {"tvm": tvm, "tvm.te": fg.te, "tvm.topi": topi, "tvm.topi.util": util}
    saved = {k: sys.modules.get(k) for k in shims}
    sys.modules.update(shims)
    try:
        scope = {"__name__": "reference_test_script"}
        with open(path) as fh:
            exec(compile(fh.read(), path, "exec"), scope)
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v
    return scope


@pytest.mark.skipif(not os.path.isfile(os.path.join(REF, "tests", "test_module_spmm.py")),
                    reason="FEATGRAPH_REFERENCE_DIR does not name a FeatGraph checkout")
def test_the_reference_spmm_test_script_passes_unmodified():
    scope = _load_script(os.path.join(REF, "tests", "test_module_spmm.py"))
    # as in the script's __main__ block
    adj = scipy.sparse.random(127, 255, density=0.1, format="csr").astype("float32")
    scope["test_vanilla_spmm_cuda"](adj)          # asserts allclose(rtol=atol=1e-4) vs scipy
    with pytest.raises(NotImplementedError):      # no x86 code path in this backend
        scope["test_vanilla_spmm_x86"](adj)


@pytest.mark.skipif(not os.path.isfile(os.path.join(REF, "tests", "test_module_sddmm.py")),
                    reason="FEATGRAPH_REFERENCE_DIR does not name a FeatGraph checkout")
def test_the_reference_sddmm_test_script_passes_unmodified():
    scope = _load_script(os.path.join(REF, "tests", "test_module_sddmm.py"))
    adj = scipy.sparse.random(127, 255, density=0.1, format="coo").astype("int32")
    scope["test_vanilla_sddmm_cuda"](adj)         # asserts allclose(rtol=atol=1e-4) vs numpy
