"""``nd`` namespace: device arrays (stands in for ``tvm.nd``)."""
from .runtime import NDArray, array, empty, zeros  # noqa: F401
