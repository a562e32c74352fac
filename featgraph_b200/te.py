"""``te`` namespace: input placeholders (stands in for ``tvm.te.placeholder``)."""
from .runtime import Placeholder, placeholder  # noqa: F401
