"""Utilities exported as in python/featgraph/util/__init__.py:1."""
from .adj_partitioning import util_convert_csr_to_dds, util_partition_adj_coo_2d

__all__ = ["util_convert_csr_to_dds", "util_partition_adj_coo_2d"]
