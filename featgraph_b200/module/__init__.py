"""Module layer: the four classes python/featgraph/module/__init__.py:1-2 exports, plus
PartitionedSDDMMcuda (the reference's 2-D edge blocking on the GPU)."""
from .spmm import SpMMbase, VanillaSpMMx86, VanillaSpMMcuda
from .sddmm import SDDMMbase, VanillaSDDMMx86, VanillaSDDMMcuda, PartitionedSDDMMcuda

__all__ = ["VanillaSpMMx86", "VanillaSpMMcuda", "VanillaSDDMMx86", "VanillaSDDMMcuda",
           "PartitionedSDDMMcuda", "SpMMbase", "SDDMMbase"]
