"""Module layer: the four classes python/featgraph/module/__init__.py:1-2 exports."""
from .spmm import SpMMbase, VanillaSpMMx86, VanillaSpMMcuda
from .sddmm import SDDMMbase, VanillaSDDMMx86, VanillaSDDMMcuda

__all__ = ["VanillaSpMMx86", "VanillaSpMMcuda", "VanillaSDDMMx86", "VanillaSDDMMcuda",
           "SpMMbase", "SDDMMbase"]
