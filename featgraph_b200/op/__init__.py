"""Op layer: the ten names python/featgraph/op/__init__.py:1-5 exports."""
from .vanilla_spmm import (vanilla_spmm_csr_cuda, schedule_vanilla_spmm_csr_cuda,
                           vanilla_spmm_csr_x86, schedule_vanilla_spmm_csr_x86,
                           vanilla_spmm_dds_x86, schedule_vanilla_spmm_dds_x86)
from .vanilla_sddmm import (vanilla_sddmm, schedule_vanilla_sddmm_cuda_tree_reduce,
                            schedule_vanilla_sddmm_cuda_single_thread_reduce,
                            schedule_vanilla_sddmm_x86)

__all__ = [
    "vanilla_spmm_csr_cuda", "schedule_vanilla_spmm_csr_cuda",
    "vanilla_spmm_csr_x86", "schedule_vanilla_spmm_csr_x86",
    "vanilla_spmm_dds_x86", "schedule_vanilla_spmm_dds_x86",
    "vanilla_sddmm", "schedule_vanilla_sddmm_cuda_tree_reduce",
    "schedule_vanilla_sddmm_cuda_single_thread_reduce", "schedule_vanilla_sddmm_x86",
]
