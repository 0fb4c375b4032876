"""scattermoe_b200: the ScatterMoE `ParallelLinear` hot path on B200 (sm_100a).

Same package surface as the reference's scattermoe/__init__.py:1-15; use it as

    import scattermoe_b200 as scattermoe

Importing the package installs the Hugging Face MoE patches (utils.replace_moe), as importing the reference
does (scattermoe/__init__.py:5 -> utils/__init__.py:1).
"""
from .parallel_experts import expert_mlp, flatten_sort_count, parallel_linear, parallel_linear_act, ParallelExperts
from . import parallel_experts
from . import kernels
from . import mlp
from . import utils
from .routing import route_topk
from ._lib import check_device_status, library_path

__all__ = [
    "flatten_sort_count",
    "parallel_linear",
    "parallel_linear_act",
    "expert_mlp",
    "route_topk",
    "ParallelExperts",
    "parallel_experts",
    "kernels",
    "mlp",
    "utils",
    "check_device_status",
    "library_path",
]
