"""`import scattermoe` for code written against shawntan/scattermoe: every name resolves to scattermoe_b200.

The reference's module tree (scattermoe/__init__.py:1-15) is `scattermoe.{parallel_experts, kernels, kernels.ops,
kernels.single, mlp, utils, utils.replace_moe}`; each of those names is bound here to the module of the same name
in `scattermoe_b200`, as attributes AND in `sys.modules`, so `from scattermoe.mlp import MLP`, `import
scattermoe.kernels.ops` and `scattermoe.kernels.ops.ALLOW_TF32 = False` (what the reference's own test does,
tests/test_mlp.py:5-8) all reach the one implementation. Importing it patches the Hugging Face MoE blocks exactly
as importing the reference does (scattermoe/utils/__init__.py:1).
"""
import sys as _sys

import scattermoe_b200 as _impl
from scattermoe_b200 import (ParallelExperts, flatten_sort_count, kernels, mlp, parallel_experts,  # noqa: F401
                             parallel_linear, utils)
import scattermoe_b200.kernels.ops  # noqa: F401
import scattermoe_b200.kernels.single  # noqa: F401
import scattermoe_b200.utils.replace_moe  # noqa: F401

for _sub in ("parallel_experts", "kernels", "kernels.ops", "kernels.single", "mlp", "utils", "utils.replace_moe"):
    _sys.modules[__name__ + "." + _sub] = _sys.modules["scattermoe_b200." + _sub]

__all__ = ["flatten_sort_count", "parallel_linear", "ParallelExperts", "parallel_experts", "kernels", "mlp", "utils"]
