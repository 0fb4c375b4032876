"""Importing this sub-package installs the Hugging Face MoE patches (`replace_moe`), which is what importing the
reference's `scattermoe.utils` does. `consolidate` turns ModuleList experts into fused tensors (the step the
reference's abandoned Qwen3 patch needed, scattermoe/utils/replace_moe.py:97-208)."""
from . import replace_moe
from . import consolidate

__all__ = ['replace_moe', 'consolidate']
