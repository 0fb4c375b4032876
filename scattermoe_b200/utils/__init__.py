"""Importing this sub-package installs the Hugging Face MoE patches (`replace_moe`), which is what importing the
reference's `scattermoe.utils` does."""
from . import replace_moe

__all__ = ['replace_moe']
