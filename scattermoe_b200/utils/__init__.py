from . import replace_moe

__all__ = ['replace_moe']
