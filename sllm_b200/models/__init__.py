"""Architectures.  Importing this package registers each of them."""
from . import gerupel, kidolorn, nutopel, qwen2, rososun  # noqa: F401
from .causal_lm import CausalLM

__all__ = ["CausalLM", "gerupel", "kidolorn", "nutopel", "qwen2", "rososun"]
