"""Generators for the sm100 artifact set: plan.json, tactics.json, toolchain.json per model shape."""
from .builder import Arena, F32, RecipeBuilder, Tensor, U32, Weight, io

__all__ = ["Arena", "F32", "RecipeBuilder", "Tensor", "U32", "Weight", "io"]
