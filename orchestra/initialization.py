"""Re-exports, same layout as the reference's orchestra/initialization.py."""
from ._api import Const, Kaiming, Lecun, LecunUniform, Normal, Uniform, UniformInclusive, Xavier, XavierUniform

__all__ = ["Const", "Kaiming", "Lecun", "LecunUniform", "Normal", "Uniform", "UniformInclusive", "Xavier", "XavierUniform"]
