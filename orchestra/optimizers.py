"""Re-exports, same layout as the reference's orchestra/optimizers.py."""
from ._api import Adam, GradientDescent, GradientDescentWithMomentum

__all__ = ["Adam", "GradientDescent", "GradientDescentWithMomentum"]
