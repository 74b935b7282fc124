"""Re-exports, same layout as the reference's orchestra/loss_fns.py."""
from ._api import CrossEntropy, Mse

__all__ = ["CrossEntropy", "Mse"]
