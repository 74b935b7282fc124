"""Re-exports, same layout as the reference's orchestra/arch.py."""
from ._api import Conv2d, Dense, MaxPooling

__all__ = ["Conv2d", "Dense", "MaxPooling"]
