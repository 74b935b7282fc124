"""Re-exports, same layout as the reference's orchestra/datasets.py."""
from ._api import InlineDataset, LocalDataset

__all__ = ["InlineDataset", "LocalDataset"]
