"""Re-exports, same layout as the reference's orchestra/store.py."""
from ._api import BlockingStore, WildStore

__all__ = ["BlockingStore", "WildStore"]
