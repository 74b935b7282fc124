"""Re-exports, same layout as the reference's orchestra/sync.py."""
from ._api import BarrierSync, NonBlockingSync

__all__ = ["BarrierSync", "NonBlockingSync"]
