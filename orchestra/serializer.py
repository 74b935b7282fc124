"""Re-exports, same layout as the reference's orchestra/serializer.py."""
from ._api import BaseSerializer, SparseSerializer

__all__ = ["BaseSerializer", "SparseSerializer"]
