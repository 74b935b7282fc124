"""Re-exports, same layout as the reference's orchestra/activations.py."""
from ._api import GELU, ReLU, Sigmoid, Softmax, Tanh

__all__ = ["GELU", "ReLU", "Sigmoid", "Softmax", "Tanh"]
