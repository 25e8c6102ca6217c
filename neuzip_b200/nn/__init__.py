from .embedding import Embedding
from .linear import Linear
from .module import Parameter

__all__ = ["Parameter", "Linear", "Embedding"]
