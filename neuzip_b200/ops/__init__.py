from .linear import CompressedLinear

__all__ = ["CompressedLinear"]
