"""neuzip_b200: the NeuZip weight codec (bf16 split + rANS-coded exponents)
written for B200 / sm_100a, behind the Python API of BorealisAI/neuzip.

Package root mirrors neuzip/__init__.py:10-35: ``nn``, ``ops``, ``Algorithm``,
``Manager`` and the two in-backward SGD hooks.
"""
import torch

from . import nn, ops
from .binding import Algorithm, Manager

__all__ = ["ops", "nn", "Algorithm", "Manager", "lomo_hook", "compressed_lomo_hook"]
__version__ = "0.1.0"


def lomo_hook(scheduler, param):
    """Plain-parameter SGD step inside backward (neuzip/__init__.py:16-22)."""
    if param.grad is None:
        return
    lr = scheduler.get_last_lr()[0]
    with torch.no_grad():
        param.data.add_(param.grad, alpha=-lr)
    del param.grad


def compressed_lomo_hook(scheduler, param):
    """SGD step on a compressed parameter inside backward: decompress, apply
    ``-lr * _gradient``, recompress under the same handle (neuzip/__init__.py:25-35)."""
    if param._gradient is None:
        return
    lr = scheduler.get_last_lr()[0]
    with torch.no_grad():
        weight = param()
        weight.add_(param._gradient, alpha=-lr)
        param._manager.write(weight, param._handle)
    param._gradient = None
    del param.grad
