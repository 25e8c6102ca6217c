"""GPT-2 style ``Conv1D`` with a compressed weight (reference: neuzip/nn/conv1d.py:15-30).
Importable but, as in the reference, not used by ``Manager.convert``."""
import torch

from ..ops import CompressedLinear
from .module import Parameter


class Conv1D(torch.nn.Module):
    def __init__(self, manager, conv) -> None:
        super().__init__()
        self.manager = manager
        self.in_features, self.out_features = conv.weight.shape
        self._p = Parameter(manager, conv.weight.data)
        if conv.bias is None:
            self.register_parameter("bias", None)
        else:
            self.bias = torch.nn.Parameter(conv.bias.data)

    def forward(self, x):
        return CompressedLinear.apply(x, self._p, self.bias)

    def extra_repr(self) -> str:
        return (f"! in_features={self.in_features}, out_features={self.out_features}, "
                f"bias={self.bias is not None}")
