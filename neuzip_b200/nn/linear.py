"""Linear layer with a compressed weight (reference: neuzip/nn/linear.py:14-35)."""
import torch

from ..ops import CompressedLinear
from .module import Parameter


class Linear(torch.nn.Module):
    def __init__(self, manager, linear: torch.nn.Linear) -> None:
        super().__init__()
        self.manager = manager
        self.in_features, self.out_features = linear.in_features, linear.out_features
        self._p = Parameter(manager, linear.weight.data, operand=True)
        if linear.bias is None:
            self.register_parameter("bias", None)
        else:
            self.bias = torch.nn.Parameter(linear.bias.data)

    @property
    def weight(self) -> Parameter:
        return self._p

    def forward(self, x):
        if not torch.is_grad_enabled():
            staged = self._p.staged()
            if staged is not None:          # decoded ahead for the whole block: a plain linear
                return torch.nn.functional.linear(x, staged, self.bias)
        if not (torch.is_grad_enabled() and (x.requires_grad or self._p.requires_grad)):
            # inference: same arithmetic without the autograd.Function round trip
            if torch.is_autocast_enabled():
                x = x.to(torch.get_autocast_gpu_dtype())
            return self._p.linear(x, self.bias)
        return CompressedLinear.apply(x, self._p, self.bias)

    # The reference's state_dict of a converted model only holds the zero-size
    # placeholder (neuzip/nn/module.py:13), so saving it loses the weights.  Here the
    # compressed bytes travel as the module's extra state: a checkpoint of a converted
    # model holds containers + fractions and loads without a bf16 staging copy.
    def get_extra_state(self):
        return self._p._manager.export_entry(self._p._handle)

    def set_extra_state(self, state):
        if state is None:
            return
        self._p._manager.import_entry(state, self._p._handle)
        self._p._shape = torch.Size(state["shape"])

    def extra_repr(self) -> str:
        return (f"! in_features={self.in_features}, out_features={self.out_features}, "
                f"bias={self.bias is not None}")
