"""Linear layer with a compressed weight (reference: neuzip/nn/linear.py:14-35)."""
import torch

from ..ops import CompressedLinear
from .module import Parameter


class Linear(torch.nn.Module):
    def __init__(self, manager, linear: torch.nn.Linear, tp=None) -> None:
        """`tp = (mode, rank, world_size, group)` (not in the reference) keeps only this
        rank's block of the weight: rows for mode "column", columns for "row"; a
        row-parallel Linear adds the ranks' partial outputs with one all-reduce."""
        super().__init__()
        self.manager = manager
        weight, bias = linear.weight.data, (None if linear.bias is None else linear.bias.data)
        self.reduce_group = None
        self.reduce_output = False
        if tp is not None:
            from ..sharding import shard_linear_weight
            mode, rank, world, group = tp
            weight, bias = shard_linear_weight(weight, bias, mode, rank, world)
            self.reduce_output = mode == "row" and world > 1
            self.reduce_group = group
        self.out_features, self.in_features = int(weight.shape[0]), int(weight.shape[1])
        self._p = Parameter(manager, weight, operand=True)
        if bias is None:
            self.register_parameter("bias", None)
        else:
            self.bias = torch.nn.Parameter(bias)

    @property
    def weight(self) -> Parameter:
        return self._p

    @classmethod
    def from_compressed(cls, manager, state, bias=None, device=None):
        """A compressed Linear straight from stored bytes (`state` = what get_extra_state
        returned): no dense weight is ever built, so a checkpoint of a converted model loads
        into a model that was never materialised."""
        self = cls.__new__(cls)
        torch.nn.Module.__init__(self)
        self.manager = manager
        self.reduce_group = None
        self.reduce_output = bool(state.get("reduce_output", False))
        self._p = Parameter.from_entry(manager, state, device=device)
        self.out_features, self.in_features = int(self._p._shape[0]), int(self._p._shape[1])
        if bias is None:
            self.register_parameter("bias", None)
        else:
            self.bias = torch.nn.Parameter(bias.to(self._p.device))
        return self

    def forward(self, x):
        if self.reduce_output and not torch.is_grad_enabled():
            # one kernel multiplies and adds over the ranks (peer stores), when switched on
            y = self._p.linear_allreduce(x, self.bias)
            if y is not None:
                return y
        y = self._forward_local(x)
        if self.reduce_output:
            # partial sums of a row-parallel Linear: one all-reduce over the ranks
            import torch.distributed as dist
            if torch.is_grad_enabled() and y.requires_grad:
                from torch.distributed.nn.functional import all_reduce
                y = all_reduce(y, group=self.reduce_group)
            else:
                dist.all_reduce(y, group=self.reduce_group)
        return y

    def _forward_local(self, x):
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
        state = self._p._manager.export_entry(self._p._handle)
        state["reduce_output"] = self.reduce_output      # a row-parallel shard (tensor parallelism)
        return state

    def set_extra_state(self, state):
        if state is None:
            return
        self._p._manager.import_entry(state, self._p._handle)
        self._p._shape = torch.Size(state["shape"])

    def extra_repr(self) -> str:
        return (f"! in_features={self.in_features}, out_features={self.out_features}, "
                f"bias={self.bias is not None}")
