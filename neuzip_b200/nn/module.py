"""Compressed parameter (reference: neuzip/nn/module.py:11-28)."""
import torch


class Parameter(torch.nn.Parameter):
    """An ``nn.Parameter`` whose own storage is empty; the values live in the
    manager under ``_handle``.  Calling the parameter decompresses it.  The
    real weight gradient is collected in ``_gradient`` by the autograd function,
    ``.grad`` only ever holds a zero-size placeholder."""

    def __new__(cls, manager, data, requires_grad=True, operand=None):
        placeholder = torch.zeros(0, dtype=data.dtype, device=data.device)
        self = super().__new__(cls, placeholder, requires_grad)
        self._manager = manager
        self._shape = data.shape
        self._gradient = None
        # operand=True: this tensor is the weight of a Linear (not in the reference's signature)
        self._handle = manager.write(data) if operand is None else manager.write(data, operand=operand)
        self._staged = None        # view of a shared decode buffer (neuzip_b200.layerwise)
        self._stage_tag = None     # (stage, block number): the view is valid while they agree
        return self

    @classmethod
    def from_entry(cls, manager, blob, device=None):
        """A parameter for bytes that are already compressed (an entry made by
        ``Manager.export_entry``, e.g. out of a checkpoint): registered under a new handle,
        nothing is decompressed or compressed.  Not in the reference, which cannot load a
        converted model at all (its state_dict holds only the empty placeholder)."""
        device = device if device is not None else ("cuda" if torch.cuda.is_available() else "cpu")
        placeholder = torch.zeros(0, dtype=torch.bfloat16, device=device)
        self = torch.nn.Parameter.__new__(cls, placeholder, True)
        self._manager = manager
        self._shape = torch.Size(blob["shape"])
        self._gradient = None
        self._handle = manager.import_entry(blob)
        self._staged = None
        self._stage_tag = None
        return self

    def staged(self):
        """The already decoded weight, if a layer-wise prefetch holds it right now."""
        tag = self._stage_tag
        if tag is not None and tag[0].current == tag[1]:
            return self._staged
        return None

    @torch.no_grad()
    def __call__(self) -> torch.Tensor:
        staged = self.staged()
        if staged is not None:
            return staged
        w = self._manager.read(self._handle).reshape(self._shape)
        return w.to(self.device).requires_grad_(False)

    def linear_allreduce(self, inputs, bias=None):
        """Row-parallel shard: the output summed over the ranks by the fused kernel, or None."""
        fn = getattr(self._manager, "linear_allreduce", None)
        if fn is None or self.staged() is not None:
            return None
        return fn(self._handle, inputs, bias)

    def linear(self, inputs, bias=None):
        staged = self.staged()
        if staged is not None:
            # a layer-wise prefetch (neuzip_b200.layerwise) already decoded this weight
            return torch.nn.functional.linear(inputs, staged, bias)
        return self._manager.linear(self._handle, inputs, bias).to(self.device)
