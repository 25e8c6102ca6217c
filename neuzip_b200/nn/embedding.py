"""Embedding with a compressed table (reference: neuzip/nn/embedding.py:13-39).
The reference decompresses the whole table for every call and then gathers;
here a lookup decodes only the units of the stored stream that hold the
requested rows (``Manager.read_rows``).  ``max_norm`` renormalises table rows in
place in torch, which a read-only compressed table cannot do: with it set the
whole table is decompressed as in the reference."""
import torch
import torch.nn.functional as F

from .module import Parameter

_COPIED = ("num_embeddings", "embedding_dim", "padding_idx", "max_norm", "norm_type",
           "scale_grad_by_freq", "sparse")


class Embedding(torch.nn.Module):
    def __init__(self, manager, embedding: torch.nn.Embedding) -> None:
        super().__init__()
        self.manager = manager
        for name in _COPIED:
            setattr(self, name, getattr(embedding, name))
        self._p = Parameter(manager, embedding.weight)

    def forward(self, x):
        staged = self._p.staged()
        if self.max_norm is not None or staged is not None or not hasattr(self.manager, "read_rows"):
            return F.embedding(x, self._p(), self.padding_idx, self.max_norm, self.norm_type,
                               self.scale_grad_by_freq, self.sparse)
        # padding_idx only masks the gradient of a row, and the table takes none
        return self.manager.read_rows(self._p._handle, x).to(self._p.device)

    def extra_repr(self) -> str:
        return "! " + ", ".join(f"{name}={getattr(self, name)}" for name in _COPIED)
