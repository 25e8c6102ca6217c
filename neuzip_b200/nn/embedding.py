"""Embedding with a compressed table (reference: neuzip/nn/embedding.py:13-39):
the whole table is decompressed for every call, then gathered."""
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
        return F.embedding(x, self._p(), self.padding_idx, self.max_norm, self.norm_type,
                           self.scale_grad_by_freq, self.sparse)

    def extra_repr(self) -> str:
        return "! " + ", ".join(f"{name}={getattr(self, name)}" for name in _COPIED)
