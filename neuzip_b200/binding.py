"""The user-facing ``Manager`` and ``Algorithm`` (reference: neuzip/binding.py).

``Manager`` hands out string handles for compressed tensors, remembers their
shapes and forwards to a backend object that has the six methods of the
reference's extension classes.  The backend is either the pass-through
``DummyBackend`` (``Algorithm.dummy``) or a ``Manager_f{precision}_n{normalizer}``
class from :mod:`neuzip_b200.backend`, looked up by name exactly as the
reference does (neuzip/binding.py:69-70).
"""
from __future__ import annotations

import enum
from typing import Dict, Optional, Tuple

import torch

from . import backend as _backend
from .backend import _cuda


class Algorithm(enum.Enum):
    """neuzip/binding.py:23-27.  Only ``ans`` and ``dummy`` are implemented."""
    ans = _cuda.Algorithm.ans
    gdeflate = _cuda.Algorithm.gdeflate
    zstd = _cuda.Algorithm.zstd
    dummy = "dummy"


class DummyBackend:
    """Stores tensors uncompressed on the GPU (neuzip/binding.py:35-52).  Unlike
    the reference's, it also answers ``linear_without_bias`` and ``split``-less
    callers get a clear error instead of an AttributeError deep in a forward."""

    def __init__(self) -> None:
        self._store: Dict[str, torch.Tensor] = {}

    def write(self, handle: str, tensor: torch.Tensor) -> None:
        self._store[handle] = tensor.cuda()

    def read(self, handle: str) -> torch.Tensor:
        return self._store[handle]

    def size(self, handle: str) -> int:
        t = self._store[handle]
        return t.numel() * t.element_size()

    @torch.no_grad()
    def linear(self, handle: str, inputs: torch.Tensor, shape, bias=None) -> torch.Tensor:
        return torch.nn.functional.linear(inputs, self.read(handle).reshape(shape), bias)

    def linear_without_bias(self, handle: str, inputs: torch.Tensor, shape) -> torch.Tensor:
        return self.linear(handle, inputs, shape, None)

    def split(self, tensor: torch.Tensor):
        raise NotImplementedError("Algorithm.dummy has no split()")


class Manager:
    """neuzip/binding.py:55-115, same constructor and methods."""

    def __init__(self, algorithm: Algorithm = Algorithm.ans, precision: int = 7,
                 normalizer_size: Optional[int] = None, chunk_size: int = 2 ** 16) -> None:
        normalizer_size = 0 if normalizer_size is None else normalizer_size
        if algorithm == Algorithm.dummy:
            self._be = DummyBackend()
        else:
            if precision not in _backend.PRECISIONS:
                raise ValueError(f"precision must be one of {_backend.PRECISIONS}, got {precision}")
            if normalizer_size not in _backend.NORMALIZER_SIZES:
                raise ValueError(f"normalizer_size must be one of {_backend.NORMALIZER_SIZES}")
            factory = getattr(_cuda, f"Manager_f{precision}_n{normalizer_size}")
            self._be = factory(algorithm.value, chunk_size)
        self.meta_dict: Dict[str, torch.Size] = {}

    def write(self, tensor: torch.Tensor, handle: Optional[str] = None,
              operand: Optional[bool] = None) -> str:
        """Compress ``tensor`` and return its handle; an existing handle is replaced.
        ``operand=True`` (not in the reference) marks a 2-D weight that will be the matrix
        of `linear`: the backend may then store it in the order the fused GEMM wants; what
        `read` returns is the same either way."""
        if handle is None:
            handle = str(len(self.meta_dict))
        self.meta_dict[handle] = tensor.shape
        if operand is None or not getattr(self._be, "supports_operand_order", False):
            self._be.write(handle, tensor)
        else:
            self._be.write(handle, tensor, operand=operand)
        return handle

    def read(self, handle: str) -> torch.Tensor:
        """Decompress to a CUDA tensor of the original shape (no grad)."""
        shape = self.meta_dict[handle]
        return self._be.read(handle).requires_grad_(False).reshape(shape)

    def size(self, handle: str) -> int:
        return self._be.size(handle)

    def linear(self, handle: str, inputs: torch.Tensor, bias=None) -> torch.Tensor:
        shape = self.meta_dict[handle]
        if bias is None:
            return self._be.linear_without_bias(handle, inputs, shape)
        return self._be.linear(handle, inputs, shape, bias)

    def convert(self, module: torch.nn.Module, tp_rank: Optional[int] = None,
                tp_world: Optional[int] = None, tp_plan=None, tp_group=None) -> torch.nn.Module:
        """neuzip/binding.py:105-106.  With ``tp_rank`` / ``tp_world`` (not in the
        reference) the Linears named in ``tp_plan`` (default: the Llama projections, see
        neuzip_b200.sharding) keep only this rank's block, row-parallel ones all-reduce
        their output over ``tp_group``; attention code that derives the head count from
        the projection width (Hugging Face Llama does) then runs tensor-parallel as is."""
        from .utils import _convert
        tp = None
        if tp_world is not None and tp_world > 1:
            if tp_rank is None or not 0 <= tp_rank < tp_world:
                raise ValueError("tp_rank must be in [0, tp_world)")
            tp = (tp_rank, tp_world, tp_plan, tp_group)
        return _convert(self, module, tp=tp)

    def load_converted(self, module: torch.nn.Module, state_dict, device=None) -> torch.nn.Module:
        """Load the state_dict of a converted model into an unconverted `module` (which may
        be on the meta device): compressed Linears are built from the stored bytes, nothing
        is compressed and no dense weight is materialised.  Not in the reference."""
        from .utils import load_converted
        return load_converted(self, module, state_dict, device=device)

    def split(self, tensor: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        exp, frac = self._be.split(tensor)
        return exp.reshape(tensor.shape), frac.reshape(tensor.shape)

    # extras (not in the reference)
    def read_many(self, handles) -> list:
        """Decompress several handles in one batched call (e.g. a whole layer)."""
        handles = list(handles)
        if hasattr(self._be, "read_many"):
            flats = self._be.read_many(handles)
        else:
            flats = [self._be.read(h) for h in handles]
        return [t.requires_grad_(False).reshape(self.meta_dict[h]) for t, h in zip(flats, handles)]

    def read_rows(self, handle: str, rows: torch.Tensor) -> torch.Tensor:
        """``self.read(handle)[rows]`` for a tensor of two or more dimensions, decoding
        only the parts of the stored stream that hold those rows."""
        shape = self.meta_dict[handle]
        if len(shape) < 2:
            raise ValueError("read_rows needs a tensor of at least two dimensions")
        row_len = 1
        for d in shape[1:]:
            row_len *= int(d)
        if hasattr(self._be, "read_rows"):
            flat = self._be.read_rows(handle, rows, row_len)
        else:
            flat = self._be.read(handle).reshape(-1, row_len)[rows.reshape(-1).long()]
        return flat.requires_grad_(False).reshape(tuple(rows.shape) + tuple(shape[1:]))

    def fuse_vector_linear(self, enabled: bool = True) -> None:
        """Let `linear` with a single input vector (batch 1, one token) multiply while
        decoding instead of decompressing the weight first.  Same fp32 arithmetic as
        the library GEMM but a different order of the sums."""
        if hasattr(self._be, "fused_vector_linear"):
            self._be.fused_vector_linear = bool(enabled)

    def fuse_linear(self, max_rows: int = 256) -> None:
        """Let `linear` with at most `max_rows` input rows (tokens) decode the weight
        straight into tensor-core operand tiles instead of decompressing it first
        (0 switches it off).  Same fp32 accumulation as the library GEMM, different order
        of the sums."""
        if hasattr(self._be, "fused_linear_max_rows"):
            self._be.fused_linear_max_rows = int(max_rows)

    def fuse_tp_allreduce(self, group=None, max_rows: int = 256,
                          workspace_bytes: int = 64 << 20) -> None:
        """Tensor parallelism on one node: let row-parallel Linears with at most `max_rows`
        input rows add their partial outputs inside the fused linear kernel, which stores them
        into every rank's memory over NVLink, instead of an all-reduce after it.  Collective:
        every rank of `group` calls it (it exchanges memory handles over the group);
        `group=None` with `max_rows=0` switches it off again."""
        old = getattr(self, "_reducer", None)
        if old is not None:
            old.close()
        self._reducer, self._reducer_rows = None, 0
        if max_rows and hasattr(self._be, "linear_allreduce"):
            from .tpcomm import PeerReducer
            self._reducer = PeerReducer(group, workspace_bytes)
            self._reducer_rows = int(max_rows)

    def linear_allreduce(self, handle: str, inputs: torch.Tensor, bias=None):
        """The summed output of a row-parallel shard, or None when the fused path is off or
        the call does not qualify (then: `linear` and an all-reduce)."""
        reducer = getattr(self, "_reducer", None)
        if reducer is None:
            return None
        limit, self._be.fused_linear_max_rows = self._be.fused_linear_max_rows, self._reducer_rows
        try:
            return self._be.linear_allreduce(handle, inputs, self.meta_dict[handle], bias, reducer)
        finally:
            self._be.fused_linear_max_rows = limit

    def export_entry(self, handle: str) -> dict:
        """Stored bytes + metadata of a handle (for checkpoints)."""
        blob = self._be.export_entry(handle)
        blob["shape"] = tuple(self.meta_dict[handle])
        return blob

    def import_entry(self, blob: dict, handle: Optional[str] = None) -> str:
        """Register compressed bytes produced by `export_entry` under a handle."""
        if handle is None:
            handle = str(len(self.meta_dict))
        self.meta_dict[handle] = torch.Size(blob["shape"])
        self._be.import_entry(handle, blob)
        return handle

    def check(self) -> None:
        """Raise if any decode so far flagged a malformed container."""
        if hasattr(self._be, "check"):
            self._be.check()

    def total_size(self) -> int:
        return sum(self.size(h) for h in self.meta_dict)
