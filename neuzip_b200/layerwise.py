"""Layer-wise decode: one batched decompress per transformer block.

The reference decompresses each weight inside its own Linear forward
(neuzip/nn/linear.py:30-31 -> neuzip/nn/module.py:27-28), i.e. seven separate
decodes per Llama block.  `attach` registers a forward pre-hook on every module
that directly owns compressed Linears below it (a decoder block) which decodes
all of them with one batched call - one kernel launch in which each matrix gets
a share of the SMs - into a set of decode buffers shared by all blocks, and
hands views of those buffers to the Linears; a forward hook takes them away
again, so that backward (which runs the blocks in the opposite order) falls back
to its own decode.  Only one block is ever held decoded.  Results are identical
to the per-Linear path.
"""
from __future__ import annotations

from typing import Callable, List, Optional

import torch

from .nn import Linear


def _compressed_linears(module: torch.nn.Module, exclude=None) -> List[Linear]:
    return [m for m in module.modules()
            if isinstance(m, Linear) and not (exclude is not None and exclude(m))]


def default_block_filter(module: torch.nn.Module) -> bool:
    """A block = an element of a ``torch.nn.ModuleList`` that contains compressed
    Linears (how transformer implementations hold their layers); attach() marks those.
    Modules whose class name ends in 'DecoderLayer' / 'Block' / 'EncoderLayer' count
    too, for models that keep their layers elsewhere."""
    if not _compressed_linears(module):
        return False
    if getattr(module, "_nz_in_module_list", False):
        return True
    return type(module).__name__.endswith(("DecoderLayer", "Block", "EncoderLayer"))


def _mark_module_list_children(model: torch.nn.Module) -> None:
    for m in model.modules():
        if isinstance(m, torch.nn.ModuleList):
            for child in m:
                # outermost list wins: children of a marked block are not blocks themselves
                child._nz_in_module_list = True


class _Stage:
    """Which block's weights the shared decode buffers hold (-1: none)."""
    __slots__ = ("current",)

    def __init__(self) -> None:
        self.current = -1


def _single_vector(args, kwargs) -> bool:
    """True when the block is called with one token of one sequence."""
    x = args[0] if args else kwargs.get("hidden_states")
    return torch.is_tensor(x) and x.dim() >= 1 and x.numel() == x.shape[-1]


def attach(model: torch.nn.Module, manager,
           is_block: Optional[Callable[[torch.nn.Module], bool]] = None,
           fuse_single_token: bool = False,
           exclude: Optional[Callable[[Linear], bool]] = None) -> List:
    """Install the hooks; returns the hook handles (call .remove() on each to undo).

    Linears for which ``exclude`` is true are left out of their block's batched decode and
    keep decoding on their own - for instance row-parallel shards that add over the ranks
    inside the fused linear kernel (``Manager.fuse_tp_allreduce``).

    With ``fuse_single_token`` a block that is called with a single token (the
    decode step of batch-1 generation) is not decoded ahead: its Linears multiply
    while decoding (``Manager.fuse_vector_linear``), which never writes the bf16
    weights out.  Larger inputs keep the batched decode."""
    is_block = is_block or default_block_filter
    backend = manager._be
    if fuse_single_token:
        manager.fuse_vector_linear(True)
    _mark_module_list_children(model)
    blocks = []
    for m in model.modules():
        # a block inside a block (nested lists) is decoded with its parent
        if is_block(m) and not any(m is not b and any(m is c for c in b.modules()) for b in blocks):
            blocks.append(m)
    # shared decode buffers: slot k is as large as the k-th Linear of the largest block
    sizes: List[int] = []
    for block in blocks:
        for k, lin in enumerate(_compressed_linears(block, exclude)):
            n = int(torch.Size(lin._p._shape).numel())
            if k == len(sizes):
                sizes.append(n)
            else:
                sizes[k] = max(sizes[k], n)
    batched = hasattr(backend, "make_batch")
    device = next((lin._p.device for b in blocks for lin in _compressed_linears(b, exclude)), "cuda")
    buffers = [torch.empty(n, dtype=torch.bfloat16, device=device) for n in sizes] if batched else []
    stage = _Stage()
    handles = []
    for number, block in enumerate(blocks):
        params = [lin._p for lin in _compressed_linears(block, exclude)]
        names = [p._handle for p in params]
        if not params:
            continue
        if batched:
            # The Linears keep their views of the shared buffers for good; a view counts
            # only while `stage.current` names its block, so staging a block is one
            # batched decode and one assignment, and un-staging is one assignment.
            batch = backend.make_batch(names, buffers[:len(names)])
            for k, p in enumerate(params):
                p._staged = buffers[k][:int(torch.Size(p._shape).numel())].view(p._shape)
                p._stage_tag = (stage, number)

            def pre(mod, args, kwargs, _batch=batch, _number=number):
                if fuse_single_token and _single_vector(args, kwargs):
                    return
                backend.run_batch(_batch)
                stage.current = _number

            def post(mod, args, output):
                stage.current = -1
        else:   # a backend without batched decode (the pass-through one)
            own = _Stage()

            def pre(mod, args, kwargs, _params=params, _names=names, _own=own):
                for p, w in zip(_params, manager.read_many(_names)):
                    p._staged = w
                    p._stage_tag = (_own, 0)
                _own.current = 0

            def post(mod, args, output, _params=params, _own=own):
                _own.current = -1
                for p in _params:
                    p._staged = None

        handles.append(block.register_forward_pre_hook(pre, with_kwargs=True))
        handles.append(block.register_forward_hook(post))
    return handles
