"""Model surgery (reference: neuzip/utils.py:19-68)."""
import logging

import torch

from .nn import Embedding, Linear

logger = logging.getLogger(__name__)


def _hf_conv1d_type():
    try:
        from transformers.pytorch_utils import Conv1D
        return Conv1D
    except Exception:   # transformers is optional for the codec itself
        return ()


def _set_module_by_name(parent_module, name, child_module):
    """Replace the sub-module at the dotted path ``name`` (neuzip/utils.py:19-31)."""
    *path, leaf = name.split(".")
    node = parent_module
    for part in path:
        node = node[int(part)] if part.isnumeric() else getattr(node, part)
    setattr(node, leaf, child_module)


def _delete_module(module):
    """Drop the parameters of a replaced module so their memory can be freed
    (neuzip/utils.py:34-38)."""
    for pname, _ in list(module.named_parameters()):
        setattr(module, pname, None)


def _unroll_convert(manager, module):
    """Flat variant that also converts embeddings (neuzip/utils.py:41-54; unused by
    ``Manager.convert``)."""
    for name, m in list(module.named_modules()):
        if isinstance(m, torch.nn.Linear):
            replacement = Linear(manager, m)
        elif isinstance(m, torch.nn.Embedding):
            replacement = Embedding(manager, m)
        else:
            continue
        logger.debug("Quantizing %s: %s", name, m)
        _set_module_by_name(module, name, replacement)
        _delete_module(m)
    return module


def _convert(manager, module, prefix="", tp=None):
    """Recursively replace ``nn.Linear`` (and HF ``Conv1D``) children by compressed
    Linears; any child whose name contains ``lm_head`` is left alone and not
    descended into (neuzip/utils.py:57-68).

    ``tp = (rank, world_size, plan, group)`` (not in the reference) makes every Linear
    whose name is in the plan keep only this rank's block (neuzip_b200.sharding);
    Linears that the plan does not name are converted whole on every rank."""
    from .sharding import tp_mode
    convertible = (torch.nn.Linear,) + ((_hf_conv1d_type(),) if _hf_conv1d_type() else ())
    for name, child in list(module.named_children()):
        full_name = f"{prefix}.{name}" if prefix else name
        if "lm_head" in name:
            continue
        if isinstance(child, convertible):
            logger.debug("Converting %s: %s", full_name, child)
            shard = None
            if tp is not None and tp[1] > 1:
                mode = tp_mode(name, tp[2])
                if mode is not None:
                    shard = (mode, tp[0], tp[1], tp[3])
            setattr(module, name, Linear(manager, child, tp=shard))
            _delete_module(child)
        else:
            _convert(manager, child, full_name, tp)
    return module


def load_converted(manager, module, state_dict, prefix="", device=None):
    """Load a checkpoint of a *converted* model (compressed bytes as module extra state)
    into `module`, which may live on the meta device and must not have been converted:
    every ``nn.Linear`` whose ``<name>._extra_state`` is in the checkpoint becomes a
    compressed Linear built from those bytes (nothing is compressed, no dense copy of
    the weight exists at any time); all other tensors of the checkpoint are assigned.
    The reference cannot do this: a converted model's state_dict loses the weights
    (neuzip/nn/module.py:13)."""
    consumed = set()

    def walk(mod, pre):
        for name, child in list(mod.named_children()):
            full = f"{pre}{name}"
            key = f"{full}._extra_state"
            if isinstance(child, torch.nn.Linear) and key in state_dict:
                bias = state_dict.get(f"{full}.bias")
                setattr(mod, name, Linear.from_compressed(manager, state_dict[key], bias, device))
                consumed.update({key, f"{full}.bias", f"{full}._p"})
            else:
                walk(child, f"{full}.")

    walk(module, prefix)
    rest = {k[len(prefix):]: v for k, v in state_dict.items()
            if k.startswith(prefix) and k not in consumed}
    if device is not None:
        rest = {k: (v.to(device) if torch.is_tensor(v) else v) for k, v in rest.items()}
    missing, unexpected = module.load_state_dict(rest, strict=False, assign=True)
    missing = [k for k in missing if not k.endswith(("._p", "._extra_state", ".bias"))
               or k in rest]
    if missing or unexpected:
        raise RuntimeError(f"load_converted: missing keys {missing}, unexpected keys {unexpected}")
    return module
