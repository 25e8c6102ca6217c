"""Autograd function of the compressed Linear (reference: neuzip/ops/linear.py:11-46).

Forward: ``y = x @ W^T (+ b)`` with ``W`` decompressed on the fly by the manager.
Backward: decompress ``W`` again, ``dX = dY @ W``, ``dW = dY^T @ X``.  ``dW`` is
accumulated in ``_p._gradient``; the gradient returned for ``_p`` is a zero-size
tensor matching its zero-size storage, which is what lets post-accumulate-grad
hooks (the in-backward optimiser step) fire for the parameter.
"""
import torch


class CompressedLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, inputs, _p, bias):
        ctx._inputs_dtype = inputs.dtype
        if torch.is_autocast_enabled():
            inputs = inputs.to(torch.get_autocast_gpu_dtype())   # autograd.Function bypasses autocast
        ctx.save_for_backward(inputs, bias)
        ctx.carry = (_p,)
        return _p.linear(inputs, bias)

    @staticmethod
    def backward(ctx, grad_output):
        inputs, bias = ctx.saved_tensors
        (_p,) = ctx.carry
        x2d = inputs.reshape(-1, inputs.shape[-1])
        g2d = grad_output.reshape(-1, grad_output.shape[-1])
        weight = _p()
        grad_inputs = torch.mm(g2d, weight).reshape(inputs.shape).to(ctx._inputs_dtype)
        del weight
        grad_weight = torch.mm(g2d.t(), x2d)
        if _p._gradient is None:
            _p._gradient = grad_weight
        else:
            _p._gradient.add_(grad_weight)
        grad_bias = g2d.sum(0) if bias is not None else None
        return grad_inputs, torch.empty_like(_p.data), grad_bias
