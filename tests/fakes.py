"""A CPU stand-in for the CUDA backend, built on the oracle, so that the
host-side logic (Manager, Parameter, Linear, autograd function, conversion,
hooks) can be exercised without a GPU.  Test infrastructure only."""
import numpy as np
import torch

from oracle import oracle as O


class OracleBackend:
    def __init__(self, precision=7):
        self.precision = precision
        self.store = {}

    def write(self, handle, tensor):
        if tensor.dtype != torch.bfloat16:
            raise RuntimeError("Unsupported data type")
        bits = tensor.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16).reshape(-1)
        cont, frac = O.compress_bf16(bits, self.precision)
        self.store[handle] = (bits.size, cont, frac)

    def read(self, handle):
        if handle not in self.store:
            raise RuntimeError("Data not found")
        n, cont, frac = self.store[handle]
        bits = O.decompress_bf16(cont, frac, n, self.precision, canonical_nan=True)
        return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)

    def size(self, handle):
        if handle not in self.store:
            return 0
        _, cont, frac = self.store[handle]
        return cont.size + frac.size

    def linear(self, handle, inputs, shape, bias):
        return torch.nn.functional.linear(inputs, self.read(handle).view(*shape), bias)

    def linear_without_bias(self, handle, inputs, shape):
        return torch.matmul(inputs, self.read(handle).view(*shape).t())

    def export_entry(self, handle):
        n, cont, frac = self.store[handle]
        return {"format": "NZR1", "precision": self.precision, "numel": n,
                "lane_symbols": O.default_lane_symbols(self.precision), "max_unit_words": 0,
                "container": torch.from_numpy(cont.copy()), "fractions": torch.from_numpy(frac.copy())}

    def import_entry(self, handle, blob):
        assert blob["format"] == "NZR1" and blob["precision"] == self.precision
        self.store[handle] = (int(blob["numel"]), blob["container"].numpy().copy(),
                              blob["fractions"].numpy().copy())

    # batched decode with the contract of CodecBackend.make_batch / run_batch: the batch
    # names handles, and every run decodes what those handles hold at that moment
    def make_batch(self, names, outs):
        return (list(names), list(outs))

    def run_batch(self, batch):
        for name, out in zip(*batch):
            w = self.read(name)
            out[:w.numel()].copy_(w)

    def split(self, tensor):
        bits = tensor.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16).reshape(-1)
        e, f = O.split(bits, 7)
        return [torch.from_numpy(e), torch.from_numpy(f)]


def cpu_manager(precision=7):
    import neuzip
    m = neuzip.Manager(algorithm=neuzip.Algorithm.dummy)
    m._be = OracleBackend(precision)
    return m
