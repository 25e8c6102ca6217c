"""Host-side logic on CPU: the API surface of the reference (names, defaults,
error behaviour) and the Manager / nn / ops / utils code running over a fake
backend that uses the oracle codec."""
import inspect

import numpy as np
import pytest
import torch

import neuzip
import neuzip_b200
from tests.fakes import OracleBackend, cpu_manager


def test_package_surface_matches_reference_names():
    import neuzip.nn, neuzip.ops, neuzip.binding, neuzip.utils  # noqa: F401
    assert neuzip.Manager is neuzip_b200.Manager
    assert set(neuzip.__all__) >= {"ops", "nn", "Algorithm", "Manager"}
    assert callable(neuzip.lomo_hook) and callable(neuzip.compressed_lomo_hook)
    assert [a.name for a in neuzip.Algorithm] == ["ans", "gdeflate", "zstd", "dummy"]
    assert neuzip.Algorithm.dummy.value == "dummy"

    assert neuzip.nn.__all__ == ["Parameter", "Linear", "Embedding"]
    assert neuzip.ops.__all__ == ["CompressedLinear"]
    from neuzip.nn import conv1d  # importable, as in the reference
    assert hasattr(neuzip.utils, "_convert") and hasattr(neuzip.utils, "_unroll_convert")
    sig = inspect.signature(neuzip.Manager.__init__)
    assert list(sig.parameters)[1:] == ["algorithm", "precision", "normalizer_size", "chunk_size"]
    assert sig.parameters["precision"].default == 7
    assert sig.parameters["chunk_size"].default == 2 ** 16
    assert sig.parameters["normalizer_size"].default is None


def test_backend_class_names_of_the_extension_exist():
    cu = neuzip._cuda
    for p in (0, 1, 3, 7):
        for n in (0, 1, 2, 4, 8, 16, 32, 64, 128, 256, 512, 1024):
            cls = getattr(cu, f"Manager_f{p}_n{n}")
            for meth in ("read", "write", "size", "linear", "linear_without_bias", "split"):
                assert callable(getattr(cls, meth))
    assert [a.name for a in cu.Algorithm] == ["ans", "bitcomp", "lz4", "zstd", "gdeflate"]
    with pytest.raises(AttributeError):
        cu.Manager_f2_n0


def test_unsupported_combinations_raise_clearly():
    with pytest.raises(ValueError):
        neuzip.Manager(precision=2)
    with pytest.raises(ValueError):
        neuzip.Manager(normalizer_size=3)
    with pytest.raises(NotImplementedError):
        neuzip.Manager(algorithm=neuzip.Algorithm.zstd)
    assert neuzip.Manager(precision=3, normalizer_size=512)._be.normalizer_size == 512
    m = neuzip.Manager()                       # constructing the real backend needs no GPU
    assert m._be.precision == 7 and m._be.lane_symbols == 256
    assert m.size("nope") == 0
    with pytest.raises(RuntimeError, match="Data not found"):
        m._be.read("nope")
    with pytest.raises(RuntimeError, match="Unsupported data type"):
        m._be.write("x", torch.zeros(4))


def test_manager_handles_shapes_and_rewrite():
    m = cpu_manager()
    a = (torch.randn(6, 10) * 0.02).to(torch.bfloat16)
    b = (torch.randn(3, 4, 5) * 0.02).to(torch.bfloat16)
    ha, hb = m.write(a), m.write(b)
    assert (ha, hb) == ("0", "1")
    assert torch.equal(m.read(ha), a) and m.read(hb).shape == b.shape
    assert not m.read(ha).requires_grad
    assert m.write(b[0], ha) == ha and m.read(ha).shape == b[0].shape
    assert m.size(ha) > 0 and m.size("missing") == 0
    e, f = m.split(a)
    assert e.shape == a.shape and f.shape == a.shape


@pytest.mark.parametrize("precision", (0, 1, 3, 7))
def test_linear_forward_backward_against_torch(precision):
    torch.manual_seed(precision)
    m = cpu_manager(precision)
    lin = torch.nn.Linear(32, 24, bias=True).to(torch.bfloat16)
    cl = neuzip.nn.Linear(m, lin)
    assert cl.weight is cl._p and cl._p.numel() == 0 and cl._p._shape == (24, 32)
    assert cl.extra_repr().startswith("! in_features=32")
    w_used = cl._p()                       # the (possibly lossy) weight actually stored
    if precision == 7:
        assert torch.equal(w_used, lin.weight.data)
    x = torch.randn(5, 7, 32, dtype=torch.bfloat16, requires_grad=True)
    y = cl(x)
    y.float().pow(2).sum().backward()
    xr = x.detach().clone().requires_grad_(True)
    wr = w_used.clone().requires_grad_(True)
    br = lin.bias.detach().clone().requires_grad_(True)
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.float().pow(2).sum().backward()
    # same library GEMMs on the same operands: tolerance only covers summation order
    assert torch.allclose(y.float(), yr.float(), atol=1e-2, rtol=1e-2)
    assert torch.allclose(x.grad.float(), xr.grad.float(), atol=1e-2, rtol=2e-2)
    assert cl._p._gradient.shape == (24, 32)
    assert torch.allclose(cl._p._gradient.float(), wr.grad.float(), atol=1e-2, rtol=2e-2)
    assert torch.allclose(cl.bias.grad.float(), br.grad.float(), atol=1e-2, rtol=2e-2)
    assert cl._p.grad is not None and cl._p.grad.numel() == 0
    # a second backward accumulates into _gradient
    g1 = cl._p._gradient.clone()
    cl(x.detach()).float().pow(2).sum().backward()
    assert torch.allclose(cl._p._gradient.float(), 2 * g1.float(), atol=2e-2, rtol=2e-2)


def test_embedding_module():
    m = cpu_manager()
    emb = torch.nn.Embedding(50, 16, padding_idx=0).to(torch.bfloat16)
    ce = neuzip.nn.Embedding(m, emb)
    idx = torch.tensor([[1, 2, 0], [49, 3, 3]])
    assert torch.equal(ce(idx), emb(idx))
    assert ce.extra_repr().startswith("! num_embeddings=50")


class Tiny(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.embed = torch.nn.Embedding(20, 8)
        self.block = torch.nn.Sequential(torch.nn.Linear(8, 16, bias=False), torch.nn.ReLU(),
                                         torch.nn.Linear(16, 8))
        self.norm = torch.nn.LayerNorm(8)
        self.lm_head = torch.nn.Linear(8, 20, bias=False)
        self.my_lm_head_extra = torch.nn.Sequential(torch.nn.Linear(8, 8))

    def forward(self, ids):
        return self.lm_head(self.norm(self.block(self.embed(ids))))


def test_convert_rules():
    torch.manual_seed(0)
    model = Tiny().to(torch.bfloat16)
    ids = torch.randint(0, 20, (2, 5))
    before = model(ids)
    m = cpu_manager()
    old_first = model.block[0]
    same = m.convert(model)
    assert same is model
    assert isinstance(model.block[0], neuzip.nn.Linear) and isinstance(model.block[2], neuzip.nn.Linear)
    assert model.block[2].bias is not None and model.block[0].bias is None
    assert isinstance(model.lm_head, torch.nn.Linear)                  # name contains lm_head
    assert isinstance(model.my_lm_head_extra[0], torch.nn.Linear)      # not descended into
    assert isinstance(model.embed, torch.nn.Embedding)
    assert old_first.weight is None                                     # old parameters dropped
    assert list(m.meta_dict) == ["0", "1"]
    assert torch.equal(model(ids), before)                              # lossless
    # zero-size placeholders show up as parameters, values do not
    names = dict(model.named_parameters())
    assert names["block.0._p"].numel() == 0


def test_unroll_convert_also_takes_embeddings():
    from neuzip.utils import _unroll_convert
    model = Tiny().to(torch.bfloat16)
    m = cpu_manager()
    _unroll_convert(m, model)
    assert isinstance(model.embed, neuzip.nn.Embedding)
    assert isinstance(model.lm_head, neuzip.nn.Linear)


def test_compressed_lomo_hook_updates_and_recompresses():
    torch.manual_seed(1)
    m = cpu_manager()
    lin = torch.nn.Linear(16, 16, bias=False).to(torch.bfloat16)
    w0 = lin.weight.data.clone()
    cl = neuzip.nn.Linear(m, lin)

    class Sched:
        def get_last_lr(self):
            return [0.5]

    sched = Sched()
    cl._p.register_post_accumulate_grad_hook(lambda p: neuzip.compressed_lomo_hook(sched, p))
    x = torch.randn(4, 16, dtype=torch.bfloat16)
    y = cl(x)
    g = torch.randn_like(y)
    y.backward(g)
    expect = w0.clone()
    expect.add_(torch.mm(g.t(), x), alpha=-0.5)
    assert cl._p._gradient is None
    assert torch.equal(cl._p(), expect)
    # plain hook
    p = torch.nn.Parameter(torch.ones(3))
    p.grad = torch.full((3,), 2.0)
    neuzip.lomo_hook(sched, p)
    assert torch.equal(p.data, torch.zeros(3)) and p.grad is None


def test_autocast_inputs_are_cast_by_hand():
    m = cpu_manager()
    lin = torch.nn.Linear(8, 8, bias=False).to(torch.bfloat16)
    cl = neuzip.nn.Linear(m, lin)
    x = torch.randn(2, 8, dtype=torch.bfloat16, requires_grad=True)
    y = cl(x)
    assert y.dtype == torch.bfloat16
    y.sum().backward()
    assert x.grad.dtype == torch.bfloat16


def test_dummy_backend_api():
    be = neuzip.binding.DummyBackend()
    for meth in ("write", "read", "size", "linear", "linear_without_bias"):
        assert callable(getattr(be, meth))


def test_state_dict_round_trip_keeps_the_compressed_weights(tmp_path):
    torch.manual_seed(3)
    src = Tiny().to(torch.bfloat16)
    ids = torch.randint(0, 20, (2, 5))
    expect = src(ids)
    m1 = cpu_manager()
    m1.convert(src)
    sd = src.state_dict()
    assert "block.0._extra_state" in sd and sd["block.0._p"].numel() == 0
    assert sd["block.0._extra_state"]["container"].dtype == torch.uint8
    path = tmp_path / "ckpt.pt"
    torch.save(sd, path)
    # a fresh model with different weights, converted, then loaded from the checkpoint
    torch.manual_seed(4)
    dst = Tiny().to(torch.bfloat16)
    m2 = cpu_manager()
    m2.convert(dst)
    assert not torch.equal(dst(ids), expect)
    dst.load_state_dict(torch.load(path, weights_only=False))
    assert torch.equal(dst(ids), expect)


class TwoBlocks(torch.nn.Module):
    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a = torch.nn.Linear(16, 16, bias=False)
            self.b = torch.nn.Linear(16, 16, bias=True)

        def forward(self, x):
            return self.b(torch.relu(self.a(x)))

    def __init__(self):
        super().__init__()
        self.blocks = torch.nn.ModuleList([TwoBlocks.Block(), TwoBlocks.Block()])

    def forward(self, x):
        for blk in self.blocks:
            x = blk(x)
        return x


def test_layerwise_hooks_stage_one_block_at_a_time_on_cpu():
    """Host logic of neuzip_b200.layerwise with the CPU stand-in backend: a block's
    weights are staged while it runs and only then; results match the per-Linear path."""
    from neuzip_b200 import layerwise
    torch.manual_seed(0)
    model = TwoBlocks().to(torch.bfloat16)
    m = cpu_manager()
    m.convert(model)
    x = torch.randn(3, 16).to(torch.bfloat16)
    with torch.no_grad():
        ref = model(x)
    hooks = layerwise.attach(model, m)
    assert len(hooks) == 4
    seen = []
    for i, blk in enumerate(model.blocks):
        blk.a.register_forward_pre_hook(
            lambda mod, args, i=i: seen.append([b.a._p.staged() is not None for b in model.blocks]))
    with torch.no_grad():
        got = model(x)
    assert torch.equal(got, ref)
    assert seen == [[True, False], [False, True]]
    assert all(b.a._p.staged() is None for b in model.blocks)      # nothing stays staged
    # training through the hooks: gradients land in _gradient as without them
    model(x).float().sum().backward()
    assert all(b.a._p._gradient is not None for b in model.blocks)
    for h in hooks:
        h.remove()
    with torch.no_grad():
        assert torch.equal(model(x), ref)


def test_layerwise_exclude_leaves_a_linear_to_decode_on_its_own():
    """attach(exclude=...) keeps the named Linears out of the per-block decode (they are never
    staged and decode themselves, e.g. through a fused kernel); results are unchanged."""
    from neuzip_b200 import layerwise
    torch.manual_seed(0)
    model = TwoBlocks().to(torch.bfloat16)
    m = cpu_manager()
    m.convert(model)
    x = torch.randn(3, 16).to(torch.bfloat16)
    with torch.no_grad():
        ref = model(x)
    layerwise.attach(model, m, exclude=lambda lin: any(lin is blk.b for blk in model.blocks))
    seen = []
    for blk in model.blocks:
        blk.b.register_forward_pre_hook(
            lambda mod, args, blk=blk: seen.append((blk.a._p.staged() is not None,
                                                     blk.b._p.staged() is not None)))
    with torch.no_grad():
        assert torch.equal(model(x), ref)
    assert seen == [(True, False), (True, False)]


def test_layerwise_hooks_follow_writes_and_loaded_state_on_cpu():
    """A handle that is written again after attach() (an optimiser step, a loaded
    checkpoint) must be decoded from its new bytes by the block's batched decode."""
    from neuzip_b200 import layerwise
    torch.manual_seed(1)
    model = TwoBlocks().to(torch.bfloat16)
    m = cpu_manager()
    m.convert(model)
    x = torch.randn(3, 16).to(torch.bfloat16)
    saved = {k: v for k, v in model.state_dict().items()}
    hooks = layerwise.attach(model, m)
    with torch.no_grad():
        first = model(x)
    # in-backward style update of every compressed weight: read -> change -> write
    for blk in model.blocks:
        for lin in (blk.a, blk.b):
            w = lin._p()
            m.write((w.float() * 1.5).to(torch.bfloat16), lin._p._handle)
    with torch.no_grad():
        hooked = model(x)
    for h in hooks:
        h.remove()
    with torch.no_grad():
        plain = model(x)
    assert torch.equal(hooked, plain) and not torch.equal(hooked, first)
    hooks = layerwise.attach(model, m)
    model.load_state_dict(saved)
    with torch.no_grad():
        assert torch.equal(model(x), first)
    for h in hooks:
        h.remove()


def test_checkpoint_of_a_converted_model_loads_into_a_meta_model_without_compressing(tmp_path):
    """A converted model's checkpoint loads into a model that was never materialised:
    the skeleton lives on the meta device, compressed Linears are built from the stored
    bytes, and the backend is never asked to compress anything."""
    torch.manual_seed(5)
    src = Tiny().to(torch.bfloat16)
    ids = torch.randint(0, 20, (2, 5))
    m1 = cpu_manager()
    m1.convert(src)
    expect = src(ids)
    path = tmp_path / "converted.pt"
    torch.save(src.state_dict(), path)

    with torch.device("meta"):
        skeleton = Tiny().to(torch.bfloat16)
    m2 = cpu_manager()
    writes = []
    real_write = m2._be.write
    m2._be.write = lambda *a, **k: (writes.append(a[0]), real_write(*a, **k))[1]
    m2.load_converted(skeleton, torch.load(path, weights_only=False), device="cpu")
    assert not writes                                   # nothing was compressed
    assert all(not p.is_meta for p in skeleton.parameters())
    assert isinstance(skeleton.block[0], neuzip.nn.Linear)
    assert torch.equal(skeleton(ids), expect)
    # and it saves again to the same bytes
    again = skeleton.state_dict()
    first = src.state_dict()
    assert torch.equal(again["block.0._extra_state"]["container"],
                       first["block.0._extra_state"]["container"])
