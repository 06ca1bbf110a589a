"""Public API behaviour: context manager rules, module reconstruction, calling convention,
input validation, the one-call API, init_weights on sharded modules."""
import pytest
import torch
import torch.nn as nn
from torch.distributed.tensor import DTensor
from torch.distributed.tensor.placement_types import Replicate, Shard

from autoparallel_b200 import AutoParallel, ForwardInputs, auto_parallel


class Inner(nn.Module):
    def __init__(self, d):
        super().__init__()
        self.lin = nn.Linear(d, d)

    def forward(self, x):
        return torch.relu(self.lin(x))


class Model(nn.Module):
    CLASS_ATTR = "kept"

    def __init__(self, d=64):
        super().__init__()
        self.d = d
        self.blocks = nn.ModuleDict({"a": Inner(d), "b": Inner(d)})
        self.head = nn.Linear(d, d, bias=False)
        self.tied = self.head  # aliased sub-module
        self.unused = nn.Parameter(torch.zeros(d))
        self.register_buffer("scale", torch.ones(d), persistent=False)
        self.note = {"user": "attribute"}

    @property
    def width(self):
        return self.d

    def helper(self):
        return "method"

    def forward(self, x, bias=None):
        for blk in self.blocks.values():
            x = blk(x)
        y = self.head(x) * self.scale
        return y if bias is None else y + bias

    def init_weights(self):
        for m in self.modules():
            if isinstance(m, nn.Linear):
                nn.init.normal_(m.weight, std=0.02)
                if m.bias is not None:
                    nn.init.zeros_(m.bias)
        self.unused = nn.Parameter(torch.full((self.d,), 3.0))  # assignment of a full tensor
        self.scale = torch.full((self.d,), 2.0)


def _build(mesh, **kw):
    with torch.device("meta"):
        m = Model()
    with AutoParallel(m, lambda: torch.randn(16, 8, 64), mesh, **kw) as ap:
        ap.add_parameter_memory_constraint()
        ap.add_input_constraints([(Shard(0),)])
        ap.add_output_constraints([(Shard(0),)])
        ap.optimize_placement()
        return ap, ap.apply_placement()


def test_context_manager_rules(mesh_1d):
    with torch.device("meta"):
        m = Model()
    ap = AutoParallel(m, lambda: torch.randn(16, 8, 64), mesh_1d)
    with pytest.raises(RuntimeError, match="context manager"):
        ap.add_parameter_memory_constraint()
    with ap:
        ap.add_input_constraints([(Shard(0),)])
        with pytest.raises(AssertionError):
            ap.add_input_constraints([(Shard(0),)])
    with pytest.raises(RuntimeError, match="re-entrant|exited"):
        ap.optimize_placement()


def test_model_must_be_on_meta(mesh_1d):
    with pytest.raises(AssertionError, match="meta"):
        AutoParallel(Model(), lambda: torch.randn(16, 8, 64), mesh_1d)


def test_failure_in_enter_unwinds(mesh_1d):
    with torch.device("meta"):
        m = Model()

    def bad_input():
        raise ValueError("boom")

    with pytest.raises(ValueError, match="boom"):
        with AutoParallel(m, bad_input, mesh_1d):
            pass
    # a fresh context works afterwards (fake mode / mesh context were unwound)
    _build(mesh_1d)


def test_parallel_module_is_users_class_with_dtensor_state(mesh_1d):
    ap, pm = _build(mesh_1d)
    assert isinstance(pm, Model) and pm.CLASS_ATTR == "kept" and pm.width == 64 and pm.helper() == "method"
    assert pm.note == {"user": "attribute"}
    assert isinstance(pm.blocks, nn.ModuleDict) and set(pm.blocks) == {"a", "b"}
    assert pm.tied is pm.head  # module alias preserved
    names = dict(pm.named_parameters())
    assert "unused" in names  # parameters forward never reads are still there
    for p in pm.parameters():
        assert isinstance(p, DTensor) and p.device.type == "meta"
    assert "scale" in dict(pm.named_buffers()) and "scale" not in pm.state_dict()  # non-persistent stays non-persistent


def test_init_weights_and_local_calling_convention(mesh_1d):
    ap, pm = _build(mesh_1d)
    pm.to_empty(device="cpu")
    pm.init_weights()
    assert torch.all(pm.unused.full_tensor() == 3.0)
    assert torch.all(pm.scale.full_tensor() == 2.0)
    x = torch.randn(2, 8, 64)  # local shard of the batch-16 input on 8 ranks
    y = pm(x)
    assert not isinstance(y, DTensor) and y.shape == (2, 8, 64)
    y.sum().backward()
    assert pm.head.weight.grad is not None
    with torch.no_grad():
        y2 = pm(x)
    assert y2.shape == y.shape and not y2.requires_grad  # (values are compared on real process groups elsewhere)
    with pytest.raises(ValueError, match="local shape"):
        pm(torch.randn(16, 8, 64))
    with pytest.raises(TypeError, match="dtype"):
        pm(x.double())
    with pytest.raises(ValueError, match="inputs"):
        pm(x, x)


def test_kwargs_any_order_and_pytree_inputs(mesh_1d):
    with torch.device("meta"):
        m = Model()

    def input_fn():
        return ForwardInputs((torch.randn(16, 8, 64),), {"bias": torch.randn(64)})

    with AutoParallel(m, input_fn, mesh_1d) as ap:
        ap.add_input_constraints([(Shard(0),), (Replicate(),)])
        ap.add_output_constraints([(Shard(0),)])
        ap.optimize_placement()
        pm = ap.apply_placement()
    pm.to_empty(device="cpu")
    pm.init_weights()
    out = pm(torch.randn(2, 8, 64), bias=torch.zeros(64))
    assert out.shape == (2, 8, 64)
    with pytest.raises(TypeError, match="unexpected keyword"):
        pm(torch.randn(2, 8, 64), other=torch.zeros(64))


def test_auto_parallel_one_call_api(mesh_1d):
    with torch.device("meta"):
        m = Model()
    pm = auto_parallel(m, mesh_1d, torch.randn(16, 8, 64), out_shardings=(Shard(0),))
    assert isinstance(pm, Model)
    assert pm._apb200_lowered.output_placements == [(Shard(0),)]
    assert pm._apb200_lowered.input_placements[0] == (Replicate(),)  # plain sample tensors are taken as replicated
