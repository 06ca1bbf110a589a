"""init_weights interception (both modes), tied parameters, buffer re-assignment and parameter shard layout."""
import pytest
import torch
import torch.nn as nn
from torch.distributed.tensor import DTensor
from torch.distributed.tensor.placement_types import Shard

from autoparallel_b200 import AutoParallel
from autoparallel_b200.parallel.lower.init_weights import wrap_init_weights


class Net(nn.Module):
    def __init__(self, v=64, d=32):
        super().__init__()
        self.emb = nn.Embedding(v, d)
        self.mid = nn.Linear(d, d)
        self.out = nn.Linear(d, v, bias=False)
        self.out.weight = self.emb.weight  # tied
        self.register_buffer("table", torch.zeros(v))

    def forward(self, t):
        return self.out(torch.relu(self.mid(self.emb(t)))) + self.table

    def init_weights(self, value=0.5):
        with torch.no_grad():
            nn.init.constant_(self.mid.weight, value)          # in-place initialiser
            self.mid.bias.copy_(torch.arange(32.0))            # copy_ from a plain tensor
            self.emb.weight = nn.Parameter(torch.arange(64.0 * 32).view(64, 32))   # slot re-assignment (tied slot)
            self.table = torch.arange(64.0)                    # buffer re-assignment
        return "done"


def _build(mesh):
    with torch.device("meta"):
        m = Net()
    with AutoParallel(m, lambda: torch.randint(0, 64, (16, 8)), mesh) as ap:
        ap.add_parameter_memory_constraint()
        ap.add_input_constraints([(Shard(0),)])
        ap.optimize_placement()
        pm = ap.apply_placement()
    pm.to_empty(device="cpu")
    return pm


@pytest.mark.parametrize("mode", ["materialize", "intercept"])
def test_init_weights_modes_give_the_same_sharded_values(mesh_1d, mode):
    pm = _build(mesh_1d)
    del pm.__dict__["init_weights"]
    wrap_init_weights(pm, mode=mode)
    assert pm.init_weights(value=0.25) == "done"  # arguments and the return value pass through
    assert isinstance(pm.mid.weight, DTensor) and isinstance(pm.table, DTensor)  # slots still hold the sharded tensors
    assert pm.out.weight is pm.emb.weight  # tie survives the re-assignment
    # fake ranks do not exchange data: check what rank 0 holds, the first shard of each global value
    def first_shard(dt, full):
        for i, pl in enumerate(dt.placements):
            if isinstance(pl, Shard):
                full = full.chunk(mesh_1d.shape[i], pl.dim)[0]
        return full

    assert torch.all(pm.mid.weight._local_tensor == 0.25)
    assert torch.equal(pm.mid.bias._local_tensor, first_shard(pm.mid.bias, torch.arange(32.0)))
    assert torch.equal(pm.emb.weight._local_tensor, first_shard(pm.emb.weight, torch.arange(64.0 * 32).view(64, 32)))
    assert torch.equal(pm.table._local_tensor, first_shard(pm.table, torch.arange(64.0)))
    assert pm.emb.weight.requires_grad
    assert any(isinstance(pl, Shard) for pl in pm.emb.weight.placements)  # the memory constraint shards it


def test_init_weights_shape_change_is_refused(mesh_1d):
    pm = _build(mesh_1d)

    def bad_init():
        pm.mid.weight = nn.Parameter(torch.zeros(3, 3))

    pm.__dict__["init_weights"] = None
    pm.init_weights = bad_init
    wrap_init_weights(pm, mode="materialize")
    with pytest.raises(RuntimeError, match="changed the shape"):
        pm.init_weights()
