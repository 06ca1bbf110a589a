"""Convolution, batch-norm and pooling rules: numerics of a small CNN on two gloo ranks under the automatic plan
and with the convolutions pinned to output-channel / input-channel sharding."""
import os

import pytest
from conftest import free_port
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn
from torch.distributed.tensor.placement_types import Replicate, Shard


class CNN(nn.Module):
    def __init__(self):
        super().__init__()
        self.c1 = nn.Conv2d(3, 8, 3, padding=1)
        self.bn = nn.BatchNorm2d(8)
        self.pool = nn.MaxPool2d(2)
        self.c2 = nn.Conv2d(8, 16, 3, padding=1, bias=False)
        self.head = nn.Linear(16, 4)

    def forward(self, x):
        y = self.pool(torch.relu(self.bn(self.c1(x))))
        y = torch.relu(self.c2(y)).mean((2, 3))
        return self.head(y)


def test_rules_offer_batch_and_channel_splits(mesh_1d):
    from autoparallel_b200 import AutoParallel

    with torch.device("meta"):
        model = CNN()
    with AutoParallel(model, lambda: torch.randn(16, 3, 16, 16), mesh_1d) as ap:
        strats = ap.sharding_optimizer.strats
        by_op = {}
        for n in ap.joint.gm.graph.nodes:
            if n.op == "call_function" and n in strats:
                by_op.setdefault(str(n.target), []).append(n)
        conv1, conv2 = by_op["aten.convolution.default"]
        outs1 = {tuple(s.output_spec.placements) for s in strats[conv1].strategies}
        outs2 = {tuple(s.output_spec.placements) for s in strats[conv2].strategies}
        assert {(Replicate(),), (Shard(0),), (Shard(1),)} <= outs1
        assert not any(p[0].is_partial() for p in outs1), "a biased convolution must not produce partial sums"
        assert any(p[0].is_partial() for p in outs2)  # input channels split: partial sums, no bias to double-count
        assert not any(p[0].is_shard() and p[0].dim >= 2 for p in outs1 | outs2)  # never the spatial dims
        bn = by_op["aten._native_batch_norm_legit_functional.default"][0]
        firsts = {tuple(s.output_specs[0].placements) for s in strats[bn].strategies}
        assert firsts == {(Replicate(),), (Shard(1),)}  # training statistics: channels only


def _worker(rank, ws, how, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(ws))
    dist.init_process_group("gloo", rank=rank, world_size=ws)
    from torch.distributed.device_mesh import init_device_mesh

    from autoparallel_b200 import AutoParallel
    from autoparallel_b200.parallel.lower.init_weights import _distribute

    torch.manual_seed(0)
    ref = CNN()
    with torch.device("meta"):
        model = CNN()
    mesh = init_device_mesh("cpu", (ws,), mesh_dim_names=("dp",))
    with AutoParallel(model, lambda: torch.randn(4, 3, 8, 8), mesh) as ap:
        ap.add_input_constraints([(Shard(0),)])
        ap.add_output_constraints([(Shard(0),)])
        if how == "channels":
            opt, params = ap.sharding_optimizer, ap.joint.param_nodes
            opt.add_node_constraint(params["c1.weight"], (Shard(0),))  # output channels
            opt.add_node_constraint(params["c2.weight"], (Shard(1),))  # input channels
        ap.optimize_placement()
        pm = ap.apply_placement()
    pm.to_empty(device="cpu")
    state = dict(ref.named_parameters())
    state.update(dict(ref.named_buffers()))
    with torch.no_grad():
        for n, t in list(pm.named_parameters()) + list(pm.named_buffers()):
            t._local_tensor.copy_(_distribute(state[n].detach().clone(), mesh, t.placements)._local_tensor)
    torch.manual_seed(1)
    x = torch.randn(4, 3, 8, 8)
    w = torch.linspace(-1, 1, 4)
    y = pm(x.chunk(ws, 0)[rank])
    (y * w).sum().backward()
    yr = ref(x)
    (yr * w).sum().backward()
    res = {
        "out": (y - yr.chunk(ws, 0)[rank]).abs().max().item(),
        "grad": max((p.grad.full_tensor() - state[n].grad).abs().max().item() for n, p in pm.named_parameters()),
        "mean": (pm.bn.running_mean.full_tensor() - ref.bn.running_mean).abs().max().item(),
        "placements": {n: str(p.placements) for n, p in pm.named_parameters()},
    }
    if rank == 0:
        q.put(res)
    dist.destroy_process_group()


@pytest.mark.parametrize("how", ["auto", "channels"])
def test_cnn_matches_single_device_on_two_ranks(how):
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    mp.spawn(_worker, args=(2, how, free_port(), q), nprocs=2, join=True)
    res = q.get()
    assert res["out"] < 1e-5 and res["grad"] < 1e-5 and res["mean"] < 1e-6, res
    if how == "channels":
        assert "Shard(dim=0)" in res["placements"]["c1.weight"] and "Shard(dim=1)" in res["placements"]["c2.weight"]
