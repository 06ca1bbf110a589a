"""Buffers that the forward mutates in place (batch-norm statistics, step counters): the joint graph returns their
new values, the solver keeps them in the buffer's placement, and the parallel module writes them back after
every forward.  (The reference's MoE model does the same with ``tokens_per_expert.add_``,
examples/../dsv3.py:1006-1008.)"""
import os

import torch
from conftest import free_port
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn
from torch.distributed.tensor.placement_types import Shard


class Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.l1 = nn.Linear(16, 32)
        self.bn = nn.BatchNorm1d(32)
        self.l2 = nn.Linear(32, 8)
        self.register_buffer("steps", torch.zeros(()))

    def forward(self, x):
        self.steps.add_(1.0)
        return self.l2(torch.relu(self.bn(self.l1(x))))


def test_joint_graph_lists_the_mutated_buffers(mesh_1d):
    from autoparallel_b200 import AutoParallel

    with torch.device("meta"):
        model = Net()
    with AutoParallel(model, lambda: torch.randn(16, 16), mesh_1d) as ap:
        j = ap.joint
        assert set(j.buffer_updates) == {"steps", "bn.running_mean", "bn.running_var", "bn.num_batches_tracked"}
        assert j.num_user_outputs == 1 and len(j.fwd_outputs) == 1 + len(j.buffer_updates)
        ap.add_input_constraints([(Shard(0),)])
        ap.add_output_constraints([(Shard(0),)])  # one constraint: the new buffer values are not user outputs
        sol = ap.optimize_placement()
        for fqn, new in j.buffer_updates.items():
            assert tuple(sol[new].output_spec.placements) == tuple(sol[j.buffer_nodes[fqn]].output_spec.placements)


def _worker(rank, ws, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(ws))
    dist.init_process_group("gloo", rank=rank, world_size=ws)
    from torch.distributed.device_mesh import init_device_mesh

    from autoparallel_b200 import AutoParallel
    from autoparallel_b200.parallel.lower.init_weights import _distribute

    torch.manual_seed(0)
    ref = Net()
    with torch.device("meta"):
        model = Net()
    mesh = init_device_mesh("cpu", (ws,), mesh_dim_names=("dp",))
    with AutoParallel(model, lambda: torch.randn(8, 16), mesh) as ap:
        ap.add_input_constraints([(Shard(0),)])
        ap.add_output_constraints([(Shard(0),)])
        ap.optimize_placement()
        pm = ap.apply_placement()
    pm.to_empty(device="cpu")
    state = dict(ref.named_parameters())
    state.update(dict(ref.named_buffers()))
    with torch.no_grad():
        for n, t in list(pm.named_parameters()) + list(pm.named_buffers()):
            t._local_tensor.copy_(_distribute(state[n].detach().clone(), mesh, t.placements)._local_tensor)
    torch.manual_seed(1)
    for _ in range(2):  # training steps: statistics move twice
        x = torch.randn(8, 16)
        y = pm(x.chunk(ws, 0)[rank])
        y.sum().backward()
        yr = ref(x)
        yr.sum().backward()
    with torch.no_grad():  # the forward-only graph updates them too
        x = torch.randn(8, 16)
        pm(x.chunk(ws, 0)[rank])
        ref(x)
    res = {
        "out": (y - yr.chunk(ws, 0)[rank]).abs().max().item(),
        "mean": (pm.bn.running_mean.full_tensor() - ref.bn.running_mean).abs().max().item(),
        "var": (pm.bn.running_var.full_tensor() - ref.bn.running_var).abs().max().item(),
        "steps": pm.steps.full_tensor().item(),
        "tracked": pm.bn.num_batches_tracked.full_tensor().item(),
        "grad": max((p.grad.full_tensor() - state[n].grad).abs().max().item() for n, p in pm.named_parameters()),
    }
    if rank == 0:
        q.put(res)
    dist.destroy_process_group()


def test_statistics_and_counters_follow_the_single_device_run_on_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    mp.spawn(_worker, args=(2, free_port(), q), nprocs=2, join=True)
    res = q.get()
    assert res["out"] < 1e-5 and res["mean"] < 1e-6 and res["var"] < 1e-6 and res["grad"] < 1e-4, res
    assert res["steps"] == 3.0 and res["tracked"] == 3
