"""index_put under the planner: dims behind the indexed rows can be split; numerics on two gloo ranks with the
operator pinned to that split (plain and accumulating forms)."""
import os

import torch
from conftest import free_port
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn
from torch.distributed.tensor.placement_types import Shard


class M(nn.Module):
    def __init__(s):
        super().__init__()
        s.l = nn.Linear(16, 16)
        s.register_buffer("perm", torch.tensor([3, 0, 2, 1, 7, 6, 5, 4]))

    def forward(s, x):
        y = s.l(x)                                   # [8, 16]
        buf = torch.zeros(8, 16).index_put((s.perm,), y)
        buf = buf.index_put((s.perm[:2],), y[:2] * 2.0, accumulate=True)
        return buf * 3.0


def _worker(rank, ws, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(ws))
    dist.init_process_group("gloo", rank=rank, world_size=ws)
    from torch.distributed.device_mesh import init_device_mesh
    from autoparallel_b200 import AutoParallel
    from autoparallel_b200.parallel.lower.init_weights import _distribute
    torch.manual_seed(0)
    ref = M()
    with torch.device("meta"):
        m = M()
    mesh = init_device_mesh("cpu", (ws,), mesh_dim_names=("dp",))
    with AutoParallel(m, lambda: torch.randn(8, 16), mesh) as ap:
        ap.add_input_constraints([(Shard(1),)])
        ap.add_output_constraints([(Shard(1),)])
        n_put = 0
        for n in ap.joint.gm.graph.nodes:
            if n.op == "call_function" and n.target is torch.ops.aten.index_put.default:
                ap.sharding_optimizer.add_node_constraint(n, (Shard(1),))
                n_put += 1
        ap.optimize_placement()
        pm = ap.apply_placement()
    pm.to_empty(device="cpu")
    state = dict(ref.named_parameters())
    state.update(dict(ref.named_buffers()))
    with torch.no_grad():
        for n, t in list(pm.named_parameters()) + list(pm.named_buffers()):
            t._local_tensor.copy_(_distribute(state[n].detach().clone(), mesh, t.placements)._local_tensor)
    torch.manual_seed(1)
    x = torch.randn(8, 16)
    w = torch.linspace(-1, 1, 16)
    y = pm(x.chunk(ws, 1)[rank])
    (y * w.chunk(ws)[rank]).sum().backward()
    yr = ref(x)
    (yr * w).sum().backward()
    err = (y - yr.chunk(ws, 1)[rank]).abs().max().item()
    g = max((p.grad.full_tensor() - state[n].grad).abs().max().item() for n, p in pm.named_parameters())
    if rank == 0:
        q.put((n_put, err, g))
    dist.destroy_process_group()


def test_index_put_split_behind_the_indexed_rows_on_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    mp.spawn(_worker, args=(2, free_port(), q), nprocs=2, join=True)
    pinned, err, grad = q.get()
    assert pinned == 2 and err < 1e-6 and grad < 1e-6


class Sel(nn.Module):
    def __init__(s):
        super().__init__()
        s.l = nn.Linear(16, 16)
        s.register_buffer("idx", torch.tensor([3, 0, 2, 1, 3, 3, 5, 4]))

    def forward(s, x):
        y = s.l(x)                                            # [8, 16]
        picked = y.index_select(0, s.idx)                     # rows re-ordered (with repeats)
        acc = torch.zeros(6, 16).index_add(0, s.idx, picked)  # and summed per target row
        return acc * 2.0


def _sel_worker(rank, ws, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(ws))
    dist.init_process_group("gloo", rank=rank, world_size=ws)
    from torch.distributed.device_mesh import init_device_mesh
    from autoparallel_b200 import AutoParallel
    from autoparallel_b200.parallel.lower.init_weights import _distribute
    torch.manual_seed(0)
    ref = Sel()
    with torch.device("meta"):
        m = Sel()
    mesh = init_device_mesh("cpu", (ws,), mesh_dim_names=("dp",))
    with AutoParallel(m, lambda: torch.randn(8, 16), mesh) as ap:
        ap.add_input_constraints([(Shard(1),)])
        ap.add_output_constraints([(Shard(1),)])
        pinned = 0
        for n in ap.joint.gm.graph.nodes:
            if n.op == "call_function" and n.target in (torch.ops.aten.index_select.default, torch.ops.aten.index_add.default):
                if n.meta["val"].ndim == 2 and n.meta["val"].shape[1] == 16:
                    ap.sharding_optimizer.add_node_constraint(n, (Shard(1),))
                    pinned += 1
        ap.optimize_placement()
        pm = ap.apply_placement()
    pm.to_empty(device="cpu")
    state = dict(ref.named_parameters())
    state.update(dict(ref.named_buffers()))
    with torch.no_grad():
        for n, t in list(pm.named_parameters()) + list(pm.named_buffers()):
            t._local_tensor.copy_(_distribute(state[n].detach().clone(), mesh, t.placements)._local_tensor)
    torch.manual_seed(1)
    x = torch.randn(8, 16)
    w = torch.linspace(-1, 1, 16)
    y = pm(x.chunk(ws, 1)[rank])
    (y * w.chunk(ws)[rank]).sum().backward()
    yr = ref(x)
    (yr * w).sum().backward()
    err = (y - yr.chunk(ws, 1)[rank]).abs().max().item()
    g = max((p.grad.full_tensor() - state[n].grad).abs().max().item() for n, p in pm.named_parameters())
    if rank == 0:
        q.put((pinned, err, g))
    dist.destroy_process_group()


def test_index_select_and_index_add_split_off_the_indexed_dim_on_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    mp.spawn(_sel_worker, args=(2, free_port(), q), nprocs=2, join=True)
    pinned, err, grad = q.get()
    assert pinned >= 2 and err < 1e-6 and grad < 1e-6
