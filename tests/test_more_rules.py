"""Sharding rules for operators that otherwise run replicated or could not be planned: ``max`` / ``min`` over a dim (two
outputs), ``flip``, prefix scans, group norm, average pooling, logical reductions.  Each is pinned to a batch split and the
parallel module is compared with the single-device model on two gloo ranks; a scalar ``.sum()`` must not stall planning."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn
import torch.nn.functional as F
from conftest import free_port
from torch.distributed.tensor.placement_types import Shard

aten = torch.ops.aten


class Zoo(nn.Module):
    def __init__(self):
        super().__init__()
        self.lin = nn.Linear(16, 16)
        self.gn = nn.GroupNorm(2, 4)

    def forward(self, x):                       # x [B, 16]
        y = self.lin(x)
        mx, arg = y.max(dim=-1)                 # two outputs
        mn = y.min(dim=1, keepdim=True)[0]
        sc = y.cumsum(-1) + y.flip(-1) + (y * 0.1 + 1.0).cumprod(-1)
        img = y.view(-1, 4, 2, 2)
        g = self.gn(img)
        pooled = F.avg_pool2d(g, 2).flatten(1) + F.adaptive_avg_pool2d(img, 1).flatten(1)   # [B, 4]
        flag = (y > 0).any(dim=-1).to(y.dtype) + (y > -10).all(dim=1).to(y.dtype)
        out = sc.sum(-1) + mx + mn.squeeze(1) + pooled.sum(-1) + flag + arg.to(y.dtype) * 0.0
        return out                              # [B]


PINNED = (aten.max.dim, aten.min.dim, aten.flip.default, aten.cumsum.default, aten.cumprod.default, aten.native_group_norm.default,
          aten.avg_pool2d.default, aten._adaptive_avg_pool2d.default, aten.any.dim, aten.any.dims, aten.all.dim, aten.all.dims)


def _worker(rank, ws, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(ws))
    dist.init_process_group("gloo", rank=rank, world_size=ws)
    from torch.distributed.device_mesh import init_device_mesh

    from autoparallel_b200 import AutoParallel
    from autoparallel_b200.parallel.lower.init_weights import _distribute

    torch.manual_seed(0)
    ref = Zoo()
    with torch.device("meta"):
        m = Zoo()
    mesh = init_device_mesh("cpu", (ws,), mesh_dim_names=("dp",))
    with AutoParallel(m, lambda: torch.randn(8, 16), mesh) as ap:
        ap.add_input_constraints([(Shard(0),)])
        ap.add_output_constraints([(Shard(0),)])
        pinned = set()
        for n in ap.joint.gm.graph.nodes:
            if n.op == "call_function" and n.target in PINNED and not n.meta.get("autograd_backward"):
                v = n.meta["val"]
                v0 = v[0] if isinstance(v, (tuple, list)) else v
                if v0.ndim >= 1 and v0.shape[0] == 8:
                    ap.sharding_optimizer.add_node_constraint(n, (Shard(0),))  # (of a multi-output node: its first output)
                    pinned.add(str(n.target))
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
    w = torch.linspace(-1, 1, 8)
    y = pm(x.chunk(ws, 0)[rank])
    (y * w.chunk(ws)[rank]).sum().backward()
    yr = ref(x)
    (yr * w).sum().backward()
    err = (y - yr.chunk(ws, 0)[rank]).abs().max().item()
    g = max((p.grad.full_tensor() - state[n].grad).abs().max().item() for n, p in pm.named_parameters())
    if rank == 0:
        q.put((sorted(pinned), err, g))
    dist.destroy_process_group()


def test_batch_split_through_less_common_operators_on_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    mp.spawn(_worker, args=(2, free_port(), q), nprocs=2, join=True)
    pinned, err, grad = q.get()
    assert len(pinned) >= 8, pinned
    assert err < 1e-5 and grad < 1e-5


def test_sum_of_a_scalar_does_not_stall_planning(mesh_1d):
    """``loss.sum()`` on a 0-d tensor traces to a reduction over an empty dim list of a tensor without dims; the graph
    clean-up must leave it alone instead of rewriting it for ever."""
    from autoparallel_b200 import AutoParallel

    class M(nn.Module):
        def __init__(self):
            super().__init__()
            self.l = nn.Linear(16, 16)

        def forward(self, x):
            return F.mse_loss(self.l(x), torch.zeros(x.shape[0], 16)).sum()

    with torch.device("meta"):
        m = M()
    with AutoParallel(m, lambda: torch.randn(64, 16), mesh_1d) as ap:
        ap.add_input_constraints([(Shard(0),)])
        ap.optimize_placement()
        assert ap.lower() is not None


class Zoo2(nn.Module):
    def __init__(self):
        super().__init__()
        self.lin = nn.Linear(16, 16)

    def forward(self, x):                       # x [B, 16]
        y = self.lin(x)
        a = F.hardtanh(y) + F.leaky_relu(y, 0.1) + F.elu(y) + F.softplus(y) + F.hardswish(y) + F.mish(y)
        var, mean = torch.var_mean(y, dim=-1)
        sd = y.std(dim=1)
        med = y.median(dim=-1)[0] + y.kthvalue(3, dim=-1)[0]
        pos = torch.searchsorted(y.detach().sort(-1)[0], y.detach()).to(y.dtype).sum(-1)
        m = y.view(-1, 4, 4)
        dist_ = torch.cdist(m, m + 1.0).sum((1, 2))
        diag = m.diagonal(dim1=1, dim2=2).sum(-1)
        return a.sum(-1) + var + mean + sd + med + pos * 0.0 + dist_ + diag


PINNED2 = (aten.hardtanh.default, aten.leaky_relu.default, aten.elu.default, aten.softplus.default, aten.hardswish.default,
           aten.mish.default, aten.var_mean.correction, aten.std.correction, aten.median.dim, aten.kthvalue.default,
           aten.searchsorted.Tensor, aten._cdist_forward.default, aten.diagonal_scatter.default, aten._cdist_backward.default,
           aten.hardtanh_backward.default, aten.leaky_relu_backward.default, aten.elu_backward.default)


def _worker2(rank, ws, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(ws))
    dist.init_process_group("gloo", rank=rank, world_size=ws)
    from torch.distributed.device_mesh import init_device_mesh

    from autoparallel_b200 import AutoParallel
    from autoparallel_b200.parallel.lower.init_weights import _distribute

    torch.manual_seed(0)
    ref = Zoo2()
    with torch.device("meta"):
        m = Zoo2()
    mesh = init_device_mesh("cpu", (ws,), mesh_dim_names=("dp",))
    with AutoParallel(m, lambda: torch.randn(8, 16), mesh) as ap:
        ap.add_input_constraints([(Shard(0),)])
        ap.add_output_constraints([(Shard(0),)])
        pinned = set()
        for n in ap.joint.gm.graph.nodes:
            if n.op == "call_function" and n.target in PINNED2:
                v = n.meta["val"]
                v0 = v[0] if isinstance(v, (tuple, list)) else v
                if v0.ndim >= 1 and v0.shape[0] == 8:
                    ap.sharding_optimizer.add_node_constraint(n, (Shard(0),))
                    pinned.add(str(n.target))
        ap.optimize_placement()
        pm = ap.apply_placement()
    pm.to_empty(device="cpu")
    state = dict(ref.named_parameters())
    with torch.no_grad():
        for n, t in pm.named_parameters():
            t._local_tensor.copy_(_distribute(state[n].detach().clone(), mesh, t.placements)._local_tensor)
    torch.manual_seed(1)
    x = torch.randn(8, 16)
    w = torch.linspace(-1, 1, 8)
    y = pm(x.chunk(ws, 0)[rank])
    (y * w.chunk(ws)[rank]).sum().backward()
    yr = ref(x)
    (yr * w).sum().backward()
    err = (y - yr.chunk(ws, 0)[rank]).abs().max().item()
    g = max((p.grad.full_tensor() - state[n].grad).abs().max().item() for n, p in pm.named_parameters())
    if rank == 0:
        q.put((sorted(pinned), err, g))
    dist.destroy_process_group()


def test_batch_split_through_activations_statistics_and_distances_on_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    mp.spawn(_worker2, args=(2, free_port(), q), nprocs=2, join=True)
    pinned, err, grad = q.get()
    assert len(pinned) >= 10, pinned
    assert err < 1e-4 and grad < 1e-4


class Zoo3(nn.Module):
    def __init__(self):
        super().__init__()
        self.conv = nn.Conv2d(2, 4, 3, padding=1)
        self.gru = nn.GRU(16, 8, batch_first=True)
        self.lstm = nn.LSTM(16, 8, batch_first=True)

    def forward(self, x):                                   # x [B, 2, 4, 4]
        y = self.conv(x)                                    # [B, 4, 4, 4]
        p = F.adaptive_max_pool2d(y, 2).flatten(1).sum(-1)
        v = F.avg_pool3d(y.unsqueeze(1), 2).flatten(1).sum(-1)
        grid = torch.zeros(x.shape[0], 3, 3, 2) + 0.25
        s = F.grid_sample(y, grid, align_corners=False).flatten(1).sum(-1)
        f = torch.fft.rfft(y.flatten(2), dim=-1).abs().flatten(1).sum(-1)
        seq, _ = self.gru(y.flatten(2))                     # [B, 4, 8]
        seq2, _ = self.lstm(y.flatten(2))                   # traced into per-step operators (no fused CPU-only operator)
        return p + v + s + f + seq.sum((1, 2)) + seq2.sum((1, 2))


PINNED3 = (aten.adaptive_max_pool2d.default, aten.avg_pool3d.default, aten.grid_sampler_2d.default, aten._fft_r2c.default,
           aten.adaptive_max_pool2d_backward.default, aten.avg_pool3d_backward.default, aten.grid_sampler_2d_backward.default)


def _worker3(rank, ws, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(ws))
    dist.init_process_group("gloo", rank=rank, world_size=ws)
    from torch.distributed.device_mesh import init_device_mesh

    from autoparallel_b200 import AutoParallel
    from autoparallel_b200.parallel.lower.init_weights import _distribute

    torch.manual_seed(0)
    ref = Zoo3()
    with torch.device("meta"):
        m = Zoo3()
    mesh = init_device_mesh("cpu", (ws,), mesh_dim_names=("dp",))
    with AutoParallel(m, lambda: torch.randn(8, 2, 4, 4), mesh) as ap:
        ap.add_input_constraints([(Shard(0),)])
        ap.add_output_constraints([(Shard(0),)])
        pinned = set()
        for n in ap.joint.gm.graph.nodes:
            if n.op == "call_function" and n.target in PINNED3:
                v = n.meta["val"]
                v0 = next(t for t in (v if isinstance(v, (tuple, list)) else [v]) if isinstance(t, torch.Tensor))
                if v0.ndim >= 1 and v0.shape[0] == 8:
                    ap.sharding_optimizer.add_node_constraint(n, (Shard(0),))
                    pinned.add(str(n.target))
        ap.optimize_placement()
        pm = ap.apply_placement()
    pm.to_empty(device="cpu")
    state = dict(ref.named_parameters())
    with torch.no_grad():
        for n, t in pm.named_parameters():
            t._local_tensor.copy_(_distribute(state[n].detach().clone(), mesh, t.placements)._local_tensor)
    torch.manual_seed(1)
    x = torch.randn(8, 2, 4, 4)
    w = torch.linspace(-1, 1, 8)
    y = pm(x.chunk(ws, 0)[rank])
    (y * w.chunk(ws)[rank]).sum().backward()
    yr = ref(x)
    (yr * w).sum().backward()
    err = (y - yr.chunk(ws, 0)[rank]).abs().max().item()
    g = max((p.grad.full_tensor() - state[n].grad).abs().max().item() for n, p in pm.named_parameters())
    if rank == 0:
        q.put((sorted(pinned), err, g))
    dist.destroy_process_group()


def test_batch_split_through_pooling_sampling_fft_a_gru_and_an_lstm_on_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    mp.spawn(_worker3, args=(2, free_port(), q), nprocs=2, join=True)
    pinned, err, grad = q.get()
    assert len(pinned) >= 4, pinned
    assert err < 1e-4 and grad < 1e-4


class Extremes(nn.Module):
    def __init__(self):
        super().__init__()
        self.lin = nn.Linear(16, 16)

    def forward(self, x):
        y = self.lin(x)                      # [B, 16], batch sharded
        spread = y.amax(dim=0) - y.amin(dim=0)   # extremes over the sharded dim
        return y / (spread + 1.0)


def _extremes_worker(rank, ws, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(ws))
    dist.init_process_group("gloo", rank=rank, world_size=ws)
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor.placement_types import Partial

    from autoparallel_b200 import AutoParallel
    from autoparallel_b200.parallel.lower.init_weights import _distribute
    from autoparallel_b200.runtime import comm_ops

    torch.manual_seed(0)
    ref = Extremes()
    with torch.device("meta"):
        m = Extremes()
    mesh = init_device_mesh("cpu", (ws,), mesh_dim_names=("dp",))
    with AutoParallel(m, lambda: torch.randn(8, 16), mesh) as ap:
        ap.add_input_constraints([(Shard(0),)])
        ap.add_output_constraints([(Shard(0),)])
        for n in ap.joint.gm.graph.nodes:
            if n.op == "call_function" and n.target is aten.amax.default:
                ap.sharding_optimizer.add_node_constraint(n, (Partial("max"),))
            if n.op == "call_function" and n.target is aten.amin.default:
                ap.sharding_optimizer.add_node_constraint(n, (Partial("min"),))
        ap.optimize_placement()
        pm = ap.apply_placement()
        n_op = sum(1 for n in ap.lowered.gm.graph.nodes if n.op == "call_function" and n.target is comm_ops.ops.all_reduce_op.default)
    pm.to_empty(device="cpu")
    state = dict(ref.named_parameters())
    with torch.no_grad():
        for n, t in pm.named_parameters():
            t._local_tensor.copy_(_distribute(state[n].detach().clone(), mesh, t.placements)._local_tensor)
    torch.manual_seed(1)
    x = torch.randn(8, 16)
    w = torch.linspace(-1, 1, 16)
    y = pm(x.chunk(ws, 0)[rank])
    (y * w).sum().backward()
    yr = ref(x)
    (yr * w).sum().backward()
    err = (y - yr.chunk(ws, 0)[rank]).abs().max().item()
    g = max((p.grad.full_tensor() - state[n].grad).abs().max().item() for n, p in pm.named_parameters())
    if rank == 0:
        q.put((n_op, err, g))
    dist.destroy_process_group()


def test_pending_maximum_and_minimum_are_completed_by_their_own_all_reduce():
    """``amax`` / ``amin`` over a sharded dim give ``Partial("max")`` / ``Partial("min")``; the lowering completes them with an
    all-reduce of that operator (a few elements) instead of gathering the operand."""
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    mp.spawn(_extremes_worker, args=(2, free_port(), q), nprocs=2, join=True)
    n_op, err, grad = q.get()
    assert n_op == 2 and err < 1e-6 and grad < 1e-5
