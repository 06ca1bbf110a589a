"""Shards of unequal size (``uneven_sharding=True``): shard arithmetic, option filtering, and numerics on gloo
ranks with extents that the mesh does not divide, an empty shard included.
(Reference behaviour: autoparallel/shardings/propagation_rules.py:146-154, autoparallel/apply_sharding.py:372-386,
tests/test_dynamic_shapes.py.)"""
import os

import pytest
from conftest import free_port
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn
from torch.distributed.tensor.placement_types import Replicate, Shard


def test_shard_extents_follow_chunk_semantics():
    from autoparallel_b200.parallel.strategies.dtensor_adapter import is_even, local_shape_at, shard_extent

    for extent in (1, 5, 7, 8, 21):
        for parts in (2, 3, 4, 8):
            sizes = [shard_extent(extent, parts, i) for i in range(parts)]
            ref = [c.shape[0] for c in torch.arange(extent).chunk(parts)]
            assert sizes == ref + [0] * (parts - len(ref)), (extent, parts)
    assert local_shape_at([7, 10], (2, 2), (Shard(0), Shard(1)), (1, 0)) == [3, 5]
    assert local_shape_at([5, 10], (4,), (Shard(0),), (3,)) == [0, 10]
    assert is_even([8, 10], (2, 2), (Shard(0), Shard(0))) and not is_even([6, 10], (2, 2), (Shard(0), Shard(0)))


def test_options_with_uneven_shards(mesh_2d):
    from torch.distributed.tensor._dtensor_spec import DTensorSpec, TensorMeta

    from autoparallel_b200.parallel.strategies.dtensor_adapter import all_options, is_valid_spec

    val = torch.empty(7, 10)
    even = {tuple(s.output_spec.placements) for s in all_options(mesh_2d, val, True).strategies}
    uneven = {tuple(s.output_spec.placements) for s in all_options(mesh_2d, val, False).strategies}
    assert (Replicate(), Shard(0)) not in even and (Replicate(), Shard(0)) in uneven  # 7 rows over tp=4: 2, 2, 2, 1
    # 6 rows over tp=4 would be 2, 2, 2, 0: a shard is only offered while every rank holds part of it
    six = {tuple(s.output_spec.placements) for s in all_options(mesh_2d, torch.empty(6, 10), False).strategies}
    assert (Replicate(), Shard(0)) not in six and (Shard(0), Replicate()) in six
    assert (Shard(1), Shard(1)) not in uneven  # 10 columns over 2 x 4 ranks: nested and uneven
    tm = TensorMeta(torch.Size([16, 10]), (10, 1), torch.float32)
    assert is_valid_spec(DTensorSpec(mesh_2d, (Shard(0), Shard(0)), tensor_meta=tm), mesh_2d, False)  # nested but even


class _MLP(nn.Module):
    def __init__(self):
        super().__init__()
        self.a = nn.Linear(10, 21, bias=True)
        self.b = nn.Linear(21, 10, bias=False)
        self.n = nn.LayerNorm(10)

    def forward(self, x):
        return self.n(x + self.b(torch.relu(self.a(x))))


def _chunks(t, parts):
    out = list(torch.chunk(t, parts, 0))
    return out + [t[:0]] * (parts - len(out))


def _worker(rank, ws, mesh_shape, batch, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(ws))
    dist.init_process_group("gloo", rank=rank, world_size=ws)
    from torch.distributed.device_mesh import init_device_mesh

    from autoparallel_b200 import AutoParallel, ForwardInputs
    from autoparallel_b200.parallel.lower.init_weights import _distribute

    torch.manual_seed(0)
    ref = _MLP()
    with torch.device("meta"):
        model = _MLP()
    S = 5
    names = ("dp", "tp")[: len(mesh_shape)]
    mesh = init_device_mesh("cpu", mesh_shape, mesh_dim_names=names)
    rest = (Replicate(),) * (len(mesh_shape) - 1)
    with AutoParallel(model, lambda: ForwardInputs((torch.randn(batch, S, 10),), {}), mesh, uneven_sharding=True) as ap:
        ap.add_parameter_memory_constraint()
        ap.add_input_constraints([(Shard(0),) + rest])
        ap.add_output_constraints([(Shard(0),) + rest])
        ap.optimize_placement()
        pm = ap.apply_placement()
    pm.to_empty(device="cpu")
    ref_state = dict(ref.named_parameters())
    uneven_params = 0
    with torch.no_grad():
        for n, t in pm.named_parameters():
            t._local_tensor.copy_(_distribute(ref_state[n].detach(), mesh, t.placements)._local_tensor)
            for m, p in zip(mesh_shape, t.placements):
                if isinstance(p, Shard) and ref_state[n].shape[p.dim] % m:
                    uneven_params += 1
    dp = mesh_shape[0]
    me = mesh.get_coordinate()[0]
    torch.manual_seed(1)
    x = torch.randn(batch, S, 10)
    w = torch.linspace(-1, 1, 10)
    y = pm(_chunks(x, dp)[me])
    (y * w).sum().backward()
    y_ref = ref(x)
    (y_ref * w).sum().backward()
    mine = _chunks(y_ref, dp)[me]
    assert y.shape == mine.shape
    err = (y - mine).abs().max().item() if y.numel() else 0.0
    worst = 0.0
    for n, p in pm.named_parameters():
        g, rg = p.grad.full_tensor(), ref_state[n].grad
        worst = max(worst, ((g - rg).abs().max() / (rg.abs().max() + 1e-12)).item())
    errs = [None] * ws
    dist.all_gather_object(errs, (err, worst, uneven_params, tuple(y.shape)))
    if rank == 0:
        q.put(errs)
    dist.destroy_process_group()


@pytest.mark.parametrize(
    "mesh_shape,batch",
    [((3,), 7), ((4,), 7), ((2, 2), 3)],  # 7 rows over 3 ranks (3, 3, 1); over 4 (2, 2, 2, 1); 2-D mesh
)
def test_uneven_shards_match_single_device(mesh_shape, batch):
    ws = 1
    for m in mesh_shape:
        ws *= m
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    mp.spawn(_worker, args=(ws, mesh_shape, batch, free_port(), q), nprocs=ws, join=True)
    per_rank = q.get()
    assert all(e < 1e-5 and w < 1e-4 for e, w, _, _ in per_rank), per_rank
    assert sum(shape[0] for _, _, _, shape in per_rank) == batch * (ws // mesh_shape[0])
    assert per_rank[0][2] > 0, "the plan was expected to shard at least one parameter unevenly"


def _redistribute_worker(rank, ws, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(ws))
    dist.init_process_group("gloo", rank=rank, world_size=ws)
    import torch.fx as fx
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor._dtensor_spec import DTensorSpec, TensorMeta
    from torch.distributed.tensor.placement_types import Partial

    import autoparallel_b200.runtime.comm_ops  # noqa: F401  (registers the collective ops)
    from autoparallel_b200.parallel.lower.apply import _Redistributor
    from autoparallel_b200.parallel.strategies.dtensor_adapter import local_shape_at

    mesh = init_device_mesh("cpu", (ws,), mesh_dim_names=("dp",))
    full = torch.arange(7 * 5, dtype=torch.float32).reshape(7, 5)
    tm = TensorMeta(full.shape, full.stride(), full.dtype)

    def shard(pl):
        if isinstance(pl, Shard):
            return _chunks(full.movedim(pl.dim, 0), ws)[rank].movedim(0, pl.dim).contiguous()
        if isinstance(pl, Partial):
            return full * (rank + 1) / (ws * (ws + 1) / 2)  # the ranks' tensors sum to ``full``
        return full.clone()

    bad = []
    cases = [(Shard(0), Replicate()), (Shard(1), Replicate()), (Replicate(), Shard(0)), (Replicate(), Shard(1)),
             (Shard(0), Shard(1)), (Shard(1), Shard(0)), (Partial(), Shard(0)), (Partial(), Shard(1)), (Partial(), Replicate())]
    for src, dst in cases:
        g = fx.Graph()
        x = g.placeholder("x")
        local = shard(src)
        x.meta["val"] = local
        redis = _Redistributor(g, mesh)
        out = redis(x, x, DTensorSpec(mesh, (src,), tensor_meta=tm), DTensorSpec(mesh, (dst,), tensor_meta=tm))
        g.output(out)
        got = fx.GraphModule(torch.nn.Module(), g)(local)
        want = shard(dst)
        planned = list(out.meta["val"].shape)
        if list(got.shape) != list(want.shape) or planned != list(want.shape) or not torch.allclose(got, want, atol=1e-5):
            bad.append((str(src), str(dst), tuple(got.shape), tuple(want.shape), planned))
        assert planned == local_shape_at(list(full.shape), (ws,), (dst,), (rank,))
    res = [None] * ws
    dist.all_gather_object(res, bad)
    if rank == 0:
        q.put(res)
    dist.destroy_process_group()


def test_every_transition_between_uneven_shards_on_three_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    mp.spawn(_redistribute_worker, args=(3, free_port(), q), nprocs=3, join=True)
    assert q.get() == [[], [], []]
