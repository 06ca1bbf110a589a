"""User-facing manual-parallelism tools: ``local_map`` regions and the collectives to use inside them.

    from autoparallel_b200.collectives import local_map, all_to_all, all_gather, axis_size

    def experts(tokens, w):                 # runs on LOCAL shards
        tokens = all_to_all(tokens, "ep", split_dim=0, concat_dim=0)
        ...
    y = local_map(experts, out_placements=((Shard(0),),), in_placements=((Shard(0),), (Shard(0),)))(x, w)

``local_map`` defaults its mesh to the mesh of the enclosing ``AutoParallel`` context; collectives
address a mesh axis by *name*; every collective is differentiable (all-gather ↔ reduce-scatter,
all-reduce ↔ all-reduce, all-to-all ↔ all-to-all with swapped dims); ``with_sharding_constraint``
pins an intermediate tensor's placement.  Reference: autoparallel/collectives.py:16-229.
"""
from __future__ import annotations

from typing import Sequence

import torch
from torch.distributed.tensor.placement_types import Placement

from .runtime import comm_ops

_C = comm_ops.ops


def _current_mesh():
    from torch.distributed.device_mesh import _mesh_resources

    try:
        return _mesh_resources.get_current_mesh()
    except Exception as e:  # no mesh context
        raise RuntimeError("no device mesh is active: call inside `with AutoParallel(...)` / `with mesh:` or pass device_mesh") from e


def local_map(func=None, out_placements=None, in_placements=None, in_grad_placements=None, device_mesh=None, *,
              redistribute_inputs: bool = True):
    """``torch.distributed.tensor.experimental.local_map`` with the mesh taken from the active
    ``AutoParallel`` context at call time."""
    from torch.distributed._tensor.experimental import local_map as _lm

    def wrap(fn):
        def call(*args, **kwargs):
            mesh = device_mesh or _current_mesh()
            return _lm(fn, out_placements=out_placements, in_placements=in_placements, in_grad_placements=in_grad_placements,
                       device_mesh=mesh, redistribute_inputs=redistribute_inputs)(*args, **kwargs)

        call.__name__ = getattr(fn, "__name__", "local_map_region")
        return call

    return wrap if func is None else wrap(func)


def _axis(mesh_axis: str, mesh=None):
    mesh = mesh or _current_mesh()
    names = mesh.mesh_dim_names or ()
    if mesh_axis not in names:
        raise ValueError(f"mesh axis {mesh_axis!r} not in {names}")
    i = names.index(mesh_axis)
    return mesh.get_group(i).group_name, mesh.shape[i], mesh, i


def axis_size(mesh_axis: str) -> int:
    return _axis(mesh_axis)[1]


def axis_index(mesh_axis: str) -> int:
    _, _, mesh, i = _axis(mesh_axis)
    return mesh.get_local_rank(i)


def all_gather(x: torch.Tensor, mesh_axis: str, gather_dim: int = 0) -> torch.Tensor:
    g, n, _, _ = _axis(mesh_axis)
    return _C.all_gather(x, gather_dim, g, n)


def reduce_scatter(x: torch.Tensor, mesh_axis: str, scatter_dim: int = 0) -> torch.Tensor:
    g, n, _, _ = _axis(mesh_axis)
    return _C.reduce_scatter(x, scatter_dim, g, n)


def all_reduce(x: torch.Tensor, mesh_axis: str) -> torch.Tensor:
    g, n, _, _ = _axis(mesh_axis)
    return _C.all_reduce(x, g, n)


def all_to_all(x: torch.Tensor, mesh_axis: str, split_dim: int = 0, concat_dim: int = 0) -> torch.Tensor:
    """Split ``x`` into equal chunks along ``split_dim``, send chunk r to rank r of the axis and
    concatenate the received chunks along ``concat_dim``."""
    g, n, _, _ = _axis(mesh_axis)
    return _C.all_to_all(x, split_dim, concat_dim, g, n)


def with_sharding_constraint(x: torch.Tensor, placements: Sequence[Placement], device_mesh=None) -> torch.Tensor:
    """Pin ``x`` to ``placements`` in the plan (an identity region whose input and output placement
    are both ``placements``).  Works between ``local_map`` regions and on N-d meshes."""
    mesh = device_mesh or _current_mesh()
    if len(placements) != mesh.ndim:
        raise ValueError(f"{len(placements)} placements for a {mesh.ndim}-d mesh")
    pl = tuple(placements)
    return local_map(lambda t: t.clone(), out_placements=(pl,), in_placements=(pl,), device_mesh=mesh)(x)
