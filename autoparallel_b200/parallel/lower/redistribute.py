"""Planning of one placement change as an ordered list of per-mesh-dim collectives.

The same plan is priced by the cost model and emitted by the lowering, so what the solver pays
for is what runs.  Ordering rules (a tensor dim sharded over several mesh dims is split
outer-mesh-dim first):

1. *unshard* steps (all-gather, all-to-all) run from the innermost mesh dim outwards;
2. a mesh dim whose shard sits *inside* a shard that changes (same tensor dim, outer mesh dim)
   is gathered first and re-sharded afterwards, so chunks stay contiguous;
3. *shard* steps (local slice, reduce-scatter) and all-reduces run from the outermost mesh dim
   inwards.

Reference: DTensor's ``redistribute_local_tensor`` as driven by
autoparallel/shardings/ordered_sharding.py:70-102 and priced by
autoparallel/cost_models/collective_runtime_estimation.py:115-229.
"""
from __future__ import annotations

from typing import NamedTuple, Optional, Sequence

from torch.distributed.tensor.placement_types import Partial, Placement, Replicate, Shard


class Step(NamedTuple):
    kind: str  # all_gather | all_reduce | reduce_scatter | all_to_all | local_chunk
    mesh_dim: int
    dim: Optional[int] = None  # gather / scatter / chunk dim (all_to_all: new shard dim)
    dim2: Optional[int] = None  # all_to_all: old shard dim (concat dim)
    op: str = "sum"  # all_reduce: the pending reduction it completes ("sum" | "max" | "min")


class RedistributeError(RuntimeError):
    pass


def plan_redistribution(src: Sequence[Placement], dst: Sequence[Placement], mesh_shape: Sequence[int],
                        order: Optional[Sequence[int]] = None) -> list[Step]:
    """``order``: mesh dims from the outermost shard to the innermost for tensor dims sharded over
    several mesh dims (default: mesh-dim order).  A different order is planned on the permuted mesh
    and the steps are mapped back, so every rule below applies unchanged."""
    if order is not None and tuple(order) != tuple(range(len(mesh_shape))):
        perm = list(order)
        steps = plan_redistribution([src[i] for i in perm], [dst[i] for i in perm], [mesh_shape[i] for i in perm])
        return [s._replace(mesh_dim=perm[s.mesh_dim]) for s in steps]
    nd = len(mesh_shape)
    cur = list(src)
    steps: list[Step] = []
    for q, p in zip(dst, src):
        if isinstance(q, Partial) and not isinstance(p, Partial):
            raise RedistributeError(f"cannot create a pending reduction: {p} -> {q}")

    def changes(i):
        return cur[i] != dst[i] and mesh_shape[i] > 1

    # tensor dims touched by a change on mesh dim i (as source shard or target shard)
    def touched(i):
        dims = set()
        if isinstance(cur[i], Shard):
            dims.add(cur[i].dim)
        if isinstance(dst[i], Shard):
            dims.add(dst[i].dim)
        return dims

    must_unshard = set()
    for i in range(nd):
        if not changes(i):
            continue
        if isinstance(cur[i], Shard):
            must_unshard.add(i)
        for j in range(i + 1, nd):
            if isinstance(cur[j], Shard) and cur[j].dim in touched(i) and mesh_shape[j] > 1:
                must_unshard.add(j)
    # phase 1: inner -> outer
    for i in sorted(must_unshard, reverse=True):
        p, q = cur[i], dst[i]
        simple_a2a = (
            isinstance(q, Shard)
            and q.dim != p.dim
            and not any(isinstance(cur[j], Shard) and cur[j].dim == q.dim for j in range(nd) if j != i)
            and not any(isinstance(dst[j], Shard) and dst[j].dim == q.dim for j in range(nd) if j != i)
            and not any(isinstance(cur[j], Shard) and cur[j].dim == p.dim for j in range(i + 1, nd))
        )
        if simple_a2a:
            steps.append(Step("all_to_all", i, q.dim, p.dim))
            cur[i] = q
        else:
            steps.append(Step("all_gather", i, p.dim))
            cur[i] = Replicate()
    # phase 2: outer -> inner
    for i in range(nd):
        p, q = cur[i], dst[i]
        if p == q or mesh_shape[i] == 1:
            cur[i] = q
            continue
        if isinstance(p, Partial) and isinstance(q, Replicate):
            steps.append(Step("all_reduce", i, op=p.reduce_op))
        elif isinstance(p, Partial) and isinstance(q, Shard):
            if p.reduce_op == "sum":
                steps.append(Step("reduce_scatter", i, q.dim))
            else:  # a pending maximum / minimum: complete it everywhere, then keep this rank's slice
                steps.append(Step("all_reduce", i, op=p.reduce_op))
                steps.append(Step("local_chunk", i, q.dim))
        elif isinstance(p, Replicate) and isinstance(q, Shard):
            steps.append(Step("local_chunk", i, q.dim))
        else:
            raise RedistributeError(f"cannot redistribute {p} -> {q} on mesh dim {i}")
        cur[i] = q
    return steps


FLAT = -1  # Step.mesh_dim of a collective that runs on the flattened mesh (all mesh dims at once)


def fuse_over_flat_mesh(steps: list[Step], nd: int, order: Optional[Sequence[int]] = None) -> list[Step]:
    """``(S(d), .., S(d)) -> (R, .., R)`` planned as one all-gather per mesh dim, or ``(P, .., P) ->
    (S(d), .., S(d))`` planned as one reduce-scatter per mesh dim, is the same data movement as ONE
    collective over the flattened mesh, because ranks of the flattened mesh are numbered in the
    default nesting order of the shards.  Only whole-mesh runs with the default order are fused.
    Reference: autoparallel/shardings/ordered_sharding.py:33-67."""
    if nd < 2 or len(steps) != nd or (order is not None and tuple(order) != tuple(range(nd))):
        return steps
    kinds = {s.kind for s in steps}
    dims = {s.dim for s in steps}
    if len(kinds) != 1 or len(dims) != 1:
        return steps
    kind = next(iter(kinds))
    mesh_dims = [s.mesh_dim for s in steps]
    if kind == "all_gather" and mesh_dims == list(range(nd - 1, -1, -1)):
        return [Step("all_gather", FLAT, steps[0].dim)]
    if kind == "reduce_scatter" and mesh_dims == list(range(nd)):
        return [Step("reduce_scatter", FLAT, steps[0].dim)]
    return steps
