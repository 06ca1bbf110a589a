"""Ordered sharding: the nesting order of mesh dims that shard the same tensor dim.

A parameter placed ``(Shard(0), Shard(0))`` on a (dp, tp) mesh is by default split dp-outer /
tp-inner.  Its uses want ``(Replicate(), Shard(0))`` – gather over dp, stay sharded over tp –
and with dp outside that takes two gathers and a re-slice, because the rows a dp-gather collects
on one tp rank are strided.  Nesting the shards the other way round (tp outer, dp inner) makes
the dp-gather return exactly the contiguous tp chunk: ONE collective on ONE mesh dim, and the
gradient's ``(Partial(), Shard(0)) -> (Shard(0), Shard(0))`` becomes ONE reduce-scatter.

This pass runs after the solver.  For every parameter whose placement nests a tensor dim over
two mesh dims it prices the redistributions on the parameter's use chain (and of its gradient)
under both nestings with the redistribution planner and keeps the cheaper one.  The chosen order
travels with the chain's nodes into the lowering, and the parameter is stored as a DTensor with a
``_StridedShard`` on the mesh dim that has become the inner one, which is how DTensor spells that
layout (checkpoints therefore round-trip through ``torch.distributed.checkpoint`` unchanged).

Reference: autoparallel/shardings/ordered_sharding.py:155-219 (use chains), :252-374 (order
choice), :70-102 (redistribution with an order).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.fx as fx
from torch.distributed.tensor.placement_types import Shard

from .redistribute import RedistributeError, plan_redistribution

Order = tuple  # mesh dims from the outermost shard to the innermost


def nested_dims(placements: Sequence) -> Optional[tuple[int, int]]:
    """The two mesh dims that shard one tensor dim, if the placement has exactly one such pair."""
    by_dim: dict[int, list[int]] = {}
    for i, p in enumerate(placements):
        if isinstance(p, Shard):
            by_dim.setdefault(p.dim, []).append(i)
    pairs = [v for v in by_dim.values() if len(v) >= 2]
    if len(pairs) != 1 or len(pairs[0]) != 2:
        return None
    return tuple(pairs[0])


def _n_collectives(src, dst, mesh_shape, order) -> Optional[int]:
    try:
        steps = plan_redistribution(src, dst, mesh_shape, order=order)
    except RedistributeError:
        return None
    return sum(1 for s in steps if s.kind != "local_chunk") * 10 + len(steps)


def compute_shard_orders(joint, solution: dict, mesh) -> dict[fx.Node, Order]:
    """node -> mesh-dim order for every node that carries a re-nested parameter layout: the
    parameter placeholder, the nodes of its use chain that keep its placement, and the node that
    produces its gradient in that layout."""
    mesh_shape = tuple(mesh.shape)
    if len(mesh_shape) < 2:
        return {}
    default = tuple(range(len(mesh_shape)))
    orders: dict[fx.Node, Order] = {}
    grads = joint.param_grads or {}
    for name, p in joint.param_nodes.items():
        if p not in solution:
            continue
        pl = tuple(solution[p].output_spec.placements)
        pair = nested_dims(pl)
        if pair is None:
            continue
        a, b = pair
        swapped = list(default)
        swapped[a], swapped[b] = b, a
        swapped = tuple(swapped)
        # nodes that keep the parameter's placement (cast / alias chain) and the edges that leave it
        chain, edges, stack, safe = [p], [], [p], True
        while stack and safe:
            n = stack.pop()
            for u in n.users:
                if u.op == "output":
                    safe = False  # the raw shard is returned to the caller in its default layout
                    break
                if u not in solution or u.op != "call_function":
                    continue
                ispecs = solution[u].input_specs or []
                tin = [i for i in u.all_input_nodes if i in solution]
                if n not in tin or tin.index(n) >= len(ispecs):
                    safe = False
                    break
                dst = tuple(ispecs[tin.index(n)].placements)
                out = solution[u].output_specs
                same_out = not isinstance(out, (tuple, list)) and tuple(out.placements) == pl
                if dst != pl:
                    edges.append((pl, dst))
                elif same_out and len(tin) == 1:
                    chain.append(u)  # elementwise on the shard: the layout passes through
                    stack.append(u)
                else:
                    safe = False  # something computes on the nested shard together with other data
                    break
        if not safe:
            continue
        # A layout can only be re-nested where a redistribution creates it.  The gradient qualifies when
        # its last node receives it through an edge whose source has no nested shard of its own
        # (e.g. (Partial, Shard(0)) -> (Shard(0), Shard(0)) is a reduce-scatter that can split either way).
        g = grads.get(name)
        grad_edge_nodes = []
        if g is not None:
            ok = False
            if g in solution and g.op == "call_function":
                gin = [i for i in g.all_input_nodes if i in solution]
                ispecs = solution[g].input_specs or []
                gout = solution[g].output_specs
                if len(gin) == 1 and ispecs and not isinstance(gout, (tuple, list)) and tuple(gout.placements) == pl:
                    prod = solution[gin[0]].output_specs
                    if not isinstance(prod, (tuple, list)) and tuple(ispecs[0].placements) == pl \
                            and nested_dims(tuple(prod.placements)) is None and all(u.op == "output" for u in g.users):
                        edges.append((tuple(prod.placements), pl))
                        grad_edge_nodes.append(g)
                        ok = True
            if not ok:
                continue
        if not edges:
            continue
        cost_d = [_n_collectives(s, d, mesh_shape, default) for s, d in edges]
        cost_s = [_n_collectives(s, d, mesh_shape, swapped) for s, d in edges]
        if any(c is None for c in cost_d + cost_s) or sum(cost_s) >= sum(cost_d):
            continue
        for n in chain + grad_edge_nodes:
            orders[n] = swapped
    return orders


def dtensor_placements(placements: Sequence, order: Optional[Order], mesh_shape: Sequence[int]) -> tuple:
    """Placements as DTensor spells them: the mesh dim that became the INNER shard of the pair gets a
    ``_StridedShard`` whose split factor is the extent of the mesh dim now outside it."""
    if order is None or tuple(order) == tuple(range(len(mesh_shape))):
        return tuple(placements)
    from torch.distributed.tensor.placement_types import _StridedShard

    pair = nested_dims(placements)
    if pair is None:
        return tuple(placements)
    a, b = pair  # a < b; default: a outer.  swapped: b outer, a inner
    out = list(placements)
    out[a] = _StridedShard(placements[a].dim, split_factor=mesh_shape[b])
    return tuple(out)


def order_of_dtensor_placements(placements: Sequence, mesh_ndim: int) -> Optional[Order]:
    from torch.distributed.tensor.placement_types import _StridedShard

    strided = [i for i, p in enumerate(placements) if isinstance(p, _StridedShard)]
    if not strided:
        return None
    plain = [Shard(p.dim) if isinstance(p, _StridedShard) else p for p in placements]
    pair = nested_dims(plain)
    if pair is None or strided != [pair[0]]:
        raise NotImplementedError(f"unsupported strided placement {placements}")
    order = list(range(mesh_ndim))
    order[pair[0]], order[pair[1]] = pair[1], pair[0]
    return tuple(order)


def local_shard(full: torch.Tensor, placements: Sequence, coord: Sequence[int], mesh_shape: Sequence[int],
                order: Optional[Order] = None) -> torch.Tensor:
    """This rank's shard of ``full``: split mesh dim by mesh dim from the outermost shard inwards."""
    out = full
    for i in (order or range(len(mesh_shape))):
        p = placements[i]
        if isinstance(p, Shard) or type(p).__name__ == "_StridedShard":
            out = out.chunk(mesh_shape[i], dim=p.dim)[coord[i]]
    return out.contiguous()
