"""Graph pass that merges a collective with the GEMM next to it into one fused node.

Patterns on the lowered per-rank graph:

* ``mm_nd(x, all_gather(w, 0))``  – FSDP parameter gather feeding a projection (forward: weight
  used transposed; backward dgrad: weight used as stored, the gathered rows are the contraction
  dim) → ``apb200_comm::ag_mm`` modes 0 / 1.  Every GEMM consumer of a gathered parameter gets its
  own fused node, i.e. the parameter is re-gathered where it is used (reshard-after-forward); with
  ``reshard_after_forward=False`` later consumers reuse the gathered operand the first node returns.
* ``mm_nd(all_gather(x, rows), w)`` – sequence-sharded activations entering a column-parallel
  projection → ``ag_mm`` modes 2 / 3 (several projections of the same gathered activation share the
  gathered operand returned by the first).
* ``reduce_scatter(mm_nd(..), rows)`` and ``reduce_scatter(mm_wgrad(..), 0)`` – row-parallel
  projection with a sequence-sharded result, and weight gradient with gradient reduce-scatter →
  ``apb200_comm::mm_rs`` modes 0 / 1 / 2.

* the same two shapes around ``apb200::scaled_mm`` (fp8 operands with tensor-wise or row-wise scales): a gathered
  float8 activation or weight shard takes its row-wise scale along (the scale's own all-gather is folded into the
  node) → ``ag_scaled_mm``; ``reduce_scatter(scaled_mm(..), rows)`` → ``scaled_mm_rs``.  These nodes are compositions of
  a collective and the library's fp8 GEMM - there is no single-kernel fp8 implementation.

Reference counterpart: ``micro_pipeline_tp_pass`` (autoparallel/graph_passes/async_tp/asynctp.py:
1265-1329), which only handles gathered *activations* and decomposes into host-side pipelines; this
pass also covers gathered weights and targets single-kernel implementations.
"""
from __future__ import annotations

import operator

import torch
import torch.fx as fx

from ...runtime import comm_ops

apb = torch.ops.apb200
comm = comm_ops.ops


def _rows_leading(shape, dim) -> bool:
    """True when ``dim`` is the outermost non-unit dim of ``shape[:-1]`` (row blocks stay contiguous
    after flattening the leading dims)."""
    lead = list(shape[:-1])
    if dim >= len(lead):
        return False
    return all(s == 1 for s in lead[:dim])


def _tangent_dependent(gm: fx.GraphModule, tangents) -> set:
    T = set(tangents)
    for n in gm.graph.nodes:
        if n.op == "call_function" and any(i in T for i in n.all_input_nodes):
            T.add(n)
    return T


def fuse_collectives(gm: fx.GraphModule, tangents=(), reshard_after_forward: bool = True,
                     fuse_contraction_gather: bool = False, patterns=("ag_mm", "mm_rs")) -> dict:
    """``fuse_contraction_gather``: also fuse a gather whose rows are the GEMM's contraction dim (the
    FSDP dgrad).  Every output tile then needs every shard, so the kernel cannot start a tile on
    local data while the rest arrives; measured slower than a prefetched gather, hence off by default.
    ``patterns``: which of the two families to rewrite (``("mm_rs",)`` keeps every gather a separate node,
    e.g. when parameter gathers are served by the copy engines and only the reductions need a kernel)."""
    g = gm.graph
    stats = {"ag_mm": 0, "mm_rs": 0, "ag_scaled_mm": 0, "scaled_mm_rs": 0}
    T = _tangent_dependent(gm, tangents)
    order = {n: i for i, n in enumerate(g.nodes)}

    def make_getitem(node, idx, like):
        with g.inserting_after(node):
            gi = g.call_function(operator.getitem, (node, idx))
        gi.meta = dict(like.meta)
        return gi

    # ---- GEMM -> reduce-scatter
    for rs in [n for n in g.nodes if "mm_rs" in patterns and n.op == "call_function" and n.target is comm.reduce_scatter.default]:
        src, dim, group, n_ranks = rs.args
        if not (isinstance(src, fx.Node) and src.op == "call_function" and len(src.users) == 1):
            continue
        if src.target is apb.mm_wgrad.default and dim == 0:
            a, b, dt = src.args
            mode = 2
        elif src.target is apb.mm_nd.default and _rows_leading(src.meta["val"].shape, dim):
            a, b, trans_b, dt = src.args
            mode = 0 if trans_b else 1
        else:
            continue
        with g.inserting_before(rs):
            fused = g.call_function(comm.mm_rs.default, (a, b, mode, dim, dt, 1.0, group, n_ranks))
        fused.meta = dict(rs.meta)
        rs.replace_all_uses_with(fused)
        g.erase_node(rs)
        g.erase_node(src)
        stats["mm_rs"] += 1

    # ---- fp8: scaled GEMM -> reduce-scatter, all-gather -> scaled GEMM
    def gathered_scale(scale, ag_src_rows, dim, group, n_ranks):
        """``scale`` as the fused node wants it: the un-gathered row-wise scale when ``scale`` is an all-gather of it over
        the same group and dim, the scale itself when it is tensor-wise, None when the pattern does not apply."""
        v = scale.meta.get("val")
        if v is not None and v.numel() == 1:
            return scale
        if (scale.op == "call_function" and scale.target is comm.all_gather.default and scale.args[1] == dim
                and scale.args[2] == group and len(scale.users) == 1):
            return scale.args[0]
        return None

    for rs in [n for n in g.nodes if "mm_rs" in patterns and n.op == "call_function" and n.target is comm.reduce_scatter.default]:
        src, dim, group, n_ranks = rs.args
        if not (isinstance(src, fx.Node) and src.op == "call_function" and src.target is apb.scaled_mm.default and len(src.users) == 1):
            continue
        if not _rows_leading(src.meta["val"].shape, dim):
            continue
        a, b, sa, sb, trans_b, dt = src.args
        with g.inserting_before(rs):
            fused = g.call_function(comm.scaled_mm_rs.default, (a, b, sa, sb, 0 if trans_b else 1, dim, dt, group, n_ranks))
        fused.meta = dict(rs.meta)
        rs.replace_all_uses_with(fused)
        g.erase_node(rs)
        g.erase_node(src)
        stats["scaled_mm_rs"] += 1

    gone: set = set()
    for ag in [n for n in g.nodes if "ag_mm" in patterns and n.op == "call_function" and n.target is comm.all_gather.default]:
        if ag in gone:
            continue
        x, dim, group, n_ranks = ag.args
        val = ag.meta["val"]
        for u in sorted(ag.users, key=lambda u: order.get(u, 1 << 30)):
            if u.op != "call_function" or u.target is not apb.scaled_mm.default:
                continue
            a, b, sa, sb, trans_b, dt = u.args
            if b is ag and a is not ag and val.ndim == 2 and dim == 0 and trans_b:
                sw = gathered_scale(sb, x, 0, group, n_ranks)
                if sw is None:
                    continue
                args, old_scale = (a, x, sa, sw, 0, 0, dt, group, n_ranks), sb
            elif a is ag and b is not ag and _rows_leading(val.shape, dim):
                sx = gathered_scale(sa, x, dim, group, n_ranks)
                if sx is None:
                    continue
                args, old_scale = (x, b, sx, sb, 2 if trans_b else 3, dim, dt, group, n_ranks), sa
            else:
                continue
            with g.inserting_before(u):
                fused = g.call_function(comm.ag_scaled_mm.default, args)
            fused.meta = dict(u.meta)
            fused.meta["val"] = (u.meta["val"], ag.meta["val"])
            order[fused] = order[u]
            y = make_getitem(fused, 0, u)
            u.replace_all_uses_with(y)
            g.erase_node(u)
            if old_scale.op == "call_function" and old_scale.target is comm.all_gather.default and len(old_scale.users) == 0:
                g.erase_node(old_scale)
                gone.add(old_scale)
            stats["ag_scaled_mm"] += 1
        if len(ag.users) == 0:
            g.erase_node(ag)
            gone.add(ag)

    # ---- all-gather -> GEMM
    for ag in [n for n in g.nodes if "ag_mm" in patterns and n.op == "call_function" and n.target is comm.all_gather.default]:
        x, dim, group, n_ranks = ag.args
        users = sorted(ag.users, key=lambda u: order.get(u, 1 << 30))
        val = ag.meta["val"]
        shared = None  # node whose second output is the gathered operand, reusable by later users
        for u in users:
            if u.op != "call_function" or u.target is not apb.mm_nd.default:
                continue
            a, b, trans_b, dt = u.args
            if b is ag and a is not ag and val.ndim == 2 and dim == 0:
                mode = 0 if trans_b else 1
                if mode == 1 and not fuse_contraction_gather:
                    continue
                args = (a, x, mode, 0, dt, group, n_ranks)
                is_weight = True
            elif a is ag and b is not ag and _rows_leading(val.shape, dim):
                mode = 2 if trans_b else 3
                args = (x, b, mode, dim, dt, group, n_ranks)
                is_weight = False
            else:
                continue
            regather = is_weight and reshard_after_forward
            if shared is not None and not regather and order[shared] < order[u] and (u in T) == (shared in T):
                # reuse the operand gathered by an earlier fused node in the same pass direction
                with g.inserting_before(u):
                    full = g.call_function(operator.getitem, (shared, 1))
                full.meta = dict(ag.meta)
                u.replace_input_with(ag, full)
                continue
            with g.inserting_before(u):
                fused = g.call_function(comm.ag_mm.default, args)
            fused.meta = dict(u.meta)
            fused.meta["val"] = (u.meta["val"], ag.meta["val"])
            order[fused] = order[u]
            if u in T:
                T.add(fused)
            y = make_getitem(fused, 0, u)
            u.replace_all_uses_with(y)
            g.erase_node(u)
            stats["ag_mm"] += 1
            if not regather:
                shared = fused
        if len(ag.users) == 0:
            g.erase_node(ag)
    g.lint()
    gm.recompile()
    return stats
