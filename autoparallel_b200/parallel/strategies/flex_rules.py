"""Sharding options of the flex-attention higher-order operators.

``flex_attention(q, k, v, score_mod, block_mask, scale, options, score_buffers, mask_buffers)`` and its
backward twin work on every (batch, head) pair independently, so each mesh dim may replicate the
call, split the batch dim (tensor dim 0) or split the head dim (tensor dim 1) of all tensors that
carry these dims: q / k / v, outputs, log-sum-exp, gradients and the block-mask index tensors.

* A tensor whose batch or head extent is 1 (a block mask built with ``B=None`` / ``H=None``, the single
  key/value head of multi-query attention) stays replicated on that mesh dim.
* Any other extent must divide by the product of the mesh dims that split it.  With grouped-query
  attention this makes head sharding available only while the *key/value* heads divide: a rank then
  holds whole groups, and local head ``h`` still reads local key/value head ``h // group``.  (The
  reference demotes the key/value tensors to replicated in that case, which changes the query →
  key/value head mapping on every rank but the first; such options are dropped here.)
* Buffers captured by ``score_mod`` / ``mask_mod`` are indexed arbitrarily and stay replicated; a captured
  buffer that requires a gradient is refused (its gradient would be a partial sum over ranks).
* ``score_mod`` / ``mask_mod`` see *local* batch and head indices; a mod that depends on the global
  batch or head index is not supported under sharding (same as the reference).

Reference: autoparallel/shardings/placement_options.py:493-649, tests/test_flex_attention.py.
"""
from __future__ import annotations

import inspect
import itertools

import torch
import torch.fx as fx
from torch.utils._pytree import tree_flatten

from .dtensor_adapter import DTensorSpec, OpSpec, OpStrategy, Replicate, Shard, tensor_meta_of

_HOP_NAMES = ("flex_attention", "flex_attention_backward")
_BUFFER_ARGS = ("score_mod_other_buffers", "mask_mod_other_buffers")


def is_flex_attention_node(node: fx.Node) -> bool:
    t = node.target
    return node.op == "call_function" and isinstance(t, torch._ops.HigherOrderOperator) and t.name() in _HOP_NAMES


def _signature(node: fx.Node) -> list[str]:
    from torch._higher_order_ops.flex_attention import flex_attention_backward_fake_tensor_mode, flex_attention_fake_impl

    fn = flex_attention_fake_impl if node.target.name() == "flex_attention" else flex_attention_backward_fake_tensor_mode
    return list(inspect.signature(fn).parameters)


def _captured_buffers(node: fx.Node) -> set[fx.Node]:
    names = _signature(node)
    found: set[fx.Node] = set()
    for arg_name in _BUFFER_ARGS:
        if arg_name in names:
            i = names.index(arg_name)
            value = node.args[i] if i < len(node.args) else node.kwargs.get(arg_name, ())
            found.update(x for x in tree_flatten(value)[0] if isinstance(x, fx.Node))
    return found


def _placement_for(t: torch.Tensor, choice: tuple, mesh):
    """Placement of one (batch, head, ...) tensor under ``choice`` (one of R / S(0) / S(1) per mesh dim), or
    None when an extent larger than 1 does not divide."""
    split = {0: 1, 1: 1}
    out = []
    for mesh_dim, p in enumerate(choice):
        if isinstance(p, Shard):
            if t.ndim <= p.dim or t.shape[p.dim] == 1:
                out.append(Replicate())
                continue
            split[p.dim] *= mesh.shape[mesh_dim]
            if t.shape[p.dim] % split[p.dim] != 0:
                return None
        out.append(p)
    return tuple(out)


def flex_attention_options(mesh, node: fx.Node, strats) -> OpStrategy:
    """One option per assignment of {Replicate, Shard(0), Shard(1)} to the mesh dims that every tensor of
    the call can follow.  ``strats`` tells which argument nodes the solver sees (sub-graphs of the mods and
    shape arithmetic are not among them)."""
    from ..frontend.graph_canon import all_input_nodes

    buffers = _captured_buffers(node)
    inputs = [a for a in all_input_nodes(node) if a in strats]
    vals = node.meta["val"]
    assert isinstance(vals, (tuple, list)), "flex attention returns a tuple"
    # forward: (out, log-sum-exp, row maxima); backward: (dq, dk, dv, gradients of captured buffers)
    top = list(vals)
    if any(isinstance(x, torch.Tensor) for v in top if isinstance(v, (tuple, list)) for x in v):
        raise NotImplementedError(
            f"{node.name}: a buffer captured by score_mod requires a gradient; sharded flex attention would have to "
            "sum it over ranks, which is not supported -- detach the buffer or wrap the call in local_map"
        )
    rep = (Replicate(),) * mesh.ndim

    options = []
    for choice in itertools.product((Replicate(), Shard(0), Shard(1)), repeat=mesh.ndim):
        ins, ok = [], True
        for a in inputs:
            v = a.meta["val"]
            if a in buffers or v.ndim < 2:
                pl = rep
            else:
                pl = _placement_for(v, choice, mesh)
                if pl is None:
                    ok = False
                    break
            ins.append(DTensorSpec(mesh, pl, tensor_meta=tensor_meta_of(v)))
        if not ok:
            continue
        outs = []
        for v in top:
            if not isinstance(v, torch.Tensor):
                outs.append(None)
                continue
            pl = _placement_for(v, choice, mesh)
            if pl is None:
                ok = False
                break
            outs.append(DTensorSpec(mesh, pl, tensor_meta=tensor_meta_of(v)))
        if ok:
            options.append(OpSpec(tuple(outs), input_specs=ins))
    # different choices collapse to the same specs when extents are 1: keep the first of each
    seen, unique = set(), []
    for o in options:
        key = (tuple(None if s is None else tuple(s.placements) for s in o.output_specs),
               tuple(tuple(s.placements) for s in o.input_specs))
        if key not in seen:
            seen.add(key)
            unique.append(o)
    return OpStrategy(unique)
