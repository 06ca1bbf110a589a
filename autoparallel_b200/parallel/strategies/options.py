"""Placement options per FX node.

``options_for_node`` returns the ``OpStrategy`` (list of candidate ``OpSpec`` = output
placement(s) + one required input placement per tensor argument) of a joint-graph node, from a
framework rule when there is one and from DTensor otherwise; results are normalised (tensor
metadata attached, invalid / duplicate candidates dropped) and memoised on a structural key.
Reference: autoparallel/shardings/placement_options.py:60-360, 652-660.
"""
from __future__ import annotations

import logging
import operator
import time
from collections import defaultdict
from typing import Any

import torch
import torch.fx as fx
from torch.utils._pytree import tree_map_only

from . import rules as _rules
from .dtensor_adapter import (
    DTensorSpec,
    OpSchema,
    OpSpec,
    OpStrategy,
    Partial,
    Replicate,
    RuntimeSchemaInfo,
    Shard,
    TupleStrategy,
    is_valid_spec,
    tensor_meta_of,
    upstream_strategy,
)

logger = logging.getLogger(__name__)

_cache: dict = {}


class OptionStats:
    """Timing / cache statistics of strategy enumeration (reference: placement_options.py:220-276)."""

    def __init__(self):
        self.reset()

    def reset(self):
        self.calls = self.hits = 0
        self.seconds = 0.0
        self.per_op = defaultdict(float)

    def summary(self, top: int = 10) -> str:
        ops = sorted(self.per_op.items(), key=lambda kv: -kv[1])[:top]
        lines = [f"placement options: {self.calls} calls, {self.hits} cache hits, {self.seconds:.3f}s"]
        lines += [f"  {t:8.3f}s  {op}" for op, t in ops]
        return "\n".join(lines)


stats = OptionStats()


def reset_caches() -> None:
    _cache.clear()
    stats.reset()


def _fp_spec(s) -> Any:
    if s is None:
        return None
    if isinstance(s, DTensorSpec):
        tm = s.tensor_meta
        return (tuple(str(p) for p in s.placements), tuple(tm.shape) if tm else None, tm.dtype if tm else None)
    if isinstance(s, (tuple, list)):
        return tuple(_fp_spec(x) for x in s)
    return repr(s)


def _fp_strategy(st) -> Any:
    if isinstance(st, OpStrategy):
        return tuple(_fp_spec(s.output_specs) for s in st.strategies)
    if isinstance(st, (list, tuple)):
        return tuple(_fp_strategy(x) for x in st)
    if isinstance(st, torch.Tensor):
        return (tuple(st.shape), st.dtype)
    return repr(st)


def _copy(st: OpStrategy) -> OpStrategy:
    return OpStrategy(
        [
            OpSpec(
                s.output_specs,
                input_specs=list(s.input_specs) if s.input_specs is not None else None,
                redistribute_cost=None,
            )
            for s in st.strategies
        ]
    )


def _attach_meta(strat: OpStrategy, out_val, in_vals, mesh) -> None:
    """DTensor leaves ``tensor_meta`` unset in places and uses ``None`` output specs for absent
    optional outputs; make both explicit so later passes need no special cases."""
    rep = (Replicate(),) * mesh.ndim
    for s in strat.strategies:
        outs = s.output_specs
        if isinstance(out_val, (tuple, list)):
            outs = list(outs) if isinstance(outs, (tuple, list)) else [outs]
            fixed = []
            for spec, v in zip(outs, out_val):
                if not isinstance(v, torch.Tensor):
                    fixed.append(None)
                    continue
                if spec is None:
                    spec = DTensorSpec(mesh, rep)
                fixed.append(DTensorSpec(mesh, spec.placements, tensor_meta=tensor_meta_of(v)))
            s.output_specs = tuple(fixed)
        elif isinstance(outs, DTensorSpec) and isinstance(out_val, torch.Tensor):
            s.output_specs = DTensorSpec(mesh, outs.placements, tensor_meta=tensor_meta_of(out_val))
        if s.input_specs is None:
            # pointwise-style upstream strategies with one tensor input follow the output
            assert len(in_vals) == 1, "strategy without input specs on a multi-input op"
            s.input_specs = [s.output_spec]
        ins = list(s.input_specs)
        if len(ins) != len(in_vals):
            raise RuntimeError(f"strategy has {len(ins)} input specs for {len(in_vals)} tensor inputs (op {getattr(strat, '_apb200_op', '?')})")
        s.input_specs = [
            DTensorSpec(mesh, spec.placements, tensor_meta=tensor_meta_of(v)) for spec, v in zip(ins, in_vals)
        ]
        s.redistribute_cost = None


def _view_keeps_counts(s, mesh) -> bool:
    """A reshape is local only if every rank's input shard has as many elements as its output shard."""
    import itertools as _it

    from .dtensor_adapter import is_even, local_shape_at

    i, o = s.input_specs[0], s.output_specs
    if i is None or o is None or isinstance(o, (tuple, list)) or i.tensor_meta is None or o.tensor_meta is None:
        return True
    if is_even(i.tensor_meta.shape, mesh.shape, i.placements) and is_even(o.tensor_meta.shape, mesh.shape, o.placements):
        return True
    for coord in _it.product(*(range(n) for n in mesh.shape)):
        a = local_shape_at(i.tensor_meta.shape, mesh.shape, i.placements, coord)
        b = local_shape_at(o.tensor_meta.shape, mesh.shape, o.placements, coord)
        na = nb = 1
        for x in a:
            na *= x
        for x in b:
            nb *= x
        if na != nb:
            return False
    return True


_RESHAPES = (torch.ops.aten.view.default, torch.ops.aten._unsafe_view.default, torch.ops.aten.reshape.default)


def _filter(strat: OpStrategy, mesh, even_only: bool, op=None) -> OpStrategy:
    kept, seen = [], set()
    for s in strat.strategies:
        outs = s.output_specs if isinstance(s.output_specs, (tuple, list)) else [s.output_specs]
        if not all(is_valid_spec(x, mesh, even_only) for x in list(outs) + list(s.input_specs)):
            continue
        if not even_only:
            if op in _RESHAPES and s.input_specs and not _view_keeps_counts(s, mesh):
                continue
        if not all(_plain_placements(x) for x in list(outs) + list(s.input_specs)):
            continue  # masked / averaging partials need op-specific local math; not lowered
        key = (_fp_spec(s.output_specs), _fp_spec(s.input_specs))
        if key in seen:
            continue
        seen.add(key)
        kept.append(s)
    return OpStrategy(kept)


def _plain_placements(spec) -> bool:
    if spec is None:
        return True
    for p in spec.placements:
        if isinstance(p, Partial) and (type(p) is not Partial or p.reduce_op not in ("sum", "max", "min")):
            return False  # masked / averaging partials need op-specific local math; sums, maxima and minima are lowered
        if not isinstance(p, (Partial, Replicate, Shard)) or type(p).__name__ == "_StridedShard":
            return False
    return True


def tensor_inputs(node: fx.Node) -> list[fx.Node]:
    """Tensor-valued argument nodes in argument order (duplicates kept)."""
    out: list[fx.Node] = []
    fx.node.map_arg((node.args, node.kwargs), lambda n: out.append(n) or n)
    return [n for n in out if isinstance(n.meta.get("val"), torch.Tensor) or isinstance(n.meta.get("val"), (tuple, list))]


def options_for_node(mesh, node: fx.Node, strats: dict[fx.Node, Any], even_only: bool = True) -> OpStrategy:
    t0 = time.perf_counter()
    op = node.target
    out_val = node.meta.get("val")
    in_nodes = tensor_inputs(node)
    in_vals = [n.meta["val"] for n in in_nodes]
    in_strats = [strats[n] for n in in_nodes]
    const_args = tree_map_only(fx.Node, lambda n: None, (node.args, node.kwargs))
    try:
        key = (op, _fp_strategy(in_strats), _fp_strategy(in_vals), repr(const_args), _fp_strategy(out_val), even_only, id(mesh))
        hash(key)
    except TypeError:
        key = None
    stats.calls += 1
    if key is not None and key in _cache:
        stats.hits += 1
        res = _copy(_cache[key])
        dt = time.perf_counter() - t0
        stats.seconds += dt
        stats.per_op[str(op)] += dt
        return res

    rule = _rules.get_rule(op)
    if rule is not None:
        ctx = _rules.RuleCtx(mesh, op, node.args, node.kwargs, in_vals, in_strats, out_val, even_only)
        strat = rule(ctx)
        if op is not operator.getitem:
            _attach_meta(strat, out_val, in_vals, mesh)
    else:
        strat = _from_dtensor(mesh, node, strats, out_val)
        flat_in_vals = [v for v in in_vals if isinstance(v, torch.Tensor)]
        _attach_meta(strat, out_val, flat_in_vals, mesh)
    if op is not operator.getitem:
        strat = _filter(strat, mesh, even_only, op)
    if len(strat.strategies) == 0:
        raise RuntimeError(f"no valid sharding strategy for node {node.name} ({op})")
    if key is not None:
        _cache[key] = _copy(strat)
    dt = time.perf_counter() - t0
    stats.seconds += dt
    stats.per_op[str(op)] += dt
    return strat


def _from_dtensor(mesh, node: fx.Node, strats, out_val) -> OpStrategy:
    op = node.target
    needs_pytree = False

    def conv(a):
        nonlocal needs_pytree
        if isinstance(a, fx.Node):
            st = strats.get(a)
            if st is not None:
                return st
            return a.meta.get("val")
        if isinstance(a, (list, tuple)) and any(isinstance(x, fx.Node) and x in strats for x in a):
            needs_pytree = True
            return TupleStrategy([conv(x) for x in a])
        return a

    args = tuple(conv(a) for a in node.args)
    kwargs = {k: conv(v) for k, v in node.kwargs.items()}
    schema = OpSchema(op, args, kwargs, RuntimeSchemaInfo(needs_pytree=needs_pytree))
    strat = upstream_strategy(op, schema, out_val)
    if isinstance(strat, TupleStrategy):
        # list-output ops (split, unbind): zip children into tuple-output strategies
        children = strat.children
        n = len(children[0].strategies)
        merged = []
        for i in range(n):
            outs = tuple(c.strategies[i].output_spec for c in children)
            merged.append(OpSpec(outs, input_specs=list(children[0].strategies[i].input_specs)))
        strat = OpStrategy(merged)
    return strat
