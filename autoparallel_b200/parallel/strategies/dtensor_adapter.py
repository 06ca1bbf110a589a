"""The single module that touches DTensor's private sharding-propagation internals.

Everything the planner needs from upstream goes through here: the strategy data model
(``OpStrategy`` / ``OpSpec`` / ``DTensorSpec``), lookup of a registered op strategy (with the
single-dim-strategy and decomposition fallbacks newer torch uses), and enumeration helpers.
A PyTorch bump is meant to be a one-file change.  Reference counterpart:
autoparallel/shardings/dtensor_sharding_helpers.py:214-361.
"""
from __future__ import annotations

import itertools
import logging
from typing import Optional, Sequence

import torch
from torch.distributed.tensor import DTensor
from torch.distributed.tensor._dtensor_spec import DTensorSpec, TensorMeta
from torch.distributed.tensor._op_schema import (  # noqa: F401
    OpSchema,
    OpSpec,
    OpStrategy,
    RuntimeSchemaInfo,
    TupleStrategy,
)
from torch.distributed.tensor.placement_types import Partial, Placement, Replicate, Shard  # noqa: F401

logger = logging.getLogger(__name__)

propagator = DTensor._op_dispatcher.sharding_propagator
_warned_replicate: set = set()


def tensor_meta_of(t: torch.Tensor) -> TensorMeta:
    return TensorMeta(torch.Size(t.shape), tuple(t.stride()), t.dtype)


def local_shape(shape: Sequence[int], mesh_shape: Sequence[int], placements: Sequence[Placement]) -> Optional[list[int]]:
    """Per-rank shape (ceil-div) or None when a shard would be smaller than the mesh dim."""
    out = list(shape)
    for n, p in zip(mesh_shape, placements):
        if isinstance(p, Shard) or type(p).__name__ == "_StridedShard":  # a re-nested shard halves the dim like any shard
            d = p.dim
            if d >= len(out) or out[d] < n:
                return None
            out[d] = -(-out[d] // n)
    return out


def shard_extent(extent: int, parts: int, index: int) -> int:
    """Rows that part ``index`` of ``parts`` holds when ``extent`` rows are cut into ceil-sized chunks
    (``torch.chunk`` / DTensor ``Shard`` semantics: full chunks first, then a shorter one, then empty ones)."""
    c = -(-extent // parts)
    return max(0, min(c, extent - index * c))


def local_shape_at(shape: Sequence[int], mesh_shape: Sequence[int], placements: Sequence[Placement], coord: Sequence[int]) -> list[int]:
    """Shape of the shard held by the rank at mesh coordinate ``coord`` (differs between ranks when a
    sharded extent does not divide; equals ``local_shape`` when everything divides)."""
    out = list(shape)
    for n, p, c in zip(mesh_shape, placements, coord):
        if isinstance(p, Shard) or type(p).__name__ == "_StridedShard":
            out[p.dim] = shard_extent(out[p.dim], n, c)
    return out


def my_local_shape(shape: Sequence[int], mesh, placements: Sequence[Placement]) -> list[int]:
    """Shape of the calling rank's own shard (rank 0's when the caller is not part of ``mesh``)."""
    coord = mesh.get_coordinate()
    if coord is None:
        coord = [0] * mesh.ndim
    return local_shape_at(shape, tuple(mesh.shape), placements, coord)


def is_even(shape: Sequence[int], mesh_shape: Sequence[int], placements: Sequence[Placement]) -> bool:
    out = list(shape)
    for n, p in zip(mesh_shape, placements):
        if isinstance(p, Shard) or type(p).__name__ == "_StridedShard":
            if out[p.dim] % n:
                return False
            out[p.dim] //= n
    return True


def is_valid_spec(spec: Optional[DTensorSpec], mesh, even_only: bool) -> bool:
    if spec is None or spec.tensor_meta is None:
        return True
    shape = list(spec.tensor_meta.shape)
    for n, p in zip(mesh.shape, spec.placements):
        if isinstance(p, Shard):
            d = p.dim
            if d >= len(shape) or shape[d] < n:
                return False
            if even_only and shape[d] % n != 0:
                return False
            chunk = -(-shape[d] // n)
            if chunk * (n - 1) >= shape[d]:
                # ceil-sized chunks would leave the last rank(s) without a row: operators such as convolution refuse empty
                # operands, and a shard is only offered while every rank holds part of it (the reference's rule)
                return False
            shape[d] = chunk
    if not even_only:
        # an uneven tensor dim may be split by one mesh dim only: the shard sizes of a second split would
        # depend on the first coordinate, which the lowered collectives do not handle
        splits: dict[int, int] = {}
        nested = set()
        for n, p in zip(mesh.shape, spec.placements):
            if isinstance(p, Shard):
                if p.dim in splits:
                    nested.add(p.dim)
                splits[p.dim] = splits.get(p.dim, 1) * n
        if any(spec.tensor_meta.shape[d] % splits[d] for d in nested):
            return False
    return True


def all_placements(mesh, ndim: int, partial: bool = False) -> list[tuple[Placement, ...]]:
    per_dim: list[Placement] = [Replicate()] + [Shard(i) for i in range(ndim)]
    if partial:
        per_dim.append(Partial())
    return list(itertools.product(per_dim, repeat=mesh.ndim))


def all_options(mesh, val: Optional[torch.Tensor], even_only: bool = True) -> OpStrategy:
    """Every product of {Replicate} ∪ {Shard(d)} per mesh dim that leaves a non-empty shard.

    Used for placeholders and redistribution points (reference:
    autoparallel/shardings/propagation_rules.py:184-201)."""
    if val is None:
        tm = TensorMeta(torch.Size(()), (), torch.float32)
    else:
        tm = tensor_meta_of(val)
    specs = []
    for pl in all_placements(mesh, len(tm.shape)):
        spec = DTensorSpec(mesh, pl, tensor_meta=tm)
        if is_valid_spec(spec, mesh, even_only):
            specs.append(OpSpec(spec, input_specs=[spec], redistribute_cost=[[0.0]]))
    return OpStrategy(specs)


def _single_dim_fallback(op, schema: OpSchema):
    info = propagator.op_single_dim_strategy_funcs.get(op) if hasattr(propagator, "op_single_dim_strategy_funcs") else None
    if info is None:
        return None
    from torch.distributed.tensor._ops.single_dim_strategy import (
        _insert_single_dim_replication_strategy,
        _ShardingPlaceholder,
    )
    from torch.distributed.tensor._ops.utils import expand_to_full_mesh_op_strategy

    mesh = schema.args_strategy[0].mesh

    def first_spec(a):
        if isinstance(a, OpStrategy):
            return a.strategies[0].output_spec
        if isinstance(a, TupleStrategy):
            return [c.strategies[0].output_spec if isinstance(c, OpStrategy) else c for c in a.children]
        return a

    spec_schema = OpSchema(op, tuple(first_spec(a) for a in schema.args_schema), schema.kwargs_schema)
    out_tm = propagator._propagate_tensor_meta_non_cached(spec_schema)
    n_out = 0 if out_tm is None else (1 if isinstance(out_tm, TensorMeta) else len(out_tm))
    n_in = len(schema.args_strategy)
    rows = info.func(op, schema.args_meta, schema.kwargs_meta)
    rows = _insert_single_dim_replication_strategy(rows, n_out, n_in)
    rows = [[Shard(p.dim) if isinstance(p, _ShardingPlaceholder) else p for p in r] for r in rows]
    return expand_to_full_mesh_op_strategy(
        mesh,
        schema,
        rows,
        input_index=n_out,
        output_tensor_meta=out_tm,
        allow_unbacked_sharding=getattr(info, "allow_unbacked_sharding", None),
        allow_uneven_sharding=getattr(info, "allow_uneven_sharding", False),
    )


def _decomp_fallback(op, schema: OpSchema):
    try:
        from torch.distributed.tensor._decompositions import DecompShardingStrategy
    except ImportError:
        return None
    if not DecompShardingStrategy.has_decomp(op):
        return None
    ds = propagator.decomp_strategy
    ds.ensure_schema_info(op)
    return ds.propagate_strategy(schema)


def replicate_only(op, schema: OpSchema, out_val) -> OpStrategy:
    mesh = next(a.mesh for a in schema.args_strategy)
    rep = (Replicate(),) * mesh.ndim

    def mk(v):
        return DTensorSpec(mesh, rep, tensor_meta=tensor_meta_of(v)) if isinstance(v, torch.Tensor) else None

    outs = tuple(mk(v) for v in out_val) if isinstance(out_val, (tuple, list)) else mk(out_val)
    ins = [DTensorSpec(mesh, rep, tensor_meta=a.strategies[0].output_spec.tensor_meta) for a in schema.args_strategy]
    return OpStrategy([OpSpec(outs, input_specs=ins)])


def upstream_strategy(op, schema: OpSchema, out_val=None):
    """Strategy for ``op`` from DTensor: registered function → single-dim expansion →
    decomposition tracing → replicate-everything (warned once per op)."""
    fn = propagator.op_strategy_funcs.get(op)
    if fn is not None:
        try:
            return fn(schema)
        except (AssertionError, IndexError, NotImplementedError, RuntimeError, TypeError, ValueError) as e:
            # the registered function does not cover this call form (e.g. ``None`` entries in an index list)
            logger.debug("registered strategy of %s failed: %s", op, e)
    for fb in (_single_dim_fallback, _decomp_fallback):
        try:
            res = fb(op, schema)
        except Exception as e:  # upstream helper could not handle this op signature
            logger.debug("%s failed for %s: %s", fb.__name__, op, e)
            res = None
        if res is not None:
            return res
    if op not in _warned_replicate:
        _warned_replicate.add(op)
        logger.warning("no sharding strategy for %s: it will run replicated", op)
    return replicate_only(op, schema, out_val)
