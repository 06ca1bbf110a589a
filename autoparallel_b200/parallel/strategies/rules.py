"""Sharding rules owned by the framework.

A rule maps ``(mesh, node, input strategies, input values, output value)`` to an
``OpStrategy``.  Rules exist for (a) every ``apb200`` operator – written as tables of
single-mesh-dim placements and expanded to the full mesh, (b) ATen ops where the planner wants
different behaviour from DTensor's default (``alias`` as a free redistribution point, factory
ops shardable at zero cost, ``getitem`` mirroring its producer, casts as pass-through).
Reference: autoparallel/shardings/propagation_rules.py:56-680.
"""
from __future__ import annotations

import itertools
import operator
from typing import Callable, Optional, Sequence

import torch

from .dtensor_adapter import (
    DTensorSpec,
    OpSpec,
    OpStrategy,
    Partial,
    Placement,
    Replicate,
    Shard,
    all_options,
    is_valid_spec,
    tensor_meta_of,
)

aten = torch.ops.aten
apb = torch.ops.apb200

R = Replicate()
P = Partial()


def S(d: int) -> Shard:
    return Shard(d)


_RULES: dict[object, Callable] = {}


def register_rule(*ops):
    def deco(fn):
        for op in ops:
            _RULES[op] = fn
        return fn

    return deco


def get_rule(op) -> Optional[Callable]:
    return _RULES.get(op)


def registered_ops():
    return list(_RULES)


class RuleCtx:
    """What a rule sees: the mesh, tensor input values/strategies (in argument order), the
    node's full args (for flags) and its output value(s)."""

    def __init__(self, mesh, op, args, kwargs, in_vals, in_strats, out_val, even_only):
        self.mesh, self.op, self.args, self.kwargs = mesh, op, args, kwargs
        self.in_vals, self.in_strats, self.out_val, self.even_only = in_vals, in_strats, out_val, even_only

    @property
    def out_vals(self):
        return list(self.out_val) if isinstance(self.out_val, (tuple, list)) else [self.out_val]


def expand_rows(ctx: RuleCtx, rows: Sequence[Sequence[Optional[Placement]]]) -> OpStrategy:
    """``rows[i] = (out_0, .., out_{m-1}, in_0, .., in_{n-1})`` placements for ONE mesh dim;
    the full-mesh strategy set is the product over mesh dims, filtered for shard validity."""
    mesh = ctx.mesh
    outs, ins = ctx.out_vals, ctx.in_vals
    n_out = len(outs)
    rep_row = tuple([R if isinstance(v, torch.Tensor) else None for v in outs] + [R] * len(ins))
    rows = [tuple(r) for r in rows]
    if rep_row not in rows:
        rows = [rep_row] + rows
    out_tms = [tensor_meta_of(v) if isinstance(v, torch.Tensor) else None for v in outs]
    in_tms = [tensor_meta_of(v) for v in ins]
    specs = []
    seen = set()
    for combo in itertools.product(rows, repeat=mesh.ndim):
        per_tensor = list(zip(*combo))  # per tensor: placements over mesh dims
        key = tuple(per_tensor)
        if key in seen:
            continue
        seen.add(key)
        o_specs = [
            DTensorSpec(mesh, tuple(pl), tensor_meta=tm) if tm is not None else None
            for pl, tm in zip(per_tensor[:n_out], out_tms)
        ]
        i_specs = [DTensorSpec(mesh, tuple(pl), tensor_meta=tm) for pl, tm in zip(per_tensor[n_out:], in_tms)]
        if not all(is_valid_spec(s, mesh, ctx.even_only) for s in o_specs + i_specs):
            continue
        out = o_specs[0] if not isinstance(ctx.out_val, (tuple, list)) else tuple(o_specs)
        specs.append(OpSpec(out, input_specs=i_specs))
    return OpStrategy(specs)


def _lead_dims(v: torch.Tensor, keep_last: int = 1):
    return range(v.ndim - keep_last)


# ------------------------------------------------------------------------------ apb200 operators
@register_rule(apb.rms_norm.default)
def _rms_norm(ctx):
    x = ctx.in_vals[0]
    return expand_rows(ctx, [(S(i), S(i), S(i), R) for i in _lead_dims(x)])


@register_rule(apb.rms_norm_bwd.default)
def _rms_norm_bwd(ctx):
    x = ctx.in_vals[1]
    return expand_rows(ctx, [(S(i), P, S(i), S(i), R, S(i)) for i in _lead_dims(x)])


@register_rule(apb.rope.default)
def _rope(ctx):
    # x [B, S, H, D]; cos/sin [S, D/2]
    return expand_rows(ctx, [(S(0), S(0), R, R), (S(1), S(1), S(0), S(0)), (S(2), S(2), R, R)])


@register_rule(apb.swiglu.default)
def _swiglu(ctx):
    return expand_rows(ctx, [(S(i), S(i), S(i)) for i in range(ctx.in_vals[0].ndim)])


@register_rule(apb.swiglu_bwd.default)
def _swiglu_bwd(ctx):
    return expand_rows(ctx, [(S(i),) * 5 for i in range(ctx.in_vals[0].ndim)])


@register_rule(apb.attention.default)
def _attention(ctx):
    # q [B,S,H,D], k/v [B,S,Hkv,D] -> o [B,S,H,D], lse [B,H,S]; batch- and head-parallel.
    return expand_rows(ctx, [(S(0), S(0), S(0), S(0), S(0)), (S(2), S(1), S(2), S(2), S(2))])


@register_rule(apb.attention_bwd.default)
def _attention_bwd(ctx):
    # (dout, q, k, v, out, lse) -> (dq, dk, dv)
    return expand_rows(
        ctx,
        [
            (S(0), S(0), S(0), S(0), S(0), S(0), S(0), S(0), S(0)),
            (S(2), S(2), S(2), S(2), S(2), S(2), S(2), S(2), S(1)),
        ],
    )


@register_rule(apb.cross_entropy.default)
def _xent(ctx):
    logits = ctx.in_vals[0]
    return expand_rows(ctx, [(S(i), S(i), S(i), S(i)) for i in _lead_dims(logits)])


@register_rule(apb.cross_entropy_bwd.default)
def _xent_bwd(ctx):
    logits = ctx.in_vals[1]
    return expand_rows(ctx, [(S(i), S(i), S(i), S(i), S(i)) for i in _lead_dims(logits)])


@register_rule(apb.mm_nd.default)
def _mm_nd(ctx):
    a, b = ctx.in_vals
    trans_b = ctx.args[2]
    last = a.ndim - 1
    kdim, ndim = (1, 0) if trans_b else (0, 1)
    rows = [(S(i), S(i), R) for i in range(last)]
    rows += [(P, S(last), S(kdim)), (S(last), R, S(ndim))]
    return expand_rows(ctx, rows)


@register_rule(apb.scaled_mm.default)
def _scaled_mm(ctx):
    # (out, a, b, scale_a, scale_b): rows of ``a`` carry their row-wise scale, columns of the result carry ``scale_b``;
    # a split of the contraction dim leaves both scales whole (they do not depend on k) and yields partial sums
    a, b, sa, sb = ctx.in_vals[:4]
    trans_b = ctx.args[4]
    last = a.ndim - 1
    kdim, ndim = (1, 0) if trans_b else (0, 1)
    row_a = sa.ndim == a.ndim and sa.numel() > 1
    row_b = sb.ndim == 2 and sb.numel() > 1
    rows = [(S(i), S(i), R, S(i) if row_a and sa.shape[i] == a.shape[i] else R, R) for i in range(last)]
    rows += [(S(last), R, S(ndim), R, S(ndim) if row_b else R), (P, S(last), S(kdim), R, R)]
    return expand_rows(ctx, rows)


@register_rule(apb.mm_wgrad.default)
def _mm_wgrad(ctx):
    a, b = ctx.in_vals
    la, lb = a.ndim - 1, b.ndim - 1
    rows = [(P, S(i), S(i)) for i in range(la)]
    rows += [(S(0), S(la), R), (S(1), R, S(lb))]
    return expand_rows(ctx, rows)


@register_rule(apb.gemm.default)
def _gemm(ctx):
    ta, tb = ctx.args[2], ctx.args[3]
    am, ak = (1, 0) if ta else (0, 1)
    bk, bn = (1, 0) if tb else (0, 1)
    return expand_rows(ctx, [(S(0), S(am), R), (S(1), R, S(bn)), (P, S(ak), S(bk))])


# ---- planner-visible mixture-of-experts ops (ops/moe_ops.py).  Tokens [T, ..] and the block dim of the
# buffer [E, nb, C, d] shard together (every rank keeps whole token blocks); the feature dim d can be
# split through scatter / gather with replicated routing.  The expert dim is never sharded INSIDE
# these ops: expert parallelism is the redistribution Shard(1) -> Shard(0) of the buffer (one
# all-to-all) between the scatter and the grouped GEMMs, which the solver prices like any other edge.
@register_rule(apb.moe_slots.default)
def _moe_slots(ctx):
    return expand_rows(ctx, [(S(0), S(0))])


@register_rule(apb.moe_scatter.default)
def _moe_scatter(ctx):
    # (buf, src, slot, w)
    return expand_rows(ctx, [(S(1), S(0), S(0), S(0)), (S(3), S(1), R, R), (P, P, R, R)])


@register_rule(apb.moe_gather.default)
def _moe_gather(ctx):
    # (out, buf, slot, w)
    return expand_rows(ctx, [(S(0), S(1), S(0), S(0)), (S(1), S(3), R, R), (P, P, R, R)])


@register_rule(apb.moe_gate_grad.default)
def _moe_gate_grad(ctx):
    # (dw, buf, slot, g): a feature-dim split leaves partial dot products
    return expand_rows(ctx, [(S(0), S(1), S(0), S(0)), (P, S(3), R, S(1))])


@register_rule(apb.grouped_mm.default)
def _grouped_mm(ctx):
    trans_b = ctx.args[2]
    kdim, ndim = (2, 1) if trans_b else (1, 2)
    # (out [E,M,N], a [E,M,K], b): experts, rows, columns, contraction
    return expand_rows(ctx, [(S(0), S(0), S(0)), (S(1), S(1), R), (S(2), R, S(ndim)), (P, S(2), S(kdim))])


@register_rule(apb.grouped_mm_wgrad.default)
def _grouped_mm_wgrad(ctx):
    # (out [E,Ka,Nb], a [E,M,Ka], b [E,M,Nb])
    return expand_rows(ctx, [(S(0), S(0), S(0)), (P, S(1), S(1)), (S(1), S(2), R), (S(2), R, S(2))])


@register_rule(apb.embedding.default)
def _embedding(ctx):
    # (out [*ids, D], weight [V, D], ids): split the tokens, or the hidden dim of the table; a table split by rows
    # would need a masked lookup and a reduction and is not offered (the table is gathered instead)
    weight, ids = ctx.in_vals
    rows = [(S(i), R, S(i)) for i in range(ids.ndim)]
    rows.append((S(ids.ndim), S(1), R))
    return expand_rows(ctx, rows)


@register_rule(apb.embedding_bwd.default)
def _embedding_bwd(ctx):
    dy, ids = ctx.in_vals
    rows = [(P, S(i), S(i)) for i in range(ids.ndim)]
    rows.append((S(1), S(dy.ndim - 1), R))
    return expand_rows(ctx, rows)


# ------------------------------------------------------------------------------ pass-through ops
def passthrough(ctx: RuleCtx, allow_partial: bool = True) -> OpStrategy:
    """One strategy per input option: output placement == input placement."""
    (strat,) = ctx.in_strats
    out_tm = tensor_meta_of(ctx.out_val)
    specs = []
    for s in strat.strategies:
        src = s.output_spec
        if not allow_partial and any(isinstance(p, Partial) for p in src.placements):
            continue
        specs.append(
            OpSpec(
                DTensorSpec(ctx.mesh, src.placements, tensor_meta=out_tm),
                input_specs=[DTensorSpec(ctx.mesh, src.placements, tensor_meta=src.tensor_meta)],
            )
        )
    return OpStrategy(specs)


@register_rule(apb.dtype_cast.default, torch.ops.prims.convert_element_type.default)
def _cast(ctx):
    return passthrough(ctx, allow_partial=True)


@register_rule(aten.alias.default)
def _alias(ctx):
    """Every placement in, same placement out: a zero-cost node whose *incoming edge* is where
    the solver pays for a redistribution shared by all consumers."""
    return all_options(ctx.mesh, ctx.out_val, ctx.even_only)


# ------------------------------------------------------------------------------ factory ops
FACTORY_OPS = [
    aten.zeros.default,
    aten.ones.default,
    aten.full.default,
    aten.empty.memory_format,
    aten.rand.default,
    aten.randn.default,
]
REPLICATED_FACTORY_OPS = [
    aten.arange.default,
    aten.arange.start,
    aten.arange.start_step,
    aten.scalar_tensor.default,
    torch.ops.prims.iota.default,
]


@register_rule(*FACTORY_OPS)
def _factory(ctx):
    """No tensor inputs: any sharding of the output is free (each rank creates its shard)."""
    strat = all_options(ctx.mesh, ctx.out_val, ctx.even_only)
    for s in strat.strategies:
        s.input_specs = []
    return strat


@register_rule(*REPLICATED_FACTORY_OPS)
def _replicated_factory(ctx):
    spec = DTensorSpec(ctx.mesh, (R,) * ctx.mesh.ndim, tensor_meta=tensor_meta_of(ctx.out_val))
    return OpStrategy([OpSpec(spec, input_specs=[])])


@register_rule(operator.getitem)
def _getitem(ctx):
    """Mirrors the producer 1:1 – strategy *i* of ``getitem`` is element ``idx`` of the
    producer's strategy *i* (the solver ties the two indices together)."""
    (strat,) = ctx.in_strats
    idx = ctx.args[1]
    specs = []
    for s in strat.strategies:
        outs = s.output_specs
        if not isinstance(outs, (tuple, list)) or idx >= len(outs):
            raise RuntimeError(
                f"getitem[{idx}] of a producer whose strategy describes {len(outs) if isinstance(outs, (tuple, list)) else 1} "
                f"outputs (producer value has {len(ctx.in_vals[0]) if isinstance(ctx.in_vals[0], (tuple, list)) else 1})"
            )
        spec = outs[idx]
        specs.append(OpSpec(spec, input_specs=[spec]))
    return OpStrategy(specs)


# ------------------------------------------------------------------------------ dropout / indexing
@register_rule(aten.native_dropout.default)
def _native_dropout(ctx):
    """(out, mask) of one input: any dim may be sharded, every rank draws its own mask for its shard."""
    (x,) = ctx.in_vals
    return expand_rows(ctx, [(S(i), S(i), S(i)) for i in range(x.ndim)])


@register_rule(aten.uniform.default, aten.normal_functional.default, aten.bernoulli.p, aten.bernoulli.default,
               aten.rand_like.default, aten.randn_like.default)
def _random_like(ctx):
    """Random values with the shape of the input (``x.uniform_()``, ``bernoulli``, ``rand_like``): the output follows any
    sharding of the input; a sharded output is drawn per shard from the shard's own stream (runtime/rng.py)."""
    x = ctx.in_vals[0]
    return expand_rows(ctx, [(S(i), S(i)) for i in range(x.ndim)])


@register_rule(aten.native_dropout_backward.default)
def _native_dropout_bwd(ctx):
    g = ctx.in_vals[0]
    return expand_rows(ctx, [(S(i), S(i), S(i)) for i in range(g.ndim)])


@register_rule(aten.constant_pad_nd.default)
def _constant_pad(ctx):
    """Padding (or cropping, with negative amounts) leaves every other dim free to shard."""
    x = ctx.in_vals[0]
    pads = list(ctx.args[1])
    touched = {x.ndim - 1 - i for i in range(len(pads) // 2) if pads[2 * i] != 0 or pads[2 * i + 1] != 0}
    return expand_rows(ctx, [(S(d), S(d)) for d in range(x.ndim) if d not in touched])


@register_rule(aten.index.Tensor)
def _index_tensor(ctx):
    """``x[..., idx, ...]`` with ONE index tensor (other entries ``None``): untouched dims of ``x`` shard
    through (shifted by the index tensor's rank), or the index tensor is sharded and ``x`` is whole along
    the indexed dim.  Other forms run replicated."""
    x = ctx.in_vals[0]
    index_list = ctx.args[1]
    pos = [i for i, a in enumerate(index_list) if a is not None]
    if len(pos) != 1 or len(ctx.in_vals) != 2:
        return expand_rows(ctx, [])
    k, idx = pos[0], ctx.in_vals[1]
    shift = idx.ndim - 1
    rows = []
    for d in range(x.ndim):
        if d == k:
            continue
        rows.append((S(d if d < k else d + shift), S(d), R))
    for j in range(idx.ndim):
        rows.append((S(k + j), R, S(j)))
    return expand_rows(ctx, rows)


@register_rule(aten.index_select.default)
def _index_select(ctx):
    """``x.index_select(dim, index)``: every other dim of ``x`` shards through; or the 1-D index is sharded and the
    result is sharded along ``dim`` (``x`` whole along it)."""
    x = ctx.in_vals[0]
    dim = ctx.args[1] % max(x.ndim, 1)
    rows = [(S(d), S(d), R) for d in range(x.ndim) if d != dim]
    rows.append((S(dim), R, S(0)))
    return expand_rows(ctx, rows)


@register_rule(aten.index_add.default)
def _index_add(ctx):
    """``x.index_add(dim, index, source)``: dims other than ``dim`` shard through ``x``, ``source`` and the result
    alike; a sharded index with the matching slice of ``source`` yields partial sums of a zero-based accumulation only
    when ``x`` itself is partial, which is not offered."""
    x = ctx.in_vals[0]
    dim = ctx.args[1] % max(x.ndim, 1)
    return expand_rows(ctx, [(S(d), S(d), R, S(d)) for d in range(x.ndim) if d != dim])


# ------------------------------------------------------------------------------ view / reshape
def _view_groups(in_shape, out_shape):
    """Split both shapes into aligned groups with equal element counts:
    ``[8, 64, 256] -> [8, 64, 8, 32]`` gives ``([0],[0]), ([1],[1]), ([2],[2,3])``."""
    groups = []
    i = j = 0
    ni, nj = len(in_shape), len(out_shape)
    while i < ni or j < nj:
        gi, gj = [], []
        pi = pj = 1
        if i < ni:
            gi.append(i)
            pi *= in_shape[i]
            i += 1
        if j < nj:
            gj.append(j)
            pj *= out_shape[j]
            j += 1
        while pi != pj:
            if pi < pj:
                if i >= ni:
                    return None
                gi.append(i)
                pi *= in_shape[i]
                i += 1
            else:
                if j >= nj:
                    return None
                gj.append(j)
                pj *= out_shape[j]
                j += 1
        # absorb trailing size-1 dims
        while i < ni and in_shape[i] == 1 and (j >= nj or out_shape[j] != 1):
            gi.append(i)
            i += 1
        while j < nj and out_shape[j] == 1 and (i >= ni or in_shape[i] != 1):
            gj.append(j)
            j += 1
        groups.append((gi, gj))
    return groups


def view_placement_map(in_shape, out_shape, mesh_shape, placements):
    """Output placements of ``x.view(out_shape)`` for a given input placement, or None when the
    view cannot be done shard-locally.  A shard on the *leading* non-unit dim of a group maps to
    the leading non-unit output dim of that group when the sizes divide."""
    groups = _view_groups(list(in_shape), list(out_shape))
    if groups is None:
        return None
    in_to_group = {}
    for g in groups:
        for d in g[0]:
            in_to_group[d] = g
    rem_out = list(out_shape)  # remaining (local) size of each out dim as mesh dims shard it
    rem_in = list(in_shape)
    out = []
    for n, p in zip(mesh_shape, placements):
        if not isinstance(p, Shard):
            out.append(p)
            continue
        d = p.dim
        gi, gj = in_to_group[d]
        lead_in = next((x for x in gi if in_shape[x] != 1), gi[0])
        if d != lead_in:
            return None
        lead_out = next((x for x in gj if out_shape[x] != 1), gj[0] if gj else None)
        if lead_out is None:
            return None
        if rem_in[d] % n != 0 or rem_out[lead_out] % n != 0:
            return None
        rem_in[d] //= n
        rem_out[lead_out] //= n
        out.append(Shard(lead_out))
    return tuple(out)


@register_rule(aten.view.default, aten._unsafe_view.default, aten.reshape.default)
def _view(ctx):
    (strat,) = ctx.in_strats
    x = ctx.in_vals[0]
    out_tm = tensor_meta_of(ctx.out_val)
    specs = []
    for s in strat.strategies:
        src = s.output_spec
        mapped = view_placement_map(x.shape, ctx.out_val.shape, ctx.mesh.shape, src.placements)
        if mapped is None:
            continue
        specs.append(
            OpSpec(
                DTensorSpec(ctx.mesh, mapped, tensor_meta=out_tm),
                input_specs=[DTensorSpec(ctx.mesh, src.placements, tensor_meta=src.tensor_meta)],
            )
        )
    return OpStrategy(specs)


# ------------------------------------------------------------------------------ layer norm
@register_rule(aten.native_layer_norm.default)
def _layer_norm(ctx):
    """(x, normalized_shape, weight?, bias?, eps) -> (out, mean, rstd); shard only outside the
    normalised dims.  (DTensor's own strategy indexes weight options by the input's option
    index and breaks when the two lists differ in length.)"""
    x = ctx.in_vals[0]
    n_norm = len(ctx.args[1])
    n_extra = len(ctx.in_vals) - 1
    rows = [(S(i), S(i), S(i), S(i)) + (R,) * n_extra for i in range(x.ndim - n_norm)]
    return expand_rows(ctx, rows)


@register_rule(aten.max.dim, aten.min.dim)
def _max_min_dim(ctx):
    """``x.max(dim)`` / ``x.min(dim)`` -> (values, indices): every dim but the reduced one shards through (renumbered
    when the reduced dim is dropped).  DTensor's strategy for these describes one output only."""
    x = ctx.in_vals[0]
    dim = ctx.args[1] % max(x.ndim, 1)
    keepdim = bool(ctx.args[2]) if len(ctx.args) > 2 else False
    rows = []
    for d in range(x.ndim):
        if d == dim:
            continue
        od = d if keepdim or d < dim else d - 1
        rows.append((S(od), S(od), S(d)))
    return expand_rows(ctx, rows)


@register_rule(aten.flip.default)
def _flip(ctx):
    x = ctx.in_vals[0]
    flipped = {d % max(x.ndim, 1) for d in ctx.args[1]}
    return expand_rows(ctx, [(S(d), S(d)) for d in range(x.ndim) if d not in flipped])


@register_rule(aten.cumsum.default, aten.cumprod.default, aten.logcumsumexp.default)
def _scan(ctx):
    """Prefix scans: every dim but the scanned one may be sharded."""
    x = ctx.in_vals[0]
    dim = ctx.args[1] % max(x.ndim, 1)
    return expand_rows(ctx, [(S(d), S(d)) for d in range(x.ndim) if d != dim])


@register_rule(aten.native_group_norm.default)
def _group_norm(ctx):
    """(x [N, C, *], weight?, bias?, N, C, HxW, groups, eps) -> (out [N, C, *], mean [N, G], rstd [N, G]): statistics are
    per sample and group, so the batch dim shards through."""
    n_extra = len(ctx.in_vals) - 1
    return expand_rows(ctx, [(S(0), S(0), S(0), S(0)) + (R,) * n_extra])


@register_rule(aten.native_group_norm_backward.default)
def _group_norm_bwd(ctx):
    """(dy, x, mean, rstd, weight?, N, C, HxW, groups, mask) -> (dx, dw?, db?): batch-sharded operands give the input
    gradient batch-sharded and partial sums for the affine parameters."""
    outs = ctx.out_vals
    n_extra = len(ctx.in_vals) - 4
    o = [S(0)] + [P if isinstance(v, torch.Tensor) else None for v in outs[1:]]
    return expand_rows(ctx, [tuple(o) + (S(0), S(0), S(0), S(0)) + (R,) * n_extra])


@register_rule(aten.native_layer_norm_backward.default)
def _layer_norm_bwd(ctx):
    """(dy, x, normalized_shape, mean, rstd, weight?, bias?, mask) -> (dx, dw?, db?)."""
    x = ctx.in_vals[1]
    n_norm = len(ctx.args[2])
    n_extra = len(ctx.in_vals) - 4
    outs = ctx.out_vals
    rows = []
    for i in range(x.ndim - n_norm):
        o = [S(i)] + [P if isinstance(v, torch.Tensor) else None for v in outs[1:]]
        rows.append(tuple(o) + (S(i), S(i), S(i), S(i)) + (R,) * n_extra)
    return expand_rows(ctx, rows)


# ------------------------------------------------------------------------------ misc ATen gaps
def _mask_rows(ctx, first_extra: int, d: int) -> tuple:
    """Placements of the tensor inputs after q/k/v(/...): an attention mask follows the batch / head shard
    where it has that dim in full and stays whole where it broadcasts (extent 1)."""
    q = ctx.in_vals[1] if first_extra == 6 else ctx.in_vals[0]
    out = []
    for v in ctx.in_vals[first_extra:]:
        follows = isinstance(v, torch.Tensor) and v.ndim == q.ndim and v.shape[d] == q.shape[d] and v.shape[d] > 1
        out.append(S(d) if follows else R)
    return tuple(out)


@register_rule(aten._scaled_dot_product_flash_attention_for_cpu.default)
def _sdpa_cpu(ctx):
    # q,k,v [B,H,S,D] (+ optional mask) -> (out [B,H,S,D], lse [B,H,S]); batch- and head-parallel
    return expand_rows(ctx, [(S(d),) * 5 + _mask_rows(ctx, 3, d) for d in (0, 1)])


@register_rule(aten._scaled_dot_product_flash_attention_for_cpu_backward.default)
def _sdpa_cpu_bwd(ctx):
    # (dout, q, k, v, out, lse, ...) -> (dq, dk, dv)
    return expand_rows(ctx, [(S(d),) * 9 + _mask_rows(ctx, 6, d) for d in (0, 1)])


# ------------------------------------------------------------------------------ convolution
# convolution(input [N,C,...], weight [O,C/groups,...], bias [O]?, stride, padding, dilation, transposed, output_padding, groups)
# Per mesh dim: split the batch; or (plain convolutions: one group, not transposed) split the output channels with
# the weight's rows, or the input channels with the weight's columns (partial sums out; only without a bias, which
# every rank would otherwise add once).  Spatial dims are never split (that would need halo exchanges).
@register_rule(aten.convolution.default)
def _convolution(ctx):
    has_bias = len(ctx.in_vals) == 3
    transposed, groups = bool(ctx.args[6]), int(ctx.args[8])
    rows = [(S(0), S(0), R) + ((R,) if has_bias else ())]
    if groups == 1 and not transposed:
        rows.append((S(1), R, S(0)) + ((S(0),) if has_bias else ()))
        if not has_bias:
            rows.append((P, S(1), S(1)))
    return expand_rows(ctx, rows)


# convolution_backward(grad_out, input, weight, bias_sizes, ..., transposed, output_padding, groups, output_mask)
#   -> (grad_input, grad_weight, grad_bias), each None where the mask says so
@register_rule(aten.convolution_backward.default)
def _convolution_bwd(ctx):
    transposed, groups = bool(ctx.args[7]), int(ctx.args[9])
    rows = [(S(0), P, P, S(0), S(0), R)]
    if groups == 1 and not transposed:
        rows.append((P, S(0), S(0), S(1), R, S(0)))    # output channels split: every rank holds a partial input gradient
        rows.append((S(1), S(1), R, R, S(1), S(1)))    # input channels split
    return expand_rows(ctx, rows)


def _channel_row(ctx):
    """Channel split of a batch-norm style op: [N, C, ...] tensors on dim 1, per-channel vectors on dim 0."""
    def pl(v):
        if not isinstance(v, torch.Tensor):
            return None
        return S(1) if v.ndim >= 2 else S(0) if v.ndim == 1 else R

    return tuple(pl(v) for v in ctx.out_vals) + tuple(pl(v) for v in ctx.in_vals)


# Batch statistics need every sample of a channel, so a training-mode batch norm is split over channels only (a batch
# split would have to combine means and variances across ranks inside the op); with fixed statistics the batch may
# be split as well.
@register_rule(aten._native_batch_norm_legit_functional.default, aten._native_batch_norm_legit.default,
               aten._native_batch_norm_legit.no_stats, aten.native_batch_norm.default, aten.native_batch_norm_backward.default)
def _batch_norm_training(ctx):
    training = next((a for a in ctx.args if isinstance(a, bool)), True)
    rows = [_channel_row(ctx)]
    if not training and ctx.op is not aten.native_batch_norm_backward.default:
        rows.append(tuple(S(0) if isinstance(v, torch.Tensor) and v.ndim >= 2 else (R if isinstance(v, torch.Tensor) else None) for v in ctx.out_vals)
                    + tuple(S(0) if v.ndim >= 2 else R for v in ctx.in_vals))
    return expand_rows(ctx, rows)


@register_rule(aten._native_batch_norm_legit_no_training.default)
def _batch_norm_eval(ctx):
    batch = tuple(S(0) if isinstance(v, torch.Tensor) and v.ndim >= 2 else (R if isinstance(v, torch.Tensor) else None) for v in ctx.out_vals) \
        + tuple(S(0) if v.ndim >= 2 else R for v in ctx.in_vals)
    return expand_rows(ctx, [_channel_row(ctx), batch])


@register_rule(aten.max_pool2d_with_indices.default, aten.max_pool2d_with_indices_backward.default)
def _max_pool(ctx):
    if ctx.in_vals[0].ndim != 4:
        return expand_rows(ctx, [])
    n = len(ctx.out_vals) + len(ctx.in_vals)
    return expand_rows(ctx, [(S(0),) * n, (S(1),) * n])  # windows never cross samples or channels


@register_rule(aten.avg_pool2d.default, aten.avg_pool2d_backward.default, aten._adaptive_avg_pool2d.default,
               aten._adaptive_avg_pool2d_backward.default)
def _avg_pool(ctx):
    """Average pooling (plain and adaptive, forward and backward): windows never cross samples or channels, so the batch
    and channel dims of a 4-D operand (the channel dim of a 3-D one) shard through every tensor of the node."""
    x = ctx.in_vals[0]
    n = len(ctx.out_vals) + len(ctx.in_vals)
    if x.ndim == 4:
        return expand_rows(ctx, [(S(0),) * n, (S(1),) * n])
    if x.ndim == 3:
        return expand_rows(ctx, [(S(0),) * n])
    return expand_rows(ctx, [])


def _pointwise_rows(ctx):
    """Rows of an elementwise operator with broadcasting: an output dim shards together with the matching dim of every
    operand that has it in full (aligned from the right); operands that broadcast along it stay whole."""
    out = ctx.out_vals[0]
    rows = []
    for d in range(out.ndim):
        row = [S(d) if isinstance(v, torch.Tensor) else None for v in ctx.out_vals]
        for v in ctx.in_vals:
            vd = d - (out.ndim - v.ndim)
            row.append(S(vd) if vd >= 0 and v.shape[vd] == out.shape[d] and out.shape[d] != 1 else R)
        rows.append(tuple(row))
    return rows


@register_rule(aten.hardtanh.default, aten.hardtanh_backward.default, aten.leaky_relu.default, aten.leaky_relu_backward.default,
               aten.elu.default, aten.elu_backward.default, aten.softplus.default, aten.softplus_backward.default,
               aten.hardswish.default, aten.hardswish_backward.default, aten.hardsigmoid.default, aten.hardsigmoid_backward.default,
               aten.mish.default, aten.mish_backward.default, aten.threshold.default, aten.threshold_backward.default,
               aten.softshrink.default, aten.hardshrink.default, aten.logit.default, aten.special_expm1.default)
def _pointwise(ctx):
    """Elementwise activations (and their backward forms) that have no registered strategy."""
    return expand_rows(ctx, _pointwise_rows(ctx))


@register_rule(aten.var_mean.correction, aten.var.correction, aten.std.correction, aten.std_mean.correction)
def _var_mean(ctx):
    """Variance / standard deviation (optionally with the mean) over some dims: no partial form, the surviving dims
    shard through every output."""
    x = ctx.in_vals[0]
    kwargs = ctx.kwargs or {}
    dims = ctx.args[1] if len(ctx.args) > 1 else kwargs.get("dim")
    dims = list(range(x.ndim)) if dims is None else ([dims] if isinstance(dims, int) else list(dims))
    dims = {d % max(x.ndim, 1) for d in dims} if dims else set(range(x.ndim))
    keepdim = bool(kwargs.get("keepdim", False))
    rows = []
    for d in range(x.ndim):
        if d in dims:
            continue
        od = d if keepdim else d - sum(1 for r in dims if r < d)
        rows.append(tuple(S(od) if isinstance(v, torch.Tensor) else None for v in ctx.out_vals) + (S(d),))
    return expand_rows(ctx, rows)


@register_rule(aten.median.dim, aten.nanmedian.dim, aten.mode.default, aten.kthvalue.default, aten.cummax.default, aten.cummin.default)
def _order_statistic(ctx):
    """(values, indices) of an order statistic along one dim: every other dim shards through."""
    x = ctx.in_vals[0]
    pos = 2 if ctx.op is aten.kthvalue.default else 1
    dim = (ctx.args[pos] if len(ctx.args) > pos else -1) % max(x.ndim, 1)
    scan = ctx.op in (aten.cummax.default, aten.cummin.default)
    keepdim = scan or (bool(ctx.args[pos + 1]) if len(ctx.args) > pos + 1 else False)
    rows = []
    for d in range(x.ndim):
        if d == dim:
            continue
        od = d if keepdim or d < dim else d - 1
        rows.append((S(od), S(od), S(d)))
    return expand_rows(ctx, rows)


@register_rule(aten.searchsorted.Tensor)
def _searchsorted(ctx):
    """``searchsorted(sorted_sequence, values)``: with an N-d sequence the leading dims pair up with those of ``values``
    and shard through; the searched (last) dim of the sequence stays whole."""
    seq, vals = ctx.in_vals[0], ctx.in_vals[1]
    if seq.ndim == 1:
        return expand_rows(ctx, [(S(d), R, S(d)) for d in range(vals.ndim)])
    return expand_rows(ctx, [(S(d), S(d), S(d)) for d in range(seq.ndim - 1)])


@register_rule(aten._cdist_forward.default)
def _cdist(ctx):
    """``cdist(x1 [.., P, M], x2 [.., R, M]) -> [.., P, R]``: batch dims shard through both; rows of either side alone."""
    x1 = ctx.in_vals[0]
    nb = x1.ndim - 2
    rows = [(S(d), S(d), S(d)) for d in range(nb)]
    rows += [(S(nb), S(nb), R), (S(nb + 1), R, S(nb))]
    return expand_rows(ctx, rows)


@register_rule(aten._cdist_backward.default)
def _cdist_bwd(ctx):
    """(grad [.., P, R], x1 [.., P, M], x2 [.., R, M], p, cdist [.., P, R]) -> dx1 [.., P, M]: batch dims and the rows of
    ``x1`` shard through; ``x2`` must be whole along its rows (every row of it contributes to every dx1 row)."""
    x1 = ctx.in_vals[1]
    nb = x1.ndim - 2
    rows = [(S(d), S(d), S(d), S(d), S(d)) for d in range(nb)]
    rows.append((S(nb), S(nb), S(nb), R, S(nb)))
    return expand_rows(ctx, rows)


@register_rule(aten.diagonal_scatter.default)
def _diagonal_scatter(ctx):
    """``diagonal_scatter(x, src, offset, dim1, dim2)``: dims of ``x`` outside the diagonal plane shard through; in ``src``
    they come first, in order, followed by the diagonal itself."""
    x = ctx.in_vals[0]
    d1 = (ctx.args[3] if len(ctx.args) > 3 else 0) % x.ndim
    d2 = (ctx.args[4] if len(ctx.args) > 4 else 1) % x.ndim
    rows, k = [], 0
    for d in range(x.ndim):
        if d in (d1, d2):
            continue
        rows.append((S(d), S(d), S(k)))
        k += 1
    return expand_rows(ctx, rows)


@register_rule(aten.adaptive_max_pool2d.default, aten.adaptive_max_pool2d_backward.default, aten.avg_pool3d.default,
               aten.avg_pool3d_backward.default, aten.max_pool3d_with_indices.default, aten.max_pool3d_with_indices_backward.default,
               aten._adaptive_avg_pool3d.default, aten._adaptive_avg_pool3d_backward.default, aten.adaptive_max_pool3d.default,
               aten.adaptive_max_pool3d_backward.default)
def _pool_nc(ctx):
    """Pooling over the spatial dims of [N, C, spatial...] operands (forward and backward forms, with or without index
    outputs): windows never cross samples or channels."""
    x = ctx.in_vals[0]
    n = len(ctx.out_vals) + len(ctx.in_vals)
    if x.ndim >= 4 and all(v.ndim == x.ndim for v in ctx.in_vals):
        return expand_rows(ctx, [(S(0),) * n, (S(1),) * n])
    return expand_rows(ctx, [])


@register_rule(aten.grid_sampler_2d.default)
def _grid_sampler(ctx):
    """``grid_sample(input [N, C, H, W], grid [N, Ho, Wo, 2]) -> [N, C, Ho, Wo]``: samples (input and grid together) or
    channels (grid whole)."""
    return expand_rows(ctx, [(S(0), S(0), S(0)), (S(1), S(1), R)])


@register_rule(aten.grid_sampler_2d_backward.default)
def _grid_sampler_bwd(ctx):
    """(grad, input, grid, ...) -> (dinput, dgrid): per-sample work."""
    o = tuple(S(0) if isinstance(v, torch.Tensor) else None for v in ctx.out_vals)
    return expand_rows(ctx, [o + (S(0), S(0), S(0))])


@register_rule(aten._fft_r2c.default, aten._fft_c2r.default, aten._fft_c2c.default)
def _fft(ctx):
    """Fourier transforms along ``dim``: every other dim shards through."""
    x = ctx.in_vals[0]
    dims = {d % max(x.ndim, 1) for d in ctx.args[1]}
    return expand_rows(ctx, [(S(d), S(d)) for d in range(x.ndim) if d not in dims])


@register_rule(aten._embedding_bag.default, aten._embedding_bag_forward_only.default)
def _embedding_bag(ctx):
    """(weight [V, D], indices, offsets, ...) -> (out [B, D], offset2bag, bag_size, max_indices): the embedding width may be
    split (every rank reduces its columns of the same rows); bags are not split - their boundaries are data."""
    n_in = len(ctx.in_vals)
    outs = ctx.out_vals
    row = (S(1),) + tuple(R if isinstance(v, torch.Tensor) else None for v in outs[1:]) + (S(1),) + (R,) * (n_in - 1)
    return expand_rows(ctx, [row])


@register_rule(aten._embedding_bag_backward.default, aten._embedding_bag_dense_backward.default)
def _embedding_bag_bwd(ctx):
    """(grad [B, D], indices, ...) -> dweight [V, D]: columns of the gradient give columns of the weight gradient."""
    n_in = len(ctx.in_vals)
    return expand_rows(ctx, [(S(1), S(1)) + (R,) * (n_in - 1)])


@register_rule(aten.any.dims, aten.any.dim, aten.all.dims, aten.all.dim)
def _any_all(ctx):
    """Logical reductions over some dims: the surviving dims shard through (no partial form of "or" / "and")."""
    x = ctx.in_vals[0]
    dims = ctx.args[1] if len(ctx.args) > 1 else None
    dims = list(range(x.ndim)) if dims is None else ([dims] if isinstance(dims, int) else list(dims))
    dims = {d % max(x.ndim, 1) for d in dims}
    keepdim = bool(ctx.args[2]) if len(ctx.args) > 2 else False
    rows = []
    for d in range(x.ndim):
        if d in dims:
            continue
        od = d if keepdim else d - sum(1 for r in dims if r < d)
        rows.append((S(od), S(d)))
    return expand_rows(ctx, rows)


@register_rule(aten.index_put.default)
def _index_put(ctx):
    # index_put(self, indices, values, accumulate): rows addressed by the index tensors must be whole on every rank,
    # so only dims behind a leading block of indexed dims are split; ``values`` follows where it has that dim in full.
    self_v, values = ctx.in_vals[0], ctx.in_vals[-1]
    indices = list(ctx.args[1])
    m = len(indices)
    if any(i is None for i in indices):
        return expand_rows(ctx, [])
    n_idx = len(ctx.in_vals) - 2
    rows = []
    for d in range(m, self_v.ndim):
        vd = values.ndim - (self_v.ndim - d)
        vpl = S(vd) if vd >= 0 and values.shape[vd] == self_v.shape[d] else R
        rows.append((S(d), S(d)) + (R,) * n_idx + (vpl,))
    return expand_rows(ctx, rows)


@register_rule(aten.copy.default)
def _copy(ctx):
    # copy(dst, src) -> src broadcast into dst's shape: split any dim of dst; src follows where it has that dim in full
    dst, src = ctx.in_vals[0], ctx.in_vals[1]
    rows = []
    for i in range(dst.ndim):
        j = i - (dst.ndim - src.ndim)
        rows.append((S(i), S(i), S(j) if j >= 0 and src.shape[j] == dst.shape[i] else R))
    return expand_rows(ctx, rows)


@register_rule(aten.squeeze.dims, aten.squeeze.dim)
def _squeeze(ctx):
    x = ctx.in_vals[0]
    dims = ctx.args[1]
    dims = [dims] if isinstance(dims, int) else list(dims)
    dims = {d % x.ndim for d in dims if x.shape[d % x.ndim] == 1}
    rows, new = [], 0
    for d in range(x.ndim):
        if d in dims:
            continue
        rows.append((S(new), S(d)))
        new += 1
    return expand_rows(ctx, rows)


@register_rule(aten.scatter.value, aten.scatter.src, aten.gather.default)
def _scatter_gather(ctx):
    """Shardable on every dim except the scatter/gather dim (all tensor operands alike)."""
    x = ctx.in_vals[0]
    dim = ctx.args[1] % x.ndim
    n = len(ctx.in_vals)
    return expand_rows(ctx, [(S(i),) * (1 + n) for i in range(x.ndim) if i != dim])
