"""Canonicalisation of the captured joint graph before strategy enumeration.

Passes (reference counterparts in autoparallel/graph_passes/graph_utils.py):

* ``cleanup_graph``            – DCE, drop autograd ``alias``/``detach`` bookkeeping nodes, fold
  ``view∘view`` and ``permute∘permute`` (graph_utils.py:23-45).
* ``rewrite_linear_patterns``  – ``view → mm → view`` chains become ``apb200::mm_nd`` and the
  weight-gradient ``permute(view) @ view`` becomes ``apb200::mm_wgrad``, so leading dims stay
  visible to the planner (the reference rewrites to einsum, graph_utils.py:270-439).
* ``insert_redistribution_points`` – an ``aten.alias`` after every multi-consumer tensor and
  before every graph output; the alias' strategy set is *all* placements, which gives the solver
  one place to pay for a redistribution shared by several consumers (graph_utils.py:99-183).
* helpers: ``is_collective``, ``assert_has_no_collectives``, ``all_input_nodes`` (duplicate
  preserving), ``param_derived_set`` / ``terminal_derived_set`` (graph_utils.py:186-197,
  255-267, 442-484).
"""
from __future__ import annotations

import operator
from typing import Iterable

import torch
import torch.fx as fx

aten = torch.ops.aten
apb = torch.ops.apb200

_VIEW_OPS = (aten.view.default, aten._unsafe_view.default, aten.reshape.default)
_COLLECTIVE_NAMESPACES = ("_c10d_functional", "c10d_functional", "_dtensor", "symm_mem", "apb200_comm")


# ------------------------------------------------------------------------------------ helpers
def is_collective(node: fx.Node) -> bool:
    t = node.target
    return (
        node.op == "call_function"
        and isinstance(t, torch._ops.OpOverload)
        and t.namespace in _COLLECTIVE_NAMESPACES
    )


def assert_has_no_collectives(gm: fx.GraphModule) -> None:
    for n in gm.graph.nodes:
        if is_collective(n):
            raise RuntimeError(
                f"the model issues a collective itself ({n.target} at {n.name}); wrap manually-parallel "
                "regions in autoparallel_b200.collectives.local_map so the planner sees them as one node"
            )


def all_input_nodes(node: fx.Node) -> list[fx.Node]:
    """Like ``node.all_input_nodes`` but a node used twice appears twice (argument order)."""
    out: list[fx.Node] = []
    fx.node.map_arg((node.args, node.kwargs), lambda n: out.append(n) or n)
    return out


def _meta_val(n):
    return n.meta.get("val") if isinstance(n, fx.Node) else None


def _is_tensor_node(n) -> bool:
    return isinstance(_meta_val(n), torch.Tensor)


def param_derived_set(gm: fx.GraphModule, param_nodes: Iterable[fx.Node]) -> set[fx.Node]:
    """Nodes reachable from a parameter through single-tensor-input ops only (cast / view /
    transpose chains) – what an FSDP all-gather may be prefetched across."""
    derived = set(param_nodes)
    for n in gm.graph.nodes:
        if n.op != "call_function":
            continue
        ins = [i for i in all_input_nodes(n) if _is_tensor_node(i)]
        if len(ins) == 1 and ins[0] in derived:
            derived.add(n)
    return derived


def terminal_derived_set(gm: fx.GraphModule, terminal_nodes: Iterable[fx.Node]) -> set[fx.Node]:
    """Nodes from which a terminal (gradient output) is reached through single-consumer,
    single-tensor-input ops only – the chain a gradient reduce-scatter may be deferred over."""
    derived = set(terminal_nodes)
    for n in reversed(list(gm.graph.nodes)):
        if n.op != "call_function" or n in derived:
            continue
        users = list(n.users)
        if len(users) == 1 and users[0] in derived:
            ins = [i for i in all_input_nodes(users[0]) if _is_tensor_node(i)]
            if len(ins) == 1:
                derived.add(n)
    return derived


# ------------------------------------------------------------------------------------ cleanup
def _copy_meta(dst: fx.Node, src: fx.Node) -> None:
    for k in ("stack_trace", "nn_module_stack", "fwd_nn_module_stack", "seq_nr", "recompute", "ac_graph_id", "custom",
              "partitioner_tag", "autograd_backward"):
        if k in src.meta:
            dst.meta[k] = src.meta[k]


def cleanup_graph(gm: fx.GraphModule) -> None:
    g = gm.graph
    changed = True
    while changed:
        changed = False
        for n in list(g.nodes):
            if n.op != "call_function":
                continue
            t = n.target
            if t in (aten.sum.dim_IntList, aten.mean.dim) and len(n.args) > 1 and n.args[1] is not None and len(n.args[1]) == 0:
                # an empty dim list means "all dims" to ATen but "no dims" to DTensor's reduction rule
                src = n.args[0]
                if _is_tensor_node(src) and src.meta["val"].ndim > 0:  # (a 0-d operand has no dims to list)
                    n.update_arg(1, list(range(src.meta["val"].ndim)))
                    changed = True
            if t in (aten.alias.default, aten.detach.default, aten.lift_fresh_copy.default):
                n.replace_all_uses_with(n.args[0])
                g.erase_node(n)
                changed = True
            elif t in _VIEW_OPS and isinstance(n.args[0], fx.Node):
                src = n.args[0]
                if src.op == "call_function" and src.target in _VIEW_OPS:
                    n.update_arg(0, src.args[0])
                    changed = True
                elif _is_tensor_node(src) and _is_tensor_node(n) and tuple(src.meta["val"].shape) == tuple(
                    n.meta["val"].shape
                ) and all(isinstance(s, int) for s in n.meta["val"].shape):
                    n.replace_all_uses_with(src)
                    g.erase_node(n)
                    changed = True
            elif t is aten.permute.default or t is aten.t.default:
                src = n.args[0]
                if (
                    isinstance(src, fx.Node)
                    and src.op == "call_function"
                    and src.target in (aten.permute.default, aten.t.default)
                    and _meta_val(src) is not None
                    and src.meta["val"].ndim == 2
                    and _is_2d_transpose(n)
                    and _is_2d_transpose(src)
                ):
                    n.replace_all_uses_with(src.args[0])
                    g.erase_node(n)
                    changed = True
        before = len(g.nodes)
        g.eliminate_dead_code()
        changed = changed or len(g.nodes) != before
    g.lint()
    gm.recompile()


def _is_2d_transpose(n: fx.Node) -> bool:
    if n.op != "call_function":
        return False
    if n.target is aten.t.default:
        return True
    if n.target is aten.permute.default:
        return list(n.args[1]) == [1, 0]
    if n.target is aten.transpose.int:
        v = _meta_val(n)
        return v is not None and v.ndim == 2 and {n.args[1] % 2, n.args[2] % 2} == {0, 1}
    return False


# ------------------------------------------------------------------------------------ linear patterns
def _flatten_source(n):
    """If ``n`` is ``view(X, [M, K])`` where ``X`` has ndim > 2 and some split ``X.shape[:i] | X.shape[i:]``
    multiplies out to ``M | K`` with ``i >= 2``, return ``(X, lead_shape)``; else None."""
    if not (isinstance(n, fx.Node) and n.op == "call_function" and n.target in _VIEW_OPS):
        return None
    x = n.args[0]
    xv, nv = _meta_val(x), _meta_val(n)
    if xv is None or nv is None or xv.ndim <= 2 or nv.ndim != 2:
        return None
    shape = list(xv.shape)
    if not all(isinstance(s, int) for s in shape):
        return None
    k = 1
    for i in range(len(shape) - 1, 1, -1):
        k *= shape[i]
        if k == nv.shape[-1]:
            return x, tuple(shape[:i])
        if k > nv.shape[-1]:
            break
    return None


def _as_nd(g: fx.Graph, before: fx.Node, src) -> fx.Node:
    """Materialise ``X`` viewed as ``[*lead, K]`` (inserting a view only when dims must merge)."""
    x, lead = src
    xv = x.meta["val"]
    if xv.ndim == len(lead) + 1:
        return x
    k = 1
    for s in xv.shape[len(lead):]:
        k *= s
    with g.inserting_before(before):
        v = g.call_function(aten.view.default, (x, [*lead, k]))
    v.meta["val"] = xv.new_empty((*lead, k))
    _copy_meta(v, before)
    return v


def rewrite_linear_patterns(gm: fx.GraphModule) -> int:
    """Returns the number of ``aten.mm`` nodes rewritten."""
    g = gm.graph
    count = 0
    for n in list(g.nodes):
        if n.op != "call_function" or n.target is not aten.mm.default:
            continue
        a, b = n.args
        out_dtype = n.meta["val"].dtype
        # weight gradient: permute(view(P)) @ view(Q)  ->  mm_wgrad(P, Q)
        if _is_2d_transpose(a):
            ps, qs = _flatten_source(a.args[0]), _flatten_source(b)
            if ps is not None and qs is not None and ps[1] == qs[1]:
                p, q = _as_nd(g, n, ps), _as_nd(g, n, qs)
                with g.inserting_before(n):
                    new = g.call_function(apb.mm_wgrad.default, (p, q, out_dtype))
                new.meta["val"] = n.meta["val"]
                _copy_meta(new, n)
                n.replace_all_uses_with(new)
                g.erase_node(n)
                count += 1
                continue
        xs = _flatten_source(a)
        if xs is None:
            continue
        x = _as_nd(g, n, xs)
        if _is_2d_transpose(b):
            w, trans_b = b.args[0], True
        else:
            w, trans_b = b, False
        lead = xs[1]
        n_out = n.meta["val"].shape[-1]
        with g.inserting_before(n):
            new = g.call_function(apb.mm_nd.default, (x, w, trans_b, out_dtype))
        new.meta["val"] = n.meta["val"].new_empty((*lead, n_out))
        _copy_meta(new, n)
        flat = None
        for u in list(n.users):
            uv = _meta_val(u)
            if u.op == "call_function" and u.target in _VIEW_OPS and uv is not None and tuple(uv.shape) == (*lead, n_out):
                u.replace_all_uses_with(new)
                g.erase_node(u)
            else:
                if flat is None:
                    with g.inserting_after(new):
                        flat = g.call_function(aten.view.default, (new, list(n.meta["val"].shape)))
                    flat.meta["val"] = n.meta["val"]
                    _copy_meta(flat, n)
                u.replace_input_with(n, flat)
        g.erase_node(n)
        count += 1
    if count:
        cleanup_graph(gm)
    return count


# ------------------------------------------------------------------------------------ alias insertion
def insert_redistribution_points(gm: fx.GraphModule) -> int:
    g = gm.graph
    added = 0
    out_node = next(n for n in g.nodes if n.op == "output")
    for n in list(g.nodes):
        if n.op in ("output",) or not _is_tensor_node(n):
            continue
        if n.op == "call_function" and n.target is aten.alias.default:
            continue
        users = [u for u in n.users]
        needs = len(users) > 1 or (out_node in users and n.op != "placeholder")
        if not needs:
            continue
        with g.inserting_after(n):
            al = g.call_function(aten.alias.default, (n,))
        al.meta["val"] = n.meta["val"]
        _copy_meta(al, n)
        al.meta["apb200_redistribution_point"] = True
        for u in users:
            u.replace_input_with(n, al)
        added += 1
    g.lint()
    gm.recompile()
    return added


def strip_redistribution_points(gm: fx.GraphModule) -> None:
    g = gm.graph
    for n in list(g.nodes):
        if n.op == "call_function" and n.target is aten.alias.default:
            n.replace_all_uses_with(n.args[0])
            g.erase_node(n)
    gm.recompile()


def rewrite_means_as_scaled_sums(gm: fx.GraphModule) -> int:
    """``mean(x, dims)`` -> ``sum(x, dims) * (1 / count)``.

    A mean over a sharded dim has no exact placement of its own (the mean of shard means needs an averaging reduction),
    so as a single node it forces the operand to be gathered first - ``loss = out.mean()`` on batch-sharded activations
    would gather every activation.  Written as a sum, the sharded reduction yields ``Partial(sum)``, which a scalar-sized
    all-reduce completes; the count is that of the global tensor, so the scaling is exact for any sharding.  (The
    reference reaches the same plans through DTensor's ``Partial("avg")`` strategies.)"""
    aten = torch.ops.aten
    g = gm.graph
    count = 0
    for n in list(g.nodes):
        if n.op != "call_function" or n.target not in (aten.mean.default, aten.mean.dim):
            continue
        x = n.args[0]
        xv, ov = _meta_val(x), _meta_val(n)
        if not isinstance(xv, torch.Tensor) or not isinstance(ov, torch.Tensor) or not ov.dtype.is_floating_point:
            continue
        if n.target is aten.mean.default:
            dims, keepdim = list(range(xv.ndim)), False
        else:
            dims = n.args[1] if len(n.args) > 1 else n.kwargs.get("dim")
            dims = list(range(xv.ndim)) if dims is None or len(dims) == 0 else [d % xv.ndim for d in dims]
            keepdim = n.args[2] if len(n.args) > 2 else n.kwargs.get("keepdim", False)
        dtype = n.kwargs.get("dtype")
        if any(not isinstance(xv.shape[d], int) for d in dims):
            continue
        numel = 1
        for d in dims:
            numel *= xv.shape[d]
        if numel == 0:
            continue
        with g.inserting_before(n):
            s = g.call_function(aten.sum.dim_IntList, (x, dims, keepdim), {"dtype": dtype} if dtype is not None else {})
            _copy_meta(s, n)
            s.meta["val"] = ov
            y = g.call_function(aten.mul.Tensor, (s, 1.0 / numel))
            _copy_meta(y, n)
            y.meta["val"] = ov
        n.replace_all_uses_with(y)
        g.erase_node(n)
        count += 1
    if count:
        g.lint()
        gm.recompile()
    return count


def canonicalize(gm: fx.GraphModule, *, linear_patterns: bool = True, aliases: bool = True) -> None:
    assert_has_no_collectives(gm)
    cleanup_graph(gm)
    rewrite_means_as_scaled_sums(gm)
    if linear_patterns:
        rewrite_linear_patterns(gm)
    if aliases:
        insert_redistribution_points(gm)


def is_getitem(node: fx.Node) -> bool:
    return node.op == "call_function" and node.target is operator.getitem
