"""Lowering: global joint graph + chosen placements → per-rank graph with collectives.

For every node, each tensor argument is moved from its producer's chosen output placement to the
placement this node's chosen strategy requires (``Shard→Replicate`` all-gather, ``Partial→
Replicate`` all-reduce, ``Partial→Shard`` reduce-scatter, ``Shard→Shard`` all-to-all,
``Replicate→Shard`` local slice), shape arguments of views / factories are rewritten to local
shapes, and the op itself is emitted unchanged on local tensors.  Redistributions of one tensor
to one target placement are emitted once and shared.  The result contains ``apb200_comm``
collective nodes (see ``runtime/comm_ops.py``).

Reference: autoparallel/apply_sharding.py:84-293 (``ApplyShardingInterpreter``) – which re-traces
with ``make_fx`` over DTensor's redistribute; here the per-rank graph is constructed directly.
"""
from __future__ import annotations

import dataclasses
import logging
import operator
from typing import Any, Optional

import torch
import torch.fx as fx

from ...runtime import comm_ops
from ..frontend.graph_canon import all_input_nodes
from ..frontend.trace import JointGraph
from ..strategies.dtensor_adapter import DTensorSpec, OpSpec, Replicate, Shard, is_even, local_shape_at, my_local_shape, shard_extent

logger = logging.getLogger(__name__)
aten = torch.ops.aten
comm = comm_ops.ops

# op -> position of the "size" argument that must be rewritten to the local output shape
_SIZE_ARG = {
    aten.view.default: 1,
    aten._unsafe_view.default: 1,
    aten.reshape.default: 1,
    aten.expand.default: 1,
    aten.zeros.default: 0,
    aten.ones.default: 0,
    aten.full.default: 0,
    aten.empty.memory_format: 0,
    aten.rand.default: 0,
    aten.randn.default: 0,
    aten.new_zeros.default: 1,
    aten.new_ones.default: 1,
    aten.new_empty.default: 1,
    aten.new_full.default: 1,
    aten.new_empty_strided.default: 1,
    aten.empty_strided.default: 0,
}
# factories whose argument after the size is a stride list
_STRIDED_FACTORIES = (aten.new_empty_strided.default, aten.empty_strided.default)


def _strides_like(old_strides, new_shape) -> list[int]:
    """Dense strides for ``new_shape`` that keep the dim order of ``old_strides`` (outermost = largest stride)."""
    order = sorted(range(len(new_shape)), key=lambda d: (-old_strides[d], d))
    out, acc = [0] * len(new_shape), 1
    for d in reversed(order):
        out[d] = acc
        acc *= max(int(new_shape[d]), 1)
    return out


def _localize_moe_slots(args, val, lval):
    # block count follows the token shard: every rank keeps whole blocks
    args[3] = args[3] * lval.shape[0] // val.shape[0]
    return args


def _localize_moe_scatter(args, val, lval):
    args[5] = lval.shape[1]
    return args


def _localize_group_norm(args, val, lval):
    # native_group_norm(x, weight, bias, N, C, HxW, groups, eps): N is the batch extent of the (possibly batch-sharded) input
    x = args[0].meta.get("val") if isinstance(args[0], fx.Node) else None
    if isinstance(x, torch.Tensor):
        args[3] = x.shape[0]
    return args


def _localize_group_norm_bwd(args, val, lval):
    # native_group_norm_backward(dy, x, mean, rstd, weight, N, C, HxW, groups, mask)
    x = args[1].meta.get("val") if isinstance(args[1], fx.Node) else None
    if isinstance(x, torch.Tensor):
        args[5] = x.shape[0]
    return args


# op -> rewrite of integer arguments that describe a global extent (args list, global value, local value)
_INT_ARG_LOCALIZERS = {
    aten.native_group_norm.default: _localize_group_norm,
    aten.native_group_norm_backward.default: _localize_group_norm_bwd,
    torch.ops.apb200.moe_slots.default: _localize_moe_slots,
    torch.ops.apb200.moe_scatter.default: _localize_moe_scatter,
}


@dataclasses.dataclass
class LoweredGraph:
    gm: fx.GraphModule
    joint: JointGraph  # re-indexed over ``gm``
    #: placements of parameters / buffers / inputs / outputs in the solution (a parameter whose shards
    #: were re-nested by the ordered-sharding pass carries a ``_StridedShard``)
    param_placements: dict[str, tuple]
    buffer_placements: dict[str, tuple]
    input_placements: list[Optional[tuple]]
    output_placements: list[Optional[tuple]]
    num_collectives: dict[str, int]


def _spec_for_input(producer_spec: OpSpec, consumer: fx.Node) -> Optional[DTensorSpec]:
    o = producer_spec.output_specs
    if isinstance(o, DTensorSpec):
        return o
    if consumer.op == "call_function" and consumer.target is operator.getitem:
        return o[consumer.args[1]]
    return next((x for x in o if x is not None), None)


class _Redistributor:
    def __init__(self, graph: fx.Graph, mesh, fuse_flat: bool = True):
        self.g = graph
        self.mesh = mesh
        self.fuse_flat = fuse_flat
        self.groups = []
        for i in range(mesh.ndim):
            pg = mesh.get_group(i)
            self.groups.append((pg.group_name, mesh.shape[i]))
        self.flat_group = None  # (name, size) of the flattened mesh, created on first use
        self.cache: dict[tuple, fx.Node] = {}
        self.counts = {"all_gather": 0, "reduce_scatter": 0, "all_reduce": 0, "all_to_all": 0, "local_chunk": 0}

    def _flat(self):
        """Process group over every rank of the mesh in row-major order (None if it cannot be made)."""
        if self.flat_group is None and self.mesh.ndim > 1:
            try:
                flat = self.mesh._flatten()
                self.flat_group = (flat.get_group().group_name, flat.size())
            except Exception as e:  # unnamed mesh dims, or a backend that cannot split: keep per-dim collectives
                logger.info("flattened mesh unavailable (%s); nested shards use one collective per mesh dim", e)
                self.flat_group = False
        return self.flat_group or None

    def _emit(self, kind: str, args: tuple, like: fx.Node, shape) -> fx.Node:
        n = self.g.call_function(getattr(comm, kind).default, args)
        v = like.meta["val"]
        n.meta["val"] = v.new_empty(shape)
        for k in ("stack_trace", "nn_module_stack", "seq_nr", "autograd_backward", "apb200_phase"):
            if k in like.meta:
                n.meta[k] = like.meta[k]
        self.counts["all_reduce" if kind == "all_reduce_op" else kind] += 1
        return n

    def _emit_all_reduce(self, cur, st, gname, n, like, shape) -> fx.Node:
        """Sums use ``all_reduce`` (own kernels, split-phase forms); a pending maximum / minimum its own operator."""
        if getattr(st, "op", "sum") == "sum":
            return self._emit("all_reduce", (cur, gname, n), like, shape)
        node = self._emit("all_reduce_op", (cur, st.op, gname, n), like, shape)
        return node

    def _local(self, target, args: tuple, like: fx.Node, shape) -> fx.Node:
        n = self.g.call_function(target, args)
        n.meta["val"] = like.meta["val"].new_empty(shape)
        for k in ("stack_trace", "nn_module_stack", "seq_nr", "autograd_backward", "apb200_phase"):
            if k in like.meta:
                n.meta[k] = like.meta[k]
        return n

    def _uneven_steps(self, cur: fx.Node, like: fx.Node, steps, full: list[int], shape: list[int], placements) -> fx.Node:
        """Collectives between shards of unequal size.  Ceil-sized chunks put all full chunks first, so a
        gather of shards padded to the chunk size has the valid rows in front: pad, gather, cut the tail.
        A scatter pads the whole extent to ``parts x chunk`` and every rank cuts its chunk down to what it
        owns (possibly nothing).  Reference: autoparallel/apply_sharding.py:372-386 (pad / slice nodes)."""
        coord = self.mesh.get_coordinate() or [0] * self.mesh.ndim
        mshape = tuple(self.mesh.shape)
        pl = list(placements)
        nd = len(shape)

        def seen_extent(m: int, d: int) -> int:
            others = [Replicate() if i == m else p for i, p in enumerate(pl)]
            return local_shape_at(full, mshape, others, coord)[d]

        def pad_to(node, d, size):
            if shape[d] == size:
                return node
            grow = size - shape[d]
            shape[d] = size
            return self._local(aten.constant_pad_nd.default, (node, _pad_spec(nd, d, grow), 0.0), like, shape)

        def cut(node, d, start, end):
            if start == 0 and end == shape[d]:
                return node
            shape[d] = max(0, end - start)
            return self._local(aten.slice.Tensor, (node, d, start, end), like, shape)

        for st in steps:
            gname, n = self.groups[st.mesh_dim]
            m, me = st.mesh_dim, coord[st.mesh_dim]
            if st.kind == "all_reduce":
                cur = self._emit_all_reduce(cur, st, gname, n, like, shape)
                pl[m] = Replicate()
            elif st.kind == "all_gather":
                d = st.dim
                extent = seen_extent(m, d)
                cur = pad_to(cur, d, -(-extent // n))
                shape[d] *= n
                cur = self._emit("all_gather", (cur, d, gname, n), like, shape)
                cur = cut(cur, d, 0, extent)
                pl[m] = Replicate()
            elif st.kind == "reduce_scatter":
                d = st.dim
                extent = shape[d]
                chunk = -(-extent // n)
                cur = pad_to(cur, d, chunk * n)
                shape[d] = chunk
                cur = self._emit("reduce_scatter", (cur, d, gname, n), like, shape)
                cur = cut(cur, d, 0, shard_extent(extent, n, me))
                pl[m] = Shard(d)
            elif st.kind == "all_to_all":
                new, old = st.dim, st.dim2
                old_extent, new_extent = seen_extent(m, old), shape[new]
                chunk = -(-new_extent // n)
                cur = pad_to(cur, old, -(-old_extent // n))
                cur = pad_to(cur, new, chunk * n)
                shape[old] *= n
                shape[new] = chunk
                cur = self._emit("all_to_all", (cur, new, old, gname, n), like, shape)
                cur = cut(cur, old, 0, old_extent)
                cur = cut(cur, new, 0, shard_extent(new_extent, n, me))
                pl[m] = Shard(new)
            elif st.kind == "local_chunk":
                d = st.dim
                extent = shape[d]
                if extent % n == 0:
                    shape[d] //= n
                    cur = self._emit("local_chunk", (cur, d, gname, n), like, shape)
                else:
                    chunk = -(-extent // n)
                    start = min(me * chunk, extent)
                    cur = cut(cur, d, start, min(start + chunk, extent))
                    self.counts["local_chunk"] += 1
                pl[m] = Shard(d)
        return cur

    def __call__(self, x: fx.Node, key_node: fx.Node, src: DTensorSpec, dst: DTensorSpec, order=None) -> fx.Node:
        """Emit (or reuse) the collectives taking local tensor ``x`` from ``src`` to ``dst``; ``order`` is
        the nesting order of mesh dims for a tensor dim sharded over several of them."""
        if src.placements == dst.placements:
            return x
        key = (key_node, tuple(dst.placements), order)
        hit = self.cache.get(key)
        if hit is not None:
            return hit
        from .redistribute import FLAT, fuse_over_flat_mesh, plan_redistribution

        cur = x
        shape = list(x.meta["val"].shape)
        steps = plan_redistribution(src.placements, dst.placements, self.mesh.shape, order=order)
        full = list(src.tensor_meta.shape) if src.tensor_meta is not None else None
        uneven = full is not None and not (
            is_even(full, self.mesh.shape, src.placements) and is_even(full, self.mesh.shape, dst.placements)
        )
        if uneven:
            cur = self._uneven_steps(cur, x, steps, full, shape, src.placements)
            self.cache[key] = cur
            return cur
        if self.fuse_flat and self._flat() is not None:
            steps = fuse_over_flat_mesh(steps, self.mesh.ndim, order)
        for st in steps:
            gname, n = self.flat_group if st.mesh_dim == FLAT else self.groups[st.mesh_dim]
            if st.kind == "all_gather":
                shape[st.dim] *= n
                cur = self._emit("all_gather", (cur, st.dim, gname, n), x, shape)
            elif st.kind == "all_reduce":
                cur = self._emit_all_reduce(cur, st, gname, n, x, shape)
            elif st.kind == "reduce_scatter":
                shape[st.dim] //= n
                cur = self._emit("reduce_scatter", (cur, st.dim, gname, n), x, shape)
            elif st.kind == "all_to_all":
                shape[st.dim2] *= n
                shape[st.dim] //= n
                cur = self._emit("all_to_all", (cur, st.dim, st.dim2, gname, n), x, shape)
            elif st.kind == "local_chunk":
                shape[st.dim] //= n
                cur = self._emit("local_chunk", (cur, st.dim, gname, n), x, shape)
        self.cache[key] = cur
        return cur


def _pad_spec(ndim: int, dim: int, amount: int) -> list[int]:
    """``constant_pad_nd`` argument that appends ``amount`` entries at the end of ``dim``."""
    return [0, 0] * (ndim - 1 - dim) + [0, amount]


def _inline_region(g: fx.Graph, body: fx.GraphModule, args) -> fx.Node:
    """Copy the body of a ``local_map`` region (already traced on local shapes) into ``g`` and return
    a node producing the tuple of its outputs."""
    env: dict[fx.Node, Any] = {}
    it = iter(args)
    out = None
    for n in body.graph.nodes:
        if n.op == "placeholder":
            env[n] = next(it)
        elif n.op == "output":
            vals = fx.node.map_arg(n.args[0], lambda a: env[a])
            out = g.call_function(_make_tuple, tuple(vals) if isinstance(vals, (tuple, list)) else (vals,))
        elif n.op == "get_attr":
            raise NotImplementedError("local_map bodies that close over tensors are not supported; pass them as arguments")
        else:
            env[n] = g.node_copy(n, lambda a: env[a])
    return out


def _make_tuple(*xs):
    return tuple(xs)


def _local_val(val, spec: Optional[DTensorSpec], mesh):
    if not isinstance(val, torch.Tensor) or spec is None:
        return val
    # this rank's own shard: smaller than rank 0's (or empty) where an extent does not divide
    return val.new_empty(my_local_shape(val.shape, mesh, spec.placements))


def lower_to_local_graph(joint: JointGraph, solution: dict[fx.Node, OpSpec], mesh, ordered_sharding: bool = True) -> LoweredGraph:
    from ..frontend.trace import index_joint_graph

    old_g = joint.gm.graph
    new_g = fx.Graph()
    env: dict[fx.Node, fx.Node] = {}
    redis = _Redistributor(new_g, mesh, fuse_flat=ordered_sharding)
    from .ordered import compute_shard_orders, dtensor_placements

    orders = compute_shard_orders(joint, solution, mesh) if ordered_sharding else {}

    for node in old_g.nodes:
        if node.op == "placeholder":
            nn_ = new_g.placeholder(node.target)
            nn_.meta = dict(node.meta)
            spec = solution[node].output_spec if node in solution else None
            nn_.meta["val"] = _local_val(node.meta.get("val"), spec, mesh)
            if spec is not None:
                nn_.meta["apb200_placements"] = tuple(spec.placements)
            env[node] = nn_
        elif node.op == "get_attr":
            nn_ = new_g.get_attr(node.target)
            nn_.meta = dict(node.meta)
            env[node] = nn_
        elif node.op == "output":
            def conv_out(a):
                return env[a] if isinstance(a, fx.Node) else a

            out = new_g.output(fx.node.map_arg(node.args[0], conv_out))
            out.meta = dict(node.meta)
        elif node.op == "call_function":
            if node not in solution:
                # shape arithmetic etc.: copy verbatim
                nn_ = new_g.node_copy(node, lambda a: env[a])
                env[node] = nn_
                continue
            spec = solution[node]
            slot = 0
            tensor_inputs = [i for i in all_input_nodes(node) if i in solution]
            it = iter(range(len(tensor_inputs)))

            def conv(a):
                nonlocal slot
                if a not in solution:
                    return env[a]
                s = next(it)
                src = _spec_for_input(solution[a], node)
                dst = spec.input_specs[s] if spec.input_specs else None
                if src is None or dst is None:
                    return env[a]
                # a re-nested layout applies to edges leaving the parameter chain and to the edge into its gradient
                return redis(env[a], a, src, dst, orders.get(a) or orders.get(node))

            new_args, new_kwargs = fx.node.map_arg((node.args, node.kwargs), conv)
            out_spec = spec.output_specs
            val = node.meta.get("val")
            if isinstance(out_spec, DTensorSpec):
                lval = _local_val(val, out_spec, mesh)
            elif isinstance(val, (tuple, list)):
                lval = tuple(_local_val(v, s, mesh) for v, s in zip(val, out_spec))
            else:
                lval = val
            if node.target in _SIZE_ARG and isinstance(lval, torch.Tensor):
                pos = _SIZE_ARG[node.target]
                new_args = list(new_args)
                if node.target is aten.expand.default:
                    old = list(node.args[pos])
                    new_args[pos] = [-1 if o == -1 else l for o, l in zip(old, lval.shape)]
                else:
                    new_args[pos] = list(lval.shape)
                    if node.target in _STRIDED_FACTORIES:
                        new_args[pos + 1] = _strides_like(list(node.args[pos + 1]), list(lval.shape))
                new_args = tuple(new_args)
            if node.target in _INT_ARG_LOCALIZERS and isinstance(lval, (torch.Tensor, tuple, list)):
                new_args = tuple(_INT_ARG_LOCALIZERS[node.target](list(new_args), val, lval))
            from ..strategies.local_map_rules import is_local_map_node, local_map_body

            rng_key = _sharded_rng_key(node, out_spec, mesh)
            if is_local_map_node(node):
                nn_ = _inline_region(new_g, local_map_body(node), new_args)
            elif rng_key is not None:
                # a random operator whose output is sharded: every rank draws from the stream of ITS shard
                # (runtime/rng.py); ranks that hold the same shard share the stream
                from ...runtime import rng

                if node.target is aten.native_dropout.default:
                    nn_ = new_g.call_function(rng.sharded_dropout, (new_args[0], new_args[1], new_args[2] if len(new_args) > 2 else True, rng_key))
                elif node.target in _RANDOM_LIKE_OPS:
                    nn_ = new_g.call_function(rng.sharded_like, (node.target, rng_key) + tuple(new_args), dict(new_kwargs))
                else:
                    nn_ = new_g.call_function(rng.sharded_rand, (new_args[0], rng_key, node.target is aten.randn.default), dict(new_kwargs))
            else:
                target = node.target
                if target in (aten.view.default, aten._unsafe_view.default):
                    # strides of a kernel's output may differ from the ones tracing assumed (attention outputs
                    # above all); reshape is the same view when one exists and a copy otherwise
                    target = aten.reshape.default
                nn_ = new_g.call_function(target, new_args, new_kwargs)
            nn_.meta = dict(node.meta)
            nn_.meta["val"] = lval
            nn_.meta["apb200_placements"] = (
                tuple(out_spec.placements)
                if isinstance(out_spec, DTensorSpec)
                else tuple(tuple(s.placements) if s is not None else None for s in out_spec)
            )
            env[node] = nn_
        else:
            raise NotImplementedError(node.op)

    new_gm = fx.GraphModule(joint.gm, new_g)
    # aliases were only redistribution points for the solver
    from ..frontend.graph_canon import strip_redistribution_points

    strip_redistribution_points(new_gm)
    new_gm.graph.eliminate_dead_code()
    sink_input_chains(new_gm)
    new_gm.graph.lint()
    new_gm.recompile()
    new_joint = index_joint_graph(new_gm, joint.traced_inputs, joint.out_spec)

    def pl(n):
        return tuple(solution[n].output_spec.placements) if isinstance(n, fx.Node) and n in solution else None

    return LoweredGraph(
        gm=new_gm,
        joint=new_joint,
        param_placements={k: (dtensor_placements(pl(v), orders.get(v), tuple(mesh.shape)) if pl(v) is not None else None)
                          for k, v in joint.param_nodes.items()},
        buffer_placements={k: pl(v) for k, v in joint.buffer_nodes.items()},
        input_placements=[pl(n) for n in joint.input_nodes],
        output_placements=[pl(n) for n in joint.fwd_outputs],
        num_collectives=dict(redis.counts),
    )


_RANDOM_LIKE_OPS = (aten.uniform.default, aten.normal_functional.default, aten.bernoulli.p, aten.bernoulli.default,
                    aten.rand_like.default, aten.randn_like.default)
_RANDOM_OPS = (aten.native_dropout.default, aten.rand.default, aten.randn.default) + _RANDOM_LIKE_OPS


def _sharded_rng_key(node: fx.Node, out_spec, mesh):
    """((mesh dim, this rank's coordinate), ...) over the mesh dims that shard the output of a random operator, or
    None when the operator is not random or its output is replicated (then every rank must draw the same numbers)."""
    if node.target not in _RANDOM_OPS:
        return None
    spec = out_spec if isinstance(out_spec, DTensorSpec) else next((s for s in out_spec if s is not None), None)
    if spec is None:
        return None
    from torch.distributed.tensor.placement_types import Shard as _Shard

    dims = [i for i, p in enumerate(spec.placements) if isinstance(p, _Shard)]
    if not dims:
        return None
    try:
        coords = [mesh.get_local_rank(i) for i in dims]
    except Exception:
        coords = [0 for _ in dims]
    return tuple(zip(dims, coords))


def sink_input_chains(gm: fx.GraphModule) -> int:
    """Move computations that depend only on graph inputs (parameter → cast → all-gather → view
    chains) down to just before their first consumer.

    The solver's redistribution points sit right after the placeholders, so without this every
    parameter gather would run – and its full-size result stay alive – from the top of the
    graph.  Sinking restores "gather right before use" (what FSDP does), which bounds memory and
    gives the overlap scheduler a meaningful first-use position to prefetch towards.
    """
    g = gm.graph
    nodes = list(g.nodes)
    input_only = {n for n in nodes if n.op == "placeholder"}
    chain = []
    for n in nodes:
        # single-input chains only (cast / gather / view of one graph input): anything that joins two
        # tensors is real computation, not parameter preparation
        if n.op == "call_function" and len(n.all_input_nodes) == 1 and n.all_input_nodes[0] in input_only:
            input_only.add(n)
            chain.append(n)
    moved = 0
    for n in reversed(chain):
        users = list(n.users)
        if not users:
            continue
        pos = {x: i for i, x in enumerate(g.nodes)}
        first = min(users, key=lambda u: pos[u])
        if first.op == "output":
            continue
        if pos[first] - pos[n] > 1:
            first.prepend(n)
            moved += 1
    g.lint()
    gm.recompile()
    return moved
