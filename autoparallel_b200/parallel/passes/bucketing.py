"""Bucketing of small parameter all-gathers and gradient reduce-scatters.

Dozens of sub-megabyte collectives per layer (norm weights, biases) are latency-bound: each costs
a kernel launch and a flag round trip for a few kilobytes.  This pass merges *adjacent* collectives
of one kind on one process group whose inputs depend only on graph inputs (gathers) or whose
results only feed graph outputs (reductions) into one collective over a packed 1-D buffer:

    all_gather(p1), all_gather(p2), ...   →  pack → one all_gather → unpack views
    reduce_scatter(g1), reduce_scatter(g2) →  pack (chunk-major) → one reduce_scatter → unpack

A bucket closes when it reaches ``max_bucket_bytes`` or when more than ``max_span`` graph nodes lie
between its first and last member (keeping members close preserves the prefetch order and bounds
how long the first member's data waits).  Dim-0 shardings only, fp32 / bf16 only – the same limits
as the reference's bucketing (autoparallel/graph_passes/autobucketing_inductor/bucket_utils.py:
487-764, size and span rules in autoparallel/graph_passes/auto_bucketing.py:19-188, 294-314).

Two ways to decide what goes into a bucket:

* static (``BucketConfig`` alone): collectives below ``small_bytes`` are merged up to the caps above;
* cost driven (``BucketCost``, ``AutoParallel(bucket_collectives="auto")``): collectives of any size are
  candidates and a member joins a bucket only if (i) the priced collective gets cheaper by at least
  ``min_saving_us`` after paying for the member's copies into and out of the packed buffers (prices come
  from the active topology, i.e. from a table calibrated on the machine when one is loaded), (ii) a gather bucket still finishes inside the compute window in front of its first
  consumer, so that merging never turns hidden communication into exposed communication, (iii) the bytes
  the bucket keeps alive longer than the separate collectives would (earlier gathered outputs, gradients
  held until the last member exists, the packed buffers) fit the memory headroom, and (iv) the bucket stays
  below ``max_fraction`` of all candidate bytes of its kind, so that a step never degenerates into one
  collective.  Reference: autoparallel/graph_passes/autobucketing_inductor/bucket_plan.py:60-330 (greedy plan
  from calibrated estimates with a memory check), estimation_utils.py:73-147.
"""
from __future__ import annotations

import dataclasses
import math
import operator

import torch
import torch.fx as fx

from ...runtime import comm_ops

aten = torch.ops.aten
C = comm_ops.ops


@dataclasses.dataclass
class BucketConfig:
    max_bucket_bytes: int = 64 << 20
    small_bytes: int = 4 << 20  # only collectives below this size are bucketed
    max_span: int = 1500


@dataclasses.dataclass
class BucketCost:
    """Prices for the cost-driven plan.  ``collective_us(kind, nbytes, n_ranks, group)`` with ``kind`` in
    {"all_gather", "reduce_scatter"} and ``nbytes`` the size of the full (gathered / pre-scatter) tensor;
    ``compute_us(node)`` for everything else."""

    collective_us: callable
    compute_us: callable
    copy_us: callable = lambda nbytes: 0.0  # device time of moving ``nbytes`` (read + write counted by the caller)
    headroom_bytes: int = 2 << 30
    min_saving_us: float = 1.0
    window_nodes: int = 12  # compute nodes in front of a consumer that a prefetched gather can hide under
    max_fraction: float = 0.2

    @classmethod
    def from_mesh(cls, mesh, plan_device=None, headroom_bytes: int = 2 << 30, **kw) -> "BucketCost":
        """Prices from the topology that is active for ``mesh`` (formula, NCCL model or a measured table)."""
        from ...parallel.cost import comm as comm_cost
        from ...utils.trace_sim import make_runtime_estimator

        topo = comm_cost.get_topology(mesh)
        group_dim = {mesh.get_group(i).group_name: i for i in range(mesh.ndim)}
        est = make_runtime_estimator(mesh, plan_device)

        def collective_us(kind, nbytes, n, group):
            dim = group_dim.get(group, 0)
            return (topo.all_gather if kind == "all_gather" else topo.reduce_scatter)(dim, n, nbytes)

        from ...parallel.cost.device import DEVICE_LIMITS, get_device_limit

        limit = DEVICE_LIMITS[plan_device] if plan_device else get_device_limit(mesh.device_type)

        def copy_us(nbytes):
            return max(limit.launch_us, nbytes / limit.bytes_per_us())

        return cls(collective_us, est, copy_us, headroom_bytes, **kw)


def _nbytes(n: fx.Node) -> int:
    v = n.meta.get("val")
    return v.numel() * v.element_size() if isinstance(v, torch.Tensor) else 0


def _pack(xs):
    return torch.cat([x.reshape(-1) for x in xs])


def _unpack_gather(buf, shapes, n):
    """buf = all_gather(pack(shards), 0) of n ranks: rank-major; rebuild each gathered tensor."""
    sizes = [math.prod(s) for s in shapes]
    per_rank = buf.view(n, -1)
    outs, off = [], 0
    for s, k in zip(shapes, sizes):
        piece = per_rank[:, off : off + k].reshape(n * s[0], *s[1:])
        outs.append(piece)
        off += k
    return tuple(outs)


def _pack_scatter(xs, n):
    """Chunk-major packing: reduce_scatter(dim 0) of the packed buffer hands rank r the r-th row block
    of every member."""
    return torch.cat([x.reshape(n, -1) for x in xs], dim=1).reshape(-1)


def _unpack_scatter(buf, shapes, n):
    sizes = [math.prod(s) // n for s in shapes]
    outs, off = [], 0
    for s, k in zip(shapes, sizes):
        outs.append(buf[off : off + k].reshape(s[0] // n, *s[1:]))
        off += k
    return tuple(outs)


def bucket_collectives(gm: fx.GraphModule, config: BucketConfig | None = None, cost: BucketCost | None = None) -> dict:
    cfg = config or BucketConfig()
    if cost is not None and config is None:
        cfg = BucketConfig(max_bucket_bytes=1 << 40, small_bytes=1 << 40)  # sizes are decided by the prices
    g = gm.graph
    order = {n: i for i, n in enumerate(g.nodes)}
    placeholders = {n for n in g.nodes if n.op == "placeholder"}
    # chains that start at a tangent belong to the backward; a bucket holding one would make the forward depend on it
    tangents = {n for n in placeholders if (n.meta.get("apb200_kind") or (None,))[0] == "tangent" or n.name.startswith("tangents")}
    input_only = set(placeholders) - tangents
    for n in g.nodes:
        # single-input chains only (cast / gather / view of one graph input): anything that joins two
        # tensors is real computation, not parameter preparation
        if n.op == "call_function" and len(n.all_input_nodes) == 1 and n.all_input_nodes[0] in input_only:
            input_only.add(n)
    out_node = next(n for n in g.nodes if n.op == "output")
    stats = {"all_gather_buckets": 0, "reduce_scatter_buckets": 0, "members": 0}
    if cost is not None:
        stats.update({"saved_us": 0.0, "rejected_saving": 0, "rejected_window": 0, "rejected_memory": 0, "rejected_fraction": 0})
    nodes_in_order = list(g.nodes)
    _compute_cache: dict = {}

    def compute_us(n):
        if n not in _compute_cache:
            t = 0.0
            if n.op == "call_function" and n.target not in comm_ops.COLLECTIVE_OPS and n.target not in comm_ops.START_OPS:
                try:
                    t = float(cost.compute_us(n))
                except Exception:
                    t = 0.0
            _compute_cache[n] = t
        return _compute_cache[n]

    def window_us(user):
        """Compute time of the ``window_nodes`` kernels in front of ``user``: what a prefetched gather can hide under."""
        i = order[user] - 1
        seen, t = 0, 0.0
        while i >= 0 and seen < cost.window_nodes:
            d = compute_us(nodes_in_order[i])
            if d > 0:
                t += d
                seen += 1
            i -= 1
        return t

    def size_of(kind, n):
        # priced mode counts the full tensor a collective moves (gathered output / pre-scatter input); the static caps
        # are defined on the node's own output
        return _nbytes(n.args[0]) if (cost is not None and kind == "rs") else _nbytes(n)

    def accept(kind, bucket, size, n, total_bytes):
        """May ``n`` join ``bucket`` (current full-tensor bytes ``size``)?"""
        nb = size_of(kind, n)
        if size + nb > cfg.max_bucket_bytes or order[n] - order[bucket[0]] > cfg.max_span:
            return False
        if cost is None:
            return True
        group, n_ranks = n.args[2], n.args[3]
        name = "all_gather" if kind == "ag" else "reduce_scatter"
        if total_bytes > 0 and size + nb > cost.max_fraction * total_bytes and len(bucket) >= 2:
            stats["rejected_fraction"] += 1
            return False
        merged = cost.collective_us(name, size + nb, n_ranks, group)
        saving = cost.collective_us(name, size, n_ranks, group) + cost.collective_us(name, nb, n_ranks, group) - merged
        # a member of a bucket is copied into the packed buffer and (gathers) out of the gathered one; alone it is not

        def packing(nbytes):
            if kind == "ag":
                return cost.copy_us(2 * nbytes // n_ranks) + cost.copy_us(2 * nbytes)
            return cost.copy_us(2 * nbytes)

        saving -= packing(nb) + (packing(size) if len(bucket) == 1 else 0.0)
        if saving < cost.min_saving_us:
            stats["rejected_saving"] += 1
            return False
        if kind == "ag":
            first_user = min((u for m in bucket for u in m.users), key=lambda u: order[u])
            latency = cost.collective_us(name, 0, n_ranks, group)
            if merged > max(window_us(first_user), 4.0 * latency):  # latency-bound buckets are always worth it
                stats["rejected_window"] += 1
                return False
            held = sum(_nbytes(m) for m in bucket[1:]) + nb  # gathered earlier than they would be
            extra = held + (size + nb) + (size + nb) // n_ranks  # + gathered buffer + packed shards
        else:
            held = sum(_nbytes(m.args[0]) for m in bucket)  # gradients wait for the last member
            extra = held + (size + nb) + (size + nb) // n_ranks
        if extra > cost.headroom_bytes:
            stats["rejected_memory"] += 1
            return False
        stats["saved_us"] += saving
        return True

    def candidates(target, pred):
        res = []
        for n in g.nodes:
            if n.op == "call_function" and n.target is target and n.args[1] == 0 and pred(n):
                v = n.meta["val"]
                if v.dtype in (torch.float32, torch.bfloat16) and _nbytes(n) <= cfg.small_bytes:
                    res.append(n)
        return res

    def close(kind, members):
        if len(members) < 2:
            return
        group, n_ranks = members[0].args[2], members[0].args[3]
        first_user = min((u for m in members for u in m.users), key=lambda u: order[u])
        srcs = [m.args[0] for m in members]
        anchor = max(srcs + [], key=lambda s: order.get(s, -1))
        insert_at = members[-1] if kind == "ag" else members[-1]
        with g.inserting_after(insert_at):
            if kind == "ag":
                shapes = [tuple(s.meta["val"].shape) for s in srcs]
                packed = g.call_function(_pack, (srcs,))
                gathered = g.call_function(C.all_gather.default, (packed, 0, group, n_ranks))
                outs = g.call_function(_unpack_gather, (gathered, shapes, n_ranks))
            else:
                shapes = [tuple(s.meta["val"].shape) for s in srcs]
                packed = g.call_function(_pack_scatter, (srcs, n_ranks))
                reduced = g.call_function(C.reduce_scatter.default, (packed, 0, group, n_ranks))
                outs = g.call_function(_unpack_scatter, (reduced, shapes, n_ranks))
        # fx inserts "after" in reverse order of creation: fix the order explicitly
        nodes = [packed, gathered if kind == "ag" else reduced, outs]
        prev = insert_at
        for nd in nodes:
            prev.append(nd)
            prev = nd
        total = sum(math.prod(s) for s in shapes)
        dt = srcs[0].meta["val"].dtype
        packed.meta["val"] = srcs[0].meta["val"].new_empty((total,))
        (gathered if kind == "ag" else reduced).meta["val"] = srcs[0].meta["val"].new_empty(
            (total * n_ranks,) if kind == "ag" else (total // n_ranks,))
        outs.meta["val"] = tuple(m.meta["val"] for m in members)
        for i, m in enumerate(members):
            with g.inserting_after(prev):
                gi = g.call_function(operator.getitem, (outs, i))
            gi.meta = dict(m.meta)
            prev = gi
            m.replace_all_uses_with(gi)
            g.erase_node(m)
        stats["all_gather_buckets" if kind == "ag" else "reduce_scatter_buckets"] += 1
        stats["members"] += len(members)

    backward_nodes = set(tangents)
    for n in g.nodes:
        if n.op == "call_function" and any(i in backward_nodes for i in n.all_input_nodes):
            backward_nodes.add(n)

    def phase(n) -> bool:
        """True for a collective that only the backward consumes (the re-gather of a parameter, say).  It must not share a
        bucket with one the forward waits for: it would run, and its result stay alive, from the forward on."""
        users = list(n.users)
        return bool(users) and all(u in backward_nodes for u in users)

    def plan(kind, cands):
        """Buckets (lists of members, graph order) of one kind; nothing in the graph is touched."""
        by_group: dict = {}
        for n in cands:
            by_group.setdefault((n.args[2], n.meta["val"].dtype, phase(n)), []).append(n)
        buckets = []
        for members in by_group.values():
            bucket, size = [], 0
            total_bytes = sum(size_of(kind, m) for m in members)
            for n in members:
                if bucket and not accept(kind, bucket, size, n, total_bytes):
                    buckets.append(bucket)
                    bucket, size = [], 0
                bucket.append(n)
                size += size_of(kind, n)
            buckets.append(bucket)
        return [b for b in buckets if len(b) >= 2]

    # Gathers of graph-input-derived shards (parameter -> cast -> gather chains).  Such a chain can
    # run anywhere after the placeholders, so the members of a bucket are first hoisted – chain and
    # all – to sit right behind the bucket's first member; every consumer stays after that point.
    def chain_of(n):
        ch, cur = [], n.args[0]
        while cur not in placeholders and cur.op == "call_function":
            ch.append(cur)
            cur = cur.all_input_nodes[0]
        return list(reversed(ch))

    ag = candidates(C.all_gather.default, lambda n: n.args[0] in input_only and all(len(c.users) == 1 for c in chain_of(n)))
    by_group: dict = {}
    for n in ag:
        by_group.setdefault((n.args[2], n.meta["val"].dtype, phase(n)), []).append(n)
    for members in by_group.values():
        bucket, size = [], 0
        total_bytes = sum(_nbytes(m) for m in members)

        def flush():
            if len(bucket) >= 2:
                prev = bucket[0]
                for m in bucket[1:]:
                    for c in chain_of(m):
                        prev.append(c)
                        prev = c
                    prev.append(m)
                    prev = m
                close("ag", list(bucket))

        for n in members:
            if bucket and not accept("ag", bucket, size, n, total_bytes):
                flush()
                bucket, size = [], 0
            bucket.append(n)
            size += _nbytes(n)
        flush()
    order = {n: i for i, n in enumerate(g.nodes)}
    nodes_in_order = list(g.nodes)
    rs = candidates(C.reduce_scatter.default, lambda n: all(u is out_node for u in n.users))

    # Reductions that feed only the graph's outputs can be delayed: the members of a bucket (and nothing else) move to
    # the position of its last member.  Reductions that stay alone keep their place.
    for bucket in plan("rs", rs):
        last = bucket[-1]
        for m in bucket[:-1]:
            last.prepend(m)
        close("rs", bucket)
    g.lint()
    gm.recompile()
    return stats
