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


def bucket_collectives(gm: fx.GraphModule, config: BucketConfig | None = None) -> dict:
    cfg = config or BucketConfig()
    g = gm.graph
    order = {n: i for i, n in enumerate(g.nodes)}
    placeholders = {n for n in g.nodes if n.op == "placeholder"}
    input_only = set(placeholders)
    for n in g.nodes:
        # single-input chains only (cast / gather / view of one graph input): anything that joins two
        # tensors is real computation, not parameter preparation
        if n.op == "call_function" and len(n.all_input_nodes) == 1 and n.all_input_nodes[0] in input_only:
            input_only.add(n)
    out_node = next(n for n in g.nodes if n.op == "output")
    stats = {"all_gather_buckets": 0, "reduce_scatter_buckets": 0, "members": 0}

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

    def run(kind, cands):
        by_group: dict = {}
        for n in cands:
            by_group.setdefault((n.args[2], n.meta["val"].dtype), []).append(n)
        for members in by_group.values():
            bucket, size = [], 0
            for n in members:
                if bucket and (size + _nbytes(n) > cfg.max_bucket_bytes or order[n] - order[bucket[0]] > cfg.max_span):
                    close(kind, bucket)
                    bucket, size = [], 0
                bucket.append(n)
                size += _nbytes(n)
            close(kind, bucket)

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
        by_group.setdefault((n.args[2], n.meta["val"].dtype), []).append(n)
    for members in by_group.values():
        bucket, size = [], 0

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
            if bucket and (size + _nbytes(n) > cfg.max_bucket_bytes or order[n] - order[bucket[0]] > cfg.max_span):
                flush()
                bucket, size = [], 0
            bucket.append(n)
            size += _nbytes(n)
        flush()
    order = {n: i for i, n in enumerate(g.nodes)}
    rs = candidates(C.reduce_scatter.default, lambda n: all(u is out_node for u in n.users))

    def rs_runs(nodes):
        # reductions feeding only the output can be delayed to the position of the last member
        return [nodes] if nodes else []

    for r in rs_runs(rs):
        # move every member (and nothing else) to the position of the last one
        last = r[-1]
        for m in r[:-1]:
            last.prepend(m)
        order = {n: i for i, n in enumerate(g.nodes)}
        run("rs", r)
    g.lint()
    gm.recompile()
    return stats
