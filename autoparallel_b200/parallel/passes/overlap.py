"""Overlap scheduling of the per-rank graphs.

Each collective becomes an issue node (``*_start``) and a ``comm_wait`` node, and the node order is
rewritten so that communication hides under independent compute:

* **parameter gathers are prefetched** – a gather whose inputs derive only from graph inputs
  (parameter → cast → gather chains, in forward and in the recomputed backward chains) is issued
  ``prefetch_depth`` gathers ahead of the one currently being waited for, bounded by
  ``max_in_flight_bytes`` of gathered-but-unused data;
* **gradient reductions are deferred** – the wait of a reduce-scatter / all-reduce whose result
  only feeds graph outputs sinks past later compute until ``max_pending_reductions`` are pending
  (each pending one pins its full-size input) and the rest drain at the end.

All ranks run the same node order, so collectives are issued in the same order everywhere.  The
reference obtains overlap from Inductor's ``schedule_overlap_bucketing`` with
``max_in_flight_gb=2``, ``max_compute_pre_fetch`` (autoparallel/compile.py:19-24,
autoparallel/graph_passes/auto_bucketing.py:294-351); this pass is the framework's own scheduler
for graphs whose nodes are its own kernels.
"""
from __future__ import annotations

import dataclasses
import operator
from typing import Optional

import torch
import torch.fx as fx

from ...runtime import comm_ops


@dataclasses.dataclass
class OverlapConfig:
    prefetch_depth: int = 12  # gathers issued ahead of the one being consumed
    max_in_flight_bytes: int = 2 << 30
    max_pending_reductions: int = 6


def _nbytes(n: fx.Node) -> int:
    v = n.meta.get("val")
    return v.numel() * v.element_size() if isinstance(v, torch.Tensor) else 0


def split_collectives(gm: fx.GraphModule) -> int:
    g = gm.graph
    count = 0
    for n in list(g.nodes):
        if n.op == "call_function" and n.target in comm_ops.START_OF:
            with g.inserting_before(n):
                start = g.call_function(comm_ops.START_OF[n.target], n.args, n.kwargs)
                wait = g.call_function(comm_ops.ops.comm_wait.default, (start,))
            start.meta = dict(n.meta)
            wait.meta = dict(n.meta)
            n.replace_all_uses_with(wait)
            g.erase_node(n)
            count += 1
    return count


def schedule_for_streams(gm: fx.GraphModule, mesh=None, config: Optional[OverlapConfig] = None) -> fx.GraphModule:
    cfg = config or OverlapConfig()
    if split_collectives(gm) == 0:
        return gm
    g = gm.graph
    nodes = list(g.nodes)
    placeholders = [n for n in nodes if n.op == "placeholder"]
    out_node = next(n for n in nodes if n.op == "output")
    body = [n for n in nodes if n.op not in ("placeholder", "output")]

    # ---- input-only chains (everything a prefetchable start depends on)
    input_only: set[fx.Node] = set(placeholders)
    for n in body:
        # single-input chains from a graph input (parameter -> cast -> gather -> view)
        if n.op == "get_attr" or (len(n.all_input_nodes) == 1 and n.all_input_nodes[0] in input_only):
            if n.op == "get_attr" or n.target is not comm_ops.ops.comm_wait.default:
                input_only.add(n)
    ag_start = comm_ops.ops.all_gather_start.default
    prefetchable = [n for n in body if n.target is ag_start and n in input_only]
    prefetch_set = set(prefetchable)
    # the chain feeding each prefetchable start (moves with it)
    chain_of: dict[fx.Node, list[fx.Node]] = {}
    claimed: set[fx.Node] = set()
    for s in prefetchable:
        chain, stack = [], [s]
        seen = set()
        while stack:
            x = stack.pop()
            for i in x.all_input_nodes:
                if i.op in ("placeholder",) or i in seen or i in claimed:
                    continue
                if len([u for u in i.users]) > 1 and not all(u in input_only for u in i.users):
                    continue  # shared with non-prefetch consumers: leave in place
                seen.add(i)
                stack.append(i)
        chain = [n for n in body if n in seen]
        claimed.update(chain)
        chain_of[s] = chain
    moved = set(prefetch_set) | claimed

    # ---- deferred waits: result feeds only the output (through single-use chains)
    wait_op = comm_ops.ops.comm_wait.default
    rs_starts = (comm_ops.ops.reduce_scatter_start.default, comm_ops.ops.all_reduce_start.default)

    def only_feeds_output(n: fx.Node) -> bool:
        cur = n
        for _ in range(8):
            users = list(cur.users)
            if len(users) != 1:
                return False
            if users[0] is out_node:
                return True
            cur = users[0]
            if cur.target in comm_ops.START_OPS or cur.target is wait_op:
                return False
            if len(cur.all_input_nodes) != 1:
                # the result joins another tensor on its way out (gradients of a tied parameter are added up): its tail
                # cannot move as a unit behind this wait alone
                return False
        return False

    deferred_waits = {
        n for n in body if n.target is wait_op and n.args[0].target in rs_starts and only_feeds_output(n)
    }
    tail_of: dict[fx.Node, list[fx.Node]] = {}
    for w in deferred_waits:
        tail, cur = [], w
        while True:
            users = list(cur.users)
            if len(users) != 1 or users[0] is out_node:
                break
            cur = users[0]
            tail.append(cur)
        tail_of[w] = tail
    deferred_tail = {t for ts in tail_of.values() for t in ts}

    # ---- emit the new order
    order: list[fx.Node] = []
    pf_queue = list(prefetchable)  # in first-use order (graph order of the original gathers)
    issued = 0
    in_flight = 0
    pending_red: list[fx.Node] = []

    def issue_prefetch(upto: int):
        nonlocal issued, in_flight
        while issued < len(pf_queue) and issued < upto:
            s = pf_queue[issued]
            if in_flight + _nbytes(s) > cfg.max_in_flight_bytes and in_flight > 0:
                break
            order.extend(chain_of[s])
            order.append(s)
            in_flight += _nbytes(s)
            issued += 1

    pf_index = {s: i for i, s in enumerate(pf_queue)}
    issue_prefetch(cfg.prefetch_depth)
    for n in body:
        if n in moved or n in deferred_tail:
            continue
        if n in deferred_waits:
            pending_red.append(n)
            while len(pending_red) > cfg.max_pending_reductions:
                w = pending_red.pop(0)
                order.append(w)
                order.extend(tail_of[w])
            continue
        if n.target is wait_op and n.args[0] in prefetch_set:
            s = n.args[0]
            # make sure this gather has been issued (budget may have held it back)
            while issued <= pf_index[s]:
                before = issued
                in_flight_backup = in_flight
                issue_prefetch(pf_index[s] + 1)
                if issued == before:
                    in_flight = 0  # nothing else can free the budget: force progress
                    issue_prefetch(pf_index[s] + 1)
            order.append(n)
            in_flight = max(0, in_flight - _nbytes(s))
            issue_prefetch(pf_index[s] + 1 + cfg.prefetch_depth)
            continue
        order.append(n)
    for w in pending_red:
        order.append(w)
        order.extend(tail_of[w])

    # ---- rebuild the graph in the new order
    new_g = fx.Graph()
    env: dict[fx.Node, fx.Node] = {}
    for p in placeholders:
        env[p] = new_g.placeholder(p.target)
        env[p].meta = dict(p.meta)
    assert len(order) == len(body), (len(order), len(body))
    for n in order:
        env[n] = new_g.node_copy(n, lambda a: env[a])
    new_g.output(fx.node.map_arg(out_node.args[0], lambda a: env[a]))
    new_g.lint()
    new_gm = fx.GraphModule(gm, new_g)
    new_gm.recompile()
    return new_gm


def exposed_collectives(gm: fx.GraphModule) -> int:
    """Number of collectives whose wait directly follows their issue (nothing overlaps them)."""
    nodes = list(gm.graph.nodes)
    n_exposed = 0
    for a, b in zip(nodes, nodes[1:]):
        if a.op == "call_function" and a.target in comm_ops.START_OPS and b.target is comm_ops.ops.comm_wait.default and b.args[0] is a:
            n_exposed += 1
    return n_exposed


def max_compute_run_between_reductions(gm: fx.GraphModule) -> int:
    """Longest run of compute nodes between two consecutive reduce-scatter / all-reduce issues (or graph ends).

    A regression metric for the scheduler: gradient reductions that are deferred too far bunch up at the end of the
    backward, where nothing is left to hide them; a small value means they are spread through the compute.
    (Reference: the ``_max_consec_compute_between_rs`` check of autoparallel/graph_passes/auto_bucketing.py:191-210.)"""
    C = comm_ops.ops
    reductions = {C.reduce_scatter.default, C.reduce_scatter_start.default, C.all_reduce.default, C.all_reduce_start.default,
                  C.mm_rs.default, C.scaled_mm_rs.default}
    passive = {C.comm_wait.default}
    longest = run = 0
    for n in gm.graph.nodes:
        if n.op != "call_function":
            continue
        if n.target in reductions:
            longest, run = max(longest, run), 0
        elif n.target in passive or n.target in comm_ops.COLLECTIVE_OPS or n.target in comm_ops.START_OPS:
            continue
        elif isinstance(n.meta.get("val"), (torch.Tensor, tuple, list)) and n.target not in _FREE_OPS:
            run += 1
    return max(longest, run)


_FREE_OPS = {torch.ops.aten.view.default, torch.ops.aten.reshape.default, torch.ops.aten._unsafe_view.default, torch.ops.aten.permute.default,
             torch.ops.aten.t.default, torch.ops.aten.alias.default, torch.ops.aten.expand.default, torch.ops.aten.unsqueeze.default,
             torch.ops.aten.squeeze.dim, torch.ops.aten.slice.Tensor, operator.getitem}
