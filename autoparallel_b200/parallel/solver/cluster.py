"""Repeated-subgraph detection by bounded colour refinement.

Transformer stacks repeat one layer many times; giving every repetition its own decision
variables multiplies the ILP for no benefit.  Each node gets an initial colour from purely
local facts (op, constant args, output metadata, candidate strategies, user-constraint salt);
then ``rounds`` times a node's colour is re-hashed together with the colours of its inputs (in
argument order) and of its users (as a multiset, with the argument slot they consume it in).
Nodes that end with equal colours have isomorphic ``rounds``-hop neighbourhoods and share one
set of ILP variables; nodes near the ends of the stack differ within the horizon and stay
separate.  The reference gets the same reduction from Dynamo's graph-region tracker
(autoparallel/graph_passes/graph_clustering.py:84-206); the algorithm here is our own.
"""
from __future__ import annotations

from typing import Callable, Hashable, Iterable

import torch.fx as fx


def refine_colors(
    nodes: Iterable[fx.Node],
    inputs_of: Callable[[fx.Node], list[fx.Node]],
    initial: Callable[[fx.Node], Hashable],
    rounds: int = 4,
) -> dict[fx.Node, int]:
    nodes = list(nodes)
    in_set = set(nodes)
    ins = {n: [i for i in inputs_of(n) if i in in_set] for n in nodes}
    users: dict[fx.Node, list[tuple[fx.Node, int]]] = {n: [] for n in nodes}
    for n in nodes:
        for slot, i in enumerate(ins[n]):
            users[i].append((n, slot))
    color = {n: hash(initial(n)) for n in nodes}
    n_classes = len(set(color.values()))
    for _ in range(rounds):
        new = {}
        for n in nodes:
            up = tuple(color[i] for i in ins[n])
            down = tuple(sorted((color[u], slot) for u, slot in users[n]))
            new[n] = hash((color[n], up, down))
        color = new
        k = len(set(color.values()))
        if k == n_classes:
            break
        n_classes = k
    # compact ids in first-appearance order (deterministic given graph order)
    ids: dict[int, int] = {}
    out = {}
    for n in nodes:
        out[n] = ids.setdefault(color[n], len(ids))
    return out
