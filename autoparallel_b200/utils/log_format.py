"""Human-readable dump of a sharding solution.

One line per graph node: name, op, chosen output placement, then per tensor argument the required
input placement and the (comm, compute, transition) cost the solver paid; totals at the end.
``verbose`` adds shapes and source locations; ``colored`` highlights edges that redistribute.
Reference format: autoparallel/log_formatting.py:19-210 and
docs/how_autoparallel_chooses_a_strategy.md:182-219.
"""
from __future__ import annotations

import torch.fx as fx

_RED, _DIM, _END = "\033[31m", "\033[2m", "\033[0m"


def _shape(node: fx.Node) -> str:
    v = node.meta.get("val")
    if hasattr(v, "shape"):
        return f"{str(v.dtype).replace('torch.', '')}{list(v.shape)}"
    if isinstance(v, (tuple, list)):
        return "(" + ", ".join(f"{str(x.dtype).replace('torch.', '')}{list(x.shape)}" if hasattr(x, "shape") else "None" for x in v) + ")"
    return ""


def format_sharding_log(optimizer, verbose: bool = False, colored: bool = False) -> str:
    from ..parallel.solver.ilp import INF_COST, _fmt_pl, _out_placements

    if optimizer.selected is None:
        return "<no solution: call get_solution() first>"
    lines = []
    tot_comm = tot_comp = 0.0
    n_redist = 0
    for node in optimizer.graph.nodes:
        if node not in optimizer.selected:
            continue
        i = optimizer.selected[node]
        spec = optimizer.strats[node].strategies[i]
        comp = float(optimizer._node_cost[node][i])
        tot_comp += comp
        target = node.op if node.op != "call_function" else str(node.target).replace("aten.", "").replace(".default", "")
        head = f"{node.name:28s} {target:34s} -> {_fmt_pl(_out_placements(spec))}"
        if verbose:
            head += f"  {_shape(node)}"
        costs = []
        for slot, p in enumerate(optimizer._inputs(node)):
            c = float(optimizer._edge_cost[(node, slot)][i, optimizer.selected[p]])
            comm = 0.0 if c >= INF_COST else c
            src = _out_placements(optimizer.strats[p].strategies[optimizer.selected[p]])
            dst = spec.input_specs[slot].placements if spec.input_specs else None
            changed = comm > 0
            n_redist += int(changed)
            tot_comm += comm
            item = f"{p.name}:{_fmt_pl(src) if not isinstance(src[0] if src else None, tuple) else '(..)'}→{_fmt_pl(dst)} comm={comm:.1f}"
            if colored and changed:
                item = f"{_RED}{item}{_END}"
            costs.append(item)
        line = head + (f"  # compute={comp:.1f}us " + " ".join(costs) if (costs or comp) else "")
        if verbose and node.meta.get("stack_trace"):
            loc = str(node.meta["stack_trace"]).strip().splitlines()[-2:]
            line += f"\n{'':8s}{_DIM if colored else ''}{loc[0].strip() if loc else ''}{_END if colored else ''}"
        lines.append(line)
    lines.append("")
    lines.append(f"total: compute {tot_comp:.1f} us, communication {tot_comm:.1f} us, {n_redist} redistributed edges, "
                 f"objective {optimizer.objective_value:.1f}")
    if getattr(optimizer, "problem_size", None):
        lines.append(f"ILP: {optimizer.problem_size}  timings: { {k: round(v, 3) for k, v in optimizer.timings.items()} }")
    return "\n".join(lines)
