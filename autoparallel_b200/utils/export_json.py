"""JSON export of a solved plan (mesh, nodes with phase / placement / edges / costs / module path,
summary) – the input of the HTML visualizer and of external tooling.
Reference: autoparallel/export_json.py:23-424."""
from __future__ import annotations

import torch
import torch.fx as fx


def _phase(node: fx.Node, tangent_dep: set) -> str:
    return "backward" if node in tangent_dep else "forward"


def _module_path(node: fx.Node) -> str:
    st = node.meta.get("nn_module_stack") or node.meta.get("fwd_nn_module_stack")
    if st:
        try:
            return list(st.values())[-1][0]
        except Exception:
            return ""
    return ""


def export_sharding_json(optimizer) -> dict:
    from ..parallel.solver.ilp import INF_COST, _fmt_pl, _out_placements

    mesh = optimizer.mesh
    tangent_dep = set(optimizer.joint.tangent_nodes)
    for n in optimizer.graph.nodes:
        if n.op == "call_function" and any(i in tangent_dep for i in n.all_input_nodes):
            tangent_dep.add(n)
    classes = optimizer._classes() if optimizer.repeated_subgraphs else {}
    nodes = []
    tot_comm = tot_comp = 0.0
    for node in optimizer.graph.nodes:
        if optimizer.selected is None or node not in optimizer.selected:
            continue
        i = optimizer.selected[node]
        spec = optimizer.strats[node].strategies[i]
        v = node.meta.get("val")
        entry = {
            "name": node.name,
            "op": node.op,
            "target": str(node.target) if node.op == "call_function" else str(node.target),
            "phase": _phase(node, tangent_dep),
            "placement": _fmt_pl(_out_placements(spec)),
            "shape": list(v.shape) if isinstance(v, torch.Tensor) else None,
            "dtype": str(v.dtype) if isinstance(v, torch.Tensor) else None,
            "module_path": _module_path(node),
            "compute_us": float(optimizer._node_cost[node][i]),
            "cluster": int(classes.get(node, -1)),
            "recompute": bool(node.meta.get("recompute")),
            "num_options": len(optimizer.strats[node].strategies),
            "kind": list(node.meta.get("apb200_kind", ())) or None,
            "edges": [],
        }
        tot_comp += entry["compute_us"]
        for slot, p in enumerate(optimizer._inputs(node)):
            c = float(optimizer._edge_cost[(node, slot)][i, optimizer.selected[p]])
            c = 0.0 if c >= INF_COST else c
            tot_comm += c
            entry["edges"].append({
                "from": p.name,
                "arg": slot,
                "src_placement": _fmt_pl(_out_placements(optimizer.strats[p].strategies[optimizer.selected[p]])),
                "dst_placement": _fmt_pl(spec.input_specs[slot].placements) if spec.input_specs else None,
                "comm_us": c,
            })
        nodes.append(entry)
    return {
        "version": 1,
        "mesh": {"shape": list(mesh.shape), "dim_names": list(mesh.mesh_dim_names or []), "device_type": mesh.device_type},
        "nodes": nodes,
        "summary": {
            "num_nodes": len(nodes),
            "compute_us": tot_comp,
            "comm_us": tot_comm,
            "objective": optimizer.objective_value,
            "ilp": getattr(optimizer, "problem_size", None),
            "timings_s": dict(optimizer.timings),
            "constraints": [{"name": c.name, "kind": c.kind, "what": c.description} for c in optimizer.constraints.values()],
        },
    }
